// Internal alias of the public header so every kernel file sees the declarations it defines.
#pragma once
#include "../../include/wukong_b200.h"
