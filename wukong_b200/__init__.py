"""wukong_b200: B200 (sm_100a) kernels behind the Wukong runtime's C ABI.

`wukong_b200.lib()` loads the in-tree CUDA library and fails loudly when it is missing;
`wukong_b200.runtime` mirrors the language's builtins over host (numpy) buffers through the
reference ABI; `wukong_b200.device` drives the device-resident API on torch CUDA tensors.
There is no CPU implementation behind any of them.
"""
from ._lib import lib, library_path, declared_symbols, WukongB200Error  # noqa: F401
