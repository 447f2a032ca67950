"""ctypes loader of libwukong_b200.so (the C-ABI boundary)."""
import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libwukong_b200.so")
_HEADER = os.path.join(_HERE, "..", "include", "wukong_b200.h")


class WukongB200Error(RuntimeError):
    pass


def library_path():
    return _SO


_lib = None

i64, f32, vp, ci = C.c_int64, C.c_float, C.c_void_p, C.c_int


def declared_symbols(header=_HEADER):
    """Names of every function the public header declares."""
    with open(header) as fh:
        text = fh.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:wukong|wkb)_[a-z0-9_]+)\s*\(", text)))


def _types_from_header(header=_HEADER):
    """Parse `ret name(args);` prototypes into ctypes signatures."""
    with open(header) as fh:
        text = fh.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#.*", "", text)
    sigs = {}
    for m in re.finditer(r"([A-Za-z_][A-Za-z0-9_ \*]*?)\s*\b((?:wukong|wkb)_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3)

        def ctype(decl):
            decl = decl.strip()
            if decl in ("void", ""):
                return None
            if "*" in decl:
                return vp
            base = decl.replace("const", "").split()
            if base[0] in ("int64_t",):
                return i64
            if base[0] == "float":
                return f32
            if base[0] == "double":
                return C.c_double
            if base[0] == "int":
                return ci
            raise WukongB200Error("unparsed parameter %r of %s" % (decl, name))

        argt = [ctype(a) for a in args.split(",")] if args.strip() not in ("", "void") else []
        rett = C.c_char_p if ("char" in ret and "*" in ret) else ctype(ret)
        sigs[name] = (rett, argt)
    return sigs


def lib():
    """The loaded library.  Raises when the CUDA extension has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            raise WukongB200Error(
                "libwukong_b200.so is missing: run `python -m wukong_b200.build` (there is no CPU fallback)")
        L = C.CDLL(_SO)
        for name, (ret, args) in _types_from_header().items():
            try:
                fn = getattr(L, name)
            except AttributeError:
                raise WukongB200Error("library does not export %s" % name)
            fn.restype = ret
            fn.argtypes = args
        _lib = L
    return _lib


def check(code, what):
    if code != 0:
        raise WukongB200Error("%s failed with status %d" % (what, code))


def require_gpu():
    if lib().wkb_device_count() < 1:
        raise WukongB200Error("no CUDA device: wukong_b200 has no CPU path")
