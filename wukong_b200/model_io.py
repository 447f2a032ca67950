"""Checkpoint containers: GGUF and safetensors tensors into host arrays or device tensors.

The names follow the reference's builtins (`gguf_read_<T>`, `gguf_find` / `gguf_rank` / `gguf_dim` / `gguf_type`,
`gguf_meta_*`, `st_read_<T>`; crates/wukong_compiler/src/sema/ml_builtins.rs:50-56) and the calls go through the
C ABI entries `wukong_rt_gguf_*` / `wukong_rt_st_read` / `wkb_*_read_device`.  Negative results are the reference's
codes: -1 open, -2 I/O, -3 dtype, -4 shape or count, -5 no such name, -6 malformed header, -7 no decoder."""
import ctypes

import numpy as np

from ._lib import lib, WukongB200Error

DT = {"f32": 0, "f64": 1, "f16": 2, "bf16": 3, "i8": 4, "i16": 5, "i32": 6, "i64": 7, "u8": 8, "u16": 9, "u32": 10, "u64": 11}
_NP = {0: np.float32, 1: np.float64, 2: np.float16, 3: np.uint16, 4: np.int8, 5: np.int16, 6: np.int32, 7: np.int64,
       8: np.uint8, 9: np.uint16, 10: np.uint32, 11: np.uint64}
CODES = {-1: "cannot open the file", -2: "I/O error", -3: "dtype mismatch", -4: "shape or element-count mismatch",
         -5: "no such tensor", -6: "malformed header", -7: "ggml type with no decoder"}


class ModelIOError(WukongB200Error):
    def __init__(self, code, what):
        super().__init__("%s: %s (%d)" % (what, CODES.get(code, "error"), code))
        self.code = code


def _b(s):
    return s if isinstance(s, bytes) else str(s).encode()


def _dims(shape):
    if shape is None:
        return None, -1
    arr = (ctypes.c_int64 * max(1, len(shape)))(*shape)
    return arr, len(shape)


def _read_host(fn, path, name, buf, shaped):
    dt = {v: k for k, v in _NP.items() if k != 3}[buf.dtype.type] if buf.dtype != np.uint16 else DT["u16"]
    dims, rank = _dims(buf.shape if shaped else None)
    return int(fn(_b(path), _b(name), buf.ctypes.data, buf.size, dt, dims, rank))


def gguf_read(path, name, buf, shaped=True):
    """Load GGUF tensor `name` into the numpy array `buf` (its dtype selects verbatim / widened / dequantized /
    raw-block loading; `shaped` checks the array's shape as a tensor view).  Returns the element count or a code."""
    return _read_host(lib().wukong_rt_gguf_read, path, name, buf, shaped)


def st_read(path, name, buf, shaped=True):
    return _read_host(lib().wukong_rt_st_read, path, name, buf, shaped)


def gguf_find(path, name):
    return int(lib().wukong_rt_gguf_query(_b(path), _b(name), 0, 0))


def gguf_rank(path, name):
    return int(lib().wukong_rt_gguf_query(_b(path), _b(name), 1, 0))


def gguf_dim(path, name, k):
    return int(lib().wukong_rt_gguf_query(_b(path), _b(name), 2, k))


def gguf_type(path, name):
    return int(lib().wukong_rt_gguf_query(_b(path), _b(name), 3, 0))


def gguf_shape(path, name):
    r = gguf_rank(path, name)
    if r < 0:
        raise ModelIOError(r, "gguf tensor %r" % name)
    return tuple(gguf_dim(path, name, k) for k in range(r))


def gguf_meta_type(path, key):
    return int(lib().wukong_rt_gguf_meta(_b(path), _b(key), 0, 0, 0))


def gguf_meta_len(path, key):
    return int(lib().wukong_rt_gguf_meta(_b(path), _b(key), 1, 0, 0))


def gguf_meta_i64(path, key, i=0, default=0):
    return int(lib().wukong_rt_gguf_meta(_b(path), _b(key), 2, i, default))


def gguf_meta_f64(path, key, i=0, default=0.0):
    return float(lib().wukong_rt_gguf_meta_f64(_b(path), _b(key), i, default))


def gguf_meta_str(path, key, i=0, cap=4096):
    """The string (bytes), or the negative code."""
    buf = ctypes.create_string_buffer(cap)
    n = int(lib().wukong_rt_gguf_meta_str(_b(path), _b(key), i, buf, cap))
    if n < 0:
        return n
    if n >= cap:
        return gguf_meta_str(path, key, i, n + 1)
    return buf.raw[:n]


# ---- device destinations -------------------------------------------------------------------------------------
def _torch_dt(t):
    import torch
    return {torch.float32: 0, torch.float64: 1, torch.float16: 2, torch.bfloat16: 3, torch.int8: 4, torch.int16: 5,
            torch.int32: 6, torch.int64: 7, torch.uint8: 8}[t.dtype]


def _read_device(fn, path, name, out, shaped, what):
    import torch
    if not out.is_cuda or not out.is_contiguous():
        raise ValueError("the destination must be a contiguous CUDA tensor")
    dims, rank = _dims(tuple(out.shape) if shaped else None)
    with torch.cuda.device(out.device):
        rc = int(fn(_b(path), _b(name), out.data_ptr(), out.numel(), _torch_dt(out), dims, rank,
                    torch.cuda.current_stream().cuda_stream))
    if rc < 0:
        raise ModelIOError(rc, "%s %r" % (what, name))
    return out


def gguf_read_device(path, name, out, shaped=True):
    """GGUF tensor `name` into the CUDA tensor `out`: f32 receives plain f32, widened halves or dequantized blocks
    (dequantized on the GPU from the raw bytes); uint8 receives the raw block rows; other dtypes load verbatim."""
    return _read_device(lib().wkb_gguf_read_device, path, name, out, shaped, "gguf tensor")


def st_read_device(path, name, out, shaped=True):
    return _read_device(lib().wkb_st_read_device, path, name, out, shaped, "safetensors tensor")


def gguf_load_q4_weight(path, name, device="cuda"):
    """A Q4_0 matrix of a GGUF checkpoint as the resident weight of the W4A16 GEMM: the [n, k/32] block rows are
    ggml's row-major layout, loaded raw and re-tiled on the device."""
    import torch
    from .device import Q4Weight
    if gguf_type(path, name) != 2:
        raise ModelIOError(-3, "gguf tensor %r is not Q4_0" % name)
    n, k = gguf_shape(path, name)
    raw = torch.empty((n, k // 32 * 18), dtype=torch.uint8, device=device)
    gguf_read_device(path, name, raw)
    return Q4Weight.from_raw(raw.reshape(-1), n, k)
