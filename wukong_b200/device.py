"""Device-resident API on torch CUDA tensors (torch supplies memory and streams only; every kernel
is this library's own).  Thin wrappers over the `wkb_*` entry points of the C ABI."""
import numpy as np
import torch

from ._lib import lib, check, vp


def _s():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def vmath(x, op, out=None):
    out = torch.empty_like(x) if out is None else out
    check(lib().wkb_vmath_f32(_p(x), _p(out), x.numel(), op, _s()), "wkb_vmath_f32")
    return out


def act_bf16(x, op, gate=None, out=None):
    out = torch.empty_like(x) if out is None else out
    check(lib().wkb_act_bf16(_p(x), _p(gate), _p(out), x.numel(), op, _s()), "wkb_act_bf16")
    return out


def norm_f32(x, op, eps=0.0, gamma=None, beta=None, affine=False, out=None):
    out = torch.empty_like(x) if out is None else out
    rows, cols = x.shape
    bits = int(np.float32(eps).view(np.uint32))
    check(lib().wkb_norm_f32(_p(x), _p(out), _p(gamma), _p(beta), rows, cols, bits, op, int(affine), _s()), "wkb_norm_f32")
    return out


def norm_fast(x, op, eps=1e-5, gamma=None, beta=None, out_dtype=None, out=None):
    rows, cols = x.shape
    out_dtype = out_dtype or x.dtype
    out = torch.empty((rows, cols), dtype=out_dtype, device=x.device) if out is None else out
    check(lib().wkb_norm_fast(_p(x), _DT[x.dtype], _p(out), _DT[out.dtype], _p(gamma), _p(beta), rows, cols, eps, op, _s()),
          "wkb_norm_fast")
    return out


def q_split(raw_u8, nblocks, q4=True):
    qs = torch.empty(nblocks * (16 if q4 else 32), dtype=torch.uint8, device=raw_u8.device)
    d = torch.empty(nblocks, dtype=torch.float16, device=raw_u8.device)
    check(lib().wkb_q_split(_p(raw_u8), _p(qs), _p(d), nblocks, int(q4), _s()), "wkb_q_split")
    return qs, d


def quantize_act(x):
    k = x.numel()
    nb = (k + 31) // 32
    xq = torch.empty(nb * 32, dtype=torch.int8, device=x.device)
    dx = torch.empty(nb, dtype=torch.float32, device=x.device)
    sx = torch.empty(nb, dtype=torch.int32, device=x.device)
    check(lib().wkb_quantize_act(_p(x), k, _p(xq), _p(dx), _p(sx), _s()), "wkb_quantize_act")
    return xq, dx, sx


def gemv_q_contract(qs, d, xq, dx, sx, n, k, q4=True, out=None):
    y = torch.empty(n, dtype=torch.float32, device=qs.device) if out is None else out
    check(lib().wkb_gemv_q_contract(_p(qs), _p(d), _p(xq), _p(dx), _p(sx), _p(y), n, k, int(q4), _s()), "wkb_gemv_q_contract")
    return y


def gemv_q4_0_bf16x(qs, d, x_bf16, n, k, out=None):
    y = torch.empty(n, dtype=torch.float32, device=qs.device) if out is None else out
    check(lib().wkb_gemv_q4_0_bf16x(_p(qs), _p(d), _p(x_bf16), _p(y), n, k, _s()), "wkb_gemv_q4_0_bf16x")
    return y


def rowargmax(x, out=None):
    rows, cols = x.shape
    out = torch.empty(rows, dtype=torch.int32, device=x.device) if out is None else out
    check(lib().wkb_rowargmax_i32(_p(x), _p(out), rows, cols, _s()), "wkb_rowargmax_i32")
    return out
