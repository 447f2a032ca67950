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


class Q4Weight:
    """Resident Q4_0 matrix [n, k] in the tiled layout of the tensor-core GEMM (wkb_q4_tile)."""

    def __init__(self, tiled, n, k):
        self.tiled, self.n, self.k = tiled, n, k

    @staticmethod
    def from_raw(raw_u8, n, k):
        """`raw_u8`: device tensor of the n * (k/32) 18-byte blocks as the reference stores them."""
        if k % 32:
            raise ValueError("k must be a multiple of 32")
        tiled = torch.empty(int(lib().wkb_q4_tiled_bytes(n, k)), dtype=torch.uint8, device=raw_u8.device)
        check(lib().wkb_q4_tile(_p(raw_u8), n, k, _p(tiled), _s()), "wkb_q4_tile")
        return Q4Weight(tiled, n, k)

    @staticmethod
    def from_planes(qs, d):
        """qs uint8 [n, k/32, 16] nibble bytes, d float16 [n, k/32] scales (device tensors)."""
        n, nb = d.shape
        raw = torch.cat([d.contiguous().view(torch.uint8).view(n, nb, 2), qs.view(n, nb, 16)], dim=2).contiguous()
        return Q4Weight.from_raw(raw.view(-1), n, nb * 32)

    def weight_bytes(self):
        return self.n * (self.k // 32) * 18


def gemm_q4_workspace(n, k, device="cuda"):
    return torch.zeros(int(lib().wkb_gemm_q4_0_workspace_bytes(n, k)), dtype=torch.uint8, device=device)


def gemm_q4_0_bf16_nt(w, x_bf16, mode=0, out=None, workspace=None):
    """out[m, n] = x . W^T (mode 0 f32, 1 bf16) or the SwiGLU of interleaved gate / up rows (mode 2, bf16 [m, n/2])."""
    m, k = x_bf16.shape
    if k != w.k or x_bf16.dtype != torch.bfloat16:
        raise ValueError("activation must be bf16 [m, k]")
    cols = w.n // 2 if mode == 2 else w.n
    if out is None:
        out = torch.empty(m, cols, dtype=torch.float32 if mode == 0 else torch.bfloat16, device=x_bf16.device)
    if workspace is None:
        workspace = gemm_q4_workspace(w.n, w.k, x_bf16.device)
    check(lib().wkb_gemm_q4_0_bf16_nt(_p(w.tiled), _p(x_bf16), x_bf16.stride(0), _p(out), out.stride(0), mode, m, w.n, k,
                                      _p(workspace), workspace.numel(), _s()), "wkb_gemm_q4_0_bf16_nt")
    return out


def rowargmax(x, out=None):
    rows, cols = x.shape
    out = torch.empty(rows, dtype=torch.int32, device=x.device) if out is None else out
    check(lib().wkb_rowargmax_i32(_p(x), _p(out), rows, cols, _s()), "wkb_rowargmax_i32")
    return out


def gemm_bf16_nt(a, b, bias=None, act=0, residual=None, out_dtype=torch.float32, out=None):
    """C = act(a @ b.T + bias) (+ residual) on the tcgen05 tensor cores; a [M,K], b [N,K] bf16."""
    m, k = a.shape
    n = b.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    ldr = residual.stride(0) if residual is not None else 0
    check(lib().wkb_gemm_bf16_nt(_p(a), a.stride(0), _p(b), b.stride(0), _p(out), out.stride(0),
                                 int(out.dtype == torch.bfloat16), m, n, k, _p(bias), act, _p(residual), ldr, _s()),
          "wkb_gemm_bf16_nt")
    return out


def gemm_e4m3_nt(a_codes, b_codes, bias=None, act=0, residual=None, out_dtype=torch.float32):
    """C = act(a @ b.T + bias) (+ residual) for E4M3FN codes held in uint8 tensors a [M,K], b [N,K]."""
    m, k = a_codes.shape
    n = b_codes.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=a_codes.device)
    ldr = residual.stride(0) if residual is not None else 0
    check(lib().wkb_gemm_e4m3_nt(_p(a_codes), a_codes.stride(0), _p(b_codes), b_codes.stride(0), _p(out), out.stride(0),
                                 int(out.dtype == torch.bfloat16), m, n, k, _p(bias), act, _p(residual), ldr, _s()),
          "wkb_gemm_e4m3_nt")
    return out


def gemm_status():
    return lib().wkb_gemm_status()


def sgemm_contract(a, b, c, m, k, n, beta=0, at=0, bt=1, bias=None, act=0, alpha=1.0, has_epi=0):
    check(lib().wkb_sgemm_contract(_p(a), _DT[a.dtype], _p(b), _DT[b.dtype], _p(c), m, k, n, beta, at, bt, _p(bias), act,
                                   alpha, has_epi, _s()), "wkb_sgemm_contract")
    return c


class PagedKV:
    """Per-layer K/V slabs, bf16 [layers][pages][kv_heads][page_tokens][head_dim]."""

    def __init__(self, layers, num_pages, kv_heads, head_dim, page_tokens=16, device="cuda"):
        self.layers, self.num_pages, self.kv_heads, self.head_dim, self.page_tokens = layers, num_pages, kv_heads, head_dim, page_tokens
        shape = (layers, num_pages, kv_heads, page_tokens, head_dim)
        self.k = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.v = torch.zeros(shape, dtype=torch.bfloat16, device=device)


def paged_kv_append(kv, layer, ksrc, vsrc, src_row_stride, block_table, row_slot, row_pos, rows, mbps):
    check(lib().wkb_paged_kv_append(_p(ksrc), _p(vsrc), src_row_stride, _p(kv.k[layer]), _p(kv.v[layer]), _p(block_table),
                                    _p(row_slot), _p(row_pos), rows, kv.kv_heads, kv.head_dim, kv.page_tokens, mbps, _s()),
          "wkb_paged_kv_append")


def paged_attn_scratch(rows, q_heads, head_dim, max_ctx, device="cuda"):
    n = lib().wkb_paged_attn_scratch_bytes(rows, q_heads, head_dim, max_ctx)
    return torch.empty(n // 4, dtype=torch.float32, device=device)


def paged_attn_decode(q, q_row_stride, kv, layer, block_table, row_slot, row_ctx, out, rows, q_heads, mbps, max_ctx, scale,
                      scratch):
    check(lib().wkb_paged_attn_decode(_p(q), q_row_stride, _p(kv.k[layer]), _p(kv.v[layer]), _p(block_table), _p(row_slot),
                                      _p(row_ctx), _p(out), int(out.dtype == torch.bfloat16), out.stride(0), rows, q_heads,
                                      kv.kv_heads, kv.head_dim, kv.page_tokens, mbps, max_ctx, scale, _p(scratch), _s()),
          "wkb_paged_attn_decode")
    return out


def prefill_tiles(row_slot, tile_rows, min_run=1):
    """Host helper: cut the runs of equal slot in `row_slot` (numpy int32, rows laid out sequence by sequence) into
    tiles of at most `tile_rows` rows -> int32 [n_tiles, 2] of (first row, row count).  Runs shorter than `min_run`
    rows are left out (the caller sends those rows through the decode kernel)."""
    import numpy as np
    rs = np.asarray(row_slot)
    n = rs.shape[0]
    if n == 0:
        return np.zeros((0, 2), np.int32)
    starts = np.flatnonzero(np.concatenate([[True], rs[1:] != rs[:-1]]))
    ends = np.concatenate([starts[1:], [n]])
    out = []
    for a, b in zip(starts.tolist(), ends.tolist()):
        if b - a < min_run:
            continue
        out.extend((r, min(tile_rows, b - r)) for r in range(a, b, tile_rows))
    return np.asarray(out, np.int32).reshape(-1, 2)


def paged_attn_prefill(q, q_row_stride, kv, layer, block_table, row_slot, row_ctx, tiles, out, q_heads, mbps, scale):
    """Causal attention of prompt-chunk rows against the paged cache; `tiles` is a device int32 [n_tiles, 2]."""
    check(lib().wkb_paged_attn_prefill(_p(q), q_row_stride, _p(kv.k[layer]), _p(kv.v[layer]), _p(block_table), _p(row_slot),
                                       _p(row_ctx), _p(tiles), tiles.shape[0], _p(out), int(out.dtype == torch.bfloat16),
                                       out.stride(0), q_heads, kv.kv_heads, kv.head_dim, kv.page_tokens, mbps, scale, _s()),
          "wkb_paged_attn_prefill")
    return out


class PagedKVInt8:
    """Per-layer int8 K/V slabs [layers][pages][kv_heads][page_tokens][head_dim] with f32 scales
    [layers][pages][kv_heads][page_tokens] (one per token and KV head)."""

    def __init__(self, layers, num_pages, kv_heads, head_dim, page_tokens=16, device="cuda"):
        self.layers, self.num_pages, self.kv_heads, self.head_dim, self.page_tokens = layers, num_pages, kv_heads, head_dim, page_tokens
        shape = (layers, num_pages, kv_heads, page_tokens, head_dim)
        self.k = torch.zeros(shape, dtype=torch.int8, device=device)
        self.v = torch.zeros(shape, dtype=torch.int8, device=device)
        self.k_scale = torch.ones(shape[:-1], dtype=torch.float32, device=device)
        self.v_scale = torch.ones(shape[:-1], dtype=torch.float32, device=device)


def paged_kv_append_int8(kv, layer, ksrc, vsrc, src_row_stride, block_table, row_slot, row_pos, rows, mbps):
    check(lib().wkb_paged_kv_append_int8(_p(ksrc), _p(vsrc), src_row_stride, _p(kv.k[layer]), _p(kv.v[layer]), _p(kv.k_scale[layer]),
                                         _p(kv.v_scale[layer]), _p(block_table), _p(row_slot), _p(row_pos), rows, kv.kv_heads,
                                         kv.head_dim, kv.page_tokens, mbps, _s()), "wkb_paged_kv_append_int8")


def paged_attn_decode_int8(q, q_row_stride, kv, layer, block_table, row_slot, row_ctx, out, rows, q_heads, mbps, max_ctx, scale, scratch):
    check(lib().wkb_paged_attn_decode_int8(_p(q), q_row_stride, _p(kv.k[layer]), _p(kv.v[layer]), _p(kv.k_scale[layer]),
                                           _p(kv.v_scale[layer]), _p(block_table), _p(row_slot), _p(row_ctx), _p(out),
                                           int(out.dtype == torch.bfloat16), out.stride(0), rows, q_heads, kv.kv_heads, kv.head_dim,
                                           kv.page_tokens, mbps, max_ctx, scale, _p(scratch), _s()), "wkb_paged_attn_decode_int8")
    return out
