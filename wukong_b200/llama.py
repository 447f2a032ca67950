"""Llama-shape decode block stack with Q4_0 weights, tensor-parallel over the GPUs of one node.

What runs per decode step and layer on each rank (all kernels are this library's; torch supplies device
memory, streams, graph capture and the process group):

    RMSNorm (fused with the previous residual add)            wkb_add_rmsnorm_bf16
    fused QKV projection, W4A16 on the tensor cores            wkb_gemm_q4_0_bf16_nt
    RoPE on q / k at the rows' positions + K / V append       wkb_rope_qk_paged_append
    paged GQA decode attention                                 wkb_paged_attn_decode
    output projection (this rank's K slice)                    wkb_gemm_q4_0_bf16_nt
    -- sum over ranks --
    residual add + RMSNorm                                     wkb_add_rmsnorm_bf16
    gate / up projection with the SwiGLU epilogue              wkb_gemm_q4_0_bf16_nt (mode 2)
    down projection (this rank's K slice)                      wkb_gemm_q4_0_bf16_nt
    -- sum over ranks --

The split is the one the reference validates on one GPU (crates/wukong_codegen_gpu/src/serving.rs:
4161-4240): QKV, gate / up and the LM head are split by output rows (whole heads, FFN columns,
vocabulary rows), O and down by input columns on Q4_0 block boundaries; the KV cache holds only this
rank's KV heads; norms and the residual stream are replicated.  Greedy sampling over a split
vocabulary gathers each rank's (value, index) candidate and applies the arg-max rule across ranks.
"""
import math

import numpy as np
import torch

from . import device as dev
from ._lib import lib, check


class LlamaConfig:
    def __init__(self, n_layer=32, d_model=4096, n_head=32, n_kv_head=8, d_ff=11008, vocab=32000, rope_base=10000.0, eps=1e-5):
        self.n_layer, self.d_model, self.n_head, self.n_kv_head = n_layer, d_model, n_head, n_kv_head
        self.d_ff, self.vocab, self.rope_base, self.eps = d_ff, vocab, rope_base, eps
        self.head_dim = d_model // n_head
        if self.head_dim not in (64, 128) or d_model % 32 or d_ff % 32:
            raise ValueError("head_dim must be 64 or 128; d_model and d_ff multiples of 32")

    def check_world(self, world):
        if self.n_kv_head % world or self.n_head % world or self.vocab % world or (self.d_ff // 32) % world:
            raise ValueError("heads, vocabulary and FFN blocks must divide by the tensor-parallel degree")

    def linear_params(self):
        d, hd = self.d_model, self.head_dim
        return self.n_layer * (2 * d * self.n_head * hd + 2 * d * self.n_kv_head * hd + 3 * d * self.d_ff)


def llama_config_from_gguf(path):
    """The block-stack shape from a GGUF file's `llama.*` metadata and its embedding table."""
    from . import model_io as io
    need = lambda key: io.gguf_meta_i64(path, key, 0, -1)
    n_layer, d, heads, ff = (need("llama." + k) for k in ("block_count", "embedding_length", "attention.head_count", "feed_forward_length"))
    if min(n_layer, d, heads, ff) <= 0:
        raise io.ModelIOError(-5, "llama.* metadata of %r" % path)
    kv = io.gguf_meta_i64(path, "llama.attention.head_count_kv", 0, heads)
    vocab = io.gguf_dim(path, "token_embd.weight", 0)
    if vocab < 0:
        raise io.ModelIOError(vocab, "token_embd.weight")
    return LlamaConfig(n_layer, d, heads, kv, ff, vocab, io.gguf_meta_f64(path, "llama.rope.freq_base", 0, 10000.0),
                       io.gguf_meta_f64(path, "llama.attention.layer_norm_rms_epsilon", 0, 1e-5))


def synth_q4_raw(rng, n, k, sigma=0.02):
    """Raw Q4_0 rows [n, k/32, 18]: uniform nibbles, f16 scale |N(0, sigma)|."""
    nb = k // 32
    raw = rng.integers(0, 256, (n, nb, 18), dtype=np.uint8)
    sc = np.abs(rng.standard_normal((n, nb)) * sigma).astype(np.float16).view(np.uint16)
    raw[:, :, 0] = (sc & 0xFF).astype(np.uint8)
    raw[:, :, 1] = (sc >> 8).astype(np.uint8)
    return raw


def synth_llama_raw(cfg, seed=0, sigma=0.02):
    """Host-side seeded weights for small configurations (the oracle consumes the same arrays).  `sigma` is the
    spread of the block scales: 0.02 is the benchmark's; a small model wants less, or its random attention and
    SwiGLU saturate and amplify any rounding difference between two implementations."""
    rng = np.random.default_rng(seed)
    d, hd, F = cfg.d_model, cfg.head_dim, cfg.d_ff
    q4 = lambda n, k: synth_q4_raw(rng, n, k, sigma)
    w = {"embed": rng.standard_normal((cfg.vocab, d)).astype(np.float32), "norm_f": np.ones(d, np.float32),
         "lm_head": q4(cfg.vocab, d), "layers": []}
    for _ in range(cfg.n_layer):
        w["layers"].append(dict(norm1=np.ones(d, np.float32), norm2=np.ones(d, np.float32), wq=q4(cfg.n_head * hd, d),
                                wk=q4(cfg.n_kv_head * hd, d), wv=q4(cfg.n_kv_head * hd, d), wo=q4(d, cfg.n_head * hd),
                                wgate=q4(F, d), wup=q4(F, d), wdown=q4(d, F)))
    return w


def shard_rows(raw, rank, world):
    n = raw.shape[0] // world
    return raw[rank * n:(rank + 1) * n]


def shard_cols(raw, rank, world):
    nb = raw.shape[1] // world
    return raw[:, rank * nb:(rank + 1) * nb]


def interleave_rows(a, b):
    out = np.empty((2 * a.shape[0],) + a.shape[1:], a.dtype)
    out[0::2], out[1::2] = a, b
    return out


class LlamaRankWeights:
    """One rank's resident weights: Q4Weight planes per linear, f32 norm gains and embedding."""

    def __init__(self):
        self.layers, self.embed, self.norm_f, self.lm_head = [], None, None, None

    @staticmethod
    def _q4(raw, device):
        n, nb, _ = raw.shape
        return dev.Q4Weight.from_raw(torch.from_numpy(np.ascontiguousarray(raw).reshape(-1)).to(device), n, nb * 32)

    @staticmethod
    def from_raw(cfg, w, rank=0, world=1, device="cuda"):
        cfg.check_world(world)
        out = LlamaRankWeights()
        f32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(device)
        out.embed, out.norm_f = f32(w["embed"]), f32(w["norm_f"])
        out.lm_head = LlamaRankWeights._q4(shard_rows(w["lm_head"], rank, world), device)
        for lw in w["layers"]:
            qkv = np.concatenate([shard_rows(lw["wq"], rank, world), shard_rows(lw["wk"], rank, world), shard_rows(lw["wv"], rank, world)])
            gu = interleave_rows(shard_rows(lw["wgate"], rank, world), shard_rows(lw["wup"], rank, world))
            out.layers.append(dict(norm1=f32(lw["norm1"]), norm2=f32(lw["norm2"]), wqkv=LlamaRankWeights._q4(qkv, device),
                                   wo=LlamaRankWeights._q4(shard_cols(lw["wo"], rank, world), device),
                                   wgu=LlamaRankWeights._q4(gu, device),
                                   wdown=LlamaRankWeights._q4(shard_cols(lw["wdown"], rank, world), device)))
        return out

    @staticmethod
    def synth_device(cfg, rank=0, world=1, seed=0, device="cuda"):
        """Full-size seeded weights generated on the device: every rank draws the same full matrices (same
        generator state) and keeps its own slice, so all tensor-parallel degrees compute one function."""
        cfg.check_world(world)
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        d, hd, F = cfg.d_model, cfg.head_dim, cfg.d_ff

        def full(n, k):
            qs = torch.randint(0, 256, (n, k // 32, 16), dtype=torch.uint8, device=device, generator=g)
            sc = (torch.randn((n, k // 32), device=device, generator=g) * 0.02).abs().to(torch.float16)
            return qs, sc

        def make(qs, sc):
            return dev.Q4Weight.from_planes(qs.contiguous(), sc.contiguous())

        rows = lambda t, n: t[rank * (n // world):(rank + 1) * (n // world)]
        cols = lambda t, nb: t[:, rank * (nb // world):(rank + 1) * (nb // world)]
        out = LlamaRankWeights()
        out.embed = torch.randn((cfg.vocab, d), device=device, generator=g)
        out.norm_f = torch.ones(d, device=device)
        qs, sc = full(cfg.vocab, d)
        out.lm_head = make(rows(qs, cfg.vocab), rows(sc, cfg.vocab))
        for _ in range(cfg.n_layer):
            (q_q, q_s), (k_q, k_s), (v_q, v_s) = full(cfg.n_head * hd, d), full(cfg.n_kv_head * hd, d), full(cfg.n_kv_head * hd, d)
            o_q, o_s = full(d, cfg.n_head * hd)
            (g_q, g_s), (u_q, u_s) = full(F, d), full(F, d)
            d_q, d_s = full(d, F)
            nq, nkv = cfg.n_head * hd, cfg.n_kv_head * hd
            qkv_q = torch.cat([rows(q_q, nq), rows(k_q, nkv), rows(v_q, nkv)])
            qkv_s = torch.cat([rows(q_s, nq), rows(k_s, nkv), rows(v_s, nkv)])
            gu_q = torch.stack([rows(g_q, F), rows(u_q, F)], dim=1).reshape(-1, d // 32, 16)
            gu_s = torch.stack([rows(g_s, F), rows(u_s, F)], dim=1).reshape(-1, d // 32)
            out.layers.append(dict(norm1=torch.ones(d, device=device), norm2=torch.ones(d, device=device),
                                   wqkv=make(qkv_q, qkv_s), wo=make(cols(o_q, nq // 32), cols(o_s, nq // 32)),
                                   wgu=make(gu_q, gu_s), wdown=make(cols(d_q, F // 32), cols(d_s, F // 32))))
        return out

    @staticmethod
    def from_gguf(path, cfg=None, rank=0, world=1, device="cuda", unpermute_qk=False):
        """One rank's weights from a GGUF checkpoint with llama.cpp's tensor names (`token_embd.weight`,
        `blk.N.attn_q.weight` ... `output.weight`).  The linears must be Q4_0: their block rows cross PCIe raw and
        are sliced for this rank and re-tiled on the device; the embedding and the norm gains may be any type the
        reader turns into f32 (dequantized on the GPU).  RoPE here pairs element i with i + head_dim/2; a file whose
        converter re-ordered the Q / K rows for adjacent pairs is restored with `unpermute_qk`."""
        from . import model_io as io
        cfg = cfg or llama_config_from_gguf(path)
        cfg.check_world(world)
        d, hd, F = cfg.d_model, cfg.head_dim, cfg.d_ff

        def f32(name, shape):
            return io.gguf_read_device(path, name, torch.empty(shape, dtype=torch.float32, device=device))

        def raw(name, n, k):
            if io.gguf_type(path, name) != 2:
                raise io.ModelIOError(-3, "gguf tensor %r must be Q4_0 for the W4A16 GEMM" % name)
            t = torch.empty((n, k // 32 * 18), dtype=torch.uint8, device=device)
            return io.gguf_read_device(path, name, t).view(n, k // 32, 18)

        def unpermute(t, heads):
            if not unpermute_qk:
                return t
            n, nb, _ = t.shape
            return t.view(heads, hd // 2, 2, nb, 18).transpose(1, 2).reshape(n, nb, 18)

        rows = lambda t: t[rank * (t.shape[0] // world):(rank + 1) * (t.shape[0] // world)]
        cols = lambda t: t[:, rank * (t.shape[1] // world):(rank + 1) * (t.shape[1] // world)]
        q4 = lambda t: dev.Q4Weight.from_raw(t.contiguous().view(-1), t.shape[0], t.shape[1] * 32)
        out = LlamaRankWeights()
        out.embed, out.norm_f = f32("token_embd.weight", (cfg.vocab, d)), f32("output_norm.weight", (d,))
        head = "output.weight" if io.gguf_find(path, "output.weight") >= 0 else "token_embd.weight"     # tied embeddings
        out.lm_head = q4(rows(raw(head, cfg.vocab, d)))
        for i in range(cfg.n_layer):
            b = "blk.%d." % i
            wq = unpermute(raw(b + "attn_q.weight", cfg.n_head * hd, d), cfg.n_head)
            wk = unpermute(raw(b + "attn_k.weight", cfg.n_kv_head * hd, d), cfg.n_kv_head)
            wv = raw(b + "attn_v.weight", cfg.n_kv_head * hd, d)
            gate, up = rows(raw(b + "ffn_gate.weight", F, d)), rows(raw(b + "ffn_up.weight", F, d))
            out.layers.append(dict(norm1=f32(b + "attn_norm.weight", (d,)), norm2=f32(b + "ffn_norm.weight", (d,)),
                                   wqkv=q4(torch.cat([rows(wq), rows(wk), rows(wv)])),
                                   wo=q4(cols(raw(b + "attn_output.weight", d, cfg.n_head * hd))),
                                   wgu=q4(torch.stack([gate, up], dim=1).reshape(-1, d // 32, 18)),
                                   wdown=q4(cols(raw(b + "ffn_down.weight", d, F)))))
        return out

    def q4_bytes(self):
        """Algorithmic weight bytes one decode step streams on this rank (18 B per 32 weights)."""
        return self.lm_head.weight_bytes() + sum(lw[key].weight_bytes() for lw in self.layers for key in ("wqkv", "wo", "wgu", "wdown"))


class PeerReduce:
    """Peer-memory plumbing of the fused sum-over-ranks + add + RMSNorm kernel (wkb_tp_reduce_add_rmsnorm): every rank
    owns two fp32 partial buffers [rows, cols] and a flag row, exports them with CUDA IPC, and maps its peers'.
    `dist` must be an initialised torch.distributed process group with one rank per GPU of the node."""

    def __init__(self, rank, world, rows, cols, device):
        import ctypes
        import torch.distributed as dist
        L = lib()
        self.rank, self.world = rank, world
        self.part = [torch.zeros((rows, cols), dtype=torch.float32, device=device) for _ in range(2)]
        self.flags = torch.zeros(256, dtype=torch.int32, device=device)
        self.step = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize()
        mine = []
        for t in self.part + [self.flags]:
            handle, off = (ctypes.c_char * 64)(), ctypes.c_int64(0)
            check(L.wkb_ipc_export(t.data_ptr(), handle, ctypes.byref(off)), "wkb_ipc_export")
            mine.append((bytes(handle.raw), int(off.value)))
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        self._mapped = []
        ptrs = [[0] * world for _ in range(3)]
        for r in range(world):
            for b in range(3):
                if r == rank:
                    ptrs[b][r] = (self.part + [self.flags])[b].data_ptr()
                else:
                    handle, off = everyone[r][b]
                    base = L.wkb_ipc_import((ctypes.c_char * 64).from_buffer_copy(handle))
                    if not base:
                        raise RuntimeError("cannot map the buffers of rank %d (CUDA IPC)" % r)
                    self._mapped.append(base)
                    ptrs[b][r] = base + off
        arr = lambda v: (ctypes.c_void_p * world)(*v)
        self.part_ptrs = [arr(ptrs[0]), arr(ptrs[1])]   # by buffer, then by rank
        self.flag_ptrs = arr(ptrs[2])
        dist.barrier()

    def close(self):
        for base in self._mapped:
            lib().wkb_ipc_close(base)
        self._mapped = []


class LlamaDecodeModel:
    """One rank of the tensor-parallel decode model.  The launch sequence lives behind the C ABI (`wkb_llama_step`, cut
    into phases at the sums over ranks); this class owns the device memory and drives the phases.  `forward(n)` runs rows
    0..n-1 of the row vectors (token, position, visible keys, slot); `reduce(t)` must sum `t` over the ranks in place
    (None: one rank); `gather(pairs, all_pairs)` must gather the ranks' arg-max candidates (None: one rank); `peer`
    (a PeerReduce) selects the library's fused peer-memory reduce instead of `reduce`."""

    def __init__(self, cfg, weights, rank, world, bcap, num_pages, max_blocks_per_seq, page_tokens=16, device="cuda",
                 reduce=None, gather=None, peer=None):
        import ctypes
        cfg.check_world(world)
        self.cfg, self.w, self.rank, self.world, self.bcap, self.device = cfg, weights, rank, world, bcap, device
        self.reduce, self.gather, self.peer = reduce, gather, peer
        self.page_tokens, self.mbps, self.max_ctx = page_tokens, max_blocks_per_seq, max_blocks_per_seq * page_tokens
        d, hd, R = cfg.d_model, cfg.head_dim, bcap
        self.hq, self.hkv, self.f = cfg.n_head // world, cfg.n_kv_head // world, cfg.d_ff // world
        self.vloc = cfg.vocab // world
        self.qkv_w = (self.hq + 2 * self.hkv) * hd
        self.kv = dev.PagedKV(cfg.n_layer, num_pages, self.hkv, hd, page_tokens, device)
        i32 = dict(dtype=torch.int32, device=device)
        self.rows = torch.zeros(4 * R, **i32)            # token | position | visible keys | slot
        self.rows[R:2 * R] = -1
        self.rows[3 * R:] = torch.arange(R, **i32)
        self.row_token, self.row_pos, self.row_ctx, self.row_slot = (self.rows[i * R:(i + 1) * R] for i in range(4))
        self.block_table = torch.zeros((bcap, max_blocks_per_seq), **i32)
        self.next_tok = torch.zeros(R, **i32)
        half = hd // 2
        inv = 1.0 / (np.float32(cfg.rope_base) ** (np.arange(half, dtype=np.float32) * np.float32(2.0 / hd)))
        self.inv_freq = torch.from_numpy(inv.astype(np.float32)).to(device)
        dims = [cfg.n_layer, d, cfg.n_head, cfg.n_kv_head, cfg.d_ff, cfg.vocab, rank, world, bcap, num_pages, max_blocks_per_seq, page_tokens,
                int(np.float32(cfg.eps).view(np.uint32))]
        self._dims = (ctypes.c_int64 * len(dims))(*dims)
        self.workspace = torch.zeros(int(lib().wkb_llama_workspace_bytes(self._dims)) + 256, dtype=torch.uint8, device=device)
        pad = (-self.workspace.data_ptr()) % 256
        ptrs = [weights.embed, weights.norm_f, weights.lm_head.tiled, self.inv_freq]
        for lw in weights.layers:
            ptrs += [lw["norm1"], lw["norm2"], lw["wqkv"].tiled, lw["wo"].tiled, lw["wgu"].tiled, lw["wdown"].tiled]
        self._wptrs = (ctypes.c_void_p * len(ptrs))(*[t.data_ptr() for t in ptrs])
        self._h = lib().wkb_llama_new(self._dims, self._wptrs, self.kv.k.data_ptr(), self.kv.v.data_ptr(), self.block_table.data_ptr(),
                                      self.rows.data_ptr(), self.next_tok.data_ptr(), self.workspace[pad:].data_ptr())
        if not self._h:
            raise ValueError("LlamaDecodeModel: geometry refused by wkb_llama_new")
        self.n_phases = int(lib().wkb_llama_num_phases(self._h))

        def view(which, dtype, *shape):
            off = lib().wkb_llama_buffer(self._h, which) - self.workspace.data_ptr()
            n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
            return self.workspace[off:off + n].view(dtype).view(*shape)
        f32, bf = torch.float32, torch.bfloat16
        self.x, self.part, self.xn = view(0, f32, R, d), view(1, f32, R, d), view(2, bf, R, d)
        self.qkv, self.att, self.h = view(3, f32, R, self.qkv_w), view(4, bf, R, self.hq * hd), view(5, bf, R, self.f)
        self.logits = view(6, f32, R, self.vloc)
        self.pairs, self.all_pairs = view(7, torch.int32, R, 2), view(8, torch.int32, world, R, 2)
        off = lib().wkb_llama_buffer(self._h, 9) - self.workspace.data_ptr()
        self.scratch = self.workspace[off:off + int(lib().wkb_paged_attn_scratch_bytes(R, self.hq, hd, self.max_ctx))].view(f32)
        # a GEMM workspace of the model's own for callers that time the linears alone (the step uses the arena's)
        ws_bytes = max(int(lib().wkb_gemm_q4_0_workspace_bytes(w.n, w.k))
                       for w in [weights.lm_head] + [lw[k] for lw in weights.layers for k in ("wqkv", "wo", "wgu", "wdown")])
        self.gemm_workspace = torch.zeros(ws_bytes, dtype=torch.uint8, device=device)
        self.scale = 1.0 / math.sqrt(hd)
        self.launches_per_forward = 0
        self._tiles = None
        if peer is not None:
            check(lib().wkb_llama_set_peer(self._h, peer.part_ptrs[0], peer.part_ptrs[1], peer.flag_ptrs, peer.step.data_ptr()), "wkb_llama_set_peer")
        # one rank, at most 64 rows: the split-K second passes are folded into the kernels that consume the results
        self.fold_slices = world == 1 and peer is None and bcap <= 64

    def __del__(self):
        if getattr(self, "_h", None):
            lib().wkb_llama_delete(self._h)
            self._h = None

    def _gemm(self, w, x, ldx, out, ldo, mode, n, what):
        p = lambda t: t.data_ptr()
        check(lib().wkb_gemm_q4_0_bf16_nt(p(w.tiled), p(x), ldx, p(out), ldo, mode, n, w.n, w.k, p(self.gemm_workspace),
                                          self.gemm_workspace.numel(), torch.cuda.current_stream().cuda_stream), what)

    def set_prefill_rows(self, row_slot_host):
        """Chunked prefill: the step's rows are laid out sequence by sequence (several consecutive positions of a
        sequence per step, at most `bcap` rows in all); `row_slot_host` is the host copy of row_slot for the live rows.
        Attention then runs on the tiled prefill kernel.  Pass None to go back to one row per sequence."""
        if row_slot_host is None:
            self._tiles = None
            check(lib().wkb_llama_set_prefill_tiles(self._h, None, 0), "wkb_llama_set_prefill_tiles")
            return
        tile_rows = int(lib().wkb_paged_attn_prefill_tile_rows(self.hq, self.hkv))
        tiles = dev.prefill_tiles(np.asarray(row_slot_host, np.int32), tile_rows)
        self._tiles = torch.from_numpy(tiles).to(self.block_table.device)
        check(lib().wkb_llama_set_prefill_tiles(self._h, self._tiles.data_ptr(), self._tiles.shape[0]), "wkb_llama_set_prefill_tiles")

    def _phases(self, n, a, b):
        check(lib().wkb_llama_step(self._h, n, a, b, torch.cuda.current_stream().cuda_stream), "wkb_llama_step")

    # ---- phases (a caller that emulates several ranks on one device runs them in lockstep) ----
    def begin(self, n):
        self._phases(n, 0, 1)

    def attn_part(self, li, n):
        self._phases(n, 1 + 4 * li, 2 + 4 * li)

    def after_attn(self, li, n):
        self._phases(n, 2 + 4 * li, 3 + 4 * li)

    def mlp_part(self, li, n):
        self._phases(n, 3 + 4 * li, 4 + 4 * li)

    def after_mlp(self, li, n):
        self._phases(n, 4 + 4 * li, 5 + 4 * li)

    def head_local(self, n):
        self._phases(n, self.n_phases - 2, self.n_phases - 1)

    def head_pick(self, n):
        self._phases(n, self.n_phases - 1, self.n_phases)

    def forward(self, n):
        P = self.n_phases
        if self.reduce is None or self.peer is not None:
            self._phases(n, 0, P - 1)                  # no host-side sum: everything up to the pairs in one call
        else:
            self.begin(n)
            for li in range(self.cfg.n_layer):
                self.attn_part(li, n)
                self.reduce(self.part)
                self.after_attn(li, n)
                self.mlp_part(li, n)
                self.reduce(self.part)
                self.after_mlp(li, n)
            self.head_local(n)
        if self.gather is not None:
            self.gather(self.pairs, self.all_pairs)
        else:
            self.all_pairs[0].copy_(self.pairs)
        self.head_pick(n)
        self.launches_per_forward = int(lib().wkb_llama_launches(self._h)) + (0 if self.gather is not None else 1)
        return self.next_tok

    def advance(self, n):
        """Device-side feedback between decode steps: the sampled token becomes the next input, positions and
        visible-key counts move on by one."""
        check(lib().wkb_llama_advance(self._h, n, torch.cuda.current_stream().cuda_stream), "wkb_llama_advance")


class LocalTensorParallel:
    """All ranks of a tensor-parallel group on ONE device, run in lockstep with the sums done in rank order.
    It exists to check the sharded model against the unsharded one where only one GPU is at hand; the
    multi-process path uses LlamaDecodeModel with a process-group reduce."""

    def __init__(self, cfg, host_weights, world, bcap, num_pages, max_blocks_per_seq, page_tokens=16, device="cuda"):
        self.world = world
        self.models = [LlamaDecodeModel(cfg, LlamaRankWeights.from_raw(cfg, host_weights, r, world, device), r, world, bcap, num_pages,
                                        max_blocks_per_seq, page_tokens, device) for r in range(world)]

    def _sum_parts(self, n):
        m0 = self.models[0]
        s = torch.cuda.current_stream().cuda_stream
        cnt = n * m0.cfg.d_model
        for m in self.models[1:]:
            check(lib().wkb_add_f32(m0.part.data_ptr(), m.part.data_ptr(), m0.part.data_ptr(), cnt, s), "sum")
        for m in self.models[1:]:
            m.part.copy_(m0.part)

    def set_rows(self, token, pos, slot, ctx, block_table):
        for m in self.models:
            m.row_token.copy_(token); m.row_pos.copy_(pos); m.row_slot.copy_(slot); m.row_ctx.copy_(ctx)
            m.block_table.copy_(block_table)

    def forward(self, n):
        ms = self.models
        for m in ms:
            m.begin(n)
        for li in range(ms[0].cfg.n_layer):
            for m in ms:
                m.attn_part(li, n)
            self._sum_parts(n)
            for m in ms:
                m.after_attn(li, n)
                m.mlp_part(li, n)
            self._sum_parts(n)
            for m in ms:
                m.after_mlp(li, n)
        for m in ms:
            m.head_local(n)
        for r, m in enumerate(ms):
            ms[0].all_pairs[r].copy_(m.pairs)
        ms[0].head_pick(n)
        return ms[0].next_tok


class DecodeStepRunner:
    """One decode step as CUDA-graph replays.  With one rank the whole step (optionally with the on-device
    feedback) is a single graph.  With several ranks the step is cut at the collectives: every run of kernels
    between two sums over ranks is one graph, and the process-group calls are issued between the replays on the
    same stream (no collective is recorded inside a graph)."""

    def __init__(self, model, n, stream, with_advance=False):
        self.m, self.n, self.stream, self.with_advance = model, n, stream, with_advance
        m, L = model, model.cfg.n_layer
        self.segments = []
        if m.world == 1:
            def whole():
                m.forward(n)
                if with_advance:
                    m.advance(n)
            self.segments.append(self._capture(whole))
            return

        if m.peer is not None:
            def body():
                m._phases(n, 0, m.n_phases - 1)
            self.segments.append(self._capture(body))

            def tail():
                m.head_pick(n)
                if with_advance:
                    m.advance(n)
            self.segments.append(self._capture(tail))
            return

        def first():
            m.begin(n)
            m.attn_part(0, n)
        self.segments.append(self._capture(first))
        for li in range(L):
            def mid(li=li):
                m.after_attn(li, n)
                m.mlp_part(li, n)
            self.segments.append(self._capture(mid))

            def nxt(li=li):
                m.after_mlp(li, n)
                if li + 1 < L:
                    m.attn_part(li + 1, n)
                else:
                    m.head_local(n)
            self.segments.append(self._capture(nxt))

        def last():
            m.head_pick(n)
            if with_advance:
                m.advance(n)
        self.segments.append(self._capture(last))

    def _capture(self, fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=self.stream):
            fn()
        return g

    def run(self):
        """Enqueue one step on the current stream (the caller makes `stream` current)."""
        m = self.m
        if m.world == 1:
            self.segments[0].replay()
            return
        segs = self.segments
        if m.peer is not None:
            segs[0].replay()
            m.gather(m.pairs, m.all_pairs)
            segs[1].replay()
            return
        segs[0].replay()
        for i in range(1, len(segs) - 1):
            m.reduce(m.part)
            segs[i].replay()
        m.gather(m.pairs, m.all_pairs)
        segs[-1].replay()
