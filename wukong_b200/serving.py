"""GPT-2-shape decode serving on device-resident tensors: weights, paged KV, the per-step forward
over a flat batch of rows, and the engine that ties the scheduler to it.

The structure follows the reference's Rust-launched serving stack (crates/wukong_codegen_gpu/src/
serving.rs: `DecodeLayer::forward_step_on` :684-937, `DecodeModel` :942, `Scheduler::step_graphed`
:1536-1575) -- norm -> QKV GEMM -> KV append through the block table -> paged decode attention ->
output projection with fused residual -> norm -> MLP GEMMs with fused activation / residual, the
whole step replayed as one CUDA graph -- widened to a real model: token + position embedding in
front, final norm, tied LM head and greedy arg-max behind (the .wk program this mirrors is
examples/gpt2_generate.wk:137-255 of the reference).

Precision recipe (what "bf16" means here, and what the CPU oracle model in the tests restates):
weights and KV cache bf16; residual stream fp32; every GEMM bf16 x bf16 with fp32 accumulation;
norm outputs, attention outputs and the MLP hidden rounded once to bf16; logits fp32.
torch is used for device memory, streams and graph capture only; every kernel is this library's.
"""
import math

import numpy as np
import torch

from . import device as dev
from ._lib import lib, check
from .paged import Scheduler


class GPT2Config:
    def __init__(self, n_layer=12, d_model=768, n_head=12, d_ff=3072, vocab=50257, n_pos=1024, eps=1e-5):
        self.n_layer, self.d_model, self.n_head, self.d_ff, self.vocab, self.n_pos, self.eps = n_layer, d_model, n_head, d_ff, vocab, n_pos, eps
        self.head_dim = d_model // n_head
        assert self.head_dim in (64, 128) and d_model % 8 == 0 and d_ff % 8 == 0

    def n_params(self):
        d, f = self.d_model, self.d_ff
        return self.vocab * d + self.n_pos * d + self.n_layer * (4 * d * d + 2 * d * f + 9 * d + f) + 2 * d


def _bf16_bits(x):
    """f32 -> bf16 bits, round to nearest even (values here are finite)."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def synth_weights(cfg, seed=0):
    """Seeded stand-in for a checkpoint: every matrix, bias and embedding ~N(0, 0.02), LayerNorm
    gamma = 1, beta = 0.  Returns host arrays: matrices as bf16 bits (uint16), vectors as f32."""
    rng = np.random.default_rng(seed)
    n = lambda *shape: (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
    d, f = cfg.d_model, cfg.d_ff
    w = {"wte": _bf16_bits(n(cfg.vocab, d)), "wpe": _bf16_bits(n(cfg.n_pos, d)), "layers": [],
         "lnf_g": np.ones(d, np.float32), "lnf_b": np.zeros(d, np.float32)}
    for _ in range(cfg.n_layer):
        w["layers"].append({
            "ln1_g": np.ones(d, np.float32), "ln1_b": np.zeros(d, np.float32),
            "w_qkv": _bf16_bits(n(3 * d, d)), "b_qkv": n(3 * d),
            "w_o": _bf16_bits(n(d, d)), "b_o": n(d),
            "ln2_g": np.ones(d, np.float32), "ln2_b": np.zeros(d, np.float32),
            "w_fc": _bf16_bits(n(f, d)), "b_fc": n(f),
            "w_proj": _bf16_bits(n(d, f)), "b_proj": n(d),
        })
    return w


def _to_dev(a, device):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if a.dtype == np.uint16:
        t = torch.from_numpy(np.ascontiguousarray(a).view(np.int16))
        return t.to(device).view(torch.bfloat16)
    return t.to(device)


class DecodeModel:
    """Device-resident GPT-2-shape model over a paged KV cache; `forward(n, n_sample)` runs the first n rows of
    the row vectors (token, position, slot, visible keys) and leaves arg-max tokens in `next_tok`.  The launch sequence
    itself lives behind the C ABI (`wkb_gpt2_step`); this class owns the device memory (torch tensors) and hands the
    library their addresses."""

    def __init__(self, cfg, weights, bcap, num_pages, max_blocks_per_seq, max_rows=None, page_tokens=16, device="cuda"):
        import ctypes
        self.cfg, self.bcap, self.device = cfg, bcap, device
        self.max_rows = max_rows or bcap
        self.page_tokens, self.mbps = page_tokens, max_blocks_per_seq
        self.max_ctx = max_blocks_per_seq * page_tokens
        d, f, R = cfg.d_model, cfg.d_ff, self.max_rows
        self.w = {k: _to_dev(v, device) for k, v in weights.items() if k != "layers"}
        self.layers = [{k: _to_dev(v, device) for k, v in lw.items()} for lw in weights["layers"]]
        self.kv = dev.PagedKV(cfg.n_layer, num_pages, cfg.n_head, cfg.head_dim, page_tokens, device)
        i32 = dict(dtype=torch.int32, device=device)
        self.rows = torch.zeros(8 * R, **i32)
        self.rows[R:2 * R] = -1                                   # every row starts inactive
        self._carve_rows()
        self.tile_rows = int(lib().wkb_paged_attn_prefill_tile_rows(cfg.n_head, cfg.n_head))
        self.block_table = torch.zeros((bcap, max_blocks_per_seq), **i32)
        self.ldl = (cfg.vocab + 7) // 8 * 8                      # logits pitch, 16-byte aligned rows
        self.logits = torch.zeros((bcap, self.ldl), dtype=torch.float32, device=device)
        self.next_tok = torch.zeros(bcap, **i32)
        self.keep_logits = False      # True: materialise fp32 logits (tests); False: arg-max fused into the LM head
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        dims = [cfg.n_layer, d, cfg.n_head, f, cfg.vocab, cfg.n_pos, bcap, R, num_pages, max_blocks_per_seq, page_tokens,
                int(np.float32(cfg.eps).view(np.uint32))]
        self._dims = (ctypes.c_int64 * len(dims))(*dims)
        self.workspace = torch.zeros(int(lib().wkb_gpt2_workspace_bytes(self._dims)) + 256, dtype=torch.uint8, device=device)
        pad = (-self.workspace.data_ptr()) % 256
        ws = self.workspace[pad:]
        ptrs = [self.w["wte"], self.w["wpe"], self.w["lnf_g"], self.w["lnf_b"]]
        for lw in self.layers:
            ptrs += [lw[k] for k in ("ln1_g", "ln1_b", "w_qkv", "b_qkv", "w_o", "b_o", "ln2_g", "ln2_b", "w_fc", "b_fc", "w_proj", "b_proj")]
        self._wptrs = (ctypes.c_void_p * len(ptrs))(*[t.data_ptr() for t in ptrs])
        self._h = lib().wkb_gpt2_new(self._dims, self._wptrs, self.kv.k.data_ptr(), self.kv.v.data_ptr(), self.block_table.data_ptr(),
                                     self.rows.data_ptr(), self.next_tok.data_ptr(), ws.data_ptr(), self.logits.data_ptr(), self.ldl)
        if not self._h:
            raise ValueError("DecodeModel: geometry refused by wkb_gpt2_new")
        # typed views of the activation buffers inside the workspace (tests, the benchmark's kernel timings)
        def view(which, dtype, rows, cols):
            off = lib().wkb_gpt2_buffer(self._h, which) - self.workspace.data_ptr()
            n = rows * cols * torch.empty((), dtype=dtype).element_size()
            return self.workspace[off:off + n].view(dtype).view(rows, cols)
        self.x, self.h = view(0, torch.float32, R, d), view(1, torch.bfloat16, R, d)
        self.q, self.att = view(2, torch.float32, R, d), view(3, torch.bfloat16, R, d)
        self.ff, self.hs = view(4, torch.bfloat16, R, f), view(5, torch.bfloat16, bcap, d)
        self.scratch = dev.paged_attn_scratch(R, cfg.n_head, cfg.head_dim, self.max_ctx, device)   # for callers that time the attention alone
        self.launches_per_forward = 0

    def _carve_rows(self):
        R = self.max_rows
        self.row_token, self.row_pos, self.row_slot, self.row_ctx, self.sample_rows, self.row_ctx_dec = (self.rows[i * R:(i + 1) * R] for i in range(6))
        self.tiles = self.rows[6 * R:8 * R]

    def __del__(self):
        if getattr(self, "_h", None):
            lib().wkb_gpt2_delete(self._h)
            self._h = None

    # -- one forward over the first n rows; n_sample rows (indices in sample_rows) reach the LM head
    def forward(self, n, n_sample, n_tiles=0):
        check(lib().wkb_gpt2_step(self._h, n, n_sample, n_tiles, int(self.keep_logits), torch.cuda.current_stream().cuda_stream), "wkb_gpt2_step")
        self.launches_per_forward = int(lib().wkb_gpt2_launches(self._h))
        return self.next_tok

    def advance(self, n):
        check(lib().wkb_gpt2_advance(self._h, n, torch.cuda.current_stream().cuda_stream), "wkb_gpt2_advance")


class StepTimeout(RuntimeError):
    """A step's device work did not finish within the engine's deadline (the work is still queued)."""


class Engine:
    """Scheduler + model: `step()` = plan rows -> upload them (and the block table when it moved) ->
    forward (one CUDA-graph replay for a decode-only step) -> read the sampled tokens -> commit.
    `step_timeout_ms` puts a host-side deadline on each step's device work (the reference's `sync_within`,
    crates/wukong_codegen_gpu/src/gpu.rs:250-262): when it passes, `step()` raises StepTimeout instead of
    blocking for ever, and the step stays uncommitted."""

    def __init__(self, cfg, weights, bcap, num_pages, max_blocks_per_seq, max_rows=None, prefill_chunk=256, page_tokens=16,
                 device="cuda", use_graph=True, step_timeout_ms=None):
        self.cfg, self.bcap = cfg, bcap
        self.step_timeout_ms = step_timeout_ms
        self.model = DecodeModel(cfg, weights, bcap, num_pages, max_blocks_per_seq, max_rows, page_tokens, device)
        self.sched = Scheduler(bcap, num_pages, page_tokens, max_blocks_per_seq, self.model.max_rows, prefill_chunk)
        R = self.model.max_rows
        pin = lambda n, dt=torch.int32: torch.zeros(n, dtype=dt).pin_memory()
        # one pinned staging block: token | pos | slot | ctx | sample_rows | ctx of the row-per-token kernel | prefill tiles
        self.h_rows = pin(8 * R)
        m = self.model
        self.d_rows = m.rows                   # the model's own row block (the library reads the step's rows from it)
        self.use_prefill_kernel = True
        self.h_table = pin(bcap * max_blocks_per_seq)
        self.h_next = pin(bcap)
        self.uploaded_epoch = -1
        self.use_graph = use_graph
        self.graph = None
        self.stream = torch.cuda.Stream(device=device)
        self.h2d_bytes = self.d2h_bytes = self.kernel_launches = 0
        self._planned = None
        self._pending = None                   # a launched step whose tokens have not been committed yet
        self._sample_rows_identity = False     # device sample_rows currently hold 0..bcap-1 (set by a decode-only step)

    def enqueue(self, prompt, gen_len):
        return self.sched.enqueue(prompt, gen_len)

    def step(self):
        s, m, R = self.sched, self.model, self.model.max_rows
        if self._pending is not None:
            raise RuntimeError("the previous step has not finished: call finish_step()")
        n = self._planned if self._planned is not None else s.plan_step()   # a caller may have planned already
        self._planned = None
        if n == 0:
            return 0
        hr = self.h_rows.numpy()
        # decode-only step: every row is the one sampled row of its slot (one token per sequence)
        decode_only = n <= self.bcap and np.array_equal(s.sample_row[s.row_slot[:n]], np.arange(n, dtype=np.int32))
        # Only the live prefix of each row vector crosses PCIe: U = the rows this step's kernels read (the whole
        # batch capacity on the graph path, whose launches are fixed at bcap rows), rounded up to 64.  Rows between
        # n and U are inactive: they write no KV (pos < 0), see no key (ctx 0) and are never sampled.
        U = min(R, (max(n, self.bcap if decode_only else 0) + 63) // 64 * 64)
        hr[0 * R:0 * R + n] = s.row_token[:n]; hr[0 * R + n:0 * R + U] = 0
        hr[1 * R:1 * R + n] = s.row_pos[:n]; hr[1 * R + n:1 * R + U] = -1
        hr[2 * R:2 * R + n] = s.row_slot[:n]; hr[2 * R + n:2 * R + U] = 0
        hr[3 * R:3 * R + n] = s.row_ctx[:n]; hr[3 * R + n:3 * R + U] = 0
        sampled_slots = np.flatnonzero(s.sample_row >= 0)
        vectors = 4
        if decode_only:
            if not self._sample_rows_identity:               # graph path: the head runs on every decode row
                hr[4 * R:4 * R + self.bcap] = np.arange(self.bcap)
                vectors = 5
        else:
            hr[4 * R:4 * R + sampled_slots.size] = s.sample_row[sampled_slots]
            vectors = 5
        n_tiles = 0
        if not decode_only and self.use_prefill_kernel and m.tile_rows:
            tiles = dev.prefill_tiles(s.row_slot[:n], m.tile_rows, min_run=2)
            n_tiles = tiles.shape[0]
            if n_tiles:
                ctx_dec = s.row_ctx[:n].copy()
                for r0, cnt in tiles:
                    ctx_dec[r0:r0 + cnt] = 0
                hr[5 * R:5 * R + n] = ctx_dec; hr[5 * R + n:5 * R + U] = 0
                hr[6 * R:6 * R + 2 * n_tiles] = tiles.reshape(-1)
                vectors = 6
        with torch.cuda.stream(self.stream):
            check(lib().wkb_upload_rows(self.d_rows.data_ptr(), self.h_rows.data_ptr(), R * 4, U * 4, vectors, self.stream.cuda_stream), "rows")
            self.h2d_bytes += vectors * U * 4
            if n_tiles:
                self.d_rows[6 * R:6 * R + 2 * n_tiles].copy_(self.h_rows[6 * R:6 * R + 2 * n_tiles], non_blocking=True)
                self.h2d_bytes += 2 * n_tiles * 4
            self._sample_rows_identity = decode_only
            ep = s.manager.layout_epoch()
            if ep != self.uploaded_epoch:
                s.manager.flat_block_table(self.h_table.numpy().view(np.uint32).reshape(self.bcap, -1))
                m.block_table.view(-1).copy_(self.h_table, non_blocking=True)
                self.uploaded_epoch = ep
                self.h2d_bytes += self.h_table.numel() * 4
            if decode_only and self.use_graph:
                if self.graph is None:
                    m.forward(self.bcap, self.bcap)          # eager once (also warms every kernel)
                    self.stream.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=self.stream):
                        m.forward(self.bcap, self.bcap)
                    self.graph = g
                    # the eager run already appended this step's K/V rows; replaying rewrites the same values
                self.graph.replay()
                nrows_head = self.bcap
            elif decode_only:
                m.forward(self.bcap, self.bcap)
                nrows_head = self.bcap
            else:
                m.forward(n, max(1, sampled_slots.size), n_tiles)
                nrows_head = sampled_slots.size
            self.kernel_launches += m.launches_per_forward
            self.h_next.copy_(m.next_tok, non_blocking=True)
            self.d2h_bytes += self.bcap * 4
        self._pending = (decode_only, sampled_slots)
        return self.finish_step(self.step_timeout_ms)

    def finish_step(self, timeout_ms=None):
        """Wait for the launched step (for ever, or up to timeout_ms) and commit its tokens.  After a StepTimeout the
        step is still pending: call this again to keep waiting, or give up on the engine."""
        if self._pending is None:
            return 0
        s = self.sched
        if timeout_ms is None:
            self.stream.synchronize()
        else:
            rc = lib().wkb_stream_sync_within(self.stream.cuda_stream, int(timeout_ms))
            if rc == -1:
                raise StepTimeout("decode step still running after %d ms" % timeout_ms)
            check(rc, "step")
        decode_only, sampled_slots = self._pending
        self._pending = None
        nxt = self.h_next.numpy()
        sampled = np.zeros(self.bcap, np.int32)
        if decode_only:
            sampled[sampled_slots] = nxt[s.sample_row[sampled_slots]]
        else:
            sampled[sampled_slots] = nxt[:sampled_slots.size]
        return s.commit_step(sampled)

    def capture_resident_loop(self):
        """A CUDA graph of one decode step that feeds itself: forward over all slots, then the
        sampled tokens become the next inputs on the device.  The caller must have extended every
        slot's block table far enough ahead (BlockManager.reserve) and uploaded it."""
        m = self.model
        def body():
            m.forward(self.bcap, self.bcap)
            m.advance(self.bcap)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self.stream):
            with torch.cuda.graph(g, stream=self.stream):
                body()
        return g

    def run_until_idle(self, max_steps=1 << 30):
        steps = 0
        while not self.sched.is_idle() and steps < max_steps:
            self.step()
            steps += 1
        return steps
