"""Host-side page allocator and continuous-batching scheduler (ctypes over the C++ implementation).

Class and method names follow the reference's `BlockManager` (crates/wukong_codegen_gpu/src/
paged_kv.rs:428-628) and `Scheduler` (serving.rs:1346-1595); `OutOfBlocks` is raised where the
reference returns `Err(OutOfBlocks)`.
"""
import ctypes as C

import numpy as np

from ._lib import lib, vp


class OutOfBlocks(RuntimeError):
    pass


class BlockManager:
    def __init__(self, num_blocks, block_size, num_slots, max_blocks_per_seq, _handle=None):
        self._own = _handle is None
        self._h = _handle or lib().wkb_blockmgr_new(num_blocks, block_size, num_slots, max_blocks_per_seq)
        if not self._h:
            raise ValueError("BlockManager: every extent must be positive")
        self.block_size, self.num_blocks, self.num_slots, self.max_blocks_per_seq = block_size, num_blocks, num_slots, max_blocks_per_seq

    def __del__(self):
        if getattr(self, "_own", False) and self._h:
            lib().wkb_blockmgr_delete(self._h)
            self._h = None

    def append(self, slot):
        phys, off = C.c_uint32(), C.c_int64()
        if lib().wkb_blockmgr_append(self._h, slot, C.byref(phys), C.byref(off)) != 0:
            raise OutOfBlocks()
        return phys.value, off.value

    def reserve(self, slot, tokens):
        start = lib().wkb_blockmgr_reserve(self._h, slot, tokens)
        if start < 0:
            raise OutOfBlocks()
        return start

    def free(self, slot):
        lib().wkb_blockmgr_release(self._h, slot)

    def can_grow(self, slot, tokens):
        return bool(lib().wkb_blockmgr_can_grow(self._h, slot, tokens))

    def free_blocks(self):
        return lib().wkb_blockmgr_free_blocks(self._h)

    def used_blocks(self):
        return lib().wkb_blockmgr_used_blocks(self._h)

    def context_len(self, slot):
        return lib().wkb_blockmgr_context_len(self._h, slot)

    def layout_epoch(self):
        return lib().wkb_blockmgr_layout_epoch(self._h)

    def locate(self, slot, pos):
        phys, off = C.c_uint32(), C.c_int64()
        if lib().wkb_blockmgr_locate(self._h, slot, pos, C.byref(phys), C.byref(off)) != 0:
            raise IndexError(pos)
        return phys.value, off.value

    def flat_block_table(self, out=None):
        out = np.empty((self.num_slots, self.max_blocks_per_seq), np.uint32) if out is None else out
        lib().wkb_blockmgr_flat_table(self._h, out.ctypes.data_as(vp))
        return out

    def ctx_lens(self, out=None):
        out = np.empty(self.num_slots, np.int32) if out is None else out
        lib().wkb_blockmgr_ctx_lens(self._h, out.ctypes.data_as(vp))
        return out


class Scheduler:
    """plan_step() -> rows for the model; commit_step(sampled) closes the step."""

    def __init__(self, bcap, num_blocks, block_size, max_blocks_per_seq, max_rows=None, prefill_chunk=256):
        self.bcap = bcap
        self.max_rows = max_rows or bcap
        self._h = lib().wkb_sched_new(bcap, num_blocks, block_size, max_blocks_per_seq, self.max_rows, prefill_chunk)
        if not self._h:
            raise ValueError("Scheduler: bad geometry")
        self.manager = BlockManager(num_blocks, block_size, bcap, max_blocks_per_seq, _handle=lib().wkb_sched_blockmgr(self._h))
        self.row_token = np.zeros(self.max_rows, np.int32)
        self.row_pos = np.zeros(self.max_rows, np.int32)
        self.row_slot = np.zeros(self.max_rows, np.int32)
        self.row_ctx = np.zeros(self.max_rows, np.int32)
        self.sample_row = np.full(bcap, -1, np.int32)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().wkb_sched_delete(self._h)
            self._h = None

    def enqueue(self, prompt, gen_len):
        p = np.ascontiguousarray(prompt, np.int32)
        rid = lib().wkb_sched_enqueue(self._h, p.ctypes.data_as(vp), p.size, gen_len)
        if rid < 0:
            raise ValueError("request does not fit a block-table row" if rid == -2 else "empty prompt or gen_len")
        return rid

    def plan_step(self):
        n = lib().wkb_sched_plan_step(self._h, *(a.ctypes.data_as(vp) for a in
                                                (self.row_token, self.row_pos, self.row_slot, self.row_ctx, self.sample_row)))
        if n == -1:
            raise OutOfBlocks()
        if n < 0:
            raise RuntimeError("plan_step: previous step not committed")
        return n

    def commit_step(self, sampled):
        s = np.ascontiguousarray(sampled, np.int32)
        return lib().wkb_sched_commit_step(self._h, s.ctypes.data_as(vp))

    def output(self, request):
        n = lib().wkb_sched_output_len(self._h, request)
        out = np.empty(max(n, 0), np.int32)
        lib().wkb_sched_output(self._h, request, out.ctypes.data_as(vp), out.size)
        return out

    num_active = lambda self: lib().wkb_sched_num_active(self._h)
    pending = lambda self: lib().wkb_sched_pending(self._h)
    emitted = lambda self: lib().wkb_sched_emitted(self._h)
    admitted = lambda self: lib().wkb_sched_admitted(self._h)
    completed = lambda self: lib().wkb_sched_completed(self._h)
    free_blocks = lambda self: self.manager.free_blocks()
    is_idle = lambda self: bool(lib().wkb_sched_is_idle(self._h))
