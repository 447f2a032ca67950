"""GPU parity of the int8 KV cache: the append quantizer is bit-exact against the reference's quantizer restated in
numpy (bytes and scales); decode attention over the int8 cache is within rtol 1e-4 of the oracle's float64 attention
over the dequantized cache (int8 * scale, exact in f32)."""
import math

import numpy as np
import pytest

from oracle import kv_int8 as Q

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from wukong_b200 import _lib, device
    _lib.require_gpu()
    return device


@pytest.mark.parametrize("q_heads,kv_heads,hd,ctx", [(12, 12, 64, [5, 300, 0, 17, 640, 256, 257]), (32, 8, 128, [128, 1000, 33, 0]),
                                                     (8, 4, 64, [31, 32, 33, 511]), (8, 2, 128, [600, 1]), (4, 4, 128, [77])])
def test_int8_append_and_decode(dev, orc, q_heads, kv_heads, hd, ctx):
    import torch
    from wukong_b200.paged import BlockManager
    rng = np.random.default_rng(3)
    slots, page, mbps = len(ctx), 16, 64
    nblk = sum((c + page - 1) // page for c in ctx) + 7
    kflat = [(rng.standard_normal((c, kv_heads, hd)) * rng.uniform(0.1, 4.0, (c, kv_heads, 1))).astype(np.float32) for c in ctx]
    vflat = [(rng.standard_normal((c, kv_heads, hd)) * rng.uniform(0.1, 4.0, (c, kv_heads, 1))).astype(np.float32) for c in ctx]
    for s in range(slots):
        if ctx[s] > 2:
            kflat[s][1, 0] = 0.0            # an all-zero row: scale 1
            vflat[s][2] *= 1e-30            # tiny values
    q = rng.standard_normal((slots, q_heads * hd)).astype(np.float32)
    scale = 1.0 / math.sqrt(hd)
    outs = []
    for perm_seed in (0, 1):
        mgr = BlockManager(nblk, page, slots, mbps)
        if perm_seed:
            mgr.reserve(slots - 1, 16 * 3); mgr.free(slots - 1)
        for s in np.random.default_rng(perm_seed).permutation(slots):
            if ctx[s]:
                mgr.reserve(int(s), int(ctx[s]))
        table = mgr.flat_block_table()
        bt = torch.from_numpy(table.astype(np.int64)).to(torch.int32).cuda()
        kv = dev.PagedKVInt8(1, nblk, kv_heads, hd, page)
        for s in range(slots):
            if not ctx[s]:
                continue
            src = torch.from_numpy(np.concatenate([kflat[s].reshape(ctx[s], -1), vflat[s].reshape(ctx[s], -1)], 1)).cuda()
            dev.paged_kv_append_int8(kv, 0, src, src[:, kv_heads * hd:], src.stride(0), bt, torch.full((ctx[s],), s, dtype=torch.int32, device="cuda"),
                                     torch.arange(ctx[s], dtype=torch.int32, device="cuda"), ctx[s], mbps)
        junk = torch.full((1, 2 * kv_heads * hd), 1e9, device="cuda")      # an inactive row writes nothing
        dev.paged_kv_append_int8(kv, 0, junk, junk[:, kv_heads * hd:], junk.stride(0), bt, torch.zeros(1, dtype=torch.int32, device="cuda"),
                                 torch.full((1,), -1, dtype=torch.int32, device="cuda"), 1, mbps)
        kq, vq = kv.k[0].cpu().numpy(), kv.v[0].cpu().numpy()
        ks, vs = kv.k_scale[0].cpu().numpy(), kv.v_scale[0].cpu().numpy()
        # every cached byte and scale is the reference quantizer's
        for s in range(slots):
            if not ctx[s]:
                continue
            wq, ws = Q.quantize_kv_int8(kflat[s])
            wvq, wvs = Q.quantize_kv_int8(vflat[s])
            t = np.arange(ctx[s])
            pages, offs = table[s, t // page], t % page
            assert np.array_equal(kq[pages, :, offs, :], wq) and np.array_equal(ks[pages, :, offs].view(np.uint32), ws.view(np.uint32))
            assert np.array_equal(vq[pages, :, offs, :], wvq) and np.array_equal(vs[pages, :, offs].view(np.uint32), wvs.view(np.uint32))
        row_slot = torch.arange(slots, dtype=torch.int32, device="cuda")
        row_ctx = torch.tensor(ctx, dtype=torch.int32, device="cuda")
        scratch = dev.paged_attn_scratch(slots, q_heads, hd, max(ctx))
        out = torch.empty((slots, q_heads * hd), dtype=torch.float32, device="cuda")
        dev.paged_attn_decode_int8(torch.from_numpy(q).cuda(), q_heads * hd, kv, 0, bt, row_slot, row_ctx, out, slots, q_heads, mbps,
                                   max(ctx), scale, scratch)
        outs.append(out.cpu().numpy())
        ref = orc.paged_attn_decode(q, Q.dequantize(kq, ks), Q.dequantize(vq, vs), 0, table, ctx, slots, q_heads, kv_heads, hd, page, mbps,
                                    scale, layout=1)
        mag = orc.paged_attn_decode(q, Q.dequantize(kq, ks), np.abs(Q.dequantize(vq, vs)), 0, table, ctx, slots, q_heads, kv_heads, hd,
                                    page, mbps, scale, layout=1)
        assert np.all(np.abs(outs[-1] - ref) <= 1e-4 * mag + 1e-6), (np.abs(outs[-1] - ref) / (mag + 1e-9)).max()
    assert outs[0].tobytes() == outs[1].tobytes(), "decode output depends on the physical page layout"
    for s in range(slots):
        if ctx[s] == 0:
            assert (outs[0][s] == 0).all()
    assert not np.isnan(outs[0]).any()
    # the quantization itself stays inside half a step per element
    for s in range(slots):
        if ctx[s]:
            wq, ws = Q.quantize_kv_int8(kflat[s])
            assert np.all(np.abs(Q.dequantize(wq, ws) - kflat[s]) <= 0.5 * ws[..., None] * (1 + 1e-4))
