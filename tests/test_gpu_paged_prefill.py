"""GPU parity of the paged prefill attention (prompt chunks against the paged bf16 cache, causal, GQA).

Bar: the tensor-core recipe of the decode path at head_dim 128 -- the softmax weights are rounded to bf16 (2^-9
relative each, in the numerator and in the normaliser), so |out - ref| <= 2 * 2^-9 * sum_i p_i |v_i| per element;
the bound's right-hand side comes from the oracle's float64 attention run on |V|.  The reference is that oracle
over the same cached bf16 keys and values; the row-per-token decode kernel of this library is a second witness."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from wukong_b200 import _lib, device
    _lib.require_gpu()
    return device


def run_case(dev, orc, q_heads, kv_heads, hd, hist, chunk, seed, ragged=False):
    import torch
    from wukong_b200._lib import lib
    from wukong_b200.paged import BlockManager
    rng = np.random.default_rng(seed)
    slots, page, mbps = len(hist), 16, 80
    total = [h + c for h, c in zip(hist, chunk)]
    nblk = sum((c + page - 1) // page for c in total) + 5
    mgr = BlockManager(nblk, page, slots, mbps)
    for s in np.random.default_rng(seed + 1).permutation(slots):
        if total[s]:
            mgr.reserve(int(s), int(total[s]))
    table = mgr.flat_block_table()
    bt = torch.from_numpy(table.astype(np.int64)).to(torch.int32).cuda()
    kv = dev.PagedKV(1, nblk, kv_heads, hd, page)
    kv.k.fill_(float("nan")); kv.v.fill_(float("nan"))
    for s in range(slots):
        if not total[s]:
            continue
        src = torch.from_numpy(rng.standard_normal((total[s], 2 * kv_heads * hd)).astype(np.float32)).cuda()
        dev.paged_kv_append(kv, 0, src, src[:, kv_heads * hd:], src.stride(0), bt, torch.full((total[s],), s, dtype=torch.int32, device="cuda"),
                            torch.arange(total[s], dtype=torch.int32, device="cuda"), total[s], mbps)
    row_slot = np.concatenate([np.full(c, s, np.int32) for s, c in enumerate(chunk)])
    row_ctx = np.concatenate([np.arange(h + 1, h + c + 1, dtype=np.int32) for h, c in zip(hist, chunk)])
    if ragged:       # visible-key counts need not be consecutive, a row may see nothing
        row_ctx = np.maximum(0, row_ctx - rng.integers(0, 40, row_ctx.shape[0])).astype(np.int32)
        row_ctx[::7] = 0
    rows = row_slot.shape[0]
    q = rng.standard_normal((rows, q_heads * hd)).astype(np.float32)
    scale = 1.0 / math.sqrt(hd)
    tile_rows = int(lib().wkb_paged_attn_prefill_tile_rows(q_heads, kv_heads))
    assert tile_rows == 128 // (q_heads // kv_heads)
    tiles = dev.prefill_tiles(row_slot, tile_rows)
    assert tiles[:, 1].sum() == rows and tiles[:, 1].max() <= tile_rows
    dq, drs, drc, dt = (torch.from_numpy(a).cuda() for a in (q, row_slot, row_ctx, tiles))
    out = torch.full((rows, q_heads * hd), 7.0, device="cuda")
    dev.paged_attn_prefill(dq, q_heads * hd, kv, 0, bt, drs, drc, dt, out, q_heads, mbps, scale)
    got = out.cpu().numpy()
    kbits = kv.k[0].view(torch.int16).cpu().numpy().view(np.uint16)
    vbits = kv.v[0].view(torch.int16).cpu().numpy().view(np.uint16)
    ref = orc.paged_attn_decode(q, kbits, vbits, 1, np.ascontiguousarray(table[row_slot]), [int(c) for c in row_ctx], rows, q_heads, kv_heads,
                                hd, page, mbps, scale, layout=1)
    seen = row_ctx > 0
    assert (got[~seen] == 7.0).all(), "a row that sees no key is not written"
    assert not np.isnan(got).any()
    mag = orc.paged_attn_decode(q, kbits, vbits & 0x7FFF, 1, np.ascontiguousarray(table[row_slot]), [int(c) for c in row_ctx], rows, q_heads,
                                kv_heads, hd, page, mbps, scale, layout=1)
    err = np.abs(got[seen] - ref[seen])
    assert np.all(err <= 2.0 ** -8 * mag[seen] + 1e-5), (err / (mag[seen] + 1e-9)).max()
    # the row-per-token kernel on the same rows
    if not (hd == 64 and q_heads // kv_heads == 8):      # a group of 8 at head_dim 64 exists only in the tiled kernel
        scratch = dev.paged_attn_scratch(rows, q_heads, hd, int(max(total)))
        dec = torch.empty((rows, q_heads * hd), device="cuda")
        dev.paged_attn_decode(dq, q_heads * hd, kv, 0, bt, drs, drc, dec, rows, q_heads, mbps, int(max(total)), scale, scratch)
        assert np.all(np.abs(got[seen] - dec.cpu().numpy()[seen]) <= 2.0 ** -7 * mag[seen] + 1e-5)
    # bf16 output = the rounding of the f32 output
    outb = torch.zeros((rows, q_heads * hd), dtype=torch.bfloat16, device="cuda")
    dev.paged_attn_prefill(dq, q_heads * hd, kv, 0, bt, drs, drc, dt, outb, q_heads, mbps, scale)
    gb = outb.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(gb[seen], orc.to_bf16_bits(got[seen].reshape(-1)).reshape(gb[seen].shape))
    # a different physical page layout of the same history gives the same bits
    return got


@pytest.mark.parametrize("q_heads,kv_heads,hd", [(12, 12, 64), (8, 4, 64), (8, 2, 64), (8, 1, 64), (4, 4, 128), (8, 4, 128), (32, 8, 128), (8, 1, 128)])
def test_prefill_matches_oracle(dev, orc, q_heads, kv_heads, hd):
    run_case(dev, orc, q_heads, kv_heads, hd, hist=[0, 37, 256, 0, 1000], chunk=[33, 16, 70, 1, 5], seed=q_heads + hd)


def test_prefill_ragged_visible_counts(dev, orc):
    run_case(dev, orc, 12, 12, 64, hist=[100, 3, 0], chunk=[50, 21, 9], seed=5, ragged=True)
    run_case(dev, orc, 32, 8, 128, hist=[100, 3, 0], chunk=[50, 21, 9], seed=6, ragged=True)

