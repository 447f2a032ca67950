"""GPU parity of the half-precision decode kernels: the tcgen05 GEMM, the fast norms, the paged KV
append / decode attention, against the CPU oracle in the same precision recipe."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch
    from wukong_b200 import _lib, device
    _lib.require_gpu()
    return device


def bf16_t(x_np, orc):
    import torch
    return torch.from_numpy(orc.to_bf16_bits(x_np).view(np.int16).reshape(x_np.shape)).cuda().view(torch.bfloat16)


def test_gemm_tc_matches_order_contract_gemm(dev, orc):
    """rtol 2e-2 on logits is the stated bf16 bar; the tensor-core GEMM differs from the
    order-contract GEMM only by fp32 summation order, so the test holds it to 1e-5 * sum|a||b|."""
    import torch
    rng = np.random.default_rng(0)
    for (m, n, k) in [(1, 1, 8), (128, 128, 64), (130, 70, 200), (64, 768, 768), (512, 2304, 768), (33, 1000, 3072),
                      (257, 129, 72), (512, 768, 3072)]:   # the last two K = 3072 shapes take the split-K path
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((n, k)).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
        res = rng.standard_normal((m, n)).astype(np.float32)
        ab, bb = orc.to_bf16_bits(a), orc.to_bf16_bits(b)
        ref = orc.sgemm_half_nt(ab, bb, m, k, n)
        at, bt = bf16_t(a, orc), bf16_t(b, orc)
        c = dev.gemm_bf16_nt(at, bt).cpu().numpy()
        bound = 1e-5 * (np.abs(orc.from_bf16_bits(ab)).reshape(m, k) @ np.abs(orc.from_bf16_bits(bb)).reshape(n, k).T) + 1e-6
        assert (np.abs(c - ref) <= bound).all(), (m, n, k, np.abs(c - ref).max())
        assert np.allclose(c, ref, rtol=2e-2, atol=1e-3)
        for act in (0, 1, 2, 3):
            refe = orc.sgemm_half_nt(ab, bb, m, k, n, bias=bias, act=act) + res
            ce = dev.gemm_bf16_nt(at, bt, bias=torch.from_numpy(bias).cuda(), act=act, residual=torch.from_numpy(res).cuda())
            # the activations are at most 1.13-Lipschitz, so the pre-activation bound carries over
            assert (np.abs(ce.cpu().numpy() - refe) <= 1.2 * bound + 1e-5).all(), (m, n, k, act)
        cb = dev.gemm_bf16_nt(at, bt, bias=torch.from_numpy(bias).cuda(), act=2, out_dtype=torch.bfloat16)
        refb = orc.sgemm_half_nt(ab, bb, m, k, n, bias=bias, act=2)
        got = cb.float().cpu().numpy()
        assert np.allclose(got, refb, rtol=2e-2, atol=2e-2)
    # split-K with the output aliasing the residual (x = x + proj(h)), exact on small integers
    a = torch.randint(-3, 4, (512, 3072), device="cuda").to(torch.bfloat16)
    b = torch.randint(-3, 4, (768, 3072), device="cuda").to(torch.bfloat16)
    xres = torch.randint(-5, 6, (512, 768), device="cuda").float()
    want = a.float() @ b.float().T + xres
    assert torch.equal(dev.gemm_bf16_nt(a, b, residual=xres, out=xres), want)
    assert dev.gemm_status() == 0
    # linearity at a size the oracle does not run: C(a1 + a2) == C(a1) + C(a2) for exactly representable inputs
    a1 = torch.randint(-4, 5, (1024, 4096), device="cuda").to(torch.bfloat16)
    a2 = torch.randint(-4, 5, (1024, 4096), device="cuda").to(torch.bfloat16)
    b = torch.randint(-4, 5, (2048, 4096), device="cuda").to(torch.bfloat16)
    c12 = dev.gemm_bf16_nt((a1 + a2), b)
    assert torch.equal(c12, dev.gemm_bf16_nt(a1, b) + dev.gemm_bf16_nt(a2, b))  # integers: exact in fp32
    assert torch.equal(c12, (a1 + a2).float() @ b.float().T)
    assert dev.gemm_status() == 0
    # a shape large enough for the 128 x 256 tile variant (ragged in M and N), exact on small integers
    a = torch.randint(-3, 4, (2100, 512), device="cuda").to(torch.bfloat16)
    b = torch.randint(-3, 4, (8200, 512), device="cuda").to(torch.bfloat16)
    bias = torch.randint(-5, 6, (8200,), device="cuda").float()
    res = torch.randint(-5, 6, (2100, 8200), device="cuda").float()
    want = torch.relu(a.float() @ b.float().T + bias) + res
    assert torch.equal(dev.gemm_bf16_nt(a, b, bias=bias, act=1, residual=res), want)
    assert torch.equal(dev.gemm_bf16_nt(a, b, bias=bias, act=1, residual=res, out_dtype=torch.bfloat16).float(), want.to(torch.bfloat16).float())
    assert dev.gemm_status() == 0


def test_gemm_fused_argmax_equals_argmax_of_logits(dev, orc):
    import torch
    from wukong_b200 import lib
    rng = np.random.default_rng(3)
    for (m, n, k) in [(5, 1000, 64), (130, 50257, 768), (512, 300, 128)]:
        a = bf16_t(rng.standard_normal((m, k)).astype(np.float32), orc)
        b = bf16_t(rng.standard_normal((n, k)).astype(np.float32), orc)
        b[7] = b[3]                      # an exact tie between two columns: the lower one must win
        logits = dev.gemm_bf16_nt(a, b)
        want = dev.rowargmax(logits.contiguous())
        tiles = lib().wkb_gemm_argmax_tiles(n)
        pv = torch.empty(m * tiles, device="cuda"); pi = torch.empty(m * tiles, dtype=torch.int32, device="cuda")
        out = torch.empty(m, dtype=torch.int32, device="cuda")
        rc = lib().wkb_gemm_bf16_nt_argmax(a.data_ptr(), k, b.data_ptr(), k, m, n, k, None, pv.data_ptr(), pi.data_ptr(),
                                           out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0 and torch.equal(out, want)
        assert list(dev.rowargmax(logits.contiguous()).cpu().numpy()) == list(orc.rowargmax(logits.cpu().numpy()))
    assert dev.gemm_status() == 0


def test_gemm_e4m3_matches_decode_then_gemm(dev, orc):
    """f8 GEMM: the reference has no CPU f8 GEMM, so the oracle is "decode every E4M3 code with the
    pinned codec, then the fp32 order-contract GEMM" (parity unpinned on the reference side).  Products
    of two E4M3 values are exact in fp32; only the fp32 summation order differs."""
    import torch
    L = orc.lib()
    table = np.array([L.wko_f8e4m3_to_f32(c) for c in range(256)], np.float32)
    rng = np.random.default_rng(4)
    for (m, n, k) in [(128, 128, 128), (70, 200, 48), (512, 768, 1024), (33, 129, 16)]:
        a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.float8_e4m3fn).view(torch.uint8)
        b = torch.from_numpy(rng.standard_normal((n, k)).astype(np.float32)).cuda().to(torch.float8_e4m3fn).view(torch.uint8)
        ac, bc = a.cpu().numpy(), b.cpu().numpy()
        # torch's encoder agrees with the pinned codec on these values
        sample = torch.from_numpy(ac[:2].copy()).view(torch.float8_e4m3fn).float().numpy()
        assert np.array_equal(sample, table[ac[:2]])
        af, bf = table[ac], table[bc]
        ref = orc.sgemm(af, bf, m, k, n, "nt")
        got = dev.gemm_e4m3_nt(a, b).cpu().numpy()
        bound = 1e-5 * (np.abs(af) @ np.abs(bf).T) + 1e-6
        assert (np.abs(got - ref) <= bound).all(), (m, n, k, np.abs(got - ref).max())
        bias = rng.standard_normal(n).astype(np.float32)
        gote = dev.gemm_e4m3_nt(a, b, bias=torch.from_numpy(bias).cuda(), act=3).cpu().numpy()
        refe = orc.sgemm(af, bf, m, k, n, bias=bias, act=3)
        assert (np.abs(gote - refe) <= 1.2 * bound + 1e-5).all()
    assert dev.gemm_status() == 0


def test_norm_fast_matches_oracle_recipe(dev, orc):
    """bf16 rows: widen -> the oracle's fp32 norm -> round once.  The fast kernel reduces in a
    different order, so outputs may differ by one bf16 ulp on a few lanes: rtol 2e-2 (the bf16 bar)."""
    import torch
    rng = np.random.default_rng(1)
    for rows, cols in [(7, 768), (33, 4096), (5, 8), (3, 8192), (64, 1024), (5000, 2048), (2371, 4096)]:
        x = rng.standard_normal((rows, cols)).astype(np.float32) * 2
        g = rng.standard_normal(cols).astype(np.float32)
        b = rng.standard_normal(cols).astype(np.float32)
        xb = orc.from_bf16_bits(orc.to_bf16_bits(x)).reshape(rows, cols)
        xt = bf16_t(x, orc)
        gt, btt = torch.from_numpy(g).cuda(), torch.from_numpy(b).cuda()
        for op, ref in ((0, orc.norm(xb, 0)), (1, orc.norm_affine(xb, g, b, 1, 1e-5)), (2, orc.norm_affine(xb, g, None, 2, 1e-5))):
            got = dev.norm_fast(xt, op, 1e-5, gt if op else None, btt if op == 1 else None).float().cpu().numpy()
            want = orc.from_bf16_bits(orc.to_bf16_bits(ref)).reshape(rows, cols)
            assert np.allclose(got, want, rtol=2e-2, atol=1e-3), (rows, cols, op, np.abs(got - want).max())
        # f32 in, f32 out agrees with the exact kernel to fp32 rounding
        xf = torch.from_numpy(x).cuda()
        got = dev.norm_fast(xf, 1, 1e-5, gt, btt).cpu().numpy()
        assert np.allclose(got, orc.norm_affine(x, g, b, 1, 1e-5), rtol=1e-4, atol=1e-5)


def _build_paged(rng, dev, orc, ctx, q_heads, kv_heads, hd, page, nblk, mbps, perm_seed):
    import torch
    slots = len(ctx)
    kflat = [rng.standard_normal((c, kv_heads, hd)).astype(np.float32) for c in ctx]
    vflat = [rng.standard_normal((c, kv_heads, hd)).astype(np.float32) for c in ctx]
    return kflat, vflat


def test_paged_append_and_decode(dev, orc):
    import torch
    from wukong_b200.paged import BlockManager
    for (q_heads, kv_heads, hd, ctx) in [(12, 12, 64, [5, 300, 0, 17, 640, 256, 257]), (32, 8, 128, [128, 1000, 33, 0]),
                                         (8, 4, 64, [31, 32, 33, 511]), (8, 2, 128, [600, 1])]:
        rng = np.random.default_rng(2)
        slots, page, mbps = len(ctx), 16, 64
        nblk = sum((c + page - 1) // page for c in ctx) + 7
        kflat = [rng.standard_normal((c, kv_heads * hd)).astype(np.float32) for c in ctx]
        vflat = [rng.standard_normal((c, kv_heads * hd)).astype(np.float32) for c in ctx]
        q = rng.standard_normal((slots, q_heads * hd)).astype(np.float32)
        scale = 1.0 / math.sqrt(hd)
        outs = []
        for perm_seed in (0, 1):
            # two physical layouts of the same logical history: pages handed out in different orders
            order = np.random.default_rng(perm_seed).permutation(slots)
            mgr = BlockManager(nblk, page, slots, mbps)
            if perm_seed:
                mgr.reserve(slots - 1, 16 * 3); mgr.free(slots - 1)   # scramble the free list
            for s in order:
                if ctx[s]:
                    mgr.reserve(int(s), int(ctx[s]))
            bt = torch.from_numpy(mgr.flat_block_table().astype(np.int64)).to(torch.int32).cuda()
            kv = dev.PagedKV(1, nblk, kv_heads, hd, page)
            kv.k.fill_(float("nan")); kv.v.fill_(float("nan"))
            # append every token through the kernel, one launch per sequence (rows = its tokens)
            for s in range(slots):
                if not ctx[s]:
                    continue
                src = torch.from_numpy(np.concatenate([kflat[s], vflat[s]], 1)).cuda()
                row_slot = torch.full((ctx[s],), s, dtype=torch.int32, device="cuda")
                row_pos = torch.arange(ctx[s], dtype=torch.int32, device="cuda")
                dev.paged_kv_append(kv, 0, src, src[:, kv_heads * hd:], src.stride(0), bt, row_slot, row_pos, ctx[s], mbps)
            # an inactive row writes nothing
            junk = torch.full((1, 2 * kv_heads * hd), 1e9, device="cuda")
            dev.paged_kv_append(kv, 0, junk, junk[:, kv_heads * hd:], junk.stride(0), bt, torch.zeros(1, dtype=torch.int32, device="cuda"),
                                torch.full((1,), -1, dtype=torch.int32, device="cuda"), 1, mbps)
            row_slot = torch.arange(slots, dtype=torch.int32, device="cuda")
            row_ctx = torch.tensor(ctx, dtype=torch.int32, device="cuda")
            scratch = dev.paged_attn_scratch(slots, q_heads, hd, max(ctx))
            out = torch.empty((slots, q_heads * hd), dtype=torch.float32, device="cuda")
            dev.paged_attn_decode(torch.from_numpy(q).cuda(), q_heads * hd, kv, 0, bt, row_slot, row_ctx, out, slots, q_heads, mbps,
                                  max(ctx), scale, scratch)
            outs.append(out.cpu().numpy())
            # block-table gather is bit-exact: every cached element is the bf16 rounding of its source
            kc = kv.k[0].view(torch.int16).cpu().numpy().view(np.uint16)
            table = mgr.flat_block_table()
            for s in range(slots):
                for t in (0, ctx[s] // 2, ctx[s] - 1):
                    if ctx[s] == 0:
                        continue
                    page_id = table[s, t // page]
                    got = kc[page_id, :, t % page, :].reshape(-1)
                    assert np.array_equal(got, orc.to_bf16_bits(kflat[s][t]))
            ref = orc.paged_attn_decode(q, kv.k[0].view(torch.int16).cpu().numpy().view(np.uint16),
                                        kv.v[0].view(torch.int16).cpu().numpy().view(np.uint16), 1, table, ctx, slots, q_heads,
                                        kv_heads, hd, page, mbps, scale, layout=1)
            # head_dim 128 with a GQA group runs on the tensor cores: the softmax weights are bf16 there (2^-9 each)
            # (values are ~N(0,1), so a weighted mean of them carries up to ~2^-9 absolute)
            mma_path = hd == 128 and q_heads != kv_heads
            rtol, atol = (4e-3, 2e-3) if mma_path else (1e-4, 1e-5)
            assert np.allclose(outs[-1], ref, rtol=rtol, atol=atol), (q_heads, kv_heads, hd, np.abs(outs[-1] - ref).max())
        assert outs[0].tobytes() == outs[1].tobytes(), "decode output depends on the physical page layout"
        for s in range(slots):
            if ctx[s] == 0:
                assert (outs[0][s] == 0).all()
        assert not np.isnan(outs[0]).any()
        # bf16 output path
        outb = torch.empty((slots, q_heads * hd), dtype=torch.bfloat16, device="cuda")
        dev.paged_attn_decode(torch.from_numpy(q).cuda(), q_heads * hd, kv, 0, bt, row_slot, row_ctx, outb, slots, q_heads, mbps,
                              max(ctx), scale, scratch)
        assert np.array_equal(outb.view(torch.int16).cpu().numpy().view(np.uint16), orc.to_bf16_bits(outs[1]).reshape(slots, -1))


def test_qkv_gemm_with_fused_append_equals_gemm_then_append(dev, orc):
    """The fused QKV projection writes the query columns like the plain GEMM and puts the K / V columns into the pages
    exactly as the separate append kernel does (same fp32 values, same rounding, same addresses); inactive rows and rows
    past the block-table row write nothing."""
    import torch
    from wukong_b200 import lib
    L, s = lib(), torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(5)
    for (rows, heads, hd, d_in) in [(70, 4, 64, 256), (512, 12, 64, 768), (33, 2, 128, 256), (600, 12, 64, 768)]:   # the last one is past one wave of 64-column tiles: 128-column tiles
        d = heads * hd
        page, mbps, slots = 16, 6, rows
        nblk = slots * mbps
        a = bf16_t(rng.standard_normal((rows, d_in)).astype(np.float32), orc)
        w = bf16_t(rng.standard_normal((3 * d, d_in)).astype(np.float32) * 0.1, orc)
        bias = torch.from_numpy(rng.standard_normal(3 * d).astype(np.float32)).cuda()
        table = torch.from_numpy(rng.permutation(nblk).astype(np.int32).reshape(slots, mbps)).cuda()
        pos = rng.integers(0, mbps * page, rows).astype(np.int32)
        pos[3] = -1                      # inactive
        pos[5] = mbps * page             # past the table: skipped and reported
        row_pos = torch.from_numpy(pos).cuda()
        row_slot = torch.from_numpy(rng.permutation(slots).astype(np.int32)).cuda()
        # reference path: plain GEMM, then the append kernel
        qkv = dev.gemm_bf16_nt(a, w, bias=bias)
        kv_ref = dev.PagedKV(1, nblk, heads, hd, page)
        kv_ref.k.fill_(7.0); kv_ref.v.fill_(7.0)
        dev.paged_kv_append(kv_ref, 0, qkv[:, d:], qkv[:, 2 * d:], qkv.stride(0), table, row_slot, row_pos, rows, mbps)
        torch.cuda.synchronize()
        assert dev.gemm_status() == 31
        # fused path
        kv = dev.PagedKV(1, nblk, heads, hd, page)
        kv.k.fill_(7.0); kv.v.fill_(7.0)
        q = torch.full((rows, d), -3.0, device="cuda")
        rc = L.wkb_gemm_bf16_nt_qkv_append(a.data_ptr(), d_in, w.data_ptr(), d_in, q.data_ptr(), d, rows, 3 * d, d_in, bias.data_ptr(), d,
                                           kv.k[0].data_ptr(), kv.v[0].data_ptr(), table.data_ptr(), row_slot.data_ptr(), row_pos.data_ptr(),
                                           heads, hd, page, mbps, s)
        torch.cuda.synchronize()
        assert rc == 0 and dev.gemm_status() == 31
        assert torch.equal(q, qkv[:, :d])
        assert torch.equal(kv.k.view(torch.int16), kv_ref.k.view(torch.int16)) and torch.equal(kv.v.view(torch.int16), kv_ref.v.view(torch.int16))


def test_addto_gemm_sums_its_k_slices_inside_a_cluster(dev, orc):
    """x += A.B^T + bias with the K slices of a tile added through distributed shared memory: exact on small integers
    whatever the split (2, 4 or 8 slices), ragged rows and columns included; shapes the rule does not offer are refused
    before anything is launched."""
    import torch
    from wukong_b200 import lib
    L, s = lib(), torch.cuda.current_stream().cuda_stream
    seen = set()
    for (m, n, k) in [(512, 768, 768), (512, 768, 3072), (64, 768, 3072), (64, 768, 768), (100, 256, 512), (130, 260, 1024), (16, 128, 4096)]:
        ks = L.wkb_gemm_bf16_addto_slices(m, n, k)
        assert ks in (2, 4, 8), (m, n, k, ks)
        seen.add(ks)
        a = torch.randint(-3, 4, (m, k), device="cuda").to(torch.bfloat16)
        b = torch.randint(-3, 4, (n, k), device="cuda").to(torch.bfloat16)
        bias = torch.randint(-5, 6, (n,), device="cuda").float()
        x = torch.randint(-9, 10, (m, n), device="cuda").float()
        want = x + a.float() @ b.float().T + bias
        assert L.wkb_gemm_bf16_nt_addto(a.data_ptr(), k, b.data_ptr(), k, x.data_ptr(), n, m, n, k, bias.data_ptr(), s) == 0
        torch.cuda.synchronize()
        assert torch.equal(x, want), (m, n, k, ks, float((x - want).abs().max()))
        # without a bias, and on real-valued inputs against the fp32 product (the bar of the dense GEMM)
        ar = bf16_t(np.random.default_rng(1).standard_normal((m, k)).astype(np.float32), orc)
        br = bf16_t(np.random.default_rng(2).standard_normal((n, k)).astype(np.float32), orc)
        x2 = torch.zeros(m, n, device="cuda")
        assert L.wkb_gemm_bf16_nt_addto(ar.data_ptr(), k, br.data_ptr(), k, x2.data_ptr(), n, m, n, k, None, s) == 0
        ref = ar.double() @ br.double().T
        mag = ar.double().abs() @ br.double().abs().T
        assert bool(((x2.double() - ref).abs() <= 1e-5 * mag + 1e-6).all())
    assert seen == {2, 4, 8}
    assert L.wkb_gemm_bf16_addto_slices(2000, 768, 768) == 0          # more tiles than one wave of clusters holds
    a = torch.zeros(2000, 768, device="cuda", dtype=torch.bfloat16)
    x = torch.zeros(2000, 768, device="cuda")
    assert L.wkb_gemm_bf16_nt_addto(a.data_ptr(), 768, a.data_ptr(), 768, x.data_ptr(), 768, 2000, 768, 768, None, s) != 0
    assert dev.gemm_status() == 0


def test_partial_gemm_slices_sum_to_the_product(dev, orc):
    import ctypes
    import torch
    from wukong_b200 import lib
    L, s = lib(), torch.cuda.current_stream().cuda_stream
    for (m, n, k) in [(64, 768, 768), (512, 768, 3072), (100, 256, 64), (2000, 768, 768)]:
        a = torch.randint(-3, 4, (m, k), device="cuda").to(torch.bfloat16)
        b = torch.randint(-3, 4, (n, k), device="cuda").to(torch.bfloat16)
        ns, st = ctypes.c_int64(), ctypes.c_int64()
        L.wkb_gemm_bf16_partial_layout(m, n, k, ctypes.byref(ns), ctypes.byref(st))
        assert ns.value >= 1 and st.value == m * n
        ws = torch.full((ns.value * m * n,), float("nan"), device="cuda")
        assert L.wkb_gemm_bf16_nt_partial(a.data_ptr(), k, b.data_ptr(), k, m, n, k, ws.data_ptr(), ws.numel() * 4, s) == 0
        got = ws.view(ns.value, m, n).sum(0)
        assert torch.equal(got, a.float() @ b.float().T)          # small integers: exact whatever the split
        assert L.wkb_gemm_bf16_nt_partial(a.data_ptr(), k, b.data_ptr(), k, m, n, k, ws.data_ptr(), ws.numel() * 4 - 4, s) != 0   # short workspace refused
    assert dev.gemm_status() == 0
