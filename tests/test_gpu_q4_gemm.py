"""GPU parity of the W4A16 tensor-core GEMM (resident Q4_0 weights, bf16 activations).

The kernel's weight is defined as bf16(bf16(d) * (nib - 8)); the checks are
  (1) against that definition with the nibbles and scales unpacked by the oracle (integer-exact
      unpack: any wrong nibble, order or scale shows up far above the fp32-accumulation band), and
  (2) against the exact f32 dequantisation d * (nib - 8), inside the rtol 2e-2 bar of the bf16 paths.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from wukong_b200 import _lib, device
    _lib.require_gpu()
    return device


def synth_q4(rng, n, k):
    """Raw Q4_0 rows as the benchmark configuration draws them: nibbles uniform, f16 scale |N(0, 0.02)|."""
    nb = k // 32
    raw = rng.integers(0, 256, (n * nb, 18), dtype=np.uint8)
    sc = np.abs(rng.standard_normal(n * nb) * 0.02).astype(np.float16).view(np.uint16)
    raw[:, 0] = sc & 0xFF
    raw[:, 1] = sc >> 8
    return raw.reshape(-1)


def kernel_weight(orc, d, q):
    """bf16(bf16(d) * q): both products are exact in f32 before the rounding."""
    d_bf = orc.from_bf16_bits(orc.to_bf16_bits(np.ascontiguousarray(d, np.float32).ravel())).reshape(np.shape(d))
    return orc.from_bf16_bits(orc.to_bf16_bits((d_bf * q).astype(np.float32).ravel())).reshape(np.shape(d_bf * q))


def reference_weights(orc, raw, n, k):
    """(exact f32 dequantisation, the kernel's bf16 weight) from the oracle's integer unpack."""
    quants, scales = orc.unpack_q4_0(raw)
    q = quants.astype(np.float32).reshape(n, k // 32, 32)
    d = scales.view(np.float16).astype(np.float32).reshape(n, k // 32, 1)
    exact = (d * q).reshape(n, k)
    return exact, kernel_weight(orc, d, q).reshape(n, k)


def run_case(dev, orc, rng, m, n, k, mode):
    import torch
    raw = synth_q4(rng, n, k)
    x = rng.standard_normal((m, k)).astype(np.float32)
    xb = orc.to_bf16_bits(x)
    xw = orc.from_bf16_bits(xb).reshape(m, k).astype(np.float64)
    exact, w_bf = reference_weights(orc, raw, n, k)
    w = dev.Q4Weight.from_raw(torch.from_numpy(raw).cuda(), n, k)
    xt = torch.from_numpy(xb.view(np.int16).reshape(m, k)).cuda().view(torch.bfloat16)
    ws = dev.gemm_q4_workspace(w.n, w.k)
    out = dev.gemm_q4_0_bf16_nt(w, xt, mode=mode, workspace=ws)
    again = dev.gemm_q4_0_bf16_nt(w, xt, mode=mode, workspace=ws)   # the arrival counters must have been re-armed
    torch.cuda.synchronize()
    assert dev.gemm_status() == 0
    assert torch.equal(out, again)
    got = out.float().cpu().numpy().astype(np.float64)
    ref_def = xw @ w_bf.astype(np.float64).T
    ref_exact = xw @ exact.astype(np.float64).T
    mag = np.abs(xw) @ np.abs(w_bf.astype(np.float64)).T
    if mode == 2:
        silu = lambda v: v / (1.0 + np.exp(-v))
        ref_def = silu(ref_def[:, 0::2]) * ref_def[:, 1::2]
        gate_exact, up_exact = ref_exact[:, 0::2], ref_exact[:, 1::2]
        ref_exact = silu(gate_exact) * up_exact
        band = 2.0 ** -8 * np.abs(ref_def) + 1e-3 * (1.0 + np.abs(ref_def))
        assert np.all(np.abs(got - ref_def) <= band), np.abs(got - ref_def).max()
    else:
        out_round = 2.0 ** -8 * np.abs(ref_def) if mode == 1 else 0.0
        assert np.all(np.abs(got - ref_def) <= 2e-6 * mag + 1e-6 + out_round), (np.abs(got - ref_def) / (mag + 1e-9)).max()
    # the stated bar against the exact dequantisation: rtol 2e-2 with the usual magnitude floor (for the
    # SwiGLU the bar is applied to both factors of the product)
    if mode == 2:
        rms_g, rms_u = np.sqrt(np.mean(gate_exact ** 2)), np.sqrt(np.mean(up_exact ** 2))
        bar = 2e-2 * (np.abs(gate_exact) + rms_g) * (np.abs(up_exact) + rms_u)
    else:
        bar = 2e-2 * np.abs(ref_exact) + 2e-2 * np.sqrt(np.mean(ref_exact ** 2))
    assert np.all(np.abs(got - ref_exact) <= bar)


@pytest.mark.parametrize("m,n,k,mode", [
    (64, 256, 256, 0),        # one stage, one slice
    (64, 384, 1024, 0),       # a full resident slice, several tiles per CTA group
    (17, 200, 2048, 0),       # ragged rows and weight rows, two K slices
    (64, 512, 4096, 1),       # four K slices, bf16 out
    (64, 1024, 1376, 0),      # K that needs row padding (43 blocks)
    (64, 512, 2048, 2),       # SwiGLU of interleaved gate / up rows
    (130, 256, 512, 0),       # more than 64 rows: three passes
    (3, 2816, 512, 2),        # few rows, SwiGLU, two single-stage K slices
    (3, 2816, 512, 0),
    (64, 256, 256, 2),        # SwiGLU without a K split
])
def test_q4_gemm_matches_definition_and_exact_dequant(dev, orc, m, n, k, mode):
    run_case(dev, orc, np.random.default_rng(1000 + m + n + k + mode), m, n, k, mode)


def test_q4_gemm_llama_shapes(dev, orc):
    """The three linear shapes of a 7B-shape block at batch 64 (column-parallel QKV, SwiGLU, down projection)."""
    rng = np.random.default_rng(7)
    run_case(dev, orc, rng, 64, 6144, 4096, 0)
    run_case(dev, orc, rng, 64, 2 * 2752, 4096, 2)
    run_case(dev, orc, rng, 64, 4096, 2752, 0)


@pytest.mark.parametrize("m,n,k", [(64, 4096, 2752), (17, 512, 4096), (64, 256, 256)])
def test_q4_gemm_partials_folded_into_add_rmsnorm(dev, orc, m, n, k):
    """out_mode 3 leaves the K-slice partials in the workspace; adding them in slice order inside the
    residual-add + RMSNorm kernel must give the residual stream and normed row of the two-kernel route."""
    import ctypes
    import torch
    from wukong_b200._lib import lib, check
    rng = np.random.default_rng(31 + m + n + k)
    raw = synth_q4(rng, n, k)
    w = dev.Q4Weight.from_raw(torch.from_numpy(raw).cuda(), n, k)
    xb = orc.to_bf16_bits(rng.standard_normal((m, k)).astype(np.float32))
    xt = torch.from_numpy(xb.view(np.int16).reshape(m, k)).cuda().view(torch.bfloat16)
    ws = dev.gemm_q4_workspace(w.n, w.k)
    full = dev.gemm_q4_0_bf16_nt(w, xt, mode=0, workspace=ws)
    res = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).cuda()
    gain = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    s = torch.cuda.current_stream().cuda_stream
    x_a, out_a = res.clone(), torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    check(lib().wkb_add_rmsnorm_bf16(x_a.data_ptr(), full.data_ptr(), gain.data_ptr(), out_a.data_ptr(), m, n, 1e-5, s), "add_rmsnorm")
    a, b, c = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    lib().wkb_gemm_q4_0_partial_layout(n, k, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
    assert a.value >= 1 and a.value * b.value * 4 <= ws.numel() and c.value >= n
    dummy = torch.empty(1, device="cuda")
    check(lib().wkb_gemm_q4_0_bf16_nt(w.tiled.data_ptr(), xt.data_ptr(), k, dummy.data_ptr(), n, 3, m, n, k, ws.data_ptr(), ws.numel(), s), "gemm mode 3")
    x_b, out_b = res.clone(), torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    check(lib().wkb_add_slices_rmsnorm_bf16(x_b.data_ptr(), ws.data_ptr(), a.value, b.value, c.value, gain.data_ptr(), out_b.data_ptr(),
                                            m, n, 1e-5, s), "add_slices_rmsnorm")
    torch.cuda.synchronize()
    assert dev.gemm_status() == 0
    # the same slices are added in the same order; only the place of the residual in the sum differs
    assert torch.allclose(x_a, x_b, rtol=0, atol=4e-6 * float(full.abs().max() + res.abs().max()))
    assert (out_a.float() - out_b.float()).abs().max() <= 2.0 ** -7 * out_a.float().abs().max()
