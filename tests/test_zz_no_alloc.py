"""The allocation-free Q4_0 GEMV entry against the ordinary one.

Some hosts of this library may not allocate device memory while they run kernels: an engine that
carved its whole arena at start-up, or a plug-in invoked from inside another runtime's managed
region.  `wkb_gemv_q4_0_f32_noalloc` serves them by keeping the per-call activation scratch in a
fixed device array of the library.  This file is collected last on purpose, so a failure here cannot
hide the result of any other test.  Two calls in a row check that the array, which keeps the previous
call's contents, is fully rewritten; both calls are also held to the CPU oracle's GEMV bit for bit; the oversize
refusal is checked too."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_gemv_matches_regular_entry_twice(orc):
    import torch
    from wukong_b200 import _lib, lib, device as dev
    _lib.require_gpu()
    L = lib()
    rng = np.random.default_rng(11)
    s = torch.cuda.current_stream().cuda_stream
    for (n, k) in [(96, 4096), (40, 257), (8, 32768)]:
        nb = (k + 31) // 32
        raw = rng.integers(0, 256, n * nb * 18, dtype=np.uint8)
        sc = np.abs(rng.standard_normal(n * nb) * 0.02).astype(np.float16).view(np.uint16)
        raw.reshape(-1, 18)[:, 0] = sc & 0xFF
        raw.reshape(-1, 18)[:, 1] = sc >> 8
        qs, d = dev.q_split(torch.from_numpy(raw).cuda(), n * nb, q4=True)
        for call in range(2):   # the second call sees the first call's scratch contents
            x_host = (rng.standard_normal(k) * (1 + 9 * call)).astype(np.float32)
            x = torch.from_numpy(x_host).cuda()
            xq, dx, sx = dev.quantize_act(x)
            want = dev.gemv_q_contract(qs, d, xq, dx, sx, n, k, q4=True)
            got = torch.full((n,), 7.0, device="cuda")
            rc = L.wkb_gemv_q4_0_f32_noalloc(qs.data_ptr(), d.data_ptr(), x.data_ptr(), got.data_ptr(), n, k, s)
            torch.cuda.synchronize()
            assert rc == 0
            assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (n, k, call)   # bit for bit
            # and against the CPU oracle's GEMV on the raw blocks (an independent implementation of the same contract)
            st, ref = orc.gemv_q(raw, x_host, n)
            assert st == 0 and got.cpu().numpy().tobytes() == ref.tobytes(), (n, k, call)
    # beyond the fixed scratch: refused, output untouched
    y = torch.full((4,), 7.0, device="cuda")
    rc = L.wkb_gemv_q4_0_f32_noalloc(qs.data_ptr(), d.data_ptr(), x.data_ptr(), y.data_ptr(), 4, 32768 + 32, s)
    torch.cuda.synchronize()
    assert rc != 0 and bool((y == 7.0).all())
