"""Host-side helpers and oracle restatements that need no GPU: prefill tiling, the int8 KV quantizer."""
import numpy as np


def test_prefill_tiles_helper():
    from wukong_b200.device import prefill_tiles
    rs = np.array([0, 0, 0, 0, 0, 2, 3, 3, 3, 7], np.int32)
    assert prefill_tiles(rs, 4).tolist() == [[0, 4], [4, 1], [5, 1], [6, 3], [9, 1]]
    assert prefill_tiles(rs, 4, min_run=2).tolist() == [[0, 4], [4, 1], [6, 3]]
    assert prefill_tiles(np.zeros(0, np.int32), 4).shape == (0, 2)


def test_quantizer_restatement_rounds_half_away_from_zero():
    from oracle.kv_int8 import quantize_kv_int8
    x = np.array([[127.0, 0.5, -0.5, 1.5, -2.5, 63.49999, 0.0, -127.0]], np.float32)
    q, s = quantize_kv_int8(x)
    assert s[0] == 1.0 and q[0].tolist() == [127, 1, -1, 2, -3, 63, 0, -127]
    q, s = quantize_kv_int8(np.zeros((1, 8), np.float32))
    assert s[0] == 1.0 and not q.any()


def test_cluster_slice_rule_is_a_function_of_the_shape():
    """The rule that offers the in-cluster K-slice sum (no device work: a machine without a GPU answers for 148 SMs):
    2, 4 or 8 slices, at least three 64-wide K steps each, no empty last slice, tiles x slices within one wave, n % 4 == 0."""
    from wukong_b200 import lib
    L = lib()
    if L.wkb_device_count() > 0:
        import pytest
        pytest.skip("the expected values are those of the 148-SM default")
    want = {(512, 768, 768): 4, (512, 768, 3072): 4, (64, 768, 3072): 8, (64, 768, 768): 4, (100, 256, 512): 2,
            (130, 260, 1024): 4, (16, 128, 4096): 8, (2000, 768, 768): 0, (512, 770, 768): 0, (64, 768, 128): 0, (0, 768, 768): 0}
    for (m, n, k), ks in want.items():
        assert L.wkb_gemm_bf16_addto_slices(m, n, k) == ks, (m, n, k)
    # a slice count is only offered when its last slice has work: 25 K steps cut in 8 would leave slice 7 empty
    for k in range(64, 64 * 64 + 1, 64):
        ks = L.wkb_gemm_bf16_addto_slices(64, 128, k)
        kit = k // 64
        if ks:
            per = (kit + ks - 1) // ks
            assert ks in (2, 4, 8) and kit // ks >= 3 and (ks - 1) * per < kit
