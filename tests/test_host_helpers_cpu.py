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
