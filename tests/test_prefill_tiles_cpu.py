"""Host helper of the paged prefill attention: cutting a step's rows into per-sequence tiles."""
import numpy as np


def test_prefill_tiles_helper():
    from wukong_b200.device import prefill_tiles
    rs = np.array([0, 0, 0, 0, 0, 2, 3, 3, 3, 7], np.int32)
    assert prefill_tiles(rs, 4).tolist() == [[0, 4], [4, 1], [5, 1], [6, 3], [9, 1]]
    assert prefill_tiles(rs, 4, min_run=2).tolist() == [[0, 4], [4, 1], [6, 3]]
    assert prefill_tiles(np.zeros(0, np.int32), 4).shape == (0, 2)
