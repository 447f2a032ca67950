"""The C-ABI library loads on a machine without a GPU and exports every symbol its header declares.
No compute call is made here."""
import os
import re

import pytest


def test_library_exports_every_declared_symbol():
    import wukong_b200
    from wukong_b200 import build
    build.build()
    L = wukong_b200.lib()
    names = wukong_b200.declared_symbols()
    assert len(names) > 80
    for n in names:
        assert hasattr(L, n), n


def test_reference_abi_names_present():
    """The hot-path rows of the reference's symbol table (runtime_abi.rs) are all exported."""
    import wukong_b200
    names = set(wukong_b200.declared_symbols())
    wanted = """wukong_sgemm wukong_sgemm_nt wukong_sgemm_tn wukong_sgemm_nt_epi wukong_sgemm_nt_alpha
    wukong_sgemm_bf16_nt wukong_sgemm_f16_nt wukong_sgemm_bf16_nt_epi wukong_sgemm_f16_nt_epi wukong_sgemm_bf16_tn
    wukong_sgemv wukong_sgemv_alpha wukong_sgemv_bf16 wukong_sgemv_f16 wukong_gemv_q4_0_f32 wukong_gemv_q8_0_f32
    wukong_quantize_q4_0_f32 wukong_quantize_q8_0_f32 wukong_dequant_i4_f32 wukong_dequant_u4_f32
    wukong_attention_kv_f32 wukong_attention_kv_batch_f32 wukong_kv_append_f32 wukong_attention_f32
    wukong_norm_f32 wukong_norm_affine_f32 wukong_vmath_f32 wukong_vmath2_f32 wukong_velem_f32 wukong_rope_f32
    wukong_embedding_f32 wukong_rowargmax_i32""".split()
    for w in wanted:
        assert w in names, w
        if w not in ("wukong_vmath2_f32", "wukong_kv_append_f32", "wukong_attention_f32", "wukong_quantize_q4_0_f32",
                     "wukong_quantize_q8_0_f32", "wukong_dequant_i4_f32", "wukong_dequant_u4_f32"):
            assert w + "_parallel" in names, w


def test_product_does_not_touch_the_oracle():
    """Nothing in the package imports, links or reads the oracle."""
    root = os.path.join(os.path.dirname(__file__), "..", "wukong_b200")
    for dirpath, _, files in os.walk(root):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"\bwko_|wk_oracle|from oracle|import oracle", text), f


def test_host_logic_no_gpu_needed():
    """Status codes that the checked entries return before touching the device."""
    import numpy as np
    import wukong_b200
    L = wukong_b200.lib()
    z = np.zeros(8, np.float32)
    p = z.ctypes.data
    assert L.wukong_gemv_q4_0_f32(p, 17, p, 32, p, 1) == -2
    assert L.wukong_sgemv_bf16(p, 5, p, 2, p, 2) == -2
    assert L.wukong_quantize_q4_0_f32(p, 8, p, 18, 0) == -2
    assert L.wukong_attention_kv_f32(p, 8, p, 8, p, 8, p, 8, 1, 1, 4, 0, 4, 3, 16, 8, 1.0, 1) == -1
    assert L.wukong_attention_kv_f32(p, 8, p, 8, p, 8, p, 8, 1, 2, 4, 0, 2, 2, 8, 8, 1.0, 1) == -2
    assert L.wukong_kv_append_f32(p, 8, p, 4, 2, 4) == -2
    assert L.wukong_dequant_i4_f32(p, 4, p, 3, 4, p, 10) == -2
    y = np.full(3, 7.0, np.float32)
    assert L.wukong_gemv_q4_0_f32(p, 0, p, 0, y.ctypes.data, 3) == 0 and (y == 0).all()  # K = 0 -> zeros
