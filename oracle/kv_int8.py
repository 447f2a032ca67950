"""TEST INFRASTRUCTURE (oracle): the reference's int8 KV quantizer restated in numpy.

crates/wukong_codegen_gpu/src/paged_attention.rs:1305-1326: per (token, KV head) scale = max_d |x| / 127 (1 when the
row is all zero), value = round(x / scale) -- half away from zero, as Rust's f32::round -- clamped to [-127, 127];
the cache stores exactly these bytes and scales, attention reads int8 * scale.  Only tests may import this module."""
import numpy as np


def quantize_kv_int8(x):
    """x: float32 [..., head_dim] -> (int8 [..., head_dim], float32 scales [...])."""
    x = np.ascontiguousarray(x, np.float32)
    amax = np.abs(x).max(axis=-1)
    scale = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    y = (x / scale[..., None]).astype(np.float32)
    a = np.abs(y)
    fl = np.floor(a)
    r = fl + ((a - fl) >= np.float32(0.5))          # exact: |y| <= 127 has an exact fractional part in f32
    q = np.clip(np.sign(y) * r, -127, 127).astype(np.int8)
    return q, scale


def dequantize(q, scale):
    return (q.astype(np.float32) * scale[..., None]).astype(np.float32)
