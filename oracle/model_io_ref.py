"""TEST INFRASTRUCTURE (oracle): checkpoint containers restated in numpy.

Independent of the C++ readers: file writers for GGUF (v2 / v3) and safetensors, and the ggml block formats
dequantized with vectorised float32 numpy (each product and sum is one float32 operation, as in
crates/wukong_runtime/src/gguf.rs:1139-1340, which follows ggml's dequantize_row_*).  Pinned on the reference's
own known-answer blocks (gguf.rs:1889-2192) in tests/test_model_io_cpu.py.  Only tests may import this module.
"""
import json
import struct

import numpy as np

# ggml type id -> (name, elements per block, bytes per block)   (gguf.rs:244-289)
GGML_TYPES = {0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
              7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110),
              12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292),
              16: ("IQ2_XXS", 256, 66), 17: ("IQ2_XS", 256, 74), 18: ("IQ3_XXS", 256, 98), 19: ("IQ1_S", 256, 50),
              20: ("IQ4_NL", 32, 18), 21: ("IQ3_S", 256, 110), 22: ("IQ2_S", 256, 82), 23: ("IQ4_XS", 256, 136),
              24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8),
              29: ("IQ1_M", 256, 56), 30: ("BF16", 1, 2), 34: ("TQ1_0", 256, 54), 35: ("TQ2_0", 256, 66), 39: ("MXFP4", 32, 17)}
DEQUANT_IDS = (2, 3, 6, 7, 8, 10, 11, 12, 13, 14, 15, 20, 23)
IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)
F = np.float32


def _half(b, at):
    return np.ascontiguousarray(b[:, at:at + 2]).view("<f2")[:, 0].astype(F)[:, None]


def _k4(j, sc):
    """6-bit scale and min of sub-block j from the 12 packed bytes [nb, 12] (ggml get_scale_min_k4)."""
    if j < 4:
        return sc[:, j] & 63, sc[:, j + 4] & 63
    return (sc[:, j + 4] & 0xF) | ((sc[:, j - 4] >> 6) << 4), (sc[:, j + 4] >> 4) | ((sc[:, j] >> 6) << 4)


def dequant(type_id, raw):
    """raw: uint8 [nblocks * bytes] -> float32 [nblocks * block]."""
    _, blk, nbytes = GGML_TYPES[type_id]
    b = np.ascontiguousarray(raw, np.uint8).reshape(-1, nbytes)
    nb = b.shape[0]
    y = np.zeros((nb, blk), F)
    if type_id in (2, 20):
        d, qs = _half(b, 0), b[:, 2:18]
        lo, hi = qs & 0xF, qs >> 4
        if type_id == 2:
            y[:, :16] = (lo.astype(np.int32) - 8).astype(F) * d
            y[:, 16:] = (hi.astype(np.int32) - 8).astype(F) * d
        else:
            y[:, :16], y[:, 16:] = d * IQ4NL[lo], d * IQ4NL[hi]
    elif type_id == 3:
        d, m, qs = _half(b, 0), _half(b, 2), b[:, 4:20]
        y[:, :16] = (qs & 0xF).astype(F) * d + m
        y[:, 16:] = (qs >> 4).astype(F) * d + m
    elif type_id in (6, 7):
        h = 4 if type_id == 7 else 2
        d = _half(b, 0)
        qh = np.ascontiguousarray(b[:, h:h + 4]).view("<u4")[:, 0][:, None]
        qs = b[:, h + 4:h + 20]
        e = np.arange(32, dtype=np.uint32)[None, :]
        nib = np.concatenate([qs & 0xF, qs >> 4], axis=1).astype(np.int32)
        x = nib | (((qh >> e) & 1).astype(np.int32) << 4)
        y[:] = x.astype(F) * d + _half(b, 2) if type_id == 7 else (x - 16).astype(F) * d
    elif type_id == 8:
        y[:] = b[:, 2:34].view(np.int8).astype(F) * _half(b, 0)
    elif type_id == 10:
        d, dmin = _half(b, 80), _half(b, 82)
        yi = 0
        for n in range(2):
            q = b[:, 16 + n * 32:16 + n * 32 + 32]
            for si, shift in enumerate((0, 2, 4, 6)):
                for h16 in range(2):
                    sc = b[:, n * 8 + si * 2 + h16][:, None]
                    dl, ml = d * (sc & 0xF).astype(F), dmin * (sc >> 4).astype(F)
                    v = (q[:, 16 * h16:16 * h16 + 16] >> shift) & 3
                    y[:, yi:yi + 16] = dl * v.astype(F) - ml
                    yi += 16
    elif type_id == 11:
        hm, sr, d_all = b[:, 0:32], b[:, 96:108], _half(b, 108)
        scales = []
        for k in range(16):
            low = (sr[:, k] & 0xF) if k < 8 else (sr[:, k - 8] >> 4)
            high = (sr[:, 8 + k % 4] >> (2 * (k // 4))) & 3
            scales.append((low | (high << 4)).astype(np.int32) - 32)
        yi, m, isc = 0, 1, 0
        for n in range(2):
            q = b[:, 32 + n * 32:32 + n * 32 + 32]
            for shift in (0, 2, 4, 6):
                for h16 in range(2):
                    dl = d_all * scales[isc].astype(F)[:, None]
                    isc += 1
                    sl = slice(16 * h16, 16 * h16 + 16)
                    v = ((q[:, sl] >> shift) & 3).astype(np.int32) - np.where(hm[:, sl] & m, 0, 4)
                    y[:, yi:yi + 16] = dl * v.astype(F)
                    yi += 16
                m <<= 1
    elif type_id in (12, 13):
        five = type_id == 13
        d, dmin, sc = _half(b, 0), _half(b, 2), b[:, 4:16]
        qh = b[:, 16:48]
        qs = b[:, 48:176] if five else b[:, 16:144]
        yi = 0
        for c in range(4):
            q = qs[:, c * 32:c * 32 + 32]
            for hi in range(2):
                s, mn = _k4(2 * c + hi, sc)
                d1, m1 = d * s.astype(F)[:, None], dmin * mn.astype(F)[:, None]
                v = ((q >> 4) if hi else (q & 0xF)).astype(np.int32)
                if five:
                    v = v + np.where(qh & ((2 if hi else 1) << (2 * c)), 16, 0)
                y[:, yi:yi + 32] = d1 * v.astype(F) - m1
                yi += 32
    elif type_id == 14:
        d = _half(b, 208)
        for n in range(2):
            ql, qh = b[:, n * 64:n * 64 + 64], b[:, 128 + n * 32:128 + n * 32 + 32]
            sc = b[:, 192 + n * 8:192 + n * 8 + 8].view(np.int8)
            isx = np.arange(32) // 16
            for grp in range(4):
                lowb = ql[:, 32 * (grp & 1):32 * (grp & 1) + 32]
                nib = (lowb >> 4) if grp >= 2 else (lowb & 0xF)
                q = (nib | (((qh >> (2 * grp)) & 3) << 4)).astype(np.int32) - 32
                s = d * sc[:, isx + 2 * grp].astype(F)
                y[:, n * 128 + grp * 32:n * 128 + grp * 32 + 32] = s * q.astype(F)
    elif type_id == 15:
        d = np.ascontiguousarray(b[:, 0:4]).view("<f4")
        y[:] = d * b[:, 4:260].view(np.int8).astype(F)
    elif type_id == 23:
        d = _half(b, 0)
        scales_h = np.ascontiguousarray(b[:, 2:4]).view("<u2")[:, 0].astype(np.int32)
        for ib in range(8):
            lo = (b[:, 4 + ib // 2] >> (4 * (ib % 2))) & 0xF
            hi = (scales_h >> (2 * ib)) & 3
            dl = d * ((lo.astype(np.int32) | (hi << 4)) - 32).astype(F)[:, None]
            q = b[:, 8 + ib * 16:8 + ib * 16 + 16]
            y[:, ib * 32:ib * 32 + 16] = dl * IQ4NL[q & 0xF]
            y[:, ib * 32 + 16:ib * 32 + 32] = dl * IQ4NL[q >> 4]
    else:
        raise ValueError("no dequantizer for ggml type %d" % type_id)
    return y.reshape(-1)


# ---------------------------------------------------------------------------------------------------------
# file writers (the inverse of the readers; used to assemble test files byte by byte)
# ---------------------------------------------------------------------------------------------------------
VT = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10, "i64": 11, "f64": 12}
_FMT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}


def gstr(s):
    s = s if isinstance(s, bytes) else s.encode()
    return struct.pack("<Q", len(s)) + s


def enc_value(kind, v):
    """Payload of a metadata value (no type id).  kind: a VT name; arrays are ("arr", elem_kind, [values])."""
    t = VT[kind]
    if t in _FMT:
        return struct.pack(_FMT[t], v)
    if kind == "str":
        return gstr(v)
    elem, items = v
    return struct.pack("<IQ", VT[elem], len(items)) + b"".join(enc_value(elem, it) for it in items)


class GgufBuilder:
    def __init__(self, version=3, align=32, magic=b"GGUF"):
        self.magic, self.version, self.align = magic, version, align
        self.kv, self.n_kv, self.ti, self.n_t, self.data = b"", 0, b"", 0, b""

    def meta(self, key, kind, v):
        return self.meta_raw(key, VT[kind], enc_value(kind, v))

    def meta_raw(self, key, type_id, payload):
        self.kv += gstr(key) + struct.pack("<I", type_id) + payload
        self.n_kv += 1
        return self

    def tensor(self, name, ne, type_id, payload):
        """ne innermost first, as the file stores it; the payload is appended at the next aligned offset."""
        pad = (-len(self.data)) % self.align
        self.data += b"\0" * pad
        self.tensor_at(name, ne, type_id, len(self.data))
        self.data += bytes(payload)
        return self

    def tensor_at(self, name, ne, type_id, offset):
        self.ti += gstr(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne) + struct.pack("<IQ", type_id, offset)
        self.n_t += 1
        return self

    def header(self):
        return self.magic + struct.pack("<IQQ", self.version, self.n_t, self.n_kv) + self.kv + self.ti

    def bytes(self):
        h = self.header()
        return h + b"\0" * ((-len(h)) % self.align) + self.data


def st_file(header, payload=b""):
    """A safetensors file from its JSON header (text, bytes or a dict) and byte buffer."""
    if isinstance(header, dict):
        header = json.dumps(header)
    if isinstance(header, str):
        header = header.encode()
    return struct.pack("<Q", len(header)) + header + bytes(payload)


def write_llama_gguf(cfg, w, embed_type=0):
    """A GGUF checkpoint (bytes) of host-side Llama-shape weights (the dictionary the oracle model consumes: raw
    Q4_0 rows [n, k/32, 18] per linear, f32 embedding and gains) under llama.cpp's tensor names."""
    b = GgufBuilder()
    b.meta("general.architecture", "str", "llama").meta("llama.block_count", "u32", cfg.n_layer)
    b.meta("llama.embedding_length", "u32", cfg.d_model).meta("llama.attention.head_count", "u32", cfg.n_head)
    b.meta("llama.attention.head_count_kv", "u32", cfg.n_kv_head).meta("llama.feed_forward_length", "u32", cfg.d_ff)
    b.meta("llama.rope.freq_base", "f32", cfg.rope_base).meta("llama.attention.layer_norm_rms_epsilon", "f32", cfg.eps)
    b.meta("tokenizer.ggml.tokens", "arr", ("str", ["<t%d>" % i for i in range(8)]))

    def q4(name, raw):
        n, nb, _ = raw.shape
        b.tensor(name, [nb * 32, n], 2, np.ascontiguousarray(raw).tobytes())

    def plain(name, a):
        a = np.ascontiguousarray(a, np.float32)
        if embed_type == 1 and a.ndim == 2:
            b.tensor(name, list(a.shape[::-1]), 1, a.astype(np.float16).tobytes())
        else:
            b.tensor(name, list(a.shape[::-1]), 0, a.tobytes())

    plain("token_embd.weight", w["embed"])
    plain("output_norm.weight", w["norm_f"])
    q4("output.weight", w["lm_head"])
    names = (("wq", "attn_q"), ("wk", "attn_k"), ("wv", "attn_v"), ("wo", "attn_output"), ("wgate", "ffn_gate"), ("wup", "ffn_up"),
             ("wdown", "ffn_down"))
    for i, lw in enumerate(w["layers"]):
        plain("blk.%d.attn_norm.weight" % i, lw["norm1"])
        plain("blk.%d.ffn_norm.weight" % i, lw["norm2"])
        for key, gname in names:
            q4("blk.%d.%s.weight" % (i, gname), lw[key])
    return b.bytes()
