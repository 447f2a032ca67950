"""Known-answer blocks of every ggml format the readers dequantize.

The parameters (scales, quant patterns) are those of the reference's own block tests
(crates/wukong_runtime/src/gguf.rs:1889-2192): each block is packed here by the format's quantizer-side layout
and the expected lanes are the format's definition evaluated in float64 -- the values are chosen so that every
float32 product and sum is exact.  `known_blocks()` returns {ggml type id: (block bytes, expected float64 lanes)}."""
import numpy as np


def f16b(x):
    return np.array([x], np.float16).tobytes()


def pack_k4_scales(sc, mn):
    s = [0] * 12
    for j in range(8):
        if j < 4:
            s[j] = sc[j]
            s[j + 4] = mn[j]
        else:
            s[j + 4] = (sc[j] & 0xF) | ((mn[j] & 0xF) << 4)
            s[j - 4] |= (sc[j] >> 4) << 6
            s[j] |= (mn[j] >> 4) << 6
    return bytes(s)


K4_SC = [63, 1, 34, 17, 50, 33, 7, 62]
K4_MN = [0, 63, 5, 40, 63, 31, 48, 2]
IQ4NL = [-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113]


def known_blocks():
    out = {}
    # Q8_0: d = -0.5, q_j = 5j - 77 with the int8 extremes at the ends
    q = [5 * j - 77 for j in range(32)]
    q[0], q[31] = -128, 127
    out[8] = (f16b(-0.5) + bytes(v & 0xFF for v in q), [v * -0.5 for v in q])
    # Q4_0: d = 2, low nibble of byte j = j, high nibble = 15 - j
    out[2] = (f16b(2.0) + bytes(j | ((15 - j) << 4) for j in range(16)),
              [((e if e < 16 else 31 - e) - 8.0) * 2.0 for e in range(32)])
    # Q4_1: d = 0.25, m = -1.5, the same nibbles
    out[3] = (f16b(0.25) + f16b(-1.5) + bytes(j | ((15 - j) << 4) for j in range(16)),
              [(e if e < 16 else 31 - e) * 0.25 - 1.5 for e in range(32)])
    # Q5_0 / Q5_1: 5-bit values v_e = (7e + 3) % 32, fifth bit of element e at bit e of qh
    v = [(7 * e + 3) % 32 for e in range(32)]
    qh, qs = 0, []
    for j in range(16):
        qs.append((v[j] & 0xF) | ((v[j + 16] & 0xF) << 4))
        qh |= ((v[j] & 0x10) >> 4) << j
        qh |= ((v[j + 16] & 0x10) >> 4) << (j + 16)
    qhb = int(qh).to_bytes(4, "little")
    out[6] = (f16b(1.5) + qhb + bytes(qs), [(x - 16.0) * 1.5 for x in v])
    out[7] = (f16b(0.5) + f16b(-4.0) + qhb + bytes(qs), [x * 0.5 - 4.0 for x in v])
    # Q2_K: scale nibble (5g + 1) % 16, min nibble (3g + 7) % 16, quants (7e + e/16) % 4, d = 0.5, dmin = 0.25
    s = [(5 * g + 1) % 16 for g in range(16)]
    m = [(3 * g + 7) % 16 for g in range(16)]
    q2 = [(e * 7 + e // 16) % 4 for e in range(256)]
    blk = bytes(s[g] | (m[g] << 4) for g in range(16))
    for n in range(2):
        blk += bytes(q2[n * 128 + l] | (q2[n * 128 + l + 32] << 2) | (q2[n * 128 + l + 64] << 4) | (q2[n * 128 + l + 96] << 6)
                     for l in range(32))
    out[10] = (blk + f16b(0.5) + f16b(0.25), [0.5 * s[e // 16] * q2[e] - 0.25 * m[e // 16] for e in range(256)])
    # Q3_K: 6-bit scales (13g + 5) % 64 biased by 32, 3-bit values (3e + e/7) % 8 biased by 4, d = 0.25
    ls = [(13 * g + 5) % 64 for g in range(16)]
    lv = [(3 * e + e // 7) % 8 for e in range(256)]
    scales = [0] * 12
    for g, l in enumerate(ls):
        if g < 8:
            scales[g] = l & 0xF
        else:
            scales[g - 8] |= (l & 0xF) << 4
        scales[g % 4 + 8] |= (l >> 4) << (2 * (g // 4))
    hmask = [0] * 32
    for e, l in enumerate(lv):
        if l > 3:
            hmask[e % 32] |= 1 << (e // 32)
    qs3 = [0] * 64
    for n in range(2):
        for l in range(32):
            b = n * 128 + l
            qs3[n * 32 + l] = (lv[b] & 3) | ((lv[b + 32] & 3) << 2) | ((lv[b + 64] & 3) << 4) | ((lv[b + 96] & 3) << 6)
    out[11] = (bytes(hmask) + bytes(qs3) + bytes(scales) + f16b(0.25),
               [0.25 * (ls[e // 16] - 32.0) * (lv[e] - 4.0) for e in range(256)])
    # Q4_K: values (5e + e/32) % 16; Q5_K: values (11e + e/64) % 32; d = 0.5, dmin = 0.125
    k4 = pack_k4_scales(K4_SC, K4_MN)
    l4 = [(5 * e + e // 32) % 16 for e in range(256)]
    qs4 = [0] * 128
    for c in range(4):
        for l in range(32):
            qs4[c * 32 + l] = l4[c * 64 + l] | (l4[c * 64 + l + 32] << 4)
    out[12] = (f16b(0.5) + f16b(0.125) + k4 + bytes(qs4),
               [0.5 * K4_SC[e // 32] * l4[e] - 0.125 * K4_MN[e // 32] for e in range(256)])
    l5 = [(11 * e + e // 64) % 32 for e in range(256)]
    qh5, ql5 = [0] * 32, [0] * 128
    for c in range(4):
        for j in range(32):
            a, b = l5[c * 64 + j], l5[c * 64 + j + 32]
            if a > 15:
                a -= 16
                qh5[j] |= 1 << (2 * c)
            if b > 15:
                b -= 16
                qh5[j] |= 2 << (2 * c)
            ql5[c * 32 + j] = a | (b << 4)
    out[13] = (f16b(0.5) + f16b(0.125) + k4 + bytes(qh5) + bytes(ql5),
               [0.5 * K4_SC[e // 32] * l5[e] - 0.125 * K4_MN[e // 32] for e in range(256)])
    # Q6_K: signed scales per 16 (the int8 extremes first), values (9e + e/5) % 64 biased by 32, d = 0.0625
    sc6 = [-128 if g == 0 else 127 if g == 1 else (g - 8) * 9 for g in range(16)]
    lq = [(9 * e + e // 5) % 64 for e in range(256)]
    ql6, qh6 = [0] * 128, [0] * 64
    for n in range(2):
        for l in range(32):
            q1, q2_, q3, q4 = (lq[n * 128 + l + 32 * t] for t in range(4))
            ql6[n * 64 + l] = (q1 & 0xF) | ((q3 & 0xF) << 4)
            ql6[n * 64 + l + 32] = (q2_ & 0xF) | ((q4 & 0xF) << 4)
            qh6[n * 32 + l] = (q1 >> 4) | ((q2_ >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)
    out[14] = (bytes(ql6) + bytes(qh6) + bytes(x & 0xFF for x in sc6) + f16b(0.0625),
               [0.0625 * sc6[e // 16] * (lq[e] - 32.0) for e in range(256)])
    # Q8_K: f32 scale 0.375, quants (13e) % 256 as int8, 32 bytes of block sums the dequantizer ignores
    q8 = [((e * 13) % 256 + 128) % 256 - 128 for e in range(256)]
    out[15] = (np.array([0.375], "<f4").tobytes() + bytes(x & 0xFF for x in q8) + bytes([0xAB] * 32), [0.375 * x for x in q8])
    # IQ4_NL: d = 0.5, nibble (3e + 1) % 16 indexes the non-uniform levels
    nib = [(3 * e + 1) % 16 for e in range(32)]
    out[20] = (f16b(0.5) + bytes(nib[j] | (nib[j + 16] << 4) for j in range(16)), [0.5 * IQ4NL[x] for x in nib])
    # IQ4_XS: 6-bit scales (23b + 9) % 64 biased by 32, nibbles (5e + e/32) % 16, d = 0.25
    lsx = [(23 * b + 9) % 64 for b in range(8)]
    scales_h, scales_l = 0, [0] * 4
    for b, l in enumerate(lsx):
        scales_l[b // 2] |= (l & 0xF) << (4 * (b % 2))
        scales_h |= (l >> 4) << (2 * b)
    nibx = [(5 * e + e // 32) % 16 for e in range(256)]
    qsx = [0] * 128
    for b in range(8):
        for j in range(16):
            qsx[b * 16 + j] = nibx[b * 32 + j] | (nibx[b * 32 + j + 16] << 4)
    out[23] = (f16b(0.25) + int(scales_h).to_bytes(2, "little") + bytes(scales_l) + bytes(qsx),
               [0.25 * (lsx[e // 32] - 32.0) * IQ4NL[nibx[e]] for e in range(256)])
    return out


def random_blocks(rng, type_id, nblocks, nbytes):
    """Random block bytes with finite, moderate scales (every f16 / f32 scale field is overwritten)."""
    raw = rng.integers(0, 256, (nblocks, nbytes), dtype=np.uint8)

    def put_half(at, lo=-2.0, hi=2.0):
        raw[:, at:at + 2] = rng.uniform(lo, hi, nblocks).astype(np.float16).view(np.uint8).reshape(nblocks, 2)

    scale_at = {2: [0], 3: [0, 2], 6: [0], 7: [0, 2], 8: [0], 10: [80, 82], 11: [108], 12: [0, 2], 13: [0, 2], 14: [208],
                20: [0], 23: [0]}
    if type_id == 15:
        raw[:, 0:4] = rng.uniform(-2, 2, nblocks).astype("<f4").view(np.uint8).reshape(nblocks, 4)
    else:
        for at in scale_at[type_id]:
            put_half(at)
    return raw.reshape(-1)
