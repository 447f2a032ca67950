"""Input constructions of the reference's end-to-end fixtures, rebuilt from their documented
formulas (tests/run/*.wk of the reference).  Shared by the oracle tests (CPU) and the parity tests
(GPU): each function returns the operands, and `expect_out.json` holds the printed values."""
import numpy as np

NAN = np.float32(np.nan)


def rust_round(x):
    """f32::round: half away from zero."""
    x = np.asarray(x, np.float64)
    return (np.sign(x) * np.floor(np.abs(x) + 0.5)).astype(np.int64)


def activations_x():
    x = (np.arange(13, dtype=np.float32) * np.float32(0.5) - np.float32(3.0)).astype(np.float32)
    return x, (x + np.float32(3.5)).astype(np.float32)


def gemv_half_operands():
    w = np.zeros((11, 13), np.float32)
    for j in range(11):
        for p in range(13):
            w[j, p] = (((j * 7 + p * 3 + (j * p) % 5) % 9) - 4.0) * 0.5
    x = np.array([(i % 5) - 2 for i in range(13)], np.float32)
    return w, x


def gemv_quant_operands():
    w8 = np.zeros((9, 40), np.float32)
    w4 = np.zeros((9, 40), np.float32)
    for j in range(9):
        for e in range(40):
            if e in (1, 33):
                w8[j, e], w4[j, e] = 127.0, -8.0
            else:
                w8[j, e] = ((j * 7 + e * 3) % 13) - 6
                w4[j, e] = ((j * 7 + e * 3) % 15) - 7
    x = np.array([127.0 if i in (0, 32) else (i % 9) - 4 for i in range(40)], np.float32)
    return w8, w4, x


def kv_batch_operands():
    lens, pos = [4, 1, 0], [2, -1, 0]
    k = np.zeros(96, np.float32)
    v = np.zeros(96, np.float32)
    for b in range(3):
        for j in range(4):
            for g in range(2):
                for c in range(4):
                    at = ((b * 4 + j) * 2 + g) * 4 + c
                    if j < lens[b]:
                        k[at] = 1.0 if c == j else 0.0
                        v[at] = 1000 * b + 100 * g + 10 * j + c
                    else:
                        k[at] = v[at] = NAN
    q = np.zeros(96, np.float32)
    qi = lambda b, i, h, c: ((b * 2 + i) * 4 + h) * 4 + c
    q[qi(0, 0, 0, 3)] = 200; q[qi(0, 0, 0, 1)] = 100; q[qi(0, 0, 1, 2)] = 200
    q[qi(0, 0, 2, 0)] = 200; q[qi(0, 0, 3, 1)] = 200
    q[qi(0, 1, 0, 3)] = 200; q[qi(0, 1, 2, 2)] = 200
    for h in range(4):
        q[qi(1, 0, h, 0)] = 200
    q[qi(1, 1, 0, 3)] = 200; q[qi(1, 1, 1, 0)] = 200
    q[64:96] = 1.0
    return dict(q=q, k=k, v=v, lens=lens, pos=pos, geo=(3, 2, 4, 4, 2, 4))


def kv_batch_gqa_operands():
    lens, pos = [2, 3], [1, 2]
    k = np.zeros(48, np.float32)
    v = np.zeros(48, np.float32)
    for b in range(2):
        for j in range(3):
            for g in range(2):
                for c in range(4):
                    at = ((b * 3 + j) * 2 + g) * 4 + c
                    if j < lens[b]:
                        k[at] = 1.0 if c == j else 0.0
                        v[at] = 1000 * b + 100 * g + 10 * j + c
                    else:
                        k[at] = v[at] = NAN
    q = np.zeros(64, np.float32)
    for h in range(8):
        t, s0, s1 = h % 4, h * 4, 32 + h * 4
        if t == 0:
            q[s0] = 200; q[s1 + 2] = 200
        if t == 1:
            q[s0 + 1] = 200; q[s1 + 1] = 200
        if t == 2:
            q[s0 + 2] = 200; q[s1] = 200
        if t == 3:
            q[s0 + 1] = 200; q[s0] = 100; q[s1 + 3] = 200; q[s1 + 2] = 100
    return dict(q=q, k=k, v=v, lens=lens, pos=pos, geo=(2, 1, 3, 8, 2, 4))


def kv_attention_steps():
    """Yields the per-step operands of the single-sequence decode fixture, then the chunked call."""
    kc = np.zeros(32, np.float32)
    vc = np.zeros(32, np.float32)
    steps = []
    for t in range(4):
        krow = np.zeros(8, np.float32)
        vrow = np.zeros(8, np.float32)
        for c in range(4):
            krow[c] = 1.0 if c == t else 0.0
            krow[4 + c] = 1.0 if c == 3 - t else 0.0
            vrow[c] = 10 * t + c
            vrow[4 + c] = 10 * t + 100 + c
        q = np.zeros(16, np.float32)
        q[t] = 200; q[4] = 200; q[8 + 3 - t] = 200; q[15] = 200
        steps.append(dict(krow=krow, vrow=vrow, q=q, t=t))
    q2 = np.zeros(40, np.float32)
    for r in range(2):
        base = r * 20
        q2[base + 3] = 200; q2[base + 1] = 100; q2[base + 8] = 200; q2[base + 10] = 100
    q2[6] = 200; q2[15] = 200
    return kc, vc, steps, q2
