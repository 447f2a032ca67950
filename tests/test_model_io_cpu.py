"""Checkpoint readers on the host (no GPU): GGUF and safetensors through the C ABI.

The cases follow the reference's own reader tests (crates/wukong_runtime/src/gguf.rs:1538-2492,
crates/wukong_runtime/src/safetensors.rs:423-664): the files are assembled byte by byte by an independent writer
(oracle/model_io_ref.py), the block known answers carry the reference's parameters (tests/ggml_known_blocks.py)."""
import ctypes
import struct

import numpy as np
import pytest

from oracle import model_io_ref as R
from tests.ggml_known_blocks import known_blocks, random_blocks
from wukong_b200 import model_io as M

BAD, OPEN, IOERR, DTYPE, SHAPE, NONAME, NOTYPE = -6, -1, -2, -3, -4, -5, -7


def write(tmp_path, name, data):
    p = tmp_path / name
    p.write_bytes(data)
    return str(p)


def f16b(x):
    return np.array([x], np.float16).tobytes()


# ---- the oracle is pinned on the reference's known-answer blocks; the host reader must agree with both ----
def test_oracle_dequant_matches_the_known_blocks():
    kb = known_blocks()
    assert sorted(kb) == sorted(R.DEQUANT_IDS)
    for tid, (blk, want) in kb.items():
        assert len(blk) == R.GGML_TYPES[tid][2], tid
        got = R.dequant(tid, np.frombuffer(blk, np.uint8))
        assert np.array_equal(got.view(np.uint32), np.asarray(want, np.float64).astype(np.float32).view(np.uint32)), R.GGML_TYPES[tid][0]


def test_host_reader_dequantizes_the_known_blocks_and_random_blocks(tmp_path):
    rng = np.random.default_rng(5)
    b = R.GgufBuilder()
    cases = {}
    for tid, (blk, want) in known_blocks().items():
        name, per, nbytes = R.GGML_TYPES[tid]
        nb = 37
        raw = np.concatenate([np.frombuffer(blk, np.uint8), random_blocks(rng, tid, nb - 1, nbytes)])
        b.tensor(name, [per, nb], tid, raw.tobytes())
        cases[name] = (tid, raw, np.asarray(want, np.float64).astype(np.float32), per, nb)
    path = write(tmp_path, "blocks.gguf", b.bytes())
    for name, (tid, raw, want, per, nb) in cases.items():
        out = np.full((nb, per), np.nan, np.float32)
        assert M.gguf_read(path, name, out) == nb * per
        assert np.array_equal(out[0].view(np.uint32), want.view(np.uint32)), name
        assert np.array_equal(out.reshape(-1).view(np.uint32), R.dequant(tid, raw).view(np.uint32)), name
        rawout = np.zeros((nb, raw.size // nb), np.uint8)
        assert M.gguf_read(path, name, rawout) == raw.size
        assert np.array_equal(rawout.reshape(-1), raw)


def test_a_multi_block_dequant_streams_across_chunks(tmp_path):
    rng = np.random.default_rng(6)
    blocks = (1 << 12) + 3
    raw = random_blocks(rng, 2, blocks, 18)
    path = write(tmp_path, "long.gguf", R.GgufBuilder().tensor("long", [32 * blocks], 2, raw.tobytes()).bytes())
    out = np.zeros(32 * blocks, np.float32)
    assert M.gguf_read(path, "long", out) == 32 * blocks
    assert np.array_equal(out.view(np.uint32), R.dequant(2, raw).view(np.uint32))
    halves = rng.standard_normal((1 << 12) + 5).astype(np.float16)
    path = write(tmp_path, "halves.gguf", R.GgufBuilder().tensor("h", [halves.size], 1, halves.tobytes()).bytes())
    out = np.zeros(halves.size, np.float32)
    assert M.gguf_read(path, "h", out) == halves.size
    assert np.array_equal(out, halves.astype(np.float32))


# ---- the container ------------------------------------------------------------------------------------------
def good():
    return R.GgufBuilder().meta("k", "u32", 1).tensor("t", [4], 0, bytes(16))


def parse_code(tmp_path, data):
    """The header's verdict as the tensor-table readers report it: 0 when it parses."""
    rc = M.gguf_find(write(tmp_path, "case.gguf", data), "t")
    return 0 if rc >= 0 or rc == NONAME else rc


def test_malformed_headers_are_rejected(tmp_path):
    assert parse_code(tmp_path, good().bytes()) == 0
    cases = []
    b = good(); b.magic = b"GGUG"; cases.append(("bad magic", b.bytes()))
    for v in (0, 1, 4, 0x03000000):
        b = good(); b.version = v; cases.append(("version", b.bytes()))
    cases.append(("unknown value type", good().meta_raw("x", 13, bytes(8)).bytes()))
    cases.append(("unknown array element type", good().meta_raw("x", 9, struct.pack("<IQ", 99, 0)).bytes()))
    cases.append(("array count past the file", good().meta_raw("x", 9, struct.pack("<IQ", 0, 1 << 40)).bytes()))
    cases.append(("duplicate key", good().meta("k", "u8", 2).bytes()))
    cases.append(("duplicate tensor", good().tensor("t", [4], 0, bytes(16)).bytes()))
    cases.append(("five dims", good().tensor_at("five", [1, 1, 1, 1, 1], 0, 0).bytes()))
    cases.append(("dim above i64::MAX", good().tensor_at("huge", [1 << 63], 0, 0).bytes()))
    cases.append(("alignment of another type", good().meta("general.alignment", "u64", 32).bytes()))
    cases.append(("zero alignment", good().meta("general.alignment", "u32", 0).bytes()))
    cases.append(("alignment not a power of two", good().meta("general.alignment", "u32", 48).bytes()))
    cases.append(("string length past the file", R.GgufBuilder().meta_raw("s", 8, struct.pack("<Q", 1 << 62)).bytes()))
    nested = b"".join(struct.pack("<IQ", 9, 1) for _ in range(65)) + struct.pack("<IQ", 0, 0)
    cases.append(("arrays nested past the limit", R.GgufBuilder().meta_raw("deep", 9, nested).bytes()))
    for what, data in cases:
        assert parse_code(tmp_path, data) == BAD, what
        assert M.gguf_meta_type(write(tmp_path, "case.gguf", data), "k") == BAD, what     # the full parse agrees
    full = good().header()
    for cut in range(len(full)):
        assert parse_code(tmp_path, full[:cut]) == BAD, cut
    # 64 arrays inside one another are allowed, the 65th is not
    for levels, verdict in ((63, 0), (64, BAD)):
        deep = b"".join(struct.pack("<IQ", 9, 1) for _ in range(levels)) + struct.pack("<IQ", 0, 0)
        assert parse_code(tmp_path, R.GgufBuilder().meta_raw("deep", 9, deep).bytes()) == verdict, levels


def test_alignment_and_data_start(tmp_path):
    w = np.arange(8, dtype=np.float32)
    for align in (8, 32, 256):
        b = R.GgufBuilder(align=align)
        if align != 32:
            b.meta("general.alignment", "u32", align)
        b.meta("pad", "str", "x" * 5).tensor("a", [3], 0, w[:3].tobytes()).tensor("b", [5], 0, w[3:].tobytes())
        path = write(tmp_path, "al.gguf", b.bytes())
        out = np.zeros(5, np.float32)
        assert M.gguf_read(path, "b", out) == 5 and np.array_equal(out, w[3:])
    # version 2 parses like version 3
    path = write(tmp_path, "v2.gguf", R.GgufBuilder(version=2).tensor("a", [3], 0, w[:3].tobytes()).bytes())
    out = np.zeros(3, np.float32)
    assert M.gguf_read(path, "a", out) == 3 and np.array_equal(out, w[:3])


def test_locate_checks_the_named_tensor_only(tmp_path):
    b = (R.GgufBuilder().tensor("ok", [32, 2], 8, bytes(68)).tensor_at("odd_row", [48], 8, 128).tensor_at("misaligned", [4], 0, 8)
         .tensor_at("past_end", [4], 0, 4096).tensor_at("unknown", [4], 4, 0).tensor_at("retired", [4], 33, 0)
         .tensor_at("future", [4], 1000, 0))
    data = b.bytes()
    path = write(tmp_path, "loc.gguf", data)
    out = np.zeros((2, 32), np.float32)
    assert M.gguf_read(path, "ok", out) == 64
    assert M.gguf_read(path, "ok", np.zeros((2, 34), np.uint8)) == 68
    f4 = np.zeros(4, np.float32)
    for name in ("odd_row", "misaligned", "past_end"):
        assert M.gguf_read(path, name, np.zeros(48 if name == "odd_row" else 4, np.float32)) == BAD, name
    for name in ("unknown", "retired", "future"):
        assert M.gguf_read(path, name, f4) == NOTYPE, name
        assert M.gguf_dim(path, name, 0) == 4          # the queries still answer
    assert M.gguf_type(path, "future") == 1000
    assert M.gguf_read(path, "absent", f4) == NONAME
    short = write(tmp_path, "short.gguf", data[:-1])   # the payload must lie inside the file: one byte short
    assert M.gguf_read(short, "ok", out) == BAD


def sample_file():
    w = np.array([1.0, -2.0, 3.0, 0.5, -0.25, 8.0], np.float32)
    hb = np.array([1.0, -0.5, 65504.0, 0.0], np.float16).tobytes()
    bb = np.array([0x3F80, 0xC040], "<u2").tobytes()
    qb, qv = b"", []
    for r, d in ((0, 0.5), (1, -2.0)):
        qb += f16b(d)
        for j in range(32):
            q = (j * 3 + r * 11) % 41 - 20
            qb += bytes([q & 0xFF])
            qv.append(q * d)
    ib = np.array([-1, 300, -32768], "<i2").tobytes()
    b = (R.GgufBuilder().meta("general.architecture", "str", "tiny").tensor("w", [3, 2], 0, w.tobytes()).tensor("h", [4], 1, hb)
         .tensor("b", [2], 30, bb).tensor("q", [32, 2], 8, qb).tensor("iq", [256], 16, bytes(66)).tensor("i", [3], 25, ib))
    return b.bytes(), np.array(qv, np.float32), np.frombuffer(qb, np.uint8)


def read(path, name, out, dt, dims):
    arr = (ctypes.c_int64 * max(1, len(dims)))(*dims) if dims is not None else None
    from wukong_b200._lib import lib
    return int(lib().wukong_rt_gguf_read(path.encode(), name.encode(), out.ctypes.data, out.size, dt, arr, len(dims) if dims is not None else -1))


def test_gguf_read_routes_every_type_and_checks_the_destination(tmp_path):
    data, qv, qb = sample_file()
    path = write(tmp_path, "s.gguf", data)
    F32, F64, F16, BF16, I8, I16, I32, U8 = 0, 1, 2, 3, 4, 5, 6, 8
    w = np.zeros(6, np.float32)
    assert read(path, "w", w, F32, [2, 3]) == 6 and w.tolist() == [1.0, -2.0, 3.0, 0.5, -0.25, 8.0]
    keep = np.full(6, 9, np.float32)
    assert read(path, "w", keep, F32, [3, 2]) == SHAPE
    assert read(path, "w", keep[:5], F32, None) == SHAPE
    assert keep.tolist() == [9.0] * 6
    h = np.zeros(4, np.float32)
    assert read(path, "h", h, F32, None) == 4 and h.tolist() == [1.0, -0.5, 65504.0, 0.0]
    hraw = np.zeros(4, np.uint16)
    assert read(path, "h", hraw, F16, None) == 4 and hraw.tolist() == [0x3C00, 0xB800, 0x7BFF, 0]
    bf = np.zeros(2, np.float32)
    assert read(path, "b", bf, F32, [2]) == 2 and bf.tolist() == [1.0, -3.0]
    braw = np.zeros(2, np.uint16)
    assert read(path, "b", braw, BF16, None) == 2 and braw.tolist() == [0x3F80, 0xC040]
    q = np.zeros(64, np.float32)
    assert read(path, "q", q, F32, [2, 32]) == 64 and np.array_equal(q, qv)
    raw = np.zeros(68, np.uint8)
    assert read(path, "q", raw, U8, [2, 34]) == 68 and np.array_equal(raw, qb)
    assert read(path, "q", raw, U8, [2, 32]) == SHAPE
    assert read(path, "q", raw, U8, None) == 68
    i = np.zeros(3, np.int16)
    assert read(path, "i", i, I16, None) == 3 and i.tolist() == [-1, 300, -32768]
    assert read(path, "i", np.full(3, 7, np.int32), I32, None) == DTYPE
    assert read(path, "w", np.zeros(6, np.float64), F64, None) == DTYPE
    assert read(path, "q", np.zeros(64, np.int8), I8, None) == DTYPE
    assert read(path, "w", np.zeros(24, np.uint8), U8, None) == DTYPE
    iq = np.full(256, 5, np.float32)
    assert read(path, "iq", iq, F32, None) == NOTYPE and iq.tolist() == [5.0] * 256
    assert read(path, "iq", np.ones(66, np.uint8), U8, None) == 66
    assert read(path, "absent", w, F32, None) == NONAME
    assert read(str(tmp_path / "wukong_gguf_absent_zz.gguf"), "w", w, F32, None) == OPEN
    assert read(write(tmp_path, "bad.gguf", b"GGUF\x01\x00\x00\x00"), "w", w, F32, None) == BAD
    assert read(write(tmp_path, "cut.gguf", data[:-1]), "i", i, I16, None) == BAD
    # the queries
    assert M.gguf_find(path, "q") == 3 and M.gguf_rank(path, "q") == 2
    assert (M.gguf_dim(path, "q", 0), M.gguf_dim(path, "q", 1)) == (2, 32)
    assert M.gguf_dim(path, "q", 2) == SHAPE and M.gguf_dim(path, "q", -1) == SHAPE
    assert M.gguf_type(path, "iq") == 16 and M.gguf_type(path, "nope") == NONAME
    from wukong_b200._lib import lib
    assert lib().wukong_rt_gguf_query(None, None, 0, 0) == OPEN
    assert lib().wukong_rt_gguf_query(path.encode(), b"q", 9, 0) == IOERR


def test_metadata_accessors_read_every_kind_and_fall_back_to_the_default(tmp_path):
    from wukong_b200._lib import lib
    b = (R.GgufBuilder().meta("general.architecture", "str", "llama").meta("llama.block_count", "u32", 12)
         .meta("llama.rope.freq_base", "f32", 10000.0).meta("big", "u64", (1 << 64) - 1).meta("flag", "bool", 1).meta("neg", "i8", -5)
         .meta("tokens", "arr", ("str", ["<s>", "wukong"])).meta("scores", "arr", ("f32", [0.5, -1.25]))
         .meta("ids", "arr", ("i32", [3, -4])))
    path = write(tmp_path, "meta.gguf", b.bytes())
    assert M.gguf_meta_type(path, "llama.block_count") == 4 and M.gguf_meta_type(path, "tokens") == 9
    assert M.gguf_meta_type(path, "absent") == NONAME
    assert M.gguf_meta_len(path, "general.architecture") == 5 and M.gguf_meta_len(path, "tokens") == 2
    assert M.gguf_meta_len(path, "flag") == 1 and M.gguf_meta_len(path, "absent") == NONAME
    geti = lambda k, i: M.gguf_meta_i64(path, k, i, -77)
    assert geti("llama.block_count", 0) == 12
    assert geti("big", 0) == -1           # a u64 keeps its bits
    assert geti("flag", 0) == 1 and geti("neg", 0) == -5 and geti("ids", 1) == -4
    for k, i in (("ids", 2), ("ids", -1), ("llama.block_count", 1), ("llama.rope.freq_base", 0), ("tokens", 0), ("absent", 0)):
        assert geti(k, i) == -77, (k, i)
    getf = lambda k, i: M.gguf_meta_f64(path, k, i, -0.5)
    assert getf("llama.rope.freq_base", 0) == 10000.0 and getf("scores", 1) == -1.25
    assert getf("llama.block_count", 0) == 12.0
    assert getf("big", 0) == float((1 << 64) - 1)       # a u64 converts by its unsigned value
    assert getf("flag", 0) == -0.5 and getf("general.architecture", 0) == -0.5
    assert M.gguf_meta_str(path, "tokens", 1) == b"wukong"
    assert M.gguf_meta_str(path, "tokens", 2) == SHAPE
    assert M.gguf_meta_str(path, "ids", 0) == DTYPE
    assert M.gguf_meta_str(path, "absent", 0) == NONAME
    buf = ctypes.create_string_buffer(b"\xaa" * 4, 4)
    assert lib().wukong_rt_gguf_meta_str(path.encode(), b"general.architecture", 0, buf, 4) == 5 and buf.raw == b"lla\0"
    keep = ctypes.create_string_buffer(b"\xaa" * 4, 4)
    assert lib().wukong_rt_gguf_meta_str(path.encode(), b"ids", 0, keep, 4) == DTYPE and keep.raw == b"\xaa" * 4
    assert lib().wukong_rt_gguf_meta_str(path.encode(), b"general.architecture", 0, keep, 0) == 5 and keep.raw == b"\xaa" * 4
    assert lib().wukong_rt_gguf_meta(None, b"general.architecture", 2, 0, 9) == 9
    assert lib().wukong_rt_gguf_meta(None, b"general.architecture", 0, 0, 9) == OPEN
    assert lib().wukong_rt_gguf_meta_f64(None, b"general.architecture", 0, 2.5) == 2.5
    # the tensor-table readers step over the metadata they do not keep and agree with the full parse
    b.tensor("t", [2], 0, np.array([1.5, -2.5], np.float32).tobytes())
    path = write(tmp_path, "meta_t.gguf", b.bytes())
    out = np.zeros(2, np.float32)
    assert M.gguf_read(path, "t", out) == 2 and out.tolist() == [1.5, -2.5]
    assert M.gguf_meta_i64(path, "ids", 0, 0) == 3


# ---- safetensors ----------------------------------------------------------------------------------------------
def st_read(path, name, out, dt, dims):
    from wukong_b200._lib import lib
    arr = (ctypes.c_int64 * max(1, len(dims)))(*dims) if dims is not None else None
    return int(lib().wukong_rt_st_read(path.encode(), name.encode(), out.ctypes.data, out.size, dt, arr, len(dims) if dims is not None else -1))


def st_code(tmp_path, header, payload=bytes(16), name="a"):
    return st_read(write(tmp_path, "c.safetensors", R.st_file(header, payload)), name, np.zeros(1, np.float32), 0, None)


def test_safetensors_json_grammar(tmp_path):
    entry = '"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}'
    ok = ['{%s,"x":[1, 0, 18446744073709551615]}', '{%s,"x":{"c":"x\\"\\u00e9\\ud83d\\ude00"}}', '{%s,"x":[true, false, null, -1, 2.5, 1e3]}',
          ' {%s,"x":18446744073709551616} ', '{%s,"x":' + "[" * 63 + "]" * 63 + "}"]
    for h in ok:
        assert st_code(tmp_path, h % entry) == 1, h
    bad = ['{%s,"x":{}', '{%s,"x":{"a" 1}}', '{%s,"x":[1,]}', '{%s,"x":{"a":1,}}', '{%s,"x":01}', '{%s,"x":"\x01"}', '{%s,"x":"\\ud800"}',
           '{%s,"x":"\\q"}', '{%s,"x":tru}', '{%s} x', '{%s,"x":' + "[" * 64 + "]" * 64 + "}", '{%s,"x":"\\udc00"}', '{%s,"x":-}', '{%s,"x":1.}']
    for h in bad:
        assert st_code(tmp_path, h % entry) == BAD, h
    assert st_code(tmp_path, b'{' + entry.encode() + b',"x":"\xff"}') == BAD        # not UTF-8
    assert st_code(tmp_path, b"") == BAD


def test_safetensors_locate(tmp_path):
    header = '{"__metadata__":{"format":"pt"},"b":{"dtype":"BF16","shape":[2],"data_offsets":[8,12]},"a":{"dtype":"F32","shape":[2],"data_offsets":[0,8]}}  '
    payload = np.array([1.5, -2.0], "<f4").tobytes() + np.array([0x3F80, 0xC040], "<u2").tobytes()
    data = R.st_file(header, payload)
    path = write(tmp_path, "l.safetensors", data)
    a = np.zeros(2, np.float32)
    assert st_read(path, "a", a, 0, [2]) == 2 and a.tolist() == [1.5, -2.0]
    assert st_read(path, "b", a, 0, None) == 2 and a.tolist() == [1.0, -3.0]
    assert st_read(path, "c", a, 0, None) == NONAME
    assert st_read(path, "__metadata__", a, 0, None) == NONAME
    assert st_read(write(tmp_path, "cut.safetensors", data[:-1]), "b", a, 0, None) == BAD
    cases = ['{"a":{"dtype":"F32","shape":[2],"data_offsets":[0,4]}}', '{"a":{"dtype":"F32","shape":[1],"data_offsets":[4,0]}}',
             '{"a":{"dtype":"F32","shape":[1]}}', '{"a":{"dtype":"F32","shape":[-1],"data_offsets":[0,4]}}',
             '{"a":{"dtype":3,"shape":[1],"data_offsets":[0,4]}}',
             '{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}', '["a"]', '{"a":']
    for h in cases:
        assert st_code(tmp_path, h) == BAD, h
    assert st_read(write(tmp_path, "long.safetensors", struct.pack("<Q", 1000) + b"{}"), "a", a, 0, None) == BAD
    assert st_read(write(tmp_path, "tiny.safetensors", bytes(4)), "a", a, 0, None) == BAD
    # a dtype with no element type here is located, then refused by the destination check
    assert st_code(tmp_path, '{"a":{"dtype":"BOOL","shape":[3],"data_offsets":[0,3]}}', bytes([1, 0, 1])) == DTYPE
    # rank 0: one element
    one = np.zeros(1, np.float32)
    p0 = write(tmp_path, "s0.safetensors", R.st_file('{"a":{"dtype":"F32","shape":[],"data_offsets":[0,4]}}', np.array([7.0], "<f4").tobytes()))
    assert st_read(p0, "a", one, 0, []) == 1 and one[0] == 7.0


def test_st_read_loads_verbatim_widens_halves_and_checks_the_destination(tmp_path):
    payload = np.array([0x3F80, 0xC000, 0x3F00, 0x4040], "<u2").tobytes() + np.array([-1, 2, 300], "<i2").tobytes()
    header = '{"w":{"dtype":"BF16","shape":[2,2],"data_offsets":[0,8]},"n":{"dtype":"I16","shape":[3],"data_offsets":[8,14]}}'
    path = write(tmp_path, "st.safetensors", R.st_file(header, payload))
    out = np.zeros(4, np.float32)
    assert st_read(path, "w", out, 0, [2, 2]) == 4 and out.tolist() == [1.0, -2.0, 0.5, 3.0]
    raw = np.zeros(4, np.uint16)
    assert st_read(path, "w", raw, 3, None) == 4 and raw.tolist() == [0x3F80, 0xC000, 0x3F00, 0x4040]
    ints = np.zeros(3, np.int16)
    assert st_read(path, "n", ints, 5, None) == 3 and ints.tolist() == [-1, 2, 300]
    keep = np.full(4, 9, np.float32)
    assert st_read(path, "w", keep, 0, [4]) == SHAPE
    assert st_read(path, "w", keep[:3], 0, None) == SHAPE
    assert st_read(path, "n", keep[:3], 0, None) == DTYPE
    assert keep.tolist() == [9.0] * 4
    assert st_read(str(tmp_path / "wukong_st_absent_zz.safetensors"), "w", keep, 0, None) == OPEN
    # f16 widening, subnormals and infinities included
    h = np.array([1.0, -0.5, 65504.0, 0.0, 6e-8, -6.1e-5, np.inf, -np.inf], np.float16)
    p = write(tmp_path, "h.safetensors", R.st_file({"h": {"dtype": "F16", "shape": [8], "data_offsets": [0, 16]}}, h.tobytes()))
    out = np.zeros(8, np.float32)
    assert st_read(p, "h", out, 0, [8]) == 8 and np.array_equal(out, h.astype(np.float32))
