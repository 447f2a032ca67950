"""GPU parity of the checkpoint loaders: tensors of GGUF / safetensors files straight into device memory.

Bit-exact bars: the device dequantizers against the numpy oracle (pinned on the reference's known-answer blocks,
crates/wukong_runtime/src/gguf.rs:1889-2192) and against the host reader of the same library; the loaded Llama-shape
weights against the ones built from the same arrays in memory."""
import numpy as np
import pytest

from oracle import model_io_ref as R
from tests.ggml_known_blocks import known_blocks, random_blocks

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def io():
    from wukong_b200 import _lib, model_io
    _lib.require_gpu()
    return model_io


def write(tmp_path, name, data):
    p = tmp_path / name
    p.write_bytes(data)
    return str(p)


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_device_dequant_every_block_format(io, tmp_path):
    import torch
    from wukong_b200._lib import lib, check
    rng = np.random.default_rng(11)
    b = R.GgufBuilder()
    cases = {}
    for tid, (blk, want) in known_blocks().items():
        name, per, nbytes = R.GGML_TYPES[tid]
        nb = 4099                                  # not a multiple of anything the kernels tile by
        raw = np.concatenate([np.frombuffer(blk, np.uint8), random_blocks(rng, tid, nb - 1, nbytes)])
        b.tensor(name, [per, nb], tid, raw.tobytes())
        cases[name] = (tid, raw, np.asarray(want, np.float64).astype(np.float32), per, nb)
    path = write(tmp_path, "blocks.gguf", b.bytes())
    for name, (tid, raw, want, per, nb) in cases.items():
        out = torch.full((nb, per), float("nan"), device="cuda")
        io.gguf_read_device(path, name, out)
        got = out.cpu().numpy()
        assert np.array_equal(bits(got[0]), bits(want)), name
        assert np.array_equal(bits(got.reshape(-1)), bits(R.dequant(tid, raw))), name
        host = np.zeros((nb, per), np.float32)
        assert io.gguf_read(path, name, host) == nb * per
        assert np.array_equal(bits(got), bits(host)), name
        # the kernel on blocks already resident
        d_raw = torch.from_numpy(raw).cuda()
        again = torch.empty(nb * per, device="cuda")
        check(lib().wkb_ggml_dequant_f32(tid, d_raw.data_ptr(), nb, again.data_ptr(), torch.cuda.current_stream().cuda_stream), "dequant")
        assert torch.equal(again, out.view(-1)), name
        rawdev = torch.zeros((nb, raw.size // nb), dtype=torch.uint8, device="cuda")
        io.gguf_read_device(path, name, rawdev)
        assert np.array_equal(rawdev.cpu().numpy().reshape(-1), raw), name


def test_device_reads_route_every_type_and_check_the_destination(io, tmp_path):
    import torch
    rng = np.random.default_rng(12)
    w = rng.standard_normal((5, 7)).astype(np.float32)
    h = rng.standard_normal(1001).astype(np.float16)
    bf = (rng.standard_normal(33).astype(np.float32).view(np.uint32) >> 16).astype("<u2")
    i16 = rng.integers(-30000, 30000, 9).astype("<i2")
    b = (R.GgufBuilder().tensor("w", [7, 5], 0, w.tobytes()).tensor("h", [1001], 1, h.tobytes()).tensor("b", [33], 30, bf.tobytes())
         .tensor("i", [9], 25, i16.tobytes()).tensor("iq", [256], 16, bytes(66)))
    path = write(tmp_path, "s.gguf", b.bytes())
    out = io.gguf_read_device(path, "w", torch.zeros((5, 7), device="cuda"))
    assert np.array_equal(out.cpu().numpy(), w)
    out = io.gguf_read_device(path, "h", torch.zeros(1001, device="cuda"))
    assert np.array_equal(out.cpu().numpy(), h.astype(np.float32))
    out = io.gguf_read_device(path, "h", torch.zeros(1001, dtype=torch.float16, device="cuda"))
    assert np.array_equal(out.cpu().numpy(), h)
    out = io.gguf_read_device(path, "b", torch.zeros(33, device="cuda"))
    assert np.array_equal(bits(out.cpu().numpy()), bf.astype(np.uint32) << 16)
    out = io.gguf_read_device(path, "b", torch.zeros(33, dtype=torch.bfloat16, device="cuda"))
    assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), bf)
    out = io.gguf_read_device(path, "i", torch.zeros(9, dtype=torch.int16, device="cuda"))
    assert np.array_equal(out.cpu().numpy(), i16)
    keep = torch.full((7, 5), 9.0, device="cuda")
    for name, dest, code in (("w", keep, -4), ("w", torch.zeros(34, device="cuda"), -4), ("i", torch.zeros(9, dtype=torch.int32, device="cuda"), -3),
                             ("iq", torch.zeros(256, device="cuda"), -7), ("absent", keep, -5)):
        with pytest.raises(io.ModelIOError) as e:
            io.gguf_read_device(path, name, dest)
        assert e.value.code == code, name
    assert bool((keep == 9.0).all())
    with pytest.raises(io.ModelIOError) as e:
        io.gguf_read_device(str(tmp_path / "absent.gguf"), "w", keep)
    assert e.value.code == -1


def test_payload_larger_than_the_staging_buffers(io, tmp_path):
    """40 MiB of Q8_0 blocks and of bf16 halves: several chunks through both staging slots."""
    import torch
    rng = np.random.default_rng(13)
    blocks = (40 << 20) // 34 + 5
    raw = random_blocks(rng, 8, blocks, 34)
    halves = rng.integers(0, 1 << 16, (20 << 20) + 3, dtype=np.uint16)
    halves[(halves & 0x7F80) == 0x7F80] = 0          # no NaN payloads in the comparison
    b = R.GgufBuilder().tensor("q", [32, blocks], 8, raw.tobytes()).tensor("b", [halves.size], 30, halves.tobytes())
    path = write(tmp_path, "big.gguf", b.bytes())
    out = io.gguf_read_device(path, "q", torch.empty((blocks, 32), device="cuda"))
    assert np.array_equal(bits(out.cpu().numpy().reshape(-1)), bits(R.dequant(8, raw)))
    rawdev = io.gguf_read_device(path, "q", torch.empty((blocks, 34), dtype=torch.uint8, device="cuda"))
    assert np.array_equal(rawdev.cpu().numpy().reshape(-1), raw)
    out = io.gguf_read_device(path, "b", torch.empty(halves.size, device="cuda"))
    assert np.array_equal(bits(out.cpu().numpy()), halves.astype(np.uint32) << 16)


def test_safetensors_into_device_memory(io, tmp_path):
    import torch
    rng = np.random.default_rng(14)
    w = rng.standard_normal((64, 48)).astype(np.float32)
    h = rng.standard_normal((3, 5)).astype(np.float16)
    header = {"__metadata__": {"format": "pt"}, "w": {"dtype": "F32", "shape": [64, 48], "data_offsets": [0, w.nbytes]},
              "h": {"dtype": "F16", "shape": [3, 5], "data_offsets": [w.nbytes, w.nbytes + h.nbytes]}}
    path = write(tmp_path, "m.safetensors", R.st_file(header, w.tobytes() + h.tobytes()))
    out = io.st_read_device(path, "w", torch.zeros((64, 48), device="cuda"))
    assert np.array_equal(out.cpu().numpy(), w)
    out = io.st_read_device(path, "h", torch.zeros((3, 5), device="cuda"))
    assert np.array_equal(out.cpu().numpy(), h.astype(np.float32))
    with pytest.raises(io.ModelIOError) as e:
        io.st_read_device(path, "w", torch.zeros((48, 64), device="cuda"))
    assert e.value.code == -4


def test_llama_weights_from_a_gguf_checkpoint(io, tmp_path):
    """The same arrays through a GGUF file and through memory give identical resident weights, on every rank
    of a tensor-parallel split; the step of the loaded model produces the in-memory model's tokens."""
    import torch
    from wukong_b200.llama import LlamaConfig, LlamaRankWeights, synth_llama_raw, llama_config_from_gguf
    cfg = LlamaConfig(n_layer=2, d_model=256, n_head=4, n_kv_head=2, d_ff=512, vocab=320)
    w = synth_llama_raw(cfg, 3, 0.008)
    path = write(tmp_path, "tiny_llama.gguf", R.write_llama_gguf(cfg, w))
    got_cfg = llama_config_from_gguf(path)
    assert (got_cfg.n_layer, got_cfg.d_model, got_cfg.n_head, got_cfg.n_kv_head, got_cfg.d_ff, got_cfg.vocab) == (2, 256, 4, 2, 512, 320)
    for rank, world in ((0, 1), (1, 2)):
        a = LlamaRankWeights.from_raw(cfg, w, rank, world, "cuda")
        b = LlamaRankWeights.from_gguf(path, None, rank, world, "cuda")
        assert torch.equal(a.embed, b.embed) and torch.equal(a.norm_f, b.norm_f)
        assert torch.equal(a.lm_head.tiled, b.lm_head.tiled)
        for la, lb in zip(a.layers, b.layers):
            for key in ("wqkv", "wo", "wgu", "wdown"):
                assert (la[key].n, la[key].k) == (lb[key].n, lb[key].k) and torch.equal(la[key].tiled, lb[key].tiled), key
            assert torch.equal(la["norm1"], lb["norm1"]) and torch.equal(la["norm2"], lb["norm2"])
    # an f16 embedding table widens on the device
    path16 = write(tmp_path, "tiny_llama_f16.gguf", R.write_llama_gguf(cfg, w, embed_type=1))
    c = LlamaRankWeights.from_gguf(path16, cfg, 0, 1, "cuda")
    assert np.array_equal(c.embed.cpu().numpy(), w["embed"].astype(np.float16).astype(np.float32))
    # a linear that is not Q4_0 is refused, not converted
    bad = R.GgufBuilder().tensor("x", [32, 2], 8, bytes(68))
    with pytest.raises(io.ModelIOError):
        io.gguf_load_q4_weight(write(tmp_path, "q8.gguf", bad.bytes()), "x")
    q = io.gguf_load_q4_weight(path, "blk.0.ffn_down.weight")
    assert (q.n, q.k) == (256, 512)
