"""Child program of tests/test_gpu_tp_peer.py (run under torch.distributed.run, one rank per GPU): the same
tensor-parallel Llama-shape decode steps once with NCCL all-reduces and once with the fused peer-memory
reduce + add + RMSNorm kernel; the two must agree (bit for bit on two ranks, where the sum has two terms)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from wukong_b200 import device as dev
from wukong_b200.llama import LlamaConfig, LlamaRankWeights, LlamaDecodeModel, PeerReduce


def main():
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = "cuda:%d" % local
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = LlamaConfig(n_layer=2, d_model=1024, n_head=8, n_kv_head=4, d_ff=2816, vocab=2048)
    w = LlamaRankWeights.synth_device(cfg, rank, world, 0, device)
    B, mbps = 16, 4

    def sum_in_rank_order(t):
        """The peer kernel adds the ranks' partials in rank order; NCCL's all-reduce gives the same bits only for two
        terms, so on more ranks the partials are gathered and added in rank order here too."""
        if world == 2:
            dist.all_reduce(t)
            return
        parts = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(parts, t.contiguous())
        acc = parts[0].clone()
        for r in range(1, world):
            acc += parts[r]
        t.copy_(acc)

    def make(peer):
        m = LlamaDecodeModel(cfg, w, rank, world, B, B * mbps, mbps, 16, device, sum_in_rank_order,
                             lambda a, b: dist.all_gather_into_tensor(b, a), peer)
        g = torch.Generator(device=device)
        g.manual_seed(5 + rank)
        m.kv.k.normal_(generator=g)
        m.kv.v.normal_(generator=g)
        m.block_table.copy_(torch.arange(B * mbps, dtype=torch.int32, device=device).view(B, mbps))
        m.row_token.copy_(torch.arange(B, dtype=torch.int32, device=device) * 37 % cfg.vocab)
        m.row_pos.fill_(20)
        m.row_ctx.fill_(21)
        return m

    peer = PeerReduce(rank, world, B, cfg.d_model, device)
    ma, mb = make(None), make(peer)
    torch.cuda.synchronize()
    dist.barrier()                      # every rank's buffers and mappings exist before the first peer kernel starts
    torch.cuda.synchronize()
    for _ in range(3):
        ta = ma.forward(B).clone()
        ma.advance(B)
        tb = mb.forward(B).clone()
        mb.advance(B)
        torch.cuda.synchronize()
        st = torch.tensor([dev.gemm_status()], dtype=torch.int32, device=device)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)            # a wait that ran out on any rank fails every rank
        assert int(st.item()) == 0
        assert torch.equal(ta, tb), "tokens differ between the NCCL and the peer-memory path"
        assert torch.equal(ma.x, mb.x), (ma.x - mb.x).abs().max().item()
    # every rank holds the same residual stream and the same tokens
    ref = mb.next_tok.clone()
    dist.broadcast(ref, 0)
    assert torch.equal(ref, mb.next_tok)
    dist.barrier()
    peer.close()
    dist.destroy_process_group()
    if rank == 0:
        print("tp_peer_check ok", flush=True)


if __name__ == "__main__":
    main()
