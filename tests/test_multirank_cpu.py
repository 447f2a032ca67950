"""The N > 1 path of the benchmark on CPU ranks (gloo, world size 2): every rank drives its own
scheduler over its own shard of the prompts, nothing is exchanged on the data path, and the job time
is the maximum over ranks."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    from wukong_b200.paged import Scheduler
    prompts = bench.shard_prompts(rank, 6, 1000)
    s = Scheduler(bcap=4, num_blocks=512, block_size=16, max_blocks_per_seq=40, max_rows=64, prefill_chunk=32)
    ids = [s.enqueue(p, 5) for p in prompts]
    steps = 0
    while not s.is_idle():
        n = s.plan_step()
        assert n > 0
        s.commit_step(((s.row_token[: s.bcap] + rank + steps) % 1000).astype(np.int32))
        steps += 1
    assert s.completed() == 6 and s.free_blocks() == 512 and s.emitted() == 30
    dist.barrier()
    ms = bench.max_over_ranks_ms(10.0 * (rank + 1), world, "cpu")
    digest = torch.tensor([float(sum(int(p.sum()) for p in prompts))], dtype=torch.float64)
    gathered = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, digest)
    if rank == 0:
        out.put((ms, [float(g.item()) for g in gathered], steps))
    dist.destroy_process_group()


def test_two_cpu_ranks_shard_and_reduce():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    ms, digests, steps = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ms == 20.0                       # the slowest rank defines the job time
    assert digests[0] != digests[1]         # ranks hold different sequences
    assert steps > 0
