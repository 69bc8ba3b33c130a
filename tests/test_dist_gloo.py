"""Two CPU ranks over gloo: the batch-sharded forward needs no collective on the data path,
and the shards put side by side equal the unsharded result bit for bit."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import reference_port as R
from trinix_b200.sharding import shard, shard_bounds


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(0)  # every rank draws the same full batch
    x = torch.randn(6, 16, 256, generator=g).bfloat16()
    w = (1 + 0.02 * torch.randn(256, generator=g)).bfloat16()
    mine = shard(x, rank, world)
    codes, scales = R.rmsnorm_quantize_ref(mine, w, 1e-6)  # the data path: no communication
    # the only communication is the untimed gather used for checking
    sizes = [shard_bounds(6, r, world) for r in range(world)]
    gathered = [torch.empty((hi - lo, 16, 256), dtype=torch.int8) for lo, hi in sizes]
    dist.all_gather(gathered, codes) if len({hi - lo for lo, hi in sizes}) == 1 else None
    ok = torch.tensor([1])
    if len({hi - lo for lo, hi in sizes}) == 1:
        full_codes, _ = R.rmsnorm_quantize_ref(x, w, 1e-6)
        ok = torch.tensor([int(torch.equal(torch.cat(gathered), full_codes))])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    # timing protocol of the benchmark: max over ranks
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        with open(os.path.join(out_dir, "result.txt"), "w") as f:
            f.write(f"{int(ok.item())} {t.item()}")
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_batch_shards_equal_unsharded(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ok, tmax = open(tmp_path / "result.txt").read().split()
    assert ok == "1" and float(tmax) == 2.0
