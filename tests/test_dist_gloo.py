"""Two CPU ranks over gloo drive the package's own sharding protocol (`trinix_b200.sharding`):
shard bounds, the untimed gather-and-compare and the max-over-ranks reduction that the
benchmark uses at N > 1. The data path itself needs no collective. The per-shard computation
here is the mirror modules' CPU path and the CPU oracle (there is no GPU in this test); on a
GPU box `bench.py --gpus N` runs the same protocol over the kernels."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import trinix_b200 as T
from oracle import reference_port as R
from trinix_b200.sharding import cross_rank_identical, gather_shards, max_over_ranks, shard


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
    x = torch.randn(7, 16, 256, generator=g).bfloat16()      # 7 sequences: ragged shards (4 + 3)
    w = (1 + 0.02 * torch.randn(256, generator=g)).bfloat16()
    norm = T.FastRMSNorm(256, eps=1e-6).bfloat16()            # 256 <= 2048: the module's torch path
    with torch.no_grad():
        norm.weight.copy_(w)
        ok_norm = cross_rank_identical(lambda t: norm(t), [x], rank, world)
    ok_int8 = cross_rank_identical(lambda t, ww: R.rmsnorm_quantize_ref(t, ww, 1e-6), [x, w],
                                   rank, world)
    glu = T.FastSwiGLU(128)
    ok_glu = cross_rank_identical(lambda t: glu(t), [x], rank, world)
    # a wrong shard must be caught: rank 1 perturbs its result
    bad = cross_rank_identical(lambda t: t.float() + (1.0 if (rank == 1 and t.shape[0] < 7) else 0.0),
                               [x], rank, world)
    gathered = gather_shards(shard(x, rank, world).contiguous(), 7, world)
    tmax = max_over_ranks(float(rank + 1))
    t2 = max_over_ranks([1.0 + rank, 5.0 - rank])
    if rank == 0:
        with open(os.path.join(out_dir, "result.txt"), "w") as f:
            f.write(f"{int(ok_norm)} {int(ok_int8)} {int(ok_glu)} {int(bad)} "
                    f"{int(torch.equal(gathered, x))} {tmax} {t2[0]} {t2[1]}")
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_batch_shards_equal_unsharded(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = open(tmp_path / "result.txt").read().split()
    assert r[:5] == ["1", "1", "1", "0", "1"]
    assert [float(v) for v in r[5:]] == [2.0, 2.0, 5.0]


def test_sharding_helpers_without_a_process_group():
    x = torch.arange(10.0).view(5, 2)
    assert cross_rank_identical(lambda t: t * 2, [x], 0, 1)
    assert max_over_ranks(3.5) == 3.5 and max_over_ranks([1.0, 2.0]) == [1.0, 2.0]
    assert torch.equal(gather_shards(x, 5, 1), x)
