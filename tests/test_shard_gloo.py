"""Batch sharding over ranks (host logic), run as two gloo ranks on the CPU.
Each rank evaluates its shard with the oracle scan (the GPU op is not
available here); the point is the sharding and the one all-reduce for inputs
broadcast over the batch."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flex_rnn_b200.shard import reduce_broadcast_grads, shard_args, shard_bounds


def test_shard_bounds_cover_batch():
    for B in (1, 7, 8, 64):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(B, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, out):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import naive_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, T, H, M, N = 4, 6, 2, 8, 8
    xs, dy, dS = O.make_case("mamba2", B, T, H, M, N, torch.float32)
    ins, sts, (lo, hi) = shard_args(xs[:-1], xs[-1:], rank, world)
    assert ins[2].shape[0] == 1 and ins[0].shape[0] == hi - lo          # A is passed whole
    y, ST, gx, gs = O.fwd_bwd(O.mamba2, ins, sts, [dy[lo:hi]], [dS[lo:hi]])
    gx = reduce_broadcast_grads(gx, ins, B)
    if rank == 0:
        torch.save({"dA": gx[2], "y0": y[0], "dx0": gx[0]}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_single_process(tmp_path):
    from oracle import naive_oracle as O
    out = str(tmp_path / "r0.pt")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = torch.load(out)
    B, T, H, M, N = 4, 6, 2, 8, 8
    xs, dy, dS = O.make_case("mamba2", B, T, H, M, N, torch.float32)
    y, ST, gx, gs = O.fwd_bwd(O.mamba2, xs[:-1], xs[-1:], [dy], [dS])
    assert O.rel_err(got["dA"], gx[2]) < 1e-5            # summed over both shards
    assert O.rel_err(got["y0"], y[0][:2]) < 1e-6 and O.rel_err(got["dx0"], gx[0][:2]) < 1e-6
