"""Multi-rank host logic on CPU (gloo, world_size 2 and 3): partition arithmetic of
e5m2effma_b200.sharding, the output all-gather and the amax max-all-reduce.  The per-rank "kernel"
is the CPU oracle run on the rank's slice, so the gathered result must equal the unsharded oracle
result bit for bit (the shards are independent: no reduction crosses ranks)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as orc
from e5m2effma_b200 import capi, sharding


def test_split_covers_everything_once():
    for total in (0, 1, 100, 128, 4096, 4097, 10_000):
        for world in (1, 2, 3, 8):
            for align in (1, 16, 128):
                parts = [sharding.split(total, world, r, align) for r in range(world)]
                assert parts[0][0] == 0 and parts[-1][1] == total
                for (a, b), (c, d) in zip(parts, parts[1:]):
                    assert b == c and a <= b
                for a, b in parts[:-1]:
                    assert (a % align == 0 or a == total) and (b % align == 0 or b == total)


def test_pointer_offsets_of_a_column_block():
    n, ldb, ldd = 1000, 4112, 515
    B = capi.tensor(0x10000, capi.E4M3, 0x500, None, None, capi.SCALING_OUTER)
    D = capi.tensor(0x900000, capi.BF16, None, 0x700, 0x800)
    sh = sharding.gemm_columns(n, ldb, 0, ldd, B, None, D, world=4, rank=2)
    assert (sh.j0, sh.j1) == (512, 768)
    assert sh.B.data == 0x10000 + 512 * ldb and sh.B.scale_inv == 0x500 + 4 * 512 and sh.B.scaling == capi.SCALING_OUTER
    assert sh.D.data == 0x900000 + 512 * ldd * 2 and sh.D.scale == 0x700 and sh.D.amax == 0x800 and sh.C is None
    i0, i1, a, b, d = sharding.gemv_rows(8192, 8192, capi.tensor(0x1000, capi.E5M2, 0x40, None, None, 1),
                                        capi.tensor(0x2000, capi.BF16), capi.tensor(0x3000, capi.BF16), 8, 3)
    assert (i0, i1) == (3072, 4096) and a.data == 0x1000 + 3072 * 8192 and a.scale_inv == 0x40 + 4 * 3072
    assert b.data == 0x2000 + 2 * 3072 and d.data == 0x3000 + 2 * 3072


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc.set_threads(1)
        rng = np.random.default_rng(11)   # same data on every rank
        m, k = 96, 64
        A = rng.integers(0, 120, m * k).astype(np.uint8)
        B = rng.integers(0, 120, n * k).astype(np.uint8)
        sb = (0.5 + rng.random(n)).astype(np.float32)
        bias = orc.encode(orc.BF16, rng.standard_normal(m).astype(np.float32))
        full = np.zeros(n * m, np.uint16)
        full_amax = orc.gemm(1, 0, m, n, k, 1.0, A, orc.E5M2, k, B, orc.E4M3, k, 0.0, None, orc.FP32, m, full, orc.BF16, m,
                             bias=bias, bias_dtype=orc.BF16, a_sinv=0.25, b_sinv=sb, b_outer=True, amax=0.0)
        j0, j1 = sharding.split(n, world, rank, 16)
        mine = np.zeros(n * m, np.uint16)
        my_amax = 0.0
        if j1 > j0:   # the rank's call: B, its scale vector and D advanced by j0 columns
            my_amax = orc.gemm(1, 0, m, j1 - j0, k, 1.0, A, orc.E5M2, k, B[j0 * k:], orc.E4M3, k, 0.0, None, orc.FP32, m,
                               mine[j0 * m:], orc.BF16, m, bias=bias, bias_dtype=orc.BF16, a_sinv=0.25, b_sinv=sb[j0:],
                               b_outer=True, amax=0.0)
        D = torch.from_numpy(mine.view(np.int16)).view(n, m)
        sharding.allgather_columns(D, n, m, world, align=16)
        am = sharding.amax_allreduce(torch.tensor([my_amax], dtype=torch.float32))
        ok = np.array_equal(D.numpy().reshape(-1).view(np.uint16), full) and float(am) == float(full_amax)
        out_q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 64), (2, 72), (3, 100)])
def test_sharded_gemm_matches_unsharded(world, n):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = dict(q.get(timeout=10) for _ in range(world))
    assert all(res.values()), res


def _worker_subgroup(rank, world, port, out_q):
    """Ranks 1 and 2 of a world of 3 form the group that shares a matrix: rank-in-group != global rank, and the
    uneven column split takes the broadcast path of allgather_columns."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        group = dist.new_group([1, 2])
        ok = True
        if rank in (1, 2):
            gr = dist.get_rank(group)
            n, m = 72, 8                   # blocks of 16 columns: 48 for group rank 0, 24 for group rank 1
            full = torch.arange(n * m, dtype=torch.int16).view(n, m)
            j0, j1 = sharding.split(n, 2, gr, 16)
            mine = torch.zeros_like(full)
            mine[j0:j1] = full[j0:j1]
            sharding.allgather_columns(mine, n, m, 2, align=16, group=group)
            am = sharding.amax_allreduce(torch.tensor([float(gr + 1)]), group=group)
            ok = torch.equal(mine, full) and float(am) == 2.0
        out_q.put((rank, bool(ok)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_gather_inside_a_subgroup():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_subgroup, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = dict(q.get(timeout=10) for _ in range(3))
    assert all(res.values()), res
