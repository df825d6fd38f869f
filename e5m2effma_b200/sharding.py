"""Multi-GPU partitioning of the hot path, one process per GPU (torch.distributed).

The reference is a single-device library; the C interface is left as it is and every rank simply
calls it on its own slice, described by pointer arithmetic:

    GEMM   columns of op(B) / D / C      B.data += j0*ldb, B.scale_inv += j0 (row-wise), D.data += j0*ldd
           (A, its scale vector and the bias are replicated on every rank)
    GEMV   rows of the weight matrix     A.data += i0*lda, A.scale_inv += i0, bias += i0, D.data += i0
    AdamW / casts   contiguous element chunks (multiples of 16 elements keep 16-byte alignment)

No step of the computation needs another rank's data.  The only collectives are the ones a caller
may want afterwards: the max-all-reduce of the scalar amax (so that every rank holds the global
statistic for the next quantisation scale) and the all-gather of the output blocks.
"""
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import capi

_ES = {capi.E4M3: 1, capi.E5M2: 1, capi.BF16: 2, capi.FP16: 2, capi.FP32: 4}


def split(total, world, rank, align):
    """[start, stop) of rank's share of `total` units: the ceil(total / align) blocks of `align`
    units are dealt out as evenly as possible in rank order; the last block may be partial."""
    blocks = -(-total // align)
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(total, b0 * align), min(total, b1 * align)


@dataclass
class GemmShard:
    """Arguments of e5ma_gemm for one rank's column block [j0, j1) of a TN problem."""
    j0: int
    j1: int
    B: capi.Tensor
    C: object
    D: capi.Tensor

    @property
    def n(self):
        return self.j1 - self.j0


def gemm_columns(n, ldb, ldc, ldd, B, C, D, world, rank, transb=capi.OP_N, align=128):
    """Column block of rank: offsets B (transb = N: K-contiguous columns), C and D by whole columns."""
    j0, j1 = split(n, world, rank, align)
    if transb != capi.OP_N:
        raise ValueError("column sharding by pointer offset needs transb = N (B stored k x n)")

    def shifted(t, ld):
        if t is None:
            return None
        sinv = t.scale_inv
        if t.scaling == capi.SCALING_OUTER and sinv:
            sinv = sinv + 4 * j0
        return capi.Tensor((t.data or 0) + j0 * ld * _ES[t.dtype], t.dtype, sinv, t.scale, t.amax, t.scaling)

    return GemmShard(j0, j1, shifted(B, ldb), shifted(C, ldc), shifted(D, ldd))


def gemv_rows(m, lda, A, bias, D, world, rank, align=32):
    """Row block [i0, i1) of a GEMV-shaped problem (transa = T): returns (i0, i1, A, bias, D)."""
    i0, i1 = split(m, world, rank, align)
    sinv = A.scale_inv
    if A.scaling == capi.SCALING_OUTER and sinv:
        sinv = sinv + 4 * i0
    a = capi.Tensor(A.data + i0 * lda * _ES[A.dtype], A.dtype, sinv, A.scale, A.amax, A.scaling)
    b = None if bias is None else capi.Tensor(bias.data + i0 * _ES[bias.dtype], bias.dtype)
    d = capi.Tensor(D.data + i0 * _ES[D.dtype], D.dtype, D.scale_inv, D.scale, D.amax, D.scaling)
    return i0, i1, a, b, d


def chunk(count, world, rank, align=16):
    """Element range of rank for AdamW / casts."""
    return split(count, world, rank, align)


def amax_allreduce(amax, group=None):
    """Global amax on every rank (max over ranks of a one-element float32 tensor), in place."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    return amax


def allgather_columns(D_full, n, ld_elems, world, align=128, group=None):
    """All-gather of the column blocks of a column-major output stored as a [n, ld] tensor whose
    column block of each rank was written in place; every rank ends with all columns.  Blocks differ
    in size when n is not a multiple of world*align, so each is broadcast from its owner."""
    if not dist.is_initialized() or world == 1:
        return D_full
    full = D_full
    D_full = D_full.view(torch.uint8)   # move bytes: every backend handles uint8, whatever the element type
    sizes = [split(n, world, r, align) for r in range(world)]
    if len({b - a for a, b in sizes}) == 1:
        rank = dist.get_rank(group)
        a, b = sizes[rank]
        dist.all_gather_into_tensor(D_full[:n], D_full[a:b].clone(), group=group)
    else:
        for r, (a, b) in enumerate(sizes):
            if b > a:       # broadcast takes the GLOBAL rank of the owner, r is its rank within `group`
                src = r if group is None else dist.get_global_rank(group, r)
                dist.broadcast(D_full[a:b], src=src, group=group)
    return full
