"""Worker of tests/test_gpu_multi.py: one rank per GPU under torch.distributed.run.  Shards a reduced dgrad GEMM
by column blocks and a reduced decode GEMV by weight rows through the unchanged C interface, gathers the output
blocks in both ways the library offers -- NCCL all-gather after e5ma_gemm, and e5b_gemm_bcast, whose epilogue stores
into every peer's buffer, closed by the device-side flag barrier e5b_peer_barrier -- and compares with the unsharded result computed on the same GPU."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from e5m2effma_b200 import capi, sharding, workloads
    from e5m2effma_b200.peer import PeerBuffer
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.current_stream().cuda_stream
    failures = []

    for name in ("c2_bf16", "c3n8", "c3n1"):
        w = workloads.make(name, dev, 4)                 # every rank builds the same full problem from the same seeds
        es = w.D.element_size()
        w.launch(stream)
        torch.cuda.synchronize()
        full = w.D.clone()
        full_amax = None if w.amax is None else w.amax.clone()

        # ---- plain call on the shard, NCCL all-gather ----
        w.D.zero_()
        if w.amax is not None:
            w.amax.zero_()
        tA, tB, tD, tb = w.tensors()
        if w.n <= 8:
            i0, i1, a, b, d = sharding.gemv_rows(w.m, w.k, tA, tb, tD, world, rank, align=16)
            args = (capi.OP_T, capi.OP_N, i1 - i0, w.n, w.k, 1.0, a, w.k, tB, w.k, 0.0, None, 0, d, w.m, b)
            off = i0 * es
        else:
            sh = sharding.gemm_columns(w.n, w.k, w.m, w.m, tB, None, tD, world, rank)
            args = (capi.OP_T, capi.OP_N, w.m, sh.n, w.k, 1.0, tA, w.k, sh.B, w.k, 0.0, None, 0, sh.D, w.m, tb)
            off = sh.j0 * w.m * es
        assert capi.gemm(*args, stream) == capi.OK, capi.last_error()
        plain_route = capi.last_route()
        if w.n <= 8:                                     # row blocks of each column: gather column by column
            for j in range(w.n):
                col = w.D[j]
                dist.all_gather_into_tensor(col, col[i0:i1].clone())
        else:
            sharding.allgather_columns(w.D, w.n, w.m, world)
        if w.amax is not None:
            sharding.amax_allreduce(w.amax)
        torch.cuda.synchronize()
        nccl = w.D.clone()
        if w.amax is not None and not torch.equal(w.amax, full_amax):
            failures.append(f"{name}: reduced amax {w.amax.item()} != {full_amax.item()}")

        # ---- e5b_gemm_bcast: the epilogue stores into every peer ----
        pb = PeerBuffer(w.D.numel() * es, dev)
        pb.local.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        Dp = capi.Tensor(pb.local.data_ptr() + off, args[13].dtype, args[13].scale_inv, args[13].scale, None, args[13].scaling)
        assert capi.gemm_bcast(*args[:13], Dp, args[14], args[15], pb.peers(off), stream) == capi.OK, capi.last_error()
        pb.device_barrier(stream)        # e5b_peer_barrier: no host-side barrier, no collective -- the flags alone order the reads below
        fused = pb.local[: w.D.numel() * es].view(w.D.dtype).view(w.D.shape).clone()
        torch.cuda.synchronize()
        # and again into a cleared buffer: the barrier counts its calls
        dist.barrier()
        pb.local.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        assert capi.gemm_bcast(*args[:13], Dp, args[14], args[15], pb.peers(off), stream) == capi.OK, capi.last_error()
        pb.device_barrier(stream)
        again = pb.local[: w.D.numel() * es].view(w.D.dtype).view(w.D.shape).clone()
        torch.cuda.synchronize()
        if not torch.equal(fused.view(torch.uint8), again.view(torch.uint8)):
            failures.append(f"{name}: second broadcast behind the device-side barrier differs from the first")

        if capi.last_route() == plain_route:
            if not torch.equal(nccl.view(torch.uint8), fused.view(torch.uint8)):
                failures.append(f"{name}: NCCL-gathered and epilogue-broadcast outputs differ")
        else:             # the broadcasting launch may prefer another tile shape (more rounds to hide the copies behind)
            diff = (nccl.view(torch.int16).int() - fused.view(torch.int16).int()).abs()
            if int(diff.max()) > 1 or float((diff != 0).float().mean()) > 0.02:
                failures.append(f"{name}: NCCL-gathered and epilogue-broadcast outputs differ by more than one code")
        if w.n <= 8:      # a row's sum does not depend on how many rows the call has: bit for bit
            if not torch.equal(nccl.view(torch.uint8), full.view(torch.uint8)):
                failures.append(f"{name}: gathered row shards differ from the unsharded GEMV")
        else:             # a tile's k-blocks may be visited in the other direction: allow one code, rarely
            a16, b16 = nccl.view(torch.int16).int(), full.view(torch.int16).int()
            diff = (a16 - b16).abs()
            if int(diff.max()) > 1 or float((diff != 0).float().mean()) > 0.02:
                failures.append(f"{name}: gathered column shards differ from the unsharded GEMM by more than one code "
                                f"(max {int(diff.max())}, {float((diff != 0).float().mean()):.4f} of the outputs)")
        if capi.gemm_fault():
            failures.append(f"{name}: a bounded wait ran out")

    # AdamW by chunks: the union of the ranks' chunks equals the unsharded step, bit for bit; amax is the global one
    a = workloads.AdamWorkload("a", 1 << 22, dev, seed=9)
    b = workloads.AdamWorkload("b", 1 << 22, dev, seed=9)
    a.launch(stream)
    i0, i1 = sharding.chunk(b.count, world, rank)
    b.launch_range(stream, i0, i1)
    sharding.amax_allreduce(b.amax)
    torch.cuda.synchronize()
    for f in ("p", "m", "v", "q"):
        if not torch.equal(getattr(a, f)[i0:i1].view(torch.uint8), getattr(b, f)[i0:i1].view(torch.uint8)):
            failures.append(f"adam: chunk of {f} differs")
    if not torch.equal(a.amax, b.amax):
        failures.append("adam: reduced amax differs")

    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    if failures:
        print(f"rank {rank}: " + "; ".join(failures), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("MULTI_GPU_OK" if int(flag.item()) == 0 else "MULTI_GPU_FAILED", flush=True)
    os._exit(0 if int(flag.item()) == 0 else 1)


if __name__ == "__main__":
    main()
