"""Device buffers that every rank of a node can store into: the plumbing under e5b_gemm_bcast.

One process per GPU (torch.distributed, NCCL).  Every rank allocates a buffer of the same size; the ranks
exchange handles once, and afterwards `ptrs[r]` is the address, valid on THIS rank's device, of rank r's
buffer.  The GEMM / GEMV epilogue writes its block of the output to all of them with plain stores, which is
the all-gather of a sharded output without a collective launch.

torch's symmetric memory does the mapping (cuMemCreate + handle exchange over the process group).  NVLink
multicast binding is switched off: only unicast peer mappings are used, nothing is ever loaded from a peer.
"""
import os

import torch
import torch.distributed as dist


class PeerBuffer:
    """`nbytes` of device memory on every rank of `group`, mapped everywhere.

    .local      uint8 tensor over this rank's buffer
    .ptrs       device addresses of all ranks' buffers, indexed by group rank (ptrs[rank] is .local)
    .peers(off) addresses of the other ranks' buffers plus a byte offset, in rank order
    .device_barrier(stream)  e5b_peer_barrier over a flag area kept behind the buffer: every rank's earlier work on
                its stream is complete and its stores into this rank's buffer are visible (no collective launched)
    """

    def __init__(self, nbytes, device, group=None):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.flag_off = (nbytes + 255) // 256 * 256          # 64 bytes of barrier flags behind the payload
        self.whole = symm.empty(self.flag_off + 64, dtype=torch.uint8, device=device)
        self.whole[self.flag_off:].zero_()
        torch.cuda.synchronize(device)
        self.local = self.whole[:nbytes]
        self.handle = symm.rendezvous(self.whole, group=self.group)      # a collective: every rank's flags are zero after it
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.ptrs) != self.world or self.ptrs[self.rank] != self.local.data_ptr():
            raise RuntimeError("symmetric memory rendezvous returned an unexpected pointer table")

    def peers(self, offset=0):
        return [p + offset for r, p in enumerate(self.ptrs) if r != self.rank]

    def device_barrier(self, stream=None):
        from . import capi
        sp = torch.cuda.current_stream().cuda_stream if stream is None else stream
        if capi.peer_barrier(self.rank, [p + self.flag_off for p in self.ptrs], sp) != capi.OK:
            raise RuntimeError(capi.last_error())

    def barrier(self):
        """All ranks' earlier work on their current streams is complete and visible (device-side barrier)."""
        self.handle.barrier()
