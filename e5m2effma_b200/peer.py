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
    """

    def __init__(self, nbytes, device, group=None):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.local = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.local, group=self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.ptrs) != self.world or self.ptrs[self.rank] != self.local.data_ptr():
            raise RuntimeError("symmetric memory rendezvous returned an unexpected pointer table")

    def peers(self, offset=0):
        return [p + offset for r, p in enumerate(self.ptrs) if r != self.rank]

    def barrier(self):
        """All ranks' earlier work on their current streams is complete and visible (device-side barrier)."""
        self.handle.barrier()
