"""Low-latency all-reduce for the tensor-parallel decoder: peer-mapped buffers from
torch.distributed's symmetric memory (plumbing) + the one-shot kernel of csrc/nb_comm.cu."""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib


class OneShotAllReduce:
    """In-place sum of an fp32 tensor over the ranks of `group`.  max_count: largest numel (multiple of 4)."""

    def __init__(self, max_count: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.max_count = (max_count + 3) // 4 * 4
        nbytes = _lib.lib().nb_allreduce_buffer_bytes(self.world, self.max_count)
        if nbytes == 0:
            raise RuntimeError(f"one-shot all-reduce supports 1..8 ranks; got {self.world}")
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.peer_array = (ctypes.c_uint64 * self.world)(*ptrs)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)          # every rank's buffer is zeroed before anyone pushes into it

    def __call__(self, t: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Sum of t over the ranks, in place or into `out` (same shape and type; t is left as it was)."""
        if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() % 4 or t.numel() > self.max_count:
            raise RuntimeError("one-shot all-reduce needs a contiguous fp32 tensor whose numel is a multiple of 4 "
                               f"and at most {self.max_count}")
        dst = t if out is None else out
        if dst.dtype != torch.float32 or not dst.is_contiguous() or dst.numel() != t.numel():
            raise RuntimeError("one-shot all-reduce: `out` must be a contiguous fp32 tensor of the input's size")
        rc = _lib.lib().nb_allreduce(t.data_ptr(), dst.data_ptr(), t.numel(), self.peer_array, self.world, self.rank,
                                     self.max_count, 0, self.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        if rc:
            _lib.check(rc, "nb_allreduce")
        return dst

    def check(self) -> None:
        """Raises if a wait for the peers ever ran out (reads the device status word: synchronises)."""
        if int(self.status.item()) != 0:
            raise RuntimeError("nb_allreduce: a peer did not arrive within the bounded wait")


class Exchange:
    """Peer-mapped exchange buffers for the all-reduce folded into the packed GEMVs (nb_gemv_tp): the
    row-sharded projection pushes its partial result into every rank's buffer, the next GEMV's prologue
    (or nb_exchange_gather) sums the ranks' vectors.  max_count: largest vector (floats, multiple of 4).
    With `local_buffers` (a list of this process's own tensors, one per emulated rank) no process group is
    needed: used by single-GPU tests that run the ranks one after another."""

    def __init__(self, max_count: int, device, group=None, rank: int | None = None, local_buffers=None, spin_limit: int = 0):
        self.max_count = (max_count + 3) // 4 * 4
        self.spin_limit = spin_limit
        if local_buffers is not None:
            self.world, self.rank = len(local_buffers), int(rank)
            self.buf = local_buffers[self.rank]
            ptrs = [int(b.data_ptr()) for b in local_buffers]
        else:
            import torch.distributed._symmetric_memory as symm_mem
            self.group = group if group is not None else dist.group.WORLD
            self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
            nbytes = self.buffer_bytes(self.world, self.max_count)
            self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            self.buf.zero_()
            self.handle = symm_mem.rendezvous(self.buf, self.group.group_name)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        peer_array = (ctypes.c_uint64 * self.world)(*ptrs)
        _lib.check(_lib.lib().nb_exchange_init(self.buf.data_ptr(), peer_array, self.world, self.rank, self.max_count),
                   "nb_exchange_init")
        if local_buffers is None:
            dist.barrier(self.group)      # every rank's buffer is zeroed and initialised before anyone pushes into it

    @staticmethod
    def buffer_bytes(world: int, max_count: int) -> int:
        nbytes = _lib.lib().nb_exchange_buffer_bytes(world, (max_count + 3) // 4 * 4)
        if nbytes == 0:
            raise RuntimeError(f"the exchange supports 1..8 ranks; got {world}")
        return int(nbytes)
