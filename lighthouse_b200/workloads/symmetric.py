"""Symmetric-memory plumbing for the fused collective kernels.

The library takes raw addresses (``lh_b200_symm_register`` / ``lh_b200_symm_set_flags``);
allocating buffers that every rank maps and binding them to an NVSwitch multicast object is
host plumbing, done here with ``torch.distributed._symmetric_memory`` on an initialised NCCL
process group. Nothing in this module touches the data.
"""

from __future__ import annotations

FLAG_PAD_WORDS = 64  # >= 2 * LH_MAX_RANKS 32-bit flags


class SymmetricBuffers:
    """Allocates the symmetric tensors of one context and registers them with it."""

    def __init__(self, ctx, group=None):
        import torch.distributed as dist

        self.ctx = ctx
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self._keep = []  # tensors and handles stay alive as long as the registrations
        self._flags_set = False

    def _rendezvous(self, tensor):
        import torch.distributed._symmetric_memory as symm_mem

        handle = symm_mem.rendezvous(tensor, self.group)
        self._keep.append((tensor, handle))
        return handle

    def empty(self, shape, dtype):
        """A symmetric tensor of this shape on every rank, registered for multicast access."""
        import torch
        import torch.distributed._symmetric_memory as symm_mem

        t = symm_mem.empty(*shape, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        handle = self._rendezvous(t)
        multicast = int(handle.multicast_ptr)
        if self.world > 1 and not multicast:
            raise RuntimeError("this system gives no NVSwitch multicast mapping for symmetric memory; use the NCCL schedule")
        base = int(handle.buffer_ptrs[self.rank])
        offset = t.data_ptr() - base
        nbytes = t.numel() * t.element_size()
        peers = [int(ptr) + offset for ptr in handle.buffer_ptrs]
        self.ctx.symm_register(t.data_ptr(), nbytes, multicast + offset if multicast else 0, peers)
        if not self._flags_set:
            self._set_flags()
        return t

    def _set_flags(self):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        flags = symm_mem.empty(FLAG_PAD_WORDS, dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))
        handle = self._rendezvous(flags)
        offset = flags.data_ptr() - int(handle.buffer_ptrs[self.rank])
        self.ctx.symm_set_flags(self.rank, self.world, [int(ptr) + offset for ptr in handle.buffer_ptrs])  # zeroes this rank's pad
        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # every pad is zero before anyone's kernel signals
        torch.cuda.synchronize()
        self._flags_set = True

    def close(self):
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # nobody unmaps while a peer's kernel may still store here
        torch.cuda.synchronize()
        self.ctx.symm_clear()
        self._keep.clear()
