"""Symmetric (peer-mapped) device memory for the fused compute+collective kernels.

Every rank of a group allocates a block of the same size; after the rendezvous each rank knows the
device address at which every peer's block is mapped into its own address space, so kernels can load
and store peer memory directly over NVLink.  The allocation and the handle exchange use PyTorch's
symmetric-memory allocator (CUDA VMM + fabric/fd handle exchange over the group's store); the reference
has no counterpart (it only ever calls NCCL: paddle/phi/core/distributed/nccl_comm_context.cc:91-249).
"""
from __future__ import annotations

import torch
import torch.distributed as tdist

_enabled_groups = set()
_live_blocks = []          # weak references to every SymmBlock, for release_all()


class SymmBlock:
    """One symmetric allocation: ``local`` is this rank's uint8 tensor, ``ptrs[r]`` the address of rank
    r's block as seen from this process."""

    def __init__(self, nbytes: int, group):
        import torch.distributed._symmetric_memory as symm_mem
        pg = group.process_group
        name = pg.group_name
        if name not in _enabled_groups:
            try:
                symm_mem.enable_symm_mem_for_group(name)
            except Exception:  # noqa: BLE001 - newer torch enables groups lazily
                pass
            _enabled_groups.add(name)
        nbytes = (nbytes + 255) // 256 * 256
        dev = torch.device("cuda", torch.cuda.current_device())
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, pg)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        # address of the NVLink multicast (NVLS) mapping of the block: a store to it lands in every rank's copy and
        # a multimem.ld_reduce sums all copies inside the switch; 0 where the fabric offers no multicast
        try:
            self.mc_ptr = int(self.handle.multicast_ptr) if multicast_enabled() else 0
        except Exception:  # noqa: BLE001 - older allocators have no multicast attribute
            self.mc_ptr = 0
        self.rank = self.handle.rank
        self.world_size = self.handle.world_size
        self.nbytes = nbytes
        torch.cuda.synchronize()
        tdist.barrier(group=pg, device_ids=[dev.index])
        import weakref
        _live_blocks.append(weakref.ref(self))

    def release(self):
        """Drop the mapping of the peers' memory and the local allocation.  Every rank has to do this before the
        process group that exchanged the handles is destroyed: the handle object keeps using the group's store and
        communicator, and tearing it down after them (at interpreter exit, in arbitrary order) can block."""
        self.handle = None
        self.local = None
        self.ptrs = []
        self.mc_ptr = 0

    def view(self, offset: int, shape, dtype):
        n = 1
        for s in shape:
            n *= int(s)
        nb = n * torch.empty(0, dtype=dtype).element_size()
        return self.local[offset:offset + nb].view(dtype).view(*shape)

    def peer_ptrs(self, offset: int):
        return [p + offset for p in self.ptrs]


def release_all():
    """Release every symmetric block of this process (after a device synchronise and a barrier by the caller: no
    kernel of any rank may still touch them).  Call before ``destroy_process_group``."""
    import gc
    for ref in _live_blocks:
        b = ref()
        if b is not None:
            b.release()
    _live_blocks.clear()
    gc.collect()


def multicast_enabled() -> bool:
    """``PD_DISABLE_NVLS=1`` keeps every kernel on plain peer loads / stores (used by tests in which a rank leaves the
    group: a process that dies while its memory is bound to a multicast object disturbs the other GPUs)."""
    import os
    return os.environ.get("PD_DISABLE_NVLS", "0") != "1"


def supported() -> bool:
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except ImportError:
        return False
    return torch.cuda.is_available()
