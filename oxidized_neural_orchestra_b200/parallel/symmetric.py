"""Symmetric peer-memory windows over NVLink: the data plane that replaces the reference's TCP
transports (comms/src/transport, comms/src/connection/{acceptor,connector}.rs).

A window is one buffer allocated at the same size on every rank; after the rendezvous every rank
holds a mapped device pointer to every peer's copy (and, where the fabric supports it, one multicast
address that reaches all copies through NVSwitch). Kernels then move gradients and parameters with
plain loads/stores or ``multimem`` instructions; no host is in the loop.

The handle exchange itself is PyTorch's symmetric-memory rendezvous (CUDA VMM allocations whose
handles travel over the process group's store), which is the framework layer's job here. With one
rank the window is an ordinary device tensor.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class SymmetricWindow:
    """``nbytes`` of device memory on every rank of ``group`` plus an epoch-flag pad.

    ``ptrs[r]`` is the address of rank r's buffer as seen from this process, ``mc_ptr`` the multicast
    address (0 when NVLS is unavailable), ``flag_ptrs[r]`` rank r's flag pad.
    """

    FLAG_WORDS = 8192  # enough for 512 blocks x 8 ranks of barrier flags plus ring flags

    def __init__(self, nbytes: int, device: torch.device, group=None):
        self.device = device
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.nbytes = _align(nbytes)
        self.flag_off = self.nbytes
        total = self.nbytes + self.FLAG_WORDS * 4
        self.handle = None
        if self.world == 1:
            self.buf = torch.zeros(total, dtype=torch.uint8, device=device)
            self.ptrs = [self.buf.data_ptr()]
            self.mc_ptr = 0
        else:
            import torch.distributed._symmetric_memory as symm_mem

            grp = group if group is not None else dist.group.WORLD
            import warnings

            with warnings.catch_warnings():       # needed by older builds; newer ones only warn that it is a no-op
                warnings.simplefilter("ignore")
                try:
                    symm_mem.enable_symm_mem_for_group(grp.group_name)
                except Exception:
                    pass
            self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
            self.handle = symm_mem.rendezvous(self.buf, grp)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
            mc = 0
            try:
                if self.handle.has_multicast_support(device.type, device.index):
                    mc = int(self.handle.multicast_ptr)
            except Exception:  # older builds expose only multicast_ptr
                mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
            self.mc_ptr = mc
            self.buf.zero_()
            torch.cuda.synchronize(device)
            dist.barrier(group=grp)
        self.flag_ptrs = [p + self.flag_off for p in self.ptrs]

    def view(self, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A local tensor over ``numel`` elements starting ``offset`` bytes into this rank's buffer."""
        nb = numel * torch.empty((), dtype=dtype).element_size()
        if offset % 16 or offset + nb > self.nbytes:
            raise ValueError("window view out of range or misaligned")
        return self.buf[offset:offset + nb].view(dtype)

    def peer_ptrs(self, offset: int) -> list[int]:
        return [p + offset for p in self.ptrs]

    def mc(self, offset: int) -> int:
        return self.mc_ptr + offset if self.mc_ptr else 0


class WindowLayout:
    """Byte offsets of named regions packed into one window (each 256-byte aligned)."""

    def __init__(self):
        self.regions: dict[str, tuple[int, int, torch.dtype]] = {}
        self.size = 0

    def add(self, name: str, numel: int, dtype: torch.dtype) -> int:
        off = self.size
        self.regions[name] = (off, numel, dtype)
        self.size = _align(off + numel * torch.empty((), dtype=dtype).element_size())
        return off

    def offset(self, name: str) -> int:
        return self.regions[name][0]

    def tensor(self, win: SymmetricWindow, name: str) -> torch.Tensor:
        off, numel, dtype = self.regions[name]
        return win.view(off, numel, dtype)
