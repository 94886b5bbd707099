"""Host expert banks: page-aligned lazy buffers that are filled first and page-locked afterwards.

Mirror of ``HostBank`` / ``pin_banks`` (``freetoken/python/freetoken/moe/host_banks.py:86-157,281-296``) and of
``device_ptr`` (``freetoken/python/freetoken/kernel/pinned.py:59-68``):

  * the buffer is a PRIVATE anonymous mmap with ``MADV_HUGEPAGE`` set before the first touch, so the fill faults in
    2 MiB pages (host-to-device copies from huge pages run closer to the link rate, and a gather kernel that reads
    the bank over the bus misses the GPU's page tables less);
  * nothing is resident until it is written: a bank of 18 GB costs address space only until the loader fills it;
  * ``pin()`` registers the filled buffer with CUDA as portable + mapped (pin-after-fill); until then the bank is
    PAGEABLE and cannot feed the GPU movement paths.
"""
from __future__ import annotations

import ctypes
import enum
import math
import mmap

import torch

_BLK = 4096
# the mappings live as long as the process: the slot cache reads from these banks forever
_LIVE_BUFFERS: list[mmap.mmap] = []


class HostResidency(str, enum.Enum):
    PINNED = "pinned"
    PAGEABLE = "pageable"


class PinFailed(RuntimeError):
    """cudaHostRegister refused a bank: the host is out of pinnable memory or over its pin quota."""


class HostBank:
    """allocate -> fill ``tensor`` -> ``pin()``."""

    __slots__ = ("tensor", "addr", "nbytes", "_buf", "_pinned")

    def __init__(self, shape: tuple[int, ...], dtype: torch.dtype, huge_pages: bool = True):
        elsize = torch.empty((), dtype=dtype).element_size()
        self.nbytes = math.prod(shape) * elsize
        asize = max(_BLK, (self.nbytes + _BLK - 1) // _BLK * _BLK)
        if huge_pages and hasattr(mmap, "MADV_HUGEPAGE"):
            self._buf = mmap.mmap(-1, asize, flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS)
            try:
                self._buf.madvise(mmap.MADV_HUGEPAGE)
            except OSError:  # kernel without transparent huge pages: plain pages
                pass
        else:
            self._buf = mmap.mmap(-1, asize)
        _LIVE_BUFFERS.append(self._buf)
        self.addr = ctypes.addressof(ctypes.c_char.from_buffer(self._buf))
        assert self.addr % _BLK == 0
        self.tensor = torch.frombuffer(self._buf, dtype=dtype, count=self.nbytes // elsize).view(*shape)
        self._pinned = False

    @property
    def residency(self) -> HostResidency:
        return HostResidency.PINNED if self._pinned else HostResidency.PAGEABLE

    def pin(self) -> None:
        """Register the (now filled) buffer with CUDA: portable + mapped."""
        if self._pinned:
            return
        from ._lib import lib

        rc = lib().b200moe_host_register(self.addr, len(self._buf))
        if rc:
            raise PinFailed(f"cudaHostRegister failed for {len(self._buf) / 2**30:.2f} GiB (code {rc})")
        self._pinned = True

    def unpin(self) -> None:
        if self._pinned:
            from ._lib import check, lib

            check(lib().b200moe_host_unregister(self.addr), "b200moe_host_unregister")
            self._pinned = False


def pin_banks(banks) -> int:
    """Pin every bank of an iterable (after the loader has filled them); returns the bytes pinned."""
    total = 0
    for b in banks:
        b.pin()
        total += b.nbytes
    return total


def device_ptr(t: torch.Tensor) -> int:
    """Base address of ``t`` as a kernel must dereference it: ``data_ptr()`` for device tensors; for pinned + mapped
    host memory the address CUDA maps it at (the same number under unified addressing)."""
    if t.is_cuda:
        return t.data_ptr()
    from ._lib import check, lib

    out = ctypes.c_void_p(0)
    check(lib().b200moe_host_device_ptr(t.data_ptr(), ctypes.byref(out)), "b200moe_host_device_ptr")
    return int(out.value)


__all__ = ["HostBank", "HostResidency", "PinFailed", "pin_banks", "device_ptr"]
