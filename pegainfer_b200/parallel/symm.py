"""Symmetric (peer-mapped) device buffers for one-process-per-GPU runs.

Every rank allocates the same-sized buffer, exports a CUDA IPC handle, all-gathers
the handles through ``torch.distributed`` and maps every peer's buffer, so kernels
can be given a table ``ptrs[rank]`` and load/store any rank's copy over NVLink.
NCCL (or gloo) is used only for this bootstrap.

Reference parity: the DeepEP shim's symmetric NCCL window
(pegainfer-kernels/csrc/deepep/deepep_shim_impl.cuh:264-283) and the K3 peer-access
setup (csrc/k3/k3_mega_moe_sm100.cu, k3_mega_open_peer_access).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native


class _CudaArray:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricBuffer:
    def __init__(self, nbytes: int, rank: int, world: int, device: torch.device, group=None):
        import torch.distributed as dist

        self.lib = _native.load()
        self.nbytes = int(nbytes)
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.group = group
        with torch.cuda.device(self.device):
            p = ctypes.c_void_p()
            _native.check(self.lib.pg_symm_alloc(ctypes.c_longlong(self.nbytes), ctypes.byref(p)))
            self.local_ptr = p.value
            h = ctypes.create_string_buffer(64)
            _native.check(self.lib.pg_ipc_export(ctypes.c_void_p(self.local_ptr), h))
            handles = [None] * world
            if world > 1:
                dist.all_gather_object(handles, h.raw, group=group)
            else:
                handles[0] = h.raw
            self.ptrs = []
            self._imported = []
            for q in range(world):
                if q == rank:
                    self.ptrs.append(self.local_ptr)
                    continue
                out = ctypes.c_void_p()
                _native.check(self.lib.pg_ipc_import(ctypes.create_string_buffer(handles[q], 64), ctypes.byref(out)))
                self.ptrs.append(out.value)
                self._imported.append(out.value)
        self.table = (ctypes.c_void_p * world)(*self.ptrs)
        self._keep = _CudaArray(self.local_ptr, self.nbytes)
        self.bytes = torch.as_tensor(self._keep, device=self.device)

    def view(self, dtype, shape, byte_offset: int = 0) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.bytes[byte_offset : byte_offset + nb].view(dtype).view(*shape)

    def sub_table(self, byte_offset: int):
        """ctypes array of every rank's pointer advanced by ``byte_offset``."""
        return (ctypes.c_void_p * self.world)(*[p + byte_offset for p in self.ptrs])

    def close(self) -> None:
        """Unmap the peers' buffers and free the local one (idempotent).  The caller makes sure no
        kernel on any rank still touches them."""
        for p in self._imported:
            self.lib.pg_ipc_close(ctypes.c_void_p(p))
        self._imported = []
        if self.local_ptr:
            if self.world > 1:
                # a buffer is freed only after every peer has unmapped it
                import torch.distributed as dist

                if dist.is_initialized():
                    dist.barrier(group=self.group)
            self.bytes = None
            self._keep = None
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                self.lib.pg_symm_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0
