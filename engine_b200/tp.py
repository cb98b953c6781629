"""Tensor-parallel exchange over peer memory: the host side of ribn_tp_* (csrc/tp.cu).

One `PeerLink` per rank.  Between processes the 64-byte handles of the ranks' blocks travel over a torch.distributed
group (any backend; they are host bytes); inside one process the blocks are connected by pointer.  The link hands out
the two partial slots as torch tensors, so that a column-split projection writes its partial output straight into the
memory the peers read.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .quantized import CudaQuantizedKernelError, RibnContext


class _DevicePointer:
    """Lets torch wrap raw device memory (the link's block) as a tensor without copying."""

    def __init__(self, pointer: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (pointer, False), "version": 3}


class PeerLink:
    def __init__(self, context: RibnContext, rank: int, world: int, slot_bytes: int, local_block: torch.Tensor | None = None):
        self.context, self.rank, self.world = context, rank, world
        self.slot_bytes = (slot_bytes + 255) // 256 * 256
        self._lib = context._lib
        self._block_tensor = local_block            # keeps caller-supplied memory alive
        handle = ctypes.c_void_p()
        status = self._lib.ribn_tp_create(context.handle, rank, world, self.slot_bytes, local_block.data_ptr() if local_block is not None else None,
                                          ctypes.byref(handle))
        if status != _lib.RIBN_OK:
            raise CudaQuantizedKernelError(status, "ribn_tp_create failed")
        self.handle = handle
        self._views = {}

    @staticmethod
    def block_bytes(slot_bytes: int) -> int:
        return _lib.load().ribn_tp_block_bytes((slot_bytes + 255) // 256 * 256)

    def close(self) -> None:
        if getattr(self, "handle", None):
            self._lib.ribn_tp_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int) -> None:
        if status != _lib.RIBN_OK:
            raise CudaQuantizedKernelError(status, self._lib.ribn_tp_last_error(self.handle).decode() or "tensor-parallel link call failed")

    def export_handle(self) -> bytes:
        raw = (ctypes.c_ubyte * 64)()
        self._check(self._lib.ribn_tp_export(self.handle, raw))
        return bytes(raw)

    def connect(self, handles: list[bytes]) -> None:
        joined = (ctypes.c_ubyte * (64 * self.world)).from_buffer_copy(b"".join(handles))
        self._check(self._lib.ribn_tp_connect(self.handle, joined))

    def connect_group(self, group=None) -> None:
        """Exchange the handles over a torch.distributed group and map the peers' blocks."""
        import torch.distributed as dist

        handles = [None] * self.world
        dist.all_gather_object(handles, self.export_handle(), group=group)
        self.connect(handles)
        dist.barrier(group=group)

    def connect_pointers(self, blocks: list[int]) -> None:
        array = (ctypes.c_void_p * self.world)(*blocks)
        self._check(self._lib.ribn_tp_connect_pointers(self.handle, array))

    def set_wait(self, microseconds: int) -> None:
        self._check(self._lib.ribn_tp_set_wait(self.handle, microseconds))

    def partial(self, slot: int, members: int, length: int, dtype: torch.dtype) -> torch.Tensor:
        """Slot `slot` (0 or 1) as a [members, length] tensor: the output buffer of this rank's column-split projection."""
        key = (slot, members, length, dtype)
        if key not in self._views:
            pointer = ctypes.c_void_p()
            self._check(self._lib.ribn_tp_partial(self.handle, slot, ctypes.byref(pointer)))
            nbytes = members * length * torch.empty(0, dtype=dtype).element_size()
            if nbytes > self.slot_bytes:
                raise ValueError(f"{members} x {length} {dtype} does not fit a slot of {self.slot_bytes} bytes")
            with torch.cuda.device(self.context.device):
                raw = torch.as_tensor(_DevicePointer(pointer.value, nbytes), device=self.context.device)
            self._views[key] = raw.view(dtype).view(members, length)
        return self._views[key]

    def allreduce_residual(self, slot: int, hidden: torch.Tensor, members: int, length: int, partial_dtype: torch.dtype) -> None:
        code = _lib.RIBN_F32 if partial_dtype == torch.float32 else _lib.RIBN_BF16
        self._check(self._lib.ribn_tp_allreduce_residual(self.context.handle, self.handle, slot, hidden.data_ptr(), members, length, code))

    def select_tokens(self, logits: torch.Tensor, members: int, index_base: int, tokens: torch.Tensor) -> None:
        self._check(self._lib.ribn_tp_select_tokens(self.context.handle, self.handle, logits.data_ptr(), members, logits.numel() // members, index_base,
                                                    tokens.data_ptr()))
