"""Tensor-parallel communicator for the fused all-reduce + residual-add + RMSNorm.

Mirror of the role CustomAllreduce plays in the reference
(fastkernels/tasks/baseline/L1/allreduce.py:95-237: IPC buffers exchanged over a
side channel, set as a module-level global with set_custom_ar / get_custom_ar),
re-designed around the fused kernel fk_allreduce_add_rmsnorm: each rank owns one
cudaMalloc'ed buffer (flag header + two data slots + two staging areas), exports
it with CUDA IPC and maps every peer's buffer.  Row-parallel projections write
their partial output straight into a slot; the norm that follows reads all ranks'
slots over NVLink, or — where that measures faster (large payloads on 8 ranks; the
reference has the same two kernels, allreduce.cu:193-250) — lets each row's owner
reduce it and push the sum into the peers' staging rows.  For small payloads the
projection kernel itself stores its output tiles into every rank's receive area
(`gemm_push`), and the norm reads only local memory.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check, lib

_TP_COMM: "TpComm | None" = None


def set_tp_comm(comm: "TpComm | None") -> None:
    global _TP_COMM
    _TP_COMM = comm


def get_tp_comm() -> "TpComm | None":
    return _TP_COMM


class _DevMem:
    """Exposes a raw device range to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nelem: int):
        self.__cuda_array_interface__ = {
            "shape": (nelem,), "typestr": "<i2", "data": (ptr, False), "version": 2}


class TpComm:
    NUM_SLOTS = 2

    def __init__(self, max_rows: int, cols: int, device, group=None):
        if not (dist.is_available() and dist.is_initialized()):
            raise _lib.FkError("TpComm needs an initialised process group")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device)
        self.max_rows, self.cols = max_rows, cols
        self.header = int(lib.fk_comm_header_bytes())
        self.slot_bytes = (max_rows * cols * 2 + 255) // 256 * 256
        # [header][slot 0][slot 1][staging 0][staging 1][receive areas of slot 0: one per
        # sender][receive areas of slot 1]; a receive area holds every output pair as
        # an 8-byte {two bf16, call number} word
        self.recv_bytes = (max_rows * cols * 4 + 255) // 256 * 256
        self.recv_base = self.header + 2 * self.NUM_SLOTS * self.slot_bytes
        total = self.recv_base + self.NUM_SLOTS * self.world * self.recv_bytes
        self.algo = "auto"                   # "auto" | "one_stage" | "two_stage" | "push"
        with torch.cuda.device(self.device):
            base = C.c_void_p()
            check(lib.fk_comm_alloc(total, C.byref(base)), "fk_comm_alloc")
            self.base = base.value
            handle = C.create_string_buffer(64)
            check(lib.fk_comm_ipc_export(self.base, handle), "fk_comm_ipc_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self.bases = (C.c_void_p * self.world)()
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.bases[r] = self.base
                else:
                    p = C.c_void_p()
                    buf = C.create_string_buffer(h, 64)
                    check(lib.fk_comm_ipc_import(buf, C.byref(p)), "fk_comm_ipc_import")
                    self.bases[r] = p.value
            torch.cuda.synchronize()
        dist.barrier(group=group)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._views: dict = {}
        self._push_dst: dict = {}
        self._epoch_offset = int(lib.fk_comm_epoch_offset())

    def slot_offset(self, slot: int) -> int:
        return self.header + (slot % self.NUM_SLOTS) * self.slot_bytes

    def staging_offset(self, slot: int) -> int:
        return self.header + (self.NUM_SLOTS + slot % self.NUM_SLOTS) * self.slot_bytes

    def two_stage(self, rows: int) -> bool:
        if self.algo != "auto":
            return self.algo == "two_stage"
        return bool(lib.fk_allreduce_two_stage_preferred(self.world, rows, self.cols))

    def pushed(self, rows: int) -> bool:
        """True when the row-parallel projection itself delivers its partial rows to
        every rank (gemm_push) and the norm only reads local memory.  The projection
        and the norm both ask this, with the same `rows`, so they always agree."""
        if self.algo != "auto":
            return self.algo == "push" and 1 <= rows <= 256     # the decode projection's limit
        return bool(lib.fk_allreduce_push_preferred(self.world, rows, self.cols))

    def recv_offset(self, slot: int) -> int:
        return self.recv_base + (slot % self.NUM_SLOTS) * self.world * self.recv_bytes

    def gemm_push(self, x: torch.Tensor, w: torch.Tensor, bias, slot: int) -> torch.Tensor:
        """x @ w.T (+ bias), this rank's partial of a row-parallel projection, stored
        by the projection kernel into the receive areas of all ranks.  Returns the
        (unwritten) slot view, which names the slot for allreduce_add_rmsnorm."""
        from . import ops
        rows = x.shape[0]
        if w.shape[0] != self.cols or rows > self.max_rows:
            raise _lib.FkError(f"receive areas hold [{self.max_rows}, {self.cols}]")
        dst = self._push_dst.get(slot % self.NUM_SLOTS)
        if dst is None:
            dst = (C.c_void_p * self.world)()
            for r in range(self.world):
                dst[r] = self.bases[r] + self.recv_offset(slot) + self.rank * self.recv_bytes
            self._push_dst[slot % self.NUM_SLOTS] = dst
        ops.gemm_bf16_push(x, w, bias, dst, self.world, self.base + self._epoch_offset,
                           status=self.status)
        return self.slot_view(slot, rows, self.cols)

    def slot_view(self, slot: int, rows: int, cols: int) -> torch.Tensor:
        """bf16 [rows, cols] tensor aliasing this rank's data slot."""
        if rows > self.max_rows or cols != self.cols:
            raise _lib.FkError(f"slot holds [{self.max_rows}, {self.cols}], asked [{rows}, {cols}]")
        key = (slot % self.NUM_SLOTS, rows)
        v = self._views.get(key)
        if v is None:
            mem = _DevMem(self.base + self.slot_offset(slot), rows * cols)
            v = torch.as_tensor(mem, device=self.device).view(torch.bfloat16).view(rows, cols)
            self._views[key] = v
        return v

    def allreduce_add_rmsnorm(self, slot: int, rows: int, residual: torch.Tensor,
                              weight: torch.Tensor, eps: float, out: torch.Tensor | None = None):
        """All ranks' partials in `slot` are summed, added to `residual` (updated in
        place) and RMS-normalised into `out`; returns (out, residual)."""
        if out is None:
            out = torch.empty((rows, self.cols), dtype=torch.bfloat16, device=self.device)
        stream = torch.cuda.current_stream().cuda_stream
        if self.pushed(rows):
            check(lib.fk_allreduce_add_rmsnorm_pushed(
                self.base, self.world, self.recv_offset(slot), self.recv_bytes,
                residual.data_ptr(), residual.stride(0), weight.data_ptr(), float(eps),
                out.data_ptr(), out.stride(0), rows, self.cols, self.status.data_ptr(), stream),
                "fk_allreduce_add_rmsnorm_pushed")
        elif self.two_stage(rows):
            check(lib.fk_allreduce_add_rmsnorm_staged(
                self.bases, self.world, self.rank, self.slot_offset(slot),
                self.staging_offset(slot), residual.data_ptr(), residual.stride(0),
                weight.data_ptr(), float(eps), out.data_ptr(), out.stride(0), rows, self.cols,
                self.status.data_ptr(), stream), "fk_allreduce_add_rmsnorm_staged")
        else:
            check(lib.fk_allreduce_add_rmsnorm(
                self.bases, self.world, self.rank, self.slot_offset(slot), residual.data_ptr(),
                residual.stride(0), weight.data_ptr(), float(eps), out.data_ptr(),
                out.stride(0), rows, self.cols, self.status.data_ptr(), stream),
                "fk_allreduce_add_rmsnorm")
        return out, residual
