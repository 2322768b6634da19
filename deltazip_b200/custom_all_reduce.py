"""All-reduce of the row-parallel layers' partial outputs over NVLink peer memory.

Host side of the library's one-shot all-reduce (`dz_allreduce_*`), in the role of
serving/vllm/model_executor/parallel_utils/custom_all_reduce.py:29-121,187-262: a
process-wide handle created once per tensor-parallel group, `custom_all_reduce(x)` returning
the reduced tensor (out of place) or None when the message does not qualify, so that the
caller falls back to NCCL exactly as the reference does (communication_op.py:32-40).

Differences by design: one kernel per call with a bounded wait (a dead or late peer yields
DZ_ERR_TIMEOUT instead of a hang), fp32 accumulation in rank order (bit-identical results on
all ranks), and a staging buffer the producer may write into directly (`staging_like`), which
removes the copy-in the reference pays outside CUDA graphs.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check, lib

_DTYPES = {torch.float16: _lib.DZ_DTYPE_F16, torch.bfloat16: _lib.DZ_DTYPE_BF16,
           torch.float32: _lib.DZ_DTYPE_F32}


class CustomAllreduce:
    """One rank's end of the peer-memory all-reduce.  All ranks of `group` must construct it
    collectively and issue the same sequence of `all_reduce` calls."""

    def __init__(self, rank: int, world_size: int, max_size: int = 8192 * 1024,
                 group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None,
                 symmetric: Optional[bool] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("CustomAllreduce needs CUDA devices")
        self.rank, self.world_size, self.max_size = rank, world_size, max_size
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self._ctx = ctypes.c_void_p()
        self.multicast = False
        self._symm = None
        if symmetric is None:
            symmetric = os.environ.get("DZ_AR_SYMMETRIC", "1") != "0"
        with torch.cuda.device(self.device):
            if world_size > 1 and symmetric and self._create_symmetric(group):
                return
            check(lib().dz_allreduce_create(ctypes.byref(self._ctx), rank, world_size, max_size),
                  "dz_allreduce_create")
            handle = (ctypes.c_ubyte * 64)()
            check(lib().dz_allreduce_export(self._ctx, handle), "dz_allreduce_export")
            if world_size > 1:
                mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.device)
                gathered = [torch.empty_like(mine) for _ in range(world_size)]
                dist.all_gather(gathered, mine, group=group)
                blob = bytes(torch.cat(gathered).cpu().tolist())
                buf = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
                check(lib().dz_allreduce_connect(self._ctx, buf), "dz_allreduce_connect")
                dist.barrier(group=group)   # every region is mapped everywhere before first use

    def _create_symmetric(self, group) -> bool:
        """Regions in torch's symmetric memory (PyTorch as the allocator: it maps every rank's
        buffer into every process and, on NVSwitch machines, binds them to one multicast
        address).  All ranks succeed or fall back together.  With a multicast address the
        in-switch kernel becomes available (`set_variant(3)` / `set_variant(4)`)."""
        ok, ptrs, mc, region, hdl = 1, None, 0, None, None
        try:
            import torch.distributed._symmetric_memory as symm_mem
            nbytes = lib().dz_allreduce_region_bytes(self.max_size)
            region = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            region.zero_()
            torch.cuda.synchronize(self.device)
            hdl = symm_mem.rendezvous(region, group if group is not None else dist.group.WORLD)
            ptrs, mc = list(hdl.buffer_ptrs), int(hdl.multicast_ptr or 0)
            if len(ptrs) != self.world_size or any(p == 0 or p % 256 for p in ptrs):
                ok = 0
        except Exception:                                      # noqa: BLE001 -- any failure: IPC path
            ok = 0
        flag = torch.tensor([ok, 1 if mc else 0], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag[0].item()) == 0:
            return False
        if int(flag[1].item()) == 0:
            mc = 0
        arr = (ctypes.c_void_p * self.world_size)(*ptrs)
        check(lib().dz_allreduce_create_external(ctypes.byref(self._ctx), self.rank, self.world_size,
                                                 self.max_size, arr, ctypes.c_void_p(mc or None)),
              "dz_allreduce_create_external")
        self._symm = (region, hdl)                             # keep the mapping alive
        self.multicast = bool(mc)
        dist.barrier(group=group)
        return True

    def should_custom_ar(self, inp: torch.Tensor) -> bool:
        nbytes = inp.numel() * inp.element_size()
        return (inp.is_cuda and inp.dtype in _DTYPES and inp.is_contiguous()
                and 0 < nbytes <= self.max_size and nbytes % 16 == 0 and inp.data_ptr() % 16 == 0)

    def staging_like(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """A tensor of `shape` aliasing the staging buffer of the NEXT all_reduce: a producer
        that writes its result there (e.g. the SBMM through `out=`) and passes the tensor to
        `all_reduce` saves the copy into peer-visible memory."""
        numel = 1
        for d in shape:
            numel *= d
        esz = torch.empty((), dtype=dtype).element_size()
        if numel * esz > self.max_size:
            raise ValueError("tensor larger than the staging buffer")
        ptr, nbytes = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().dz_allreduce_staging(self._ctx, ctypes.byref(ptr), ctypes.byref(nbytes)),
              "dz_allreduce_staging")
        return _alias(ptr.value, tuple(shape), dtype, self.device)

    def all_reduce(self, inp: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty_like(inp)
        stream = torch.cuda.current_stream(inp.device).cuda_stream
        check(lib().dz_allreduce_run(self._ctx, inp.data_ptr(), out.data_ptr(), inp.numel(),
                                     _DTYPES[inp.dtype], stream), "dz_allreduce_run")
        return out

    # -- fused form: the producer pushes its tiles, the reduction sums local slots ------------
    PUSH_SLOT_BYTES = 2 << 20

    def can_push(self, rows: int, cols: int, dtype: torch.dtype) -> bool:
        """Whether an [rows, cols] partial output of `dtype` can take the fused path."""
        return (self.world_size > 1 and dtype in (torch.float16, torch.bfloat16) and cols % 128 == 0
                and 0 < rows * cols * 2 <= self.PUSH_SLOT_BYTES
                and ((rows + 127) // 128) * (cols // 128) <= 256)

    def push_target(self, rows: int, cols: int, dtype: torch.dtype) -> "_lib.PushTarget":
        """Addresses for the producer of the NEXT reduction (pass as `push=` to ops.sbmm, then
        call all_reduce_pushed with the same shape)."""
        t = _lib.PushTarget()
        check(lib().dz_allreduce_push_target(self._ctx, rows, cols, _DTYPES[dtype], ctypes.byref(t)),
              "dz_allreduce_push_target")
        return t

    def all_reduce_pushed(self, rows: int, cols: int, dtype: torch.dtype,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty((rows, cols), dtype=dtype, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        check(lib().dz_allreduce_run_pushed(self._ctx, out.data_ptr(), rows, cols, _DTYPES[dtype], stream),
              "dz_allreduce_run_pushed")
        return out

    def set_variant(self, variant: int) -> None:
        """0: kernel chosen by message size and rank count; 1: always the one-shot kernel;
        2: the two-stage kernel whenever there are more than two ranks; 3: always the in-switch
        (multimem) kernel; 4: like 0 with the in-switch kernel from 64 KB on more than two ranks
        (3 and 4 need `self.multicast`).  All ranks alike."""
        check(lib().dz_allreduce_set_variant(self._ctx, variant), "dz_allreduce_set_variant")

    def status(self) -> int:
        st = ctypes.c_int()
        check(lib().dz_allreduce_status(self._ctx, ctypes.byref(st)), "dz_allreduce_status")
        return st.value

    def close(self) -> None:
        if self._ctx:
            lib().dz_allreduce_destroy(self._ctx)
            self._ctx = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _CudaArray:
    """Minimal __cuda_array_interface__ carrier so torch can alias raw device memory."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False),
                                         "version": 3, "strides": None}


def _alias(ptr: int, shape, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    # bf16 has no numpy typestr: alias as int16 and reinterpret
    if dtype == torch.float32:
        return torch.as_tensor(_CudaArray(ptr, shape, "<f4"), device=device)
    t = torch.as_tensor(_CudaArray(ptr, shape, "<i2"), device=device)
    return t.view(dtype)


_HANDLE: Optional[CustomAllreduce] = None


def init_custom_ar(rank: int, world_size: int, max_size: int = 8192 * 1024,
                   group: Optional[dist.ProcessGroup] = None) -> Optional[CustomAllreduce]:
    """Creates the process-wide handle (no-op for one rank or without CUDA)."""
    global _HANDLE
    if _HANDLE is not None or world_size == 1 or not torch.cuda.is_available():
        return _HANDLE
    if world_size > 8:
        return None
    _HANDLE = CustomAllreduce(rank, world_size, max_size, group)
    return _HANDLE


def get_handle() -> Optional[CustomAllreduce]:
    return _HANDLE


def destroy_custom_ar() -> None:
    global _HANDLE
    if _HANDLE is not None:
        _HANDLE.close()
        _HANDLE = None


def custom_all_reduce(inp: torch.Tensor) -> Optional[torch.Tensor]:
    """Reduced tensor, or None when the handle is absent or the message does not qualify."""
    h = _HANDLE
    if h is None or not h.should_custom_ar(inp):
        return None
    return h.all_reduce(inp)
