"""Row-parallel reduce + residual + RMSNorm as one kernel over peer memory.

``tp.row_parallel_gemm`` sums the ranks' integer accumulators with ``ncclAllReduce`` and
converts afterwards; that stays the default.  For decode-sized batches the collective's
latency dominates the step, so this module offers the same arithmetic as ONE kernel per
rank: every rank publishes its accumulators in a peer-mapped buffer, pulls its share of the
rows from all ranks over NVLink, adds them as integers (any rank count gives the same bits),
applies the GEMM epilogue, the residual add and the RMSNorm, and pushes the finished rows to
every rank.  Same bits as all-reduce + ``rms_norm_fxp_from_int``.  The reference has no
counterpart.

The buffers are plain ``cudaMalloc`` memory shared with CUDA IPC handles (one allocation per
rank: accumulators | residual | output | flags); no multicast object is created.  Waits in the
kernel are bounded and report through the library's status word (``check_device_status``).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _native as nat
from ._lib import _INT_DTYPE, _status_word, _on_device
from .config import get_runtime_config


class _RawCuda:
    """Zero-copy window on device memory for ``torch.as_tensor``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3}


def _window(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device)


class PeerReduceNorm:
    """Buffers and launcher of ``fxpr_tp_reduce_norm`` for one process (one rank).

    ``acc``, ``residual`` and ``y`` are ``[max_rows, hidden]`` views of this rank's buffer: the
    row-parallel int GEMM writes ``acc[:rows]``, ``residual[:rows]`` holds the running residual
    (the kernel keeps every rank's copy current), and ``reduce_norm`` returns ``y[:rows]``,
    valid until the next call."""

    def __init__(self, max_rows: int, hidden: int, io_dtype: torch.dtype, int_bits: int = 64, *,
                 group=None, device=None, timeout_cycles: int = 0, _fake_world: int = 0):
        self.lib = nat.load()
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.max_rows, self.hidden, self.io_dtype, self.int_bits = max_rows, hidden, io_dtype, int_bits
        self.timeout_cycles = int(timeout_cycles)
        self.group = group
        if _fake_world:
            # test aid: `_fake_world` ranks' buffers all live on this device and only rank 0
            # ever runs, so the other ranks' flags never arrive
            self.world, self.rank = _fake_world, 0
        elif dist.is_available() and dist.is_initialized():
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        if self.world > 8:
            raise ValueError("PeerReduceNorm supports at most 8 ranks")
        off = [ctypes.c_int64() for _ in range(5)]
        nat.check(self.lib.fxpr_tp_buffer_bytes(max_rows, hidden, int_bits, nat.DTYPE_CODE[io_dtype],
                                                *[ctypes.byref(o) for o in off]), "tp_buffer_bytes")
        self.acc_off, self.res_off, self.y_off, self.flags_off, self.nbytes = (o.value for o in off)
        self._owned, self._opened = [], []
        # Set-up is collective.  A rank whose allocation or mapping fails still takes part in
        # every exchange below, and the outcome is agreed on at the end, so that either every
        # rank gets the object or every rank raises (no rank is left waiting in a collective).
        failure = None
        own, handle = 0, b""
        bases = [None] * self.world
        with _on_device(torch.empty(0, device=self.device)):
            try:
                own, handle = self._alloc()
                bases[self.rank] = own
                if _fake_world:
                    for p in range(1, _fake_world):
                        bases[p], _ = self._alloc()
            except (RuntimeError, ValueError, TypeError) as e:
                failure = f"allocation: {e}"
            if self.world > 1 and not _fake_world:
                handles = [None] * self.world
                dist.all_gather_object(handles, handle if failure is None else None, group=group)
                if failure is None and any(h is None for h in handles):
                    failure = "a peer could not allocate its buffer"
                if failure is None:
                    try:
                        for p in range(self.world):
                            if p != self.rank:
                                ptr = ctypes.c_void_p()
                                buf = (ctypes.c_char * 64).from_buffer_copy(handles[p])
                                nat.check(self.lib.fxpr_tp_open(buf, ctypes.byref(ptr)), "tp_open")
                                self._opened.append(ptr.value)
                                bases[p] = ptr.value
                    except (RuntimeError, ValueError, TypeError) as e:
                        failure = f"mapping a peer's buffer: {e}"
                ok = torch.tensor([0 if failure else 1], device=self.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)    # also: every buffer is zeroed and mapped
                if int(ok.item()) != 1 and failure is None:
                    failure = "a peer could not map the buffers"
        if failure is not None:
            self.acc = self.residual = self.y = None
            self._release()
            raise RuntimeError(f"PeerReduceNorm set-up failed on rank {self.rank}: {failure}")
        self._bases = (ctypes.c_void_p * self.world)(*bases)
        self.ctl = torch.zeros(2, dtype=torch.int32, device=self.device)
        isz, osz = int_bits // 8, torch.empty(0, dtype=io_dtype).element_size()
        self.acc = _window(own + self.acc_off, max_rows * hidden * isz, self.device) \
            .view(_INT_DTYPE[int_bits]).view(max_rows, hidden)
        self.residual = _window(own + self.res_off, max_rows * hidden * osz, self.device) \
            .view(io_dtype).view(max_rows, hidden)
        self.y = _window(own + self.y_off, max_rows * hidden * osz, self.device) \
            .view(io_dtype).view(max_rows, hidden)

    def _alloc(self):
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_char * 64)()
        nat.check(self.lib.fxpr_tp_alloc(self.nbytes, ctypes.byref(ptr), handle), "tp_alloc")
        self._owned.append(ptr.value)
        return ptr.value, bytes(handle)

    def reduce_norm(self, rows: int, weight: torch.Tensor, bias: torch.Tensor | None, eps: float,
                    gemm_frac_bits: int, local_residual: bool = False) -> torch.Tensor:
        """Sum ``acc[:rows]`` over the ranks, update ``residual[:rows]`` on every rank and
        return the normalised rows (a view of ``y``).  With ``local_residual`` a rank updates only
        its own rows of its own residual copy (rows ``[rank * ceil(rows / world), ...)``): enough
        when the residual is only ever fed back into this call, and less traffic."""
        if not 0 <= rows <= self.max_rows:
            raise ValueError(f"rows={rows} exceeds the buffer's {self.max_rows}")
        if weight.dtype != self.io_dtype or weight.numel() != self.hidden:
            raise TypeError("reduce_norm: weight must be [hidden] in the io dtype")
        b = None if bias is None else bias.to(self.io_dtype).contiguous()
        with _on_device(self.ctl):
            st = self.lib.fxpr_tp_reduce_norm(
                self._bases, self.world, self.rank, self.ctl.data_ptr(), self.acc_off, self.res_off,
                self.y_off, self.flags_off, self.int_bits, nat.ptr(b), weight.contiguous().data_ptr(),
                nat.DTYPE_CODE[self.io_dtype], rows, self.hidden, float(eps), int(gemm_frac_bits),
                get_runtime_config().fxp_frac_bits, self.timeout_cycles,
                nat.TP_LOCAL_RESIDUAL if local_residual else 0,
                _status_word(self.device).data_ptr(), nat.stream_ptr(self.device))
        nat.check(st, "tp_reduce_norm")
        return self.y[:rows]

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (all ranks must be done with them)."""
        torch.cuda.synchronize(self.device)
        if self.world > 1 and self._opened and dist.is_initialized():
            dist.barrier(group=self.group)
        self.acc = self.residual = self.y = None
        self._release(barrier=bool(self._opened) and dist.is_initialized())

    def _release(self, barrier: bool = False) -> None:
        for p in self._opened:
            self.lib.fxpr_tp_close(ctypes.c_void_p(p))
        self._opened = []
        if barrier:
            dist.barrier(group=self.group)     # nobody still maps the buffer freed below
        for p in self._owned:
            self.lib.fxpr_tp_free(ctypes.c_void_p(p))
        self._owned = []
