"""GEMM-fused all-reduce for row-parallel block-FP8 linears on one NVSwitch node.

Stands where the reference runs the block GEMM and then `tensor_model_parallel_all_reduce`
(python/sglang/srt/layers/linear.py:1365-1393, python/sglang/srt/distributed/parallel_state.py:544-623; its
custom all-reduce with IPC-registered buffers is sgl-kernel/csrc/allreduce/custom_all_reduce.cuh).  Here the
all-reduce is two-shot and its first shot happens inside the GEMM: each output tile is stored by the GEMM's
epilogue into the staging buffer of the rank that owns those rows, while later tiles are still being computed;
one more kernel sums the staged blocks in rank order and fetches the other ranks' reduced rows with peer loads.
Every rank ends with bit-identical rows (the NCCL ring does not promise that).

Buffers that peers touch come from the library's own `cudaMalloc` and travel as CUDA IPC handles through the
group's `all_gather_object`; one process drives one GPU.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from ..._lib import check, lib

_BM = 128  # rows of a GEMM output tile: ownership of output rows changes on these boundaries


def _alloc(nbytes: int) -> int:
    p = C.c_void_p()
    check(lib.sglb200_comm_alloc(nbytes, C.byref(p)))
    return p.value


def _exchange(group, world: int, rank: int, ptr: int) -> List[int]:
    """Device pointers of every rank's buffer as mapped in this process (own pointer for `rank`)."""
    handle = (C.c_char * 64)()
    check(lib.sglb200_comm_ipc_export(ptr, handle))
    handles: List[Optional[bytes]] = [None] * world
    dist.all_gather_object(handles, bytes(handle.raw), group=group)
    out = []
    for r, h in enumerate(handles):
        if r == rank:
            out.append(ptr)
            continue
        q = C.c_void_p()
        buf = (C.c_char * 64).from_buffer_copy(h)
        check(lib.sglb200_comm_ipc_open(buf, C.byref(q)))
        out.append(q.value)
    return out


class FusedRowParallelComm:
    """Staging, reduced-row and flag buffers of one tensor-parallel group, sized for `max_elems` output elements."""

    def __init__(self, group, world: int, rank: int, max_elems: int, device: torch.device):
        assert 2 <= world <= 8
        self.group, self.world, self.rank, self.device = group, world, rank, device
        self.max_elems = int(max_elems)
        with torch.cuda.device(device):
            self._stage = _alloc(self.max_elems * 2)
            self._reduced = _alloc(((self.max_elems + world - 1) // world + 8) * 2)
            self._flags = _alloc(lib.sglb200_comm_flag_bytes())
            self.stage_ptrs = _exchange(group, world, rank, self._stage)
            self.reduced_ptrs = _exchange(group, world, rank, self._reduced)
            self.flag_ptrs = _exchange(group, world, rank, self._flags)
        arr = C.c_void_p * world
        self._stage_arr = arr(*self.stage_ptrs)
        self._reduced_arr = arr(*self.reduced_ptrs)
        self._flag_arr = arr(*self.flag_ptrs)
        # Cutting large outputs into row chunks (see `_chunks`) is off: measured on 8 GPUs (8192 x 8192 outputs, K
        # per rank 1024 and 3584) the chunked form took 2.14 ms per layer against 1.73 ms unchunked, because 16 CTAs
        # do not keep NVLink busy and the chunked GEMMs lose SMs and waves; on 2 GPUs 4.87 against 4.65 ms.
        self.pipeline = False
        self.min_comm_ratio = 0.4  # pipeline only where gather time / GEMM time exceeds this (see `_chunks`)
        self.min_waves = 3       # a chunk keeps at least this many waves of GEMM tiles
        self.sm_margin = 16      # SMs the GEMM of a later chunk leaves to the reduce-and-gather of an earlier one
        self.sms = torch.cuda.get_device_properties(device).multi_processor_count
        self._side = torch.cuda.Stream(device=device, priority=-1)
        dist.barrier(group=group)  # nobody launches before every rank has mapped every buffer

    def supports(self, M: int, N: int) -> bool:
        """At least one tile of rows per rank; the staging buffer holds world x (M / world rounded up to whole tiles)
        rows."""
        if M < self.world * _BM or N % 8 != 0:
            return False
        return self.world * lib.sglb200_push_rows_per_owner(M, self.world) * N <= self.max_elems

    def _chunks(self, M: int, N: int, K: int) -> int:
        """Row chunks to pipeline over: the reduce-and-gather of chunk c runs beside the GEMM of chunk c + 1 on the
        SMs that GEMM leaves free.  Chunks keep at least `min_waves` waves of GEMM tiles each.  Pipelining costs
        the later chunks' GEMMs `sm_margin` SMs, so it is used only where the exposed gather is a sizeable part of
        the GEMM time: gather / GEMM = ((p-1)/p * 2MN B / ~700 GB/s) / (2MNK FLOP / ~1.8 PFLOP/s) ~ (p-1)/p * 2570 / K."""
        if not self.pipeline or (self.world - 1) / self.world * 2570.0 / K < self.min_comm_ratio:
            return 1
        tiles_n = (N + 191) // 192
        for c in (4, 2):
            if M % (c * self.world * _BM) == 0 and (M // c // _BM) * tiles_n >= self.min_waves * (self.sms - self.sm_margin):
                return c
        return 1

    def linear(self, xq: torch.Tensor, xs: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
               out_dtype: torch.dtype) -> torch.Tensor:
        """sum over ranks of blockscaled(xq, weight): xq [M, K_local] e4m3, xs [M, K_local/128] float32."""
        M, K = xq.shape
        N = weight.shape[0]
        if not self.supports(M, N):
            raise RuntimeError(f"fused row-parallel all-reduce does not take M={M}, N={N} at world {self.world}")
        if not (xq.is_contiguous() and xs.is_contiguous()):
            xq, xs = xq.contiguous(), xs.contiguous()
        main = torch.cuda.current_stream(xq.device)
        dt = 0 if out_dtype == torch.bfloat16 else 1
        out = torch.empty(M, N, device=xq.device, dtype=out_dtype)
        C_ = self._chunks(M, N, K)
        Mc = M // C_
        arr = C.c_void_p * self.world
        side = self._side if C_ > 1 else main
        if C_ > 1:
            out.record_stream(side)
        for c in range(C_):
            stage_off, red_off = c * Mc * N * 2, c * (Mc // self.world) * N * 2
            stage = self._stage_arr if C_ == 1 else arr(*[p + stage_off for p in self.stage_ptrs])
            reduced = self._reduced_arr if C_ == 1 else arr(*[p + red_off for p in self.reduced_ptrs])
            check(lib.sglb200_fp8_blockwise_scaled_mm_push(
                xq.data_ptr() + c * Mc * K, weight.data_ptr(), xs.data_ptr() + c * Mc * xs.stride(0) * 4,
                weight_scale.data_ptr(), stage, self.world, self.rank, Mc, N, K, xs.stride(0), xs.stride(1), dt,
                self.sm_margin if c > 0 else 0, main.cuda_stream))
            if C_ > 1:
                ev = torch.cuda.Event()
                ev.record(main)
                side.wait_event(ev)
            check(lib.sglb200_reduce_gather(
                self._stage + stage_off, reduced, self._flag_arr, out.data_ptr() + c * Mc * N * 2, self.world,
                self.rank, Mc, N, dt, self.sm_margin if c < C_ - 1 else 0, side.cuda_stream))
        if C_ > 1:
            done = torch.cuda.Event()
            done.record(side)
            main.wait_event(done)
        return out

    def prepare(self, M: int, N: int, out_dtype: torch.dtype = torch.bfloat16) -> None:
        """Builds the device table of per-owner tensor maps for outputs of `M` x `N` now (a small allocation and a
        synchronous copy) instead of inside the first `linear` call of that shape, where it would delay this rank
        against its peers.  Call it for the shapes the layer will serve, before the first forward pass."""
        if self.supports(M, N):
            check(lib.sglb200_push_prepare(self._stage_arr, self.world, M, N, 0 if out_dtype == torch.bfloat16 else 1))

    def check_status(self) -> None:
        """Raises if a wait for a peer (or a GEMM pipeline wait) has expired since the library was loaded: the outputs
        of the affected calls are incomplete.  Synchronises the device."""
        if lib.sglb200_comm_status() != 0:
            raise RuntimeError("fused all-reduce: a wait for a peer's flag expired (a rank stalled for about a second); "
                               "outputs of that call are incomplete")
        if lib.sglb200_gemm_status() != 0:
            raise RuntimeError("fused all-reduce: a GEMM pipeline wait expired; outputs of that call are incomplete")

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        failed = None
        try:
            self.check_status()
        except RuntimeError as e:  # release the buffers first, then report
            failed = e
        dist.barrier(group=self.group)
        for ptrs in (self.stage_ptrs, self.reduced_ptrs, self.flag_ptrs):
            for r, p in enumerate(ptrs):
                if r != self.rank:
                    check(lib.sglb200_comm_ipc_close(p))
        dist.barrier(group=self.group)
        for p in (self._stage, self._reduced, self._flags):
            check(lib.sglb200_comm_free(p))
        if failed is not None:
            raise failed


def comm_status() -> int:
    """0, or 1 if a wait for a peer's flag inside the reduce kernel expired since the library was loaded."""
    return lib.sglb200_comm_status()
