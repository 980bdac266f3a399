"""Tensor-level entry points: torch tensors in, C-ABI calls out.

Each function validates what the reference op validates (`CHECK_INPUT`,
`TORCH_CHECK`), hands raw device pointers plus the current CUDA stream to
`libsglang_b200.so`, and raises `RuntimeError` on a rejected call.  Nothing
here computes on the host and nothing synchronises the device.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ._lib import check, lib

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
FP8_MIN = -448.0
ALIGN_BLOCK = 128  # row-block of the grouped GEMM; moe_align must be called with this block size

_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _cuda_contig(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _dt(t: torch.Tensor, allow=(torch.bfloat16, torch.float16)) -> int:
    if t.dtype not in allow:
        raise RuntimeError(f"unsupported dtype {t.dtype}")
    return _DT[t.dtype]


# --------------------------------------------------------------------------------------------
# quantizer
# --------------------------------------------------------------------------------------------


def per_token_group_quant_fp8_out(
    x: torch.Tensor,
    x_q: torch.Tensor,
    x_s: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    fp8_min: float = FP8_MIN,
    fp8_max: float = FP8_MAX,
) -> None:
    """Writes codes into `x_q` and scales into `x_s` (any 2-D strides: row-major or the
    M-major "column_major_scales" view)."""
    _cuda_contig(x, "input")
    _cuda_contig(x_q, "output_q")
    if x_q.dtype != FP8:
        raise RuntimeError("output_q must be float8_e4m3fn")
    if x_s.dtype != torch.float32 or not x_s.is_cuda:
        raise RuntimeError("output_s must be a float32 CUDA tensor")
    hidden = x.shape[-1]
    tokens = x.numel() // hidden if hidden else 0
    if x_q.numel() != x.numel():
        raise RuntimeError("output_q has the wrong number of elements")
    groups = hidden // group_size if group_size else 0
    if x_s.numel() == 0 and tokens == 0:
        return
    s2 = x_s.reshape(tokens, groups) if x_s.is_contiguous() else x_s
    if s2.dim() != 2 or s2.shape[0] != tokens or s2.shape[1] != groups:
        raise RuntimeError(f"output_s has shape {tuple(x_s.shape)}, expected [{tokens}, {groups}]")
    check(
        lib.sglb200_per_token_group_quant_fp8(
            x.data_ptr(), _dt(x, _DT), x_q.data_ptr(), s2.data_ptr(), tokens, hidden, int(group_size),
            float(eps), float(fp8_min), float(fp8_max), s2.stride(0), s2.stride(1), _stream(x),
        )
    )


def per_token_group_quant_fp8(
    x: torch.Tensor, group_size: int = 128, eps: float = 1e-10, column_major_scales: bool = False,
    scale_tma_aligned: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    x_q = torch.empty_like(x, dtype=FP8)
    tokens = x.numel() // x.shape[-1]
    groups = x.shape[-1] // group_size
    if column_major_scales:
        pad = (tokens + 3) // 4 * 4 if scale_tma_aligned else tokens
        x_s = torch.empty((groups, pad), device=x.device, dtype=torch.float32).t()[:tokens, :]
    else:
        x_s = torch.empty(x.shape[:-1] + (groups,), device=x.device, dtype=torch.float32)
    if tokens > 0:
        per_token_group_quant_fp8_out(x, x_q, x_s, group_size, eps)
    return x_q, x_s


# --------------------------------------------------------------------------------------------
# activation / reduction / gather
# --------------------------------------------------------------------------------------------


def silu_and_mul_out(out: torch.Tensor, x: torch.Tensor) -> None:
    _cuda_contig(x, "input")
    _cuda_contig(out, "out")
    d = x.shape[-1] // 2
    rows = x.numel() // x.shape[-1] if x.shape[-1] else 0
    if out.dtype != x.dtype or out.numel() != rows * d:
        raise RuntimeError("silu_and_mul: out must have input's dtype and half its last dimension")
    check(lib.sglb200_silu_and_mul(out.data_ptr(), x.data_ptr(), _dt(x), rows, d, _stream(x)))


def silu_and_mul_quant_fp8(
    x: torch.Tensor, group_size: int = 128, eps: float = 1e-10, num_rows: Optional[torch.Tensor] = None
) -> Tuple[torch.Tensor, torch.Tensor]:
    """[rows, 2d] -> (codes [rows, d], scales [rows, d/group]).  `num_rows` (device int32 scalar)
    limits the rows processed; the remaining rows of the outputs are left untouched."""
    _cuda_contig(x, "input")
    d = x.shape[-1] // 2
    rows = x.numel() // x.shape[-1]
    q = torch.empty(x.shape[:-1] + (d,), device=x.device, dtype=FP8)
    s = torch.empty(x.shape[:-1] + (d // group_size,), device=x.device, dtype=torch.float32)
    nr = num_rows.data_ptr() if num_rows is not None else None
    check(
        lib.sglb200_silu_and_mul_quant_fp8(
            x.data_ptr(), _dt(x), q.data_ptr(), s.data_ptr(), rows, d, int(group_size), float(eps), nr, _stream(x)
        )
    )
    return q, s


def silu_and_mul_masked_quant_fp8_out(x: torch.Tensor, out_q: torch.Tensor, out_s: torch.Tensor, masked_m: torch.Tensor,
                                      group_size: int = 128, eps: float = 1e-10) -> None:
    """Masked expert layout: x [E, T_pad, 2d]; rows t < masked_m[e] of expert e are activated and quantised into
    out_q [E, T_pad, d] / out_s [E, T_pad, d/group] (float32), every other row of the outputs is left untouched."""
    for t, n in ((x, "input"), (out_q, "output"), (out_s, "output_scale"), (masked_m, "masked_m")):
        _cuda_contig(t, n)
    if x.dim() != 3 or x.shape[-1] % 2:
        raise RuntimeError("silu_and_mul_masked_quant: input must be [experts, padded tokens, 2d]")
    E, T, d2 = x.shape
    d = d2 // 2
    if out_q.dtype != FP8 or tuple(out_q.shape) != (E, T, d):
        raise RuntimeError("silu_and_mul_masked_quant: output must be float8_e4m3fn [experts, padded tokens, d]")
    if out_s.dtype != torch.float32 or tuple(out_s.shape) != (E, T, d // group_size):
        raise RuntimeError("silu_and_mul_masked_quant: output_scale must be float32 [experts, padded tokens, d/group]")
    if masked_m.dtype != torch.int32 or tuple(masked_m.shape) != (E,):
        raise RuntimeError("silu_and_mul_masked_quant: masked_m must be int32 [experts]")
    check(lib.sglb200_silu_and_mul_masked_quant_fp8(x.data_ptr(), _dt(x), out_q.data_ptr(), out_s.data_ptr(), E, T, d,
                                                    int(group_size), float(eps), masked_m.data_ptr(), _stream(x)))


def moe_sum_reduce_out(x: torch.Tensor, out: torch.Tensor, routed_scaling_factor: float) -> None:
    _cuda_contig(x, "input")
    _cuda_contig(out, "output")
    if x.dim() != 3 or out.dim() != 2 or out.shape[0] != x.shape[0] or out.shape[1] != x.shape[2]:
        raise RuntimeError("moe_sum_reduce: input [tokens, topk, hidden], output [tokens, hidden]")
    if out.dtype != x.dtype:
        raise RuntimeError("moe_sum_reduce: dtype mismatch")
    t, k, h = x.shape
    check(lib.sglb200_moe_sum_reduce(x.data_ptr(), out.data_ptr(), _dt(x), t, k, h, float(routed_scaling_factor), _stream(x)))


def moe_sum_reduce_masked_out(x: torch.Tensor, topk_ids: torch.Tensor, out: torch.Tensor,
                              routed_scaling_factor: float) -> None:
    """moe_sum_reduce over the slots whose id in `topk_ids` [tokens, topk] (int32) is not negative."""
    _cuda_contig(x, "input")
    _cuda_contig(out, "output")
    _cuda_contig(topk_ids, "topk_ids")
    if x.dim() != 3 or out.dim() != 2 or out.shape[0] != x.shape[0] or out.shape[1] != x.shape[2]:
        raise RuntimeError("moe_sum_reduce: input [tokens, topk, hidden], output [tokens, hidden]")
    if out.dtype != x.dtype or topk_ids.dtype != torch.int32 or tuple(topk_ids.shape) != tuple(x.shape[:2]):
        raise RuntimeError("moe_sum_reduce: dtype or shape mismatch")
    t, k, h = x.shape
    check(lib.sglb200_moe_sum_reduce_masked(x.data_ptr(), topk_ids.data_ptr(), out.data_ptr(), _dt(x), t, k, h,
                                            float(routed_scaling_factor), _stream(x)))


def gather_sum_rows(src: torch.Tensor, slot: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t] = scale * sum_j src[slot[t, j]] (float32 accumulation); slots outside [0, len(src)) are skipped."""
    _cuda_contig(src, "src")
    _cuda_contig(slot, "slot")
    if src.dim() != 2 or slot.dim() != 2 or slot.dtype != torch.int64:
        raise RuntimeError("gather_sum_rows: src [rows, hidden], slot [tokens, per_token] int64")
    out = torch.empty((slot.shape[0], src.shape[1]), dtype=src.dtype, device=src.device)
    check(lib.sglb200_gather_sum_rows(src.data_ptr(), slot.data_ptr(), out.data_ptr(), _dt(src), slot.shape[0],
                                      slot.shape[1], src.shape[0], src.shape[1], float(scale), _stream(src)))
    return out


def shuffle_mul_sum_out(input: torch.Tensor, output: torch.Tensor, permutation: torch.Tensor,
                        factors: Optional[torch.Tensor] = None) -> None:
    """output[t] = sum_j factors[t, j] * input[permutation[t * topk + j]] (float32 accumulation)."""
    _cuda_contig(input, "input")
    _cuda_contig(output, "output")
    _cuda_contig(permutation, "permutation")
    tokens, hidden = output.shape
    if permutation.dtype != torch.int32 or tokens == 0 or permutation.numel() % max(tokens, 1):
        raise RuntimeError("apply_shuffle_mul_sum: permutation must be int32 with tokens * topk entries")
    topk = permutation.numel() // tokens
    if input.dtype != output.dtype or input.shape[1] != hidden:
        raise RuntimeError("apply_shuffle_mul_sum: input [tokens * topk, hidden] and output [tokens, hidden] of one dtype")
    f = 0
    if factors is not None:
        _cuda_contig(factors, "factors")
        if factors.dtype != output.dtype or factors.numel() != permutation.numel():
            raise RuntimeError("apply_shuffle_mul_sum: factors must match the output dtype and have tokens * topk entries")
        f = factors.data_ptr()
    check(lib.sglb200_shuffle_mul_sum(input.data_ptr(), output.data_ptr(), permutation.data_ptr(), f, _dt(output), tokens,
                                      topk, hidden, _stream(output)))


_GATE_DT = (torch.bfloat16, torch.float16, torch.float32)


def _gate_io(gating: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, what: str):
    _cuda_contig(gating, "gating_output")
    _cuda_contig(topk_weights, "topk_weights")
    _cuda_contig(topk_ids, "topk_ids")
    if gating.dim() != 2 or topk_weights.shape != topk_ids.shape or topk_weights.shape[0] != gating.shape[0]:
        raise RuntimeError(f"{what}: gating [tokens, experts], outputs [tokens, topk]")
    if topk_weights.dtype != torch.float32 or topk_ids.dtype != torch.int32:
        raise RuntimeError(f"{what}: topk_weights must be float32 and topk_ids int32")
    return gating.shape[0], gating.shape[1], topk_weights.shape[1]


def _gate_bias(correction_bias: Optional[torch.Tensor], experts: int, what: str) -> int:
    if correction_bias is None:
        return 0
    _cuda_contig(correction_bias, "correction_bias")
    if correction_bias.dtype != torch.float32 or correction_bias.numel() != experts:
        raise RuntimeError(f"{what}: correction_bias must be float32 [num_experts]")
    return correction_bias.data_ptr()


def topk_softmax_out(topk_weights, topk_ids, gating, renormalize=False, moe_softcapping=0.0, correction_bias=None) -> None:
    rows, experts, k = _gate_io(gating, topk_weights, topk_ids, "topk_softmax")
    check(lib.sglb200_topk_softmax(gating.data_ptr(), _dt(gating, _GATE_DT), rows, experts, k, int(bool(renormalize)),
                                   float(moe_softcapping), _gate_bias(correction_bias, experts, "topk_softmax"),
                                   topk_weights.data_ptr(), topk_ids.data_ptr(), _stream(gating)))


def topk_sigmoid_out(topk_weights, topk_ids, gating, renormalize=False, correction_bias=None) -> None:
    rows, experts, k = _gate_io(gating, topk_weights, topk_ids, "topk_sigmoid")
    check(lib.sglb200_topk_sigmoid(gating.data_ptr(), _dt(gating, _GATE_DT), rows, experts, k, int(bool(renormalize)),
                                   _gate_bias(correction_bias, experts, "topk_sigmoid"), topk_weights.data_ptr(),
                                   topk_ids.data_ptr(), _stream(gating)))


def moe_fused_gate(input: torch.Tensor, bias: torch.Tensor, num_expert_group: int, topk_group: int, topk: int,
                   num_fused_shared_experts: int = 0, routed_scaling_factor: float = 0.0,
                   apply_routed_scaling_factor_on_output: bool = False):
    _cuda_contig(input, "input")
    _cuda_contig(bias, "bias")
    if input.dim() != 2 or bias.numel() != input.shape[1] or bias.dtype != input.dtype:
        raise RuntimeError("moe_fused_gate: input [tokens, experts] and bias [experts] of the same dtype")
    rows, experts = input.shape
    w = torch.empty(rows, topk, dtype=torch.float32, device=input.device)
    ids = torch.empty(rows, topk, dtype=torch.int32, device=input.device)
    check(lib.sglb200_moe_fused_gate(input.data_ptr(), bias.data_ptr(), _dt(input, _GATE_DT), rows, experts, int(num_expert_group),
                                     int(topk_group), int(topk), int(num_fused_shared_experts),
                                     float(routed_scaling_factor), int(bool(apply_routed_scaling_factor_on_output)),
                                     w.data_ptr(), ids.data_ptr(), _stream(input)))
    return w, ids


def gather_rows_fp8(
    src_q: torch.Tensor, src_s: torch.Tensor, sorted_token_ids: torch.Tensor, num_rows: torch.Tensor,
    numel: int, topk: int, max_rows: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows of (src_q, src_s) in expert-sorted order; padding rows are zero."""
    _cuda_contig(src_q, "src_q")
    _cuda_contig(src_s, "src_s")
    hidden, groups = src_q.shape[-1], src_s.shape[-1]
    if max_rows is None:
        max_rows = sorted_token_ids.numel()
    dst_q = torch.empty((max_rows, hidden), device=src_q.device, dtype=src_q.dtype)
    dst_s = torch.empty((max_rows, groups), device=src_q.device, dtype=torch.float32)
    check(
        lib.sglb200_gather_rows_fp8(
            src_q.data_ptr(), src_s.data_ptr(), dst_q.data_ptr(), dst_s.data_ptr(), sorted_token_ids.data_ptr(),
            num_rows.data_ptr(), max_rows, numel, topk, hidden, groups, _stream(src_q),
        )
    )
    return dst_q, dst_s


# --------------------------------------------------------------------------------------------
# moe_align_block_size
# --------------------------------------------------------------------------------------------


def moe_align_block_size_out(
    topk_ids: torch.Tensor, num_experts: int, block_size: int, sorted_token_ids: torch.Tensor,
    experts_ids: torch.Tensor, num_tokens_post_pad: torch.Tensor, cumsum_buffer: torch.Tensor,
    pad_sorted_token_ids: bool = False,
) -> None:
    """`num_experts` is the bucket count (model experts + 1), as the reference op is called."""
    _cuda_contig(topk_ids, "topk_ids")
    if topk_ids.dtype != torch.int32:
        raise RuntimeError("topk_ids must be int32")
    for t, n in ((sorted_token_ids, "sorted_token_ids"), (experts_ids, "experts_ids"),
                 (num_tokens_post_pad, "num_tokens_post_pad"), (cumsum_buffer, "cumsum_buffer")):
        _cuda_contig(t, n)
        if t.dtype != torch.int32:
            raise RuntimeError(f"{n} must be int32")
    numel = topk_ids.numel()
    if cumsum_buffer.numel() < num_experts + 1:
        raise RuntimeError("cumsum_buffer needs num_experts + 1 entries")
    if sorted_token_ids.numel() < numel + num_experts * (block_size - 1) and numel > 0:
        # the exact worst case is min(numel, buckets) * (block-1); accept the reference's allocation
        pass
    ws_bytes = lib.sglb200_moe_align_workspace_bytes(numel, int(num_experts))
    ws = torch.empty(ws_bytes, device=topk_ids.device, dtype=torch.uint8) if ws_bytes else None
    check(
        lib.sglb200_moe_align_block_size(
            topk_ids.data_ptr(), numel, int(num_experts), int(block_size), sorted_token_ids.data_ptr(),
            experts_ids.data_ptr(), num_tokens_post_pad.data_ptr(), cumsum_buffer.data_ptr(),
            1 if pad_sorted_token_ids else 0, ws.data_ptr() if ws is not None else None, ws_bytes, _stream(topk_ids),
        )
    )


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """Python-level wrapper with the reference's allocation rules
    (fused_moe_triton/moe_align_block_size.py:57-81).  `num_experts` = model experts."""
    max_padded = topk_ids.numel() + (num_experts + 1) * (block_size - 1)
    dev = topk_ids.device
    sorted_ids = torch.empty((max_padded,), dtype=torch.int32, device=dev)
    expert_ids = torch.empty(((max_padded + block_size - 1) // block_size,), dtype=torch.int32, device=dev)
    post = torch.empty((1,), dtype=torch.int32, device=dev)
    cumsum = torch.empty((num_experts + 2,), dtype=torch.int32, device=dev)
    moe_align_block_size_out(topk_ids, num_experts + 1, block_size, sorted_ids, expert_ids, post, cumsum, True)
    return sorted_ids, expert_ids, post


def moe_align_block_size_local(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """The sort without its segment of filtered ids (-1 = expert of another rank): rows of local experts only."""
    max_padded = topk_ids.numel() + (num_experts + 1) * (block_size - 1)
    dev = topk_ids.device
    nblk = (max_padded + block_size - 1) // block_size
    sorted_ids = torch.empty((2, max_padded), dtype=torch.int32, device=dev)
    expert_ids = torch.empty((2, nblk), dtype=torch.int32, device=dev)
    post = torch.empty((2,), dtype=torch.int32, device=dev)
    cumsum = torch.empty((num_experts + 2,), dtype=torch.int32, device=dev)
    moe_align_block_size_out(topk_ids, num_experts + 1, block_size, sorted_ids[0], expert_ids[0], post[0:1], cumsum, True)
    check(lib.sglb200_moe_align_drop_filtered(
        sorted_ids[0].data_ptr(), expert_ids[0].data_ptr(), cumsum.data_ptr(), post[0:1].data_ptr(),
        sorted_ids[1].data_ptr(), expert_ids[1].data_ptr(), post[1:2].data_ptr(), max_padded, int(block_size),
        _stream(topk_ids)))
    return sorted_ids[1], expert_ids[1], post[1:2]


# --------------------------------------------------------------------------------------------
# GEMMs
# --------------------------------------------------------------------------------------------


def w8a8_block_fp8_matmul(
    A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor, block_size=(128, 128),
    output_dtype: torch.dtype = torch.bfloat16, bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """A [..., K] e4m3, B [N, K] e4m3, As [..., ceil(K/128)] f32 (any strides), Bs [ceil(N/128), ceil(K/128)] f32."""
    if list(block_size) != [128, 128]:
        raise RuntimeError("only block_size [128, 128] is supported")
    _cuda_contig(A, "A")
    _cuda_contig(B, "B")
    if A.dtype != FP8 or B.dtype != FP8:
        raise RuntimeError("A and B must be float8_e4m3fn")
    if output_dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError("output dtype must be bfloat16 or float16")
    K = A.shape[-1]
    M = A.numel() // K if K else 0
    N = B.shape[0]
    if B.dim() != 2 or B.shape[1] != K:
        raise RuntimeError("B must be [N, K] with K matching A")
    kb, nb = (K + 127) // 128, (N + 127) // 128
    Bs = Bs.contiguous()
    if Bs.dtype != torch.float32 or tuple(Bs.shape) != (nb, kb):
        raise RuntimeError(f"Bs must be float32 [{nb}, {kb}]")
    As2 = As.reshape(M, kb) if As.is_contiguous() else As
    if As2.dtype != torch.float32 or As2.dim() != 2 or tuple(As2.shape) != (M, kb):
        raise RuntimeError(f"As must be float32 [{M}, {kb}]")
    C = torch.empty(A.shape[:-1] + (N,), device=A.device, dtype=output_dtype)
    if bias is not None:
        bias = bias.to(output_dtype).contiguous()
    if M > 0:
        ws_bytes = lib.sglb200_gemm_workspace_bytes(M, N, K)  # split-K scratch for the small-M regime
        ws = torch.empty(ws_bytes, device=A.device, dtype=torch.uint8) if ws_bytes else None
        check(
            lib.sglb200_fp8_blockwise_scaled_mm(
                A.data_ptr(), B.data_ptr(), As2.data_ptr(), Bs.data_ptr(), C.data_ptr(),
                bias.data_ptr() if bias is not None else None, M, N, K, As2.stride(0), As2.stride(1),
                0 if output_dtype == torch.bfloat16 else 1, ws.data_ptr() if ws is not None else None, ws_bytes,
                _stream(A),
            )
        )
    return C


def grouped_block_fp8_matmul(
    A: torch.Tensor, As: torch.Tensor, B: torch.Tensor, Bs: torch.Tensor, sorted_token_ids: torch.Tensor,
    expert_ids: torch.Tensor, num_rows: torch.Tensor, *, numel: int, scatter: bool,
    row_weights: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
    output_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """Grouped GEMM over expert-sorted rows (see sglb200_fp8_blockwise_grouped_mm)."""
    for t, n in ((A, "A"), (As, "As"), (B, "B"), (Bs, "Bs")):
        _cuda_contig(t, n)
    E, N, K = B.shape
    max_rows = A.shape[0]
    if out is None:
        out = torch.empty((numel if scatter else max_rows, N), device=A.device, dtype=output_dtype)
    if row_weights is not None:
        row_weights = row_weights.reshape(-1)
        if row_weights.dtype != torch.float32 or not row_weights.is_contiguous():
            raise RuntimeError("row_weights must be contiguous float32")
    check(
        lib.sglb200_fp8_blockwise_grouped_mm(
            A.data_ptr(), As.data_ptr(), B.data_ptr(), Bs.data_ptr(), out.data_ptr(), sorted_token_ids.data_ptr(),
            expert_ids.data_ptr(), num_rows.data_ptr(), row_weights.data_ptr() if row_weights is not None else None,
            max_rows, numel, E, N, K, 1 if scatter else 0, 0 if out.dtype == torch.bfloat16 else 1, _stream(A),
        )
    )
    return out


def gemm_status() -> int:
    """0, or 1 if a pipeline wait inside a GEMM kernel expired since the library was loaded (synchronises)."""
    return lib.sglb200_gemm_status()


def stream_status() -> int:
    """0, or 1 if a wait for a staged tile inside a streaming kernel (quantizer, fused silu_and_mul + quantizer)
    expired since the library was loaded (synchronises)."""
    return lib.sglb200_stream_status()
