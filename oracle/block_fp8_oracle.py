"""CPU restatement of SGLang's block-wise FP8 W8A8 hot path (TEST INFRASTRUCTURE ONLY).

This module is the parity oracle.  It is imported by the tests, by the smoke
check and by the CPU-baseline leg of the benchmark, and by nothing else: the
product path (`sglang_b200`) never imports it and has no CPU fallback.

Everything here is numpy on float32 / uint8 / int32 arrays so the arithmetic is
explicit.  bfloat16 values travel as uint16 bit patterns, float8_e4m3fn values
as uint8 codes.  Each function cites the reference code it restates (paths are
relative to the reference repository root).

Pinning: the functions are checked (tests/test_oracle_golden.py) against
fixtures produced by executing the reference's own torch-native test oracles
(python/sglang/test/test_block_fp8.py) and against the constructive
known-answer cases of test/srt/quant/test_fp8_kernel.py and the worked example
in python/sglang/srt/layers/moe/fused_moe_triton/moe_align_block_size.py:43-55.
"""
from __future__ import annotations

import numpy as np

FP8_MAX = np.float32(448.0)
FP8_MIN = np.float32(-448.0)

# ----------------------------------------------------------------------------
# bfloat16 / float8_e4m3fn bit-level helpers
# ----------------------------------------------------------------------------


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bfloat16 patterns -> float32 (exact)."""
    b = np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)
    return b.view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 patterns, round-to-nearest-even (what
    `__float2bfloat16_rn` and torch's `.to(torch.bfloat16)` do)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    nan = np.isnan(x)
    rounding = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    r = ((u + rounding) >> np.uint32(16)).astype(np.uint16)
    r[nan] = np.uint16(0x7FC0)
    return r


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def _build_e4m3_tables():
    codes = np.arange(256, dtype=np.uint32)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    exp = (codes >> 3) & 0xF
    man = codes & 0x7
    val = np.where(exp == 0, man / 8.0 * 2.0**-6, (1.0 + man / 8.0) * 2.0 ** (exp.astype(np.float64) - 7))
    val = sign * val
    val[0x7F] = np.nan
    val[0xFF] = np.nan
    dec = val.astype(np.float32)
    pos = val[:0x7F].astype(np.float64)  # codes 0x00..0x7E: 0 .. 448, strictly increasing
    mid = (pos[:-1] + pos[1:]) / 2.0
    return dec, pos, mid


E4M3_DECODE, _E4M3_POS, _E4M3_MID = _build_e4m3_tables()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    """uint8 float8_e4m3fn codes -> float32 (exact)."""
    return E4M3_DECODE[np.ascontiguousarray(codes, dtype=np.uint8)]


def e4m3_encode_rne_sat(x: np.ndarray) -> np.ndarray:
    """float32 -> float8_e4m3fn code, round-to-nearest-even, saturating to +-448.

    This is `__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)`, which is
    what `__nv_fp8_e4m3(float)` performs in
    sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:111, and equals torch's
    `.to(torch.float8_e4m3fn)` on values already clamped to [-448, 448]
    (python/sglang/test/test_block_fp8.py:44).  NaN maps to 0x7F.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    a = np.minimum(a, 448.0)
    idx = np.searchsorted(_E4M3_MID, a, side="left")  # number of midpoints strictly below a
    idx = np.minimum(idx, 0x7E)
    tie = np.zeros(a.shape, dtype=bool)
    inb = idx < 0x7E
    tie[inb] = a[inb] == _E4M3_MID[idx[inb]]
    # a == mid[idx] means a sits exactly between code idx and idx+1: pick the even code
    idx = np.where(tie & ((idx & 1) == 1), idx + 1, idx)
    code = idx.astype(np.uint8)
    code = np.where(np.signbit(x), code | np.uint8(0x80), code).astype(np.uint8)
    code = np.where(np.isnan(x), np.uint8(0x7F), code).astype(np.uint8)
    return code


# ----------------------------------------------------------------------------
# R1: per-token-group quantizer
# ----------------------------------------------------------------------------


def per_token_group_quant_fp8(x_f32: np.ndarray, group_size: int = 128, eps: float = 1e-10):
    """Canonical 1 x `group_size` activation quantizer.

    Restates sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:44-113 (CUDA
    default path) == python/sglang/test/test_block_fp8.py:23-48 (torch-native)
    == the column-major Triton kernel
    python/sglang/srt/layers/quantization/fp8_kernel.py:168-216:

        amax = max(|x|, eps)             (float32)
        s    = amax / 448                (IEEE float32 division)
        q    = e4m3_rne_sat(clamp(x / s, -448, 448))   (IEEE float32 division)

    `x_f32` holds the bf16/fp16 input values widened to float32, shape [..., K]
    with K % group_size == 0.  Returns (codes uint8 [..., K], scales float32
    [..., K/group_size]).
    """
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    K = x.shape[-1]
    assert K % group_size == 0
    g = x.reshape(-1, group_size)
    amax = np.maximum(np.max(np.abs(g), axis=-1, keepdims=True), np.float32(eps)).astype(np.float32)
    s = (amax / FP8_MAX).astype(np.float32)
    q = (g / s).astype(np.float32)
    q = np.minimum(np.maximum(q, FP8_MIN), FP8_MAX)
    codes = e4m3_encode_rne_sat(q).reshape(x.shape)
    scales = s.reshape(x.shape[:-1] + (K // group_size,))
    return codes, scales


def quant_weight_block_fp8(w_f32: np.ndarray, block_n: int = 128, block_k: int = 128):
    """Weight preparation used by every config: one float32 scale (block amax /
    448) per block_n x block_k block, codes = e4m3(clamp(w / s)).  Follows the
    recipe of test/srt/cpu/utils.py:39-87 (`convert_weight`) with the zero-block
    guard (an all-zero block gets scale 1).  Works on [..., N, K].
    """
    w = np.ascontiguousarray(w_f32, dtype=np.float32)
    *lead, N, K = w.shape
    nb, kb = -(-N // block_n), -(-K // block_k)
    wp = np.zeros(tuple(lead) + (nb * block_n, kb * block_k), dtype=np.float32)
    wp[..., :N, :K] = w
    blk = wp.reshape(tuple(lead) + (nb, block_n, kb, block_k))
    amax = np.max(np.abs(blk), axis=(-3, -1), keepdims=True).astype(np.float32)
    s = (amax / FP8_MAX).astype(np.float32)
    s = np.where(s == 0, np.float32(1.0), s).astype(np.float32)
    q = np.minimum(np.maximum((blk / s).astype(np.float32), FP8_MIN), FP8_MAX)
    codes = e4m3_encode_rne_sat(q).reshape(wp.shape)[..., :N, :K]
    scales = s.reshape(tuple(lead) + (nb, kb))
    return np.ascontiguousarray(codes), np.ascontiguousarray(scales)


# ----------------------------------------------------------------------------
# R2: block-scaled GEMM
# ----------------------------------------------------------------------------


def w8a8_block_fp8_matmul(a_codes, b_codes, a_s, b_s, block_n: int = 128, block_k: int = 128, out_bf16: bool = True):
    """C[m,n] = sum_kb a_s[m,kb] * b_s[n//block_n,kb] * sum_{k in kb} A[m,k]*B[n,k].

    Restates python/sglang/test/test_block_fp8.py:273-325
    (`native_w8a8_block_fp8_matmul`): dequantised float32 operands, float32
    accumulation block by block, result rounded to bf16 when `out_bf16`.
    a_codes [M,K] uint8, b_codes [N,K] uint8, a_s [M,ceil(K/bk)] f32,
    b_s [ceil(N/bn), ceil(K/bk)] f32.  Returns float32 (bf16-rounded values).
    """
    A = e4m3_decode(a_codes)
    B = e4m3_decode(b_codes)
    M, K = A.shape
    N = B.shape[0]
    kt = -(-K // block_k)
    nt = -(-N // block_n)
    assert a_s.shape == (M, kt) and b_s.shape == (nt, kt)
    C = np.zeros((M, N), dtype=np.float32)
    for i in range(kt):
        a = A[:, i * block_k : (i + 1) * block_k]
        for j in range(nt):
            b = B[j * block_n : (j + 1) * block_n, i * block_k : (i + 1) * block_k]
            s = (a_s[:, i : i + 1] * b_s[j, i]).astype(np.float32)
            C[:, j * block_n : (j + 1) * block_n] += (a @ b.T).astype(np.float32) * s
    return bf16_round(C) if out_bf16 else C


# ----------------------------------------------------------------------------
# R3: moe_align_block_size
# ----------------------------------------------------------------------------


def moe_align_block_size(topk_ids: np.ndarray, block_size: int, num_experts: int):
    """Stable counting sort of the flat `topk_ids` into block-padded expert segments.

    Restates sgl-kernel/csrc/moe/moe_align_kernel.cu:56-228 plus the scatter at
    :28-41, called as in
    python/sglang/srt/layers/moe/fused_moe_triton/moe_align_block_size.py:57-81
    (the wrapper passes num_experts+1 buckets; ids are shifted by +1 so that id
    -1, a non-local expert under expert parallelism, falls in bucket 0 and is
    reported as expert -1).  Intra-expert order is ascending flat index, the
    order produced by the reference's CPU implementation
    (sgl-kernel/csrc/cpu/moe.cpp:134-189) and Triton test oracle
    (sgl-kernel/tests/test_moe_align.py:21-144); the CUDA kernel's atomicAdd
    scatter yields some permutation of it.

    Returns (sorted_token_ids int32 [numel + (E+1)*(block-1)], expert_ids int32
    [ceil(that/block)], num_tokens_post_pad int32 [1]).  Only
    sorted_token_ids[:num_tokens_post_pad] and
    expert_ids[:num_tokens_post_pad/block] are defined; the rest is filled with
    a sentinel (-7) here and is uninitialised memory in the reference.
    """
    ids = np.ascontiguousarray(topk_ids, dtype=np.int32).reshape(-1)
    numel = ids.size
    buckets = num_experts + 1
    max_padded = numel + buckets * (block_size - 1)
    sorted_ids = np.full(max_padded, -7, dtype=np.int32)
    expert_ids = np.full(-(-max_padded // block_size), -7, dtype=np.int32)
    b = ids + 1
    assert b.min(initial=0) >= 0 and b.max(initial=0) < buckets
    counts = np.bincount(b, minlength=buckets).astype(np.int64)
    padded = (counts + block_size - 1) // block_size * block_size
    cumsum = np.concatenate([[0], np.cumsum(padded)]).astype(np.int64)
    total = int(cumsum[-1])
    sorted_ids[:total] = numel
    for e in range(buckets):
        expert_ids[cumsum[e] // block_size : cumsum[e + 1] // block_size] = e - 1
    order = np.argsort(b, kind="stable")
    starts = np.concatenate([[0], np.cumsum(counts)])[:-1]
    rank_in_bucket = np.arange(numel) - np.repeat(starts, counts)
    sorted_ids[cumsum[b[order]] + rank_in_bucket] = order.astype(np.int32)
    return sorted_ids, expert_ids, np.array([total], dtype=np.int32)


# ----------------------------------------------------------------------------
# R5: silu_and_mul (+ requantisation), R6: top-k weighted sum
# ----------------------------------------------------------------------------


def silu_and_mul(x_f32: np.ndarray) -> np.ndarray:
    """h = bf16( bf16(silu_f32(gate)) * up ), gate = x[..., :d], up = x[..., d:].

    Restates sgl-kernel/csrc/elementwise/activation.cu:55-60,85-105 (FlashInfer
    `act_and_mul_kernel`): silu is evaluated in float32 as x / (1 + expf(-x)),
    rounded to the tensor dtype, then multiplied by `up` in that dtype.
    Input: bf16 values widened to float32.  Output float32 holding bf16 values.
    """
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    d = x.shape[-1] // 2
    gate, up = x[..., :d], x[..., d:]
    with np.errstate(over="ignore"):
        act = (gate / (np.float32(1.0) + np.exp(-gate, dtype=np.float32))).astype(np.float32)
    act = bf16_round(act)
    return bf16_round((act * up).astype(np.float32))


def moe_sum_reduce(x_f32: np.ndarray, routed_scaling_factor: float = 1.0) -> np.ndarray:
    """out[t,:] = bf16( scale * sum_k x[t,k,:] ) with float32 accumulation in
    ascending k.  Restates sgl-kernel/csrc/moe/moe_sum_reduce.cu:56-116."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    acc = np.zeros((x.shape[0], x.shape[2]), dtype=np.float32)
    for k in range(x.shape[1]):
        acc = (acc + x[:, k, :]).astype(np.float32)
    return bf16_round((acc * np.float32(routed_scaling_factor)).astype(np.float32))


# ----------------------------------------------------------------------------
# R4-R6: the MoE layer
# ----------------------------------------------------------------------------


def fused_experts_block_fp8(
    x_f32,
    w13_codes,
    w13_s,
    w2_codes,
    w2_s,
    topk_weights,
    topk_ids,
    routed_scaling_factor: float = 1.0,
    block: int = 128,
):
    """Block-FP8 MoE layer with the reference's rounding points.

    Restates `fused_experts_impl`
    (python/sglang/srt/layers/moe/fused_moe_triton/fused_moe.py:369-667) for
    use_fp8_w8a8 with block_shape [128,128]: quantise x per 1x128 group
    (fused_moe_triton_kernels.py:632-633); GEMM #1 -> bf16 (:572);
    silu_and_mul in bf16 (fused_moe.py:555-556); re-quantise; GEMM #2, scaled by
    the top-k weight in float32 before the bf16 cast
    (fused_moe_triton_kernels.py:566-572); float32 sum over top-k times
    routed_scaling_factor -> bf16 (moe_sum_reduce.cu:82-103).  Entries with
    expert id -1 contribute zeros (fused_moe_triton_kernels.py:421-437).

    x_f32 [T,H] bf16 values as float32; w13_codes [E,2I,H]; w2_codes [E,H,I].
    Returns float32 [T,H] holding bf16 values.
    """
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    T, H = x.shape
    E = w13_codes.shape[0]
    topk = topk_ids.shape[1]
    xq, xs = per_token_group_quant_fp8(x, block)
    ic3 = np.zeros((T, topk, H), dtype=np.float32)
    for e in range(E):
        tok, slot = np.nonzero(topk_ids == e)
        if tok.size == 0:
            continue
        ic1 = w8a8_block_fp8_matmul(xq[tok], w13_codes[e], xs[tok], w13_s[e], block, block)
        h = silu_and_mul(ic1)
        hq, hs = per_token_group_quant_fp8(h, block)
        o = w8a8_block_fp8_matmul(hq, w2_codes[e], hs, w2_s[e], block, block, out_bf16=False)
        w = topk_weights[tok, slot].astype(np.float32)[:, None]
        ic3[tok, slot] = bf16_round((o * w).astype(np.float32))
    return moe_sum_reduce(ic3, routed_scaling_factor)


def block_fp8_linear(x_f32, w_codes, w_s, bias_f32=None, block: int = 128):
    """`Fp8LinearMethod.apply` for block quantisation:
    python/sglang/srt/layers/quantization/fp8_utils.py:306-326 — quantise,
    block GEMM to bf16, add bias in bf16."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    xq, xs = per_token_group_quant_fp8(x.reshape(-1, x.shape[-1]), block)
    out = w8a8_block_fp8_matmul(xq, w_codes, xs, w_s, block, block)
    if bias_f32 is not None:
        out = bf16_round((out + bias_f32).astype(np.float32))
    return out.reshape(x.shape[:-1] + (w_codes.shape[0],))


# ----------------------------------------------------------------------------
# Routing used by the MoE configs (input generators; not on the graded path)
# ----------------------------------------------------------------------------


def grouped_sigmoid_topk(logits_f32, topk=8, n_group=8, topk_group=4, renormalize=True):
    """DeepSeek-V3 routing with a zero correction bias: sigmoid scores, group
    score = sum of the group's top-2, keep `topk_group` groups, take top-k
    experts, weights = sigmoid scores renormalised.  Follows
    python/sglang/srt/layers/moe/topk.py:665-738 (`biased_grouped_topk_impl`)."""
    s = 1.0 / (1.0 + np.exp(-logits_f32.astype(np.float64)))
    T, E = s.shape
    g = s.reshape(T, n_group, E // n_group)
    gs = np.sort(g, axis=-1)[..., -2:].sum(-1)
    keep = np.argsort(-gs, axis=-1, kind="stable")[:, :topk_group]
    mask = np.zeros((T, n_group), dtype=bool)
    np.put_along_axis(mask, keep, True, axis=1)
    masked = np.where(np.repeat(mask, E // n_group, axis=1), s, -np.inf)
    ids = np.argsort(-masked, axis=-1, kind="stable")[:, :topk]
    w = np.take_along_axis(s, ids, axis=1)
    if renormalize:
        w = w / w.sum(-1, keepdims=True)
    return w.astype(np.float32), ids.astype(np.int32)


def softmax_topk(logits_f32, topk=8, renormalize=True):
    """softmax -> top-k -> renormalise (python/sglang/srt/layers/moe/topk.py:427-456)."""
    z = logits_f32.astype(np.float64)
    z = z - z.max(-1, keepdims=True)
    p = np.exp(z)
    p /= p.sum(-1, keepdims=True)
    ids = np.argsort(-p, axis=-1, kind="stable")[:, :topk]
    w = np.take_along_axis(p, ids, axis=1)
    if renormalize:
        w = w / w.sum(-1, keepdims=True)
    return w.astype(np.float32), ids.astype(np.int32)


def _round_to(v_f32, dtype):
    """float32 values rounded to the arithmetic type of the gate ("f32", "bf16", "f16")."""
    if dtype == "f32":
        return v_f32.astype(np.float32)
    if dtype == "bf16":
        return bf16_round(v_f32.astype(np.float32))
    return v_f32.astype(np.float16).astype(np.float32)


def _topk_desc(sel, k):
    """Indices of the k largest entries per row, best first, lower index first on equal values."""
    return np.argsort(-sel, axis=-1, kind="stable")[:, :k]


def moe_fused_gate(x_f32, bias_f32, num_expert_group, topk_group, topk, num_fused_shared_experts=0,
                   routed_scaling_factor=0.0, apply_routed_scaling_factor_on_output=False, dtype="f32"):
    """DeepSeek-V3 grouped gate as the reference's kernel computes it (sgl-kernel/csrc/moe/moe_fused_gate.cu:52-260;
    torch form python/sglang/srt/layers/moe/topk.py:665-738): every score is held in the input type `dtype`.
    `x_f32` / `bias_f32` hold values already representable in that type.  Picks come out best first."""
    x = x_f32.astype(np.float32)
    s = _round_to(np.float32(1.0) / (np.float32(1.0) + np.exp(-x)), dtype)
    b = _round_to(s + bias_f32.astype(np.float32)[None, :], dtype)
    T, E = b.shape
    gs = E // num_expert_group
    top2 = -np.sort(-b.reshape(T, num_expert_group, gs), axis=-1)[..., :2]
    gscore = _round_to(top2[..., 0] + top2[..., 1], dtype)
    keep = _topk_desc(gscore, topk_group)
    mask = np.zeros((T, num_expert_group), dtype=bool)
    np.put_along_axis(mask, keep, True, axis=1)
    sel = np.where(np.repeat(mask, gs, axis=1), b, -np.inf)
    k_routed = topk - num_fused_shared_experts
    ids = _topk_desc(sel, k_routed)
    w = np.take_along_axis(s, ids, axis=1).astype(np.float32)
    total = np.zeros(T, dtype=np.float32)
    for j in range(k_routed):  # the kernel adds the picks in order, in float32
        total = (total + w[:, j]).astype(np.float32)
    if num_fused_shared_experts:
        shared_w = (total / np.float32(routed_scaling_factor)).astype(np.float32)
        w = np.concatenate([w, np.repeat(shared_w[:, None], num_fused_shared_experts, axis=1)], axis=1)
        shared_ids = np.broadcast_to(E + np.arange(num_fused_shared_experts), (T, num_fused_shared_experts))
        ids = np.concatenate([ids, shared_ids], axis=1)
    w = (w / total[:, None]).astype(np.float32)
    if apply_routed_scaling_factor_on_output:
        w = (w * np.float32(routed_scaling_factor)).astype(np.float32)
    return w, ids.astype(np.int32)


def topk_softmax(x_f32, topk, renormalize=False, moe_softcapping=0.0, correction_bias=None):
    """sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:75-215: optional tanh cap, optional bias added to the
    logits, float32 softmax, picks best first (lower index on ties), weights = probabilities."""
    v = x_f32.astype(np.float32)
    if moe_softcapping != 0.0:
        v = (np.tanh(v / np.float32(moe_softcapping)) * np.float32(moe_softcapping)).astype(np.float32)
    if correction_bias is not None:
        v = (v + correction_bias.astype(np.float32)[None, :]).astype(np.float32)
    p = np.exp(v - v.max(-1, keepdims=True)).astype(np.float32)
    p = (p * (np.float32(1.0) / p.sum(-1, keepdims=True, dtype=np.float32))).astype(np.float32)
    ids = _topk_desc(p, topk)
    w = np.take_along_axis(p, ids, axis=1)
    if renormalize:
        w = (w * (np.float32(1.0) / w.sum(-1, keepdims=True, dtype=np.float32))).astype(np.float32)
    return w.astype(np.float32), ids.astype(np.int32)


def topk_sigmoid(x_f32, topk, renormalize=False, correction_bias=None):
    """sgl-kernel/csrc/moe/moe_topk_sigmoid_kernels.cu:75-170: c = sigmoid(x) + bias selects; the reported weight
    is c - bias (float32, so not always the sigmoid bit for bit)."""
    x = x_f32.astype(np.float32)
    c = (np.float32(1.0) / (np.float32(1.0) + np.exp(-x))).astype(np.float32)
    if correction_bias is not None:
        c = (c + correction_bias.astype(np.float32)[None, :]).astype(np.float32)
    ids = _topk_desc(c, topk)
    w = np.take_along_axis(c, ids, axis=1)
    if correction_bias is not None:
        w = (w - correction_bias.astype(np.float32)[ids]).astype(np.float32)
    if renormalize:
        w = (w * (np.float32(1.0) / w.sum(-1, keepdims=True, dtype=np.float32))).astype(np.float32)
    return w.astype(np.float32), ids.astype(np.int32)
