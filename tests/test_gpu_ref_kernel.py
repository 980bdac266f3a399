"""This library's block GEMM against the reference's own CUDA kernel on the same device buffers.

`oracle/_ref/libsgl_gpu_ref.so` is sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu compiled unmodified for
sm_100a (oracle/Makefile, target `ref_gpu`).  Both kernels form the same float32 partial sums per 128-wide K slab
and add them in the same order, so wherever this library does not split K the outputs must agree bit for bit;
with split-K (few output tiles, long K) the float32 summation order differs and the bf16 results may differ by
one rounding.  The reference kernel wants N to be a multiple of 128 and M-major activation scales.
"""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libsgl_gpu_ref.so")


@pytest.fixture(scope="module")
def ref_mm():
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libsgl_gpu_ref.so not built (make -C oracle ref_gpu)")
    torch.ops.load_library(LIB)
    return torch.ops.sgl_gpu_ref.fp8_blockwise_scaled_mm


def _inputs(M, N, K, seed):
    from sglang_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    x[torch.rand(M, K, device="cuda", generator=g) < 0.001] *= 10
    xq, xs = ops.per_token_group_quant_fp8(x, 128)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    blk = w.view(N // 128, 128, K // 128, 128)
    ws = blk.abs().amax(dim=(1, 3)) / 448.0
    wq = (blk / ws[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(N, K).contiguous()
    return xq, xs, wq, ws.contiguous()


# (700 and 520 rows end in a partial 128-row block, of 60 and 8 rows; 130 and 513 rows in one of 2 and 1)
@pytest.mark.parametrize("M,N,K", [(4096, 7168, 2048), (2048, 4608, 7168), (513, 1536, 1536), (130, 24576, 1536),
                                   (1024, 7168, 18432), (4, 512, 512), (128, 256, 128), (700, 1536, 2048),
                                   (520, 768, 2048), (8192, 1280, 3584)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_bitwise_equal_to_reference_kernel(ref_mm, M, N, K, out_dtype):
    from sglang_b200 import ops
    xq, xs, wq, ws = _inputs(M, N, K, M + N + K)
    from sglang_b200._lib import lib
    mine = ops.w8a8_block_fp8_matmul(xq, wq, xs, ws, [128, 128], out_dtype)
    ref = ref_mm(xq, wq.t(), xs.t().contiguous().t(), ws.t(), out_dtype)
    torch.cuda.synchronize()
    if lib.sglb200_gemm_workspace_bytes(M, N, K) == 0:
        assert torch.equal(mine.view(torch.int16), ref.view(torch.int16))
    else:
        # the tiles of the last wave are split along K: same partial sums, added in another order
        differ = (mine.view(torch.int16) != ref.view(torch.int16)).float().mean().item()
        assert differ < 0.05
        assert torch.allclose(mine.float(), ref.float(), rtol=2 ** -7, atol=2e-3)


@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (16, 7168, 16384), (1, 7168, 18432)])
def test_split_k_regime_against_reference_kernel(ref_mm, M, N, K):
    from sglang_b200 import ops
    xq, xs, wq, ws = _inputs(M, N, K, M + N + K)
    mine = ops.w8a8_block_fp8_matmul(xq, wq, xs, ws, [128, 128], torch.bfloat16).float()
    ref = ref_mm(xq, wq.t(), xs.t().contiguous().t(), ws.t(), torch.bfloat16).float()
    torch.cuda.synchronize()
    # one bf16 rounding apart at most: 2^-8 relative, plus a little absolute slack near zero
    assert torch.allclose(mine, ref, rtol=2 ** -7, atol=2e-3)
    assert torch.nn.functional.cosine_similarity(mine.flatten(), ref.flatten(), dim=0).item() > 0.99999


def test_op_surface_matches_reference_call(ref_mm):
    """The same positional call through torch.ops.sgl_kernel (this library) and the reference's op."""
    import sglang_b200.sgl_kernel  # noqa: F401  (registers torch.ops.sgl_kernel.*)
    xq, xs, wq, ws = _inputs(256, 1024, 1024, 5)
    a_s = xs.t().contiguous().t()
    mine = torch.ops.sgl_kernel.fp8_blockwise_scaled_mm.default(xq, wq.t(), a_s, ws.t(), torch.bfloat16)
    ref = ref_mm(xq, wq.t(), a_s, ws.t(), torch.bfloat16)
    assert torch.equal(mine.view(torch.int16), ref.view(torch.int16))


# ------------------------------------------------------------------------------------------------------------------
# the expert-grouped kernel
# ------------------------------------------------------------------------------------------------------------------
LIB_MOE = os.path.join(os.path.dirname(LIB), "libsgl_gpu_ref_moe.so")


@pytest.fixture(scope="module")
def ref_grouped():
    """sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu compiled with its one-CTA tile configurations (oracle/Makefile,
    target `ref_gpu_moe`): more than 2048 rows with K >= 2048 run its 128x128x128 tiles, K < 2048 its 64x128x128
    tiles; at most 2048 rows with K >= 2048 would take the two-CTA cluster configuration, which is not built."""
    if not os.path.exists(LIB_MOE):
        pytest.skip("oracle/_ref/libsgl_gpu_ref_moe.so not built (make -C oracle ref_gpu_moe)")
    torch.ops.load_library(LIB_MOE)
    return torch.ops.sgl_gpu_ref.fp8_blockwise_scaled_grouped_mm


@pytest.mark.parametrize("E,R,N,K", [(8, 2600, 512, 2048), (16, 4096, 1024, 768), (8, 300, 256, 512),
                                     (32, 6000, 1536, 2048), (4, 2100, 4096, 7168)])
def test_grouped_bitwise_equal_to_reference_kernel(ref_grouped, E, R, N, K):
    """Same arguments to both (the call of python/sglang/srt/layers/moe/cutlass_moe.py:179-198): per expert the rows
    off_e .. off_e + M_e of `a` times that expert's [N, K] weights.  Neither kernel splits K, both add the per-slab
    float32 partial products in ascending K order, so the outputs must agree bit for bit."""
    import sglang_b200.sgl_kernel as sk
    from sglang_b200 import ops
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(E * 1000 + R)
    cuts = torch.sort(torch.randperm(R - 1, device=dev, generator=g)[: E - 1] + 1).values
    offs = torch.cat([torch.zeros(1, device=dev, dtype=torch.int64), cuts, torch.tensor([R], device=dev)]).to(torch.int32)
    counts = (offs[1:] - offs[:-1]).to(torch.int32)
    assert int(counts.min()) >= 1 and int(counts.sum()) == R
    x = torch.randn(R, K, device=dev, generator=g).bfloat16()
    aq, a_s = ops.per_token_group_quant_fp8(x, 128)
    w = torch.randn(E, N, K, device=dev, generator=g) * 0.02
    blk = w.view(E, N // 128, 128, K // 128, 128)
    ws = (blk.abs().amax(dim=(2, 4)) / 448.0).contiguous()
    wq = (blk / ws[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(E, N, K).contiguous()
    ps = torch.stack([counts, torch.full_like(counts, N), torch.full_like(counts, K)], dim=1).contiguous()
    i64 = dict(dtype=torch.int64, device=dev)
    ptrs = [torch.empty(E, **i64) for _ in range(5)]
    ab, cs = torch.full((E,), K, **i64), torch.full((E,), N, **i64)
    lay_a, lay_b = (torch.empty(E, 5, dtype=torch.int32, device=dev) for _ in range(2))
    # (the reference's 90 000 bytes, fp8.py:1196, fit the CUTLASS it pins; the CUTLASS this comparator is built with
    # keeps about 0.3 MB of tensor-map copies per grouped launch and does not check the size it is given)
    work = torch.empty(4 << 20, device=dev, dtype=torch.uint8)
    out_ref = torch.zeros(R, N, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(R, N, device=dev, dtype=torch.bfloat16)
    args = (*ptrs, aq, wq.transpose(1, 2), a_s, ws.transpose(1, 2), ab, ab, cs, lay_a, lay_b, ps, offs[:-1].contiguous(), work)
    ref_grouped(out_ref, *args)
    sk.fp8_blockwise_scaled_grouped_mm(out, *args)
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    assert torch.allclose(out.float(), out_ref.float(), rtol=2 ** -7, atol=2e-3)
    differ = (out.view(torch.int16) != out_ref.view(torch.int16)).float().mean().item()
    assert differ == 0.0, f"{differ:.2e} of the outputs differ in their bf16 bits"


# ------------------------------------------------------------------------------------------------------------------
# the reference's CUDA quantizer and moe_align kernel
# ------------------------------------------------------------------------------------------------------------------
LIB_AUX = os.path.join(os.path.dirname(LIB), "libsgl_gpu_ref_aux.so")


@pytest.fixture(scope="module")
def ref_aux():
    """sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu and sgl-kernel/csrc/moe/moe_align_kernel.cu compiled
    unmodified (oracle/Makefile, target `ref_gpu_aux`; without the reference build's fast-math flag, so its
    `val / y_s` is an IEEE division like the torch-native form the oracle restates)."""
    if not os.path.exists(LIB_AUX):
        pytest.skip("oracle/_ref/libsgl_gpu_ref_aux.so not built (make -C oracle ref_gpu_aux)")
    torch.ops.load_library(LIB_AUX)
    return torch.ops.sgl_gpu_ref


@pytest.mark.parametrize("tokens,hidden,dtype", [(83, 7168, torch.bfloat16), (2048, 4096, torch.bfloat16),
                                                 (7, 512, torch.float16), (300, 2048, torch.float32),
                                                 (4096, 7168, torch.bfloat16)])
def test_quantizer_bitwise_equal_to_reference_kernel(ref_aux, tokens, hidden, dtype):
    """The division form (`y_s = absmax / 448`, `q = clamp(x / y_s)`, per_token_group_quant_8bit.cu:86-111): codes and
    scales must agree bit for bit."""
    from sglang_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(tokens + hidden)
    x = torch.randn(tokens, hidden, device="cuda", generator=g)
    x[torch.rand(tokens, hidden, device="cuda", generator=g) < 0.001] *= 30
    x[0, :128] = 0                                   # a group below eps
    x = x.to(dtype)
    q_ref = torch.empty(tokens, hidden, device="cuda", dtype=torch.float8_e4m3fn)
    s_ref = torch.empty(tokens, hidden // 128, device="cuda", dtype=torch.float32)
    ref_aux.sgl_per_token_group_quant_8bit(x, q_ref, s_ref, 128, 1e-10, -448.0, 448.0, False)
    q, s = ops.per_token_group_quant_fp8(x, 128)
    torch.cuda.synchronize()
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))


@pytest.mark.parametrize("T,topk,E,filtered", [(1, 8, 256, False), (64, 8, 256, False), (4096, 8, 256, False),
                                                (16384, 8, 128, False), (300, 2, 8, True), (4096, 8, 32, True)])
def test_moe_align_agrees_with_reference_kernel(ref_aux, T, topk, E, filtered):
    """Same padded total, same expert of every block, and the same set of flat indices in every expert's segment (the
    reference kernel orders a segment by atomics, this library by ascending flat index)."""
    from sglang_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(T * 31 + E)
    ids = torch.randint(0, E, (T, topk), device="cuda", generator=g, dtype=torch.int32)
    if filtered:
        ids[torch.rand(T, topk, device="cuda", generator=g) < 0.15] = -1
    block, numel = 128, T * topk
    mine_sorted, mine_experts, mine_post = ops.moe_align_block_size(ids, block, E)
    max_padded = numel + (E + 1) * (block - 1)
    i32 = dict(dtype=torch.int32, device="cuda")
    ref_sorted = torch.empty(max_padded, **i32)
    ref_experts = torch.empty((max_padded + block - 1) // block, **i32)
    ref_post, cumsum = torch.empty(1, **i32), torch.empty(E + 2, **i32)
    ref_aux.moe_align_block_size(ids, E + 1, block, ref_sorted, ref_experts, ref_post, cumsum, True)
    torch.cuda.synchronize()
    n = int(ref_post.item())
    assert int(mine_post.item()) == n and n % block == 0
    assert torch.equal(mine_experts[: n // block], ref_experts[: n // block])

    def keys(sorted_ids, experts):
        e = experts[: n // block].long().repeat_interleave(block) + 1
        return torch.sort(e * (numel + 1) + sorted_ids[:n].long()).values

    assert torch.equal(keys(mine_sorted, mine_experts), keys(ref_sorted, ref_experts))
