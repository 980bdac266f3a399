"""GPU parity of the block-scaled GEMM (dense and grouped) and of the MoE layer, through the C ABI.

Tolerance (from the path's specification): rtol 1e-2, atol 1e-2 and cosine >= 0.9999 against the
dequantised float32 reference computed by the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import block_fp8_oracle as O
from tests.util import assert_close_fp, bf16_bits, codes_to_fp8, cosine, fp8_codes, make_act, make_weight, to_f32_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from sglang_b200 import ops as _ops
    return _ops


def _dense_case(ops, M, N, K, seed=0, out_dtype=torch.bfloat16):
    x = make_act(M, K, seed, outliers=False)
    wq, ws = make_weight(N, K, seed + 1)
    xq, xs = O.per_token_group_quant_fp8(to_f32_np(x))
    ref = O.w8a8_block_fp8_matmul(xq, wq, xs, ws, out_bf16=(out_dtype == torch.bfloat16))
    c = ops.w8a8_block_fp8_matmul(codes_to_fp8(xq), codes_to_fp8(wq), torch.from_numpy(xs).cuda(),
                                  torch.from_numpy(ws).cuda(), [128, 128], out_dtype)
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    return to_f32_np(c), ref


@pytest.mark.parametrize("M", [1, 3, 5, 127, 128, 129, 300])
@pytest.mark.parametrize("N,K", [(128, 128), (256, 512), (320, 512), (2112, 1024), (1024, 7168)])
def test_dense_gemm_matches_oracle(ops, M, N, K):
    got, ref = _dense_case(ops, M, N, K, seed=M + N + K)
    assert_close_fp(got, ref)


def test_dense_gemm_many_tiles_and_fp16(ops):
    got, ref = _dense_case(ops, 1000, 4096, 2048, seed=11)
    assert_close_fp(got, ref)
    got, ref = _dense_case(ops, 200, 512, 1536, seed=12, out_dtype=torch.float16)
    assert_close_fp(got, ref)


def test_dense_gemm_golden_and_known_answer(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "gemm_native.npz"))
    c = ops.w8a8_block_fp8_matmul(codes_to_fp8(g["xq"]), codes_to_fp8(g["wq"]), torch.from_numpy(g["xs"]).cuda(),
                                  torch.from_numpy(g["ws"]).cuda(), [128, 128], torch.bfloat16)
    assert_close_fp(to_f32_np(c), O.bf16_bits_to_f32(g["c"]))
    k = np.load(os.path.join(golden_dir, "kat_fp8_kernel.npz"))
    c = ops.w8a8_block_fp8_matmul(codes_to_fp8(k["A_q"]), codes_to_fp8(k["B_q_t"]), torch.from_numpy(k["A_s"]).cuda(),
                                  torch.from_numpy(k["B_s_t"]).cuda(), [128, 128], torch.bfloat16)
    np.testing.assert_allclose(to_f32_np(c), O.bf16_bits_to_f32(k["C_gt"]), atol=0.5, rtol=1e-4)


def test_dense_gemm_column_major_scales_and_bias(ops):
    M, N, K = 70, 384, 1024
    x = make_act(M, K, 21).cuda()
    wq, ws = make_weight(N, K, 22)
    xq, xs_cm = ops.per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True)
    xq2, xs_rm = ops.per_token_group_quant_fp8(x, 128)
    bias = torch.randn(N, dtype=torch.bfloat16, device="cuda")
    w_t, ws_t = codes_to_fp8(wq), torch.from_numpy(ws).cuda()
    c1 = ops.w8a8_block_fp8_matmul(xq, w_t, xs_cm, ws_t, [128, 128], torch.bfloat16)
    c2 = ops.w8a8_block_fp8_matmul(xq2, w_t, xs_rm, ws_t, [128, 128], torch.bfloat16)
    assert torch.equal(c1, c2)
    c3 = ops.w8a8_block_fp8_matmul(xq2, w_t, xs_rm, ws_t, [128, 128], torch.bfloat16, bias=bias)
    ref = O.block_fp8_linear(to_f32_np(x), wq, ws, to_f32_np(bias))
    assert_close_fp(to_f32_np(c3), ref, atol=2e-2)


def test_dense_gemm_linearity_at_full_size(ops):
    # DeepSeek-V3 gate_up shape at M=4096: C(2*a_s) == 2*C(a_s) exactly (power-of-two scaling commutes with
    # every rounding), and a sampled set of rows matches the oracle
    M, N, K = 4096, 36864, 7168
    g = torch.Generator(device="cuda").manual_seed(0)
    xq = torch.randint(0, 0x7E, (M, K), device="cuda", dtype=torch.uint8, generator=g).view(torch.float8_e4m3fn)
    wq = torch.randint(0, 0x7E, (N, K), device="cuda", dtype=torch.uint8, generator=g)
    wq = (wq | (torch.randint(0, 2, (N, K), device="cuda", dtype=torch.uint8, generator=g) << 7)).view(torch.float8_e4m3fn)
    xs = torch.rand(M, K // 128, device="cuda", generator=g) * 1e-3 + 1e-4
    ws = torch.rand(N // 128, K // 128, device="cuda", generator=g) * 1e-3 + 1e-4
    c1 = ops.w8a8_block_fp8_matmul(xq, wq, xs, ws, [128, 128], torch.bfloat16)
    c2 = ops.w8a8_block_fp8_matmul(xq, wq, xs * 2, ws, [128, 128], torch.bfloat16)
    assert torch.equal(c1.float() * 2, c2.float())
    rows = [0, 1, 127, 128, 2049, 4095]
    ref = O.w8a8_block_fp8_matmul(fp8_codes(xq[rows]), fp8_codes(wq[:1024]), xs[rows].cpu().numpy(),
                                  ws[:8].cpu().numpy())
    assert_close_fp(to_f32_np(c1[rows][:, :1024]), ref, atol=1e-2 * float(np.abs(ref).max()))
    assert ops.gemm_status() == 0


def _moe_inputs(T, E, H, I, topk, seed, filtered=False):
    g = torch.Generator().manual_seed(seed)
    x = make_act(T, H, seed, outliers=False)
    w13q, w13s = make_weight(2 * I, H, seed + 1, std=0.05, experts=E)
    w2q, w2s = make_weight(H, I, seed + 2, std=0.05, experts=E)
    logits = torch.randn(T, E, generator=g)
    w, ids = torch.topk(torch.softmax(logits, -1), topk)
    w = (w / w.sum(-1, keepdim=True)).float()
    ids = ids.to(torch.int32)
    if filtered:
        ids = torch.where(ids >= E // 2, torch.full_like(ids, -1), ids)
    return x, w13q, w13s, w2q, w2s, w, ids


@pytest.mark.parametrize("T,E,H,I,topk,filtered", [
    (9, 4, 256, 128, 2, False), (1, 8, 512, 256, 4, False), (64, 16, 1024, 256, 8, False),
    (300, 8, 512, 384, 2, True), (130, 32, 2048, 768, 8, True),
])
def test_fused_experts_matches_oracle(ops, T, E, H, I, topk, filtered):
    from sglang_b200.srt.layers.moe.fused_moe_triton.fused_moe import fused_experts_impl
    x, w13q, w13s, w2q, w2s, w, ids = _moe_inputs(T, E, H, I, topk, seed=T + E, filtered=filtered)
    ref = O.fused_experts_block_fp8(to_f32_np(x), w13q, w13s, w2q, w2s, w.numpy(), ids.numpy(), 1.0)
    out = fused_experts_impl(
        x.cuda(), codes_to_fp8(w13q), codes_to_fp8(w2q), w.cuda(), ids.cuda(), use_fp8_w8a8=True,
        w1_scale=torch.from_numpy(w13s).cuda(), w2_scale=torch.from_numpy(w2s).cuda(), block_shape=[128, 128])
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    # intermediate fp8 codes may differ by one code where silu's expf differs by an ulp: same tolerance
    assert_close_fp(to_f32_np(out), ref, atol=2e-2)
    # the expert-parallel form, which drops the rows of filtered (-1) ids instead of carrying them as zeros, must
    # give the very same bits (also when there is nothing to drop)
    out2 = fused_experts_impl(
        x.cuda(), codes_to_fp8(w13q), codes_to_fp8(w2q), w.cuda(), ids.cuda(), use_fp8_w8a8=True,
        w1_scale=torch.from_numpy(w13s).cuda(), w2_scale=torch.from_numpy(w2s).cuda(), block_shape=[128, 128],
        has_filtered_ids=True)
    assert torch.equal(out, out2)


def test_fused_experts_all_ids_filtered(ops):
    from sglang_b200.srt.layers.moe.fused_moe_triton.fused_moe import fused_experts_impl
    x, w13q, w13s, w2q, w2s, w, ids = _moe_inputs(40, 8, 512, 256, 4, seed=5)
    ids = torch.full_like(ids, -1)
    out = fused_experts_impl(
        x.cuda(), codes_to_fp8(w13q), codes_to_fp8(w2q), w.cuda(), ids.cuda(), use_fp8_w8a8=True,
        w1_scale=torch.from_numpy(w13s).cuda(), w2_scale=torch.from_numpy(w2s).cuda(), block_shape=[128, 128],
        has_filtered_ids=True)
    assert out.shape == (40, 512) and not out.float().abs().any()


def test_moe_golden_fixture(ops, golden_dir):
    from sglang_b200.srt.layers.moe.fused_moe_triton.fused_moe import fused_experts_impl
    g = np.load(os.path.join(golden_dir, "moe_native.npz"))
    x = torch.from_numpy(g["a"].view(np.int16)).view(torch.bfloat16).cuda()
    out = fused_experts_impl(
        x, codes_to_fp8(g["w1q"]), codes_to_fp8(g["w2q"]), torch.from_numpy(g["topk_w"]).cuda(),
        torch.from_numpy(g["topk_ids"]).cuda(), use_fp8_w8a8=True, w1_scale=torch.from_numpy(g["w1s"]).cuda(),
        w2_scale=torch.from_numpy(g["w2s"]).cuda(), block_shape=[128, 128])
    ref = O.bf16_bits_to_f32(g["out"])
    assert_close_fp(to_f32_np(out), ref, rtol=2e-2, atol=2e-2)


def test_quant_method_surface(ops):
    """Fp8LinearMethod.apply / Fp8MoEMethod.apply through the layer classes, single rank."""
    from sglang_b200.srt.layers.linear import RowParallelLinear
    from sglang_b200.srt.layers.moe.fused_moe_triton.layer import FusedMoE
    from sglang_b200.srt.layers.moe.token_dispatcher import StandardTopKOutput
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
    cfg = Fp8Config(weight_block_size=[128, 128])
    lin = RowParallelLinear(1024, 384, quant_config=cfg, device="cuda")
    wq, ws = make_weight(384, 1024, 5)
    lin.load_full_weight(codes_to_fp8(wq), torch.from_numpy(ws).cuda())
    x = make_act(33, 1024, 6)
    y, _ = lin(x.cuda())
    assert_close_fp(to_f32_np(y), O.block_fp8_linear(to_f32_np(x), wq, ws))
    # pre-quantised tuple input (fp8.py:500-508)
    xq, xs = ops.per_token_group_quant_fp8(x.cuda(), 128)
    y2 = lin.quant_method.apply(lin, (xq, xs))
    assert torch.equal(y, y2)
    T, E, H, I, topk = 40, 8, 512, 256, 2
    x, w13q, w13s, w2q, w2s, w, ids = _moe_inputs(T, E, H, I, topk, seed=3)
    moe = FusedMoE(E, H, I, topk, quant_config=cfg, routed_scaling_factor=2.5, device="cuda")
    moe.load_full_weights(codes_to_fp8(w13q), torch.from_numpy(w13s).cuda(), codes_to_fp8(w2q), torch.from_numpy(w2s).cuda())
    out = moe(x.cuda(), StandardTopKOutput(w.cuda(), ids.cuda(), None))
    ref = O.fused_experts_block_fp8(to_f32_np(x), w13q, w13s, w2q, w2s, w.numpy(), ids.numpy(), 2.5)
    assert_close_fp(to_f32_np(out), ref, atol=5e-2)


def test_sgl_kernel_gemm_op_surface(ops):
    import sglang_b200.sgl_kernel as sk
    M, N, K = 65, 256, 512
    x = make_act(M, K, 31).cuda()
    wq, ws = make_weight(N, K, 32)
    xq = torch.empty(M, K, device="cuda", dtype=torch.float8_e4m3fn)
    xs = torch.empty(K // 128, M, device="cuda", dtype=torch.float32).t()  # M-major, as the CUTLASS op takes it
    sk.sgl_per_token_group_quant_fp8(x, xq, xs, 128, 1e-10, -448.0, 448.0)
    w = codes_to_fp8(wq)
    c = sk.fp8_blockwise_scaled_mm(xq, w.t(), xs, torch.from_numpy(ws).cuda().t(), torch.bfloat16)
    assert_close_fp(to_f32_np(c), O.block_fp8_linear(to_f32_np(x), wq, ws))


def test_cutlass_moe_path_ops(ops):
    """The op sequence of the reference's CUTLASS MoE runner (python/sglang/srt/layers/moe/cutlass_moe.py:125-260:
    prepare_moe_input -> quantise -> shuffle_rows -> grouped GEMM -> silu_and_mul -> quantise -> grouped GEMM ->
    apply_shuffle_mul_sum), with the tensor layouts fp8.py:1071-1104 passes, against the fused-experts oracle."""
    import sglang_b200.sgl_kernel as sk
    T, E, H, I, topk = 70, 8, 512, 256, 4
    x, w13q, w13s, w2q, w2s, w, ids = _moe_inputs(T, E, H, I, topk, seed=31, filtered=False)
    dev = "cuda"
    a = x.cuda()
    w1 = codes_to_fp8(w13q).transpose(1, 2)            # [E, k, 2n] view
    w2 = codes_to_fp8(w2q).transpose(1, 2)             # [E, n, k] view
    w1_s = torch.from_numpy(w13s).cuda().transpose(1, 2)
    w2_s = torch.from_numpy(w2s).cuda().transpose(1, 2)
    topk_ids, topk_w = ids.cuda(), w.cuda()
    m, k, n = T, H, I
    i32 = dict(dtype=torch.int32, device=dev)
    expert_offsets = torch.empty(E + 1, **i32)
    ps1, ps2 = torch.empty(E, 3, **i32), torch.empty(E, 3, **i32)
    a_map, c_map = torch.empty(m * topk, **i32), torch.empty(m * topk, **i32)
    sk.prepare_moe_input(topk_ids, expert_offsets, ps1, ps2, a_map, c_map, E, n, k)
    counts = np.bincount(ids.numpy().reshape(-1), minlength=E)
    assert expert_offsets.cpu().tolist() == [0] + np.cumsum(counts).tolist()
    assert ps1.cpu().tolist() == [[int(c), 2 * n, k] for c in counts] and ps2.cpu().tolist() == [[int(c), k, n] for c in counts]
    flat = ids.numpy().reshape(-1)
    assert np.array_equal(flat[c_map.cpu().numpy().argsort()], np.sort(flat))          # expert-major order
    assert np.array_equal(a_map.cpu().numpy()[c_map.cpu().numpy()], np.arange(m * topk) // topk)
    a_q, a1_scale = ops.per_token_group_quant_fp8(a, 128)
    rep_a_q = sk.shuffle_rows(a_q, a_map, (m * topk, k))
    rep_a1_s = sk.shuffle_rows(a1_scale, a_map, (m * topk, k // 128))
    c1 = torch.empty(m * topk, 2 * n, device=dev, dtype=torch.bfloat16)
    c2 = torch.empty(m * topk, k, device=dev, dtype=torch.bfloat16)
    scratch = torch.empty(E, dtype=torch.int64, device=dev)
    lay = torch.empty(E, 5, **i32)
    sk.fp8_blockwise_scaled_grouped_mm(c1, scratch, scratch, scratch, scratch, scratch, rep_a_q, w1, rep_a1_s, w1_s,
                                       scratch, scratch, scratch, lay, lay, ps1, expert_offsets[:-1], scratch)
    inter = torch.empty(m * topk, n, device=dev, dtype=torch.bfloat16)
    sk.silu_and_mul(c1, inter)
    inter_q, a2_scale = ops.per_token_group_quant_fp8(inter, 128)
    sk.fp8_blockwise_scaled_grouped_mm(c2, scratch, scratch, scratch, scratch, scratch, inter_q, w2, a2_scale, w2_s,
                                       scratch, scratch, scratch, lay, lay, ps2, expert_offsets[:-1], scratch)
    out = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
    sk.apply_shuffle_mul_sum(c2, out, c_map, topk_w.to(torch.bfloat16))
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    # the CUTLASS path rounds the routing weights to bf16 and applies them after the bf16 rounding of GEMM 2
    ref = O.fused_experts_block_fp8(to_f32_np(x), w13q, w13s, w2q, w2s,
                                    w.to(torch.bfloat16).float().numpy(), ids.numpy(), 1.0)
    assert_close_fp(to_f32_np(out), ref, rtol=3e-2, atol=3e-2)
