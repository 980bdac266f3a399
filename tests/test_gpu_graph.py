"""The hot path inside CUDA graphs: every entry point only enqueues work on the stream it is given (no
synchronisation, no host round trip), so quantise -> GEMM and the whole MoE layer can be captured and replayed,
which is how the reference's model runner executes decode steps (cuda_graph_runner.py)."""
import numpy as np
import pytest
import torch

from oracle import block_fp8_oracle as O
from tests.util import assert_close_fp, codes_to_fp8, make_act, make_weight, to_f32_np

pytestmark = pytest.mark.gpu


def test_linear_captured_and_replayed_with_new_inputs():
    from sglang_b200 import ops
    M, N, K = 48, 1536, 2048          # small M: the split-K form with its workspace and second kernel
    wq, ws = make_weight(N, K, 3)
    w, s = codes_to_fp8(wq), torch.from_numpy(ws).cuda()
    x_static = make_act(M, K, 4).cuda()

    def step():
        xq, xs = ops.per_token_group_quant_fp8(x_static, 128)
        return ops.w8a8_block_fp8_matmul(xq, w, xs, s, [128, 128], torch.bfloat16)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y_static = step()
    for seed in (11, 12):
        x = make_act(M, K, seed)
        x_static.copy_(x.cuda())
        g.replay()
        torch.cuda.synchronize()
        assert_close_fp(to_f32_np(y_static), O.block_fp8_linear(to_f32_np(x), wq, ws))
    assert ops.gemm_status() == 0


def test_moe_layer_captured_and_replayed():
    from sglang_b200 import ops
    from sglang_b200.srt.layers.moe.fused_moe_triton.fused_moe import fused_experts_impl
    T, E, H, I, topk = 32, 16, 512, 256, 4
    w13q, w13s = make_weight(2 * I, H, 5, std=0.05, experts=E)
    w2q, w2s = make_weight(H, I, 6, std=0.05, experts=E)
    w13, w2 = codes_to_fp8(w13q), codes_to_fp8(w2q)
    s13, s2 = torch.from_numpy(w13s).cuda(), torch.from_numpy(w2s).cuda()
    x_static = make_act(T, H, 7).cuda()
    logits_static = torch.randn(T, E, generator=torch.Generator().manual_seed(8)).cuda()

    def step():
        w = torch.empty(T, topk, device="cuda")
        ids = torch.empty(T, topk, dtype=torch.int32, device="cuda")
        ops.topk_softmax_out(w, ids, logits_static, True)
        return fused_experts_impl(x_static, w13, w2, w, ids, use_fp8_w8a8=True, w1_scale=s13, w2_scale=s2,
                                  block_shape=[128, 128]), w, ids

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out_static, w_static, ids_static = step()
    for seed in (21, 22):
        x = make_act(T, H, seed)
        logits = torch.randn(T, E, generator=torch.Generator().manual_seed(seed))
        x_static.copy_(x.cuda())
        logits_static.copy_(logits.cuda())
        g.replay()
        torch.cuda.synchronize()
        rw, rids = O.topk_softmax(logits.numpy(), topk, True)
        assert np.array_equal(ids_static.cpu().numpy(), rids)
        ref = O.fused_experts_block_fp8(to_f32_np(x), w13q, w13s, w2q, w2s, w_static.cpu().numpy(), rids, 1.0)
        assert_close_fp(to_f32_np(out_static), ref, atol=2e-2)
    assert ops.gemm_status() == 0
