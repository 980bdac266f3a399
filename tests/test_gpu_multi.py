"""Two-GPU parity of the tensor-parallel linears and the expert-parallel MoE layer (NCCL).
Skipped on boxes with a single GPU; the host logic of both is also covered on CPU (gloo) in
tests/test_host_logic.py."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import block_fp8_oracle as O
from tests.util import assert_close_fp, codes_to_fp8, make_act, make_weight, to_f32_np

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from sglang_b200.srt.distributed import initialize_model_parallel
        from sglang_b200.srt.layers.linear import MergedColumnParallelLinear, RowParallelLinear
        from sglang_b200.srt.layers.moe.fused_moe_triton.layer import FusedMoE
        from sglang_b200.srt.layers.moe.token_dispatcher import StandardTopKOutput
        from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
        initialize_model_parallel(world, world)
        cfg = Fp8Config()
        # ---- tensor parallel: gate_up (column) -> down (row + all-reduce) on replicated tokens ----
        H, I, M = 512, 768, 70
        w1q, w1s = make_weight(2 * I, H, 1)
        w2q, w2s = make_weight(H, I, 2)
        x = make_act(M, H, 3, outliers=False)
        gate_up = MergedColumnParallelLinear(H, [I, I], quant_config=cfg, device=dev)
        down = RowParallelLinear(I, H, quant_config=cfg, device=dev)
        gate_up.load_full_weight(codes_to_fp8(w1q, dev), torch.from_numpy(w1s).to(dev))
        down.load_full_weight(codes_to_fp8(w2q, dev), torch.from_numpy(w2s).to(dev))
        gu, _ = gate_up(x.to(dev))          # [M, 2I/world]: this rank's slice of gate and of up
        h = (torch.nn.functional.silu(gu[:, : I // world].float()) * gu[:, I // world :].float()).to(torch.bfloat16)
        y, _ = down(h)                        # all-reduced
        # ---- expert parallel with all-to-all dispatch/combine; every rank owns different tokens ----
        E, Hm, Im, topk, T = 8, 512, 256, 2, 33 + rank
        w13q, w13s = make_weight(2 * Im, Hm, 5, std=0.05, experts=E)
        wdq, wds = make_weight(Hm, Im, 6, std=0.05, experts=E)
        g = torch.Generator().manual_seed(100 + rank)
        xt = make_act(T, Hm, 7 + rank, outliers=False)
        tw, ti = torch.topk(torch.softmax(torch.randn(T, E, generator=g), -1), topk)
        tw = (tw / tw.sum(-1, keepdim=True)).float()
        ti = ti.to(torch.int32)
        # the replicate-and-mask form needs every rank to hold the same tokens: all ranks build rank 0's
        g0 = torch.Generator().manual_seed(100)
        x0 = make_act(33, Hm, 7, outliers=False)
        tw0, ti0 = torch.topk(torch.softmax(torch.randn(33, E, generator=g0), -1), topk)
        tw0 = (tw0 / tw0.sum(-1, keepdim=True)).float()
        ti0 = ti0.to(torch.int32)
        outs = {}
        for backend, (xi, wi, ii) in (("nccl", (xt, tw, ti)), ("none", (x0, tw0, ti0))):
            moe = FusedMoE(E, Hm, Im, topk, quant_config=cfg, a2a_backend=backend, device=dev)
            moe.load_full_weights(codes_to_fp8(w13q, dev), torch.from_numpy(w13s).to(dev), codes_to_fp8(wdq, dev),
                                  torch.from_numpy(wds).to(dev))
            outs[backend] = moe(xi.to(dev), StandardTopKOutput(wi.to(dev), ii.to(dev), None)).float().cpu().numpy()
        # decode-sized batches of equal size per rank: all-gather, local experts, reduce-scatter
        moe = FusedMoE(E, Hm, Im, topk, quant_config=cfg, a2a_backend="nccl", device=dev,
                       equal_tokens_gather_below=1024)
        moe.load_full_weights(codes_to_fp8(w13q, dev), torch.from_numpy(w13s).to(dev), codes_to_fp8(wdq, dev),
                              torch.from_numpy(wds).to(dev))
        outs["gather"] = moe(xt[:33].to(dev), StandardTopKOutput(tw[:33].to(dev), ti[:33].to(dev), None)).float().cpu().numpy()
        # redundant copies of the two hottest experts on every rank (srt/eplb): hot rows are served by the sender's own copy
        from sglang_b200.srt.eplb import ExpertLocationMetadata
        count = torch.bincount(ti.flatten().long(), minlength=E).float().to(dev)
        dist.all_reduce(count)
        for key, make in (("replicas", ExpertLocationMetadata.init_by_hot_replication),
                          ("packed", ExpertLocationMetadata.init_by_load)):  # (hot copies; hot copies + cold experts by load)
            loc = make(count, world, rank, 2)
            moe = FusedMoE(E, Hm, Im, topk, quant_config=cfg, a2a_backend="nccl", device=dev, expert_location=loc)
            moe.load_full_weights(codes_to_fp8(w13q, dev), torch.from_numpy(w13s).to(dev), codes_to_fp8(wdq, dev),
                                  torch.from_numpy(wds).to(dev))
            outs[key] = moe(xt.to(dev), StandardTopKOutput(tw.to(dev), ti.to(dev), None)).float().cpu().numpy()
        torch.cuda.synchronize()
        from sglang_b200 import ops
        ret[rank] = dict(moe_rep=outs["replicas"], moe_packed=outs["packed"], moe_gather=outs["gather"], y=y.float().cpu().numpy(), gu=gu.float().cpu().numpy(), moe_a2a=outs["nccl"],
                         moe_std=outs["none"], x=to_f32_np(xt), tw=tw.numpy(), ti=ti.numpy(), status=ops.gemm_status())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_and_ep_on_two_gpus():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    H, I, M = 512, 768, 70
    w1q, w1s = make_weight(2 * I, H, 1)
    w2q, w2s = make_weight(H, I, 2)
    x = to_f32_np(make_act(M, H, 3, outliers=False))
    gu = O.block_fp8_linear(x, w1q, w1s)
    h = O.bf16_round((gu[:, :I] / (1 + np.exp(-gu[:, :I]))).astype(np.float32) * gu[:, I:])
    y_ref = O.block_fp8_linear(h, w2q, w2s)
    E, Hm, Im, topk = 8, 512, 256, 2
    w13q, w13s = make_weight(2 * Im, Hm, 5, std=0.05, experts=E)
    wdq, wds = make_weight(Hm, Im, 6, std=0.05, experts=E)
    for r in range(world):
        d = ret[r]
        assert d["status"] == 0
        # column-parallel slices: rank r holds columns [r*I/2, (r+1)*I/2) of gate and of up
        lo, hi = r * I // world, (r + 1) * I // world
        assert_close_fp(d["gu"], np.concatenate([gu[:, lo:hi], gu[:, I + lo : I + hi]], 1))
        # row-parallel: bf16 partial sums are added by the all-reduce, one extra bf16 rounding per rank
        assert_close_fp(d["y"], y_ref, rtol=2e-2, atol=2e-2, min_cos=0.9995)
        ref = O.fused_experts_block_fp8(d["x"], w13q, w13s, wdq, wds, d["tw"], d["ti"], 1.0)
        assert_close_fp(d["moe_a2a"], ref, rtol=2e-2, atol=2e-2)
        assert_close_fp(d["moe_rep"], ref, rtol=2e-2, atol=2e-2)
        assert_close_fp(d["moe_packed"], ref, rtol=2e-2, atol=2e-2)
        assert d["moe_gather"].shape == (33, Hm)
        assert_close_fp(d["moe_gather"], ref[:33], rtol=2e-2, atol=2e-2)
    ref0 = O.fused_experts_block_fp8(ret[0]["x"], w13q, w13s, wdq, wds, ret[0]["tw"], ret[0]["ti"], 1.0)
    for r in range(world):
        assert_close_fp(ret[r]["moe_std"], ref0, rtol=2e-2, atol=2e-2)


def _fused_sizes(world):
    # whole multiples of 128 x world, one size below the fused path's minimum, and two ragged row counts (the last
    # owners hold a partial block of rows; with 8 ranks and 128 x world + 44 rows six of them hold none)
    return (4 * 128 * world // 2, 128 * world, 70, 4 * 128 * world, 128 * world + 44, 4 * 128 * world - 24)


def _fused_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from sglang_b200 import ops
        from sglang_b200.srt.distributed import (destroy_model_parallel, enable_fused_row_parallel,
                                                 initialize_model_parallel)
        from sglang_b200.srt.distributed.fused_row_parallel import comm_status
        from sglang_b200.srt.layers.linear import RowParallelLinear
        from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
        initialize_model_parallel(world, 1)
        K, N = 1024, 712  # N is not a multiple of the 192-column tile nor of its 64-column store groups
        wq, ws = make_weight(N, K, 21)
        down = RowParallelLinear(K, N, quant_config=Fp8Config(), device=dev)
        down.load_full_weight(codes_to_fp8(wq, dev), torch.from_numpy(ws).to(dev))
        k = K // world
        sizes = _fused_sizes(world)
        xs = [make_act(M, K, 30 + i, outliers=False)[:, rank * k : (rank + 1) * k].contiguous().to(dev)
              for i, M in enumerate(sizes)]
        nccl = [down(x)[0].clone() for x in xs]            # plain path: GEMM, then NCCL all-reduce
        comm = enable_fused_row_parallel(max(sizes) * N)
        assert comm.supports(sizes[4], N) and comm.supports(sizes[5], N)
        assert comm.supports(sizes[0], N) and comm.supports(sizes[3], N) and not comm.supports(70, N)
        fused = [down(x)[0].clone() for x in xs]           # 70 rows fall back to the plain path
        fused2 = [down(x)[0].clone() for x in xs]          # flags and staging are reused by later calls
        comm.pipeline, comm.min_waves, comm.min_comm_ratio = True, 0, 0.0  # row chunks wherever the row count allows:
        piped = [down(x)[0].clone() for x in xs]           # reduce-and-gather of a chunk beside the next chunk's GEMM
        assert comm._chunks(sizes[3], N, k) == 4 and comm._chunks(sizes[0], N, k) == 2 and comm._chunks(sizes[1], N, k) == 1
        torch.cuda.synchronize()
        ret[rank] = dict(nccl=[t.float().cpu().numpy() for t in nccl], fused=[t.float().cpu().numpy() for t in fused],
                         again=all(torch.equal(a, b) for a, b in zip(fused, fused2)) and
                         all(torch.equal(a, b) for a, b in zip(fused, piped)),
                         status=(ops.gemm_status(), comm_status()))
        destroy_model_parallel()
    finally:
        dist.destroy_process_group()


def _check_fused(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_fused_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    K, N = 1024, 712
    wq, ws = make_weight(N, K, 21)
    for r in range(world):
        assert ret[r]["status"] == (0, 0) and ret[r]["again"]
    for i, M in enumerate(_fused_sizes(world)):
        for r in range(world):
            if world == 2 or M == 70:
                # with two ranks, adding two bf16 partial sums in float32 and rounding once is what NCCL's bf16 sum does
                assert np.array_equal(ret[r]["fused"][i], ret[r]["nccl"][i])
            if M != 70:  # (the ring all-reduce of the plain path does not promise identical rows on every rank)
                assert np.array_equal(ret[r]["fused"][i], ret[0]["fused"][i])
        x = to_f32_np(make_act(M, K, 30 + i, outliers=False))
        assert_close_fp(ret[0]["fused"][i], O.block_fp8_linear(x, wq, ws), rtol=2e-2, atol=2e-2, min_cos=0.9995)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_row_parallel_all_reduce_on_two_gpus():
    """The GEMM whose epilogue pushes tiles to their owner + the reduce-and-gather kernel against GEMM + NCCL."""
    _check_fused(2)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs or more")
def test_fused_row_parallel_all_reduce_on_all_gpus():
    _check_fused(8 if torch.cuda.device_count() >= 8 else 4)
