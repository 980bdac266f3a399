"""Extra sections of bench.py: the per-M GEMM sweep of BASELINE config 1, the tensor-parallel Llama-3-70B
layer of config 2 and the expert-parallel DeepSeek-V3 MoE layer of config 3.  Each returns a dict that
bench.py merges into its JSON line.  Times are CUDA-event times on the launching stream, max over ranks.
"""
from __future__ import annotations

import torch

SWEEP_M = [1, 16, 64, 256, 1024, 4096, 8192]
L2_BYTES = 126 * 1024 * 1024


def _barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def _max_ms(ms, world, dev):
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _time(fn, iters, warmup, world, dev):
    for _ in range(warmup):
        fn()
    _barrier(world)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return _max_ms(e0.elapsed_time(e1) / iters, world, dev)


def _time_graph(fn, iters, warmup, dev):
    """One call of `fn` captured into a CUDA graph and replayed: the launch-bound small-batch sizes are served from
    graphs (as the reference serves its decode batches), so their eager time measures Python, not the GPU."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    ms = _time(g.replay, iters, 2, 1, dev)
    del g
    return ms


def _fill_weight(dst_q, dst_s, gen, std=0.02, chunk=8):
    """Random N(0,std) weights quantised per 128x128 block, written expert-chunk by expert-chunk."""
    from bench import make_block_fp8_weight
    if dst_q.dim() == 2:
        q, s = make_block_fp8_weight(dst_q.shape[0], dst_q.shape[1], dst_q.device, gen, std)
        dst_q.copy_(q)
        dst_s.copy_(s)
        return
    E, N, K = dst_q.shape
    for e0 in range(0, E, chunk):
        n = min(chunk, E - e0)
        q, s = make_block_fp8_weight(N, K, dst_q.device, gen, std, experts=n)
        dst_q[e0 : e0 + n].copy_(q)
        dst_s[e0 : e0 + n].copy_(s)
        del q, s


# ------------------------------------------------------------------------------------------------
# config 1: GEMM sweep over M
# ------------------------------------------------------------------------------------------------


def gemm_sweep(args, ctx, peaks):
    from bench import DSV3_LAYERS, make_block_fp8_weight
    from sglang_b200 import ops
    rank, world, dev = ctx
    gen = torch.Generator(device=dev).manual_seed(7)
    out = {}
    for name, N, K in DSV3_LAYERS:
        wq, ws = make_block_fp8_weight(N, K, dev, gen)
        # rotate over enough copies of the weight that successive launches cannot hit L2
        copies = max(1, -(-2 * L2_BYTES // (N * K)))
        wqs = [wq] + [wq.clone() for _ in range(copies - 1)]
        res = {}
        for M in SWEEP_M:
            x = torch.randn(M, K, device=dev, generator=gen).bfloat16()
            xq, xs = ops.per_token_group_quant_fp8(x, 128)
            state = {"i": 0}

            def run():
                w = wqs[state["i"] % copies]
                state["i"] += 1
                ops.w8a8_block_fp8_matmul(xq, w, xs, ws, [128, 128], torch.bfloat16)

            iters = 20 if M <= 1024 else 10
            # the launches are replayed from a CUDA graph so that what is timed is the device, not the Python
            # call overhead (the reference times its kernels the same way: bench_fp8_blockwise_gemm.py:162-170)
            for _ in range(3):
                run()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(iters):
                    run()
            ms = _time(graph.replay, 3, 1, world, dev) / iters
            del graph
            flops = 2.0 * M * N * K
            nbytes = M * K + N * K + 2 * M * N + 4 * M * (K // 128) + 4 * ((N + 127) // 128) * (K // 128)
            res[str(M)] = {"us": ms * 1e3, "tflops": flops / ms / 1e9, "gbs": nbytes / ms / 1e6}
        out[name] = res
        del wqs, wq
        torch.cuda.empty_cache()
    return {"gemm_sweep": {"unit": "us / TFLOP/s / GB/s (algorithmic bytes)", "l2": "weight copies rotated so that "
                           "consecutive launches exceed the 126 MB L2", "layers": out,
                           "hbm_peak_gbs": peaks["hbm_gbs"], "fp8_peak_tflops": 2 * peaks["bf16"]}}


# ------------------------------------------------------------------------------------------------
# config 2: Llama-3-70B-shaped layer, tensor parallel
# ------------------------------------------------------------------------------------------------


def tp_layer(args, ctx, peaks):
    """QKV (column) -> o_proj (row + all-reduce) -> gate_up (column) -> silu_and_mul + quantizer -> down (row + all-reduce).
    Attention itself is not on this path: o_proj is fed a tensor of the attention output's shape."""
    from sglang_b200 import ops
    from sglang_b200.srt.distributed import initialize_model_parallel
    from sglang_b200.srt.layers.linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
    rank, world, dev = ctx
    initialize_model_parallel(world, world)
    cfg = Fp8Config()
    H, I, heads, kv_heads, hd = 8192, 28672, 64, 8, 128
    gen = torch.Generator(device=dev).manual_seed(11 + rank)
    qkv = QKVParallelLinear(H, hd, heads, kv_heads, quant_config=cfg, device=dev)
    o_proj = RowParallelLinear(heads * hd, H, quant_config=cfg, device=dev)
    gate_up = MergedColumnParallelLinear(H, [I, I], quant_config=cfg, device=dev)
    down = RowParallelLinear(I, H, quant_config=cfg, device=dev)
    for lin in (qkv, o_proj, gate_up, down):
        _fill_weight(lin.weight.data, lin.weight_scale_inv.data, gen)
    flops_per_token = 2.0 * (H * (heads + 2 * kv_heads) * hd + heads * hd * H + H * 2 * I + I * H)
    res = {}
    sizes = (8, 128, 2048, 8192)
    inputs = {M: (torch.randn(M, H, device=dev, generator=gen).bfloat16(),
                  torch.randn(M, heads * hd // world, device=dev, generator=gen).bfloat16()) for M in sizes}

    def run_all(key):
        for M in sizes:
            x, attn = inputs[M]

            def layer():
                qkv(x)
                h, _ = o_proj(attn)
                gu, _ = gate_up(h)
                # activation and the 1x128 quantisation of down's input in one pass; `apply` takes (codes, scales)
                down(ops.silu_and_mul_quant_fp8(gu, 128))

            ms = _time(layer, 10 if M >= 2048 else 20, 3, world, dev)
            res.setdefault(str(M), {"allreduce_bytes": 2 * M * H * 2})[key] = ms
            if world == 1 and M <= 128:
                res[str(M)]["ms_eager"] = ms
                res[str(M)][key] = _time_graph(layer, 20, 3, dev)
                res[str(M)]["launch"] = "cuda graph"

    run_all("ms_nccl" if world > 1 else "ms")
    if world > 1:
        # the same layer with the all-reduce of o_proj and down fused into their GEMMs where the shape allows
        # (at least 128 x world rows); smaller batches keep the NCCL all-reduce and repeat the number above
        from sglang_b200.srt.distributed import destroy_model_parallel, enable_fused_row_parallel
        from sglang_b200.srt.distributed.fused_row_parallel import comm_status
        comm = enable_fused_row_parallel(max(sizes) * H)
        run_all("ms_fused")
        for M in sizes:
            r = res[str(M)]
            r["fused_all_reduce"] = bool(comm.supports(M, H))
            r["ms"] = r["ms_fused"] if r["fused_all_reduce"] else r["ms_nccl"]
        status = comm_status()
        destroy_model_parallel()
    else:
        status = 0
    for M in sizes:
        res[str(M)]["tflops"] = flops_per_token * M / res[str(M)]["ms"] / 1e9
    return {"tp_layer": {"config": "BASELINE config 2: Llama-3-70B layer (hidden 8192, inter 28672, 64q/8kv x 128), "
                                   "QKV + gate_up column-parallel, o_proj + down row-parallel; the sum over ranks is "
                                   "an NCCL all-reduce (ms_nccl) or the GEMM-fused all-reduce over peer memory "
                                   "(ms_fused); ms is the fused form where the shape allows it",
                         "tp": world, "scaling": "strong", "comm_status": status, "results": res}}


# ------------------------------------------------------------------------------------------------
# config 3: DeepSeek-V3-shaped MoE layer, expert parallel
# ------------------------------------------------------------------------------------------------


def moe_layer(args, ctx, peaks):
    from sglang_b200 import ops
    from sglang_b200.srt.distributed import initialize_model_parallel
    from sglang_b200.srt.layers.linear import ColumnParallelLinear
    from sglang_b200.srt.layers.moe.fused_moe_triton.layer import FusedMoE
    from sglang_b200.srt.layers.moe.token_dispatcher import StandardTopKOutput
    from sglang_b200.srt.layers.moe.topk import biased_grouped_topk
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
    rank, world, dev = ctx
    initialize_model_parallel(1, world)
    cfg = Fp8Config()
    E, H, I, topk = 256, 7168, 2048, 8
    gen = torch.Generator(device=dev).manual_seed(23 + rank)
    # (every rank holds the same number of tokens here, so decode-sized batches may take the gather form)
    moe = FusedMoE(E, H, I, topk, quant_config=cfg, a2a_backend="nccl", device=dev, equal_tokens_gather_below=2048)
    _fill_weight(moe.w13_weight.data, moe.w13_weight_scale_inv.data, gen)
    _fill_weight(moe.w2_weight.data, moe.w2_weight_scale_inv.data, gen)
    # the shared expert is a dense block-FP8 MLP replicated on every rank (models/deepseek_v2.py:826-882)
    sh_gate_up = ColumnParallelLinear(H, 2 * I, quant_config=cfg, device=dev)
    sh_down = ColumnParallelLinear(I, H, quant_config=cfg, device=dev)
    for lin in (sh_gate_up, sh_down):
        _fill_weight(lin.weight.data, lin.weight_scale_inv.data, gen)
    res = {}
    for T in (1, 64, 512, 4096):
        x = torch.randn(T, H, device=dev, generator=gen).bfloat16()
        logits = torch.randn(T, E, device=dev, generator=gen)
        w, ids = biased_grouped_topk(logits, None, topk, True, 8, 4)
        top = StandardTopKOutput(w, ids, None)

        def layer():
            routed = moe(x, top)
            gu, _ = sh_gate_up(x)
            shared, _ = sh_down(ops.silu_and_mul_quant_fp8(gu, 128))
            return routed + shared

        ms = _time(layer, 10, 3, world, dev)
        extra = {}
        if world == 1 and T <= 512:
            extra = {"ms_eager": ms, "launch": "cuda graph"}
            ms = _time_graph(layer, 10, 3, dev)
        flops = 6.0 * T * topk * H * I + 6.0 * T * H * I
        res[str(T)] = {"ms": ms, "tokens_per_s": world * T / ms * 1e3, "tflops_per_gpu": flops / ms / 1e9, **extra}
    return {"moe_layer": {"config": "BASELINE config 3: DeepSeek-V3 MoE, 256 routed experts + 1 shared, hidden 7168, "
                                    "moe_intermediate 2048, top-8 grouped sigmoid routing (8 groups, top-4), "
                                    "tokens per GPU as keyed; expert-parallel with NCCL all-to-all dispatch/combine (batches of at "
                                    "most 2048 tokens over all ranks: all-gather, local experts, reduce-scatter)",
                          "ep": world, "scaling": "weak", "results": res}}


# ------------------------------------------------------------------------------------------------
# config 4: Qwen3-30B-A3B-shaped MoE layer under Zipf-skewed expert popularity
# ------------------------------------------------------------------------------------------------


def moe_layer_skewed(args, ctx, peaks):
    """128 experts, hidden 2048, moe_intermediate 768, top-8 softmax routing; the logits carry log(p_e) with
    p_e ~ rank^-1.2 over a seeded permutation of the experts.  Reports the layer time (max over ranks), this
    rank's own time and the spread of tokens per local expert, i.e. the load-imbalance tail."""
    from sglang_b200.srt.distributed import initialize_model_parallel
    from sglang_b200.srt.layers.moe.fused_moe_triton.layer import FusedMoE
    from sglang_b200.srt.layers.moe.token_dispatcher import StandardTopKOutput
    from sglang_b200.srt.layers.moe.topk import fused_topk
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
    rank, world, dev = ctx
    initialize_model_parallel(1, world)
    E, H, I, topk = 128, 2048, 768, 8
    gen = torch.Generator(device=dev).manual_seed(41 + rank)
    moe = FusedMoE(E, H, I, topk, quant_config=Fp8Config(), a2a_backend="nccl", device=dev,
                   equal_tokens_gather_below=2048)
    _fill_weight(moe.w13_weight.data, moe.w13_weight_scale_inv.data, gen)
    _fill_weight(moe.w2_weight.data, moe.w2_weight_scale_inv.data, gen)
    perm = torch.randperm(E, generator=torch.Generator().manual_seed(7))  # the same popularity order on every rank
    logp = torch.empty(E)
    logp[perm] = -1.2 * torch.log(torch.arange(1, E + 1, dtype=torch.float32))
    logp = logp.to(dev)
    res = {}
    for T in (32, 1024, 16384):
        x = torch.randn(T, H, device=dev, generator=gen).bfloat16()
        logits = torch.randn(T, E, device=dev, generator=gen) + logp
        w, ids = fused_topk(logits, topk, True)
        top = StandardTopKOutput(w, ids, None)
        counts = torch.bincount(ids.flatten().long(), minlength=E).float()
        ms = _time(lambda: moe(x, top), 10, 3, world, dev)
        extra = {}
        if world == 1 and T <= 1024:
            extra = {"ms_eager": ms, "launch": "cuda graph"}
            ms = _time_graph(lambda: moe(x, top), 10, 3, dev)
        # this rank alone, without the barrier-and-max: the gap to `ms` at EP > 1 is the wait for the busiest rank
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(10):
            moe(x, top)
        e1.record()
        torch.cuda.synchronize()
        res[str(T)] = {"ms": ms, "ms_this_rank": e0.elapsed_time(e1) / 10, "tokens_per_s": world * T / ms * 1e3,
                       "tflops_per_gpu": 6.0 * T * topk * H * I / ms / 1e9,
                       "routed_per_expert_max_over_mean": float(counts.max() / counts.mean()),
                       "experts_hit": int((counts > 0).sum()), **extra}
    return {"moe_layer_skewed": {"config": "BASELINE config 4: Qwen3-30B-A3B MoE, 128 experts, hidden 2048, "
                                           "moe_intermediate 768, top-8 softmax routing, Zipf(1.2) expert popularity, "
                                           "tokens per GPU as keyed",
                                 "ep": world, "scaling": "weak", "results": res}}


# ------------------------------------------------------------------------------------------------
# the memory-bound kernels of the path: GB/s of algorithmic bytes against the measured HBM copy rate
# ------------------------------------------------------------------------------------------------


def hbm_kernels(args, ctx, peaks):
    from sglang_b200 import ops
    rank, world, dev = ctx
    gen = torch.Generator(device=dev).manual_seed(5)
    out = {}

    def graph_time(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        ms = _time(g.replay, 3, 1, world, dev) / iters
        del g
        return ms

    # 1x128 quantizer at the largest activation of config 1 (8192 x 18432 bf16: 453 MB of traffic per call)
    M, K = 8192, 18432
    x = torch.randn(M, K, device=dev, generator=gen).bfloat16()
    ms = graph_time(lambda: ops.per_token_group_quant_fp8(x, 128))
    nbytes = M * K * 3 + M * (K // 128) * 4
    out["per_token_group_quant_fp8"] = {"shape": [M, K], "us": ms * 1e3, "gbs": nbytes / ms / 1e6,
                                        "frac_of_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"]}
    del x
    # fused silu_and_mul + quantizer on the config-3 intermediate of 4096 tokens x top-8 (32768 x 4096 bf16)
    R, I = 32768, 2048
    y = torch.randn(R, 2 * I, device=dev, generator=gen).bfloat16()
    ms = graph_time(lambda: ops.silu_and_mul_quant_fp8(y, 128))
    nbytes = R * (2 * I * 2 + I + (I // 128) * 4)
    out["silu_and_mul_quant_fp8"] = {"shape": [R, 2 * I], "us": ms * 1e3, "gbs": nbytes / ms / 1e6,
                                     "frac_of_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"]}
    del y
    # top-k sum on [4096, 8, 7168]
    z = torch.randn(4096, 8, 7168, device=dev, generator=gen).bfloat16()
    o = torch.empty(4096, 7168, device=dev, dtype=torch.bfloat16)
    ms = graph_time(lambda: ops.moe_sum_reduce_out(z, o, 1.0))
    nbytes = z.numel() * 2 + o.numel() * 2
    out["moe_sum_reduce"] = {"shape": [4096, 8, 7168], "us": ms * 1e3, "gbs": nbytes / ms / 1e6,
                             "frac_of_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"]}
    del z, o
    # moe_align_block_size: the layer sizes (latency regime) and a bandwidth-regime input (8M tokens x 8)
    align = {}
    for name, T, E in (("config3_T4096", 4096, 256), ("config4_T16384", 16384, 128), ("bandwidth_8M_tokens", 8 * 1024 * 1024, 256)):
        ids = torch.randint(0, E, (T, 8), device=dev, dtype=torch.int32, generator=gen)
        ms = graph_time(lambda: ops.moe_align_block_size(ids, 128, E), iters=5)
        post = int(ops.moe_align_block_size(ids, 128, E)[2].item())
        nbytes = 4 * (ids.numel() + post + post // 128 + 1)
        align[name] = {"ids": ids.numel(), "experts": E, "us": ms * 1e3, "gbs": nbytes / ms / 1e6,
                       "frac_of_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"]}
        del ids
    out["moe_align_block_size"] = align
    return {"hbm_kernels": {"unit": "us, GB/s of algorithmic bytes, fraction of MEASURED_PEAKS hbm_gbs", "kernels": out}}


def run(sections, args, ctx, peaks):
    out = {}
    rank, world, dev = ctx
    if "sweep" in sections and world == 1:
        out.update(gemm_sweep(args, ctx, peaks))
        torch.cuda.empty_cache()
    if "hbm" in sections and world == 1:
        out.update(hbm_kernels(args, ctx, peaks))
        torch.cuda.empty_cache()
    if "tp" in sections:
        out.update(tp_layer(args, ctx, peaks))
        torch.cuda.empty_cache()
    if "moe" in sections:
        out.update(moe_layer(args, ctx, peaks))
        torch.cuda.empty_cache()
        out.update(moe_layer_skewed(args, ctx, peaks))
        torch.cuda.empty_cache()
    return out
