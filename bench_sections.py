"""Extra sections of bench.py: the per-M GEMM sweep of BASELINE config 1, the tensor-parallel Llama-3-70B
layer of config 2 and the expert-parallel DeepSeek-V3 MoE layer of config 3.  Each returns a dict that
bench.py merges into its JSON line.  Times are CUDA-event times on the launching stream, max over ranks.
"""
from __future__ import annotations

import torch

SWEEP_M = [1, 16, 64, 256, 1024, 4096, 8192]
L2_BYTES = 126 * 1024 * 1024
# Expert-parallel batches of at most this many tokens over all ranks (the same count on every rank) take the gather
# form (quantise, all-gather the codes, local experts, reduce-scatter: no host synchronisation); larger ones the
# all-to-all form, whose fixed host-side cost (about a millisecond of split-size exchange and index kernels) they amortise.
GATHER_BELOW = 16384


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


def _time_graph(fn, iters, warmup, dev, world=1):
    """One call of `fn` captured into a CUDA graph and replayed: the launch-bound small-batch sizes are served from
    graphs (as the reference serves its decode batches), so their eager time measures Python, not the GPU.
    With `world` > 1 every rank captures the same call (its NCCL collectives and cross-rank kernels included) and the
    replays are timed like any other step: barrier, CUDA events, max over ranks.  Returns None if any rank could not
    capture (the ranks agree on that before anything is replayed)."""
    for _ in range(warmup):
        fn()
    _barrier(world)
    torch.cuda.synchronize()
    g, ok = torch.cuda.CUDAGraph(), 1.0
    try:
        with torch.cuda.graph(g):
            fn()
    except Exception:  # noqa: BLE001  (reported by the caller as a missing graph number)
        ok = 0.0
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        flag = torch.tensor([ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = float(flag.item())
    if ok < 1.0:
        del g
        return None
    ms = _time(g.replay, iters, 2, world, dev)
    del g
    return ms


def _time_graph_alone(fn, iters, warmup, world, dev):
    """`_time_graph` of a call without collectives, timed by every rank for itself: the slowest rank's time, or None
    if some rank could not capture."""
    ms = _time_graph(fn, iters, warmup, dev)
    worst = _max_ms(ms if ms is not None else float("inf"), world, dev)
    return None if worst == float("inf") else worst


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
    # the reference's own CUDA kernel, where its comparator library is built (one GPU only): timed right after this
    # library's kernel, same inputs, same graph-replay protocol, same clocks
    import os
    ref_mm = None
    ref_lib = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "libsgl_gpu_ref.so")
    if world == 1 and os.path.exists(ref_lib):
        try:
            torch.ops.load_library(ref_lib)
            ref_mm = torch.ops.sgl_gpu_ref.fp8_blockwise_scaled_mm
        except Exception:  # noqa: BLE001  (the comparator is optional)
            ref_mm = None
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
            if ref_mm is not None and N % 128 == 0 and M >= 256:  # (it wants whole 128-column blocks)
                xs_m = xs.t().contiguous().t()  # M-major activation scales, as the reference kernel wants them
                ws_t = ws.t()

                def run_ref():
                    w = wqs[state["i"] % copies]
                    state["i"] += 1
                    ref_mm(xq, w.t(), xs_m, ws_t, torch.bfloat16)

                try:
                    for _ in range(3):
                        run_ref()
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        for _ in range(iters):
                            run_ref()
                    ms_ref = _time(graph.replay, 3, 1, world, dev) / iters
                    del graph
                    res[str(M)].update({"ref_us": ms_ref * 1e3, "ref_tflops": flops / ms_ref / 1e9})
                except Exception:  # noqa: BLE001
                    ref_mm = None
        out[name] = res
        del wqs, wq
        torch.cuda.empty_cache()
    return {"gemm_sweep": {"unit": "us / TFLOP/s / GB/s (algorithmic bytes)", "l2": "weight copies rotated so that "
                           "consecutive launches exceed the 126 MB L2", "layers": out,
                           "hbm_peak_gbs": peaks["hbm_gbs"],
                           "fp8_peak_tflops": peaks.get("fp8_measured", 2 * peaks["bf16"]),
                           "fp8_peak_source": "the same denominator as roofline.peak of this line",
                           "ref": "ref_us / ref_tflops: the reference's own CUDA kernel (sgl-kernel fp8_blockwise_scaled_mm, "
                                  "compiled unmodified into oracle/_ref) timed right after this library's kernel on the same "
                                  "inputs with the same protocol; absent where that library is not built"}}


def config0_gpu(args, ctx, peaks):
    """BASELINE config 0 on the GPU: one block-FP8 linear, M = 64, N = K = 4096 (quantizer + GEMM, graph-replayed,
    weight copies rotated past L2); the CPU arm's time for the same shape is `config0_cpu` / the reference arm's
    `config0`."""
    from bench import make_block_fp8_weight
    from sglang_b200 import ops
    rank, world, dev = ctx
    gen = torch.Generator(device=dev).manual_seed(0)
    M, N, K = 64, 4096, 4096
    wq, ws = make_block_fp8_weight(N, K, dev, gen)
    copies = -(-2 * L2_BYTES // (N * K))
    wqs = [wq] + [wq.clone() for _ in range(copies - 1)]
    x = torch.randn(M, K, device=dev, generator=gen).bfloat16()
    state = {"i": 0}

    def run():
        w = wqs[state["i"] % copies]
        state["i"] += 1
        xq, xs = ops.per_token_group_quant_fp8(x, 128)
        ops.w8a8_block_fp8_matmul(xq, w, xs, ws, [128, 128], torch.bfloat16)

    for _ in range(3):
        run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(20):
            run()
    ms = _time(graph.replay, 3, 1, world, dev) / 20
    del graph
    nbytes = N * K + M * K * 3 + 2 * M * N
    return {"config0": {"workload": "BASELINE config 0: M=64, N=K=4096 block-FP8 linear (quantizer + GEMM)",
                        "us": ms * 1e3, "tflops": 2.0 * M * N * K / ms / 1e9, "gbs": nbytes / ms / 1e6,
                        "frac_of_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"]}}


# ------------------------------------------------------------------------------------------------
# config 2: Llama-3-70B-shaped layer, tensor parallel
# ------------------------------------------------------------------------------------------------


def tp_layer(args, ctx, peaks):
    """QKV (column) -> o_proj (row + all-reduce) -> gate_up (column) -> silu_and_mul + quantizer -> down (row + all-reduce).
    Attention itself is not on this path: o_proj is fed a tensor of the attention output's shape.
    With more than one rank: a parity check of the sharded layer first (`tp_parity`), then the unsharded layer timed
    on every GPU by itself (`ms_1gpu_eager`, the numerator of the strong-scaling efficiency), then the sharded layer
    with the NCCL all-reduce and with the GEMM-fused all-reduce.  Every size is timed from eager launches at every
    rank count (`ms_eager`); on one GPU the launch-bound sizes are also replayed from a CUDA graph (`ms`)."""
    from sglang_b200 import ops
    from sglang_b200.srt.distributed import destroy_model_parallel, enable_fused_row_parallel, initialize_model_parallel
    from sglang_b200.srt.distributed.fused_row_parallel import comm_status
    from sglang_b200.srt.layers.linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
    rank, world, dev = ctx
    parity = tp_parity(ctx) if world > 1 else None
    cfg = Fp8Config()
    H, I, heads, kv_heads, hd = 8192, 28672, 64, 8, 128
    flops_per_token = 2.0 * (H * (heads + 2 * kv_heads) * hd + heads * hd * H + H * 2 * I + I * H)
    sizes = (8, 128, 2048, 8192)
    res = {str(M): {"allreduce_bytes": 2 * M * H * 2} for M in sizes}

    def build(tp):
        initialize_model_parallel(tp, tp)
        gen = torch.Generator(device=dev).manual_seed(11 + rank)
        qkv = QKVParallelLinear(H, hd, heads, kv_heads, quant_config=cfg, device=dev)
        o_proj = RowParallelLinear(heads * hd, H, quant_config=cfg, device=dev)
        gate_up = MergedColumnParallelLinear(H, [I, I], quant_config=cfg, device=dev)
        down = RowParallelLinear(I, H, quant_config=cfg, device=dev)
        for lin in (qkv, o_proj, gate_up, down):
            _fill_weight(lin.weight.data, lin.weight_scale_inv.data, gen)
        inputs = {M: (torch.randn(M, H, device=dev, generator=gen).bfloat16(),
                      torch.randn(M, heads * hd // tp, device=dev, generator=gen).bfloat16()) for M in sizes}

        def layer_for(M):
            x, attn = inputs[M]

            def layer():
                qkv(x)
                h, _ = o_proj(attn)
                gu, _ = gate_up(h)
                # activation and the 1x128 quantisation of down's input in one pass; `apply` takes (codes, scales)
                down(ops.silu_and_mul_quant_fp8(gu, 128))

            return layer

        return layer_for

    def time_all(layer_for, key, ranks):
        for M in sizes:
            res[str(M)][key] = _time(layer_for(M), 10 if M >= 2048 else 20, 3, ranks, dev)

    status = 0
    if world == 1:
        layer_for = build(1)
        time_all(layer_for, "ms_eager", 1)
        for M in sizes:
            r = res[str(M)]
            r["ms"] = r["ms_eager"]
            if M <= 128:
                g_ms = _time_graph(layer_for(M), 20, 3, dev)
                if g_ms is not None:
                    r["ms"], r["launch"] = g_ms, "cuda graph"
    else:
        small = [M for M in sizes if M <= 128]  # launch-bound: also replayed from CUDA graphs, alone and sharded
        layer_for = build(1)  # the whole layer on this GPU alone: no collective, every rank times its own copy
        time_all(layer_for, "ms_1gpu_eager", world)
        for M in small:
            res[str(M)]["ms_1gpu_graph"] = _time_graph_alone(layer_for(M), 20, 3, world, dev)
        del layer_for
        torch.cuda.empty_cache()
        layer_for = build(world)
        time_all(layer_for, "ms_nccl", world)
        for M in small:
            res[str(M)]["ms_nccl_graph"] = _time_graph(layer_for(M), 20, 3, dev, world)
        # the same layer with the all-reduce of o_proj and down fused into their GEMMs where the shape allows
        # (at least 128 x world rows); smaller batches keep the NCCL all-reduce and repeat the number above
        comm = enable_fused_row_parallel(max(sizes) * H)
        time_all(layer_for, "ms_fused", world)
        for M in sizes:
            r = res[str(M)]
            r["fused_all_reduce"] = bool(comm.supports(M, H))
            r["ms"] = r["ms_fused"] if r["fused_all_reduce"] else r["ms_nccl"]
            r["ms_eager"] = r["ms"]
            r["efficiency_vs_1gpu"] = r["ms_1gpu_eager"] / (world * r["ms"])
            if M in small and r.get("ms_nccl_graph") and r.get("ms_1gpu_graph") and not r["fused_all_reduce"]:
                # graph against graph: what a decode batch costs when both arms are served from CUDA graphs
                r["launch"] = "cuda graph"
                r["ms"] = r["ms_nccl_graph"]
                r["efficiency_vs_1gpu"] = r["ms_1gpu_graph"] / (world * r["ms"])
        status = comm_status()
        destroy_model_parallel()
    for M in sizes:
        res[str(M)]["tflops"] = flops_per_token * M / res[str(M)]["ms"] / 1e9
    out = {"config": "BASELINE config 2: Llama-3-70B layer (hidden 8192, inter 28672, 64q/8kv x 128), "
                     "QKV + gate_up column-parallel, o_proj + down row-parallel; the sum over ranks is "
                     "an NCCL all-reduce (ms_nccl) or the GEMM-fused all-reduce over peer memory "
                     "(ms_fused); ms is the fused form where the shape allows it; ms_1gpu_eager = the unsharded "
                     "layer on one GPU of this box in this run",
           "tp": world, "scaling": "strong", "comm_status": status, "results": res}
    if parity is not None:
        out["parity"] = parity
    return {"tp_layer": out}


# ------------------------------------------------------------------------------------------------
# config 3: DeepSeek-V3-shaped MoE layer, expert parallel
# ------------------------------------------------------------------------------------------------


def moe_layer(args, ctx, peaks):
    """With more than one rank: `ep_parity` first, then the whole layer (all 256 experts) timed on every GPU by itself
    (`ms_1gpu_eager`: the numerator of the weak-scaling efficiency), then the expert-parallel layer."""
    from sglang_b200 import ops
    from sglang_b200.srt.distributed import initialize_model_parallel
    from sglang_b200.srt.layers.linear import ColumnParallelLinear
    from sglang_b200.srt.layers.moe.fused_moe_triton.layer import FusedMoE
    from sglang_b200.srt.layers.moe.token_dispatcher import StandardTopKOutput
    from sglang_b200.srt.layers.moe.topk import biased_grouped_topk, fused_topk
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
    rank, world, dev = ctx
    parity = ep_parity(ctx) if world > 1 else None
    cfg = Fp8Config()
    E, H, I, topk = 256, 7168, 2048, 8
    sizes = (1, 64, 512, 4096)
    reduced = bool(getattr(args, "moe_experts", 0) or getattr(args, "moe_tokens", 0))
    if reduced:  # a reduced case for profiler captures (a few GB on the device, one size)
        E = args.moe_experts or E
        sizes = (args.moe_tokens,) if args.moe_tokens else sizes
    res = {str(T): {} for T in sizes}

    def build(ep):
        initialize_model_parallel(1, ep)
        gen = torch.Generator(device=dev).manual_seed(23 + rank)
        # (every rank holds the same number of tokens here, so decode-sized batches may take the gather form)
        moe = FusedMoE(E, H, I, topk, quant_config=cfg, a2a_backend="nccl", device=dev, equal_tokens_gather_below=GATHER_BELOW)
        _fill_weight(moe.w13_weight.data, moe.w13_weight_scale_inv.data, gen)
        _fill_weight(moe.w2_weight.data, moe.w2_weight_scale_inv.data, gen)
        # the shared expert is a dense block-FP8 MLP replicated on every rank (models/deepseek_v2.py:826-882)
        sh_gate_up = ColumnParallelLinear(H, 2 * I, quant_config=cfg, device=dev)
        sh_down = ColumnParallelLinear(I, H, quant_config=cfg, device=dev)
        for lin in (sh_gate_up, sh_down):
            _fill_weight(lin.weight.data, lin.weight_scale_inv.data, gen)

        def layer_for(T):
            x = torch.randn(T, H, device=dev, generator=gen).bfloat16()
            logits = torch.randn(T, E, device=dev, generator=gen)
            w, ids = biased_grouped_topk(logits, None, topk, True, 8, min(4, max(1, E // 8 // 2))) if E % 8 == 0 and E >= 64 \
                else fused_topk(logits, topk, True)
            top = StandardTopKOutput(w, ids, None)

            def layer():
                routed = moe(x, top)
                gu, _ = sh_gate_up(x)
                shared, _ = sh_down(ops.silu_and_mul_quant_fp8(gu, 128))
                return routed + shared

            return layer

        def compare(T):
            x = torch.randn(T, H, device=dev, generator=gen).bfloat16()
            w, ids = biased_grouped_topk(torch.randn(T, E, device=dev, generator=gen), None, topk, True, 8, 4)
            return grouped_vs_reference(moe.w13_weight.data, moe.w13_weight_scale_inv.data, moe.w2_weight.data,
                                        moe.w2_weight_scale_inv.data, x, ids, w, dev)

        layer_for.compare = compare
        return layer_for

    # sizes that take the gather form at this rank count have no host synchronisation: they are replayed from CUDA
    # graphs as well, alone and expert-parallel (graph against graph)
    graphed = [T for T in sizes if T <= 512 and (world == 1 or T * world <= GATHER_BELOW)]
    if world > 1:
        layer_for = build(1)
        for T in sizes:
            res[str(T)]["ms_1gpu_eager"] = _time(layer_for(T), 10, 3, world, dev)
            if T in graphed:
                res[str(T)]["ms_1gpu_graph"] = _time_graph_alone(layer_for(T), 10, 3, world, dev)
        del layer_for
        torch.cuda.empty_cache()
    layer_for = build(world)
    for T in sizes:
        layer = layer_for(T)
        ms = _time(layer, 10, 3, world, dev)
        r = res[str(T)]
        r["ms_eager"] = r["ms"] = ms
        if world > 1:
            r["efficiency_vs_1gpu"] = r["ms_1gpu_eager"] / ms
        if T in graphed:
            g_ms = _time_graph(layer, 10, 3, dev, world)
            if g_ms is not None:
                r["launch"] = "cuda graph"
                r["ms"] = g_ms
                if world > 1 and r.get("ms_1gpu_graph"):
                    r["efficiency_vs_1gpu"] = r["ms_1gpu_graph"] / g_ms
        flops = 6.0 * T * topk * H * I + 6.0 * T * H * I
        r.update({"tokens_per_s": world * T / r["ms"] * 1e3, "tflops_per_gpu": flops / r["ms"] / 1e9})
    if world == 1 and not reduced:
        cmp_ = layer_for.compare(max(sizes))
        if cmp_ is not None:
            res[str(max(sizes))]["grouped_gemms_vs_reference_kernel"] = cmp_
    out = {"config": "BASELINE config 3: DeepSeek-V3 MoE, 256 routed experts + 1 shared, hidden 7168, "
                     "moe_intermediate 2048, top-8 grouped sigmoid routing (8 groups, top-4), "
                     "tokens per GPU as keyed; expert-parallel with NCCL all-to-all dispatch/combine (batches of at "
                     f"most {GATHER_BELOW} tokens over all ranks: quantise, all-gather, local experts, reduce-scatter); ms_1gpu_eager = "
                     "the layer with all experts on one GPU of this box in this run",
           "ep": world, "scaling": "weak", "results": res}
    if reduced:
        out["reduced_case"] = {"experts": E, "tokens": list(sizes)}
    if parity is not None:
        out["parity"] = parity
    return {"moe_layer": out}


# ------------------------------------------------------------------------------------------------
# the two expert-grouped GEMMs of a MoE layer call against the reference's own CUDA kernel (one GPU only)
# ------------------------------------------------------------------------------------------------
def grouped_vs_reference(w13, w13_s, w2, w2_s, x, ids, wts, dev, iters=5):
    """This library's grouped kernel and the reference's `fp8_blockwise_scaled_grouped_mm` (its
    sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu compiled here with its one-CTA tile configurations, `make -C oracle
    ref_gpu_moe`) on the same quantised rows and the same expert weights, each in the row order its own pipeline
    uses: 128-row padded expert blocks here, compact expert-major rows there (python/sglang/srt/layers/moe/
    cutlass_moe.py:140-232).  Returns None where the comparator library is not built; not part of any `value`."""
    import os
    lib = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "libsgl_gpu_ref_moe.so")
    if not os.path.exists(lib):
        return None
    try:
        import sglang_b200.sgl_kernel as sk
        from sglang_b200 import ops
        from sglang_b200.srt.layers.moe.fused_moe_triton.fused_moe import _max_padded_rows
        T, H = x.shape
        E, N1, _ = w13.shape
        I, topk = N1 // 2, ids.shape[1]
        R = T * topk
        if R <= 2048 and (H >= 2048 or I >= 2048):
            return {"unavailable": "at most 2048 rows with K >= 2048: the reference routes this shape to its two-CTA "
                                   "cluster configuration, which is left out of the comparator build"}
        torch.ops.load_library(lib)
        ref = torch.ops.sgl_gpu_ref.fp8_blockwise_scaled_grouped_mm
        i32, i64 = dict(dtype=torch.int32, device=dev), dict(dtype=torch.int64, device=dev)
        offs, ps1, ps2 = torch.empty(E + 1, **i32), torch.empty(E, 3, **i32), torch.empty(E, 3, **i32)
        a_map, c_map = torch.empty(R, **i32), torch.empty(R, **i32)
        sk.prepare_moe_input(ids, offs, ps1, ps2, a_map, c_map, E, I, H)
        if int(ps1[:, 0].min()) == 0:
            return {"unavailable": "an expert without rows in this batch; the comparator is only run on batches that "
                                   "give every expert at least one row"}
        xq, xs = ops.per_token_group_quant_fp8(x, 128)
        rep_a, rep_s = sk.shuffle_rows(xq, a_map, (R, H)), sk.shuffle_rows(xs, a_map, (R, H // 128))
        c1 = torch.empty(R, 2 * I, device=dev, dtype=torch.bfloat16)
        c2 = torch.empty(R, H, device=dev, dtype=torch.bfloat16)
        ptrs = [torch.empty(E, **i64) for _ in range(5)]
        ab1, cs1 = torch.full((E,), H, **i64), torch.full((E,), 2 * I, **i64)
        ab2, cs2 = torch.full((E,), I, **i64), torch.full((E,), H, **i64)
        lay_a, lay_b = torch.empty(E, 5, **i32), torch.empty(E, 5, **i32)
        # The reference allocates 90 000 bytes (fp8.py:1196), enough for the CUTLASS it pins.  The CUTLASS this
        # comparator is compiled against keeps 8 + epilogue stages + 2 tensor-map copies per SM for a grouped kernel
        # (about 0.3 MB on 148 SMs) and does not check the size it is given: a larger workspace is passed.
        work = torch.empty(4 << 20, device=dev, dtype=torch.uint8)
        w13_t, w13_st, w2_t, w2_st = w13.transpose(1, 2), w13_s.transpose(1, 2), w2.transpose(1, 2), w2_s.transpose(1, 2)

        def ref1():
            ref(c1, *ptrs, rep_a, w13_t, rep_s, w13_st, ab1, ab1, cs1, lay_a, lay_b, ps1, offs[:-1], work)

        ref1()
        inter_q, inter_s = ops.per_token_group_quant_fp8(sk.silu_and_mul(c1), 128)

        def ref2():
            ref(c2, *ptrs, inter_q, w2_t, inter_s, w2_st, ab2, ab2, cs2, lay_a, lay_b, ps2, offs[:-1], work)

        sorted_ids, expert_ids, post = ops.moe_align_block_size(ids, ops.ALIGN_BLOCK, E)
        a1, a1s = ops.gather_rows_fp8(xq, xs, sorted_ids, post, R, topk, _max_padded_rows(R, E, ops.ALIGN_BLOCK))
        ic1 = torch.empty(a1.shape[0], 2 * I, device=dev, dtype=torch.bfloat16)

        def mine1():
            ops.grouped_block_fp8_matmul(a1, a1s, w13, w13_s, sorted_ids, expert_ids, post, numel=R, scatter=False,
                                         out=ic1)

        mine1()
        a2, a2s = ops.silu_and_mul_quant_fp8(ic1, 128, num_rows=post)
        o2 = torch.empty(R, H, device=dev, dtype=torch.bfloat16)

        def mine2(weights=wts):
            ops.grouped_block_fp8_matmul(a2, a2s, w2, w2_s, sorted_ids, expert_ids, post, numel=R, scatter=True,
                                         row_weights=weights, out=o2)

        # parity of the two kernels on these inputs: row p of the padded order is flat slot sorted_ids[p], which the
        # reference's order holds at row c_map[slot]
        ref2()
        mine2(None)
        n_pad = int(post.item())
        slot = sorted_ids[:n_pad].long()
        valid = slot < R
        same1 = bool(torch.equal(ic1[:n_pad][valid].view(torch.int16), c1[c_map[slot[valid]].long()].view(torch.int16)))
        same2 = bool(torch.equal(o2.view(torch.int16), c2[c_map.long()].view(torch.int16)))
        close2 = bool(torch.allclose(o2.float(), c2[c_map.long()].float(), rtol=2 ** -6, atol=1e-2))
        fl1, fl2 = 2.0 * R * 2 * I * H, 2.0 * R * H * I
        out = {"rows": R, "experts": E,
               "reference_kernel": "sgl-kernel fp8_blockwise_scaled_grouped_mm, one-CTA configurations "
                                   "(128x128x128 tiles for K >= 2048, 64x128x128 below)",
               "bit_identical": {"gemm1": same1, "gemm2": same2}, "gemm2_close": close2}
        for name, mine, theirs, fl in (("gemm1", mine1, ref1, fl1), ("gemm2", mine2, ref2, fl2)):
            ms, ms_ref = _time(mine, iters, 3, 1, dev), _time(theirs, iters, 3, 1, dev)
            out[name] = {"ms": ms, "ref_ms": ms_ref, "tflops": fl / ms / 1e9, "ref_tflops": fl / ms_ref / 1e9}
        return out
    except Exception as e:  # the comparator is optional: never let it break the section
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


# ------------------------------------------------------------------------------------------------
# config 4: Qwen3-30B-A3B-shaped MoE layer under Zipf-skewed expert popularity
# ------------------------------------------------------------------------------------------------


def moe_layer_skewed(args, ctx, peaks):
    """128 experts, hidden 2048, moe_intermediate 768, top-8 softmax routing; the logits carry log(p_e) with
    p_e ~ rank^-1.2 over a seeded permutation of the experts.  Reports the layer time (max over ranks), this
    rank's own time and the spread of tokens per local expert, i.e. the load-imbalance tail.  With more than one
    rank the whole layer (all experts) is first timed on every GPU by itself (`ms_1gpu_eager`), then the
    expert-parallel layer with the static block placement (`ms`), then with redundant copies of the hottest experts on
    every rank and the other experts packed onto the ranks by load (`ms_redundant`: `srt/eplb`, eight copies per
    rank, chosen from the routed-row counts of the batch itself summed over the ranks; a hot expert's rows are served
    by the sender's own copy and never cross NVLink)."""
    from sglang_b200.srt.distributed import initialize_model_parallel
    from sglang_b200.srt.eplb import ExpertLocationMetadata
    from sglang_b200.srt.layers.moe.fused_moe_triton.layer import FusedMoE
    from sglang_b200.srt.layers.moe.token_dispatcher import StandardTopKOutput
    from sglang_b200.srt.layers.moe.topk import fused_topk
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
    rank, world, dev = ctx
    E, H, I, topk = 128, 2048, 768, 8
    sizes = (32, 1024, 16384)
    redundant_per_rank = 8
    perm = torch.randperm(E, generator=torch.Generator().manual_seed(7))  # the same popularity order on every rank
    logp = torch.empty(E)
    logp[perm] = -1.2 * torch.log(torch.arange(1, E + 1, dtype=torch.float32))
    logp = logp.to(dev)
    res = {str(T): {} for T in sizes}

    def routing(T, gen):
        x = torch.randn(T, H, device=dev, generator=gen).bfloat16()
        logits = torch.randn(T, E, device=dev, generator=gen) + logp
        w, ids = fused_topk(logits, topk, True)
        counts = torch.bincount(ids.flatten().long(), minlength=E).float()
        return x, StandardTopKOutput(w, ids, None), counts

    def build(ep, location=None):
        initialize_model_parallel(1, ep)
        gen = torch.Generator(device=dev).manual_seed(41 + rank)
        moe = FusedMoE(E, H, I, topk, quant_config=Fp8Config(), a2a_backend="nccl", device=dev,
                       equal_tokens_gather_below=GATHER_BELOW, expert_location=location)
        _fill_weight(moe.w13_weight.data, moe.w13_weight_scale_inv.data, gen)
        _fill_weight(moe.w2_weight.data, moe.w2_weight_scale_inv.data, gen)
        return moe

    batches = {}
    gen_in = torch.Generator(device=dev).manual_seed(4100 + rank)
    for T in sizes:
        batches[T] = routing(T, gen_in)
    graphed = [T for T in sizes if T <= 1024 and (world == 1 or T * world <= GATHER_BELOW)]  # (as in the config-3 section)
    if world > 1:
        moe = build(1)
        for T in sizes:
            x, top, _ = batches[T]
            res[str(T)]["ms_1gpu_eager"] = _time(lambda: moe(x, top), 10, 3, world, dev)
            if T in graphed:
                res[str(T)]["ms_1gpu_graph"] = _time_graph_alone(lambda: moe(x, top), 10, 3, world, dev)
        del moe
        torch.cuda.empty_cache()
    moe = build(world)
    for T in sizes:
        x, top, counts = batches[T]
        layer = lambda: moe(x, top)
        ms = _time(layer, 10, 3, world, dev)
        r = res[str(T)]
        r["ms_eager"] = r["ms"] = ms
        if world > 1:
            r["efficiency_vs_1gpu"] = r["ms_1gpu_eager"] / ms
        if T in graphed:
            g_ms = _time_graph(layer, 10, 3, dev, world)
            if g_ms is not None:
                r["launch"] = "cuda graph"
                r["ms"] = g_ms
                if world > 1 and r.get("ms_1gpu_graph"):
                    r["efficiency_vs_1gpu"] = r["ms_1gpu_graph"] / g_ms
        # this rank alone, without the barrier-and-max: the gap to `ms` at EP > 1 is the wait for the busiest rank
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(10):
            layer()
        e1.record()
        torch.cuda.synchronize()
        r.update({"ms_this_rank": e0.elapsed_time(e1) / 10, "tokens_per_s": world * T / r["ms"] * 1e3,
                  "tflops_per_gpu": 6.0 * T * topk * H * I / r["ms"] / 1e9,
                  "routed_per_expert_max_over_mean": float(counts.max() / counts.mean()),
                  "experts_hit": int((counts > 0).sum())})
    if world == 1:
        x, top, _ = batches[max(sizes)]
        cmp_ = grouped_vs_reference(moe.w13_weight.data, moe.w13_weight_scale_inv.data, moe.w2_weight.data,
                                    moe.w2_weight_scale_inv.data, x, top[1], top[0], dev)
        if cmp_ is not None:
            res[str(max(sizes))]["grouped_gemms_vs_reference_kernel"] = cmp_
    del moe
    torch.cuda.empty_cache()
    if world > 1:
        import torch.distributed as dist
        for T in sizes:
            x, top, counts = batches[T]
            total = counts.clone()
            dist.all_reduce(total)
            loc = ExpertLocationMetadata.init_by_load(total, world, rank, redundant_per_rank)
            moe = build(world, loc)
            ms = _time(lambda: moe(x, top), 10, 3, world, dev)
            r = res[str(T)]
            r["ms_redundant"] = ms
            r["efficiency_vs_1gpu_redundant"] = r["ms_1gpu_eager"] / ms
            # share of this rank's routed rows that its own copies serve
            hot = loc.physical_to_logical_map[loc.num_local_physical_experts - redundant_per_rank: loc.num_local_physical_experts]
            r["rows_served_by_own_copies"] = float(counts[hot.long()].sum() / counts.sum())
            del moe
            torch.cuda.empty_cache()
    return {"moe_layer_skewed": {"config": "BASELINE config 4: Qwen3-30B-A3B MoE, 128 experts, hidden 2048, "
                                           "moe_intermediate 768, top-8 softmax routing, Zipf(1.2) expert popularity, "
                                           "tokens per GPU as keyed; ms = static block placement, ms_redundant = eight "
                                           "redundant copies of the hottest experts on every rank",
                                 "ep": world, "scaling": "weak", "redundant_experts_per_rank": redundant_per_rank,
                                 "results": res}}


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


# ------------------------------------------------------------------------------------------------
# parity of the sharded paths, checked inside the run (no second GPU is needed to see the result: it is part of
# the JSON line, and a mismatch fails the run)
# ------------------------------------------------------------------------------------------------


class ParityError(AssertionError):
    pass


def _close(out: torch.Tensor, ref: torch.Tensor, what: str, rtol=2e-2, atol=2e-2, min_cos=0.9995):
    """The tolerance of the multi-GPU tests: |out - ref| <= atol + rtol |ref| everywhere, cosine >= min_cos."""
    o, r = out.double(), ref.double()
    bad = (o - r).abs() > atol + rtol * r.abs()
    den = (o * o).sum().sqrt() * (r * r).sum().sqrt()
    cos = float((o * r).sum() / den) if float(den) > 0 else 1.0
    if bool(bad.any()) or cos < min_cos or not bool(torch.isfinite(o).all()):
        raise ParityError(f"{what}: {int(bad.sum())} of {bad.numel()} elements outside rtol {rtol} / atol {atol}, "
                          f"cosine {cos:.6f} (needs {min_cos}), max |diff| {float((o - r).abs().max()):.4g}")
    return cos


def _same_on_all_ranks(t: torch.Tensor, world: int, what: str):
    import torch.distributed as dist
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous())
    for r, q in enumerate(parts):
        if not torch.equal(q, parts[0]):
            raise ParityError(f"{what}: rank {r} differs from rank 0 bit for bit")


def tp_parity(ctx):
    """A small tensor-parallel MLP (gate_up column-parallel -> silu_and_mul + quantiser -> down row-parallel) against
    the same layer computed on this GPU alone from the unsharded weights; with the fused all-reduce, every rank's
    rows bit-identical, and at two ranks bit-identical to GEMM + NCCL."""
    from sglang_b200 import ops
    from sglang_b200.srt.distributed import destroy_model_parallel, enable_fused_row_parallel, initialize_model_parallel
    from sglang_b200.srt.distributed.fused_row_parallel import comm_status
    from sglang_b200.srt.layers.linear import MergedColumnParallelLinear, RowParallelLinear
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
    from bench import make_block_fp8_weight
    rank, world, dev = ctx
    initialize_model_parallel(world, world)
    cfg = Fp8Config()
    H, I = 1024, 2048
    gen = torch.Generator(device=dev).manual_seed(97)  # the same full weights and tokens on every rank
    w1q, w1s = make_block_fp8_weight(2 * I, H, dev, gen)
    w2q, w2s = make_block_fp8_weight(H, I, dev, gen)
    gate_up = MergedColumnParallelLinear(H, [I, I], quant_config=cfg, device=dev)
    down = RowParallelLinear(I, H, quant_config=cfg, device=dev)
    gate_up.load_full_weight(w1q, w1s)
    down.load_full_weight(w2q, w2s)
    sizes = (70, 128 * world + 44, 4 * 128 * world)
    xs = [torch.randn(M, H, device=dev, generator=gen).bfloat16() for M in sizes]

    def alone(x):
        xq, xsc = ops.per_token_group_quant_fp8(x, 128)
        gu = ops.w8a8_block_fp8_matmul(xq, w1q, xsc, w1s, [128, 128], torch.bfloat16)
        hq, hs = ops.silu_and_mul_quant_fp8(gu, 128)
        return ops.w8a8_block_fp8_matmul(hq, w2q, hs, w2s, [128, 128], torch.bfloat16)

    def sharded(x):
        gu, _ = gate_up(x)
        y, _ = down(ops.silu_and_mul_quant_fp8(gu, 128))
        return y

    refs = [alone(x) for x in xs]
    nccl = [sharded(x).clone() for x in xs]
    comm = enable_fused_row_parallel(max(sizes) * H)
    fused = [sharded(x).clone() for x in xs]
    fused2 = [sharded(x).clone() for x in xs]  # flags and staging are reused by later calls
    torch.cuda.synchronize()
    cos = 1.0
    for M, r, a, b, b2 in zip(sizes, refs, nccl, fused, fused2):
        cos = min(cos, _close(a, r, f"TP layer, NCCL all-reduce, M={M}"), _close(b, r, f"TP layer, fused all-reduce, M={M}"))
        if not torch.equal(b, b2):
            raise ParityError(f"TP layer, fused all-reduce, M={M}: a repeated call differs")
        if comm.supports(M, H):
            _same_on_all_ranks(b, world, f"TP layer, fused all-reduce, M={M}")
            if world == 2 and not torch.equal(a, b):
                raise ParityError(f"TP layer, M={M}: fused all-reduce differs from GEMM + NCCL at two ranks")
    status = (ops.gemm_status(), comm_status())
    destroy_model_parallel()
    if status != (0, 0):
        raise ParityError(f"TP parity: status words {status}")
    return {"ok": True, "min_cosine": cos, "sizes": list(sizes)}


def ep_parity(ctx):
    """A small expert-parallel MoE layer in its three forms (all-to-all, gather, replicate + all-reduce) against
    fused_experts_impl on this GPU alone with all experts."""
    from sglang_b200 import ops
    from sglang_b200.srt.distributed import initialize_model_parallel
    from sglang_b200.srt.layers.moe.fused_moe_triton.fused_moe import fused_experts_impl
    from sglang_b200.srt.layers.moe.fused_moe_triton.layer import FusedMoE
    from sglang_b200.srt.layers.moe.token_dispatcher import StandardTopKOutput
    from sglang_b200.srt.layers.moe.topk import fused_topk
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
    from bench import make_block_fp8_weight
    rank, world, dev = ctx
    initialize_model_parallel(1, world)
    E, H, I, topk = 16, 512, 256, 2
    gen = torch.Generator(device=dev).manual_seed(131)  # the same full weights on every rank
    w13q, w13s = make_block_fp8_weight(2 * I, H, dev, gen, std=0.05, experts=E)
    w2q, w2s = make_block_fp8_weight(H, I, dev, gen, std=0.05, experts=E)
    gen_r = torch.Generator(device=dev).manual_seed(1000 + rank)  # this rank's own tokens
    cos = 1.0
    import torch.distributed as dist
    from sglang_b200.srt.eplb import ExpertLocationMetadata
    for form, T in (("a2a", 33 + rank), ("gather", 32), ("allreduce", 32), ("a2a + redundant hot experts", 33 + rank)):
        g = gen if form == "allreduce" else gen_r  # the replicate form holds the same tokens on every rank
        x = torch.randn(T, H, device=dev, generator=g).bfloat16()
        w, ids = fused_topk(torch.randn(T, E, device=dev, generator=g), topk, True)
        loc = None
        if "redundant" in form:  # the eight most-routed experts on every rank, the other eight packed by load
            count = torch.bincount(ids.flatten().long(), minlength=E).float()
            dist.all_reduce(count)
            loc = ExpertLocationMetadata.init_by_load(count, world, rank, E // 2)
        moe = FusedMoE(E, H, I, topk, quant_config=Fp8Config(), a2a_backend="none" if form == "allreduce" else "nccl",
                       device=dev, equal_tokens_gather_below=1024 if form == "gather" else None, expert_location=loc)
        moe.load_full_weights(w13q, w13s, w2q, w2s)
        out = moe(x, StandardTopKOutput(w, ids, None))
        ref = fused_experts_impl(x, w13q, w2q, w, ids, use_fp8_w8a8=True, w1_scale=w13s, w2_scale=w2s,
                                 block_shape=[128, 128])
        torch.cuda.synchronize()
        cos = min(cos, _close(out, ref, f"EP layer, {form} form, {T} tokens"))
    if ops.gemm_status() != 0:
        raise ParityError("EP parity: a GEMM pipeline wait expired")
    return {"ok": True, "min_cosine": cos}


def sharded_summary(out, world):
    """The sharded layers of one run in a few hundred characters, printed as the LAST key of the JSON line: per size
    the eager time (max over ranks) and its efficiency against the same layer timed on ONE GPU of the same box in
    the same run with the same (eager) protocol: strong scaling t1 / (N tN) for the tensor-parallel layer, weak
    scaling t1 / tN for the expert-parallel layers (tokens per GPU fixed)."""
    s = {}
    tp = out.get("tp_layer", {}).get("results", {})
    for M in ("8192", "2048", "128"):
        r = tp.get(M)
        if r and "ms_eager" in r:
            d = {"ms": round(r["ms_eager"], 4)}
            if "ms_1gpu_eager" in r:
                d["eff"] = round(r["ms_1gpu_eager"] / (world * r["ms_eager"]), 3)
            if r.get("ms_nccl_graph") and r.get("ms_1gpu_graph"):  # both arms replayed from CUDA graphs
                d["ms_g"] = round(r["ms_nccl_graph"], 4)
                d["eff_g"] = round(r["ms_1gpu_graph"] / (world * r["ms_nccl_graph"]), 3)
            s[f"tp_M{M}"] = d
    for key, name, sizes in (("moe_layer", "ep3", ("4096", "64", "1")), ("moe_layer_skewed", "ep4", ("16384", "32"))):
        res = out.get(key, {}).get("results", {})
        for T in sizes:
            r = res.get(T)
            if r and "ms_eager" in r:
                d = {"ms": round(r["ms_eager"], 4)}
                if "ms_1gpu_eager" in r:
                    d["eff"] = round(r["ms_1gpu_eager"] / r["ms_eager"], 3)
                if r.get("launch") == "cuda graph" and r.get("ms_1gpu_graph"):  # both arms replayed from CUDA graphs
                    d["ms_g"] = round(r["ms"], 4)
                    d["eff_g"] = round(r["ms_1gpu_graph"] / r["ms"], 3)
                if "ms_redundant" in r:  # with redundant copies of the hot experts (srt/eplb)
                    d["ms_red"] = round(r["ms_redundant"], 4)
                    d["eff_red"] = round(r["ms_1gpu_eager"] / r["ms_redundant"], 3)
                s[f"{name}_T{T}"] = d
    par = [out.get(k, {}).get("parity") for k in ("tp_layer", "moe_layer")]
    par = [p for p in par if p is not None]
    s["parity"] = (all(p.get("ok") for p in par) if par else None) if world > 1 else None
    s["n_gpus"] = world
    s["protocol"] = "eager launches (ms, eff) or graph replays on both arms (ms_g, eff_g); CUDA events, max over ranks"
    return s


def run(sections, args, ctx, peaks):
    out = {}
    rank, world, dev = ctx
    if "sweep" in sections and world == 1:
        out.update(config0_gpu(args, ctx, peaks))
        out.update(gemm_sweep(args, ctx, peaks))
        torch.cuda.empty_cache()
    if "hbm" in sections and world == 1:
        out.update(hbm_kernels(args, ctx, peaks))
        torch.cuda.empty_cache()
    if "tp" in sections:
        out.update(tp_layer(args, ctx, peaks))
        torch.cuda.empty_cache()
    if "moe" in sections or "moe3" in sections:
        out.update(moe_layer(args, ctx, peaks))
        torch.cuda.empty_cache()
    reduced = getattr(args, "moe_experts", 0) or getattr(args, "moe_tokens", 0)  # (a profiler's reduced case)
    if ("moe" in sections and not reduced) or "moe4" in sections:
        out.update(moe_layer_skewed(args, ctx, peaks))
        torch.cuda.empty_cache()
    if sections & {"tp", "moe", "moe3", "moe4"}:
        out["sharded"] = sharded_summary(out, world)  # last key of the JSON line
    return out
