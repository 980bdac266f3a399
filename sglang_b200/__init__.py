"""sglang_b200 — B200 (sm_100a) implementation of SGLang's block-wise FP8 W8A8 hot path.

Layout mirrors the reference so that call sites read the same:

    sglang_b200.sgl_kernel                         <-> sgl_kernel (op names, torch.ops.sgl_kernel.*)
    sglang_b200.srt.layers.quantization.fp8        <-> sglang.srt.layers.quantization.fp8
    sglang_b200.srt.layers.quantization.fp8_kernel <-> ....fp8_kernel
    sglang_b200.srt.layers.quantization.fp8_utils  <-> ....fp8_utils
    sglang_b200.srt.layers.moe.*                   <-> sglang.srt.layers.moe.*
    sglang_b200.srt.layers.linear                  <-> sglang.srt.layers.linear (TP linears)
    sglang_b200.srt.distributed                    <-> sglang.srt.distributed (TP / EP groups)

All compute goes through the C ABI in include/sglang_b200.h (sglang_b200/lib/libsglang_b200.so).
"""
__version__ = "0.1.0"
