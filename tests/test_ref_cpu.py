"""The reference's own CPU kernels (oracle/_ref/libsgl_cpu_ref.so: sgl-kernel/csrc/cpu/{gemm_fp8,moe}.cpp compiled
unmodified) against the oracle.  These kernels are the timed CPU baseline of the benchmark; this file checks that the
library built from them computes what the oracle says the path computes.  The CPU path is W8A16: it dequantises the
FP8 weights and multiplies bf16 activations (it never quantises activations), so the linear is compared with the product of the
oracle's dequantised weights (rtol / atol 3e-2: bf16 rounding of the kernel's partial sums) and the MoE layer, whose
oracle also quantises activations, at rtol / atol 3e-2 and cosine >= 0.999.  Skipped where the library was not built or the host lacks AMX / AVX512-BF16.
"""
import os

import numpy as np
import pytest
import torch

from oracle import block_fp8_oracle as O
from tests.util import cosine, make_act, make_weight, to_f32_np

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libsgl_cpu_ref.so")


def _host_ok():
    try:
        flags = open("/proc/cpuinfo").read()
    except OSError:
        return False
    return all(f in flags for f in ("avx512f", "avx512_bf16", "amx_bf16"))


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libsgl_cpu_ref.so not built (make -C oracle ref)")
    if not _host_ok():
        pytest.skip("host CPU lacks AVX512-BF16 / AMX")
    torch.ops.load_library(LIB)
    return torch.ops.sgl_cpu_ref


def _dequant(q, s):
    """[.., N, K] codes and [.., N/128, K/128] scales -> float32 weights."""
    w = O.e4m3_decode(q).astype(np.float32)
    sc = np.repeat(np.repeat(s, 128, axis=-2), 128, axis=-1)[..., : w.shape[-2], : w.shape[-1]]
    return w * sc


@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (7, 512, 1024)])
def test_fp8_scaled_mm_cpu_matches_oracle(ref, M, N, K):
    wq, ws = make_weight(N, K, 1)
    x = make_act(M, K, 2, outliers=False)
    wt = torch.from_numpy(wq).view(torch.float8_e4m3fn)
    y = ref.fp8_scaled_mm_cpu(x, ref.convert_weight_packed(wt), torch.from_numpy(ws), [128, 128], None, torch.bfloat16, True)
    want = to_f32_np(x) @ _dequant(wq, ws).T
    got = to_f32_np(y)
    np.testing.assert_allclose(got, want, rtol=3e-2, atol=3e-2)
    assert cosine(got, want) >= 0.9999
    # the W8A8 result of the path proper differs from it by the activation quantisation only
    assert cosine(got, O.block_fp8_linear(to_f32_np(x), wq, ws)) >= 0.999


def test_fused_experts_cpu_matches_oracle(ref):
    E, H, I, topk, T = 8, 512, 256, 2, 33
    w13q, w13s = make_weight(2 * I, H, 5, std=0.05, experts=E)
    w2q, w2s = make_weight(H, I, 6, std=0.05, experts=E)
    x = make_act(T, H, 7, outliers=False)
    g = torch.Generator().manual_seed(9)
    tw, ti = torch.topk(torch.softmax(torch.randn(T, E, generator=g), -1), topk)
    tw = (tw / tw.sum(-1, keepdim=True)).float()
    ti = ti.to(torch.int32)
    w13 = ref.convert_weight_packed(torch.from_numpy(w13q).view(torch.float8_e4m3fn))
    w2 = ref.convert_weight_packed(torch.from_numpy(w2q).view(torch.float8_e4m3fn))
    y = ref.fused_experts_cpu(x, w13, w2, tw, ti, False, False, True, torch.from_numpy(w13s), torch.from_numpy(w2s),
                              [128, 128], None, None, True)
    got = to_f32_np(y)
    # W8A16 by hand: dequantised weights, bf16 activations, bf16 intermediates
    w13f, w2f, xf = _dequant(w13q, w13s), _dequant(w2q, w2s), to_f32_np(x)
    want = np.zeros((T, H), np.float32)
    for t in range(T):
        for j in range(topk):
            e = int(ti[t, j])
            gu = O.bf16_round(w13f[e] @ xf[t])
            h = O.bf16_round(O.bf16_round(gu[:I] / (1.0 + np.exp(-gu[:I]))) * gu[I:])
            want[t] += float(tw[t, j]) * O.bf16_round(w2f[e] @ h)
    np.testing.assert_allclose(got, want, rtol=3e-2, atol=3e-2)
    assert cosine(got, want) >= 0.9999
    # the W8A8 layer of the path proper differs from it by the two activation quantisations only
    w8a8 = O.fused_experts_block_fp8(xf, w13q, w13s, w2q, w2s, tw.numpy(), ti.numpy(), 1.0)
    assert cosine(got, w8a8) >= 0.999
