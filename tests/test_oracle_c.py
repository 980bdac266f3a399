"""oracle/oracle.c (fast C restatement) against oracle/block_fp8_oracle.py and the fixtures."""
import os

import numpy as np

from oracle import block_fp8_oracle as O
from oracle import c_oracle as CO


def test_c_e4m3_encode_exhaustive_ish():
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(300000).astype(np.float32) * 200,
        rng.standard_normal(300000).astype(np.float32) * 0.02,
        O.E4M3_DECODE[:0x7F], -O.E4M3_DECODE[:0x7F], O._E4M3_MID.astype(np.float32), -O._E4M3_MID.astype(np.float32),
        np.nextafter(O._E4M3_MID.astype(np.float32), np.float32(0)), np.nextafter(O._E4M3_MID.astype(np.float32), np.float32(1e9)),
        np.array([0.0, -0.0, 1e-30, 448.0, 449.0, 1e30, -1e30, np.inf, -np.inf], dtype=np.float32),
    ])
    assert np.array_equal(CO.e4m3_encode(x), O.e4m3_encode_rne_sat(x))


def test_c_quant_matches_numpy_and_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "quant_native.npz"))
    for i in range(4):
        code = int(g[f"dtype{i}"])
        q, s = CO.quant(g[f"x{i}"], code)
        x = O.bf16_bits_to_f32(g[f"x{i}"]) if code == 0 else g[f"x{i}"].view(np.float16).astype(np.float32)
        q2, s2 = O.per_token_group_quant_fp8(x)
        assert np.array_equal(q, q2) and np.array_equal(s.view(np.uint32), s2.view(np.uint32))
        assert np.array_equal(q, g[f"q{i}"])
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((64, 1024)) * rng.choice([1e-3, 1, 50], size=(64, 1))).astype(np.float32)
    q, s = CO.quant(x, 2)
    q2, s2 = O.per_token_group_quant_fp8(x)
    assert np.array_equal(q, q2) and np.array_equal(s, s2)


def test_c_moe_align_matches_numpy():
    rng = np.random.default_rng(2)
    for (T, topk, E, block) in [(1, 8, 256, 128), (77, 8, 64, 32), (4096, 8, 256, 128), (300, 6, 257, 64), (0, 8, 8, 16)]:
        ids = rng.integers(-1, E, size=(T, topk)).astype(np.int32)
        a = CO.moe_align(ids, block, E)
        b = O.moe_align_block_size(ids, block, E)
        P = int(b[2][0])
        assert a[2][0] == P
        assert np.array_equal(a[0][:P], b[0][:P])
        assert np.array_equal(a[1][: P // block], b[1][: P // block])


def test_c_block_gemm_matches_numpy(golden_dir):
    g = np.load(os.path.join(golden_dir, "gemm_native.npz"))
    c = O.bf16_bits_to_f32(CO.block_gemm(g["xq"], g["xs"], g["wq"], g["ws"]))
    ref = O.w8a8_block_fp8_matmul(g["xq"], g["wq"], g["xs"], g["ws"])
    np.testing.assert_allclose(c, ref, rtol=1e-2, atol=1e-3)


def test_c_silu_and_sum_match_numpy():
    rng = np.random.default_rng(4)
    x = O.f32_to_bf16_bits((rng.standard_normal((19, 256)) * 3).astype(np.float32))
    h = O.bf16_bits_to_f32(CO.silu_and_mul(x))
    ref = O.silu_and_mul(O.bf16_bits_to_f32(x))
    assert (np.abs(h - ref) <= np.abs(ref) * 2.0**-7).all() and (h != ref).mean() < 1e-2
    y = O.f32_to_bf16_bits(rng.standard_normal((7, 8, 128)).astype(np.float32))
    assert np.array_equal(O.bf16_bits_to_f32(CO.moe_sum_reduce(y, 2.5)), O.moe_sum_reduce(O.bf16_bits_to_f32(y), 2.5))
