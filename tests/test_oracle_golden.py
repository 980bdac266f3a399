"""The oracle against fixtures produced by the reference's own torch-native
functions (tests/golden/make_golden.py) and its documented known answers."""
import os

import numpy as np
import pytest

from oracle import block_fp8_oracle as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def _fp16_bits_to_f32(bits):
    return bits.view(np.float16).astype(np.float32)


def test_e4m3_roundtrip_all_codes():
    codes = np.arange(256, dtype=np.uint8)
    vals = O.e4m3_decode(codes)
    finite = ~np.isnan(vals)
    back = O.e4m3_encode_rne_sat(vals[finite])
    expect = codes[finite].copy()
    expect[expect == 0x80] = 0x80  # -0 keeps its sign
    assert np.array_equal(back, expect)
    assert vals[0x7E] == 448.0 and vals[0x08] == 2.0**-6 and vals[0x01] == 2.0**-9


def test_e4m3_ties_to_even_and_saturation():
    # halfway between 0x7D (416) and 0x7E (448) -> even mantissa (0x7E); 464 saturates to 448
    x = np.array([432.0, 464.0, 1e9, -1e9, 2.0**-10, 2.0**-10 * 1.0001, 3 * 2.0**-10], dtype=np.float32)
    assert list(O.e4m3_encode_rne_sat(x)) == [0x7E, 0x7E, 0x7E, 0xFE, 0x00, 0x01, 0x02]


def test_e4m3_matches_torch_cast():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * 100,
        rng.standard_normal(200000).astype(np.float32) * 0.01,
        O.E4M3_DECODE[:0x7F], (O._E4M3_MID).astype(np.float32),
    ])
    x = np.clip(x, -448, 448).astype(np.float32)
    t = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode_rne_sat(x), t)


def test_bf16_round_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(100000) * 10).astype(np.float32)
    t = torch.from_numpy(x).bfloat16().float().numpy()
    assert np.array_equal(O.bf16_round(x), t)


def test_quant_matches_reference_native(golden_dir):
    g = _load(golden_dir, "quant_native.npz")
    for i in range(4):
        bits = g[f"x{i}"]
        x = O.bf16_bits_to_f32(bits) if int(g[f"dtype{i}"]) == 0 else _fp16_bits_to_f32(bits)
        q, s = O.per_token_group_quant_fp8(x, 128)
        # An all-zero group is the one place the reference's variants disagree: the torch-native
        # function clamps with eps rounded to the input dtype, the CUDA kernel
        # (per_token_group_quant_8bit.cu:45,86) uses float32 1e-10f, which the oracle follows.
        zero = np.abs(x.reshape(-1, 128)).max(-1).reshape(s.shape) == 0
        assert np.array_equal(s.view(np.uint32)[~zero], g[f"s{i}"].view(np.uint32)[~zero]), i
        assert np.all(s[zero] == np.float32(1e-10) / np.float32(448.0))
        assert zero.sum() == (1 if i == 1 else 0)
        assert np.array_equal(q, g[f"q{i}"]), i


def test_quant_known_answer_construction(golden_dir):
    # test/srt/quant/test_fp8_kernel.py:89-100: scales must be recovered, codes mismatch < 1e-4
    g = _load(golden_dir, "kat_fp8_kernel.npz")
    q, s = O.per_token_group_quant_fp8(g["A"], 128)
    np.testing.assert_allclose(s, g["A_s"], rtol=1.3e-6, atol=1e-5)
    diff = np.abs(O.e4m3_decode(q) - O.e4m3_decode(g["A_q"])) > 1e-5
    assert diff.mean() < 1e-4


def test_gemm_matches_reference_native(golden_dir):
    g = _load(golden_dir, "gemm_native.npz")
    x = O.bf16_bits_to_f32(g["x"])
    xq, xs = O.per_token_group_quant_fp8(x)
    assert np.array_equal(xq, g["xq"]) and np.array_equal(xs, g["xs"])
    wq, ws = g["wq"], g["ws"]
    c = O.w8a8_block_fp8_matmul(xq, wq, xs, ws)
    ref = O.bf16_bits_to_f32(g["c"])
    # same formula in float32: differences only from summation order inside a 128-block
    np.testing.assert_allclose(c, ref, rtol=1e-2, atol=1e-3)
    assert (c != ref).mean() < 0.05


def test_gemm_known_answer(golden_dir):
    # test/srt/quant/test_fp8_kernel.py:103-122 (atol .5, rtol 1e-4 vs bf16 matmul)
    g = _load(golden_dir, "kat_fp8_kernel.npz")
    c = O.w8a8_block_fp8_matmul(g["A_q"], g["B_q_t"], g["A_s"], g["B_s_t"])
    np.testing.assert_allclose(c, O.bf16_bits_to_f32(g["C_gt"]), atol=0.5, rtol=1e-4)


def test_weight_quant_matches_fixture_recipe(golden_dir):
    torch = pytest.importorskip("torch")
    torch.manual_seed(0)
    torch.randn(17, 512)
    w = (torch.randn(320, 512) * 0.02).numpy()
    g = _load(golden_dir, "gemm_native.npz")
    q, s = O.quant_weight_block_fp8(w)
    assert np.array_equal(q, g["wq"]) and np.array_equal(s, g["ws"])


def test_moe_matches_reference_native(golden_dir):
    g = _load(golden_dir, "moe_native.npz")
    out = O.fused_experts_block_fp8(
        O.bf16_bits_to_f32(g["a"]), g["w1q"], g["w1s"], g["w2q"], g["w2s"], g["topk_w"], g["topk_ids"]
    )
    ref = O.bf16_bits_to_f32(g["out"])
    # the torch-native MoE multiplies by the weight and sums in bf16; the kernels' rounding
    # points (restated by the oracle) differ in the last bf16 bits only
    np.testing.assert_allclose(out, ref, rtol=2e-2, atol=2e-2)
    cos = (out * ref).sum() / np.sqrt((out * out).sum() * (ref * ref).sum())
    assert cos > 0.9999


def test_moe_align_documented_example():
    # python/sglang/srt/layers/moe/fused_moe_triton/moe_align_block_size.py:43-55
    ids = np.array([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=np.int32)
    s, e, n = O.moe_align_block_size(ids, 4, 5)
    assert n[0] == 16
    assert list(s[:16]) == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    assert list(e[:4]) == [1, 2, 3, 4]


def test_moe_align_properties_and_filtered_bucket():
    rng = np.random.default_rng(3)
    for (T, topk, E, block) in [(1, 8, 256, 128), (33, 8, 64, 32), (512, 8, 256, 128), (100, 4, 257, 64), (0, 8, 16, 16)]:
        ids = rng.integers(-1, E, size=(T, topk)).astype(np.int32)
        s, e, n = O.moe_align_block_size(ids, block, E)
        P = int(n[0])
        assert P % block == 0
        flat = ids.reshape(-1)
        numel = flat.size
        valid = s[:P][s[:P] < numel]
        assert np.array_equal(np.sort(valid), np.arange(numel))
        for b in range(P // block):
            seg = s[b * block : (b + 1) * block]
            real = seg[seg < numel]
            assert np.all(flat[real] == e[b])
            assert np.all(np.diff(real) > 0)  # stable: ascending flat index
            assert np.all(seg[len(real):] == numel)
        assert np.all(np.diff(e[: P // block]) >= 0)
        counts = np.bincount(flat + 1, minlength=E + 1)
        assert P == int(((counts + block - 1) // block * block).sum())


def test_silu_and_mul_matches_torch_bf16():
    torch = pytest.importorskip("torch")
    torch.manual_seed(5)
    x = torch.randn(37, 512).bfloat16() * 3
    h = O.silu_and_mul(x.float().numpy())
    d = 256
    ref = (torch.nn.functional.silu(x[:, :d].float()).bfloat16() * x[:, d:]).float().numpy()
    ulp = np.abs(h - ref) / np.maximum(np.abs(ref), 1e-30)
    assert (ulp < 2 ** -7).all()
    assert (h != ref).mean() < 1e-2


def test_moe_sum_reduce():
    rng = np.random.default_rng(7)
    x = O.bf16_round(rng.standard_normal((5, 8, 64)).astype(np.float32))
    out = O.moe_sum_reduce(x, 2.5)
    np.testing.assert_allclose(out, x.sum(1) * 2.5, rtol=1e-2, atol=1e-2)


# ---- routing: oracle against the reference's torch-native functions (tests/golden/make_golden_topk.py) ----
def _same_picks(ids_a, ids_b):
    return np.array_equal(np.sort(ids_a, axis=1), np.sort(ids_b, axis=1))


def _weights_by_id(w, ids):
    order = np.argsort(ids, axis=1, kind="stable")
    return np.take_along_axis(w, order, axis=1)


def test_oracle_fused_gate_matches_reference_native(golden_dir):
    from oracle import block_fp8_oracle as O

    z = _load(golden_dir, "topk_native.npz")
    for i in range(3):
        for apply in (0, 1):
            tag = f"g{i}a{apply}"
            E, G, tg, k = (int(v) for v in z[tag + "_cfg"])
            w, ids = O.moe_fused_gate(z[tag + "_x"], z[tag + "_bias"], G, tg, k, 0, 2.5, bool(apply), dtype="f32")
            # the reference's topk is unsorted: compare the picked sets and the weight attached to each id
            assert _same_picks(ids, z[tag + "_ids"]), tag
            np.testing.assert_allclose(_weights_by_id(w, ids), _weights_by_id(z[tag + "_w"], z[tag + "_ids"]),
                                       rtol=2e-6, atol=1e-7, err_msg=tag)


def test_oracle_topk_softmax_matches_reference_native(golden_dir):
    from oracle import block_fp8_oracle as O

    z = _load(golden_dir, "topk_native.npz")
    for i in range(4):
        for renorm in (0, 1):
            tag = f"s{i}r{renorm}"
            w, ids = O.topk_softmax(z[tag + "_x"], int(z[tag + "_k"]), bool(renorm))
            assert np.array_equal(ids, z[tag + "_ids"]), tag  # torch.topk sorted: same order, best first
            np.testing.assert_allclose(w, z[tag + "_w"], rtol=3e-6, atol=1e-8, err_msg=tag)


def test_oracle_gate_tie_rules():
    from oracle import block_fp8_oracle as O

    # equal scores everywhere: lower groups are kept, lower experts are picked, weights are equal
    x = np.zeros((2, 16), dtype=np.float32)
    w, ids = O.moe_fused_gate(x, np.zeros(16, np.float32), 4, 2, 3)
    assert ids.tolist() == [[0, 1, 2], [0, 1, 2]]
    np.testing.assert_allclose(w, 1.0 / 3.0, rtol=1e-6)
    # fused shared expert: id E, weight 1/factor after normalisation (times the factor when applied)
    w, ids = O.moe_fused_gate(x, np.zeros(16, np.float32), 4, 2, 4, 1, 2.5, False)
    assert ids[0].tolist() == [0, 1, 2, 16]
    np.testing.assert_allclose(w[0], [1 / 3, 1 / 3, 1 / 3, 0.4], rtol=1e-6)
    w, _ = O.moe_fused_gate(x, np.zeros(16, np.float32), 4, 2, 4, 1, 2.5, True)
    np.testing.assert_allclose(w[0], [2.5 / 3, 2.5 / 3, 2.5 / 3, 1.0], rtol=1e-6)
    w, ids = O.topk_softmax(np.zeros((1, 8), np.float32), 2, True)
    assert ids.tolist() == [[0, 1]] and np.allclose(w, 0.5)
    b = np.linspace(0, 0.7, 8).astype(np.float32)
    w, ids = O.topk_sigmoid(np.zeros((1, 8), np.float32), 2, False, b)
    assert ids.tolist() == [[7, 6]] and np.allclose(w, 0.5, atol=1e-6)
