"""GPU parity of the quantizer and the elementwise MoE kernels, through the C ABI (bit-exact)."""
import os

import numpy as np
import pytest
import torch

from oracle import block_fp8_oracle as O
from oracle import c_oracle as CO
from tests.util import bf16_bits, codes_to_fp8, fp8_codes, make_act, to_f32_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from sglang_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("tokens", [1, 7, 83, 2048])
@pytest.mark.parametrize("hidden", [128, 512, 4096, 7168])
def test_quant_bf16_bit_exact(ops, tokens, hidden):
    x = make_act(tokens, hidden, tokens * 10000 + hidden)
    q, s = ops.per_token_group_quant_fp8(x.cuda(), 128)
    rq, rs = CO.quant(bf16_bits(x), 0, 128)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), rs.view(np.uint32))
    assert np.array_equal(fp8_codes(q), rq)


@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 0), (torch.float16, 1), (torch.float32, 2)])
def test_quant_groups_and_dtypes(ops, group, dtype, code):
    x = make_act(37, 1024, 1234 + group, dtype=dtype)
    x[3, :group] = 0  # all-zero group -> eps path
    x[5, 7] = 6.0e4 if dtype != torch.bfloat16 else 3.0e38
    q, s = ops.per_token_group_quant_fp8(x.cuda(), group)
    raw = x.numpy() if code == 2 else x.view(torch.int16).numpy().view(np.uint16)
    rq, rs = CO.quant(raw, code, group)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), rs.view(np.uint32))
    assert np.array_equal(fp8_codes(q), rq)


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 0), (torch.float16, 1), (torch.float32, 2)])
def test_quant_special_values(ops, dtype, code):
    # NaN, infinities and signed zeros: a group holding a NaN or an infinity leaves the fast path of the kernel and
    # must still follow the reference arithmetic (NaN-ignoring maximum, clamp that maps a NaN quotient to -448)
    x = make_act(64, 1024, 77, dtype=dtype)
    x[1, 3] = float("nan")
    x[2, 130] = float("inf")
    x[3, 260] = float("-inf")
    x[4, 5] = float("nan")
    x[4, 6] = float("inf")
    x[5, :8] = -0.0
    x[6, 128:256] = -0.0  # an all-zero group of negative zeros
    x[7, 511] = float("nan")
    q, s = ops.per_token_group_quant_fp8(x.cuda(), 128)
    raw = x.numpy() if code == 2 else x.view(torch.int16).numpy().view(np.uint16)
    rq, rs = CO.quant(raw, code, 128)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), rs.view(np.uint32))
    assert np.array_equal(fp8_codes(q), rq)
    assert ops.stream_status() == 0


def test_quant_ragged_tile_edges(ops):
    # sizes around the kernel's 8192-element tiles and its ring of staged tiles
    for tokens, hidden in [(1, 8192), (1, 8192 + 128), (3, 8192 - 128), (5 * 148 * 3 + 1, 8192), (33, 24576 + 384)]:
        x = make_act(tokens, hidden, tokens + hidden)
        q, s = ops.per_token_group_quant_fp8(x.cuda(), 128)
        rq, rs = CO.quant(bf16_bits(x), 0, 128)
        assert np.array_equal(s.cpu().numpy().view(np.uint32), rs.view(np.uint32))
        assert np.array_equal(fp8_codes(q), rq)
    assert ops.stream_status() == 0


def test_quant_column_major_scales(ops):
    x = make_act(83, 2048, 5)
    q, s = ops.per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True)
    assert s.shape == (83, 16) and s.stride() == (1, 84)
    rq, rs = CO.quant(bf16_bits(x), 0, 128)
    assert np.array_equal(s.cpu().numpy(), rs) and np.array_equal(fp8_codes(q), rq)


def test_quant_golden_fixtures(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "quant_native.npz"))
    for i in range(4):
        dt = torch.bfloat16 if int(g[f"dtype{i}"]) == 0 else torch.float16
        x = torch.from_numpy(g[f"x{i}"].view(np.int16)).view(dt).cuda()
        q, s = ops.per_token_group_quant_fp8(x, 128)
        assert np.array_equal(fp8_codes(q), g[f"q{i}"])
        xs = np.abs(to_f32_np(x).reshape(-1, 128)).max(-1).reshape(s.shape)
        nz = xs != 0
        assert np.array_equal(s.cpu().numpy()[nz], g[f"s{i}"][nz])
    k = np.load(os.path.join(golden_dir, "kat_fp8_kernel.npz"))
    q, s = ops.per_token_group_quant_fp8(torch.from_numpy(k["A"]).cuda(), 128)
    np.testing.assert_allclose(s.cpu().numpy(), k["A_s"], rtol=1.3e-6, atol=1e-5)
    assert (np.abs(O.e4m3_decode(fp8_codes(q)) - O.e4m3_decode(k["A_q"])) > 1e-5).mean() < 1e-4


def test_quant_large_round_trip_property(ops):
    # full BASELINE size (8192 x 18432): scale * 448 recovers amax exactly enough, dequantised error bounded
    x = torch.randn(8192, 18432, device="cuda", dtype=torch.bfloat16)
    q, s = ops.per_token_group_quant_fp8(x, 128)
    amax = x.view(8192, -1, 128).abs().amax(-1).float()
    # tensor / tensor is a true IEEE division on the device (tensor / python-scalar becomes a reciprocal multiply)
    assert torch.equal(s, amax.clamp(min=1e-10) / torch.full_like(amax, 448.0))
    deq = q.view(8192, -1, 128).float() * s.unsqueeze(-1)
    err = (deq - x.view(8192, -1, 128).float()).abs()
    assert bool((err <= amax.unsqueeze(-1) * (2.0 ** -4) + 1e-12).all())


def test_quant_rejects_bad_shapes(ops):
    x = torch.zeros(4, 100, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.per_token_group_quant_fp8(x, 128)
    q, s = ops.per_token_group_quant_fp8(torch.zeros(0, 256, device="cuda", dtype=torch.bfloat16), 128)
    assert q.shape == (0, 256) and s.shape == (0, 2)


@pytest.mark.parametrize("rows,d", [(1, 128), (19, 768), (300, 2048)])
def test_silu_and_mul(ops, rows, d):
    x = (make_act(rows, 2 * d, rows + d, outliers=False) * 3).cuda()
    out = torch.empty(rows, d, device="cuda", dtype=torch.bfloat16)
    ops.silu_and_mul_out(out, x)
    ref = O.bf16_bits_to_f32(CO.silu_and_mul(bf16_bits(x)))
    got = to_f32_np(out)
    # expf differs between libm and the device by an ulp or two: after bf16 rounding almost all agree
    assert (np.abs(got - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-30).all()
    assert (got != ref).mean() < 5e-3


@pytest.mark.parametrize("rows,d", [(1, 128), (19, 768), (300, 2048), (2777, 768), (37, 14336), (4500, 2048), (3, 8192)])
def test_silu_mul_quant_equals_unfused_pipeline(ops, rows, d):
    x = (make_act(rows, 2 * d, 77 + rows, outliers=False) * 3).cuda()
    h = torch.empty(rows, d, device="cuda", dtype=torch.bfloat16)
    ops.silu_and_mul_out(h, x)
    q_ref, s_ref = ops.per_token_group_quant_fp8(h, 128)
    q, s = ops.silu_and_mul_quant_fp8(x, 128)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s, s_ref)
    # and the quantiser half is bit-exact against the oracle given the same h
    rq, rs = CO.quant(bf16_bits(h), 0, 128)
    assert np.array_equal(fp8_codes(q), rq) and np.array_equal(s.cpu().numpy(), rs)
    # row limit read from device memory
    lim = torch.tensor([rows // 2], device="cuda", dtype=torch.int32)
    q2, s2 = ops.silu_and_mul_quant_fp8(x, 128, num_rows=lim)
    assert torch.equal(q2.view(torch.uint8)[: rows // 2], q.view(torch.uint8)[: rows // 2])
    assert ops.stream_status() == 0


@pytest.mark.parametrize("E,T_pad,d,group", [(4, 64, 2048, 128), (32, 128, 768, 128), (3, 40, 256, 64), (1, 5, 128, 128),
                                             (256, 16, 512, 128), (8, 200, 7168, 128), (1000, 8, 128, 32)])
def test_silu_mul_masked_quant(ops, E, T_pad, d, group):
    """`silu_and_mul_masked_post_quant_fwd` (python/sglang/srt/layers/moe/ep_moe/kernels.py:287-420, float32 scales):
    the first masked_m[e] rows of every expert equal the unfused pair silu_and_mul + quantizer bit for bit, and the
    quantizer half equals the oracle on the same h; rows at or beyond masked_m[e] keep what the outputs held."""
    from sglang_b200.srt.layers.moe.ep_moe.kernels import silu_and_mul_masked_post_quant_fwd
    g = torch.Generator().manual_seed(E * 7 + T_pad)
    masked_m = torch.randint(0, T_pad + 1, (E,), generator=g, dtype=torch.int32)
    masked_m[0] = T_pad                      # a full expert
    if E > 2:
        masked_m[1], masked_m[E - 1] = 0, 1  # an empty one; a single row in the last
    x = (make_act(E * T_pad, 2 * d, 5 + E, outliers=False) * 3).cuda().view(E, T_pad, 2 * d)
    q = torch.full((E, T_pad, d), 0x55, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    s = torch.full((E, T_pad, d // group), -7.0, device="cuda")
    silu_and_mul_masked_post_quant_fwd(x, q, s, group, masked_m.cuda())
    h = torch.empty(E * T_pad, d, device="cuda", dtype=torch.bfloat16)
    ops.silu_and_mul_out(h, x.view(E * T_pad, 2 * d))
    q_ref, s_ref = ops.per_token_group_quant_fp8(h, group)
    rq, rs = CO.quant(bf16_bits(h), 0, group)
    valid = (torch.arange(T_pad)[None, :] < masked_m[:, None]).cuda()          # [E, T_pad]
    qb, sb = q.view(torch.uint8), s
    assert torch.equal(qb[valid], q_ref.view(torch.uint8).view(E, T_pad, d)[valid])
    assert torch.equal(sb[valid], s_ref.view(E, T_pad, -1)[valid])
    v = valid.cpu().numpy().reshape(-1)
    assert np.array_equal(fp8_codes(q).reshape(E * T_pad, d)[v], rq[v])
    assert np.array_equal(s.cpu().numpy().reshape(E * T_pad, -1)[v], rs[v])
    assert bool((qb[~valid] == 0x55).all()) and bool((sb[~valid] == -7.0).all())
    assert ops.stream_status() == 0


def test_silu_mul_masked_quant_rejects(ops):
    from sglang_b200.srt.layers.moe.ep_moe.kernels import silu_and_mul_masked_post_quant_fwd
    x = torch.zeros(2, 4, 256, device="cuda", dtype=torch.bfloat16)
    q = torch.zeros(2, 4, 128, device="cuda", dtype=torch.float8_e4m3fn)
    s = torch.zeros(2, 4, 1, device="cuda")
    m = torch.zeros(2, device="cuda", dtype=torch.int32)
    with pytest.raises(NotImplementedError):
        silu_and_mul_masked_post_quant_fwd(x, q, s, 128, m, scale_ue8m0=True)
    with pytest.raises(RuntimeError):
        ops.silu_and_mul_masked_quant_fp8_out(x, q, torch.zeros(2, 4, 2, device="cuda"), m, 128)
    with pytest.raises(RuntimeError):
        ops.silu_and_mul_masked_quant_fp8_out(x, q, s, torch.zeros(3, device="cuda", dtype=torch.int32), 128)


@pytest.mark.parametrize("tokens,topk,hidden", [(1, 8, 7168), (33, 8, 2048), (512, 6, 1024), (5, 1, 128)])
def test_moe_sum_reduce_bit_exact(ops, tokens, topk, hidden):
    x = make_act(tokens * topk, hidden, 99 + tokens, outliers=False).view(tokens, topk, hidden).cuda()
    out = torch.empty(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    ops.moe_sum_reduce_out(x, out, 2.5)
    ref = CO.moe_sum_reduce(bf16_bits(x), 2.5)
    assert np.array_equal(bf16_bits(out), ref)


@pytest.mark.parametrize("tokens,per_token,hidden,src_rows", [(1, 2, 7168, 2), (97, 8, 1024, 300), (512, 4, 2048, 1000)])
def test_gather_sum_rows_bit_exact(ops, tokens, per_token, hidden, src_rows):
    """The expert-parallel combine: gathering the rows and summing them with the plain sum-reduce oracle."""
    g = torch.Generator().manual_seed(tokens + per_token)
    src = make_act(src_rows, hidden, 7 + tokens, outliers=False).cuda()
    slot = torch.randint(0, src_rows + 1, (tokens, per_token), generator=g)  # src_rows = "no row"
    slot[0, 0] = src_rows
    out = ops.gather_sum_rows(src, slot.cuda(), 2.5)
    padded = torch.cat([src.cpu(), torch.zeros(1, hidden, dtype=src.dtype)])
    ref = CO.moe_sum_reduce(bf16_bits(padded[slot].contiguous()), 2.5)  # adding a zero row changes nothing
    assert np.array_equal(bf16_bits(out), ref)


def test_gather_rows(ops):
    T, topk, H, E = 50, 4, 512, 16
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(-1, E, (T, topk), generator=g, dtype=torch.int32).cuda()
    q = torch.randint(0, 255, (T, H), generator=g, dtype=torch.uint8).cuda().view(torch.float8_e4m3fn)
    s = torch.rand(T, H // 128, generator=g).cuda()
    sorted_ids, expert_ids, post = ops.moe_align_block_size(ids, 128, E)
    dq, ds = ops.gather_rows_fp8(q, s, sorted_ids, post, T * topk, topk)
    P = int(post.item())
    sid = sorted_ids[:P].cpu().numpy()
    exp_q = np.zeros((P, H), np.uint8)
    exp_s = np.zeros((P, H // 128), np.float32)
    ok = sid < T * topk
    exp_q[ok] = fp8_codes(q)[sid[ok] // topk]
    exp_s[ok] = s.cpu().numpy()[sid[ok] // topk]
    assert np.array_equal(fp8_codes(dq)[:P], exp_q) and np.array_equal(ds.cpu().numpy()[:P], exp_s)
