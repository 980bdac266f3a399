"""GPU parity of the routing kernels (topk_softmax, topk_sigmoid, moe_fused_gate) through the C ABI.

Ids are compared exactly with the oracle, in pick order.  The device exponential and numpy's may differ in the
last float32 bit, which can flip a pick between two experts whose scores are within an ulp (or, for 16-bit
inputs, flip the rounding of one score), so a row may disagree in rare cases: at most 0.5 % of the rows, and the
weights are compared on the rows that agree.  The fixtures produced by the reference's torch-native functions
must be met on every row.
"""
import os

import numpy as np
import pytest
import torch

from oracle import block_fp8_oracle as O

pytestmark = pytest.mark.gpu

NP_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


@pytest.fixture(scope="module")
def ops():
    from sglang_b200 import ops as _ops
    return _ops


def _compare(w, ids, rw, rids, rtol, max_bad_frac=0.005):
    w, ids = w.cpu().numpy(), ids.cpu().numpy()
    assert ids.shape == rids.shape and w.shape == rw.shape
    same = (ids == rids).all(axis=1)
    bad = int((~same).sum())
    assert bad <= max(1, int(max_bad_frac * len(same))) if len(same) > 8 else bad == 0, f"{bad} of {len(same)} rows differ"
    np.testing.assert_allclose(w[same], rw[same], rtol=rtol, atol=1e-7)


@pytest.mark.parametrize("rows", [1, 7, 64, 1000, 4096])
@pytest.mark.parametrize("cfg", [(128, 4, 2, 4), (256, 8, 4, 8), (512, 16, 8, 16), (96, 3, 2, 5), (1024, 32, 4, 8)])
@pytest.mark.parametrize("shared,apply", [(0, False), (0, True), (1, False), (2, True)])
def test_fused_gate_f32(ops, rows, cfg, shared, apply):
    E, G, tg, k = cfg
    g = torch.Generator().manual_seed(rows * 7 + E + shared)
    x = torch.rand(rows, E, generator=g)
    bias = torch.rand(E, generator=g)
    w, ids = ops.moe_fused_gate(x.cuda(), bias.cuda(), G, tg, k + shared, shared, 2.5, apply)
    rw, rids = O.moe_fused_gate(x.numpy(), bias.numpy(), G, tg, k + shared, shared, 2.5, apply, dtype="f32")
    _compare(w, ids, rw, rids, rtol=2e-5)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("rows", [3, 513, 4096])
def test_fused_gate_16bit_types(ops, dtype, rows):
    E, G, tg, k = 256, 8, 4, 8
    g = torch.Generator().manual_seed(rows + len(dtype))
    x = (torch.randn(rows, E, generator=g) * 1.5).to(NP_DT[dtype])
    bias = (torch.rand(E, generator=g) * 0.1).to(NP_DT[dtype])
    w, ids = ops.moe_fused_gate(x.cuda(), bias.cuda(), G, tg, k, 0, 2.5, True)
    rw, rids = O.moe_fused_gate(x.float().numpy(), bias.float().numpy(), G, tg, k, 0, 2.5, True, dtype=dtype)
    # scores rounded to 16 bits tie often: the tie rules (lower group, lower expert) are what this case checks
    _compare(w, ids, rw, rids, rtol=1e-5, max_bad_frac=0.01)


def test_fused_gate_ties_and_errors(ops):
    x = torch.zeros(5, 64, device="cuda")
    w, ids = ops.moe_fused_gate(x, torch.zeros(64, device="cuda"), 8, 3, 6)
    assert ids.cpu().tolist() == [[0, 1, 2, 3, 4, 5]] * 5
    assert torch.allclose(w, torch.full_like(w, 1 / 6))
    with pytest.raises(RuntimeError):
        ops.moe_fused_gate(x, torch.zeros(64, device="cuda"), 7, 3, 6)  # 64 experts do not split into 7 groups
    with pytest.raises(RuntimeError):
        ops.moe_fused_gate(x, torch.zeros(64, device="cuda", dtype=torch.bfloat16), 8, 3, 6)  # dtype mismatch


def test_fixtures_of_the_reference(ops, golden_dir):
    z = np.load(os.path.join(golden_dir, "topk_native.npz"))
    for i in range(3):
        for apply in (0, 1):
            tag = f"g{i}a{apply}"
            E, G, tg, k = (int(v) for v in z[tag + "_cfg"])
            w, ids = ops.moe_fused_gate(torch.from_numpy(z[tag + "_x"]).cuda(), torch.from_numpy(z[tag + "_bias"]).cuda(),
                                        G, tg, k, 0, 2.5, bool(apply))
            ids, w = ids.cpu().numpy(), w.cpu().numpy()
            order, rorder = np.argsort(ids, axis=1), np.argsort(z[tag + "_ids"], axis=1)
            assert np.array_equal(np.take_along_axis(ids, order, 1), np.take_along_axis(z[tag + "_ids"], rorder, 1)), tag
            np.testing.assert_allclose(np.take_along_axis(w, order, 1), np.take_along_axis(z[tag + "_w"], rorder, 1),
                                       rtol=1e-5, err_msg=tag)
    for i in range(4):
        for renorm in (0, 1):
            tag = f"s{i}r{renorm}"
            x = torch.from_numpy(z[tag + "_x"]).cuda()
            k = int(z[tag + "_k"])
            w = torch.empty(x.shape[0], k, device="cuda")
            ids = torch.empty(x.shape[0], k, dtype=torch.int32, device="cuda")
            ops.topk_softmax_out(w, ids, x, bool(renorm))
            assert np.array_equal(ids.cpu().numpy(), z[tag + "_ids"]), tag
            np.testing.assert_allclose(w.cpu().numpy(), z[tag + "_w"], rtol=1e-5, err_msg=tag)


@pytest.mark.parametrize("rows,E,k", [(1, 8, 2), (130, 60, 4), (4096, 128, 8), (777, 256, 8), (64, 1024, 6)])
@pytest.mark.parametrize("renorm", [False, True])
@pytest.mark.parametrize("softcap,with_bias", [(0.0, False), (30.0, False), (0.0, True), (2.0, True)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_topk_softmax(ops, rows, E, k, renorm, softcap, with_bias, dtype):
    g = torch.Generator().manual_seed(rows + E + k)
    x = (torch.randn(rows, E, generator=g) * 3).to(NP_DT[dtype])
    bias = torch.randn(E, generator=g) if with_bias else None
    w = torch.empty(rows, k, device="cuda")
    ids = torch.empty(rows, k, dtype=torch.int32, device="cuda")
    ops.topk_softmax_out(w, ids, x.cuda(), renorm, softcap, None if bias is None else bias.cuda())
    rw, rids = O.topk_softmax(x.float().numpy(), k, renorm, softcap, None if bias is None else bias.numpy())
    _compare(w, ids, rw, rids, rtol=3e-5)


@pytest.mark.parametrize("rows,E,k", [(2, 16, 3), (300, 64, 6), (4096, 256, 8)])
@pytest.mark.parametrize("renorm", [False, True])
@pytest.mark.parametrize("with_bias", [False, True])
def test_topk_sigmoid(ops, rows, E, k, renorm, with_bias):
    g = torch.Generator().manual_seed(rows * 3 + E)
    x = torch.randn(rows, E, generator=g) * 2
    bias = torch.rand(E, generator=g) if with_bias else None
    w = torch.empty(rows, k, device="cuda")
    ids = torch.empty(rows, k, dtype=torch.int32, device="cuda")
    ops.topk_sigmoid_out(w, ids, x.cuda(), renorm, None if bias is None else bias.cuda())
    rw, rids = O.topk_sigmoid(x.numpy(), k, renorm, None if bias is None else bias.numpy())
    _compare(w, ids, rw, rids, rtol=3e-5)


def test_sgl_kernel_surface(ops):
    import sglang_b200.sgl_kernel as sk

    x = torch.rand(33, 256, device="cuda")
    bias = torch.rand(256, device="cuda")
    w, ids = sk.moe_fused_gate(x, bias, num_expert_group=8, topk_group=4, topk=8, routed_scaling_factor=2.5,
                               apply_routed_scaling_factor_on_output=True)
    rw, rids = O.moe_fused_gate(x.cpu().numpy(), bias.cpu().numpy(), 8, 4, 8, 0, 2.5, True)
    _compare(w, ids, rw, rids, rtol=2e-5)
    tw = torch.empty(33, 4, device="cuda")
    ti = torch.empty(33, 4, dtype=torch.int32, device="cuda")
    torch.ops.sgl_kernel.topk_softmax.default(tw, ti, x, True, 0.0, None)
    rw, rids = O.topk_softmax(x.cpu().numpy(), 4, True)
    _compare(tw, ti, rw, rids, rtol=3e-5)
    sk.topk_sigmoid(tw, ti, x, renormalize=False, correction_bias=bias)
    rw, rids = O.topk_sigmoid(x.cpu().numpy(), 4, False, bias.cpu().numpy())
    _compare(tw, ti, rw, rids, rtol=3e-5)
    from sglang_b200.srt.layers.moe.topk import biased_grouped_topk, fused_topk
    w2, ids2 = biased_grouped_topk(x, bias, 8, True, 8, 4, 2.5)
    assert torch.equal(ids2, ids) and torch.equal(w2, w)
    w3, ids3 = fused_topk(x, 4, True)
    rw, rids = O.topk_softmax(x.cpu().numpy(), 4, True)
    _compare(w3, ids3, rw, rids, rtol=3e-5)
