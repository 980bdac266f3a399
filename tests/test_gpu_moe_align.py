"""GPU parity of moe_align_block_size through the C ABI: bit-exact against the oracle."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as CO

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from sglang_b200 import ops as _ops
    return _ops


def _check(ops, ids_np, block, E):
    ids = torch.from_numpy(ids_np).cuda()
    s, e, n = ops.moe_align_block_size(ids, block, E)
    rs, re, rn = CO.moe_align(ids_np, block, E)
    P = int(rn[0])
    assert int(n.item()) == P
    assert np.array_equal(s.cpu().numpy()[:P], rs[:P])
    assert np.array_equal(e.cpu().numpy()[: P // block], re[: P // block])


def test_documented_example(ops):
    ids = np.array([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=np.int32)
    s, e, n = ops.moe_align_block_size(torch.from_numpy(ids).cuda(), 4, 5)
    assert int(n.item()) == 16
    assert s[:16].tolist() == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    assert e[:4].tolist() == [1, 2, 3, 4]


@pytest.mark.parametrize("block", [32, 64, 128, 256])
@pytest.mark.parametrize("tokens", [1, 2, 33, 256, 257, 1024, 1025, 4096])
@pytest.mark.parametrize("topk,E", [(1, 64), (8, 256), (6, 160), (9, 257), (8, 8)])
def test_random_ids(ops, block, tokens, topk, E):
    rng = np.random.default_rng(tokens * 131 + topk * 7 + E + block)
    ids = rng.integers(0, E, size=(tokens, topk)).astype(np.int32)
    _check(ops, ids, block, E)


@pytest.mark.parametrize("tokens", [1, 64, 512, 4096, 16384])
def test_filtered_experts_and_skew(ops, tokens):
    # expert parallelism: ids of experts on other ranks are -1; Zipf-like skew piles load on few experts
    rng = np.random.default_rng(tokens)
    E = 32
    p = 1.0 / np.arange(1, E + 2) ** 1.2
    ids = rng.choice(E + 1, size=(tokens, 8), p=p / p.sum()).astype(np.int32) - 1
    _check(ops, ids, 128, E)


def test_all_one_expert_and_empty(ops):
    _check(ops, np.full((3000, 8), 5, dtype=np.int32), 128, 256)
    _check(ops, np.full((7, 8), -1, dtype=np.int32), 128, 256)
    s, e, n = ops.moe_align_block_size(torch.zeros((0, 8), dtype=torch.int32, device="cuda"), 128, 256)
    assert int(n.item()) == 0


def test_three_launch_form(ops):
    """The histogram / scan / scatter launches that stand in where a cooperative launch is not possible."""
    from sglang_b200._lib import lib
    lib.sglb200_moe_align_set_cooperative(0)
    try:
        rng = np.random.default_rng(11)
        for tokens, topk, E in ((300, 8, 256), (4096, 8, 256), (16384, 8, 128), (100000, 6, 160)):
            _check(ops, rng.integers(-1, E, size=(tokens, topk)).astype(np.int32), 128, E)
    finally:
        lib.sglb200_moe_align_set_cooperative(1)


def test_large_input_properties(ops):
    # 2M ids: multi-chunk path at a size the python checks still finish quickly
    rng = np.random.default_rng(0)
    E, block = 256, 128
    ids = rng.integers(0, E, size=(262144, 8)).astype(np.int32)
    _check(ops, ids, block, E)
    # 3.2M ids with filtered entries: chunks longer than 8192 ids (more than two CTAs per SM otherwise)
    ids = rng.integers(-1, E, size=(400000, 8)).astype(np.int32)
    _check(ops, ids, block, E)
    # ragged length, every id in one bucket: a tile of the large-input path is a single run
    _check(ops, np.full((1300001, 1), 7, dtype=np.int32), 64, 16)
    # many buckets under Zipf skew, ragged length
    E = 1000
    p = 1.0 / np.arange(1, E + 2) ** 1.2
    ids = rng.choice(E + 1, size=(1500003, 1), p=p / p.sum()).astype(np.int32) - 1
    _check(ops, ids, 128, E)


def test_sgl_kernel_op_surface(ops):
    import sglang_b200.sgl_kernel  # registers torch.ops.sgl_kernel.*
    E, block = 64, 32
    ids = torch.randint(0, E, (100, 4), dtype=torch.int32, device="cuda")
    max_padded = ids.numel() + (E + 1) * (block - 1)
    s = torch.empty(max_padded, dtype=torch.int32, device="cuda")
    e = torch.empty((max_padded + block - 1) // block, dtype=torch.int32, device="cuda")
    n = torch.empty(1, dtype=torch.int32, device="cuda")
    c = torch.empty(E + 2, dtype=torch.int32, device="cuda")
    torch.ops.sgl_kernel.moe_align_block_size.default(ids, E + 1, block, s, e, n, c, True)
    rs, re, rn = CO.moe_align(ids.cpu().numpy(), block, E)
    P = int(rn[0])
    assert int(n.item()) == P and np.array_equal(s.cpu().numpy()[:P], rs[:P])
    assert int(c[E + 1].item()) == P
