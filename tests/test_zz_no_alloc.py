"""The allocation-free moe_align entry point against the regular one, through the C ABI.

Collected last on purpose (file name): a failure here cannot hide the results of the other tests in a
run that stops at the first failure.  The entry point serves callers that cannot allocate device memory
at call time (graph capture with a frozen allocator, a pool fully given to the KV cache, hosts without
torch); its scratch is a fixed array inside the library, so the test also runs two calls back to back to
show that what one call leaves in the array does not leak into the next.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(ids, block, E):
    from sglang_b200 import ops
    return ops.moe_align_block_size(ids, block, E)


def _noalloc(ids, block, E):
    from sglang_b200._lib import check, lib
    numel = ids.numel()
    max_padded = numel + (E + 1) * (block - 1)
    s = torch.full((max_padded,), -3, dtype=torch.int32, device=ids.device)
    e = torch.full(((max_padded + block - 1) // block,), -3, dtype=torch.int32, device=ids.device)
    n = torch.zeros(1, dtype=torch.int32, device=ids.device)
    check(lib.sglb200_moe_align_block_size_noalloc(
        ids.data_ptr(), numel, E + 1, block, s.data_ptr(), e.data_ptr(), n.data_ptr(), 1,
        torch.cuda.current_stream().cuda_stream))
    return s, e, n


def _same(a, b, block):
    P = int(b[2].item())
    assert int(a[2].item()) == P
    assert torch.equal(a[0][:P], b[0][:P])
    assert torch.equal(a[1][: P // block], b[1][: P // block])


def test_noalloc_matches_regular_on_two_calls_in_a_row():
    g = torch.Generator(device="cuda").manual_seed(0)
    # first call: multi-chunk path (fills the histogram area), many experts
    ids1 = torch.randint(-1, 256, (16384, 8), device="cuda", dtype=torch.int32, generator=g)
    # second call: fewer experts and a single chunk, so it reads a region the first call left non-zero
    ids2 = torch.randint(-1, 64, (300, 8), device="cuda", dtype=torch.int32, generator=g)
    out1 = _noalloc(ids1, 128, 256)
    out2 = _noalloc(ids2, 128, 64)
    _same(out1, _regular(ids1, 128, 256), 128)
    _same(out2, _regular(ids2, 128, 64), 128)
    # and again in the other order, multi-chunk after single-chunk
    out3 = _noalloc(ids2, 32, 64)
    out4 = _noalloc(ids1, 64, 256)
    _same(out3, _regular(ids2, 32, 64), 32)
    _same(out4, _regular(ids1, 64, 256), 64)


def test_noalloc_rejects_oversized_calls():
    from sglang_b200._lib import lib
    ids = torch.zeros(8, dtype=torch.int32, device="cuda")
    out = torch.zeros(4096, dtype=torch.int32, device="cuda")
    rc = lib.sglb200_moe_align_block_size_noalloc(ids.data_ptr(), 8, 2000, 128, out.data_ptr(), out.data_ptr(),
                                                  out.data_ptr(), 1, None)
    assert rc == -1 and b"exceed the built-in scratch" in lib.sglb200_last_error()
    rc = lib.sglb200_moe_align_block_size_noalloc(ids.data_ptr(), (1 << 20) + 1, 257, 128, out.data_ptr(),
                                                  out.data_ptr(), out.data_ptr(), 1, None)
    assert rc == -1 and b"exceed the built-in scratch" in lib.sglb200_last_error()
