"""The bounded waits of the kernels, made to run out on a healthy GPU (nothing faults, traps or hangs): each kernel
must return promptly with its status word set, leave the context usable, and the next ordinary call must be right.

* GEMM and streaming kernels: the probe limit is set to "give up at once" (`*_set_wait_probes(UINT32_MAX)`), so every
  pipeline wait expires before anything was loaded.
* reduce-and-gather kernel of the fused all-reduce: one process plays rank 0 of a two-rank group whose "peer" buffers
  are this GPU's own memory; nothing ever writes the peer's flag, so the wait for it runs out after a small number of
  probes.  Then the flags the peer would have written are set from the host and the same call completes: rank 0's
  rows are the float32 sum of the two staged blocks, the peer's rows come from its buffer of reduced rows.
"""
import ctypes as C
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
GIVE_UP_AT_ONCE = 0xFFFFFFFF


def _inputs(M, N, K):
    from sglang_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    xq, xs = ops.per_token_group_quant_fp8(x, 128)
    wq = (torch.randn(N, K, device="cuda", generator=g) * 20).clamp(-448, 448).to(torch.float8_e4m3fn)
    ws = torch.rand((N + 127) // 128, K // 128, device="cuda", generator=g) * 1e-3
    return x, xq, xs, wq, ws


@pytest.mark.parametrize("M,N,K", [(300, 512, 1024), (1024, 768, 2048), (16, 7168, 16384)])
def test_gemm_wait_runs_out_and_recovers(M, N, K):
    from sglang_b200 import ops
    from sglang_b200._lib import check, lib
    _, xq, xs, wq, ws = _inputs(M, N, K)
    good = ops.w8a8_block_fp8_matmul(xq, wq, xs, ws, [128, 128], torch.bfloat16)
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    lib.sglb200_gemm_set_wait_probes(GIVE_UP_AT_ONCE)
    try:
        t0 = time.perf_counter()
        ops.w8a8_block_fp8_matmul(xq, wq, xs, ws, [128, 128], torch.bfloat16)
        torch.cuda.synchronize()  # returns: no role is left waiting
        assert time.perf_counter() - t0 < 5.0
        assert ops.gemm_status() == 1
    finally:
        lib.sglb200_gemm_set_wait_probes(0)
        check(lib.sglb200_gemm_status_clear())
    again = ops.w8a8_block_fp8_matmul(xq, wq, xs, ws, [128, 128], torch.bfloat16)
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0 and torch.equal(again, good)


def test_stream_kernels_wait_runs_out_and_recover():
    from sglang_b200 import ops
    from sglang_b200._lib import check, lib
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(777, 4096, device="cuda", generator=g).bfloat16()
    y = torch.randn(333, 2 * 1024, device="cuda", generator=g).bfloat16()
    good_q, good_s = ops.per_token_group_quant_fp8(x, 128)
    good_hq, good_hs = ops.silu_and_mul_quant_fp8(y, 128)
    torch.cuda.synchronize()
    assert ops.stream_status() == 0
    lib.sglb200_stream_set_wait_probes(GIVE_UP_AT_ONCE)
    try:
        t0 = time.perf_counter()
        ops.per_token_group_quant_fp8(x, 128)
        ops.silu_and_mul_quant_fp8(y, 128)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 5.0
        assert ops.stream_status() == 1
    finally:
        lib.sglb200_stream_set_wait_probes(0)
        check(lib.sglb200_stream_status_clear())
    q, s = ops.per_token_group_quant_fp8(x, 128)
    hq, hs = ops.silu_and_mul_quant_fp8(y, 128)
    torch.cuda.synchronize()
    assert ops.stream_status() == 0
    assert torch.equal(q.view(torch.uint8), good_q.view(torch.uint8)) and torch.equal(s, good_s)
    assert torch.equal(hq.view(torch.uint8), good_hq.view(torch.uint8)) and torch.equal(hs, good_hs)


def test_reduce_gather_peer_never_arrives_then_completes():
    from sglang_b200._lib import check, lib
    world, rank, M, N = 2, 0, 256, 512
    rpo = lib.sglb200_push_rows_per_owner(M, world)  # 128 rows per owner
    g = torch.Generator(device="cuda").manual_seed(11)
    stage = torch.randn(world, rpo, N, device="cuda", generator=g).bfloat16()      # what two GEMMs would have pushed
    reduced_peer = torch.randn(rpo, N, device="cuda", generator=g).bfloat16()     # the peer's reduced rows
    reduced_own = torch.zeros(rpo, N, device="cuda", dtype=torch.bfloat16)
    nflag = lib.sglb200_comm_flag_bytes() // 4
    flags_own = torch.zeros(nflag, device="cuda", dtype=torch.int32)
    flags_peer = torch.zeros(nflag, device="cuda", dtype=torch.int32)               # rank 0's arrivals land here
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    arr = C.c_void_p * world
    reduced = arr(reduced_own.data_ptr(), reduced_peer.data_ptr())
    flags = arr(flags_own.data_ptr(), flags_peer.data_ptr())
    st = torch.cuda.current_stream().cuda_stream

    def call():
        check(lib.sglb200_reduce_gather(stage.data_ptr(), reduced, flags, out.data_ptr(), world, rank, M, N, 0, 0, st))

    lib.sglb200_comm_set_wait_probes(2000)  # about a millisecond
    try:
        t0 = time.perf_counter()
        call()
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 2.0
        assert lib.sglb200_comm_status() == 1
        assert not out.any()  # the kernel left without touching the output
        check(lib.sglb200_comm_status_clear())
        # the second call's epoch is 2 in every block (each block counts its own calls): play the peer's arrivals at
        # both barriers by writing 2 into the words rank 1 would write, for every block
        blocks, max_world = 148, 8
        peer_words = flags_own[: 2 * blocks * max_world].view(2, blocks, max_world)
        peer_words[:, :, 1] = 2
        torch.cuda.synchronize()
        call()
        torch.cuda.synchronize()
        assert lib.sglb200_comm_status() == 0
    finally:
        lib.sglb200_comm_set_wait_probes(0)
        check(lib.sglb200_comm_status_clear())
    want_own = (stage[0].float() + stage[1].float()).bfloat16()
    assert torch.equal(out[:rpo], want_own) and torch.equal(reduced_own, want_own)
    assert torch.equal(out[rpo:], reduced_peer)
    # rank 0 told the peer about both barriers of both calls
    assert int(flags_peer[: 2 * blocks * max_world].view(2, blocks, max_world)[:, 0, 0].max()) == 2
