"""Host-side logic that needs no GPU: sharding rules, quant-method checks, and the expert-parallel
exchange run as two gloo ranks on CPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_fp8_config_and_divisibility_checks():
    from sglang_b200.srt.layers.quantization.fp8 import Fp8Config, Fp8LinearMethod, Fp8MoEMethod
    cfg = Fp8Config.from_config({"quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128]})
    assert cfg.weight_block_size == [128, 128] and cfg.get_name() == "fp8"
    with pytest.raises(ValueError):
        Fp8Config(activation_scheme="static")
    with pytest.raises(ValueError):
        Fp8Config(weight_block_size=[64, 64])
    layer = torch.nn.Module()
    m = Fp8LinearMethod(cfg)
    m.create_weights(layer, 7168, [2112], 7168, 2112, torch.bfloat16)
    assert layer.weight.shape == (2112, 7168) and layer.weight.dtype == torch.float8_e4m3fn
    assert layer.weight_scale_inv.shape == (17, 56)
    with pytest.raises(ValueError):  # merged layers must split on 128-row boundaries (fp8.py:249-259)
        m.create_weights(torch.nn.Module(), 512, [192, 192], 512, 384, torch.bfloat16)
    moe = torch.nn.Module()
    mm = Fp8MoEMethod(cfg)
    mm.create_weights(moe, 4, 512, 256, torch.bfloat16)
    assert moe.w13_weight.shape == (4, 512, 512) and moe.w13_weight_scale_inv.shape == (4, 4, 4)
    assert moe.w2_weight.shape == (4, 512, 256) and moe.w2_weight_scale_inv.shape == (4, 4, 2)
    with pytest.raises(ValueError):
        mm.create_weights(torch.nn.Module(), 4, 512, 192, torch.bfloat16)


def test_max_padded_rows_bound():
    from sglang_b200.srt.layers.moe.fused_moe_triton.fused_moe import _max_padded_rows
    from oracle import block_fp8_oracle as O
    rng = np.random.default_rng(0)
    for T, topk, E in [(1, 8, 256), (5, 2, 4), (64, 8, 256), (4096, 8, 32)]:
        ids = rng.integers(-1, E, size=(T, topk)).astype(np.int32)
        _, _, n = O.moe_align_block_size(ids, 128, E)
        assert int(n[0]) <= _max_padded_rows(T * topk, E, 128)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ep_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sglang_b200.srt.distributed import get_moe_ep_group, initialize_model_parallel
        from sglang_b200.srt.layers.moe.fused_moe_triton import ep_a2a
        initialize_model_parallel(1, world, backend="gloo")
        group = get_moe_ep_group()
        E, E_local, T, H, topk = 8, 8 // world, 6 + rank, 256, 3
        g = torch.Generator().manual_seed(100 + rank)
        xq = torch.randint(0, 120, (T, H), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
        xs = torch.rand(T, H // 128, generator=g)
        ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]).to(torch.int32)
        w = torch.rand(T, topk, generator=g)
        plan = ep_a2a.plan_dispatch(ids, E_local, group)
        q, s, local, rw = ep_a2a.dispatch(xq, xs, ids, w, plan, group, E_local)
        # stand-in for the local experts: row value = sum of weights of the experts this rank owns
        owned = (local >= 0).float()
        out_rows = ((rw * owned).sum(1, keepdim=True) * torch.ones(1, H)).to(torch.bfloat16)
        out = ep_a2a.combine(out_rows, plan, group, T, 1.0)
        ret[rank] = dict(
            out=out.float().numpy(), w=w.numpy(), ids=ids.numpy(), recv_rows=q.shape[0], local=local.numpy(),
            q_first=q.view(torch.uint8)[:1].numpy() if q.shape[0] else None,
            send_splits=plan.send_splits, recv_splits=plan.recv_splits)
    finally:
        dist.destroy_process_group()


def test_ep_dispatch_combine_two_gloo_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_ep_worker, args=(world, port, ret), nprocs=world, join=True)
    for r in range(world):
        d = ret[r]
        # every token's weights are all counted exactly once across the ranks that own its experts
        expect = d["w"].sum(1)
        got = d["out"][:, 0]
        np.testing.assert_allclose(got, expect, rtol=2e-2)
        # a row is sent once per destination rank even when several of its experts live there
        dest = d["ids"] // (8 // world)
        pairs = sum(len(set(row)) for row in dest.tolist())
        assert sum(d["send_splits"]) == pairs
        assert d["recv_rows"] == sum(d["recv_splits"])
        assert ((d["local"] >= -1) & (d["local"] < 8 // world)).all()
    assert ret[0]["send_splits"][1] == ret[1]["recv_splits"][0]


def test_dispatch_mask_mixed_filtered_and_valid_ids():
    """Rows that mix a filtered slot (-1), an id past the last expert and valid ids: a token goes to a rank exactly
    when one of its VALID slots names an expert of that rank, whatever the order of its slots."""
    from sglang_b200.srt.distributed import GroupCoordinator
    from sglang_b200.srt.layers.moe.fused_moe_triton import ep_a2a

    class FakeGroup(GroupCoordinator):  # four ranks' worth of planning on one process: only the mask is looked at
        def __init__(self):
            self.ranks, self.world_size, self.rank, self.rank_in_group, self.device_group = [0, 1, 2, 3], 4, 0, 0, None

        def all_to_all_single(self, out, inp, out_splits, in_splits):
            out.copy_(inp)
            return out

    E_local = 2  # experts 0-1 on rank 0, 2-3 on rank 1, 4-5 on rank 2, 6-7 on rank 3
    ids = torch.tensor([[-1, 0, 1],      # filtered slot first, then two experts of rank 0 -> rank 0 only
                        [1, -1, -1],     # valid slot first, filtered after it -> rank 0 (the -1s must not erase it)
                        [-1, -1, -1],    # nothing valid -> nowhere
                        [7, 8, 2],       # 8 is past the last expert -> ranks 3 and 1, not clamped onto rank 3 twice
                        [9, -1, 100],    # nothing valid -> nowhere
                        [6, 0, 3]], dtype=torch.int32)
    plan = ep_a2a.plan_dispatch(ids, E_local, FakeGroup())
    sent = {(int(t), r) for r, n in enumerate(plan.send_splits) for t in
            plan.send_token[sum(plan.send_splits[:r]): sum(plan.send_splits[:r]) + n]}
    assert sent == {(0, 0), (1, 0), (3, 1), (3, 3), (5, 0), (5, 1), (5, 3)}
    assert plan.send_splits == [3, 2, 0, 2]
    S = int(plan.send_token.numel())
    assert (plan.slot[2] == S).all() and (plan.slot[4] == S).all()  # tokens that go nowhere point at the zero row


def test_expert_location_hot_replication():
    """Placement with redundant copies of the hottest experts: every rank keeps its block of logical experts plus a copy
    of the same hot ones, sends a hot expert's rows to its own copy (to the original where it is the owner), and the
    physical-to-logical map tells each slot which weights to load."""
    from sglang_b200.srt.eplb import ExpertLocationMetadata, topk_ids_logical_to_physical
    count = torch.tensor([5.0, 1, 9, 2, 7, 7, 0, 3])  # experts 2 and 4 are the hottest (4 wins the tie with 5)
    metas = [ExpertLocationMetadata.init_by_hot_replication(count, 2, r, 2) for r in range(2)]
    for m in metas:
        assert m.num_physical_experts == 12 and m.num_local_physical_experts == 6
        assert m.physical_to_logical_map.tolist() == [0, 1, 2, 3, 2, 4, 4, 5, 6, 7, 2, 4]
    assert metas[0].logical_to_rank_dispatch_physical_map.tolist() == [0, 1, 2, 3, 5, 7, 8, 9]
    assert metas[1].logical_to_rank_dispatch_physical_map.tolist() == [0, 1, 10, 3, 6, 7, 8, 9]
    ids = torch.tensor([[2, 4, -1], [0, 7, 5]], dtype=torch.int32)
    for r, m in enumerate(metas):
        phys = topk_ids_logical_to_physical(ids, m)
        assert phys.dtype == torch.int32 and int(phys[0, 2]) == -1
        # every physical slot a rank names holds the logical expert that was routed, and hot rows stay on the rank
        ok = phys >= 0
        assert torch.equal(m.physical_to_logical_map[phys[ok].long()], ids[ok])
        assert all(int(phys[0, j]) // 6 == r for j in (0, 1))
    assert metas[0].local_logical_experts(1).tolist() == [4, 5, 6, 7, 2, 4]
    assert topk_ids_logical_to_physical(ids, None) is ids


def test_expert_location_by_load():
    """Hot experts on every rank only, cold experts packed by routed rows: every logical expert has a slot, every rank
    the same number of slots, the cold load is spread evenly, and all ranks agree on the cold experts' places."""
    from sglang_b200.srt.eplb import ExpertLocationMetadata, topk_ids_logical_to_physical
    g = torch.Generator().manual_seed(5)
    E, p, R = 20, 4, 4
    count = (torch.arange(1, E + 1, dtype=torch.float64) ** -1.2)[torch.randperm(E, generator=g)] * 1e6
    metas = [ExpertLocationMetadata.init_by_load(count, p, r, R) for r in range(p)]
    hot = set(torch.topk(count, R).indices.tolist())
    local = (E - R) // p + R
    for r, m in enumerate(metas):
        assert m.num_local_physical_experts == local and m.num_physical_experts == p * local
        assert torch.equal(m.physical_to_logical_map, metas[0].physical_to_logical_map)
        l2p = m.logical_to_rank_dispatch_physical_map
        assert torch.equal(m.physical_to_logical_map[l2p.long()], torch.arange(E, dtype=torch.int32))
        for e in range(E):
            owner = int(l2p[e]) // local
            assert (owner == r) if e in hot else (int(l2p[e]) == int(metas[0].logical_to_rank_dispatch_physical_map[e]))
        assert set(m.local_logical_experts(r)[-R:].tolist()) == hot
    # cold rows per rank: within 15 % of their mean (they are 16 experts with a 1 : 9 spread of loads)
    cold_load = [sum(float(count[e]) for e in metas[0].local_logical_experts(r)[:-R].tolist()) for r in range(p)]
    assert max(cold_load) <= 1.15 * (sum(cold_load) / p)
    ids = torch.tensor([[0, 5, -1]], dtype=torch.int32)
    assert int(topk_ids_logical_to_physical(ids, metas[2])[0, 2]) == -1


def _tp_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sglang_b200.srt.distributed import initialize_model_parallel, tensor_model_parallel_all_reduce
        from sglang_b200.srt.layers.linear import MergedColumnParallelLinear, RowParallelLinear
        from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
        initialize_model_parallel(world, 1, backend="gloo")
        cfg = Fp8Config()
        col = MergedColumnParallelLinear(512, [256, 256], quant_config=cfg)
        row = RowParallelLinear(512, 384, quant_config=cfg)
        g = torch.Generator().manual_seed(0)
        w = torch.randint(0, 255, (512, 512), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
        s = torch.rand(4, 4, generator=g)
        col.load_full_weight(w, s)
        w2 = torch.randint(0, 255, (384, 512), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
        s2 = torch.rand(3, 4, generator=g)
        row.load_full_weight(w2, s2)
        x = torch.full((2, 3), float(rank + 1))
        tensor_model_parallel_all_reduce(x)
        from sglang_b200.srt.distributed import get_tp_group
        rs = get_tp_group().reduce_scatter(torch.arange(4.0).reshape(4, 1) * (rank + 1))  # rows [2r, 2r+2) of the sum
        ret[rank] = dict(rs=rs.numpy(),
            col_w=col.weight.view(torch.uint8).numpy(), col_s=col.weight_scale_inv.numpy(),
            row_w=row.weight.view(torch.uint8).numpy(), row_s=row.weight_scale_inv.numpy(),
            full_w=w.view(torch.uint8).numpy(), full_s=s.numpy(), full_w2=w2.view(torch.uint8).numpy(),
            full_s2=s2.numpy(), ar=x.numpy())
    finally:
        dist.destroy_process_group()


def test_tp_sharding_two_gloo_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_tp_worker, args=(world, port, ret), nprocs=world, join=True)
    for r in range(world):
        d = ret[r]
        # merged column layer: rank r holds rows [128r,128r+128) of part 0 and of part 1
        exp_w = np.concatenate([d["full_w"][128 * r : 128 * r + 128], d["full_w"][256 + 128 * r : 256 + 128 * r + 128]])
        exp_s = np.concatenate([d["full_s"][r : r + 1], d["full_s"][2 + r : 3 + r]])
        assert np.array_equal(d["col_w"], exp_w) and np.array_equal(d["col_s"], exp_s)
        assert np.array_equal(d["row_w"], d["full_w2"][:, 256 * r : 256 * r + 256])
        assert np.array_equal(d["row_s"], d["full_s2"][:, 2 * r : 2 * r + 2])
        assert np.all(d["ar"] == 3.0)
        assert np.array_equal(d["rs"], 3.0 * np.arange(4.0).reshape(4, 1)[2 * r : 2 * r + 2])


def test_sgl_kernel_ops_have_shape_only_implementations():
    """torch.ops.sgl_kernel.* can be traced without a GPU (meta tensors), as torch.compile needs."""
    import torch
    import sglang_b200.sgl_kernel  # noqa: F401

    a = torch.empty(33, 256, dtype=torch.float8_e4m3fn, device="meta")
    b = torch.empty(256, 384, dtype=torch.float8_e4m3fn, device="meta")
    sa = torch.empty(33, 2, device="meta")
    sb = torch.empty(2, 3, device="meta")
    out = torch.ops.sgl_kernel.fp8_blockwise_scaled_mm.default(a, b, sa, sb, torch.bfloat16)
    assert out.shape == (33, 384) and out.dtype == torch.bfloat16 and out.device.type == "meta"
    x = torch.empty(33, 256, dtype=torch.bfloat16, device="meta")
    q = torch.empty(33, 256, dtype=torch.float8_e4m3fn, device="meta")
    s = torch.empty(33, 2, device="meta")
    assert torch.ops.sgl_kernel.sgl_per_token_group_quant_8bit.default(x, q, s, 128, 1e-10, -448.0, 448.0, False) is None
    w, ids = torch.ops.sgl_kernel.moe_fused_gate.default(torch.empty(7, 256, device="meta"), torch.empty(256, device="meta"),
                                                         8, 4, 8, 0, 2.5, True)
    assert w.shape == (7, 8) and w.dtype == torch.float32 and ids.dtype == torch.int32
    tw = torch.empty(7, 4, device="meta")
    ti = torch.empty(7, 4, dtype=torch.int32, device="meta")
    assert torch.ops.sgl_kernel.topk_softmax.default(tw, ti, torch.empty(7, 64, device="meta"), True, 0.0, None) is None


def test_fused_row_parallel_shape_rules():
    """Which outputs the GEMM-fused all-reduce takes and how rows are owned (host logic only, no GPU)."""
    from sglang_b200._lib import lib
    from sglang_b200.srt.distributed.fused_row_parallel import FusedRowParallelComm
    assert lib.sglb200_push_rows_per_owner(8192, 8) == 1024
    assert lib.sglb200_push_rows_per_owner(300, 2) == 256      # owner 0: 256 rows, owner 1: 44
    assert lib.sglb200_push_rows_per_owner(1068, 8) == 256     # owners 0-3 full, owner 4: 44 rows, owners 5-7: none
    comm = object.__new__(FusedRowParallelComm)
    comm.world, comm.max_elems = 8, 8192 * 8192
    assert comm.supports(8192, 8192) and comm.supports(1024, 8192) and comm.supports(5000, 8192)
    assert not comm.supports(1023, 8192)        # fewer than one tile of rows per rank
    assert not comm.supports(8192, 8196)        # rows of 16-byte pieces only
    assert not comm.supports(8192 + 1, 8192)    # its staging copy (8 x 1152 rows) does not fit
    comm.pipeline, comm.min_comm_ratio, comm.min_waves, comm.sms, comm.sm_margin = False, 0.4, 3, 148, 16
    assert comm._chunks(8192, 8192, 1024) == 1  # chunked pipelining is off by default
    comm.pipeline = True
    assert comm._chunks(8192, 8192, 1024) == 4 and comm._chunks(8192, 8192, 14336) == 1
    assert comm._chunks(5000, 8192, 1024) == 1  # ragged row counts are never chunked
