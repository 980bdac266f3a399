"""Loading a serialized block-FP8 checkpoint (safetensors, Hugging Face names, `weight` + `weight_scale_inv`) into the
tensor-parallel and expert-parallel layers of the path: every rank must end up with exactly its rows / columns /
experts of the checkpoint tensors and 1/128 of them, rounded up, of the block scales
(python/sglang/srt/layers/linear.py:737-746, :917-973, :1314-1352; fused_moe_triton/layer.py:575-918;
models/deepseek_v2.py:3749-3960).  Runs on CPU: loading moves bytes, it launches nothing."""
import numpy as np
import pytest
import torch
from torch import nn

from sglang_b200.srt.distributed import parallel_state as ps
from sglang_b200.srt.eplb import ExpertLocationMetadata
from sglang_b200.srt.layers.linear import (ColumnParallelLinear, MergedColumnParallelLinear, QKVParallelLinear,
                                           ReplicatedLinear, RowParallelLinear)
from sglang_b200.srt.layers.moe.fused_moe_triton.layer import FusedMoE
from sglang_b200.srt.layers.quantization.fp8 import Fp8Config
from sglang_b200.srt.model_loader import load_block_fp8_weights, safetensors_weights_iterator

H, Q_LORA, KV_A, Q_B, O_IN, I_DENSE, E, I_MOE = 512, 256, 192, 1024, 1024, 1024, 8, 512
HEAD, NQ, NKV = 128, 8, 2


def _fake_group(world, rank):
    g = ps.GroupCoordinator.__new__(ps.GroupCoordinator)
    g.ranks, g.world_size, g.rank, g.rank_in_group, g.device_group = list(range(world)), world, rank, rank, None
    return g


@pytest.fixture
def parallel():
    def set_(tp=1, tp_rank=0, ep=1, ep_rank=0):
        ps._TP, ps._MOE_EP = _fake_group(tp, tp_rank), _fake_group(ep, ep_rank)
    yield set_
    ps._TP = ps._MOE_EP = None


def _codes(gen, *shape):
    # any byte but the two NaN encodings of e4m3
    c = torch.randint(0, 0x7F, shape, generator=gen, dtype=torch.uint8) | (torch.randint(0, 2, shape, generator=gen, dtype=torch.uint8) << 7)
    return c.view(torch.float8_e4m3fn)


def _pair(gen, n, k):
    return _codes(gen, n, k), torch.rand((n + 127) // 128, (k + 127) // 128, generator=gen) + 0.5


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    """Two safetensors files named as the DeepSeek-V3 and Llama FP8 releases name their tensors."""
    from safetensors.torch import save_file
    gen = torch.Generator().manual_seed(7)
    t = {}

    def add(name, n, k):
        t[f"{name}.weight"], t[f"{name}.weight_scale_inv"] = _pair(gen, n, k)

    a = "model.layers.0.self_attn"
    add(f"{a}.q_a_proj", Q_LORA, H)
    add(f"{a}.kv_a_proj_with_mqa", KV_A, H)           # 1.5 blocks of rows: two scale rows, the second half used
    add(f"{a}.q_b_proj", Q_B, Q_LORA)
    add(f"{a}.o_proj", H, O_IN)
    for proj in ("q_proj", "k_proj", "v_proj"):
        add(f"{a}.{proj}", (NQ if proj == "q_proj" else NKV) * HEAD, H)
    m = "model.layers.0.mlp"
    add(f"{m}.gate_proj", I_DENSE, H)
    add(f"{m}.up_proj", I_DENSE, H)
    add(f"{m}.down_proj", H, I_DENSE)
    x = "model.layers.1.mlp"
    for e in range(E):
        add(f"{x}.experts.{e}.gate_proj", I_MOE, H)
        add(f"{x}.experts.{e}.up_proj", I_MOE, H)
        add(f"{x}.experts.{e}.down_proj", H, I_MOE)
    add(f"{x}.shared_experts.gate_proj", I_MOE, H)
    add(f"{x}.shared_experts.up_proj", I_MOE, H)
    add(f"{x}.shared_experts.down_proj", H, I_MOE)
    t[f"{a}.rotary_emb.inv_freq"] = torch.rand(4)
    d = tmp_path_factory.mktemp("ckpt")
    names = sorted(t)
    files = [str(d / "model-00001-of-00002.safetensors"), str(d / "model-00002-of-00002.safetensors")]
    save_file({n: t[n] for n in names[::2]}, files[0])
    save_file({n: t[n] for n in names[1::2]}, files[1])
    return files, t


class _Attn(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.fused_qkv_a_proj_with_mqa = ReplicatedLinear(H, Q_LORA + KV_A, quant_config=cfg, prefix="fused_qkv_a")
        self.q_b_proj = ColumnParallelLinear(Q_LORA, Q_B, quant_config=cfg, prefix="q_b")
        self.o_proj = RowParallelLinear(O_IN, H, quant_config=cfg, prefix="o_proj")
        self.qkv_proj = QKVParallelLinear(H, HEAD, NQ, NKV, quant_config=cfg, prefix="qkv")


class _Mlp(nn.Module):
    def __init__(self, cfg, inter):
        super().__init__()
        self.gate_up_proj = MergedColumnParallelLinear(H, [inter, inter], quant_config=cfg, prefix="gate_up")
        self.down_proj = RowParallelLinear(inter, H, quant_config=cfg, prefix="down")


class _MoeBlock(nn.Module):
    def __init__(self, cfg, location=None):
        super().__init__()
        self.experts = FusedMoE(E, H, I_MOE, 2, quant_config=cfg, expert_location=location)
        self.shared_experts = _Mlp(cfg, I_MOE)


class _Layer(nn.Module):
    def __init__(self, mlp, attn=None):
        super().__init__()
        if attn is not None:
            self.self_attn = attn
        self.mlp = mlp


class _Model(nn.Module):
    def __init__(self, location=None):
        super().__init__()
        cfg = Fp8Config()
        inner = nn.Module()
        inner.layers = nn.ModuleList([_Layer(_Mlp(cfg, I_DENSE), _Attn(cfg)), _Layer(_MoeBlock(cfg, location))])
        self.model = inner

    def load_weights(self, weights):
        return load_block_fp8_weights(
            self, weights,
            stacked_params_mapping=[("gate_up_proj", "gate_proj", 0), ("gate_up_proj", "up_proj", 1),
                                    ("qkv_proj", "q_proj", "q"), ("qkv_proj", "k_proj", "k"), ("qkv_proj", "v_proj", "v")],
            expert_params_mapping=FusedMoE.make_expert_params_mapping("gate_proj", "down_proj", "up_proj", E),
            concat_params_mapping={"fused_qkv_a_proj_with_mqa": ["q_a_proj", "kv_a_proj_with_mqa"]})


def _same(param, expect):
    got = param.data
    if got.dtype == torch.float8_e4m3fn:
        got, expect = got.view(torch.uint8), expect.view(torch.uint8)
    assert tuple(got.shape) == tuple(expect.shape)
    assert torch.equal(got, expect)


def _rows(t, lo, n, scale):
    return t[lo // 128: (lo + n + 127) // 128] if scale else t[lo: lo + n]


@pytest.mark.parametrize("tp,tp_rank", [(1, 0), (2, 0), (2, 1), (4, 3)])
def test_dense_layers_take_their_shard(parallel, checkpoint, tp, tp_rank):
    files, t = checkpoint
    parallel(tp=tp, tp_rank=tp_rank)
    model = _Model()
    written = model.load_weights(safetensors_weights_iterator(files))
    a, m = model.model.layers[0].self_attn, model.model.layers[0].mlp
    pa, pm = "model.layers.0.self_attn", "model.layers.0.mlp"
    for kind in ("weight", "weight_scale_inv"):
        sc = kind.endswith("inv")
        # replicated, joined from two checkpoint tensors: 256 + 192 rows -> 448 rows, 2 + 2 scale rows
        _same(getattr(a.fused_qkv_a_proj_with_mqa, kind),
              torch.cat([t[f"{pa}.q_a_proj.{kind}"].view(torch.uint8) if not sc else t[f"{pa}.q_a_proj.{kind}"],
                         t[f"{pa}.kv_a_proj_with_mqa.{kind}"].view(torch.uint8) if not sc else t[f"{pa}.kv_a_proj_with_mqa.{kind}"]]))
        n = Q_B // tp
        _same(getattr(a.q_b_proj, kind), _rows(t[f"{pa}.q_b_proj.{kind}"], tp_rank * n, n, sc))
        k = O_IN // tp
        full = t[f"{pa}.o_proj.{kind}"]
        _same(getattr(a.o_proj, kind), full[:, tp_rank * k // 128: (tp_rank + 1) * k // 128] if sc else full[:, tp_rank * k: (tp_rank + 1) * k])
        n = I_DENSE // tp
        gate, up = t[f"{pm}.gate_proj.{kind}"], t[f"{pm}.up_proj.{kind}"]
        if not sc:
            gate, up = gate.view(torch.uint8), up.view(torch.uint8)
        _same(getattr(m.gate_up_proj, kind), torch.cat([_rows(gate, tp_rank * n, n, sc), _rows(up, tp_rank * n, n, sc)]))
        k = I_DENSE // tp
        full = t[f"{pm}.down_proj.{kind}"]
        _same(getattr(m.down_proj, kind), full[:, tp_rank * k // 128: (tp_rank + 1) * k // 128] if sc else full[:, tp_rank * k: (tp_rank + 1) * k])
        # grouped-query attention: 8 query heads split over the ranks, 2 KV heads split (tp <= 2) or held twice (tp = 4)
        nq = NQ * HEAD // tp
        kv_rank = tp_rank if tp <= NKV else tp_rank // (tp // NKV)
        nkv = max(NKV // tp, 1) * HEAD
        parts = [_rows(t[f"{pa}.q_proj.{kind}"], tp_rank * nq, nq, sc), _rows(t[f"{pa}.k_proj.{kind}"], kv_rank * nkv, nkv, sc),
                 _rows(t[f"{pa}.v_proj.{kind}"], kv_rank * nkv, nkv, sc)]
        _same(getattr(a.qkv_proj, kind), torch.cat([p if sc else p.view(torch.uint8) for p in parts]))
    assert f"{pa}.fused_qkv_a_proj_with_mqa.weight" in written and f"{pm}.gate_up_proj.weight_scale_inv" in written


def test_weight_loader_agrees_with_load_full_weight(parallel, checkpoint):
    files, t = checkpoint
    for tp_rank in (0, 1):
        parallel(tp=2, tp_rank=tp_rank)
        cfg = Fp8Config()
        a, b = MergedColumnParallelLinear(H, [I_DENSE, I_DENSE], quant_config=cfg), MergedColumnParallelLinear(H, [I_DENSE, I_DENSE], quant_config=cfg)
        m = "model.layers.0.mlp"
        full_w = torch.cat([t[f"{m}.gate_proj.weight"].view(torch.uint8), t[f"{m}.up_proj.weight"].view(torch.uint8)]).view(torch.float8_e4m3fn)
        full_s = torch.cat([t[f"{m}.gate_proj.weight_scale_inv"], t[f"{m}.up_proj.weight_scale_inv"]])
        a.load_full_weight(full_w, full_s)
        b.weight_loader(b.weight, full_w)               # stored fused on disk: no shard id
        b.weight_loader(b.weight_scale_inv, full_s)
        _same(a.weight, b.weight.data)
        _same(a.weight_scale_inv, b.weight_scale_inv.data)


@pytest.mark.parametrize("ep,ep_rank", [(1, 0), (2, 0), (2, 1), (4, 2)])
def test_experts_take_their_block(parallel, checkpoint, ep, ep_rank):
    files, t = checkpoint
    parallel(ep=ep, ep_rank=ep_rank)
    model = _Model()
    model.load_weights(safetensors_weights_iterator(files))
    blk = model.model.layers[1].mlp
    x = "model.layers.1.mlp"
    local = E // ep
    for j in range(local):
        e = ep_rank * local + j
        for kind in ("weight", "weight_scale_inv"):
            gate, up, down = (t[f"{x}.experts.{e}.{p}.{kind}"] for p in ("gate_proj", "up_proj", "down_proj"))
            w13 = getattr(blk.experts, f"w13_{kind}").data[j]
            w2 = getattr(blk.experts, f"w2_{kind}").data[j]
            if kind == "weight":
                gate, up, down, w13, w2 = (v.view(torch.uint8) for v in (gate, up, down, w13, w2))
            assert torch.equal(w13, torch.cat([gate, up])) and torch.equal(w2, down)
    # the shared expert is an ordinary merged / row-parallel pair under the same stacked mapping
    _same(blk.shared_experts.down_proj.weight, t[f"{x}.shared_experts.down_proj.weight"])
    _same(blk.shared_experts.gate_up_proj.weight_scale_inv,
          torch.cat([t[f"{x}.shared_experts.gate_proj.weight_scale_inv"], t[f"{x}.shared_experts.up_proj.weight_scale_inv"]]))


def test_redundant_experts_are_loaded_into_every_copy(parallel, checkpoint):
    files, t = checkpoint
    counts = torch.tensor([50., 1, 1, 40, 1, 1, 1, 1])
    for ep_rank in (0, 1):
        parallel(ep=2, ep_rank=ep_rank)
        loc = ExpertLocationMetadata.init_by_hot_replication(counts, 2, ep_rank, 2)
        model = _Model(loc)
        model.load_weights(safetensors_weights_iterator(files))
        experts = model.model.layers[1].mlp.experts
        mine = loc.local_logical_experts(ep_rank).tolist()
        assert len(mine) == E // 2 + 2 and sorted(mine[-2:]) == [0, 3]
        for j, e in enumerate(mine):
            down = t[f"model.layers.1.mlp.experts.{e}.down_proj.weight"]
            assert torch.equal(experts.w2_weight.data[j].view(torch.uint8), down.view(torch.uint8))
            gs = t[f"model.layers.1.mlp.experts.{e}.gate_proj.weight_scale_inv"]
            assert torch.equal(experts.w13_weight_scale_inv.data[j][: I_MOE // 128], gs)


def test_loader_errors(parallel, checkpoint):
    files, t = checkpoint
    parallel()
    model = _Model()
    with pytest.raises(KeyError):
        model.load_weights([("model.layers.0.mlp.nothing.weight", torch.zeros(1))])
    with pytest.raises(KeyError):   # one piece of a concatenated parameter is missing
        model.load_weights([("model.layers.0.self_attn.q_a_proj.weight", t["model.layers.0.self_attn.q_a_proj.weight"])])
    with pytest.raises(ValueError):  # a bf16 tensor where serialized fp8 is expected
        model.load_weights([("model.layers.0.self_attn.q_b_proj.weight", torch.zeros(Q_B, Q_LORA, dtype=torch.bfloat16))])
    with pytest.raises(ValueError):  # wrong shape
        model.load_weights([("model.layers.0.self_attn.o_proj.weight_scale_inv", torch.zeros(3, 3))])
