"""Reading a serialized block-FP8 checkpoint into the layers of the path.

The on-disk format (DeepSeek-V3 / Qwen3 FP8 releases): safetensors files whose tensors are named after the
Hugging Face modules; every quantised projection `<module>.weight` (float8_e4m3fn, [N, K]) comes with
`<module>.weight_scale_inv` (float32, [ceil(N/128), ceil(K/128)]), the multiplier that dequantises its 128x128
block.  After python/sglang/srt/model_loader/weight_utils.py (`safetensors_weights_iterator`, :547-590) and the
`load_weights` loop of python/sglang/srt/models/deepseek_v2.py:3749-3960, reduced to what the dense and MoE layers
of this path need:

* stacked parameters: checkpoint tensors that are one logical part of a merged layer
  (`gate_proj` / `up_proj` -> `gate_up_proj` parts 0 / 1; `q_proj` / `k_proj` / `v_proj` -> `qkv_proj`);
* expert parameters: `experts.<e>.<gate|up|down>_proj.*` -> `experts.w13_*` / `experts.w2_*`
  (`FusedMoE.make_expert_params_mapping`);
* concatenated parameters: tensors that the model keeps as one replicated matrix, joined along the output rows once
  all of them have been read (`q_a_proj` + `kv_a_proj_with_mqa` -> `fused_qkv_a_proj_with_mqa`, deepseek_v2.py:3346-3354);
* everything else by its own name.

Sharding is the layers' business (their `weight_loader`s); this file only routes names.
"""
from __future__ import annotations

from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch
from torch import nn


def safetensors_weights_iterator(files: Sequence[str], device: str = "cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    """(name, tensor) for every tensor of every file, in file order and name order within a file."""
    from safetensors import safe_open

    for path in files:
        with safe_open(path, framework="pt", device=device) as f:
            for name in sorted(f.keys()):
                yield name, f.get_tensor(name)


def _default_loader(param, loaded_weight: torch.Tensor) -> None:
    if tuple(param.shape) != tuple(loaded_weight.shape):
        raise ValueError(f"checkpoint tensor of shape {tuple(loaded_weight.shape)} for a parameter of shape "
                         f"{tuple(param.shape)}")
    if param.dtype == torch.float8_e4m3fn:
        param.data.view(torch.uint8).copy_(loaded_weight.view(torch.uint8))
    else:
        param.data.copy_(loaded_weight)


def load_block_fp8_weights(
    model: nn.Module,
    weights: Iterable[Tuple[str, torch.Tensor]],
    stacked_params_mapping: Sequence[Tuple[str, str, object]] = (),
    expert_params_mapping: Sequence[Tuple[str, str, int, str]] = (),
    concat_params_mapping: Optional[Dict[str, List[str]]] = None,
    ignore_unmatched: bool = False,
) -> List[str]:
    """Routes every checkpoint tensor to `param.weight_loader` of the parameter it belongs to and returns the names of
    the parameters that were written.  Raises KeyError for a tensor that matches nothing (unless
    `ignore_unmatched`) and for a concatenated parameter some of whose pieces never arrived."""
    params = dict(model.named_parameters())
    concat_params_mapping = concat_params_mapping or {}
    pending: Dict[str, Dict[str, torch.Tensor]] = {}
    written: List[str] = []

    def concat_target(name: str):
        for fused, pieces in concat_params_mapping.items():
            for piece in pieces:
                tag = f".{piece}."
                if tag in name:
                    return name.replace(tag, f".{fused}."), fused, piece, pieces
        return None

    for name, tensor in weights:
        if "rotary_emb.inv_freq" in name:
            continue
        done = False
        for param_name, weight_name, shard_id in stacked_params_mapping:
            if f".{weight_name}." not in name:
                continue
            if ".experts." in name and name not in params:  # per-expert tensors are handled below
                continue
            target = name.replace(f".{weight_name}.", f".{param_name}.")
            if target not in params:
                continue
            p = params[target]
            p.weight_loader(p, tensor, shard_id)
            written.append(target)
            done = True
            break
        if done:
            continue
        for param_name, weight_name, expert_id, shard_id in expert_params_mapping:
            if weight_name not in name:
                continue
            target = name.replace(weight_name, param_name)
            if target not in params:
                continue
            p = params[target]
            p.weight_loader(p, tensor, name, shard_id=shard_id, expert_id=expert_id)
            written.append(target)
            done = True
            break
        if done:
            continue
        hit = concat_target(name)
        if hit is not None and hit[0] in params:
            target, fused, piece, pieces = hit
            got = pending.setdefault(target, {})
            got[piece] = tensor
            if len(got) == len(pieces):
                joined = torch.cat([got[q].view(torch.uint8) if got[q].dtype == torch.float8_e4m3fn else got[q]
                                    for q in pieces], dim=0)
                if got[pieces[0]].dtype == torch.float8_e4m3fn:
                    joined = joined.view(torch.float8_e4m3fn)
                p = params[target]
                getattr(p, "weight_loader", _default_loader)(p, joined)
                written.append(target)
                del pending[target]
            continue
        if name in params:
            p = params[name]
            getattr(p, "weight_loader", _default_loader)(p, tensor)
            written.append(name)
        elif not ignore_unmatched:
            raise KeyError(f"checkpoint tensor {name} matches no parameter of the model")
    if pending:
        missing = {t: [q for q in concat_params_mapping[t.rsplit('.', 2)[-2]] if q not in got] for t, got in pending.items()}
        raise KeyError(f"concatenated parameters with pieces that never arrived: {missing}")
    return written
