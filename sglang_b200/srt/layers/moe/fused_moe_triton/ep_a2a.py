"""Expert-parallel dispatch / combine over one all-to-all each way.

Replaces the DeepEP normal-mode dispatcher of the reference
(python/sglang/srt/layers/moe/token_dispatcher/deepep.py:377-390 quantise-before-send, :449-461
`buffer.dispatch`, :502-509 `buffer.combine`) with `all_to_all_single` of the process group (NCCL over
NVLink on GPUs; gloo in the CPU tests of this host logic).

Wire format of one dispatched row (one per (token, destination rank) pair, sent once even if several of
the token's experts live on that rank): H bytes of e4m3 codes, H/128 float32 scales, top_k int32 global
expert ids, top_k float32 weights.  Rows arrive ordered by (source rank, source token); the receiver
rewrites ids of experts it does not own to -1 (the convention of
token_dispatcher/standard.py:146-173) and runs the single-GPU MoE path on them.  Combine returns one
bf16 row per dispatched row; the source adds the rows of each token in ascending rank order in float32.
"""
from __future__ import annotations

from typing import List, NamedTuple, Tuple

import torch

from ....distributed import GroupCoordinator, get_moe_ep_group


class EPDispatchPlan(NamedTuple):
    send_token: torch.Tensor      # [S] source token of every sent row, grouped by destination rank
    send_splits: List[int]        # rows sent to each rank
    recv_splits: List[int]        # rows received from each rank
    slot: torch.Tensor            # [T, p] index of the returned row for (token, rank), or S (a zero row)


def plan_dispatch(topk_ids: torch.Tensor, num_local_experts: int, group: GroupCoordinator) -> EPDispatchPlan:
    """Which rows go where.  One host synchronisation (the split sizes) as in DeepEP's normal mode."""
    T, _ = topk_ids.shape
    p = group.world_size
    dest = torch.div(topk_ids.long(), num_local_experts, rounding_mode="floor")
    valid = (topk_ids >= 0) & (dest < p)  # -1 (no expert) and ids past the last expert go nowhere
    # a token goes to rank r if ANY of its valid slots names an expert of r (an OR over the slots: a row that
    # mixes a filtered slot with a valid one must not depend on which write lands last)
    ranks = torch.arange(p, device=topk_ids.device)
    mask = ((dest.unsqueeze(-1) == ranks) & valid.unsqueeze(-1)).any(dim=1)
    pairs = torch.nonzero(mask.t())            # rows sorted by (rank, token)
    send_token = pairs[:, 1].contiguous()
    counts = mask.sum(0).to(torch.int64)
    recv_counts = torch.empty_like(counts)
    group.all_to_all_single(recv_counts, counts, [1] * p, [1] * p)
    both = torch.stack([counts, recv_counts]).cpu()
    send_splits, recv_splits = both[0].tolist(), both[1].tolist()
    _check_kernel_status(topk_ids)  # the device has just been synchronised: a cheap place to notice a failed kernel
    S = int(send_token.numel())
    slot = torch.full((T, p), S, dtype=torch.int64, device=topk_ids.device)
    slot[pairs[:, 1], pairs[:, 0]] = torch.arange(S, device=topk_ids.device)
    return EPDispatchPlan(send_token, send_splits, recv_splits, slot)


def _check_kernel_status(t: torch.Tensor) -> None:
    """Raises if a bounded wait inside one of this library's kernels has expired (their outputs are then
    incomplete).  Called where the host has synchronised with the device anyway."""
    if not t.is_cuda:
        return
    from ..... import ops as _ops

    if _ops.gemm_status() != 0 or _ops.stream_status() != 0:
        raise RuntimeError("a pipeline wait inside a block-FP8 kernel expired: outputs of earlier calls are incomplete")


def pack_rows(xq: torch.Tensor, xs: torch.Tensor, ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    n = xq.shape[0]
    return torch.cat(
        [xq.view(torch.uint8).reshape(n, -1), xs.contiguous().view(torch.uint8).reshape(n, -1),
         ids.to(torch.int32).contiguous().view(torch.uint8).reshape(n, -1),
         w.to(torch.float32).contiguous().view(torch.uint8).reshape(n, -1)], dim=1).contiguous()


def unpack_rows(buf: torch.Tensor, hidden: int, groups: int, topk: int):
    o = 0
    q = buf[:, o : o + hidden].contiguous().view(torch.float8_e4m3fn); o += hidden
    s = buf[:, o : o + 4 * groups].contiguous().view(torch.float32); o += 4 * groups
    ids = buf[:, o : o + 4 * topk].contiguous().view(torch.int32); o += 4 * topk
    w = buf[:, o : o + 4 * topk].contiguous().view(torch.float32)
    return q, s, ids, w


def dispatch(xq, xs, topk_ids, topk_w, plan: EPDispatchPlan, group: GroupCoordinator, num_local_experts: int):
    """-> (codes [R,H], scales [R,H/128], local ids [R,k] with -1 for foreign experts, weights [R,k])."""
    hidden, groups, topk = xq.shape[1], xs.shape[1], topk_ids.shape[1]
    t = plan.send_token
    send = pack_rows(xq[t] if xq.dtype != torch.float8_e4m3fn else xq.view(torch.uint8)[t].view(torch.float8_e4m3fn),
                     xs[t], topk_ids[t], topk_w[t])
    recv = torch.empty((sum(plan.recv_splits), send.shape[1]), dtype=torch.uint8, device=send.device)
    group.all_to_all_single(recv, send, plan.recv_splits, plan.send_splits)
    q, s, ids, w = unpack_rows(recv, hidden, groups, topk)
    lo = max(group.rank_in_group, 0) * num_local_experts
    local = ids - lo
    local = torch.where((local >= 0) & (local < num_local_experts), local, torch.full_like(local, -1))
    return q, s, local.contiguous(), w.contiguous()


def combine(out_rows: torch.Tensor, plan: EPDispatchPlan, group: GroupCoordinator, num_tokens: int,
            routed_scaling_factor: float = 1.0) -> torch.Tensor:
    """Returns rows to their sources and sums them per token (float32, ascending rank) -> [T,H]."""
    H = out_rows.shape[1]
    S = int(plan.send_token.numel())
    if out_rows.is_cuda and H % 8 == 0 and out_rows.dtype in (torch.bfloat16, torch.float16):
        from ..... import ops as _ops

        back = torch.empty((S, H), dtype=out_rows.dtype, device=out_rows.device)
        group.all_to_all_single(back, out_rows.contiguous(), plan.send_splits, plan.recv_splits)
        return _ops.gather_sum_rows(back, plan.slot, routed_scaling_factor)  # slot S = "no row": skipped
    back = torch.zeros((S + 1, H), dtype=out_rows.dtype, device=out_rows.device)  # last row stays zero
    group.all_to_all_single(back[:S], out_rows.contiguous(), plan.send_splits, plan.recv_splits)
    acc = torch.zeros((num_tokens, H), dtype=torch.float32, device=out_rows.device)
    for r in range(group.world_size):
        acc += back[plan.slot[:, r]].float()
    if routed_scaling_factor != 1.0:
        acc *= routed_scaling_factor
    return acc.to(out_rows.dtype)


def ep_all_to_all_forward(layer, hidden_states: torch.Tensor, topk_output) -> torch.Tensor:
    """dispatch -> local block-FP8 experts -> combine, for `FusedMoE` with a2a_backend "nccl"."""
    from ..... import ops as _ops
    from .fused_moe import fused_experts_impl

    group = get_moe_ep_group()
    topk_w, topk_ids = topk_output[0], topk_output[1]
    T = hidden_states.shape[0]
    xq, xs = _ops.per_token_group_quant_fp8(hidden_states, 128)
    plan = plan_dispatch(topk_ids, layer.num_local_experts, group)
    q, s, local_ids, w = dispatch(xq, xs, topk_ids, topk_w, plan, group, layer.num_local_experts)
    if q.shape[0] > 0:
        out_rows = fused_experts_impl(
            q, layer.w13_weight, layer.w2_weight, w, local_ids, inplace=False, use_fp8_w8a8=True,
            w1_scale=layer.w13_weight_scale_inv, w2_scale=layer.w2_weight_scale_inv, block_shape=[128, 128],
            routed_scaling_factor=1.0, a1_scale=s, out_dtype=hidden_states.dtype, has_filtered_ids=True)
    else:
        out_rows = torch.empty((0, hidden_states.shape[1]), dtype=hidden_states.dtype, device=hidden_states.device)
    rsf = layer.moe_runner_config.routed_scaling_factor or 1.0
    return combine(out_rows, plan, group, T, rsf)
