"""Where the experts of an expert-parallel MoE layer live, with redundant copies of the hot ones.

After python/sglang/srt/eplb/expert_location.py (`ExpertLocationMetadata`: `physical_to_logical_map`,
`logical_to_rank_dispatch_physical_map`, `num_physical_experts`, server argument `ep_num_redundant_experts`) and
python/sglang/srt/eplb/expert_location_dispatch.py:88-92 (`_topk_ids_logical_to_physical_static`: one gather of the
routed logical ids through this rank's dispatch map).  The reference places the redundant experts with its balancing
algorithms (`eplb_algorithms/`) from recorded expert distributions; here the placement is the simplest one that
removes the tail of a skewed routing, in two forms.  `init_by_hot_replication`: every rank keeps its block of the logical
experts and, after them, a copy of the same `num_redundant_per_rank` hottest logical experts, and every rank sends the
rows of a hot expert to its OWN copy; hot rows then never cross NVLink and are spread as evenly as the tokens are, and
only the cold experts keep their owners.  `init_by_load`: the hot experts live on every rank only, and the cold ones
are packed onto the ranks by their routed-row counts instead of by index, which also evens out what still travels.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class ExpertLocationMetadata:
    """One layer's placement, as seen from one rank."""

    physical_to_logical_map: torch.Tensor                # [num_physical_experts] int32, all ranks' slots in rank order
    logical_to_rank_dispatch_physical_map: torch.Tensor  # [num_logical_experts] int32: where THIS rank sends each expert
    num_logical_experts: int
    num_physical_experts: int
    num_local_physical_experts: int
    ep_size: int

    @staticmethod
    def init_by_hot_replication(logical_count: torch.Tensor, ep_size: int, ep_rank: int,
                                num_redundant_per_rank: int) -> "ExpertLocationMetadata":
        """`logical_count` [num_logical_experts]: routed rows per logical expert (summed over ranks, the same tensor
        on every rank).  Ties are broken towards the lower expert index so that every rank derives the same placement."""
        E = int(logical_count.numel())
        assert E % ep_size == 0 and 0 <= num_redundant_per_rank <= E
        owned = E // ep_size
        local = owned + num_redundant_per_rank
        count = logical_count.detach().to("cpu", torch.float64)
        order = sorted(range(E), key=lambda e: (-float(count[e]), e))
        hot = order[:num_redundant_per_rank]
        p2l = torch.empty(ep_size * local, dtype=torch.int32)
        for r in range(ep_size):
            base = r * local
            p2l[base : base + owned] = torch.arange(r * owned, (r + 1) * owned, dtype=torch.int32)
            for j, e in enumerate(hot):
                p2l[base + owned + j] = e
        # this rank's dispatch map: a cold expert goes to its owner's slot, a hot one to this rank's own copy (to the
        # original where this rank is the owner)
        l2p = torch.empty(E, dtype=torch.int32)
        for e in range(E):
            l2p[e] = (e // owned) * local + (e % owned)
        for j, e in enumerate(hot):
            if e // owned != ep_rank:
                l2p[e] = ep_rank * local + owned + j
        dev = logical_count.device
        return ExpertLocationMetadata(p2l.to(dev), l2p.to(dev), E, ep_size * local, local, ep_size)

    @staticmethod
    def init_by_load(logical_count: torch.Tensor, ep_size: int, ep_rank: int,
                     num_redundant_per_rank: int) -> "ExpertLocationMetadata":
        """Hot experts replicated, cold experts packed by load.  The `num_redundant_per_rank` most-routed logical
        experts live on EVERY rank (each rank serves its own tokens' rows of them) and nowhere else; the other experts
        are dealt out, most-routed first, each to the rank with the fewest routed rows so far that still has a free
        slot (longest-processing-time packing, the same number of slots on every rank), so that the rows that do cross
        NVLink arrive evenly.  Needs (experts - redundant) divisible by the number of ranks.  Deterministic: every rank
        derives the same placement from the same counts."""
        E = int(logical_count.numel())
        R = int(num_redundant_per_rank)
        assert 0 <= R < E and (E - R) % ep_size == 0, "(experts - redundant copies) must be divisible by the ranks"
        cold_slots = (E - R) // ep_size
        local = cold_slots + R
        count = logical_count.detach().to("cpu", torch.float64)
        order = sorted(range(E), key=lambda e: (-float(count[e]), e))
        hot, cold = order[:R], order[R:]
        owned = [[] for _ in range(ep_size)]
        load = [0.0] * ep_size
        for e in cold:
            r = min((r for r in range(ep_size) if len(owned[r]) < cold_slots), key=lambda r: (load[r], r))
            owned[r].append(e)
            load[r] += float(count[e])
        p2l = torch.empty(ep_size * local, dtype=torch.int32)
        l2p = torch.empty(E, dtype=torch.int32)
        for r in range(ep_size):
            base = r * local
            for j, e in enumerate(sorted(owned[r])):
                p2l[base + j] = e
                l2p[e] = base + j
            for j, e in enumerate(hot):
                p2l[base + cold_slots + j] = e
        for j, e in enumerate(hot):
            l2p[e] = ep_rank * local + cold_slots + j
        dev = logical_count.device
        return ExpertLocationMetadata(p2l.to(dev), l2p.to(dev), E, ep_size * local, local, ep_size)

    def local_logical_experts(self, ep_rank: int) -> torch.Tensor:
        """Logical expert held by each physical slot of rank `ep_rank` (for loading its weights)."""
        n = self.num_local_physical_experts
        return self.physical_to_logical_map[ep_rank * n : (ep_rank + 1) * n]


def topk_ids_logical_to_physical(topk_ids: torch.Tensor, info: ExpertLocationMetadata | None) -> torch.Tensor:
    """Static dispatch: routed logical ids -> physical slots through this rank's map; negative ids (no expert) stay."""
    if info is None:
        return topk_ids
    m = info.logical_to_rank_dispatch_physical_map
    phys = m[topk_ids.clamp_min(0).long()]
    return torch.where(topk_ids >= 0, phys, topk_ids.to(phys.dtype)).to(torch.int32)
