"""Generate `topk_native.npz` from the reference's torch-native routing functions.

    python tests/golden/make_golden_topk.py /path/to/reference

Pulls `biased_grouped_topk_impl` (python/sglang/srt/layers/moe/topk.py:665-738) and `fused_topk_torch_native`
(:427-456) out of the reference with `ast` (the `sglang` package itself cannot be imported here) and runs exactly
that source on seeded CPU tensors drawn the way sgl-kernel/tests/test_moe_fused_gate.py:30-33 and
sgl-kernel/tests/test_moe_topk_softmax.py draw them.  The two helpers the function calls after the arithmetic
(logical-to-physical id mapping, masking of padded tokens) are identity stubs: neither is used on this path.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from make_golden import HERE, _extract  # noqa: E402


def main(ref_root: str):
    ns = {
        "torch": torch, "F": F, "Optional": None.__class__, "ExpertLocationDispatchInfo": None,
        "topk_ids_logical_to_physical": lambda ids, info: ids,
        "_mask_topk_ids_padded_region": lambda ids, n: None,
    }
    src = _extract(os.path.join(ref_root, "python/sglang/srt/layers/moe/topk.py"),
                   ["biased_grouped_topk_impl", "fused_topk_torch_native"])
    exec("from __future__ import annotations\n" + src, ns)
    grouped, softmax_topk = ns["biased_grouped_topk_impl"], ns["fused_topk_torch_native"]

    out = {}
    # grouped gate: (experts, groups, topk_group, topk) of test_moe_fused_gate.py:15-19, 24 tokens each
    for i, (E, G, tg, k) in enumerate([(128, 4, 2, 4), (256, 8, 4, 8), (512, 16, 8, 16)]):
        for apply in (0, 1):
            torch.manual_seed(100 + i)
            x = torch.rand(24, E)
            bias = torch.rand(E)
            w, ids = grouped(x, x.clone(), bias, topk=k, renormalize=True, num_expert_group=G, topk_group=tg,
                             num_fused_shared_experts=0, routed_scaling_factor=2.5,
                             apply_routed_scaling_factor_on_output=bool(apply))
            tag = f"g{i}a{apply}"
            out[tag + "_x"], out[tag + "_bias"] = x.numpy(), bias.numpy()
            out[tag + "_w"], out[tag + "_ids"] = w.numpy(), ids.numpy().astype(np.int32)
            out[tag + "_cfg"] = np.array([E, G, tg, k], dtype=np.int32)
    # softmax top-k: (tokens, experts, topk)
    for i, (T, E, k) in enumerate([(19, 8, 2), (33, 64, 6), (16, 128, 8), (7, 60, 4)]):
        for renorm in (0, 1):
            torch.manual_seed(200 + i)
            x = torch.randn(T, E)
            w, ids = softmax_topk(x, x, k, bool(renorm))
            tag = f"s{i}r{renorm}"
            out[tag + "_x"] = x.numpy()
            out[tag + "_w"], out[tag + "_ids"] = w.float().numpy(), ids.numpy().astype(np.int32)
            out[tag + "_k"] = np.array(k, dtype=np.int32)
    path = os.path.join(HERE, "topk_native.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))
