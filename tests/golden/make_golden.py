"""Generate the golden fixtures in this directory from the reference's own code.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It does not import the `sglang` package (it cannot be imported without its
serving dependencies).  Instead it pulls the torch-native oracle functions out
of the reference's test modules with `ast`, executes exactly that source on
CPU tensors, and stores seeded inputs and the outputs as small `.npz` files:

* python/sglang/test/test_block_fp8.py
    native_per_token_group_quant_fp8 (:23-48)
    native_w8a8_block_fp8_matmul     (:273-325)
    torch_w8a8_block_fp8_moe         (:418-447)
* test/srt/quant/test_fp8_kernel.py
    TestFP8Base._make_A / _make_B    (:22-100)  (constructive known answers;
    the only edit is device="cuda" -> "cpu")

The fixtures travel with the repository; the reference checkout is not needed
to run the tests.
"""
from __future__ import annotations

import ast
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def _extract(path: str, names, replace=()):
    src = open(path).read()
    tree = ast.parse(src)
    out = []
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in names:
            seg = ast.get_source_segment(src, node)
            # drop decorators such as @staticmethod; dedent methods
            lines = seg.splitlines()
            indent = len(lines[0]) - len(lines[0].lstrip())
            seg = "\n".join(l[indent:] if l.strip() else l for l in lines)
            for a, b in replace:
                seg = seg.replace(a, b)
            out.append(seg)
    assert len(out) == len(names), (names, len(out))
    return "\n\n".join(out)


class _SiluAndMul:
    # python/sglang/srt/layers/activation.py:68-70
    def forward_native(self, x):
        d = x.shape[-1] // 2
        return F.silu(x[..., :d]) * x[..., d:]


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def fp8_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy().copy()


def quant_w(w: torch.Tensor, bn=128, bk=128):
    """Weight block quantisation used for fixtures (per-block amax / 448)."""
    N, K = w.shape[-2:]
    nb, kb = -(-N // bn), -(-K // bk)
    wp = torch.zeros(*w.shape[:-2], nb * bn, kb * bk)
    wp[..., :N, :K] = w
    blk = wp.view(*w.shape[:-2], nb, bn, kb, bk)
    amax = blk.abs().amax(dim=(-3, -1), keepdim=True)
    s = amax / 448.0
    s = torch.where(s == 0, torch.ones_like(s), s)
    q = (blk / s).clamp(-448, 448).to(torch.float8_e4m3fn)
    q = q.view(*w.shape[:-2], nb * bn, kb * bk)[..., :N, :K].contiguous()
    return q, s.view(*w.shape[:-2], nb, kb).contiguous()


def main(ref_root: str):
    ns = {"torch": torch, "SiluAndMul": _SiluAndMul}
    exec(
        _extract(
            os.path.join(ref_root, "python/sglang/test/test_block_fp8.py"),
            ["native_per_token_group_quant_fp8", "native_w8a8_block_fp8_matmul", "torch_w8a8_block_fp8_moe"],
        ),
        ns,
    )
    kat = {"torch": torch}
    exec(
        _extract(
            os.path.join(ref_root, "test/srt/quant/test_fp8_kernel.py"),
            ["_make_A", "_make_B"],
            replace=[('device="cuda"', 'device="cpu"'), ("@staticmethod\n", "")],
        ),
        kat,
    )
    quant = ns["native_per_token_group_quant_fp8"]
    matmul = ns["native_w8a8_block_fp8_matmul"]
    moe = ns["torch_w8a8_block_fp8_moe"]

    # ---- quantizer: seeded N(0,1) bf16 with x10 outliers (sgl_kernel/test_utils.py:4-62) ----
    out = {}
    for i, (tokens, hidden, dt) in enumerate(
        [(7, 512, torch.bfloat16), (83, 1024, torch.bfloat16), (33, 2048, torch.bfloat16), (5, 384, torch.float16)]
    ):
        g = torch.Generator().manual_seed(tokens * 10000 + hidden)
        x = torch.randn(tokens, hidden, generator=g).to(dt)
        x[torch.randn(x.shape, generator=g) < 0.001] *= 10
        if i == 1:
            x[3, 128:256] = 0  # an all-zero group -> eps path
            x[4, 0] = 3.0e4  # large magnitude
        q, s = quant(x, 128)
        out[f"x{i}"] = bf16_bits(x) if dt == torch.bfloat16 else x.view(torch.int16).numpy().view(np.uint16).copy()
        out[f"q{i}"] = fp8_bits(q)
        out[f"s{i}"] = s.numpy().copy()
        out[f"dtype{i}"] = np.array(0 if dt == torch.bfloat16 else 1)
    np.savez_compressed(os.path.join(HERE, "quant_native.npz"), **out)

    # ---- block GEMM: M=17, N=320 (partial last block), K=512 ----
    torch.manual_seed(0)
    M, N, K = 17, 320, 512
    x = torch.randn(M, K).bfloat16()
    w = torch.randn(N, K) * 0.02
    wq, ws = quant_w(w)
    xq, xs = quant(x, 128)
    c = matmul(xq, wq, xs, ws, [128, 128], output_dtype=torch.bfloat16)
    np.savez_compressed(
        os.path.join(HERE, "gemm_native.npz"),
        x=bf16_bits(x), xq=fp8_bits(xq), xs=xs.numpy(), wq=fp8_bits(wq), ws=ws.numpy(), c=bf16_bits(c),
    )

    # ---- MoE: T=9, E=4, H=256, I=128, top-2 ----
    torch.manual_seed(1)
    T, E, H, I, topk = 9, 4, 256, 128, 2
    a = torch.randn(T, H).bfloat16()
    w1 = torch.randn(E, 2 * I, H) * 0.05
    w2 = torch.randn(E, H, I) * 0.05
    w1q, w1s = quant_w(w1)
    w2q, w2s = quant_w(w2)
    score = torch.randn(T, E)
    o = moe(a, w1q, w2q, w1s, w2s, score, topk, [128, 128])
    sm = torch.softmax(score, dim=-1, dtype=torch.float32)
    tw, ti = torch.topk(sm, topk)
    np.savez_compressed(
        os.path.join(HERE, "moe_native.npz"),
        a=bf16_bits(a), w1q=fp8_bits(w1q), w1s=w1s.numpy(), w2q=fp8_bits(w2q), w2s=w2s.numpy(),
        topk_w=tw.numpy(), topk_ids=ti.numpy().astype(np.int32), out=bf16_bits(o),
    )

    # ---- constructive known answers (test_fp8_kernel.py) ----
    torch.manual_seed(2)
    A, A_q, A_s = kat["_make_A"](64, 512, 128, torch.float8_e4m3fn)
    B, B_q, B_s = kat["_make_B"](512, 128 + 64, 128, torch.float8_e4m3fn)
    C_gt = A.to(torch.bfloat16) @ B.to(torch.bfloat16)
    np.savez_compressed(
        os.path.join(HERE, "kat_fp8_kernel.npz"),
        A=A.numpy(), A_q=fp8_bits(A_q), A_s=A_s.numpy(),
        B_q_t=fp8_bits(B_q.T.contiguous()), B_s_t=B_s.T.contiguous().numpy(), C_gt=bf16_bits(C_gt),
    )
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))
