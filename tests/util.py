"""Helpers shared by the tests: seeded inputs and torch <-> oracle conversions."""
import numpy as np
import torch

from oracle import block_fp8_oracle as O


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def to_f32_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().float().numpy()


def fp8_codes(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def codes_to_fp8(a: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to(device).view(torch.float8_e4m3fn)


def make_weight(n, k, seed, std=0.02, experts=None):
    g = torch.Generator().manual_seed(seed)
    shape = (n, k) if experts is None else (experts, n, k)
    w = (torch.randn(*shape, generator=g) * std).numpy()
    q, s = O.quant_weight_block_fp8(w)
    return q, s


def make_act(m, k, seed, dtype=torch.bfloat16, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).to(dtype)
    if outliers:
        x[torch.randn(x.shape, generator=g) < 0.001] *= 10
    return x


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    den = np.sqrt((a * a).sum() * (b * b).sum())
    return float((a * b).sum() / den) if den > 0 else 1.0


def assert_close_fp(out: np.ndarray, ref: np.ndarray, rtol=1e-2, atol=1e-2, min_cos=0.9999):
    """The tolerance of the block-FP8 GEMM / MoE outputs: rtol 1e-2, atol 1e-2, cosine >= 0.9999."""
    np.testing.assert_allclose(out, ref, rtol=rtol, atol=atol)
    assert cosine(out, ref) >= min_cos
