"""ctypes bindings for oracle/oracle.c (TEST INFRASTRUCTURE ONLY).

`load()` builds oracle/_build/liboracle.so with gcc on first use if it is
missing.  Same semantics as oracle/block_fp8_oracle.py, fast enough for
BASELINE-sized parity cases.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        subprocess.check_call(
            ["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-o", _SO, src, "-lm"]
        )
    return _SO


def load():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def e4m3_encode(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    load().oracle_e4m3_encode(_p(x), C.c_int64(x.size), _p(out))
    return out


def quant(x, dtype_code: int, group_size: int = 128, eps: float = 1e-10):
    """x: uint16 bits (dtype_code 0 bf16 / 1 fp16) or float32 (2), shape [..., K]."""
    x = np.ascontiguousarray(x)
    K = x.shape[-1]
    groups = x.size // group_size
    q = np.empty(x.shape, dtype=np.uint8)
    s = np.empty(x.shape[:-1] + (K // group_size,), dtype=np.float32)
    load().oracle_quant(_p(x), C.c_int(dtype_code), C.c_int64(groups), C.c_int(group_size), C.c_float(eps), _p(q), _p(s))
    return q, s


def moe_align(topk_ids, block_size: int, num_experts: int):
    ids = np.ascontiguousarray(topk_ids, dtype=np.int32).reshape(-1)
    max_padded = ids.size + (num_experts + 1) * (block_size - 1)
    sorted_ids = np.full(max_padded, -7, dtype=np.int32)
    expert_ids = np.full(-(-max_padded // block_size), -7, dtype=np.int32)
    post = np.zeros(1, dtype=np.int32)
    load().oracle_moe_align(_p(ids), C.c_int64(ids.size), C.c_int(num_experts), C.c_int(block_size), _p(sorted_ids), _p(expert_ids), _p(post))
    return sorted_ids, expert_ids, post


def block_gemm(a, a_s, b, b_s, bn: int = 128, bk: int = 128):
    a = np.ascontiguousarray(a, dtype=np.uint8)
    b = np.ascontiguousarray(b, dtype=np.uint8)
    a_s = np.ascontiguousarray(a_s, dtype=np.float32)
    b_s = np.ascontiguousarray(b_s, dtype=np.float32)
    M, K = a.shape
    N = b.shape[0]
    c = np.empty((M, N), dtype=np.uint16)
    load().oracle_block_gemm(_p(a), _p(a_s), _p(b), _p(b_s), C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int(bn), C.c_int(bk), _p(c), None)
    return c


def silu_and_mul(x_bits):
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, d2 = x.shape
    out = np.empty((rows, d2 // 2), dtype=np.uint16)
    load().oracle_silu_and_mul(_p(x), C.c_int64(rows), C.c_int64(d2 // 2), _p(out))
    return out


def moe_sum_reduce(x_bits, scale: float):
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    T, topk, H = x.shape
    out = np.empty((T, H), dtype=np.uint16)
    load().oracle_moe_sum_reduce(_p(x), C.c_int64(T), C.c_int64(topk), C.c_int64(H), C.c_float(scale), _p(out))
    return out
