"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "sglang_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(sglb200_\w+)\s*\(", src)))


def test_header_symbols_exported():
    from sglang_b200 import _lib, build
    build.build()
    names = _declared()
    assert len(names) >= 12
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/sglang_b200.h but not exported"
    assert set(_lib.SIGNATURES) == set(names)


def test_abi_version_and_error_channel():
    from sglang_b200._lib import check, lib
    assert lib.sglb200_abi_version() == 2
    # a rejected call launches nothing and reports through the message channel (no GPU needed)
    rc = lib.sglb200_per_token_group_quant_fp8(None, 0, None, None, 4, 100, 128, 1e-10, -448.0, 448.0, 1, 1, None)
    assert rc == -1
    assert b"not divisible" in lib.sglb200_last_error()
    with pytest.raises(RuntimeError):
        check(rc)
    assert lib.sglb200_moe_align_workspace_bytes(100, 257) == 0
    assert lib.sglb200_moe_align_workspace_bytes(131072, 257) == (128 + 1) * 257 * 4  # 128 chunks of 1024 ids


def test_product_never_imports_the_oracle():
    bad = []
    for base, _, files in os.walk(os.path.join(ROOT, "sglang_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                if re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M) or "oracle/" in text:
                    bad.append(f)
    assert not bad, bad
