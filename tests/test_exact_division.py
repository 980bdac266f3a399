"""CPU proof obligation of the quantizer's division-free quotient (see quant8 in sglang_b200/csrc/quant.cu):
the reciprocal + two-FMA sequence must equal the IEEE quotient for every input the kernel can meet."""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def checker(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("exactdiv") / "exact_div_check")
    subprocess.check_call(["gcc", "-O2", "-mfma", "-fopenmp", "-ffp-contract=off", "-o", exe,
                           os.path.join(HERE, "exact_div_check.c"), "-lm"])
    return exe


@pytest.mark.parametrize("mode,min_pairs", [(0, 10**9), (1, 10**9), (2, 5 * 10**7)])
def test_reciprocal_fma_quotient_is_exact(checker, mode, min_pairs):
    bad, total = map(int, subprocess.check_output([checker, str(mode)]).split())
    assert total >= min_pairs
    assert bad == 0
