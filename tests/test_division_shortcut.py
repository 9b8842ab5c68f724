"""The 16-bit step kernels replace the IEEE division by one residual correction on an approximate reciprocal
(div16 in optimi_b200/csrc/mta_common.cuh).  That is only legitimate if the result is the correctly rounded
quotient for every operand pair the guard lets through; `oracle/div_shortcut_check.c` checks exactly that on the
host, exhaustively for bfloat16 operands and for float16 operands (here on every third significand to keep the
CPU suite short; the program's default visits all of them)."""

import os
import subprocess

import pytest

ORACLE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle")


@pytest.fixture(scope="module")
def checker():
    res = subprocess.run(["make", "-C", ORACLE, "_build/div_shortcut_check"], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    return os.path.join(ORACLE, "_build", "div_shortcut_check")


@pytest.mark.parametrize("args", [("bf16",), ("f16", "3")], ids=["bf16-exhaustive", "f16-every-third-significand"])
def test_shortcut_quotient_is_correctly_rounded(checker, args):
    res = subprocess.run([checker, *args], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert " 0 wrong" in res.stdout, res.stdout
