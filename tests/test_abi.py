"""The C-ABI library loads without a GPU and exports exactly what
include/flashrec_b200.h declares; the ctypes table matches the declarations."""

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "flashrec_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    decls = {}
    for m in re.finditer(r"\b(?:int|int64_t|const char\*)\s+(fr_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        n = 0 if args in ("", "void") else args.count(",") + 1
        decls[m.group(1)] = n
    return decls


def test_every_declared_symbol_is_exported(lib):
    decls = _declared()
    assert len(decls) >= 20
    for name in decls:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_ctypes_table_matches_header():
    from flashrec_b200 import _lib

    decls = _declared()
    assert set(decls) == set(_lib._SIGNATURES), set(decls) ^ set(_lib._SIGNATURES)
    for name, nargs in decls.items():
        assert len(_lib._SIGNATURES[name]) == nargs, name


def test_version_and_struct_layout(lib):
    from flashrec_b200 import _lib

    assert b"sm_100a" in lib.fr_version()
    assert ctypes.sizeof(_lib.FrTrie) == 112


def test_cpu_tensors_are_rejected_not_computed():
    import pytest
    import torch

    from flashrec_b200 import FlashRecKernelError
    from flashrec_b200.kernel.rms_fp8 import rmsnorm_per_token_quant_fp8

    with pytest.raises(FlashRecKernelError):
        rmsnorm_per_token_quant_fp8(torch.zeros(2, 64, dtype=torch.bfloat16), torch.ones(64, dtype=torch.bfloat16), 1e-6)
