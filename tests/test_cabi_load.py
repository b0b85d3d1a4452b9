"""The C-ABI library builds, loads without a GPU, and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "hils_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hils_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_all_declared_symbols():
    from hils_attention_b200 import _lib, build
    path = build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/hils_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes table and header disagree"
    assert _lib.load().hils_version() >= 100


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    import hils_attention_b200 as hb
    x = torch.zeros(1, 4, 1, 8)
    with pytest.raises(RuntimeError):
        hb.flex_attn_tl(x, x, x, 2, 2)
