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


def _prototypes():
    """name -> (return type, [parameter types]) parsed from the header."""
    text = open(os.path.join(ROOT, "include", "hils_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(int|size_t|const char\*)\s+(hils_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text, flags=re.S):
        ret, name, params = m.group(1), m.group(2), m.group(3).strip()
        plist = [] if params in ("", "void") else [" ".join(x.split()) for x in params.split(",")]
        out[name] = (ret, plist)
    return out


def _kind(ctype_decl):
    """C parameter declaration -> the ctypes class the binding table must use."""
    d = ctype_decl
    if "*" in d:
        return ctypes.c_void_p
    base = d.rsplit(" ", 1)[0].replace("const ", "").strip()
    return {"int": ctypes.c_int, "float": ctypes.c_float, "size_t": ctypes.c_size_t, "int64_t": ctypes.c_int64}[base]


def test_binding_table_matches_header_prototypes():
    """Every ctypes signature has the header's arity, parameter kinds and return type: a wrong count
    or a float passed where the C side reads an int would corrupt the call silently."""
    from hils_attention_b200 import _lib
    protos = _prototypes()
    assert set(protos) == set(_lib.SIGNATURES)
    for name, (ret, params) in protos.items():
        restype, argtypes = _lib.SIGNATURES[name]
        want_ret = {"int": ctypes.c_int, "size_t": ctypes.c_size_t, "const char*": ctypes.c_char_p}[ret]
        assert restype is want_ret, f"{name}: return type {restype} vs header {ret}"
        assert len(argtypes) == len(params), f"{name}: {len(argtypes)} bound arguments vs {len(params)} in the header"
        for i, (a, d) in enumerate(zip(argtypes, params)):
            assert a is _kind(d), f"{name}: argument {i} ({d}) bound as {a}"


class _FakeCudaTensor:
    """Stands in for a CUDA tensor on a box without a GPU: only what _lib.ptr() reads."""
    is_cuda = True

    def __init__(self, index):
        import torch
        self.device = torch.device("cuda", index)

    def data_ptr(self):
        return 4096


def test_tensors_on_different_devices_are_refused_before_any_launch():
    """A call assembled from tensors of two devices raises on the host; nothing reaches the library."""
    import pytest
    from hils_attention_b200 import _lib
    _lib._pending().clear()
    _lib.ptr(_FakeCudaTensor(0))
    _lib.ptr(_FakeCudaTensor(1))
    with pytest.raises(RuntimeError, match="different devices"):
        _lib.stream()
    assert _lib._pending() == []
    # one device: the call's device is that device, whatever the process-wide current device is
    _lib.ptr(_FakeCudaTensor(1))
    _lib.ptr(_FakeCudaTensor(1))
    assert _lib._call_device().index == 1
    _lib._pending().clear()
