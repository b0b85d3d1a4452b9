"""Argument checks of the C ABI that happen on the host before anything is launched: they can be exercised
without a GPU (no call below reaches a kernel launch or a CUDA API call)."""
import ctypes as C

import pytest

from hils_attention_b200 import _lib

BAD_ARG, WORKSPACE = -1, -4
BF16 = _lib.BF16


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


def _err(lib):
    return lib.hils_last_error().decode()


def _paged_step(lib, *, chunk_size=64, D=64, K=4, h_q=4, h_kv=2, h_lmk=4, max_len=100, page_stride=4, ptr=0x1000,
                workspace=None, workspace_bytes=0):
    p = C.c_void_p(ptr)
    return lib.hils_decode_step_paged(p, p, p, p, p, p, p, page_stride, 8, p, max_len, p, None, 16, p, None, 2, h_q, h_kv, h_lmk,
                                      D, K, chunk_size, 128, 0, 0.125, BF16, workspace, workspace_bytes, None)


def test_paged_decode_step_refuses_what_its_kernels_do_not_cover(lib):
    assert _paged_step(lib, chunk_size=32) == BAD_ARG and "64 tokens" in _err(lib)
    assert _paged_step(lib, D=96) == BAD_ARG and "head dimension" in _err(lib)
    assert _paged_step(lib, K=64) == BAD_ARG and "topk" in _err(lib)
    assert _paged_step(lib, h_q=5) == BAD_ARG
    assert _paged_step(lib, h_lmk=3) == BAD_ARG and "chunk keys" in _err(lib)
    assert _paged_step(lib, h_q=32, h_kv=2, h_lmk=2) == BAD_ARG and "8 query heads" in _err(lib)


def test_paged_decode_step_checks_the_table_width_pointers_alignment_and_workspace(lib):
    assert _paged_step(lib, max_len=4 * 64, page_stride=4) == BAD_ARG and "page table" in _err(lib)     # token 257 needs a 5th page
    assert _paged_step(lib, max_len=17 * 64, page_stride=32) == BAD_ARG and "chunk keys" in _err(lib)   # 17 chunks, room for 16 keys
    assert _paged_step(lib, ptr=0) == BAD_ARG and "null" in _err(lib)
    assert _paged_step(lib, ptr=0x1002) == BAD_ARG and "aligned" in _err(lib)
    assert _paged_step(lib) == WORKSPACE and "workspace" in _err(lib)
    need = lib.hils_decode_step_paged_workspace_bytes(2, 4, 2, 4, 64, 4, 16, 0, BF16)
    assert need > 0 and need % 256 == 0
    assert _paged_step(lib, workspace=C.c_void_p(0x2000), workspace_bytes=need - 1) == WORKSPACE


def test_workspace_queries_are_host_arithmetic(lib):
    q = lib.hils_decode_step_paged_workspace_bytes
    assert q(2, 4, 2, 3, 64, 4, 16, 0, BF16) == 0                 # chunk keys with neither h_kv nor h_q heads
    assert q(2, 5, 2, 5, 64, 4, 16, 0, BF16) == 0                 # h_q not a multiple of h_kv
    assert q(4, 4, 2, 4, 64, 4, 16, 0, BF16) > q(2, 4, 2, 4, 64, 4, 16, 0, BF16)
    assert q(2, 4, 2, 4, 64, 4, 16, 1, BF16) >= q(2, 4, 2, 4, 64, 4, 16, 0, BF16)     # softmax1 adds a weight column
    # the streamed-keys selection needs its dot products: only from 512 chunk keys on, bf16
    big, small = q(2, 4, 2, 4, 64, 4, 1024, 0, BF16), q(2, 4, 2, 4, 64, 4, 256, 0, BF16)
    assert big - small >= 2 * 4 * 1024 * 4
    d = lib.hils_decode_step_workspace_bytes
    assert d(8, 4, 8, 64, 4, 16, 0, BF16) > 0 and d(8, 3, 8, 64, 4, 16, 0, BF16) == 0


def test_selection_and_sparse_entries_check_sizes_before_launching(lib):
    p = C.c_void_p(0x1000)
    rc = lib.hils_topk_fwd(p, p, p, None, None, None, p, p, None, None, 1, 8, 4, 2, 1, 64, 200, 64, 128, 1, 0, 0, 0.125, BF16, BF16,
                           None, 0, None)
    assert rc == BAD_ARG and "topk" in _err(lib)
    rc = lib.hils_topk_fwd(p, p, p, None, None, None, p, p, None, None, 1, 8, 4, 2, 1, 62, 4, 64, 128, 1, 0, 0, 0.125, BF16, BF16,
                           None, 0, None)
    assert rc == BAD_ARG and "multiple of 4" in _err(lib)
    # the selection of an empty call is a no-op that succeeds without touching the device
    assert lib.hils_topk_fwd(p, p, p, None, None, None, p, p, None, None, 1, 0, 4, 2, 1, 64, 4, 64, 128, 1, 0, 0, 0.125, BF16, BF16,
                             None, 0, None) == 0
