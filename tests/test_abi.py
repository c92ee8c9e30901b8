"""The C-ABI library loads without a GPU, exports every symbol its headers declare, and its host-only
entry points agree with the reference's arithmetic.  No compute call is made here."""
import ctypes
import os
import re
import subprocess

import pytest

from all_quant_b200 import uq_cuda

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_c_symbols():
    text = open(os.path.join(ROOT, "include", "uq_b200.h")).read()
    return sorted(set(re.findall(r"\b(uqb_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    L = uq_cuda.lib()
    names = _declared_c_symbols()
    assert set(names) == set(uq_cuda.EXPORTS), (names, uq_cuda.EXPORTS)
    for n in names:
        assert hasattr(L, n), n


def test_cxx_surface_of_the_reference_header_is_exported():
    """The reference's binding and harness link against C++-mangled names (its header has no extern "C")."""
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", uq_cuda._LIB_PATH], capture_output=True, text=True).stdout
    for sig in ("uq_block_m(int, int, int)", "uq_mo_elems(UQParams const&)", "uq_ml_elems(UQParams const&)",
                "uq_workspace_bytes(UQParams const&)", "uq_decode_launch(UQParams const&, int, int, CUstream_st*)",
                "uq_decode_launch_ws(UQParams, void*, int, int, CUstream_st*)", "uq_has_sm90()"):
        assert sig in out, sig


def test_params_struct_is_136_bytes():
    assert ctypes.sizeof(uq_cuda.UQParams) == 136
    assert uq_cuda.UQParams.B.offset == 80 and uq_cuda.UQParams.v_ts.offset == 132


@pytest.mark.parametrize("K,HQ,HKV,bm", [(1, 64, 8, 16), (2, 64, 8, 16), (4, 64, 8, 32), (8, 64, 8, 64), (16, 64, 8, 128),
                                         (3, 14, 2, 32), (1, 8, 8, 16), (8, 32, 8, 32), (3, 8, 8, 16)])
def test_block_m_and_scratch_sizes(K, HQ, HKV, bm):
    e = uq_cuda.ext()
    assert e.block_m(K, HQ, HKV) == bm     # max(16, pow2(K * pow2(G))), reference cuda/uq_decode.cu:398
    assert uq_cuda._block_m(K, HQ, HKV) == bm   # the Python twin the call path uses
    B, D, ns = 8, 128, 9
    assert e.workspace_floats(B, K, HQ, HKV, D, ns) == B * HKV * ns * bm * (D + 1)
    assert e.has_sm90() == 0


def test_auto_nsplit_arithmetic():
    # reference tests/test_attn.py:85-93 / cuda/uq_cuda.py:34-37
    assert uq_cuda.auto_nsplit(8, 8, 512, 148) == 9
    assert uq_cuda.auto_nsplit(1, 1, 4, 148) == 4
    assert uq_cuda.auto_nsplit(64, 8, 512, 148) == 1
    assert uq_cuda.auto_nsplit(1, 1, 100000, 148) == 128


def test_cpu_tensors_are_refused_not_served_by_a_fallback():
    import torch
    q = torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16)
    c = torch.zeros(1, 1, 64, 64, dtype=torch.uint8)
    s = torch.zeros(1, 1, 64, 4, dtype=torch.uint8)
    with pytest.raises(RuntimeError):
        uq_cuda.uq_decode_cuda(q, c, s, c, s, torch.zeros(1, 1, dtype=torch.int32), torch.ones(1, dtype=torch.int32))


def _fake_params(**over):
    """A UQParams whose pointers are made-up, well-aligned addresses: only for calls that must be refused by the host-side
    checks before anything touches the device."""
    p = uq_cuda.UQParams()
    base = 0x7F0000000000
    for i, n in enumerate(("q", "kc", "ks", "vc", "vs", "block_table", "seq_lens", "mo", "ml", "out")):
        setattr(p, n, base + i * 0x100000)
    p.B, p.K, p.HQ, p.HKV, p.D, p.PAGE, p.max_pages, p.nsplit = 2, 4, 8, 2, 128, 64, 16, 4
    p.sm_scale = 128 ** -0.5
    for k, v in over.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("field,delta", [("kc", 1), ("kc", 8), ("q", 2), ("q", 8), ("mo", 4), ("ml", 2), ("out", 2), ("seq_lens", 1),
                                         ("block_table", 2)])
def test_misaligned_pointers_are_refused_before_any_launch(field, delta):
    """The alignment contract of the launch (q and kc 16 bytes, mo 8, ml / out / tables 4): a pointer that breaks it is
    answered with cudaErrorInvalidValue and nothing is enqueued - no kernel ever sees it."""
    L = uq_cuda.lib()
    p = _fake_params()
    setattr(p, field, getattr(p, field) + delta)
    n0 = L.uqb_launch_count()
    assert L.uqb_decode_launch(ctypes.byref(p), 0, 0, None) == uq_cuda.cudaErrorInvalidValue
    assert L.uqb_decode_partial_launch(ctypes.byref(p), None, ctypes.c_void_p(0x7F1000000000), ctypes.c_void_p(0x7F1000100000), None) == uq_cuda.cudaErrorInvalidValue
    assert L.uqb_launch_count() == n0


@pytest.mark.parametrize("over", [dict(K=0), dict(K=1 << 20), dict(HQ=7), dict(HKV=0), dict(D=96), dict(nsplit=0), dict(nsplit=129),
                                  dict(B=-1), dict(K=64, HQ=64, HKV=8), dict(PAGE=0), dict(fmt=2), dict(HQ=1 << 30, HKV=1)])
def test_out_of_range_arguments_are_refused_and_sizes_do_not_wrap(over):
    L = uq_cuda.lib()
    p = _fake_params(**over)
    n0 = L.uqb_launch_count()
    assert L.uqb_decode_launch(ctypes.byref(p), 0, 0, None) == uq_cuda.cudaErrorInvalidValue
    assert L.uqb_decode_launch_static(ctypes.byref(p), 0, 0, None) == uq_cuda.cudaErrorInvalidValue
    assert L.uqb_launch_count() == n0
    # the size helpers return (no endless loop, no wrapped product): zero elements for arguments outside the served ranges
    assert L.uqb_workspace_bytes(ctypes.byref(p)) < (1 << 62)
    assert L.uqb_block_m(1 << 30, 1 << 30, 1) == 1 << 30
