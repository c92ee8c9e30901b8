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
