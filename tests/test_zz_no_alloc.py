"""The allocation-free launch (uqb_decode_launch_static) against the ordinary launch, through the C ABI.

Some hosts of this library cannot allocate device memory around an attention call (all memory already belongs to
the engine's pool, or the framework they plug into forbids it once serving has started), so the library carries a
fixed scratch array for them.  This file is named to be collected last: a run that stops at the first failure has
then already exercised every other test.  Needs a B200."""
import ctypes

import numpy as np
import pytest
import torch

from all_quant_b200 import uq_cuda
from tests.cases import check_close, load_cases

pytestmark = pytest.mark.gpu


def _dev(a, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dt is None else t.view(dt)


@pytest.mark.parametrize("name", ["ref_cuda_main_K8", "gen_d256_K8"])
def test_static_scratch_launch_matches_the_ordinary_launch_twice_in_a_row(name):
    c = [x for x in load_cases() if x.name == name][0]
    L = uq_cuda.lib()
    q = _dev(c.q.view(np.int16), torch.bfloat16)
    kc, ks, vc, vs, bt, sl = (_dev(a) for a in (c.kc, c.ks, c.vc, c.vs, c.bt, c.sl))
    nsplit = 4
    # the ordinary entry point, with a caller-owned workspace
    ws = torch.empty(uq_cuda.workspace_floats(c.B, c.K, c.HQ, c.HKV, c.D, nsplit), dtype=torch.float32, device="cuda")
    want = torch.empty_like(q)
    p = uq_cuda._params(q, kc, ks, vc, vs, bt, sl, nsplit, c.sm_scale)
    p.out = want.data_ptr()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.uqb_decode_launch_ws(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), 0, 0, stream) == 0
    torch.cuda.synchronize()
    want = want.float().cpu().numpy()
    check_close(want, c.ref, "ordinary launch")
    # the allocation-free entry point: no scratch pointers at all, two calls back to back on the same stream
    assert int(L.uqb_workspace_bytes(ctypes.byref(p))) <= int(L.uqb_static_scratch_bytes())
    for attempt in range(2):
        got = torch.full_like(q, float("nan"))
        ps = uq_cuda._params(q, kc, ks, vc, vs, bt, sl, nsplit, c.sm_scale)
        ps.mo, ps.ml, ps.out = None, None, got.data_ptr()
        before = torch.cuda.memory_allocated()
        assert L.uqb_decode_launch_static(ctypes.byref(ps), 0, 0, stream) == 0
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        g = got.float().cpu().numpy()
        check_close(g, want, f"static launch, call {attempt + 1}, vs ordinary launch")
        check_close(g, c.ref, f"static launch, call {attempt + 1}, vs reference answer")
    assert uq_cuda.last_status()[0] == 0


def test_static_scratch_launch_refuses_what_does_not_fit():
    L = uq_cuda.lib()
    p = uq_cuda.UQParams()
    p.B, p.K, p.HQ, p.HKV, p.D, p.PAGE, p.max_pages, p.nsplit = 64, 8, 64, 8, 128, 64, 512, 128
    assert int(L.uqb_workspace_bytes(ctypes.byref(p))) > int(L.uqb_static_scratch_bytes())
    assert L.uqb_decode_launch_static(ctypes.byref(p), 0, 0, None) == uq_cuda.cudaErrorInvalidValue
    q = torch.zeros(64, 8, 64, 128, dtype=torch.bfloat16, device="cuda")
    c8 = torch.zeros(1, 8, 64, 64, dtype=torch.uint8, device="cuda")
    s8 = torch.zeros(1, 8, 64, 4, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="built-in scratch"):
        uq_cuda.uq_decode_static(q, c8, s8, c8, s8, torch.zeros(64, 512, dtype=torch.int32, device="cuda"),
                                 torch.ones(64, dtype=torch.int32, device="cuda"), torch.empty_like(q), nsplit=128)
