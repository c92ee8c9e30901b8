"""The reference's own callers, built unchanged against this library: its C++ vector harness (reference
cuda/test_vectors.cu:21-72: every case of the frozen vectors under a sweep of variant / mb / nwarps / stages / nsplit, a
combination answered with cudaErrorInvalidValue is skipped, the rest must satisfy |d| - |ref|/64 <= tol) and its torch
binding (reference cuda/uq_ext.cpp:6-37, module `uq_cuda_ext`).  Both are compiled where the reference checkout is
(baseline/ref_gpu.py build_boundary: -I include, -luq_b200) and only run here; the vectors are written out from the
repacked fixtures in the reference's file layout.  Skipped when the two artefacts have not been built.  Needs a B200."""
import importlib.util
import os
import re
import subprocess

import numpy as np
import pytest
import torch

from tests.cases import GOLDEN, check_close

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HARNESS = os.path.join(ROOT, "baseline", "_ref", "test_vectors_b200")
EXT = os.path.join(ROOT, "baseline", "_ref", "uq_cuda_ext.so")
SETS = ("main", "gqa8_p128", "d64_p32", "p16_g4", "edge_short")


def write_vectors(dirname):
    """ref_cuda_<name>.npz -> <name>_{kc,ks,vc,vs,bt,sl}.bin, <name>_K<k>_{q,ref}.bin and manifest.txt (reference
    tools/gen_vectors.py:112: `case name K B HQ HKV D PAGE pages max_pages seq_lens...`)."""
    lines = []
    for name in SETS:
        z = np.load(os.path.join(GOLDEN, f"ref_cuda_{name}.npz"))
        B, HQ, HKV, D, PAGE, pages, mp = (int(x) for x in z["meta"])
        for key in ("kc", "ks", "vc", "vs", "bt", "sl"):
            np.ascontiguousarray(z[key]).tofile(os.path.join(dirname, f"{name}_{key}.bin"))
        for K in z["Ks"]:
            np.ascontiguousarray(z[f"q_K{K}"]).tofile(os.path.join(dirname, f"{name}_K{K}_q.bin"))
            np.ascontiguousarray(z[f"ref_K{K}"], dtype=np.float32).tofile(os.path.join(dirname, f"{name}_K{K}_ref.bin"))
            lines.append(" ".join(["case", name, str(int(K)), str(B), str(HQ), str(HKV), str(D), str(PAGE), str(pages), str(mp)] + [str(int(v)) for v in z["sl"]]))
    with open(os.path.join(dirname, "manifest.txt"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return len(lines)


@pytest.mark.skipif(not os.path.exists(HARNESS), reason="the reference's harness has not been built against this library (python baseline/ref_gpu.py --build)")
def test_the_references_vector_harness_passes_against_this_library(tmp_path):
    n = write_vectors(str(tmp_path))
    r = subprocess.run([HARNESS, str(tmp_path), "1e-2"], capture_output=True, text=True, timeout=600)
    tail = r.stdout[-1500:] + r.stderr[-500:]
    m = re.search(r"RESULT runs=(\d+) fails=(\d+)", r.stdout)
    assert m, tail
    runs, fails = int(m.group(1)), int(m.group(2))
    # 288 combinations per case in the harness's sweep (variant 1: 72, variant 2: 216); this library takes the hints as hints,
    # so every one of them is served
    assert r.returncode == 0 and fails == 0 and runs == 288 * n, tail
    assert r.stdout.count(" done") == n


@pytest.mark.skipif(not os.path.exists(EXT), reason="the reference's torch binding has not been built against this library (python baseline/ref_gpu.py --build)")
def test_the_references_torch_binding_runs_on_this_library():
    spec = importlib.util.spec_from_file_location("uq_cuda_ext", EXT)
    ext = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ext)
    assert ext.block_m(8, 64, 8) == 64 and ext.has_sm90() == 0
    assert ext.workspace_floats(8, 8, 64, 8, 128, 9) == 8 * 8 * 9 * 64 * 129
    z = np.load(os.path.join(GOLDEN, "ref_cuda_main.npz"))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for K in z["Ks"]:
        q = dev(z[f"q_K{K}"].view(np.int16)).view(torch.bfloat16)
        out = ext.decode(q, dev(z["kc"]), dev(z["ks"]), dev(z["vc"]), dev(z["vs"]), dev(z["bt"]), dev(z["sl"]),
                         4, 0, 0, 0, 0, float(q.shape[-1]) ** -0.5, None, None, None, 0, 1.0, 1.0)
        torch.cuda.synchronize()
        check_close(out.float().cpu().numpy(), z[f"ref_K{K}"], f"uq_cuda_ext.decode K={K}")
    with pytest.raises(RuntimeError, match="bt/sl must be int32"):
        ext.decode(q, dev(z["kc"]), dev(z["ks"]), dev(z["vc"]), dev(z["vs"]), dev(z["bt"]).long(), dev(z["sl"]), 4, 0, 0, 0, 0, 0.1, None, None, None, 0, 1.0, 1.0)
