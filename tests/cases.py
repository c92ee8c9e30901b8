"""Fixture loading and the two tolerance rules shared by the parity tests."""
import glob
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


class Case:
    """One known-answer attention case: cache bytes, page table, lengths, bf16 query bits, fp32 answer."""

    def __init__(self, name, z, K):
        self.name = f"{name}_K{K}"
        self.B, self.HQ, self.HKV, self.D, self.PAGE, self.pages, self.max_pages = (int(x) for x in z["meta"])
        self.K = K
        self.kc, self.ks, self.vc, self.vs = z["kc"], z["ks"], z["vc"], z["vs"]
        self.bt, self.sl = z["bt"], z["sl"]
        self.q = z[f"q_K{K}"]
        self.ref = z[f"ref_K{K}"]
        self.sm_scale = float(z["sm_scale"]) if "sm_scale" in z else self.D ** -0.5
        # NVFP4 sets carry the per-tensor scales; their scale arrays are e4m3fn bytes per 16 channels
        self.fmt = 1 if "ts" in z else 0
        self.k_ts, self.v_ts = (float(z["ts"][0]), float(z["ts"][1])) if "ts" in z else (1.0, 1.0)

    def __repr__(self):
        return self.name


def load_cases(pattern="*"):
    """Attention cases of the fixtures matching `pattern`; the NVFP4 sets only when the pattern names them."""
    out = []
    for f in sorted(glob.glob(os.path.join(GOLDEN, pattern + ".npz"))):
        base = os.path.basename(f)[:-4]
        if base in ("gen_codec", "gen_append", "tree_cases", "gen_rotate", "gen_nvfp4_quant", "gen_upstream"):
            continue
        if base.startswith("nvfp4_") and not pattern.startswith("nvfp4_"):
            continue
        z = np.load(f)
        for K in z["Ks"]:
            out.append(Case(base, z, int(K)))
    return out


def load(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def check_close(got, ref, what=""):
    """The acceptance rule of the benchmark contract: max|d| <= 1e-2 * max|ref| and mean|d| <= 1e-3."""
    got = np.asarray(got, np.float32)
    ref = np.asarray(ref, np.float32)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    d = np.abs(got - ref)
    mx = float(np.abs(ref).max()) if ref.size else 0.0
    assert d.max(initial=0.0) <= 1e-2 * mx + 1e-30, f"{what}: max|d|={d.max():.3e} > 1e-2*max|ref|={1e-2 * mx:.3e}"
    assert (d.mean() if d.size else 0.0) <= 1e-3, f"{what}: mean|d|={d.mean():.3e}"


def check_harness_rule(got, ref, what="", tol=1e-2):
    """The reference C++ harness rule for bf16 outputs (cuda/test_vectors.cu:54-63): |d| - |ref|/64 <= tol."""
    d = np.abs(np.asarray(got, np.float32) - ref) - np.abs(ref) / 64.0
    assert d.max(initial=0.0) <= tol, f"{what}: excess {d.max():.3e}"
