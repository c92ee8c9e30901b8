"""The reference's own CUDA kernels as the same-box GPU bar.

`build()` compiles the reference checkout's `cuda/uq_decode.cu` (its variants 1 and 2: the mma.sync split kernels, reference
cuda/uq_decode.cu:114-350 and cuda/uq_decode_w.cuh:55-310, with the combine kernel :353-388) for sm_100a, straight from
the checkout named by $UQ_REFERENCE, into the git-ignored baseline/_ref/ - no reference source
is copied into this repository.  It is built WITHOUT -DUQ_ENABLE_SM100: the reference's tcgen05 kernel (variant 4) ends a
wait that runs out in `__trap()` (reference cuda/uq_decode_sm100.cuh:23-30), which on a shared GPU is a fault, so it is
not run here; the figures the reference publishes for it were measured on another chip.

`sweep()` times the built library on a case of bench.py with the reference's own tuning protocol (reference
cuda/bench_cuda.py:62-75: variant x warps x stages x nsplit, CUDA events around back-to-back launches) and returns the
best configuration per K.  The library is loaded with RTLD_LOCAL through ctypes and called by its C++-mangled names, so it
lives beside libuq_b200.so (which exports the same names) without either seeing the other; all_quant_b200 never loads it.

    python baseline/ref_gpu.py --build            # here, where the checkout is
    python baseline/ref_gpu.py --sweep full       # on a B200: every candidate of the reference's tuning grid, K = 1 2 4 8
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
OUT_DIR = os.path.join(ROOT, "baseline", "_ref")
LIB = os.path.join(OUT_DIR, "libuq_ref_v12.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
LAUNCH = "_Z16uq_decode_launchRK8UQParamsiiP11CUstream_st"          # uq_decode_launch(UQParams const&, int, int, CUstream_st*)
DEFAULT_REFERENCE = os.path.join(os.sep, "root", "reference")   # where the build container keeps the checkout; $UQ_REFERENCE overrides
NSPLITS = (4, 5, 6, 7, 8, 9, 10, 11, 12, 14, 16, 18, 20, 24, 32, 48)   # reference cuda/bench_cuda.py:58


def build(force=False):
    """Compile the reference's kernels where its checkout is present; returns the library path or None."""
    ref = os.environ.get("UQ_REFERENCE", DEFAULT_REFERENCE)
    src = os.path.join(ref, "cuda", "uq_decode.cu")
    if not os.path.exists(src):
        return LIB if os.path.exists(LIB) else None
    if os.path.exists(LIB) and not force and os.path.getmtime(LIB) >= os.path.getmtime(src):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    # the reference's own flags (cuda/uq_cuda.py:19, cuda/setup.py:11) for the one architecture of this repository
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math", "-lineinfo", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "-I", os.path.join(ref, "cuda"), src, "-o", LIB]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the reference's CUDA kernels failed:\n" + r.stderr[-2000:])
    return LIB


HARNESS = os.path.join(OUT_DIR, "test_vectors_b200")
EXT = os.path.join(OUT_DIR, "uq_cuda_ext.so")


def build_boundary(force=False):
    """The reference's own callers built against THIS library, unchanged and straight from the checkout: its vector harness
    (cuda/test_vectors.cu:21-72) as a binary and its torch binding (cuda/uq_ext.cpp:6-37) as the module `uq_cuda_ext`, both
    compiled with -I include (this repository's uq_decode.h) and linked with libuq_b200.so.  Outputs go to baseline/_ref/.
    Returns the paths that exist afterwards."""
    ref = os.environ.get("UQ_REFERENCE", DEFAULT_REFERENCE)
    inc, libdir = os.path.join(ROOT, "include"), os.path.join(ROOT, "all_quant_b200")
    src_h, src_e = os.path.join(ref, "cuda", "test_vectors.cu"), os.path.join(ref, "cuda", "uq_ext.cpp")
    os.makedirs(OUT_DIR, exist_ok=True)
    rpath = "-Wl,-rpath,$ORIGIN/../../all_quant_b200"
    if os.path.exists(src_h) and (force or not os.path.exists(HARNESS)):
        cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-I", inc, src_h, "-L", libdir, "-luq_b200",
               "-Xlinker", "-rpath=$ORIGIN/../../all_quant_b200", "-o", HARNESS]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("building the reference's vector harness against libuq_b200.so failed:\n" + r.stderr[-2000:])
    if os.path.exists(src_e) and (force or not os.path.exists(EXT)):
        import sysconfig
        import torch
        from torch.utils import cpp_extension as ce
        incs = [inc, sysconfig.get_paths()["include"], "/usr/local/cuda/include"] + ce.include_paths()
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=uq_cuda_ext", "-DTORCH_API_INCLUDE_EXTENSION_H",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"] + [f"-I{i}" for i in incs] + [src_e, "-L", libdir, "-luq_b200", rpath,
               "-L", tlib, "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10", "-lc10_cuda", "-L", "/usr/local/cuda/lib64", "-lcudart", "-o", EXT]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("building the reference's torch binding against libuq_b200.so failed:\n" + r.stderr[-2000:])
    return [f for f in (HARNESS, EXT) if os.path.exists(f)]


def candidates(K, G, mode):
    """The reference's tuning grid (cuda/bench_cuda.py:62-69), or a short list around the configurations that won it."""
    bm = max(16, 1 << (K * G - 1).bit_length())
    if mode == "full":
        nws = {16: (1, 2, 4), 32: (2, 4), 64: (4, 8), 128: (8,)}[bm]
        c = [dict(variant=1, nwarps=nw, stages=st, nsplit=ns, mb=0) for nw in nws for st in (2, 3, 4) for ns in NSPLITS]
        c += [dict(variant=2, nwarps=nw, stages=st, nsplit=ns, mb=mb) for mb in (1, 2) for nw in (2, 4, 8, 16) for st in (2, 3, 4) for ns in NSPLITS]
        return c
    # (winners of the full grid on a B200 at the headline shape: K=1, 2 variant 2 / 2 warps / 2 stages / nsplit 9 / mb 1;
    #  K=4 variant 1 / 4 warps / 2 stages / nsplit 16; K=8 variant 1 / 4 warps / 3 stages / nsplit 9)
    nws = {16: (2, 4), 32: (4,), 64: (4, 8), 128: (8,)}[bm]
    c = [dict(variant=1, nwarps=nw, stages=st, nsplit=ns, mb=0) for nw in nws for st in (2, 3) for ns in (9, 16)]
    c += [dict(variant=2, nwarps=nw, stages=st, nsplit=ns, mb=1) for nw in (2, 4) for st in (2, 3) for ns in (9, 16)]
    c += [dict(variant=0, nwarps=0, stages=0, nsplit=9, mb=0)]   # the reference's own default choice
    return c


def sweep(case, K, HQ, HKV, D, PAGE, mode="short", iters=30, check_against=None):
    """Best reference configuration for this case: {"us": ..., "variant": ..., ...}, or {"unavailable": why}."""
    import torch
    from all_quant_b200 import uq_cuda
    if not os.path.exists(LIB):
        return {"unavailable": "baseline/_ref/libuq_ref_v12.so has not been built (python baseline/ref_gpu.py --build where the reference checkout is)"}
    L = ctypes.CDLL(LIB, mode=ctypes.RTLD_LOCAL)
    launch = getattr(L, LAUNCH)
    launch.argtypes = [ctypes.POINTER(uq_cuda.UQParams), ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    q, bt, sl, caches = case["q"], case["bt"], case["sl"], case["caches"]
    B = q.shape[0]
    bm = max(16, 1 << (K * (HQ // HKV) - 1).bit_length())
    ns_max = max(NSPLITS)
    mo = torch.empty(B * HKV * ns_max * bm * D, dtype=torch.float32, device=q.device)
    ml = torch.empty(B * HKV * ns_max * bm, dtype=torch.float32, device=q.device)
    out = torch.empty_like(q)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def params(c, i):
        kc, ks, vc, vs = caches[i % len(caches)]
        p = uq_cuda._params(q, kc, ks, vc, vs, bt, sl, c["nsplit"], D ** -0.5, c["variant"], c["mb"])
        p.mo, p.ml, p.out = mo.data_ptr(), ml.data_ptr(), out.data_ptr()
        return p

    def run(c, n):
        ps = [params(c, i) for i in range(len(caches))]
        for i in range(3):
            e = launch(ctypes.byref(ps[i % len(ps)]), c["nwarps"], c["stages"], stream)
            if e != 0:
                return None, e
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            launch(ctypes.byref(ps[i % len(ps)]), c["nwarps"], c["stages"], stream)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / n, 0

    best, tried, refused = None, 0, 0
    for c in candidates(K, HQ // HKV, mode):
        us, err = run(c, 10 if mode == "full" else iters)
        if us is None:
            if err != 1:   # 1 = cudaErrorInvalidValue = "this combination is not built": skipped, as the reference's own sweep does
                return {"unavailable": f"reference launch failed with cudaError {err} at {c}"}
            refused += 1
            continue
        tried += 1
        if best is None or us < best["us"]:
            best = dict(c, us=us)
    if best is None:
        return {"unavailable": "no candidate configuration was accepted"}
    us, _ = run(best, iters)     # the winner once more with the full iteration count
    best["us"] = us
    best.update(candidates=tried, refused=refused, mode=mode, iters=iters)
    if check_against is not None:   # the reference kernel's own answer next to this library's, same inputs
        run(best, 1)
        torch.cuda.synchronize()
        d = (out.float() - check_against.float()).abs()
        best["max_abs_diff_vs_this_library"] = float(d.max())
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--build", action="store_true")
    ap.add_argument("--sweep", choices=["short", "full"])
    ap.add_argument("--ks", type=int, nargs="+", default=[1, 2, 4, 8])
    a = ap.parse_args()
    if a.build:
        print(build(force=True))
        print(build_boundary(force=True))
    if a.sweep:
        import torch
        import bench
        from all_quant_b200 import uq_cuda
        cfg = bench.CONFIGS[1]
        res = {}
        for K in a.ks:
            case = bench.build_case(cfg, bench.shard_plan(cfg, 0, 1), K, 1001, torch.device("cuda", 0), copies=2)
            kc, ks, vc, vs = case["caches"][0]
            mine = uq_cuda.uq_decode_cuda(case["q"], kc, ks, vc, vs, case["bt"], case["sl"])
            res[K] = sweep(case, K, cfg["HQ"], cfg["HKV"], cfg["D"], cfg["PAGE"], a.sweep, check_against=mine)
            print(json.dumps({"K": K, "reference_gpu": res[K]}), flush=True)
            del case
            torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
