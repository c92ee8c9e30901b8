"""Benchmark of the one hot path: speculative-verify attention over a paged UltraQuant FP4 KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--kq 8] [--config 1]

A step is one attention layer call on the headline configuration: B=8 sequences at context 32768,
Hq=64 / Hkv=8 / D=128, page 64, K draft queries (default 8), seeded synthetic data (bf16 N(0,1) queries,
fp32 N(0,1) K/V with a lognormal(0,0.5) multiplier per K channel, encoded to UltraQuant FP4 by this
library's append kernel, physical pages randomly permuted).  The metric is the KV-read throughput
(algorithmic KV bytes of the call / time) and, in ms_per_step, the time per layer call.

N > 1 (launched with torch.distributed.run, one rank per GPU): KV heads are partitioned across ranks with no
collective; every rank owns Hkv=8 heads of its own (per-GPU work fixed: weak scaling) and the value is the
bytes all ranks read over the slowest rank's time.

--impl reference times the CPU implementation of the same path (the C restatement of the reference's
uqmt.attn.reference, all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    1: dict(name="cfg1: B8 ctx32768 Hq64 Hkv8 D128 page64", B=8, ctx=32768, HQ=64, HKV=8, D=128, PAGE=64),
}


def peaks():
    """Measured roofline denominators of this pool (driver-written file), else the stated fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def kv_bytes(cfg, seq_lens):
    return int(sum(int(n) for n in seq_lens) * cfg["HKV"] * 2 * (cfg["D"] // 2 + cfg["D"] // 32))


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {getattr(nv, n): n[len("nvmlClocksEventReason"):] for n in dir(nv) if n.startswith("nvmlClocksEventReason") and isinstance(getattr(nv, n), int)}
        if not names:
            names = {getattr(nv, n): n[len("nvmlClocksThrottleReason"):] for n in dir(nv) if n.startswith("nvmlClocksThrottleReason") and isinstance(getattr(nv, n), int)}
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if bit and bits & bit and name not in ("None", "All", "GpuIdle"):
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------ data
def build_case(cfg, K, seed, device, copies=2):
    """Seeded synthetic cache(s) and queries on `device`; the cache is encoded by the library's append kernel."""
    import torch
    from all_quant_b200 import uq_cuda
    B, ctx, HQ, HKV, D, PAGE = (cfg[k] for k in ("B", "ctx", "HQ", "HKV", "D", "PAGE"))
    g = torch.Generator(device=device).manual_seed(seed)
    npg = (ctx + PAGE - 1) // PAGE
    pages = B * npg
    chan = torch.exp(0.5 * torch.randn(1, HKV, D, generator=g, device=device))
    perm = torch.randperm(pages, generator=g, device=device)
    bt = perm.reshape(B, npg).to(torch.int32).contiguous()
    kc = torch.empty(pages, HKV, PAGE, D // 2, dtype=torch.uint8, device=device)
    ks = torch.empty(pages, HKV, PAGE, D // 32, dtype=torch.uint8, device=device)
    vc, vs = torch.empty_like(kc), torch.empty_like(ks)
    pos = torch.arange(ctx, device=device)
    for b in range(B):
        k = torch.randn(ctx, HKV, D, generator=g, device=device) * chan
        v = torch.randn(ctx, HKV, D, generator=g, device=device)
        slots = bt[b].long()[pos // PAGE] * PAGE + pos % PAGE
        uq_cuda.append_kv(kc, ks, vc, vs, k, v, slots)
    q = torch.randn(B, K, HQ, D, generator=g, device=device).bfloat16()
    sl = torch.full((B,), ctx, dtype=torch.int32, device=device)
    caches = [(kc, ks, vc, vs)]
    for _ in range(copies - 1):   # identical bytes at other addresses, so consecutive steps never hit L2
        caches.append(tuple(t.clone() for t in (kc, ks, vc, vs)))
    return dict(q=q, bt=bt, sl=sl, caches=caches)


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_sample(cfg, K, case_np, steps, warmup):
    """Times the CPU oracle on sequence 0 (all KV heads, full context): 1/B of a layer call per step."""
    from oracle import uq_oracle as O
    q, kc, ks, vc, vs, bt, sl = case_np
    ts = []
    out = None
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        out = O.reference(q[:1], kc, ks, vc, vs, bt[:1], sl[:1])
        if i >= warmup:
            ts.append(time.perf_counter() - t0)
    return float(np.mean(ts)), out, O.max_threads()


def case_to_numpy(case, cache=0):
    kc, ks, vc, vs = (t.cpu().numpy() for t in case["caches"][cache])
    import torch
    q = case["q"].view(torch.int16).cpu().numpy().view(np.uint16)
    return q, kc, ks, vc, vs, case["bt"].cpu().numpy(), case["sl"].cpu().numpy()


def run_reference_arm(args, cfg):
    """The reference's CPU path (C restatement, all host threads) on a bounded sample; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import uq_oracle as O
    rng = np.random.default_rng(1001)
    B, ctx, HQ, HKV, D, PAGE = (cfg[k] for k in ("B", "ctx", "HQ", "HKV", "D", "PAGE"))
    K = args.kq
    npg = ctx // PAGE
    chan = np.exp(0.5 * rng.standard_normal((1, HKV, 1, D))).astype(np.float32)
    k = rng.standard_normal((npg, HKV, PAGE, D)).astype(np.float32) * chan
    v = rng.standard_normal((npg, HKV, PAGE, D)).astype(np.float32)
    kc, ks = O.quantize_fp4(k)
    vc, vs = O.quantize_fp4(v)
    bt = rng.permutation(npg).astype(np.int32).reshape(1, npg)
    inv = np.empty(npg, np.int64)
    inv[bt[0]] = np.arange(npg)
    kc, ks, vc, vs = (a[inv] for a in (kc, ks, vc, vs))
    q = O.bf16_bits(rng.standard_normal((1, K, HQ, D)).astype(np.float32))
    sl = np.array([ctx], np.int32)
    steps = max(1, args.steps)
    # keep the whole run within a few minutes: at most ~90 s of timed CPU work
    t0 = time.perf_counter()
    O.reference(q, kc, ks, vc, vs, bt, sl)
    one = time.perf_counter() - t0
    frac_heads = HKV
    while frac_heads > 1 and one * frac_heads / HKV * (steps + args.warmup) > 90.0:
        frac_heads //= 2
    sub = slice(0, frac_heads)
    kc2, ks2, vc2, vs2 = (np.ascontiguousarray(a[:, sub]) for a in (kc, ks, vc, vs))
    q2 = np.ascontiguousarray(q.reshape(1, K, HKV, HQ // HKV, D)[:, :, sub].reshape(1, K, -1, D))
    ts = []
    for i in range(args.warmup + steps):
        t0 = time.perf_counter()
        O.reference(q2, kc2, ks2, vc2, vs2, bt, sl)
        if i >= args.warmup:
            ts.append(time.perf_counter() - t0)
    sample_frac = frac_heads / (HKV * B)                 # of one layer call
    t_call = float(np.mean(ts)) / sample_frac            # seconds per full layer call, scaled linearly
    by = kv_bytes(cfg, [ctx] * B)
    val = by / t_call / 1e12
    sample = f"1 of {B} sequences x {frac_heads} of {HKV} kv heads, full context, K={K}; scaled linearly to a layer call"
    line = {"impl": "reference", "metric": "kv_read_throughput", "value": val, "unit": "TB/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": t_call * 1e3, "us_per_layer_call": t_call * 1e6, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg["name"] + f" K={K}", "kq": K},
            "cpu_baseline": {"value": val, "unit": "TB/s", "cores": O.max_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "tokens_verified_per_s": B * K / t_call}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ GPU arm
def run_ours(args, cfg):
    import torch
    import torch.distributed as dist
    from all_quant_b200 import uq_cuda

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    K = args.kq
    B, ctx, HQ, HKV, D, PAGE = (cfg[k] for k in ("B", "ctx", "HQ", "HKV", "D", "PAGE"))
    case = build_case(cfg, K, 1001 + rank, dev, copies=2)
    q, bt, sl, caches = case["q"], case["bt"], case["sl"], case["caches"]
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    nsplit = uq_cuda.auto_nsplit(B, HKV, bt.shape[1], sms, K, HQ // HKV)
    ws = torch.empty(uq_cuda.workspace_floats(B, K, HQ, HKV, D, nsplit), dtype=torch.float32, device=dev)
    out = torch.empty_like(q)
    by = kv_bytes(cfg, [ctx] * B)
    lib = uq_cuda.lib()

    def step(i, qq=q, oo=out):
        kc, ks, vc, vs = caches[i % len(caches)]
        return uq_cuda.uq_decode_cuda(qq, kc, ks, vc, vs, bt, sl, nsplit=nsplit, workspace=ws, out=oo)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    # ---- device-resident timing: exactly `steps` layer calls
    n0 = uq_cuda.launch_count()
    with ClockSampler(local) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
        barrier()
        ms_total = e0.elapsed_time(e1)
        launches = uq_cuda.launch_count() - n0
        # ---- dominant kernel alone: events recorded by the library around the verify kernel of each call
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for i, (a, b) in enumerate(pairs):
            a.record()
            b.record()      # a torch event gets its handle at its first record
            lib.uqb_debug_events(a.cuda_event, b.cuda_event)
            step(i)
        lib.uqb_debug_events(None, None)
        torch.cuda.synchronize()
        kern_ms = float(np.mean([a.elapsed_time(b) for a, b in pairs]))
        # ---- end to end through the public API with host buffers
        hq = q.cpu().pin_memory()
        hbt, hsl = bt.cpu().pin_memory(), sl.cpu().pin_memory()
        hout = torch.empty_like(hq).pin_memory()
        dq, dbt, dsl = torch.empty_like(q), torch.empty_like(bt), torch.empty_like(sl)

        def e2e_step(i):
            dq.copy_(hq, non_blocking=True)
            dbt.copy_(hbt, non_blocking=True)
            dsl.copy_(hsl, non_blocking=True)
            kc, ks, vc, vs = caches[i % len(caches)]
            o = uq_cuda.uq_decode_cuda(dq, kc, ks, vc, vs, dbt, dsl, nsplit=nsplit, workspace=ws, out=out)
            hout.copy_(o, non_blocking=True)

        for i in range(3):
            e2e_step(i)
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for i in range(args.steps):
            e2e_step(i)
        f1.record()
        barrier()
        e2e_ms = f0.elapsed_time(f1)
    ms_step = max_over_ranks(ms_total / args.steps)
    e2e_step_ms = max_over_ranks(e2e_ms / args.steps)
    status = uq_cuda.last_status()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = peaks()
    value = world * by / (ms_step * 1e-3) / 1e12
    achieved = by / (kern_ms * 1e-3) / 1e9
    line = {"metric": "kv_read_throughput", "value": value, "unit": "TB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_step, "us_per_layer_call": ms_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": cfg["name"] + f" K={K}", "kq": K, "nsplit": nsplit, "l2": f"two cache copies alternate; each {by / 1e6:.0f} MB copy exceeds the 126 MB L2" if by > 126e6 else "two cache copies alternate (each smaller than L2: not a valid bench size)",
                       "sharding": "kv heads partitioned across ranks, no collective" if world > 1 else "single GPU",
                       "kernel_path": {1: "cuda-core", 2: "tcgen05"}.get(uq_cuda.last_path(), "?")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "peak_kind": peak_kind, "kernel_us": kern_ms * 1e3, "algorithmic_bytes": by},
            "e2e": {"value": world * by / (e2e_step_ms * 1e-3) / 1e12, "unit": "TB/s", "us_per_layer_call": e2e_step_ms * 1e3,
                    "h2d_bytes_per_step": int(hq.numel() * 2 + hbt.numel() * 4 + hsl.numel() * 4), "d2h_bytes_per_step": int(hout.numel() * 2)},
            "gpu_launches": int(launches), "tokens_verified_per_s": world * B * K / (ms_step * 1e-3),
            "clocks": clk.summary(), "device_status": list(status)}
    # ---- CPU baseline beside it (N = 1 only), and a parity check of sequence 0 for free
    if world == 1 and not args.no_cpu:
        t_seq, ref0, cores = cpu_sample(cfg, K, case_to_numpy(case), steps=2, warmup=1)
        t_call = t_seq * B
        line["cpu_baseline"] = {"value": by / t_call / 1e12, "unit": "TB/s", "cores": cores, "kind": "port", "us_per_layer_call": t_call * 1e6,
                                "sample": f"sequence 0 of {B} (all kv heads, full context, K={K}), 2 timed runs; scaled x{B} to a layer call"}
        got = step(0).float().cpu().numpy()[:1]
        d = np.abs(got - ref0)
        line["parity"] = {"max_abs_err": float(d.max()), "mean_abs_err": float(d.mean()), "max_abs_ref": float(np.abs(ref0).max()),
                          "ok": bool(d.max() <= 1e-2 * np.abs(ref0).max() and d.mean() <= 1e-3), "checked": "sequence 0 vs CPU oracle"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kq", type=int, default=8, help="draft queries per sequence (K)")
    ap.add_argument("--config", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=0, help="override the context length (profiler captures use a shorter one; the JSON says so)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.ctx:
        cfg["ctx"] = args.ctx
        cfg["name"] = cfg["name"].replace("ctx32768", f"ctx{args.ctx}")
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
