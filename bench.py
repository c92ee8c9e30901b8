"""Benchmark of the one hot path: speculative-verify attention over a paged UltraQuant FP4 KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--kq 8] [--config 1]

Default (--config 1, the headline): a step is one attention layer call with B=8 sequences at context 32768,
Hq=64 / Hkv=8 / D=128, page 64, K draft queries (default 8), seeded synthetic data (bf16 N(0,1) queries,
fp32 N(0,1) K/V with a lognormal(0,0.5) multiplier per K channel, encoded to UltraQuant FP4 by this
library's append kernel, physical pages randomly permuted).  The metric is the KV-read throughput
(algorithmic KV bytes of the step / time) and, in ms_per_step, the time per step.

N > 1 (launched with torch.distributed.run, one rank per GPU), by configuration:
  1  every rank owns Hkv=8 heads of its own and runs the whole call (per-GPU work fixed: weak scaling, no collective);
  2  Mistral-7B-shaped step: 32 layers, each the append-quantize of the K new tokens per sequence and the verify
     call, B=8, context uniform in [8192, 16384], Hq=32 / Hkv=8; KV heads are divided across ranks (strong, no collective);
  3  ragged serving batch: B=32, context uniform in [4096, 65536], Hq=64 / Hkv=8; KV heads divided across ranks (strong);
  4  one long sequence: B=1, context 131072, Hq=32 / Hkv=4 / D=256; context pages divided across ranks, every rank
     emits partials, an NCCL all-gather and the log-sum-exp merge kernel follow inside the timed step (strong).
The value is the KV bytes all ranks read over the slowest rank's time.

The `e2e` object is the same metric through the public API with host buffers: every step copies its queries, page table
and lengths (and the append leg's new tokens) in from pinned host memory and its output back; two buffer sets, with the
copies on streams of their own beside the kernels, as a serving loop would run it (`serial_us_per_layer_call` is the
same steps with everything on one stream).

--impl reference times the CPU implementation of the same path (the C restatement of the reference's
uqmt.attn.reference, all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    1: dict(name="cfg1: B8 ctx32768 Hq64 Hkv8 D128 page64", B=8, ctx=32768, HQ=64, HKV=8, D=128, PAGE=64, shard="replicas", layers=1, append=False),
    2: dict(name="cfg2: 32 layers x (append + verify) B8 ctx U[8192,16384] Hq32 Hkv8 D128 page64", B=8, ctx=(8192, 16384), HQ=32, HKV=8, D=128,
            PAGE=64, shard="heads", layers=32, append=True),
    3: dict(name="cfg3: B32 ctx U[4096,65536] Hq64 Hkv8 D128 page64", B=32, ctx=(4096, 65536), HQ=64, HKV=8, D=128, PAGE=64, shard="heads",
            layers=1, append=False),
    4: dict(name="cfg4: B1 ctx131072 Hq32 Hkv4 D256 page64", B=1, ctx=131072, HQ=32, HKV=4, D=256, PAGE=64, shard="context", layers=1, append=False),
}


def seq_lengths(cfg):
    """Per-sequence context lengths (drafts included): fixed, or seeded uniform in the configured range; the same on every rank."""
    if isinstance(cfg["ctx"], tuple):
        lo, hi = cfg["ctx"]
        return np.random.default_rng(7).integers(lo, hi + 1, cfg["B"]).astype(np.int64)
    return np.full(cfg["B"], cfg["ctx"], np.int64)


def shard_plan(cfg, rank, world):
    """What this rank holds: its head counts, per-sequence local token counts and the global position of its first key."""
    lens = seq_lengths(cfg)
    mode = cfg["shard"] if world > 1 else "single"
    plan = dict(mode=mode, lens=lens, local=lens.copy(), off=0, hkv=cfg["HKV"], hq=cfg["HQ"])
    if mode == "heads":
        if cfg["HKV"] % world:
            raise SystemExit(f"config needs Hkv={cfg['HKV']} divisible by the number of ranks")
        plan["hkv"], plan["hq"] = cfg["HKV"] // world, cfg["HQ"] // world
    elif mode == "context":
        page = cfg["PAGE"]
        max_pages = int(-(-lens.max() // page))
        per = -(-max_pages // world)
        plan["off"] = rank * per * page
        plan["local"] = np.clip(lens - plan["off"], 0, per * page)
    return plan


def scale_bytes(cfg):
    """Scale bytes per cache row: one UE8M0 byte per 32 channels, or (--fmt 1, NVFP4) one e4m3fn byte per 16."""
    return cfg["D"] // (16 if cfg.get("fmt", 0) == 1 else 32)


def local_kv_bytes(cfg, plan):
    return int(plan["local"].sum() * plan["hkv"] * 2 * (cfg["D"] // 2 + scale_bytes(cfg)))


def peaks():
    """The measured copy bandwidth of MEASURED_PEAKS.json when the file is there, else the stated fallback figure."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# DRAM traffic of one launch of the attention kernel from the ncu capture summarised in the named file (dram__bytes_read.sum +
# dram__bytes_write.sum of a half-size headline call, whose algorithmic bytes are given beside it); None = no capture on record
TRAFFIC_PROFILE = {"source": "profiles/uq_verify_tc_kernel_ctx16384_K8_ncu_full.md", "dram_bytes": 145.7e6 + 12.5e6, "algorithmic_bytes": 142606336}


def kv_bytes(cfg, seq_lens):
    return int(sum(int(n) for n in seq_lens) * cfg["HKV"] * 2 * (cfg["D"] // 2 + scale_bytes(cfg)))


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """SM clock and throttle reasons while the timed regions run, sampled by an `nvidia-smi` child process every 20 ms (a
    sampling thread inside this process would take the interpreter lock from the loop that launches the steps: with 20 timed
    steps that showed as 7 us per step).  Falls back to "unsampled" when nvidia-smi cannot be started."""

    FIELDS = ("clocks.sm", "clocks.max.sm", "clocks_event_reasons.hw_slowdown", "clocks_event_reasons.hw_thermal_slowdown",
              "clocks_event_reasons.sw_thermal_slowdown", "clocks_event_reasons.sw_power_cap")
    NAMES = ("HwSlowdown", "HwThermalSlowdown", "SwThermalSlowdown", "SwPowerCap")

    def __init__(self, index):
        self.index, self.proc, self.lines = str(index), None, []
        try:   # the device's UUID names it whatever CUDA_VISIBLE_DEVICES does to the numbering
            import torch
            self.index = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
        except Exception:
            pass

    def __enter__(self):
        import subprocess
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", "--query-gpu=" + ",".join(self.FIELDS), "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            first = self.proc.stdout.readline()     # the child is up and sampling before anything is timed
            if first:
                self.lines.append(first)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                out, _ = self.proc.communicate(timeout=5)
                self.lines += out.splitlines()
            except Exception:
                self.proc.kill()

    def summary(self):
        mhz, max_mhz, reasons = [], None, set()
        for ln in self.lines:
            t = [x.strip() for x in ln.split(",")]
            if len(t) != len(self.FIELDS):
                continue
            try:
                mhz.append(float(t[0]))
                max_mhz = int(float(t[1]))
            except ValueError:
                continue
            for name, v in zip(self.NAMES, t[2:]):
                if v == "Active":
                    reasons.add(name)
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": max_mhz, "reasons": ["unsampled"]}
        # the median of the samples taken under load (the block also holds host-side pauses, where the clock may idle down)
        busy = [m for m in mhz if m >= 0.6 * max(mhz)] or mhz
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": max_mhz, "reasons": sorted(reasons), "samples": len(mhz), "how": "nvidia-smi -lms 20"}


# ------------------------------------------------------------------------------------------------ data
def build_case(cfg, plan, K, seed, device, copies=2, q_seed=None):
    """Seeded synthetic cache(s) and queries on `device` for this rank's shard; the cache is encoded by the
    library's append kernel.  Returns q, the page table, global seq_lens, pos_offset, `copies` caches with the
    same bytes at different addresses, and (for the append leg) the K newest tokens of every sequence with their slots."""
    import torch
    from all_quant_b200 import uq_cuda
    B, D, PAGE = cfg["B"], cfg["D"], cfg["PAGE"]
    hkv, hq, local, off = plan["hkv"], plan["hq"], plan["local"], plan["off"]
    g = torch.Generator(device=device).manual_seed(seed)
    npgs = [int(-(-n // PAGE)) for n in local]
    pages, width = max(1, sum(npgs)), max(1, max(npgs))
    chan = torch.exp(0.5 * torch.randn(1, hkv, D, generator=g, device=device))
    perm = torch.randperm(pages, generator=g, device=device).to(torch.int32)
    bt = torch.zeros(B, width, dtype=torch.int32, device=device)
    kc = torch.empty(pages, hkv, PAGE, D // 2, dtype=torch.uint8, device=device)
    ks = torch.empty(pages, hkv, PAGE, scale_bytes(cfg), dtype=torch.uint8, device=device)
    vc, vs = torch.empty_like(kc), torch.empty_like(ks)
    nvfp4 = cfg.get("fmt", 0) == 1
    # NVFP4: fixed per-tensor scales that put a block maximum of 32 (K) / 8 (V) at the top of the e4m3fn range
    k_ts, v_ts = (32.0 / (6 * 448), 8.0 / (6 * 448)) if nvfp4 else (1.0, 1.0)
    new_k, new_v, new_slots = [], [], []
    first = 0
    for b in range(B):
        n, npg = int(local[b]), npgs[b]
        bt[b, :npg] = perm[first:first + npg]
        first += npg
        if n == 0:
            continue
        pos = torch.arange(n, device=device)
        k = torch.randn(n, hkv, D, generator=g, device=device) * chan
        v = torch.randn(n, hkv, D, generator=g, device=device)
        slots = bt[b].long()[pos // PAGE] * PAGE + pos % PAGE
        if nvfp4:
            uq_cuda.append_kv_nvfp4(kc, ks, vc, vs, k, v, slots, k_ts, v_ts)
        else:
            uq_cuda.append_kv(kc, ks, vc, vs, k, v, slots)
        # the K newest tokens of the sequence (global positions len-K .. len-1) that fall into this shard
        lo = max(0, int(plan["lens"][b]) - K - off)
        if lo < n:
            new_k.append(k[lo:].bfloat16())
            new_v.append(v[lo:].bfloat16())
            new_slots.append(slots[lo:])
    # (a context split hands every rank the same queries: they come from a generator of their own there)
    gq = g if q_seed is None else torch.Generator(device=device).manual_seed(q_seed)
    q = torch.randn(B, K, hq, D, generator=gq, device=device).bfloat16()
    sl = torch.tensor(plan["lens"], dtype=torch.int32, device=device)
    po = torch.full((B,), off, dtype=torch.int32, device=device)
    caches = [(kc, ks, vc, vs)]
    for _ in range(copies - 1):   # identical bytes at other addresses, so consecutive calls never hit L2
        caches.append(tuple(t.clone() for t in (kc, ks, vc, vs)))
    cat = lambda xs: torch.cat(xs).contiguous() if xs else None
    return dict(q=q, bt=bt.contiguous(), sl=sl, po=po, caches=caches, new_k=cat(new_k), new_v=cat(new_v), new_slots=cat(new_slots),
                k_ts=k_ts, v_ts=v_ts)


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_sample(case_np, steps, warmup, nvfp4=None):
    """Times the CPU oracle on sequence 0 (all KV heads, full context) of one layer; nvfp4 = (k_ts, v_ts) for an NVFP4 cache."""
    from oracle import uq_oracle as O
    O.set_threads(0)
    q, kc, ks, vc, vs, bt, sl = case_np
    ts = []
    out = None
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        out = O.reference_nvfp4(q[:1], kc, ks, vc, vs, bt[:1], sl[:1], *nvfp4) if nvfp4 else O.reference(q[:1], kc, ks, vc, vs, bt[:1], sl[:1])
        if i >= warmup:
            ts.append(time.perf_counter() - t0)
    return float(np.mean(ts)), out, O.max_threads()


def case_to_numpy(case, cache=0):
    import torch
    kc, ks, vc, vs = (t.cpu().numpy() for t in case["caches"][cache])
    q = case["q"].view(torch.int16).cpu().numpy().view(np.uint16)
    return q, kc, ks, vc, vs, case["bt"].cpu().numpy(), case["sl"].cpu().numpy()


def run_reference_arm(args, cfg):
    """The reference's CPU path (C restatement, all host threads) on a bounded sample; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import uq_oracle as O
    O.set_threads(0)   # all host cores: a launcher's OMP_NUM_THREADS=1 for its workers is not this arm's choice
    rng = np.random.default_rng(1001)
    B, HQ, HKV, D, PAGE = (cfg[k] for k in ("B", "HQ", "HKV", "D", "PAGE"))
    lens = seq_lengths(cfg)
    ctx = int(lens[0])
    K = args.kq
    npg = -(-ctx // PAGE)
    chan = np.exp(0.5 * rng.standard_normal((1, HKV, 1, D))).astype(np.float32)
    k = rng.standard_normal((npg, HKV, PAGE, D)).astype(np.float32) * chan
    v = rng.standard_normal((npg, HKV, PAGE, D)).astype(np.float32)
    nvfp4 = cfg.get("fmt", 0) == 1
    if nvfp4:   # the time does not depend on the values: random codes, scale bytes around one
        kc, vc = (rng.integers(0, 256, (npg, HKV, PAGE, D // 2), dtype=np.uint8) for _ in range(2))
        ks, vs = (rng.integers(0x30, 0x40, (npg, HKV, PAGE, D // 16)).astype(np.uint8) for _ in range(2))
        ref = lambda *a: O.reference_nvfp4(*a, 0.05, 0.05)
    else:
        kc, ks = O.quantize_fp4(k)
        vc, vs = O.quantize_fp4(v)
        ref = O.reference
    bt = rng.permutation(npg).astype(np.int32).reshape(1, npg)
    inv = np.empty(npg, np.int64)
    inv[bt[0]] = np.arange(npg)
    kc, ks, vc, vs = (a[inv] for a in (kc, ks, vc, vs))
    q = O.bf16_bits(rng.standard_normal((1, K, HQ, D)).astype(np.float32))
    sl = np.array([ctx], np.int32)
    steps = max(1, args.steps)
    # keep the whole run within a few minutes: at most ~90 s of timed CPU work
    t0 = time.perf_counter()
    ref(q, kc, ks, vc, vs, bt, sl)
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
        ref(q2, kc2, ks2, vc2, vs2, bt, sl)
        if i >= args.warmup:
            ts.append(time.perf_counter() - t0)
    # fraction of one step the sample covers: its tokens x heads over all sequences, heads and layers
    sample_frac = ctx * frac_heads / (float(lens.sum()) * HKV * cfg["layers"])
    t_step = float(np.mean(ts)) / sample_frac            # seconds per full step, scaled linearly
    by = kv_bytes(cfg, lens) * cfg["layers"]
    val = by / t_step / 1e12
    sample = (f"sequence 0 ({ctx} tokens) of {B} x {frac_heads} of {HKV} kv heads, one layer of {cfg['layers']}, K={K}; "
              "scaled linearly by tokens x heads x layers to a step" + ("; the append leg is not in the sample" if cfg["append"] else ""))
    line = {"impl": "reference", "metric": "kv_read_throughput", "value": val, "unit": "TB/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": t_step * 1e3, "us_per_layer_call": t_step * 1e6 / cfg["layers"], "higher_is_better": True,
            "scaling": "weak" if cfg["shard"] == "replicas" else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg["name"] + f" K={K}", "kq": K},
            "cpu_baseline": {"value": val, "unit": "TB/s", "cores": O.max_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "tokens_verified_per_s": B * K / t_step}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ GPU arm
Q_SEED = 4242   # the queries of a context split are the same on every rank


class Run:
    """This rank's share of one configuration: the seeded case, caller-owned scratch and output, and the step function."""

    def __init__(self, cfg, K, rank, world, dev, exchange="peer", copies=None, group=None):
        import torch
        from all_quant_b200 import uq_cuda
        self.cfg, self.K, self.rank, self.world, self.dev = cfg, K, rank, world, dev
        self.plan = shard_plan(cfg, rank, world)
        self.mode, hkv, hq = self.plan["mode"], self.plan["hkv"], self.plan["hq"]
        self.layers, self.fmt = cfg["layers"], cfg.get("fmt", 0)
        # one cache per layer; a single-layer configuration alternates two copies so that no call finds its cache in L2
        self.case = build_case(cfg, self.plan, K, 1001 + rank, dev, copies=copies or (self.layers if self.layers > 1 else 2),
                               q_seed=Q_SEED if cfg["shard"] == "context" else None)
        c = self.case
        self.q, self.bt, self.sl, self.po, self.caches = c["q"], c["bt"], c["sl"], c["po"], c["caches"]
        B, D = cfg["B"], cfg["D"]
        self.nsplit = uq_cuda.auto_nsplit(B, hkv, self.bt.shape[1], uq_cuda._sm_count(dev), K, hq // hkv)
        self.ws = torch.empty(uq_cuda.workspace_floats(B, K, hq, hkv, D, self.nsplit), dtype=torch.float32, device=dev)
        self.out = torch.empty_like(self.q)
        self.by_local = local_kv_bytes(cfg, self.plan)                                         # one layer, this rank
        self.by_step = kv_bytes(cfg, self.plan["lens"]) * self.layers * (world if self.mode == "replicas" else 1)   # one step, all ranks
        self.cache_bytes = sum(t.numel() for t in self.caches[0])
        self.exchange = exchange if self.mode == "context" else None
        self.cs = uq_cuda.ContextSplit(B * K * hq, D, group=group) if self.exchange == "peer" else None
        self.uq = uq_cuda

    def step(self, i, q=None, bt=None, sl=None, out=None, fused=True):
        uq, c, cfg = self.uq, self.case, self.cfg
        q = self.q if q is None else q
        bt = self.bt if bt is None else bt
        sl = self.sl if sl is None else sl
        out = self.out if out is None else out
        o = None
        for layer in range(self.layers):
            kc, ks, vc, vs = self.caches[(i * self.layers + layer) % len(self.caches)]
            if cfg["append"] and c["new_k"] is not None:
                uq.append_kv(kc, ks, vc, vs, c["new_k"], c["new_v"], c["new_slots"])
            if self.exchange == "peer":
                o = self.cs.run(q, kc, ks, vc, vs, bt, sl, self.po, out=out, nsplit=self.nsplit)
            elif self.exchange == "nccl":
                o = uq.uq_decode_context_split(q, kc, ks, vc, vs, bt, sl, self.po, nsplit=self.nsplit)
            elif fused:
                o = uq.uq_decode_cuda(q, kc, ks, vc, vs, bt, sl, nsplit=self.nsplit, workspace=self.ws, out=out, fmt=self.fmt,
                                      k_ts=c["k_ts"], v_ts=c["v_ts"])
            else:   # the reference's no-sharing mode: K single-query problems, the cache read K times (it allocates its own scratch)
                o = uq.uq_decode_cuda(q, kc, ks, vc, vs, bt, sl, fused=False, fmt=self.fmt, k_ts=c["k_ts"], v_ts=c["v_ts"])
        return o

    def close(self):
        if self.cs is not None:
            self.cs.close()


def parity_of(run, got):
    """Sequence 0 of this rank's output against the CPU oracle on the cache bytes the kernel read (rank 0 calls this).
    Head-partitioned and replicated runs: this rank's own heads.  Context split: the other ranks' shards are rebuilt here from
    their seeds and sequence 0's pages put in logical order, so the merged output is checked against the whole context."""
    import torch
    from oracle import uq_oracle as O
    O.set_threads(0)
    cfg, K = run.cfg, run.K
    nv = (run.case["k_ts"], run.case["v_ts"]) if run.fmt == 1 else None
    if run.mode == "context" and run.world > 1:
        PAGE = cfg["PAGE"]
        parts = []
        for r in range(run.world):
            pl = shard_plan(cfg, r, run.world)
            cr = run.case if r == run.rank else build_case(cfg, pl, K, 1001 + r, run.dev, copies=1, q_seed=Q_SEED)
            npg = int(-(-int(pl["local"][0]) // PAGE))
            idx = cr["bt"][0, :npg].long()
            parts.append(tuple(t[idx].cpu().numpy() for t in cr["caches"][0]))
            del cr
        kc, ks, vc, vs = (np.concatenate([p[i] for p in parts]) for i in range(4))
        bt = np.arange(kc.shape[0], dtype=np.int32)[None]
        q = run.q.view(torch.int16).cpu().numpy().view(np.uint16)[:1]
        ref = O.reference(q, kc, ks, vc, vs, bt, run.plan["lens"][:1].astype(np.int32))
        what = f"sequence 0 (whole context, {run.world} shards reassembled on rank 0) vs CPU oracle"
    else:
        q, kc, ks, vc, vs, bt, sl = case_to_numpy(run.case)
        ref = O.reference_nvfp4(q[:1], kc, ks, vc, vs, bt[:1], sl[:1], *nv) if nv else O.reference(q[:1], kc, ks, vc, vs, bt[:1], sl[:1])
        what = "sequence 0 vs CPU oracle" + (f" (rank 0's {run.plan['hkv']} kv heads)" if run.world > 1 else "")
    d = np.abs(got[:1] - ref)
    return {"max_abs_err": float(d.max()), "mean_abs_err": float(d.mean()), "max_abs_ref": float(np.abs(ref).max()),
            "ok": bool(d.max() <= 1e-2 * np.abs(ref).max() and d.mean() <= 1e-3), "checked": what}


def append_prompt(dev, peak, HKV, D, PAGE, tokens, iters=10, seed=77):
    """The append-quantize of a prompt: `tokens` tokens' keys and values (the benchmark's distributions: N(0,1), keys with a
    lognormal(0, 0.5) multiplier per channel) encoded and scattered into randomly permuted pages, as bf16 and as fp32 input.
    Algorithmic bytes = both input tensors + the codes and scale bytes written + the slot list; inputs (over a gigabyte at
    the default size) and the cache written are larger than L2.  The rows of the first 512 tokens are checked against the
    CPU oracle, and the per-row kernel (the one a decode step takes) is timed on the same call for contrast."""
    import torch
    from all_quant_b200 import uq_cuda
    from oracle import uq_oracle as O
    g = torch.Generator(device=dev).manual_seed(seed)
    pages = (tokens + PAGE - 1) // PAGE
    chan = torch.exp(0.5 * torch.randn(1, HKV, D, generator=g, device=dev))
    k32 = torch.randn(tokens, HKV, D, generator=g, device=dev) * chan
    v32 = torch.randn(tokens, HKV, D, generator=g, device=dev)
    perm = torch.randperm(pages, generator=g, device=dev)
    slots = (perm[:, None] * PAGE + torch.arange(PAGE, device=dev)[None, :]).reshape(-1)[:tokens].contiguous()
    kc = torch.zeros(pages, HKV, PAGE, D // 2, dtype=torch.uint8, device=dev)
    ks = torch.zeros(pages, HKV, PAGE, D // 32, dtype=torch.uint8, device=dev)
    vc, vs = torch.zeros_like(kc), torch.zeros_like(ks)
    out = {"workload": f"append of {tokens} tokens x {HKV} kv heads x D{D}, keys and values, page {PAGE}, pages permuted", "peak_GBs": peak}
    for name, dt in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        k, v = k32.to(dt), v32.to(dt)
        by = 2 * tokens * HKV * (D * k.element_size() + D // 2 + D // 32) + tokens * 8
        ent = {"algorithmic_bytes": by}
        for kernel in ("bulk", "rows"):
            n = iters if kernel == "bulk" else 3
            for _ in range(3):
                uq_cuda.append_kv(kc, ks, vc, vs, k, v, slots, kernel=kernel)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                uq_cuda.append_kv(kc, ks, vc, vs, k, v, slots, kernel=kernel)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / n
            ent[f"{kernel}_kernel_us"] = us
            if kernel == "bulk":
                ent["GB/s"] = by / us / 1e3
                ent["frac"] = by / us / 1e3 / peak
        n_chk = min(tokens, 512)
        want_p, want_s = O.quantize_fp4(k[:n_chk].float().cpu().numpy().reshape(n_chk * HKV, D))
        sl = slots[:n_chk].cpu().numpy()
        got_p = kc.cpu().numpy()[sl // PAGE, :, sl % PAGE].reshape(n_chk * HKV, D // 2)
        got_s = ks.cpu().numpy()[sl // PAGE, :, sl % PAGE].reshape(n_chk * HKV, D // 32)
        ent["parity"] = {"rows_checked": n_chk * HKV, "bit_exact": bool((got_p == want_p).all() and (got_s == want_s).all())}
        out[name] = ent
        del k, v
    return out


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
    json_fd = 1
    if world > 1:
        # the one JSON line must be alone on stdout: libraries of the multi-GPU run (NCCL's version banner) write there too,
        # so stdout proper is kept aside for the line and everything else goes to stderr
        json_fd = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)
    lib = uq_cuda.lib()
    peak, peak_kind = peaks()
    if args.append_only:   # the prompt-sized append alone (what the profiler capture of that kernel runs)
        ent = append_prompt(dev, peak, cfg["HKV"], cfg["D"], cfg["PAGE"], args.append_tokens, iters=max(1, args.steps))
        os.write(json_fd, (json.dumps({"append": ent, "peak_kind": peak_kind}) + "\n").encode())
        return

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

    def time_steps(fn, steps, warm=3):
        """ms per step of fn(i): `warm` untimed, then exactly `steps` between two events, barrier + synchronize on both sides, max over ranks."""
        for i in range(warm):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    def time_kernel(fn, n):
        """ms of the attention kernel alone: events recorded by the library around that kernel (of a step's last layer)."""
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for i, (a, b) in enumerate(pairs):
            a.record()
            b.record()      # a torch event gets its handle at its first record
            lib.uqb_debug_events(a.cuda_event, b.cuda_event)
            fn(i)
        lib.uqb_debug_events(None, None)
        barrier()
        return max_over_ranks(float(np.mean([a.elapsed_time(b) for a, b in pairs])))

    K = args.kq
    B, HQ, HKV, D, PAGE, layers = (cfg[k] for k in ("B", "HQ", "HKV", "D", "PAGE", "layers"))
    run = Run(cfg, K, rank, world, dev, exchange=args.exchange)
    mode, hkv, hq = run.mode, run.plan["hkv"], run.plan["hq"]
    q, bt, sl, caches, case, fmt, nsplit = run.q, run.bt, run.sl, run.caches, run.case, run.fmt, run.nsplit
    step = run.step

    # ---- device-resident timing: exactly `steps` steps.  The clock sampler is a child process that takes a few hundred
    # milliseconds to come up, during which the GPU would idle down: the warm-up steps run once it is sampling, directly
    # before the timed region
    with ClockSampler(local) as clk:
        for i in range(max(3, args.warmup)):
            step(i)
        barrier()
        n0 = uq_cuda.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
        barrier()
        ms_total = e0.elapsed_time(e1)
        launches = uq_cuda.launch_count() - n0
        # ---- dominant kernel alone
        kern_ms = time_kernel(step, min(args.steps, 50))
        # ---- the same steps replayed from a CUDA graph (the call allocates nothing and reads nothing back, so a caller can
        # capture it once warmed): len(caches) steps per graph, so the alternation of the cache copies is kept
        graph_ms = None
        if mode != "context":
            try:
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    per_graph = 2 if layers == 1 else 1
                    with torch.cuda.graph(graph, stream=side):
                        for i in range(per_graph):
                            step(i)
                    for _ in range(3):
                        graph.replay()
                    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    reps = max(1, args.steps // per_graph)
                    g0.record()
                    for _ in range(reps):
                        graph.replay()
                    g1.record()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph_ms = g0.elapsed_time(g1) / (reps * per_graph)
            except Exception as e:   # capture is a convenience measurement: say why it is missing
                graph_ms = f"unavailable: {type(e).__name__}: {e}"[:200]
                torch.cuda.synchronize()
        # ---- end to end through the public API with host buffers: per step the queries, page table and lengths
        # (and the new tokens of the append leg) come from pinned host memory and the step's output goes back
        hq_, hbt, hsl = q.cpu().pin_memory(), bt.cpu().pin_memory(), sl.cpu().pin_memory()
        hout = torch.empty_like(hq_).pin_memory()
        dq, dbt, dsl = torch.empty_like(q), torch.empty_like(bt), torch.empty_like(sl)
        h2d = int(hq_.numel() * 2 + hbt.numel() * 4 + hsl.numel() * 4)
        hnew = None
        if cfg["append"] and case["new_k"] is not None:
            hnew = (case["new_k"].cpu().pin_memory(), case["new_v"].cpu().pin_memory())
            h2d += int(2 * hnew[0].numel() * 2)

        def e2e_step(i):
            dq.copy_(hq_, non_blocking=True)
            dbt.copy_(hbt, non_blocking=True)
            dsl.copy_(hsl, non_blocking=True)
            if hnew is not None:
                case["new_k"].copy_(hnew[0], non_blocking=True)
                case["new_v"].copy_(hnew[1], non_blocking=True)
            hout.copy_(step(i, dq, dbt, dsl, run.out), non_blocking=True)

        for i in range(3):
            e2e_step(i)
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for i in range(args.steps):
            e2e_step(i)
        f1.record()
        barrier()
        e2e_serial_ms = f0.elapsed_time(f1)
        # ---- the same steps as a serving loop would run them: two sets of buffers, the input copy of step i + 1 and the
        # output copy of step i - 1 on streams of their own, overlapping the kernels of step i.  Every step still copies its
        # inputs in and its output out inside the timed region.
        cur, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
        dqs, dbts, dsls = ([torch.empty_like(t) for _ in range(2)] for t in (q, bt, sl))
        outs = [torch.empty_like(q) for _ in range(2)]
        houts = [torch.empty_like(hq_).pin_memory() for _ in range(2)]
        ev_in, ev_k, ev_out = ([torch.cuda.Event() for _ in range(2)] for _ in range(3))

        def e2e_pipe_step(i):
            j = i & 1
            s_in.wait_event(ev_k[j])        # the step that read these input buffers is done
            with torch.cuda.stream(s_in):
                dqs[j].copy_(hq_, non_blocking=True)
                dbts[j].copy_(hbt, non_blocking=True)
                dsls[j].copy_(hsl, non_blocking=True)
                ev_in[j].record(s_in)
            cur.wait_event(ev_in[j])
            cur.wait_event(ev_out[j])       # the output buffer's previous contents have left
            if hnew is not None:
                case["new_k"].copy_(hnew[0], non_blocking=True)
                case["new_v"].copy_(hnew[1], non_blocking=True)
            o = step(i, dqs[j], dbts[j], dsls[j], outs[j])
            ev_k[j].record(cur)
            s_out.wait_event(ev_k[j])
            o.record_stream(s_out)
            with torch.cuda.stream(s_out):
                houts[j].copy_(o, non_blocking=True)
                ev_out[j].record(s_out)

        for i in range(4):
            e2e_pipe_step(i)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(cur)
        s_in.wait_event(g0)
        for i in range(args.steps):
            e2e_pipe_step(i)
        cur.wait_event(ev_out[0])
        cur.wait_event(ev_out[1])
        g1.record(cur)
        barrier()
        e2e_ms = g0.elapsed_time(g1)
    ms_step = max_over_ranks(ms_total / args.steps)
    e2e_step_ms = max_over_ranks(e2e_ms / args.steps)
    e2e_serial_step_ms = max_over_ranks(e2e_serial_ms / args.steps)
    status = uq_cuda.last_status()
    by_local, by_step, cache_bytes = run.by_local, run.by_step, run.cache_bytes
    value = by_step / (ms_step * 1e-3) / 1e12
    achieved = by_local / (kern_ms * 1e-3) / 1e9
    sharding = {"single": "single GPU", "replicas": "every rank runs the whole call on kv heads of its own, no collective",
                "heads": f"kv heads divided across ranks ({hkv} per rank), no collective",
                "context": "context pages divided across ranks; " + ("every rank's combine kernel stores its packed partial into all ranks' exchange buffers over NVLink "
                           "(plain peer stores, a flag behind them) and the merge kernel waits for the flags: no collective call" if run.exchange == "peer" else
                           "partials all-gathered over NCCL and merged by the log-sum-exp kernel") + ", inside the step"}[mode]
    # DRAM bytes per launch of the attention kernel: from the ncu capture named in `traffic_source`, taken on a half-size case
    # (the capture-size rule) and scaled by the bytes of this call; given only for the captured kernel and shape family
    traffic, traffic_source = None, None
    if args.config == 1 and fmt == 0 and K == 8 and world == 1 and TRAFFIC_PROFILE:
        traffic = int(round(by_local * TRAFFIC_PROFILE["dram_bytes"] / TRAFFIC_PROFILE["algorithmic_bytes"]))
        traffic_source = dict(TRAFFIC_PROFILE, kind="scaled_from_profile")
    l2 = (f"{len(caches)} cache copies alternate; each {cache_bytes / 1e6:.0f} MB copy exceeds the 126 MB L2" if cache_bytes > 126e6 else
          f"{len(caches)} caches of {cache_bytes / 1e6:.0f} MB are read in turn ({len(caches) * cache_bytes / 1e6:.0f} MB between two reads of the same bytes; L2 is 126 MB)")
    line = {"metric": "kv_read_throughput", "value": value, "unit": "TB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_step, "us_per_layer_call": ms_step * 1e3 / layers, "higher_is_better": True,
            "scaling": "weak" if cfg["shard"] == "replicas" else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": cfg["name"] + f" K={K}", "kq": K, "nsplit": nsplit, "layers": layers, "l2": l2, "sharding": sharding,
                       "kernel_path": {1: "cuda-core", 2: "tcgen05"}.get(uq_cuda.last_path(), "?")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                         "traffic_source": traffic_source, "peak_kind": peak_kind, "kernel_us": kern_ms * 1e3, "algorithmic_bytes": by_local},
            "e2e": {"value": by_step / (e2e_step_ms * 1e-3) / 1e12, "unit": "TB/s", "us_per_layer_call": e2e_step_ms * 1e3 / layers,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(hout.numel() * 2),
                    "how": "two buffer sets; the input copy of the next step and the output copy of the previous one run on streams of their own beside the kernels",
                    "serial_us_per_layer_call": e2e_serial_step_ms * 1e3 / layers},
            "graph_replay_ms_per_step": graph_ms, "gpu_launches": int(launches), "tokens_verified_per_s": B * K * (world if mode == "replicas" else 1) / (ms_step * 1e-3),
            "clocks": clk.summary(), "device_status": list(status)}
    # ---- parity of sequence 0 against the CPU oracle (rank 0, every world size), and the CPU baseline beside it at N = 1
    got = step(0).float().cpu().numpy()
    if rank == 0:
        line["parity"] = parity_of(run, got)
    if world == 1 and not args.no_cpu:
        t_seq, _, cores = cpu_sample(case_to_numpy(case), steps=2, warmup=1, nvfp4=(case["k_ts"], case["v_ts"]) if fmt == 1 else None)
        scale = float(run.plan["lens"].sum()) / float(run.plan["lens"][0]) * layers
        t_step = t_seq * scale
        line["cpu_baseline"] = {"value": by_step / t_step / 1e12, "unit": "TB/s", "cores": cores, "kind": "port", "us_per_layer_call": t_step * 1e6 / layers,
                                "sample": f"sequence 0 ({int(run.plan['lens'][0])} tokens) of {B}, all kv heads, one layer of {layers}, K={K}, 2 timed runs; "
                                          f"scaled x{scale:.2f} (tokens x layers) to a step"}

    # ---- the whole metric of the headline configuration in the same line (N = 1): every K, the no-sharing mode, and the
    # reference's own CUDA kernels timed on this GPU
    if world == 1 and args.config == 1 and fmt == 0 and not args.ctx and not args.lean:
        per_k, no_sharing, gpu_ref = {}, {}, {}
        n_k = 20
        for k in (1, 2, 4, 8):
            rk = run if k == K else Run(cfg, k, rank, world, dev)
            t = time_steps(rk.step, n_k)
            tk = time_kernel(rk.step, n_k)
            per_k[str(k)] = {"us_per_layer_call": t * 1e3, "kernel_us": tk * 1e3, "frac": rk.by_local / (tk * 1e-3) / 1e9 / peak}
            # the no-sharing mode (reference cuda/uq_cuda.py:58-61): K single-query problems over B*K pseudo-sequences
            no_sharing[str(k)] = {"us_per_layer_call": (t if k == 1 else time_steps(lambda i: rk.step(i, fused=False), n_k)) * 1e3}
            no_sharing[str(k)]["fused_gain"] = no_sharing[str(k)]["us_per_layer_call"] / (t * 1e3)
            try:
                sys.path.insert(0, os.path.join(ROOT, "baseline"))
                import ref_gpu
                gpu_ref[str(k)] = ref_gpu.sweep(rk.case, k, HQ, HKV, D, PAGE, mode="short", iters=30, check_against=rk.step(0))
            except Exception as e:
                gpu_ref[str(k)] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
            if "us" in gpu_ref[str(k)]:
                gpu_ref[str(k)]["speedup_of_this_library"] = gpu_ref[str(k)]["us"] / (t * 1e3)
            if rk is not run:
                del rk
                torch.cuda.empty_cache()
        torch.cuda.empty_cache()
        line["append"] = append_prompt(dev, peak, HKV, D, PAGE, B * cfg["ctx"])   # the prompt that fills this very cache: B x ctx tokens
        line["per_k"] = per_k
        line["k8_over_k1"] = per_k["8"]["us_per_layer_call"] / per_k["1"]["us_per_layer_call"]
        line["no_sharing"] = no_sharing
        line["gpu_reference"] = {"what": "the reference's own CUDA kernels (its variants 1 and 2, mma.sync) built for sm_100a from its checkout and tuned "
                                         "with its own protocol on this GPU, same inputs; its tcgen05 variant is not run (its waits end in a trap)",
                                 "per_k": gpu_ref}

    # ---- the two sharded configurations in the scaling run's line (N > 1, default configuration): heads divided (config 3)
    # and the context split (config 4), each with its parity and the same configuration timed on rank 0's GPU alone
    if world > 1 and args.config == 1 and fmt == 0 and not args.lean:
        run.close()
        del run, case, caches
        torch.cuda.empty_cache()
        sharded = {}
        for cid in (3, 4):
            c2 = dict(CONFIGS[cid])
            r2 = Run(c2, K, rank, world, dev)
            t = time_steps(r2.step, 30)
            tk = time_kernel(r2.step, 20)
            ent = {"workload": c2["name"] + f" K={K}", "us_per_call": t * 1e3, "kernel_us": tk * 1e3, "tokens_verified_per_s": c2["B"] * K / (t * 1e-3),
                   "per_gpu_frac": r2.by_local / (tk * 1e-3) / 1e9 / peak, "per_gpu_algorithmic_bytes": r2.by_local,
                   "sharding": "context pages divided; partials exchanged by peer stores, merged after a flag wait" if r2.mode == "context" else f"{r2.plan['hkv']} kv heads per rank, no collective"}
            got2 = r2.step(0).float().cpu().numpy()
            if rank == 0:
                ent["parity"] = parity_of(r2, got2)
            if r2.mode == "context":   # the NCCL all-gather variant of the same step, for comparison
                r2.close()
                r3 = Run(c2, K, rank, world, dev, exchange="nccl")
                ent["us_per_call_nccl_allgather"] = time_steps(r3.step, 30) * 1e3
                del r3
            r2.close()
            del r2
            torch.cuda.empty_cache()
            barrier()
            if rank == 0:   # the whole configuration on one GPU, in the same run
                r1 = Run(c2, K, 0, 1, dev)
                for i in range(3):
                    r1.step(i)
                torch.cuda.synchronize()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for i in range(20):
                    r1.step(i)
                a1.record()
                torch.cuda.synchronize()
                ent["single_gpu_us_per_call"] = a0.elapsed_time(a1) / 20 * 1e3
                ent["speedup_over_single_gpu"] = ent["single_gpu_us_per_call"] / ent["us_per_call"]
                del r1
                torch.cuda.empty_cache()
            barrier()
            sharded[f"cfg{cid}"] = ent
        line["sharded"] = sharded
    if rank == 0:
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="timed steps (default 200; 10 for the 32-layer configuration)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kq", type=int, default=8, help="draft queries per sequence (K)")
    ap.add_argument("--config", type=int, default=1, choices=sorted(CONFIGS))
    ap.add_argument("--ctx", type=int, default=0, help="override the context length (profiler captures use a shorter one; the JSON says so)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--fmt", type=int, default=0, choices=[0, 1], help="cache format: 0 UltraQuant (the headline), 1 NVFP4 (configurations 1 and 3)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="context split (configuration 4, N > 1): partials by peer stores and flags, or by an NCCL all-gather")
    ap.add_argument("--append-only", action="store_true", help="time only the append-quantize of a prompt (--append-tokens tokens of the configuration's heads)")
    ap.add_argument("--append-tokens", type=int, default=262144)
    ap.add_argument("--lean", action="store_true", help="only the headline measurement: no per-K table, no reference-GPU sweep, no sharded configurations")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.steps <= 0:
        args.steps = 200 if cfg["layers"] == 1 else 10
    if args.fmt == 1:
        if cfg["append"] or cfg["shard"] == "context":
            raise SystemExit("--fmt 1 (NVFP4) runs configurations 1 and 3: the append kernel and the context split serve the UltraQuant cache")
        cfg["fmt"] = 1
        cfg["name"] += " NVFP4 cache (e4m3fn scale per 16 channels)"
    if args.ctx:
        cfg["ctx"] = args.ctx
        cfg["name"] += f" (context overridden to {args.ctx})"
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
