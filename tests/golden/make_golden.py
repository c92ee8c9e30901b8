"""Generates the fixtures in this directory.  Needs the reference checkout: its path is argv[1] or the environment
variable UQ_REFERENCE; the tests themselves never read the reference, only the .npz files written here.

Two kinds of fixture:
  ref_cuda_<set>.npz / ref_sycl_<case>.npz   the reference's own frozen known-answer vectors
      (cuda/vectors, sycl/vectors: cache bytes, page table, seq_lens, bf16 queries, fp32 outputs),
      repacked unchanged into one compressed file per case set.
  gen_*.npz   inputs and outputs of the reference's Python functions run here
      (uqmt.attn.quantize_fp4 / dequantize_fp4 / reference / build_paged_cache,
       uqmt.vllm_adapter.append_kv, uqmt.tree.tree_reference), for the cases the frozen vectors do not cover.
  nvfp4_cuda_<set>.npz   the reference's frozen NVFP4 vectors (cuda/vectors_nvfp4), repacked the same way; the scale
      arrays are e4m3fn bytes [pages,Hkv,PAGE,D/16] and `ts` holds the per-tensor scales (k_ts, v_ts).
gen_upstream.npz holds the upstream engines' slot layout (the converter of cuda/UPSTREAM_COMPAT.md:81-88 applied with torch) and the
bytes of the upstream encoder vendored by the reference (cuda/compat/upstream/reference.py, run the way
cuda/compat/paper_rule_cpu_check.py runs it) beside the reference's own 'paper'-rule bytes; `--upstream-only` writes it alone.
`--sycl-only` repacks the sycl vectors alone.
`--tree-only` regenerates tree_cases.npz alone, `--nvfp4-only` the nvfp4_cuda_* files alone, `--rotate-only` gen_rotate.npz
(uqmt.quant.fwht and the 'paper' scale rule of uqmt.quant.quantize) and gen_nvfp4_quant.npz (uqmt.quant.quantize_nvfp4) alone.
"""
import os
import sys

import numpy as np
import torch

_args = [a for a in sys.argv[1:] if not a.startswith("--")]
REF = _args[0] if _args else os.environ.get("UQ_REFERENCE")
if not REF:
    raise SystemExit("usage: make_golden.py <path of the reference checkout> [--tree-only | --nvfp4-only | --rotate-only]")
OUT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REF)
from uqmt.attn import build_paged_cache, dequantize_fp4, quantize_fp4, reference  # noqa: E402
from uqmt.vllm_adapter import append_kv  # noqa: E402


def save(name, **arrs):
    np.savez_compressed(os.path.join(OUT, name), **arrs)
    print(name, {k: getattr(v, "shape", v) for k, v in arrs.items()})


def repack_cuda_vectors(sub="vectors", prefix="ref_cuda_", group=32):
    d = os.path.join(REF, "cuda", sub)
    sets = {}
    for line in open(os.path.join(d, "manifest.txt")):
        t = line.split()
        name, K = t[1], int(t[2])
        B, HQ, HKV, D, PAGE, pages, max_pages = map(int, t[3:10])
        s = sets.setdefault(name, dict(meta=np.array([B, HQ, HKV, D, PAGE, pages, max_pages], np.int32), Ks=[]))
        if group == 16:   # NVFP4 manifest: two more columns, the per-tensor scales
            s["ts"] = np.array([float(t[10]), float(t[11])], np.float64)
        s["Ks"].append(K)
    for name, s in sets.items():
        B, HQ, HKV, D, PAGE, pages, max_pages = (int(x) for x in s["meta"])
        f = lambda suf, dt: np.fromfile(os.path.join(d, f"{name}_{suf}.bin"), dtype=dt)
        arrs = dict(meta=s["meta"], Ks=np.array(s["Ks"], np.int32),
                    kc=f("kc", np.uint8).reshape(pages, HKV, PAGE, D // 2), ks=f("ks", np.uint8).reshape(pages, HKV, PAGE, D // group),
                    vc=f("vc", np.uint8).reshape(pages, HKV, PAGE, D // 2), vs=f("vs", np.uint8).reshape(pages, HKV, PAGE, D // group),
                    bt=f("bt", np.int32).reshape(B, max_pages), sl=f("sl", np.int32))
        for K in s["Ks"]:
            arrs[f"q_K{K}"] = f(f"K{K}_q", np.uint16).reshape(B, K, HQ, D)
            arrs[f"ref_K{K}"] = f(f"K{K}_ref", np.float32).reshape(B, K, HQ, D)
        if "ts" in s:
            arrs["ts"] = s["ts"]
        save(f"{prefix}{name}.npz", **arrs)


SYCL_KEEP = ("b2k16_d128_p32", "b3k2_d64_p16", "b4k3_d128_p64_g1", "edge_short_k4", "b1k8_d128_p64",
             "b2k1_d128_p64", "b2k4_d128_p64", "rot_h128_b2k4", "paper_rule_b2k4")   # all nine cases of sycl/vectors/manifest.txt


def repack_sycl_vectors():
    d = os.path.join(REF, "sycl", "vectors")
    for line in open(os.path.join(d, "manifest.txt")):
        t = line.split()
        name = t[0]
        if name not in SYCL_KEEP:
            continue
        B, K, HQ, HKV, D, PAGE, max_pages = map(int, t[1:8])
        f = lambda suf, dt: np.fromfile(os.path.join(d, f"{name}.{suf}.bin"), dtype=dt)
        kc = f("kc", np.uint8)
        pages = kc.size // (HKV * PAGE * (D // 2))
        save(f"ref_sycl_{name}.npz", meta=np.array([B, HQ, HKV, D, PAGE, pages, max_pages], np.int32), Ks=np.array([K], np.int32),
             sm_scale=np.float32(t[8]), kc=kc.reshape(pages, HKV, PAGE, D // 2), ks=f("ks", np.uint8).reshape(pages, HKV, PAGE, D // 32),
             vc=f("vc", np.uint8).reshape(pages, HKV, PAGE, D // 2), vs=f("vs", np.uint8).reshape(pages, HKV, PAGE, D // 32),
             bt=f("bt", np.int32).reshape(B, max_pages), sl=f("sl", np.int32),
             **{f"q_K{K}": f("q", np.uint16).reshape(B, K, HQ, D), f"ref_K{K}": f("ref", np.float32).reshape(B, K, HQ, D)})


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def gen_codec():
    """Encoder known answers: wide dynamic range, bf16/fp16 inputs (exact rounding ties), all-zero
    groups, +-1e30 / 1e-30 extremes, signed zeros, and amax on both sides of every power-of-two
    boundary of amax/6 (the place where a sloppy log2 flips the scale byte)."""
    g = torch.Generator().manual_seed(11)
    wide = torch.randn(256, 128, generator=g) * torch.exp2(torch.randint(-40, 40, (256, 1), generator=g).float())
    b16 = torch.randn(512, 128, generator=g).bfloat16().float()
    f16 = (torch.randn(256, 128, generator=g) * 3).half().float()
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0,
                         0.0, -0.0, 0.1, -0.1, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 7.0, -7.0, 0.2500001, 0.7499999, 5.0000005, 4.9999995])
    ties = torch.stack([ties * (2.0 ** k) for k in (-3, 0, 5)] + [ties * 0.9, ties * 1.1]).reshape(-1, 32)
    special = torch.zeros(8, 32)
    special[1, 3] = 1e30
    special[2, 5] = -1e30
    special[3, 7] = 1e-30
    special[4, :] = 1e-38
    special[5, 0] = -0.0
    special[6, :] = torch.tensor([-1e-9] * 31 + [6.0])
    special[7, :] = 3e38
    ks = torch.arange(-120, 121, dtype=torch.float32)
    base = 6.0 * torch.exp2(ks)
    ulps = []
    for j in (-2, -1, 0, 1, 2, 3):
        u = base.clone().view(torch.int32) + j
        ulps.append(u.view(torch.float32))
    edge_amax = torch.cat(ulps)
    edges = torch.zeros(edge_amax.numel(), 32)
    edges[:, 0] = edge_amax
    edges[:, 1] = -edge_amax * 0.41
    edges[:, 2] = edge_amax * 0.13
    x32 = torch.cat([ties, special, edges])
    arrs = {}
    for name, x in (("wide", wide), ("bf16in", b16), ("fp16in", f16), ("g32", x32)):
        p, s = quantize_fp4(x)
        arrs[f"{name}_x"] = x.numpy()
        arrs[f"{name}_packed"] = p.numpy()
        arrs[f"{name}_scales"] = s.numpy()
        arrs[f"{name}_deq"] = dequantize_fp4(p, s).numpy()
    # every (nibble, scale byte) pair decodes exactly
    allb = torch.arange(256, dtype=torch.uint8).reshape(1, 16, 16).repeat(256, 1, 1)   # [scale byte, group, 16 packed bytes]
    arrs["all_packed"] = allb.numpy()
    arrs["all_scales"] = torch.arange(256, dtype=torch.uint8).reshape(256, 1, 1).repeat(1, 16, 1).numpy()
    arrs["all_deq"] = dequantize_fp4(torch.from_numpy(arrs["all_packed"]), torch.from_numpy(arrs["all_scales"])).numpy()
    save("gen_codec.npz", **arrs)


def make_case(B, K, HQ, HKV, D, PAGE, seq_lens, seed, keep_raw_pages=0):
    """Seeded synthetic case: bf16 N(0,1) queries; fp32 N(0,1) K/V with a lognormal(0, 0.5)
    multiplier per K channel; encoded by the reference encoder; physical pages permuted."""
    g = torch.Generator().manual_seed(seed)
    T = max(max(seq_lens), 1)
    chan = torch.exp(0.5 * torch.randn(1, HKV, 1, D, generator=g))
    k = torch.randn(B, HKV, T, D, generator=g) * chan
    v = torch.randn(B, HKV, T, D, generator=g)
    q = torch.randn(B, K, HQ, D, generator=g).bfloat16()
    c = build_paged_cache(k, v, page_size=PAGE, seq_lens=seq_lens, shuffle=True, generator=g)
    ref = reference(q, c.kc, c.ks, c.vc, c.vs, c.block_table, c.seq_lens)
    arrs = dict(meta=np.array([B, HQ, HKV, D, PAGE, c.kc.shape[0], c.block_table.shape[1]], np.int32), Ks=np.array([K], np.int32),
                kc=c.kc.numpy(), ks=c.ks.numpy(), vc=c.vc.numpy(), vs=c.vs.numpy(), bt=c.block_table.numpy(), sl=c.seq_lens.numpy(),
                **{f"q_K{K}": bits(q), f"ref_K{K}": ref.numpy()})
    if keep_raw_pages:
        # fp32 K/V of the first logical pages of sequence 0 (+ the physical ids they landed on): encoder check
        n = keep_raw_pages
        arrs["raw_k"] = k[0, :, : n * PAGE].reshape(HKV, n, PAGE, D).permute(1, 0, 2, 3).contiguous().numpy()
        arrs["raw_v"] = v[0, :, : n * PAGE].reshape(HKV, n, PAGE, D).permute(1, 0, 2, 3).contiguous().numpy()
        arrs["raw_pages"] = c.block_table[0, :n].numpy()
    return arrs


def gen_cases():
    # configuration 0 of the benchmark contract: the CPU-runnable parity case
    save("gen_cfg0.npz", **make_case(2, 4, 8, 2, 128, 64, [1000, 777], 0, keep_raw_pages=4))
    # head_dim 256 (136 B per head per token): no frozen vector exists for it
    save("gen_d256.npz", **make_case(2, 8, 16, 2, 256, 64, [700, 130], 1005))
    # K=8, G=8 (64 rows) with ragged lengths incl. an empty sequence and seq_len < K
    save("gen_k8g8.npz", **make_case(4, 8, 16, 2, 128, 64, [515, 0, 5, 128], 1006))
    # G=7 (not a power of two), K=3, PAGE=32
    save("gen_g7.npz", **make_case(2, 3, 14, 2, 128, 32, [100, 33], 1007))
    # D=64, PAGE=64, K=8
    save("gen_d64.npz", **make_case(2, 8, 16, 2, 64, 64, [321, 64], 1008))


def gen_append():
    """append_kv known answer: 8 new bf16 tokens per sequence written through a permuted page table."""
    g = torch.Generator().manual_seed(21)
    pages, HKV, PAGE, D, B, Kn = 12, 2, 64, 128, 3, 8
    kc = torch.randint(0, 256, (pages, HKV, PAGE, D // 2), generator=g, dtype=torch.uint8)
    ks = torch.randint(100, 140, (pages, HKV, PAGE, D // 32), generator=g, dtype=torch.uint8)
    vc = torch.randint(0, 256, (pages, HKV, PAGE, D // 2), generator=g, dtype=torch.uint8)
    vs = torch.randint(100, 140, (pages, HKV, PAGE, D // 32), generator=g, dtype=torch.uint8)
    before = [t.clone() for t in (kc, ks, vc, vs)]
    bt = torch.randperm(pages, generator=g).reshape(B, 4)
    seq = torch.tensor([70, 8, 250])   # lengths AFTER the append; new tokens are the last 8 positions
    pos = torch.stack([torch.arange(int(n) - Kn, int(n)) for n in seq])          # [B, 8]
    slots = (bt.gather(1, pos // PAGE) * PAGE + pos % PAGE).reshape(-1)
    key = (torch.randn(B * Kn, HKV, D, generator=g) * 2).bfloat16()
    val = torch.randn(B * Kn, HKV, D, generator=g).bfloat16()
    key[3, 1, 32:64] = 0   # an all-zero group
    append_kv(kc, ks, vc, vs, key, val, slots)
    save("gen_append.npz", kc0=before[0].numpy(), ks0=before[1].numpy(), vc0=before[2].numpy(), vs0=before[3].numpy(),
         key=bits(key), value=bits(val), slots=slots.numpy().astype(np.int64),
         kc1=kc.numpy(), ks1=ks.numpy(), vc1=vc.numpy(), vs1=vs.numpy())


def gen_rotate():
    """The engine-side options of the append: uqmt.quant.fwht (orthonormal Hadamard of K and Q) and the 'paper' scale rule
    of uqmt.quant.quantize, on seeded rows with a wide range of magnitudes, zero rows and exact powers of two included."""
    from uqmt.quant import PAPER_C, fwht, quantize
    g = torch.Generator().manual_seed(77)
    arrs = {"c": np.float32(PAPER_C)}
    for D in (64, 128, 256):
        x = torch.randn(24, 2, D, generator=g) * torch.exp(2.0 * torch.randn(24, 2, 1, generator=g))
        x[3] = 0.0
        x[5] = torch.exp2(torch.randint(-6, 6, (2, D), generator=g).float())
        xr = fwht(x)
        arrs[f"d{D}_x"] = x.numpy()
        arrs[f"d{D}_fwht"] = xr.numpy()
        for name, src in (("plain", x), ("rot", xr)):
            for rule in ("ceil", "paper"):
                p, sc = quantize(src, rule, PAPER_C)
                arrs[f"d{D}_{name}_{rule}_codes"], arrs[f"d{D}_{name}_{rule}_scales"] = p.numpy(), sc.numpy()
        q = torch.randn(6, 4, D, generator=g).bfloat16()
        arrs[f"d{D}_q"] = q.view(torch.int16).numpy().view(np.uint16)
        arrs[f"d{D}_q_fwht"] = fwht(q).view(torch.int16).numpy().view(np.uint16)
    save("gen_rotate.npz", **arrs)


def gen_nvfp4_quant():
    """uqmt.quant.quantize_nvfp4 with a given tensor scale (the NVFP4 append's encoder) on seeded rows: wide magnitudes, zero
    rows, rows far below and far above the range the tensor scale covers (scale bytes at both clamps)."""
    from uqmt.quant import quantize_nvfp4
    g = torch.Generator().manual_seed(99)
    arrs = {}
    for D in (64, 128, 256):
        x = torch.randn(32, 2, D, generator=g) * torch.exp(2.0 * torch.randn(32, 2, 1, generator=g))
        x[3] = 0.0
        x[5] *= 1e-7
        x[7] *= 1e4
        ts = 32.0 / (6 * 448)
        p, s, _ = quantize_nvfp4(x, ts)
        arrs[f"d{D}_x"], arrs[f"d{D}_codes"], arrs[f"d{D}_scales"] = x.numpy(), p.numpy(), s.view(torch.uint8).numpy()
        arrs[f"d{D}_ts"] = np.float64(ts)
    save("gen_nvfp4_quant.npz", **arrs)


def gen_tree():
    """Tree-masked verify: answers of the reference's own oracle (uqmt/tree.py tree_reference) for chain, star and seeded
    random parent trees, one case with a different tree per sequence.  One file, cases t0..tN."""
    from uqmt.tree import chain_mask, parents_to_mask, star_mask, tree_reference
    specs = [  # B, K, HQ, HKV, D, PAGE, seq_lens, seed, kind
        (2, 4, 8, 2, 128, 64, [300, 129], 2001, "chain"),
        (2, 8, 16, 2, 128, 64, [515, 70], 2002, "star"),
        (3, 8, 16, 2, 128, 64, [400, 128, 9], 2003, "random"),     # K x G = 64 rows, a sequence of K + 1 tokens
        (2, 6, 8, 4, 64, 16, [77, 200], 2004, "random"),
        (2, 16, 4, 2, 128, 32, [260, 17], 2005, "random"),          # K = 16: the widest mask
        (1, 5, 8, 2, 128, 64, [3], 2006, "random"),                 # fewer tokens than drafts
    ]
    arrs = {"n": np.array([len(specs)], np.int32)}
    for i, (B, K, HQ, HKV, D, PAGE, lens, seed, kind) in enumerate(specs):
        g = torch.Generator().manual_seed(seed)
        T = max(max(lens), 1)
        chan = torch.exp(0.5 * torch.randn(1, HKV, 1, D, generator=g))
        k = torch.randn(B, HKV, T, D, generator=g) * chan
        v = torch.randn(B, HKV, T, D, generator=g)
        q = torch.randn(B, K, HQ, D, generator=g).bfloat16()
        c = build_paged_cache(k, v, page_size=PAGE, seq_lens=lens, shuffle=True, generator=g)
        if kind == "chain":
            tm = chain_mask(K, B)
        elif kind == "star":
            tm = star_mask(K).expand(B, K).contiguous()
        else:
            rng = np.random.default_rng(seed)
            tm = parents_to_mask(np.stack([[-1] + [int(rng.integers(-1, j)) for j in range(1, K)] for _ in range(B)]))
        ref = tree_reference(q, c.kc, c.ks, c.vc, c.vs, c.block_table, c.seq_lens, tm)
        arrs.update({f"t{i}_meta": np.array([B, K, HQ, HKV, D, PAGE], np.int32), f"t{i}_kc": c.kc.numpy(), f"t{i}_ks": c.ks.numpy(),
                     f"t{i}_vc": c.vc.numpy(), f"t{i}_vs": c.vs.numpy(), f"t{i}_bt": c.block_table.numpy(), f"t{i}_sl": c.seq_lens.numpy(),
                     f"t{i}_q": bits(q), f"t{i}_tm": tm.numpy().astype(np.int32), f"t{i}_ref": ref.numpy()})
    save("tree_cases.npz", **arrs)


def gen_upstream():
    import importlib.util
    import re
    import types
    from uqmt import quant as UQ
    here = os.path.join(REF, "cuda", "compat")

    def load(name, path):
        sp = importlib.util.spec_from_file_location(name, path)
        m = importlib.util.module_from_spec(sp)
        sys.modules[name] = m
        sp.loader.exec_module(m)
        return m
    for pkg in ("vllm", "vllm.v1", "vllm.v1.attention", "vllm.v1.attention.ops", "vllm.v1.attention.ops.ultraquant"):
        sys.modules.setdefault(pkg, types.ModuleType(pkg))
    load("vllm.v1.attention.ops.ultraquant.format", os.path.join(here, "upstream", "format.py"))
    UR = load("vllm.v1.attention.ops.ultraquant.reference", os.path.join(here, "upstream", "reference.py"))
    # canon_negzero as the reference's check script defines it (the script itself writes into the checkout when run)
    text = open(os.path.join(here, "paper_rule_cpu_check.py")).read()
    ns = {"torch": torch}
    exec(re.search(r"def canon_negzero\(pk\):.*?\n    return [^\n]*\n", text, re.S).group(0), ns)
    canon = ns["canon_negzero"]
    torch.manual_seed(5)
    arrs = {}
    for D in (64, 128, 256):
        G = D // 32
        pages, HKV, PAGE = 3, 2, 16
        n = pages * HKV * PAGE
        x = torch.randn(2, n, D) * torch.exp(0.7 * torch.randn(2, n, G, 1)).expand(2, n, G, 32).reshape(2, n, D)
        x = x * (torch.rand(2, n, G, 1) > 0.2).float().expand(2, n, G, 32).reshape(2, n, D)     # a fifth of the groups all zero
        pk, sc = UQ.quantize(x, "paper", 0.156)
        if D in (128, 256):   # the vendored encoder asserts these head sizes
            enc = UR.ultraquant_encode(x.reshape(-1, D), rotate=False)
            up_codes, up_scales = enc.codes_packed.reshape(pk.shape), enc.scale_bytes.reshape(sc.shape)
            assert torch.equal(canon(pk), up_codes)
        else:
            up_codes, up_scales = canon(pk), None
        kc, vc = (t.reshape(pages, HKV, PAGE, D // 2).contiguous() for t in pk)
        ks, vs = (t.reshape(pages, HKV, PAGE, G).contiguous() for t in sc)
        aos = torch.cat([kc, ks, vc, vs], -1).permute(0, 2, 1, 3).contiguous()          # ours_to_upstream
        pad = torch.nn.functional.pad(aos, (0, 8))                                      # a slot size 8 bytes above the payload
        c = aos.permute(0, 2, 1, 3)                                                     # upstream_to_ours
        back = (c[..., :D // 2], c[..., D // 2:D // 2 + G], c[..., D // 2 + G:D + G], c[..., D + G:D + 2 * G])
        assert all(torch.equal(a.contiguous(), b) for a, b in zip(back, (kc, ks, vc, vs)))
        arrs.update({f"d{D}_kc": kc.numpy(), f"d{D}_ks": ks.numpy(), f"d{D}_vc": vc.numpy(), f"d{D}_vs": vs.numpy(), f"d{D}_aos": aos.numpy(),
                     f"d{D}_aos_pad8": pad.numpy(), f"d{D}_canon_kc": canon(kc).numpy(), f"d{D}_canon_vc": canon(vc).numpy()})
        if up_scales is not None:
            arrs.update({f"d{D}_up_ks": up_scales[0].reshape(ks.shape).numpy(), f"d{D}_up_vs": up_scales[1].reshape(vs.shape).numpy()})
    save("gen_upstream.npz", **arrs)


if __name__ == "__main__":
    if "--upstream-only" in sys.argv:
        gen_upstream()
        sys.exit(0)
    if "--sycl-only" in sys.argv:
        repack_sycl_vectors()
        sys.exit(0)
    if "--nvfp4-only" in sys.argv:
        repack_cuda_vectors("vectors_nvfp4", "nvfp4_cuda_", 16)
        sys.exit(0)
    if "--rotate-only" in sys.argv:
        gen_rotate()
        gen_nvfp4_quant()
        sys.exit(0)
    if "--tree-only" in sys.argv:
        gen_tree()
        sys.exit(0)
    repack_cuda_vectors()
    repack_cuda_vectors("vectors_nvfp4", "nvfp4_cuda_", 16)
    repack_sycl_vectors()
    gen_codec()
    gen_cases()
    gen_append()
    gen_tree()
    gen_rotate()
    gen_nvfp4_quant()
