"""NVFP4 cache (fmt = 1: e2m1 codes, one e4m3fn scale byte per 16 channels, per-tensor fp32 scales k_ts / v_ts).

The known answers are the reference's own frozen vectors (cuda/vectors_nvfp4, repacked into golden/nvfp4_cuda_*.npz):
the oracle is pinned to them on the CPU, and the CUDA-core kernel is compared with them through the C ABI on a GPU."""
import numpy as np
import pytest
import torch

from tests.cases import check_close, check_harness_rule, load_cases
from oracle import uq_oracle as O

CASES = load_cases("nvfp4_cuda_*")


def test_fixture_set_is_complete():
    assert len(CASES) == 13
    assert {c.name.split("_K")[0] for c in CASES} == {f"nvfp4_cuda_{s}" for s in ("main", "gqa8_p128", "d64_p32", "p16_g4", "edge_short")}
    for c in CASES:
        assert c.fmt == 1 and c.ks.shape[-1] == c.D // 16 and c.vs.shape[-1] == c.D // 16


def test_e4m3fn_table_matches_torch():
    want = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    got = O.e4m3fn_table()
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok], want[ok])


@pytest.mark.parametrize("c", CASES, ids=repr)
def test_oracle_reproduces_the_reference_vectors(c):
    out = O.reference_nvfp4(c.q, c.kc, c.ks, c.vc, c.vs, c.bt, c.sl, c.k_ts, c.v_ts, c.sm_scale)
    assert np.abs(out - c.ref).max() <= 1e-5 * max(1.0, np.abs(c.ref).max())


def test_unit_tensor_scales_and_power_of_two_blocks_equal_the_ultraquant_answer():
    """A cache whose e4m3fn scales are powers of two, equal within each 32-channel block, is the same tensor as the
    UltraQuant cache with the matching UE8M0 bytes: both oracles must give the same answer."""
    rng = np.random.default_rng(5)
    B, K, HQ, HKV, D, PAGE, pages = 2, 3, 4, 2, 64, 16, 6
    kc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
    vc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
    e = rng.integers(-3, 3, (2, pages, HKV, PAGE, D // 32))
    ue = (e + 127).astype(np.uint8)
    e4 = np.repeat(((e + 7) << 3).astype(np.uint8), 2, axis=-1)      # exponent field only: 2^e
    bt = np.arange(pages, dtype=np.int32).reshape(B, pages // B)
    sl = np.array([40, 33], np.int32)
    q = O.bf16_bits(rng.standard_normal((B, K, HQ, D)).astype(np.float32))
    a = O.reference(q, kc, ue[0], vc, ue[1], bt, sl)
    b = O.reference_nvfp4(q, kc, e4[0], vc, e4[1], bt, sl, 1.0, 1.0)
    assert np.array_equal(a, b)


# ---------------------------------------------------------------------------------------------------- GPU
def _dev(c):
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    q = torch.from_numpy(c.q.view(np.int16)).cuda().view(torch.bfloat16)
    return q, t(c.kc), t(c.ks), t(c.vc), t(c.vs), t(c.bt), t(c.sl)


@pytest.mark.gpu
@pytest.mark.parametrize("path", ["tc", "fma"])
@pytest.mark.parametrize("c", CASES, ids=repr)
def test_kernel_matches_the_reference_vectors(c, path, monkeypatch):
    from all_quant_b200 import uq_cuda
    monkeypatch.setenv("UQ_B200_CFG", f"path={path}")
    q, kc, ks, vc, vs, bt, sl = _dev(c)
    for nsplit in (None, 1, 3):
        out = uq_cuda.uq_decode_cuda(q, kc, ks, vc, vs, bt, sl, nsplit=nsplit, sm_scale=c.sm_scale, fmt=1, k_ts=c.k_ts, v_ts=c.v_ts)
        torch.cuda.synchronize()
        assert uq_cuda.last_path() == {"fma": 1, "tc": 2}[path]
        assert uq_cuda.last_status()[0] == 0
        got = out.float().cpu().numpy()
        check_close(got, c.ref, f"{c} nsplit={nsplit}")
        check_harness_rule(got, c.ref, f"{c} nsplit={nsplit}")


@pytest.mark.gpu
def test_unfused_mode_and_tensor_scales():
    from all_quant_b200 import uq_cuda
    c = [x for x in CASES if x.name == "nvfp4_cuda_main_K4"][0]
    q, kc, ks, vc, vs, bt, sl = _dev(c)
    out = uq_cuda.uq_decode_cuda(q, kc, ks, vc, vs, bt, sl, fused=False, fmt=1, k_ts=c.k_ts, v_ts=c.v_ts)
    check_close(out.float().cpu().numpy(), c.ref, "unfused")
    # other tensor scales: the oracle gives the answer
    for k_ts, v_ts in ((2.0 * c.k_ts, 0.5 * c.v_ts), (0.25 * c.k_ts, 1.5 * c.v_ts)):   # outputs stay of order one: the rule's mean bound is absolute
        want = O.reference_nvfp4(c.q, c.kc, c.ks, c.vc, c.vs, c.bt, c.sl, k_ts, v_ts)
        out = uq_cuda.uq_decode_cuda(q, kc, ks, vc, vs, bt, sl, fmt=1, k_ts=k_ts, v_ts=v_ts)
        check_close(out.float().cpu().numpy(), want, f"k_ts={k_ts} v_ts={v_ts}")


@pytest.mark.gpu
@pytest.mark.parametrize("path", ["tc", "fma"])
def test_larger_nvfp4_call_against_the_oracle(path, monkeypatch):
    """Longer contexts than the frozen vectors hold, D = 256 included (the reference ships no NVFP4 vector for it); scale
    bytes over the whole exponent range of the format, subnormals included."""
    from all_quant_b200 import uq_cuda
    monkeypatch.setenv("UQ_B200_CFG", f"path={path}")
    rng = np.random.default_rng(11)
    for D, PAGE, K, HQ, HKV in ((128, 64, 8, 16, 2), (256, 32, 2, 8, 4), (64, 128, 5, 6, 2)):
        B, ctx = 2, 1500
        npg = -(-ctx // PAGE)
        pages = B * npg
        kc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
        vc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
        # scale bytes: K exponent fields 4..10 with any mantissa, sign clear (what an amax / 6 scale can be);
        # V any finite non-negative byte (0x00..0x7e: zero, subnormals, up to 448), mostly small so that outputs stay of order one
        ks = (rng.integers(4, 11, (pages, HKV, PAGE, D // 16)) << 3 | rng.integers(0, 8, (pages, HKV, PAGE, D // 16))).astype(np.uint8)
        vs = rng.integers(0, 0x48, (pages, HKV, PAGE, D // 16)).astype(np.uint8)
        vs[rng.random(vs.shape) < 0.01] = 0x7e
        bt = rng.permutation(pages).astype(np.int32).reshape(B, npg)
        sl = np.array([ctx, ctx - 777], np.int32)
        qf = rng.standard_normal((B, K, HQ, D)).astype(np.float32)
        qb = O.bf16_bits(qf)
        k_ts, v_ts = 0.05, 0.02
        want = O.reference_nvfp4(qb, kc, ks, vc, vs, bt, sl, k_ts, v_ts)
        t = lambda a: torch.from_numpy(a).cuda()
        q = torch.from_numpy(qb.view(np.int16)).cuda().view(torch.bfloat16)
        out = uq_cuda.uq_decode_cuda(q, t(kc), t(ks), t(vc), t(vs), t(bt), t(sl), fmt=1, k_ts=k_ts, v_ts=v_ts)
        assert uq_cuda.last_path() == {"fma": 1, "tc": 2}[path] and uq_cuda.last_status()[0] == 0
        check_close(out.float().cpu().numpy(), want, f"D={D}")


@pytest.mark.gpu
def test_unknown_format_is_refused():
    from all_quant_b200 import uq_cuda
    c = CASES[0]
    q, kc, ks, vc, vs, bt, sl = _dev(c)
    with pytest.raises(RuntimeError):
        uq_cuda.uq_decode_cuda(q, kc, ks, vc, vs, bt, sl, fmt=2)


# ---------------------------------------------------------------------------------------------------- the NVFP4 append
QZ = None


def _qz():
    global QZ
    if QZ is None:
        from tests.cases import load
        QZ = load("gen_nvfp4_quant")
    return QZ


@pytest.mark.parametrize("D", (64, 128, 256))
def test_oracle_nvfp4_quantiser_matches_the_reference_bytes(D):
    z = _qz()
    codes, scales = O.quantize_nvfp4(z[f"d{D}_x"], float(z[f"d{D}_ts"]))
    assert np.array_equal(codes, z[f"d{D}_codes"])
    assert np.array_equal(scales, z[f"d{D}_scales"])
    assert scales.min() == 0x01 and scales.max() == 0x7e      # both clamps of the scale are in the fixture


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["rows", "bulk"])
@pytest.mark.parametrize("D", (64, 128, 256))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_nvfp4_append_kernel_bit_exact(D, dtype, kernel):
    from all_quant_b200 import uq_cuda
    z = _qz()
    x = torch.from_numpy(z[f"d{D}_x"]).to(dtype)
    ts = float(z[f"d{D}_ts"])
    if dtype == torch.float32:
        want_c, want_s = z[f"d{D}_codes"], z[f"d{D}_scales"]
    else:   # 16-bit input: the oracle (pinned above) on the rounded values
        want_c, want_s = O.quantize_nvfp4(x.float().numpy(), ts)
    T, HKV, _ = x.shape
    PAGE, pages = 16, 3
    kc = torch.zeros(pages, HKV, PAGE, D // 2, dtype=torch.uint8, device="cuda")
    ks = torch.zeros(pages, HKV, PAGE, D // 16, dtype=torch.uint8, device="cuda")
    vc, vs = torch.zeros_like(kc), torch.zeros_like(ks)
    slots = torch.from_numpy(np.random.default_rng(4).permutation(pages * PAGE)[:T].astype(np.int64)).cuda()
    uq_cuda.append_kv_nvfp4(kc, ks, vc, vs, x.cuda(), x.cuda(), slots, ts, ts, kernel=kernel)
    pg, at = (slots // PAGE).cpu(), (slots % PAGE).cpu()
    for codes, scales in ((kc, ks), (vc, vs)):
        assert np.array_equal(codes.cpu()[pg, :, at].numpy(), want_c)
        assert np.array_equal(scales.cpu()[pg, :, at].numpy(), want_s)


def _nv_steps(v, dtype, k):
    """v (fp32 numpy, > 0) moved k representable steps of `dtype`."""
    if dtype == torch.bfloat16:
        b = (v.view(np.uint32) >> 16).astype(np.int64) + k
        return (b.astype(np.uint32) << 16).view(np.float32)
    t, iv = (np.float32, np.int32) if dtype == torch.float32 else (np.float16, np.int16)
    return (v.astype(t).view(iv) + iv(k)).view(t).astype(np.float32)


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["rows", "bulk"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_nvfp4_append_on_and_beside_every_code_boundary(dtype, kernel):
    """Blocks whose scale is exactly a power of two (maximum 6 * 2^k, ts = 1) hold the code boundaries themselves, where the
    reference takes the smaller magnitude, their nearest neighbours in the input's type, zeros of both signs and tiny values;
    the bulk kernel brackets the quotient and must fall back to the division exactly there.  A second tensor scale (0.3:
    quotients that are not exact) runs the same values through rounded quotients."""
    from all_quant_b200 import uq_cuda
    thr = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    cand = np.concatenate([_nv_steps(thr, dtype, k) for k in (-2, -1, 0, 1, 2)])
    cand = np.concatenate([cand, -cand, np.array([0.0, -0.0, 1e-30, -1e-30, 6.0, -6.0, 0.5, -1.0, 4.0, -3.0, -1e-38, 2e-45, -2e-45], np.float32)])
    blocks = []
    for k in (-6, -1, 0, 3, 7):
        v = cand * np.float32(2.0 ** k)
        n = (v.size + 14) // 15
        g = np.zeros((n, 16), np.float32)
        g[:, 0] = 6.0 * 2.0 ** k
        g[:, 1:].reshape(-1)[: v.size] = v
        blocks.append(g)
    x = np.concatenate(blocks)
    x = np.concatenate([x, np.zeros(((-x.shape[0]) % 4, 16), np.float32)]).reshape(-1, 1, 64)
    xt = torch.from_numpy(x).to(dtype)
    T = xt.shape[0]
    for ts in (1.0, 0.3):
        want_c, want_s = O.quantize_nvfp4(xt.float().numpy(), ts)
        PAGE = 16
        pages = (T + PAGE - 1) // PAGE
        kc = torch.zeros(pages, 1, PAGE, 32, dtype=torch.uint8, device="cuda")
        ks = torch.zeros(pages, 1, PAGE, 4, dtype=torch.uint8, device="cuda")
        vc, vs = torch.zeros_like(kc), torch.zeros_like(ks)
        uq_cuda.append_kv_nvfp4(kc, ks, vc, vs, xt.cuda(), xt.cuda(), torch.arange(T, device="cuda"), ts, ts, kernel=kernel)
        assert np.array_equal(ks.reshape(-1, 1, 4)[:T].cpu().numpy(), want_s)
        assert np.array_equal(kc.reshape(-1, 1, 32)[:T].cpu().numpy(), want_c)
        assert np.array_equal(vc.reshape(-1, 1, 32)[:T].cpu().numpy(), want_c)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,HKV,PAGE", [(64, 1, 16), (128, 3, 48), (128, 8, 64), (256, 5, 32)])
def test_nvfp4_bulk_kernel_writes_the_bytes_of_the_row_kernel_and_the_oracle(D, HKV, PAGE, dtype):
    """Seeded keys and values of very different magnitude (scale bytes from the lower clamp to the upper one), scattered
    slots with skipped tokens, head counts and page sizes that do not line up with a warp's run of rows."""
    from all_quant_b200 import uq_cuda
    g = torch.Generator(device="cuda").manual_seed(3 * D + HKV + PAGE)
    T = 1000 + HKV
    pages = (T + PAGE - 1) // PAGE + 2
    mag = torch.exp2(torch.randint(-12, 9, (T, HKV, D // 16, 1), generator=g, device="cuda").float())
    k = (torch.randn(T, HKV, D // 16, 16, generator=g, device="cuda") * mag).reshape(T, HKV, D).to(dtype)
    v = (torch.randn(T, HKV, D, generator=g, device="cuda") * 0.3).to(dtype)
    slots = torch.randperm(pages * PAGE, generator=g, device="cuda")[:T]
    slots[::11] = -1
    k_ts, v_ts = 0.013, 0.0021
    out = {}
    for kernel in ("rows", "bulk"):
        kc = torch.full((pages, HKV, PAGE, D // 2), 0xA5, dtype=torch.uint8, device="cuda")
        ks = torch.full((pages, HKV, PAGE, D // 16), 0x5A, dtype=torch.uint8, device="cuda")
        vc, vs = kc.clone(), ks.clone()
        uq_cuda.append_kv_nvfp4(kc, ks, vc, vs, k, v, slots, k_ts, v_ts, kernel=kernel)
        torch.cuda.synchronize()
        out[kernel] = [t.cpu().numpy() for t in (kc, ks, vc, vs)]
    for a, b in zip(out["rows"], out["bulk"]):
        assert np.array_equal(a, b)
    sl = slots.cpu().numpy()
    keep = sl >= 0
    for x, ts, (codes, scales) in ((k, k_ts, out["bulk"][:2]), (v, v_ts, out["bulk"][2:])):
        want_c, want_s = O.quantize_nvfp4(x.float().cpu().numpy(), ts)
        ref_c = np.full((pages, HKV, PAGE, D // 2), 0xA5, np.uint8)
        ref_s = np.full((pages, HKV, PAGE, D // 16), 0x5A, np.uint8)
        ref_c[sl[keep] // PAGE, :, sl[keep] % PAGE] = want_c[keep]
        ref_s[sl[keep] // PAGE, :, sl[keep] % PAGE] = want_s[keep]
        assert np.array_equal(codes, ref_c) and np.array_equal(scales, ref_s)
    ks_written = out["bulk"][1][sl[keep] // PAGE, :, sl[keep] % PAGE]
    assert ks_written.min() <= 0x08 and ks_written.max() >= 0x70      # both ends of the scale's range are in the data


@pytest.mark.gpu
def test_nvfp4_append_then_decode_follows_the_oracle():
    """A cache written by the NVFP4 append and read by the verify call, against the oracle on the same float data."""
    from all_quant_b200 import uq_cuda
    rng = np.random.default_rng(17)
    B, K, HQ, HKV, D, PAGE, ctx = 2, 4, 8, 2, 128, 64, 600
    npg = -(-ctx // PAGE)
    k = rng.standard_normal((B * ctx, HKV, D)).astype(np.float32) * 2.0
    v = rng.standard_normal((B * ctx, HKV, D)).astype(np.float32)
    k_ts, v_ts = 16.0 / (6 * 448), 8.0 / (6 * 448)
    bt = rng.permutation(B * npg).astype(np.int32).reshape(B, npg)
    pos = np.tile(np.arange(ctx), B)
    slots = bt[np.repeat(np.arange(B), ctx), pos // PAGE].astype(np.int64) * PAGE + pos % PAGE
    kc = torch.zeros(B * npg, HKV, PAGE, D // 2, dtype=torch.uint8, device="cuda")
    ks = torch.zeros(B * npg, HKV, PAGE, D // 16, dtype=torch.uint8, device="cuda")
    vc, vs = torch.zeros_like(kc), torch.zeros_like(ks)
    uq_cuda.append_kv_nvfp4(kc, ks, vc, vs, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), torch.from_numpy(slots).cuda(), k_ts, v_ts)
    # the same bytes from the oracle's quantiser, scattered on the host
    kcw, ksw = O.quantize_nvfp4(k, k_ts)
    vcw, vsw = O.quantize_nvfp4(v, v_ts)
    pg, at = slots // PAGE, slots % PAGE
    assert np.array_equal(kc.cpu().numpy()[pg, :, at], kcw) and np.array_equal(ks.cpu().numpy()[pg, :, at], ksw)
    assert np.array_equal(vc.cpu().numpy()[pg, :, at], vcw) and np.array_equal(vs.cpu().numpy()[pg, :, at], vsw)
    qb = O.bf16_bits(rng.standard_normal((B, K, HQ, D)).astype(np.float32))
    sl = np.full(B, ctx, np.int32)
    want = O.reference_nvfp4(qb, kc.cpu().numpy(), ks.cpu().numpy(), vc.cpu().numpy(), vs.cpu().numpy(), bt, sl, k_ts, v_ts)
    q = torch.from_numpy(qb.view(np.int16)).cuda().view(torch.bfloat16)
    out = uq_cuda.uq_decode_cuda(q, kc, ks, vc, vs, torch.from_numpy(bt).cuda(), torch.from_numpy(sl).cuda(), fmt=1, k_ts=k_ts, v_ts=v_ts)
    check_close(out.float().cpu().numpy(), want, "append + decode")
