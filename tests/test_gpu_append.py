"""KV append-quantize kernel: bytes identical to the reference encoder (fixtures made by the reference's
quantize_fp4 / append_kv) and to the CPU oracle on seeded inputs.  Needs a B200."""
import numpy as np
import pytest
import torch

from all_quant_b200 import uq_cuda
from oracle import uq_oracle as O
from tests.cases import load

pytestmark = pytest.mark.gpu


KERNELS = ["rows", "bulk"]   # one warp per row (decode steps) and the bulk kernel (prompts): same bytes


def encode_on_gpu(x, dtype=torch.float32, rule="ceil", c=None, kernel=None):
    """x fp32 numpy [N, D] -> (packed, scales) via quantize_on_write into a fresh one-head cache."""
    N, D = x.shape
    PAGE = 64
    pages = (N + PAGE - 1) // PAGE
    code = torch.zeros(pages, 1, PAGE, D // 2, dtype=torch.uint8, device="cuda")
    scale = torch.zeros(pages, 1, PAGE, D // 32, dtype=torch.uint8, device="cuda")
    xt = torch.from_numpy(x).cuda().to(dtype).reshape(N, 1, D)
    uq_cuda.quantize_on_write(xt, code, scale, torch.arange(N, device="cuda"), rule=rule, c=c, kernel=kernel)
    torch.cuda.synchronize()
    return code.reshape(-1, D // 2)[:N].cpu().numpy(), scale.reshape(-1, D // 32)[:N].cpu().numpy()


@pytest.mark.parametrize("name,dtype", [("wide", torch.float32), ("bf16in", torch.float32), ("bf16in", torch.bfloat16),
                                        ("fp16in", torch.float32), ("fp16in", torch.float16)])
@pytest.mark.parametrize("kernel", KERNELS)
def test_encoder_bit_exact_with_reference_fixture(name, dtype, kernel):
    z = load("gen_codec")
    p, s = encode_on_gpu(z[f"{name}_x"], dtype, kernel=kernel)
    assert np.array_equal(s, z[f"{name}_scales"])
    assert np.array_equal(p, z[f"{name}_packed"])


@pytest.mark.parametrize("kernel", KERNELS)
def test_encoder_ties_specials_and_every_scale_boundary(kernel):
    z = load("gen_codec")
    x = z["g32_x"]                                   # [n, 32] single groups
    n = x.shape[0] // 2 * 2
    p, s = encode_on_gpu(x[:n].reshape(n // 2, 64), kernel=kernel)  # two groups per row of a D=64 cache
    assert np.array_equal(s.reshape(-1), z["g32_scales"][:n].reshape(-1))
    assert np.array_equal(p.reshape(n, 16), z["g32_packed"][:n])


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("rule", ["ceil", "paper"])
def test_scale_exponent_around_its_deciding_points(rule, kernel):
    """Group maxima a few ulp either side of every point where the exponent steps (6 * 2^n for 'ceil', 2^(n + 1/2) / c for
    'paper'), plus a dense random sweep: the kernel's fp32 shortcut for the logarithm must never change the byte."""
    c = 0.156
    n = np.arange(-100, 101, dtype=np.float64)
    centre = (6.0 * 2.0 ** n) if rule == "ceil" else (2.0 ** (n + 0.5) / np.float64(np.float32(c)))
    centre = centre.astype(np.float32)
    amax = []
    for k in range(-6, 7):
        a = centre.copy()
        for _ in range(abs(k)):
            a = np.nextafter(a, np.float32(np.inf if k > 0 else 0), dtype=np.float32)
        amax.append(a)
    rng = np.random.default_rng(21)
    amax.append(np.exp2(rng.uniform(-100, 100, 40000)).astype(np.float32))
    amax = np.concatenate(amax)
    amax = amax[: amax.size // 2 * 2]
    x = (rng.uniform(-1, 1, (amax.size, 32)).astype(np.float32)) * amax[:, None]
    x[:, 7] = amax * np.where(rng.random(amax.size) < 0.5, -1, 1).astype(np.float32)     # the group's maximum itself
    want_p, want_s = O.quantize(x, rule, c)
    p, s = encode_on_gpu(x.reshape(-1, 64), rule=rule, c=c, kernel=kernel)
    assert np.array_equal(s.reshape(-1), want_s.reshape(-1))
    assert np.array_equal(p.reshape(-1, 16), want_p)


_NP_OF = {torch.float32: np.float32, torch.float16: np.float16}


def _steps(v, dtype, k):
    """v moved k representable steps of `dtype` away from / towards zero (v > 0, fp32 numpy array in, fp32 out)."""
    if dtype == torch.bfloat16:
        b = (v.view(np.uint32) >> 16).astype(np.int64) + k
        return (b.astype(np.uint32) << 16).view(np.float32)
    t = _NP_OF[dtype]
    iv = np.int32 if t is np.float32 else np.int16
    return (v.astype(t).view(iv) + iv(k)).view(t).astype(np.float32)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_values_on_and_beside_every_code_boundary(dtype, kernel):
    """The code boundaries (.25 .75 1.25 1.75 2.5 3.5 5 times the group's scale) themselves, where the reference takes the
    smaller magnitude, and the nearest values of the input's type either side of them, both signs, at several scales; the
    bulk kernel's hardware conversion rounds half-way values to even and is corrected to the reference's rule."""
    thr = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    cand = np.concatenate([_steps(thr, dtype, k) for k in (-2, -1, 0, 1, 2)])
    cand = np.concatenate([cand, -cand, np.array([0.0, -0.0, 1e-30, -1e-30, 6.0, -6.0, 0.5, -1.0, 4.0, -3.0], np.float32)])
    groups = []
    for k in (-10, -1, 0, 3, 10):
        v = cand * np.float32(2.0 ** k)
        n = (v.size + 30) // 31
        g = np.zeros((n, 32), np.float32)
        g[:, 0] = 6.0 * 2.0 ** k                      # the group's maximum: scale 2^k
        g[:, 1:].reshape(-1)[: v.size] = v
        groups.append(g)
    x = np.concatenate(groups)
    x = np.concatenate([x, x[: x.shape[0] % 2]])       # two groups per row of a D=64 cache
    want_p, want_s = O.quantize(x, "ceil")
    p, s = encode_on_gpu(x.reshape(-1, 64), dtype, kernel=kernel)
    assert np.array_equal(s.reshape(-1), want_s.reshape(-1))
    assert np.array_equal(p.reshape(-1, 16), want_p)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_negative_values_that_underflow_under_the_scale_take_code_zero(dtype, kernel):
    """A negative value so far below the group's maximum that x / scale rounds to -0 is not 'y < 0' in the reference: code 0,
    not the minus-zero code; a negative value that survives the division as a denormal keeps its sign bit."""
    tiny = np.float32(2.0 ** -133)                    # representable in bf16 and fp32
    g = np.zeros((4, 32), np.float32)
    g[0, 0] = 6.0 * 2.0 ** 40; g[0, 1:5] = [-tiny, tiny, -0.0, -tiny * 4]          # y = -2^-173: gone
    g[1, 0] = 6.0 * 2.0 ** 16; g[1, 1:5] = [-tiny, tiny, -0.0, -tiny * 4]          # y = -2^-149: the smallest denormal survives
    g[2, 0] = 6.0 * 2.0 ** 17; g[2, 1:5] = [-tiny, tiny, -0.0, -tiny * 4]          # y = -2^-150: half way, rounds to -0
    g[3, 0] = -6.0 * 2.0 ** 100; g[3, 1:5] = [-tiny, -1e-20, -0.0, 1e-20]
    want_p, want_s = O.quantize(g, "ceil")
    p, s = encode_on_gpu(g.reshape(-1, 64), dtype, kernel=kernel)
    assert np.array_equal(s.reshape(-1), want_s.reshape(-1))
    assert np.array_equal(p.reshape(-1, 16), want_p)
    assert want_p[0, 0] >> 4 == 0 and want_p[1, 0] >> 4 == 8      # the oracle itself: gone / kept


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_bulk_kernel_on_every_16_bit_value_up_to_the_group_maximum(dtype):
    """All bit patterns of the input type with |x| <= 6 (and the same a few binades up and down), beside a 6 that fixes the
    scale: the bulk kernel's one-step-down multiplier must give the reference's code for each of them."""
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    v = bits.view(dtype).float().numpy()
    v = v[np.isfinite(v) & (np.abs(v) <= 6.0)]
    groups = []
    for k in (0, -7, 5):
        w = v * np.float32(2.0 ** k)
        n = (w.size + 30) // 31
        g = np.zeros((n, 32), np.float32)
        g[:, 0] = 6.0 * 2.0 ** k
        g[:, 1:].reshape(-1)[: w.size] = w
        groups.append(g)
    x = np.concatenate(groups)
    x = np.concatenate([x, x[: x.shape[0] % 2]])
    want_p, want_s = O.quantize(x, "ceil")
    p, s = encode_on_gpu(x.reshape(-1, 64), dtype, kernel="bulk")
    assert np.array_equal(s.reshape(-1), want_s.reshape(-1))
    assert np.array_equal(p.reshape(-1, 16), want_p)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,HKV,PAGE", [(64, 1, 16), (128, 3, 48), (128, 8, 64), (256, 5, 32), (64, 7, 80)])
@pytest.mark.parametrize("rule", ["ceil", "paper"])
def test_bulk_kernel_writes_the_bytes_of_the_row_kernel_and_the_oracle(D, HKV, PAGE, dtype, rule):
    """Both streams, scattered slots with skipped tokens, head counts that do not divide a warp's run of rows, page sizes
    that are not powers of two, a token count that leaves a ragged last warp."""
    g = torch.Generator(device="cuda").manual_seed(D + HKV + PAGE)
    T = 1000 + HKV
    pages = (T + PAGE - 1) // PAGE + 2
    chan = torch.exp(0.5 * torch.randn(1, HKV, D, generator=g, device="cuda"))
    k = (torch.randn(T, HKV, D, generator=g, device="cuda") * chan * 37.0).to(dtype)
    v = (torch.randn(T, HKV, D, generator=g, device="cuda") * 0.01).to(dtype)
    slots = torch.randperm(pages * PAGE, generator=g, device="cuda")[:T]
    slots[::13] = -1
    out = {}
    for kernel in KERNELS:
        kc = torch.full((pages, HKV, PAGE, D // 2), 0xA5, dtype=torch.uint8, device="cuda")
        ks = torch.full((pages, HKV, PAGE, D // 32), 0x5A, dtype=torch.uint8, device="cuda")
        vc, vs = kc.clone(), ks.clone()
        uq_cuda.append_kv(kc, ks, vc, vs, k, v, slots, rule=rule, kernel=kernel)
        torch.cuda.synchronize()
        out[kernel] = [t.cpu().numpy() for t in (kc, ks, vc, vs)]
    for a, b in zip(out["rows"], out["bulk"]):
        assert np.array_equal(a, b)
    sl = slots.cpu().numpy()
    keep = sl >= 0
    for x, (codes, scales) in ((k, out["bulk"][:2]), (v, out["bulk"][2:])):
        want_p, want_s = O.quantize(x.float().cpu().numpy().reshape(T * HKV, D), rule)
        ref_c = np.full((pages, HKV, PAGE, D // 2), 0xA5, np.uint8)
        ref_s = np.full((pages, HKV, PAGE, D // 32), 0x5A, np.uint8)
        ref_c[sl[keep] // PAGE, :, sl[keep] % PAGE] = want_p.reshape(T, HKV, D // 2)[keep]
        ref_s[sl[keep] // PAGE, :, sl[keep] % PAGE] = want_s.reshape(T, HKV, D // 32)[keep]
        assert np.array_equal(codes, ref_c) and np.array_equal(scales, ref_s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,HKV", [(64, 3), (128, 8), (256, 2)])
def test_bulk_kernel_rotates_keys_like_the_row_kernel(D, HKV, dtype):
    """Rotated keys (the transform across the D / 8 lanes of a row, its result rounded to the input's type) and unrotated
    values in one call: the bulk kernel's bytes equal the row kernel's, whose rotation is pinned to the reference's function."""
    g = torch.Generator(device="cuda").manual_seed(7 * D + HKV)
    T, PAGE = 777, 32
    pages = (T + PAGE - 1) // PAGE
    k = (torch.randn(T, HKV, D, generator=g, device="cuda") * torch.exp(torch.randn(1, HKV, D, generator=g, device="cuda"))).to(dtype)
    v = torch.randn(T, HKV, D, generator=g, device="cuda").to(dtype)
    slots = torch.randperm(pages * PAGE, generator=g, device="cuda")[:T]
    out = {}
    for kernel in KERNELS:
        kc = torch.zeros(pages, HKV, PAGE, D // 2, dtype=torch.uint8, device="cuda")
        ks = torch.zeros(pages, HKV, PAGE, D // 32, dtype=torch.uint8, device="cuda")
        vc, vs = kc.clone(), ks.clone()
        uq_cuda.append_kv(kc, ks, vc, vs, k, v, slots, rotate_k=True, rule="paper", kernel=kernel)
        torch.cuda.synchronize()
        out[kernel] = [t.cpu().numpy() for t in (kc, ks, vc, vs)]
    for a, b in zip(out["rows"], out["bulk"]):
        assert np.array_equal(a, b)
    assert out["bulk"][0].any() and out["bulk"][2].any()


def test_bulk_kernel_named_for_a_call_it_does_not_serve_is_an_error():
    kc = torch.zeros(4, 1, 16, 64, dtype=torch.uint8, device="cuda")
    ks = torch.zeros(4, 1, 16, 4, dtype=torch.uint8, device="cuda")
    x = torch.randn(8 * 128 + 1, device="cuda")[1:].view(8, 1, 128)   # contiguous, 4 bytes off a 16-byte boundary
    with pytest.raises(RuntimeError):
        uq_cuda.append_kv(kc, ks, kc.clone(), ks.clone(), x, x, torch.arange(8, device="cuda"), kernel="bulk")
    uq_cuda.append_kv(kc, ks, kc.clone(), ks.clone(), x, x, torch.arange(8, device="cuda"))          # by size: the row kernel takes it
    with pytest.raises(ValueError):
        uq_cuda.append_kv(kc, ks, kc.clone(), ks.clone(), x, x, torch.arange(8, device="cuda"), kernel="both")


def test_append_kv_matches_reference_fixture():
    z = load("gen_append")
    kc, ks, vc, vs = (torch.from_numpy(z[n].copy()).cuda() for n in ("kc0", "ks0", "vc0", "vs0"))
    key = torch.from_numpy(z["key"].view(np.int16)).cuda().view(torch.bfloat16)
    val = torch.from_numpy(z["value"].view(np.int16)).cuda().view(torch.bfloat16)
    uq_cuda.append_kv(kc, ks, vc, vs, key, val, torch.from_numpy(z["slots"]).cuda())
    torch.cuda.synchronize()
    for got, name in ((kc, "kc1"), (ks, "ks1"), (vc, "vc1"), (vs, "vs1")):
        assert np.array_equal(got.cpu().numpy(), z[name]), name


@pytest.mark.parametrize("D", [64, 128, 256])
def test_cache_build_bit_exact_with_oracle_on_seeded_kv(D):
    """The benchmark's cache is built by this kernel: lognormal-channel K, N(0,1) V, fp32 in."""
    g = torch.Generator(device="cuda").manual_seed(1000 + D)
    T, HKV, PAGE = 4096, 2, 64
    chan = torch.exp(0.5 * torch.randn(1, HKV, D, generator=g, device="cuda"))
    k = torch.randn(T, HKV, D, generator=g, device="cuda") * chan
    v = torch.randn(T, HKV, D, generator=g, device="cuda")
    pages = T // PAGE
    kc = torch.zeros(pages, HKV, PAGE, D // 2, dtype=torch.uint8, device="cuda")
    ks = torch.zeros(pages, HKV, PAGE, D // 32, dtype=torch.uint8, device="cuda")
    vc, vs = torch.zeros_like(kc), torch.zeros_like(ks)
    slots = torch.randperm(T, generator=g, device="cuda")
    uq_cuda.append_kv(kc, ks, vc, vs, k, v, slots)
    torch.cuda.synchronize()
    rkc, rks, rvc, rvs = (np.zeros_like(t.cpu().numpy()) for t in (kc, ks, vc, vs))
    O.append_kv(rkc, rks, rvc, rvs, k.cpu().numpy(), v.cpu().numpy(), slots.cpu().numpy())
    for got, ref in ((kc, rkc), (ks, rks), (vc, rvc), (vs, rvs)):
        assert np.array_equal(got.cpu().numpy(), ref)


def test_negative_slots_are_skipped_and_empty_append_is_a_no_op():
    kc = torch.full((2, 1, 16, 64), 7, dtype=torch.uint8, device="cuda")
    ks = torch.full((2, 1, 16, 4), 9, dtype=torch.uint8, device="cuda")
    vc, vs = kc.clone(), ks.clone()
    x = torch.randn(3, 1, 128, device="cuda")
    uq_cuda.append_kv(kc, ks, vc, vs, x, x, torch.tensor([-1, 5, -1], device="cuda"))
    uq_cuda.append_kv(kc, ks, vc, vs, x[:0], x[:0], torch.zeros(0, dtype=torch.long, device="cuda"))
    torch.cuda.synchronize()
    untouched = torch.ones(32, dtype=torch.bool)
    untouched[5] = False
    assert (kc.reshape(32, 64)[untouched.cuda()] == 7).all() and (ks.reshape(32, 4)[untouched.cuda()] == 9).all()
    p, s = O.quantize_fp4(x[1].cpu().numpy())
    assert np.array_equal(kc.reshape(32, 64)[5].cpu().numpy(), p[0]) and np.array_equal(vs.reshape(32, 4)[5].cpu().numpy(), s[0])
