"""The engine adapter (reference uqmt/vllm_adapter.py) and the options of the append it exposes: Hadamard-rotated keys and
the 'paper' scale rule (reference uqmt/quant.py).  The fixtures of gen_rotate.npz were written by the reference's own
functions (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import uq_oracle as O
from tests.cases import check_close, load, load_cases

Z = load("gen_rotate")
DIMS = (64, 128, 256)


# ---------------------------------------------------------------------------------------------------- CPU: oracle
@pytest.mark.parametrize("D", DIMS)
def test_oracle_fwht_is_the_reference_transform_bit_for_bit(D):
    got = O.fwht(Z[f"d{D}_x"])
    assert np.array_equal(got.view(np.uint32), Z[f"d{D}_fwht"].view(np.uint32))
    # orthonormal and its own inverse
    back = O.fwht(got)
    assert np.allclose(back, Z[f"d{D}_x"], rtol=1e-5, atol=1e-5 * np.abs(Z[f"d{D}_x"]).max())


@pytest.mark.parametrize("D", DIMS)
@pytest.mark.parametrize("rule", ["ceil", "paper"])
@pytest.mark.parametrize("src", ["plain", "rot"])
def test_oracle_quantiser_rules_match_the_reference_bytes(D, rule, src):
    x = Z[f"d{D}_x"] if src == "plain" else Z[f"d{D}_fwht"]
    codes, scales = O.quantize(x, rule, float(Z["c"]))
    assert np.array_equal(codes, Z[f"d{D}_{src}_{rule}_codes"])
    assert np.array_equal(scales, Z[f"d{D}_{src}_{rule}_scales"])


def test_eligible_reasons():
    from all_quant_b200 import vllm_adapter as A
    q = torch.zeros(12, 8, 128, dtype=torch.bfloat16)
    loc = torch.tensor([0, 4, 8, 12])
    assert A.eligible(q, loc, 64) == (True, "ok", 4)
    assert A.eligible(q, loc, 64, sliding_window=-1) == (True, "ok", 4)
    assert A.eligible(q, loc, 64, sliding_window=4096) == (False, "sliding_window", 0)
    assert A.eligible(q, loc, 64, softcap=30.0) == (False, "softcap", 0)
    assert A.eligible(q.float(), loc, 64) == (False, "q_dtype", 0)
    assert A.eligible(torch.zeros(12, 8, 96, dtype=torch.bfloat16), loc, 64) == (False, "head_dim", 0)
    assert A.eligible(torch.zeros(12, 8, 256, dtype=torch.bfloat16), loc, 64) == (True, "ok", 4)
    assert A.eligible(q, loc, 8) == (False, "page_size", 0)
    assert A.eligible(q, loc, 48) == (False, "page_size", 0)
    assert A.eligible(q, torch.tensor([0, 4, 9, 12]), 64) == (False, "non_uniform_k", 0)
    assert A.eligible(torch.zeros(34, 8, 128, dtype=torch.bfloat16), torch.tensor([0, 17, 34]), 64) == (False, "non_uniform_k", 0)
    assert set(r for r in A.REASONS) >= {"ok", "non_uniform_k", "head_dim", "page_size", "q_dtype", "sliding_window", "softcap"}


def test_adapter_refuses_cpu_tensors():
    from all_quant_b200 import vllm_adapter as A
    c = load_cases("ref_cuda_main")[0]
    q = torch.zeros(c.B * c.K, c.HQ, c.D, dtype=torch.bfloat16)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    with pytest.raises(RuntimeError):
        A.uq_verify_attention(q, t(c.kc), t(c.ks), t(c.vc), t(c.vs), t(c.bt), t(c.sl), c.K)


# ---------------------------------------------------------------------------------------------------- GPU
def _bf16(bits):
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)


@pytest.mark.gpu
@pytest.mark.parametrize("D", DIMS)
def test_fwht_kernel_bit_exact(D):
    from all_quant_b200 import uq_cuda
    x = torch.from_numpy(Z[f"d{D}_x"]).cuda()
    got = uq_cuda.fwht(x)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), Z[f"d{D}_fwht"].view(np.uint32))
    q = _bf16(Z[f"d{D}_q"])
    gq = uq_cuda.fwht(q)
    assert np.array_equal(gq.view(torch.int16).cpu().numpy().view(np.uint16), Z[f"d{D}_q_fwht"])
    uq_cuda.fwht(q, out=q)   # in place
    assert torch.equal(q, gq)


@pytest.mark.gpu
@pytest.mark.parametrize("D", DIMS)
@pytest.mark.parametrize("rule", ["ceil", "paper"])
@pytest.mark.parametrize("rotate", [False, True])
@pytest.mark.parametrize("kernel", ["rows", "bulk"])
def test_append_options_bit_exact(D, rule, rotate, kernel):
    """append_kv(rotate_k, rule): the key stream equals quantize(fwht(key), rule) of the reference, the value stream
    quantize(value, rule) (values are never rotated)."""
    from all_quant_b200 import vllm_adapter as A
    x = Z[f"d{D}_x"]
    T, HKV, _ = x.shape
    PAGE, pages = 16, 4
    kc = torch.zeros(pages, HKV, PAGE, D // 2, dtype=torch.uint8, device="cuda")
    ks = torch.zeros(pages, HKV, PAGE, D // 32, dtype=torch.uint8, device="cuda")
    vc, vs = torch.zeros_like(kc), torch.zeros_like(ks)
    slots = torch.from_numpy(np.random.default_rng(3).permutation(pages * PAGE)[:T].astype(np.int64)).cuda()
    xd = torch.from_numpy(x).cuda()
    A.append_kv(kc, ks, vc, vs, xd, xd, slots, rotate_k=rotate, rule=rule, c=float(Z["c"]), kernel=kernel)
    pg, at = (slots // PAGE).cpu(), (slots % PAGE).cpu()
    src = "rot" if rotate else "plain"
    assert np.array_equal(kc.cpu()[pg, :, at].numpy(), Z[f"d{D}_{src}_{rule}_codes"])
    assert np.array_equal(ks.cpu()[pg, :, at].numpy(), Z[f"d{D}_{src}_{rule}_scales"])
    assert np.array_equal(vc.cpu()[pg, :, at].numpy(), Z[f"d{D}_plain_{rule}_codes"])
    assert np.array_equal(vs.cpu()[pg, :, at].numpy(), Z[f"d{D}_plain_{rule}_scales"])


@pytest.mark.gpu
def test_bf16_keys_rotate_like_the_reference_function():
    """A 16-bit input: the reference's transform returns its input's type, so the rotated row is rounded to bf16 before it is
    encoded; the oracle restates that (fwht in fp32, round to bf16, quantize)."""
    from all_quant_b200 import uq_cuda
    D, T, HKV, PAGE = 128, 24, 2, 32
    xb = torch.from_numpy(Z["d128_x"]).bfloat16()
    want_c, want_s = O.quantize(torch.from_numpy(O.fwht(xb.float().numpy())).bfloat16().float().numpy(), "ceil")
    kc = torch.zeros(1, HKV, PAGE, D // 2, dtype=torch.uint8, device="cuda")
    ks = torch.zeros(1, HKV, PAGE, D // 32, dtype=torch.uint8, device="cuda")
    for kernel in ("rows", "bulk"):
        kc.zero_(); ks.zero_()
        uq_cuda.append_kv(kc, ks, torch.zeros_like(kc), torch.zeros_like(ks), xb.cuda(), xb.cuda(), torch.arange(T, device="cuda"), rotate_k=True, kernel=kernel)
        assert np.array_equal(kc.cpu().numpy()[0, :, :T].transpose(1, 0, 2), want_c)
        assert np.array_equal(ks.cpu().numpy()[0, :, :T].transpose(1, 0, 2), want_s)


@pytest.mark.gpu
def test_verify_attention_varlen_layout_matches_the_reference_answer():
    from all_quant_b200 import uq_cuda, vllm_adapter as A
    for c in load_cases("ref_cuda_main") + load_cases("gen_d256"):
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        q = _bf16(c.q).reshape(c.B * c.K, c.HQ, c.D)
        loc = torch.arange(0, c.B * c.K + 1, c.K)
        ok, why, K = A.eligible(q, loc, c.PAGE)
        assert (ok, why, K) == (True, "ok", c.K)
        args = (t(c.kc), t(c.ks), t(c.vc), t(c.vs), t(c.bt), t(c.sl))
        out = A.uq_verify_attention(q, *args, K, sm_scale=c.sm_scale)
        assert out.shape == q.shape
        check_close(out.float().cpu().numpy().reshape(c.ref.shape), c.ref, str(c))
        # caller-owned scratch and output: same answer
        ws = torch.empty(uq_cuda.workspace_floats(c.B, c.K, c.HQ, c.HKV, c.D, 4), dtype=torch.float32, device="cuda")
        o2 = torch.empty_like(q)
        A.uq_verify_attention(q, *args, K, sm_scale=c.sm_scale, workspace=ws, out=o2)
        check_close(o2.float().cpu().numpy().reshape(c.ref.shape), c.ref, str(c) + " scratch")


@pytest.mark.gpu
@pytest.mark.parametrize("D", (64, 128))
def test_rotated_cache_end_to_end(D):
    """Keys appended with rotate_k, queries rotated by the adapter: the answer is the oracle's on the same cache bytes with
    the oracle's rotated queries, and strongly correlated with the answer of the unrotated cache (q.k is invariant up to quantisation)."""
    from all_quant_b200 import vllm_adapter as A
    rng = np.random.default_rng(9)
    B, K, HQ, HKV, PAGE, ctx = 2, 4, 8, 2, 64, 700
    npg = -(-ctx // PAGE)
    k = (rng.standard_normal((B * ctx, HKV, D)) * np.exp(0.5 * rng.standard_normal((1, HKV, D)))).astype(np.float32)
    v = rng.standard_normal((B * ctx, HKV, D)).astype(np.float32)
    bt = rng.permutation(B * npg).astype(np.int32).reshape(B, npg)
    pos = np.tile(np.arange(ctx), B)
    slots = (bt[np.repeat(np.arange(B), ctx), pos // PAGE].astype(np.int64) * PAGE + pos % PAGE)
    qf = rng.standard_normal((B * K, HQ, D)).astype(np.float32)
    qb = O.bf16_bits(qf)
    sl = np.full(B, ctx, np.int32)
    outs = {}
    for rot in (False, True):
        kc = torch.zeros(B * npg, HKV, PAGE, D // 2, dtype=torch.uint8, device="cuda")
        ks = torch.zeros(B * npg, HKV, PAGE, D // 32, dtype=torch.uint8, device="cuda")
        vc, vs = torch.zeros_like(kc), torch.zeros_like(ks)
        A.append_kv(kc, ks, vc, vs, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), torch.from_numpy(slots).cuda(), rotate_k=rot)
        out = A.uq_verify_attention(_bf16(qb), kc, ks, vc, vs, torch.from_numpy(bt).cuda(), torch.from_numpy(sl).cuda(), K, rotate_q=rot)
        q_or = qb
        if rot:   # the oracle's rotated queries: transform in fp32, rounded to bf16 like the reference's function
            q_or = O.bf16_bits(O.fwht(O.bf16_to_f32(qb)))   # (bf16_bits rounds to nearest even, as the conversion to bf16 does)
        want = O.reference(q_or.reshape(B, K, HQ, D), kc.cpu().numpy(), ks.cpu().numpy(), vc.cpu().numpy(), vs.cpu().numpy(), bt, sl)
        got = out.float().cpu().numpy().reshape(B, K, HQ, D)
        check_close(got, want, f"rot={rot}")
        outs[rot] = got
    # two FP4 encodings of the same keys in two bases: the answers differ by quantisation noise only (correlation 0.92 / 0.96 here)
    assert np.corrcoef(outs[True].ravel(), outs[False].ravel())[0, 1] >= 0.8
