"""Parity of the CUDA verify/decode attention with the reference's known answers and with the CPU oracle,
through the C ABI (all_quant_b200.uq_cuda -> libuq_b200.so).  Needs a B200."""
import numpy as np
import pytest
import torch

from all_quant_b200 import uq_cuda
from oracle import uq_oracle as O
from tests.cases import check_close, check_harness_rule, load_cases

pytestmark = pytest.mark.gpu
CASES = load_cases()


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


def run_case(c, **kw):
    q = dev(c.q.view(np.int16), torch.bfloat16)
    out = uq_cuda.uq_decode_cuda(q, dev(c.kc), dev(c.ks), dev(c.vc), dev(c.vs), dev(c.bt), dev(c.sl), sm_scale=c.sm_scale, **kw)
    torch.cuda.synchronize()
    assert uq_cuda.last_status()[0] == 0
    return out.float().cpu().numpy()


@pytest.mark.parametrize("c", CASES, ids=repr)
def test_known_answers(c):
    got = run_case(c)
    check_close(got, c.ref, c.name)
    check_harness_rule(got, c.ref, c.name)
    for b in range(c.B):            # rows that see no key are exact zeros
        for j in range(c.K):
            if c.sl[b] - c.K + j + 1 <= 0:
                assert not got[b, j].any()


@pytest.mark.parametrize("c", [x for x in CASES if x.name in ("ref_cuda_main_K8", "gen_k8g8_K8", "ref_cuda_p16_g4_K3", "gen_d256_K8")], ids=repr)
@pytest.mark.parametrize("nsplit", [1, 2, 3, 7, 16])
def test_nsplit_invariance(c, nsplit):
    check_close(run_case(c, nsplit=nsplit), c.ref, f"{c.name} nsplit={nsplit}")


@pytest.mark.parametrize("c", [x for x in CASES if x.name in ("ref_cuda_main_K4", "gen_cfg0_K4", "gen_g7_K3")], ids=repr)
def test_fused_equals_no_sharing(c):
    a = run_case(c, fused=True)
    b = run_case(c, fused=False)
    check_close(b, c.ref, c.name + " no-sharing")
    assert np.abs(a - b).max() <= 2e-2 * max(1.0, np.abs(c.ref).max())


@pytest.mark.parametrize("path", ["fma", "tc"])
def test_both_kernels_on_the_same_case(path, monkeypatch):
    c = [x for x in CASES if x.name == "ref_cuda_main_K8"][0]
    monkeypatch.setenv("UQ_B200_CFG", f"path={path}")
    try:
        got = run_case(c)
    except RuntimeError as e:   # a forced kernel that does not serve the shape answers invalid value, never garbage
        assert "InvalidValue" in str(e)
        pytest.skip(f"{path} kernel does not serve this shape")
    assert uq_cuda.last_path() == (1 if path == "fma" else 2)
    check_close(got, c.ref, f"{c.name} {path}")


def test_caller_workspace_int64_tables_and_out_argument():
    c = [x for x in CASES if x.name == "ref_cuda_main_K4"][0]
    q = dev(c.q.view(np.int16), torch.bfloat16)
    ns = 5
    ws = torch.full((uq_cuda.workspace_floats(c.B, c.K, c.HQ, c.HKV, c.D, ns),), float("nan"), device="cuda")
    out = torch.full_like(q, float("nan"))
    r = uq_cuda.uq_decode_cuda(q, dev(c.kc), dev(c.ks), dev(c.vc), dev(c.vs), dev(c.bt).long(), dev(c.sl).long(), nsplit=ns,
                               workspace=ws, out=out)
    assert r.data_ptr() == out.data_ptr()
    check_close(out.float().cpu().numpy(), c.ref, "workspace")


def test_poisoned_tail_and_unused_table_entries():
    """Bytes after seq_len in the last page and page-table entries past the sequence may hold anything."""
    c = [x for x in CASES if x.name == "gen_cfg0_K4"][0]
    kc, ks, vc, vs, bt = (a.copy() for a in (c.kc, c.ks, c.vc, c.vs, c.bt))
    for b in range(c.B):
        n = int(c.sl[b])
        last = bt[b, (n - 1) // c.PAGE]
        t = n % c.PAGE
        if t:
            for a in (kc, ks, vc, vs):
                a[last, :, t:] = 0xFF
        bt[b, (n + c.PAGE - 1) // c.PAGE:] = -1
    q = dev(c.q.view(np.int16), torch.bfloat16)
    out = uq_cuda.uq_decode_cuda(q, dev(kc), dev(ks), dev(vc), dev(vs), dev(bt), dev(c.sl))
    check_close(out.float().cpu().numpy(), c.ref, "poisoned tail")


def test_scale_extremes():
    """Scale bytes far from 127 (2^+-20): outputs follow the oracle on the same bytes."""
    c = [x for x in CASES if x.name == "ref_cuda_main_K2"][0]
    ks = (c.ks.astype(np.int32) - 20).clip(0, 255).astype(np.uint8)
    vs = (c.vs.astype(np.int32) + 20).clip(0, 255).astype(np.uint8)
    ref = O.reference(c.q, c.kc, ks, c.vc, vs, c.bt, c.sl, c.sm_scale)
    q = dev(c.q.view(np.int16), torch.bfloat16)
    out = uq_cuda.uq_decode_cuda(q, dev(c.kc), dev(ks), dev(c.vc), dev(vs), dev(c.bt), dev(c.sl))
    mx = np.abs(ref).max()      # outputs are ~2^20 here: apply the acceptance rule to outputs normalised to O(1)
    check_close(out.float().cpu().numpy() / mx, ref / mx, "scale extremes")


@pytest.mark.parametrize("K,HQ,HKV,D", [(16, 16, 2, 128), (12, 16, 2, 128), (8, 32, 2, 64), (16, 8, 1, 256), (13, 14, 2, 128)])
def test_more_than_64_query_rows_run_as_draft_chunks_on_the_tensor_core_kernel(K, HQ, HKV, D):
    """K * group between 65 and 128 rows: consecutive drafts are verified in chunks of at most 64 rows, each chunk against
    the sequence cut after it; answers follow the oracle, short sequences (fewer tokens than drafts) included."""
    rng = np.random.default_rng(K * 100 + HQ)
    B, PAGE = 3, 32
    sl = np.array([900, 5, 333], np.int32)       # 5 < K: some drafts see nothing or only part of the tokens
    npg = -(-int(sl.max()) // PAGE)
    pages = B * npg
    k = rng.standard_normal((pages, HKV, PAGE, D)).astype(np.float32) * np.exp(0.5 * rng.standard_normal((1, HKV, 1, D))).astype(np.float32)
    v = rng.standard_normal((pages, HKV, PAGE, D)).astype(np.float32)
    kc, ks = O.quantize_fp4(k)
    vc, vs = O.quantize_fp4(v)
    bt = rng.permutation(pages).astype(np.int32).reshape(B, npg)
    qb = O.bf16_bits(rng.standard_normal((B, K, HQ, D)).astype(np.float32))
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl)
    q = dev(qb.view(np.int16), torch.bfloat16)
    args = (dev(kc), dev(ks), dev(vc), dev(vs), dev(bt), dev(sl))
    for nsplit in (None, 2):
        out = uq_cuda.uq_decode_cuda(q, *args, nsplit=nsplit)
        assert uq_cuda.last_path() == 2 and uq_cuda.last_status() == (0, 0, 0, 0)
        check_close(out.float().cpu().numpy(), ref, f"K={K} nsplit={nsplit}")
    # the context-split form writes its partial rows through the same mapping
    o, lse = uq_cuda.uq_decode_partial(q, *args)
    merged = uq_cuda.uq_merge(o.unsqueeze(0), lse.unsqueeze(0))
    check_close(merged.float().cpu().numpy(), ref, f"K={K} partial")


@pytest.mark.parametrize("PAGE,D,fmt", [(16, 128, 0), (256, 128, 0), (512, 128, 0), (256, 64, 0), (1024, 256, 0), (256, 128, 1), (48, 128, 0),
                                         (96, 128, 0), (80, 64, 0), (192, 256, 0), (48, 128, 1), (144, 128, 0), (24, 128, 0), (40, 64, 0)])
def test_page_sizes_from_16_to_1024_tokens(PAGE, D, fmt):
    """Pages smaller than the 128-key tile are copied whole, larger ones in 128-token parts, and a page size that neither
    divides 128 nor is a multiple of it (48, 80, 96, 144, 192 ...) in parts of gcd(PAGE, 128) tokens, three to eight copies per
    stream and tile; only a page size that is not a multiple of 16 runs on the CUDA-core kernel.  Ragged lengths that end
    inside a page and inside a part of a page."""
    rng = np.random.default_rng(PAGE + D)
    B, K, HQ, HKV = 3, 4, 8, 2
    sl = np.array([2 * PAGE + 77, 130, 3 * PAGE], np.int32)
    npg = -(-int(sl.max()) // PAGE)
    pages = B * npg
    kc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
    vc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
    if fmt == 0:
        ks = rng.integers(125, 130, (pages, HKV, PAGE, D // 32)).astype(np.uint8)
        vs = rng.integers(125, 130, (pages, HKV, PAGE, D // 32)).astype(np.uint8)
    else:
        ks = rng.integers(0x30, 0x40, (pages, HKV, PAGE, D // 16)).astype(np.uint8)
        vs = rng.integers(0x30, 0x40, (pages, HKV, PAGE, D // 16)).astype(np.uint8)
    bt = rng.permutation(pages).astype(np.int32).reshape(B, npg)
    qb = O.bf16_bits(0.3 * rng.standard_normal((B, K, HQ, D)).astype(np.float32))
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl) if fmt == 0 else O.reference_nvfp4(qb, kc, ks, vc, vs, bt, sl, 0.5, 0.5)
    q = dev(qb.view(np.int16), torch.bfloat16)
    kw = dict(fmt=1, k_ts=0.5, v_ts=0.5) if fmt else {}
    for nsplit in (None, 3):
        out = uq_cuda.uq_decode_cuda(q, dev(kc), dev(ks), dev(vc), dev(vs), dev(bt), dev(sl), nsplit=nsplit, **kw)
        assert uq_cuda.last_status() == (0, 0, 0, 0)
        assert uq_cuda.last_path() == (2 if PAGE % 16 == 0 else 1)
        mx = np.abs(ref).max()      # random codes and scales give outputs of order ten: the rule is applied to outputs normalised to O(1)
        check_close(out.float().cpu().numpy() / mx, ref / mx, f"PAGE={PAGE} D={D} fmt={fmt} nsplit={nsplit}")


@pytest.mark.parametrize("B,HKV,G,K", [(700, 8, 2, 2), (1000, 4, 8, 1), (300, 8, 8, 8)])
def test_many_short_sequences_put_more_segments_on_a_cta_than_its_list_holds(B, HKV, G, K):
    """Hundreds of sequences of one or two tiles (some empty): a CTA's share of the work list then spans more items than the 32
    candidates listed at set-up, so every role goes on with the walker from where the list ends; with one partial slot per item
    (nsplit 1) the items are dealt out by index, the list's other form."""
    rng = np.random.default_rng(B + HKV)
    D, PAGE = 128, 64
    HQ = HKV * G
    sl = rng.integers(1, 4 * PAGE, B).astype(np.int32)
    sl[rng.random(B) < 0.05] = 0
    sl[rng.random(B) < 0.05] = K
    npg = -(-int(sl.max()) // PAGE)
    pages = B * npg
    kc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
    vc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
    ks = rng.integers(125, 130, (pages, HKV, PAGE, D // 32)).astype(np.uint8)
    vs = rng.integers(125, 130, (pages, HKV, PAGE, D // 32)).astype(np.uint8)
    bt = rng.permutation(pages).astype(np.int32).reshape(B, npg)
    qb = O.bf16_bits(0.3 * rng.standard_normal((B, K, HQ, D)).astype(np.float32))
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl)
    q = dev(qb.view(np.int16), torch.bfloat16)
    mx = np.abs(ref).max()
    for nsplit in (None, 1, 2):
        out = uq_cuda.uq_decode_cuda(q, dev(kc), dev(ks), dev(vc), dev(vs), dev(bt), dev(sl), nsplit=nsplit)
        assert uq_cuda.last_status() == (0, 0, 0, 0) and uq_cuda.last_path() == 2
        check_close(out.float().cpu().numpy() / mx, ref / mx, f"B={B} HKV={HKV} nsplit={nsplit}")


def test_late_outliers_take_the_second_pass():
    """Keys whose scores (and V scales) dwarf those of a segment's first tile arrive late in every sequence: the quick path
    marks the segment and the careful pass redoes it; outputs follow the oracle on the same bytes."""
    c = [x for x in CASES if x.name == "ref_cuda_main_K8"][0]
    ks, vs = c.ks.copy(), c.vs.copy()
    for b in range(c.B):
        npg = -(-int(c.sl[b]) // c.PAGE)
        first, late = c.bt[b, : max(1, 128 // c.PAGE)], c.bt[b, npg // 2]
        ks[first] = (ks[first].astype(np.int32) - 10).clip(0, 255).astype(np.uint8)
        ks[late] = (ks[late].astype(np.int32) + 3).clip(0, 255).astype(np.uint8)
        vs[late] = (vs[late].astype(np.int32) + 5).clip(0, 255).astype(np.uint8)
    ref = O.reference(c.q, c.kc, ks, c.vc, vs, c.bt, c.sl, c.sm_scale)
    q = dev(c.q.view(np.int16), torch.bfloat16)
    for nsplit in (1, 4):
        out = uq_cuda.uq_decode_cuda(q, dev(c.kc), dev(ks), dev(c.vc), dev(vs), dev(c.bt), dev(c.sl), nsplit=nsplit)
        assert uq_cuda.last_status() == (0, 0, 0, 0)
        mx = np.abs(ref).max()
        check_close(out.float().cpu().numpy() / mx, ref / mx, f"late outliers nsplit={nsplit}")


def test_repeated_calls_are_bitwise_identical():
    """No result depends on which warp or CTA got somewhere first: the same call gives the same bits."""
    c = [x for x in CASES if x.name == "ref_cuda_main_K8"][0]
    q = dev(c.q.view(np.int16), torch.bfloat16)
    args = (dev(c.kc), dev(c.ks), dev(c.vc), dev(c.vs), dev(c.bt), dev(c.sl))
    outs = [uq_cuda.uq_decode_cuda(q, *args, nsplit=4).clone() for _ in range(6)]
    assert all(torch.equal(outs[0], o) for o in outs[1:])


def test_unserved_shapes_answer_invalid_value_before_any_work():
    c = [x for x in CASES if x.name == "ref_cuda_main_K1"][0]
    q = dev(c.q.view(np.int16), torch.bfloat16)
    args = (dev(c.kc), dev(c.ks), dev(c.vc), dev(c.vs), dev(c.bt), dev(c.sl))
    with pytest.raises(RuntimeError, match="InvalidValue"):
        uq_cuda.uq_decode_cuda(q, *args, fmt=2)
    with pytest.raises(RuntimeError, match="scale"):   # an NVFP4 call needs D/16 scale bytes per row
        uq_cuda.uq_decode_cuda(q, *args, fmt=1)
    with pytest.raises(RuntimeError, match="InvalidValue"):
        uq_cuda.uq_decode_cuda(q, *args, nsplit=129)
    with pytest.raises(RuntimeError, match="InvalidValue"):
        uq_cuda.uq_decode_cuda(q, *args, nsplit=0)
    with pytest.raises(RuntimeError, match="bf16"):
        uq_cuda.uq_decode_cuda(q.float(), *args)
    # the tuning hints of the reference's kernels are accepted and ignored
    out = uq_cuda.uq_decode_cuda(q, *args, variant=4, mb=2, nwarps=8, stages=4)
    check_close(out.float().cpu().numpy(), c.ref, "hints")


@pytest.mark.parametrize("R", [2, 4, 8])
def test_context_split_partials_merge_to_the_unsplit_answer(R):
    c = [x for x in CASES if x.name == "gen_d256_K8"][0]
    q = dev(c.q.view(np.int16), torch.bfloat16)
    per = -(-c.max_pages // R)
    os_, ls_ = [], []
    for r in range(R):
        lo, hi = min(r * per, c.max_pages), min((r + 1) * per, c.max_pages)
        bt = np.zeros((c.B, max(per, 1)), np.int32)
        bt[:, : hi - lo] = c.bt[:, lo:hi]
        off = np.full(c.B, lo * c.PAGE, np.int32)
        o, l = uq_cuda.uq_decode_partial(q, dev(c.kc), dev(c.ks), dev(c.vc), dev(c.vs), dev(bt), dev(c.sl), dev(off))
        # each shard's partial against the oracle's partial on the same shard
        nloc = np.clip(c.sl - lo * c.PAGE, 0, (hi - lo) * c.PAGE).astype(np.int32)
        ro, rl = O.reference(c.q, c.kc, c.ks, c.vc, c.vs, bt, c.sl, pos_offset=off, n_local=nloc, return_lse=True)
        check_close(o.cpu().numpy(), ro, f"shard {r} o")
        lse = l.cpu().numpy() * np.log(2.0)
        fin = np.isfinite(rl)
        assert np.array_equal(np.isfinite(lse), fin)
        assert np.abs(lse[fin] - rl[fin]).max(initial=0) <= 2e-3
        os_.append(o)
        ls_.append(l)
    out = uq_cuda.uq_merge(torch.stack(os_), torch.stack(ls_))
    check_close(out.float().cpu().numpy(), c.ref, f"merge R={R}")
    # the packed form (what one all-gather of per-rank buffers gives): same shards, same bits
    B, K, HQ, D = q.shape
    n = B * K * HQ * (D + 1)
    packed = torch.empty(R, n, dtype=torch.float32, device="cuda")
    for r in range(R):
        lo, hi = min(r * per, c.max_pages), min((r + 1) * per, c.max_pages)
        bt = np.zeros((c.B, max(per, 1)), np.int32)
        bt[:, : hi - lo] = c.bt[:, lo:hi]
        off = np.full(c.B, lo * c.PAGE, np.int32)
        uq_cuda.uq_decode_partial(q, dev(c.kc), dev(c.ks), dev(c.vc), dev(c.vs), dev(bt), dev(c.sl), dev(off), into=packed[r])
    out2 = uq_cuda.uq_merge_packed(packed, B * K * HQ, D, torch.empty_like(q))
    assert torch.equal(out2, out)


def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_unaffected(monkeypatch):
    """The give-up path of the tcgen05 kernel on a healthy GPU: with UQ_B200_CFG=expire=30 the softmax role never announces a
    segment's query tile (an arrival that nothing makes), so the issuing thread's wait for it - barrier id 30, bounded at one
    second like every wait of the kernel - runs out.  The kernel must return (every role drains to the common exit, the copy
    warps wait for their copies in flight, TMEM goes back), the status record must name a wait that ran out (code 1; the
    issuing thread's, or the softmax role's own wait for scores that were never computed, ids 62-64, whichever CTA reports
    first), and the next ordinary calls on the device must be right."""
    c = [x for x in CASES if x.name == "gen_cfg0_K4"][0]
    q = dev(c.q.view(np.int16), torch.bfloat16)
    args = (dev(c.kc), dev(c.ks), dev(c.vc), dev(c.vs), dev(c.bt), dev(c.sl))
    monkeypatch.setenv("UQ_B200_CFG", "path=tc,expire=30")
    bad = uq_cuda.uq_decode_cuda(q, *args)     # not an answer: the combine writes NaN rows while the status code is set
    assert torch.isnan(bad.float()).all()
    st = uq_cuda.last_status()
    assert st[0] == 1 and st[2] in (30, 62, 63, 64), st
    monkeypatch.delenv("UQ_B200_CFG")
    for _ in range(2):
        out = uq_cuda.uq_decode_cuda(q, *args)
        assert uq_cuda.last_status() == (0, 0, 0, 0) and uq_cuda.last_path() == 2
        check_close(out.float().cpu().numpy(), c.ref, "call after a wait that ran out")
