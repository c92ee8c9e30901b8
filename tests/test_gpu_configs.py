"""Parity at the shape families of the benchmark's other configurations, which the frozen vectors do not cover: ragged
serving batches at the Mistral-7B-shaped and the large-batch head counts (also divided by KV head, as the ranks of a
multi-GPU run hold them), a multi-layer append-then-verify step with bf16 tokens, a long head_dim-256 sequence split into
context shards with a ragged last shard, and scale / query value ranges that stress the kernels' fp16 and e4m3 operand
tiles.  Everything is compared with the CPU oracle on the bytes the kernel consumed.  Needs a B200."""
import numpy as np
import pytest
import torch

from all_quant_b200 import uq_cuda
from oracle import uq_oracle as O
from tests.cases import check_close

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


def make_cache(rng, lens, HKV, D, PAGE, shuffle=True):
    """fp32 K/V of the given lengths -> UltraQuant bytes in pages (physical pages permuted), page table, raw values."""
    B = len(lens)
    npgs = [-(-int(n) // PAGE) for n in lens]
    width, pages = max(1, max(npgs)), max(1, sum(npgs))
    chan = np.exp(0.5 * rng.standard_normal((1, HKV, 1, D))).astype(np.float32)
    k = rng.standard_normal((pages, HKV, PAGE, D)).astype(np.float32) * chan
    v = rng.standard_normal((pages, HKV, PAGE, D)).astype(np.float32)
    kc, ks = O.quantize_fp4(k)
    vc, vs = O.quantize_fp4(v)
    perm = rng.permutation(pages).astype(np.int32) if shuffle else np.arange(pages, dtype=np.int32)
    bt = np.zeros((B, width), np.int32)
    first = 0
    for b, n in enumerate(npgs):
        bt[b, :n] = perm[first:first + n]
        first += n
    return kc, ks, vc, vs, bt


RAGGED = [1537, 5, 4096, 777, 129, 2050, 64, 3001, 1000]   # not multiples of the 128-key tile or the page; one shorter than K; one a whole page


@pytest.mark.parametrize("HQ,HKV", [(64, 8), (32, 8)], ids=["large-batch heads", "mistral heads"])
@pytest.mark.parametrize("K", [8, 3])
def test_ragged_batch_against_the_oracle(HQ, HKV, K):
    rng = np.random.default_rng(HQ + K)
    D, PAGE = 128, 64
    sl = np.array(RAGGED, np.int32)
    kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
    qb = O.bf16_bits(rng.standard_normal((len(sl), K, HQ, D)).astype(np.float32))
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl)
    q = dev(qb.view(np.int16), torch.bfloat16)
    out = uq_cuda.uq_decode_cuda(q, dev(kc), dev(ks), dev(vc), dev(vs), dev(bt), dev(sl))
    assert uq_cuda.last_path() == 2 and uq_cuda.last_status() == (0, 0, 0, 0)
    got = out.float().cpu().numpy()
    check_close(got, ref, "ragged batch")
    for j in range(K):   # sequence 1 has 5 tokens: drafts that see nothing are exact zeros
        if 5 - K + j + 1 <= 0:
            assert not got[1, j].any()


@pytest.mark.parametrize("world", [2, 8])
def test_kv_head_partition_gives_the_rows_of_the_whole_call(world):
    """What each rank of the head-partitioned configurations computes (its own kv heads and their query heads, the same page
    table and lengths) put side by side is the whole call's answer; at 8 ranks a rank holds one kv head."""
    rng = np.random.default_rng(world)
    HQ, HKV, D, PAGE, K = 64, 8, 128, 64, 8
    sl = np.array(RAGGED[:6], np.int32)
    kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
    qb = O.bf16_bits(rng.standard_normal((len(sl), K, HQ, D)).astype(np.float32))
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl)
    q = dev(qb.view(np.int16), torch.bfloat16)
    caches = tuple(dev(a) for a in (kc, ks, vc, vs))
    parts = []
    for r in range(world):
        qs, *cs = uq_cuda.head_shard(q, *caches, r, world)
        parts.append(uq_cuda.uq_decode_cuda(qs, *cs, dev(bt), dev(sl)))
        assert uq_cuda.last_status() == (0, 0, 0, 0)
    check_close(torch.cat(parts, dim=2).float().cpu().numpy(), ref, f"{world} head shards")


def test_layers_of_append_then_verify_with_bf16_tokens():
    """The decode step of the 32-layer configuration, three layers of it: the K newest tokens of every sequence arrive as
    bf16, are quantized into their slots (bytes equal to the reference encoder applied to the same values as fp32), and the
    verify call then reads the cache that holds them."""
    rng = np.random.default_rng(11)
    HQ, HKV, D, PAGE, K, L = 32, 8, 128, 64, 8, 3
    sl = np.array([1300, 2049, 515, 8, 3071], np.int32)
    B = len(sl)
    for layer in range(L):
        kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
        d_kc, d_ks, d_vc, d_vs = (dev(a) for a in (kc, ks, vc, vs))
        # the K newest positions of every sequence, through the page table
        pos = np.concatenate([np.arange(max(0, n - K), n) for n in sl])
        seq = np.concatenate([np.full(min(K, n), b) for b, n in enumerate(sl)])
        slots = bt[seq, pos // PAGE].astype(np.int64) * PAGE + pos % PAGE
        chan = np.exp(0.5 * rng.standard_normal((1, HKV, D))).astype(np.float32)
        new_k = torch.from_numpy(rng.standard_normal((len(pos), HKV, D)).astype(np.float32) * chan).bfloat16()
        new_v = torch.from_numpy(rng.standard_normal((len(pos), HKV, D)).astype(np.float32)).bfloat16()
        uq_cuda.append_kv(d_kc, d_ks, d_vc, d_vs, new_k.cuda(), new_v.cuda(), torch.from_numpy(slots).cuda())
        # the oracle's append on the same values widened to fp32: every byte of the four arrays must agree
        O.append_kv(kc, ks, vc, vs, new_k.float().numpy(), new_v.float().numpy(), slots)
        for name, a, d in (("kc", kc, d_kc), ("ks", ks, d_ks), ("vc", vc, d_vc), ("vs", vs, d_vs)):
            assert np.array_equal(a, d.cpu().numpy()), f"layer {layer}: {name} differs from the reference encoder"
        qb = O.bf16_bits(rng.standard_normal((B, K, HQ, D)).astype(np.float32))
        ref = O.reference(qb, kc, ks, vc, vs, bt, sl)
        out = uq_cuda.uq_decode_cuda(dev(qb.view(np.int16), torch.bfloat16), d_kc, d_ks, d_vc, d_vs, dev(bt), dev(sl))
        assert uq_cuda.last_status() == (0, 0, 0, 0)
        check_close(out.float().cpu().numpy(), ref, f"layer {layer}")


@pytest.mark.parametrize("R", [2, 4, 8])
def test_long_head_dim_256_sequence_in_context_shards(R):
    """One sequence of a few thousand tokens at head_dim 256 (Hq 32 / Hkv 4), its pages divided over R shards by
    context_shard (the last shard ragged, at 8 shards the last but one too): the packed partials of the shards merge to the
    oracle's answer for the whole sequence."""
    rng = np.random.default_rng(R)
    HQ, HKV, D, PAGE, K = 32, 4, 256, 64, 8
    sl = np.array([5000], np.int32)   # 79 pages: 8 shards of 10 pages hold 640 tokens each, the last one 520
    kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
    qb = O.bf16_bits(rng.standard_normal((1, K, HQ, D)).astype(np.float32))
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl)
    q = dev(qb.view(np.int16), torch.bfloat16)
    caches = tuple(dev(a) for a in (kc, ks, vc, vs))
    n = K * HQ * (D + 1)
    packed = torch.empty(R, n, dtype=torch.float32, device="cuda")
    for r in range(R):
        bt_r, off_r = uq_cuda.context_shard(dev(bt), r, R, PAGE)
        uq_cuda.uq_decode_partial(q, *caches, bt_r, dev(sl), off_r, into=packed[r])
        assert uq_cuda.last_status() == (0, 0, 0, 0)
    out = uq_cuda.uq_merge_packed(packed, K * HQ, D, torch.empty_like(q))
    check_close(out.float().cpu().numpy(), ref, f"{R} context shards")


@pytest.mark.parametrize("D", [128, 256, 64])
def test_scale_groups_of_one_key_thirty_binades_apart(D):
    """Inside one key the 32-channel groups of K and of V carry scales up to 2^30 apart (the frozen vectors and the uniform
    shift of the scale-extremes test never do that).  The kernels hold a key's fp16 operand values relative to the key's
    largest scale, so a group more than 24 binades below it reads as zero there; what it would have contributed is below
    2^-24 of the key's largest term, far inside the tolerance, which is applied to outputs normalised to O(1)."""
    rng = np.random.default_rng(D)
    HQ, HKV, PAGE, K = 16, 2, 64, 4
    sl = np.array([700, 333], np.int32)
    kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
    G = D // 32
    spread = np.linspace(-15, 15, G).round().astype(np.int32)             # group g of every key: 2^spread[g]
    ks = (ks.astype(np.int32) + spread).clip(1, 254).astype(np.uint8)
    vs = (vs.astype(np.int32) + spread[::-1]).clip(1, 254).astype(np.uint8)
    # and some keys the other way round, so that neighbouring keys of a tile disagree about which group is the large one
    flip = rng.random(ks.shape[:3]) < 0.3
    ks[flip] = ks[flip][:, ::-1]
    vs[flip] = vs[flip][:, ::-1]
    qb = O.bf16_bits(rng.standard_normal((2, K, HQ, D)).astype(np.float32))
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl)
    out = uq_cuda.uq_decode_cuda(dev(qb.view(np.int16), torch.bfloat16), dev(kc), dev(ks), dev(vc), dev(vs), dev(bt), dev(sl))
    assert uq_cuda.last_status() == (0, 0, 0, 0)
    mx = np.abs(ref).max()
    check_close(out.float().cpu().numpy() / mx, ref / mx, f"scale spread D={D}")


@pytest.mark.parametrize("D", [128, 256])
def test_query_block_with_one_entry_far_above_the_rest(D):
    """A query whose 32-channel blocks each hold one entry 2^8 above the others: at head_dim 128 the query tile is two e4m3
    tiles with one power-of-two scale per row and block (about nine significant bits relative to the block's largest entry),
    so the small entries keep only their leading bits; the answer still follows the oracle within the tolerance."""
    rng = np.random.default_rng(D + 1)
    HQ, HKV, PAGE, K = 16, 2, 64, 4
    sl = np.array([1500, 260], np.int32)
    kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
    qf = rng.standard_normal((2, K, HQ, D)).astype(np.float32) * 0.25
    big = rng.integers(0, 32, (2, K, HQ, D // 32))
    for blk in range(D // 32):
        idx = blk * 32 + big[..., blk]
        np.put_along_axis(qf, idx[..., None], np.take_along_axis(qf, idx[..., None], -1) * 256.0, -1)
    qb = O.bf16_bits(qf)
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl, sm_scale=D ** -0.5 / 16)   # (scores stay in a range where the softmax is not one-hot)
    out = uq_cuda.uq_decode_cuda(dev(qb.view(np.int16), torch.bfloat16), dev(kc), dev(ks), dev(vc), dev(vs), dev(bt), dev(sl), sm_scale=D ** -0.5 / 16)
    assert uq_cuda.last_status() == (0, 0, 0, 0)
    check_close(out.float().cpu().numpy(), ref, f"query outliers D={D}")


@pytest.mark.parametrize("R", [2, 4, 8])
def test_context_split_over_exchange_buffers_in_one_process(R):
    """The two launches of the peer-memory context split - the shard's attention whose combine stores the packed partial
    into every rank's exchange buffer and raises its flag, and the merge that waits for all flags - with the R ranks'
    buffers living in one process on one GPU (the launches run in stream order, so no kernel waits for a later one).  Every
    rank's merged output equals the oracle's answer for the whole sequence, on two calls in a row (the second on the other
    parity of the double-buffered slots)."""
    rng = np.random.default_rng(40 + R)
    HQ, HKV, D, PAGE, K = 32, 4, 256, 64, 8
    sl = np.array([3000], np.int32)
    kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
    caches = tuple(dev(a) for a in (kc, ks, vc, vs))
    ranks = uq_cuda.ContextSplit.in_one_process(R, K * HQ, D)
    try:
        for call in range(2):
            qb = O.bf16_bits(rng.standard_normal((1, K, HQ, D)).astype(np.float32))
            ref = O.reference(qb, kc, ks, vc, vs, bt, sl)
            q = dev(qb.view(np.int16), torch.bfloat16)
            for r, cs in enumerate(ranks):
                bt_r, off_r = uq_cuda.context_shard(dev(bt), r, R, PAGE)
                cs.push(q, *caches, bt_r, dev(sl), off_r, seq=call + 1)
            for cs in ranks:
                out = cs.merge(q, seq=call + 1)
                assert uq_cuda.last_status() == (0, 0, 0, 0)
                check_close(out.float().cpu().numpy(), ref, f"{R} ranks, call {call}, rank {cs.rank}")
    finally:
        torch.cuda.synchronize()
        ranks[0].close()


def test_a_rank_that_never_arrives_ends_the_merge_wait_with_a_status():
    """The merge's wait for the other ranks is bounded: with a limit of two milliseconds and a second rank that never stores
    anything (its flag is never set), the kernel returns, the status record names the wait (code 3), the missing rank and
    the sequence number, and the next ordinary call on the device is unaffected."""
    rng = np.random.default_rng(77)
    HQ, HKV, D, PAGE, K = 8, 2, 128, 64, 2
    sl = np.array([300], np.int32)
    kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
    caches = tuple(dev(a) for a in (kc, ks, vc, vs))
    qb = O.bf16_bits(rng.standard_normal((1, K, HQ, D)).astype(np.float32))
    q = dev(qb.view(np.int16), torch.bfloat16)
    ranks = uq_cuda.ContextSplit.in_one_process(2, K * HQ, D, wait_ns=2_000_000)
    try:
        bt_0, off_0 = uq_cuda.context_shard(dev(bt), 0, 2, PAGE)
        ranks[0].push(q, *caches, bt_0, dev(sl), off_0, seq=1)     # rank 1 never pushes
        ranks[0].merge(q, seq=1)
        code, _, who, seq = uq_cuda.last_status()
        assert (code, who, seq) == (3, 1, 1)
        out = uq_cuda.uq_decode_cuda(q, *caches, dev(bt), dev(sl))
        assert uq_cuda.last_status() == (0, 0, 0, 0)
        check_close(out.float().cpu().numpy(), O.reference(qb, kc, ks, vc, vs, bt, sl), "call after the timed-out wait")
    finally:
        torch.cuda.synchronize()
        ranks[0].close()


@pytest.mark.parametrize("HQ,HKV,K", [(2, 2, 1), (2, 2, 2), (4, 2, 1), (4, 2, 4), (8, 8, 3)])
def test_few_query_rows_run_on_the_tensor_core_kernel_and_both_kernels_agree(HQ, HKV, K, monkeypatch):
    """One to eight query rows per (sequence, kv head): measured on a B200 at the headline context the tcgen05 kernel is 3.7 to
    5 times faster than the CUDA-core kernel even for a single row, so the dispatch sends every served shape there
    (last_path() == 2); the CUDA-core kernel, forced, gives the same answer."""
    rng = np.random.default_rng(HQ * 10 + K)
    D, PAGE = 128, 64
    sl = np.array([1100, 3, 640], np.int32)
    kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
    qb = O.bf16_bits(rng.standard_normal((len(sl), K, HQ, D)).astype(np.float32))
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl)
    args = (dev(qb.view(np.int16), torch.bfloat16), dev(kc), dev(ks), dev(vc), dev(vs), dev(bt), dev(sl))
    out = uq_cuda.uq_decode_cuda(*args)
    assert uq_cuda.last_path() == 2
    check_close(out.float().cpu().numpy(), ref, "tcgen05, few rows")
    monkeypatch.setenv("UQ_B200_CFG", "path=fma")
    out = uq_cuda.uq_decode_cuda(*args)
    assert uq_cuda.last_path() == 1 and uq_cuda.last_status() == (0, 0, 0, 0)
    check_close(out.float().cpu().numpy(), ref, "CUDA cores, few rows")


@pytest.mark.parametrize("K,HQ,HKV,D,fmt", [(8, 8, 2, 128, 0), (4, 32, 4, 256, 0), (16, 8, 1, 64, 0), (5, 14, 2, 128, 0)])
def test_cuda_core_kernel_with_many_rows_and_unaligned_value_arrays(K, HQ, HKV, D, fmt, monkeypatch):
    """The CUDA-core kernel at 16 to 128 rows (passes of 32 rows, every tile staged once per pass), with the V codes and both
    scale arrays at odd byte offsets (only q and the K codes have an alignment contract), on a page size that is not a power
    of two."""
    rng = np.random.default_rng(K * 7 + D)
    PAGE = 48
    sl = np.array([500, 47, 1000], np.int32)
    kc, ks, vc, vs, bt = make_cache(rng, sl, HKV, D, PAGE)
    qb = O.bf16_bits(rng.standard_normal((len(sl), K, HQ, D)).astype(np.float32))
    ref = O.reference(qb, kc, ks, vc, vs, bt, sl)

    def odd(a):   # the same bytes starting one byte into a larger allocation
        buf = torch.empty(a.size + 1, dtype=torch.uint8, device="cuda")
        view = buf[1:].view(a.shape)
        view.copy_(dev(a))
        return view
    out = uq_cuda.uq_decode_cuda(dev(qb.view(np.int16), torch.bfloat16), dev(kc), odd(ks), odd(vc), odd(vs), dev(bt), dev(sl))
    assert uq_cuda.last_path() == 1 and uq_cuda.last_status() == (0, 0, 0, 0)
    check_close(out.float().cpu().numpy(), ref, "CUDA cores, odd offsets")
