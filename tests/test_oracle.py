"""Pins the CPU oracle (oracle/uq_oracle.c) to the reference's frozen vectors and to fixtures produced
by the reference's own Python functions.  Runs without a GPU."""
import numpy as np
import pytest

from oracle import uq_oracle as O
from tests.cases import load, load_cases

CASES = load_cases()


@pytest.mark.parametrize("c", CASES, ids=repr)
def test_attention_matches_reference_vectors(c):
    out = O.reference(c.q, c.kc, c.ks, c.vc, c.vs, c.bt, c.sl, c.sm_scale)
    assert np.abs(out - c.ref).max() <= 2e-5, np.abs(out - c.ref).max()
    # rows with no visible key are exact zeros (uqmt/attn.py:418-419)
    for b in range(c.B):
        for j in range(c.K):
            if c.sl[b] - c.K + j + 1 <= 0:
                assert not out[b, j].any()


@pytest.mark.parametrize("name", ["wide", "bf16in", "fp16in", "g32"])
def test_encoder_bit_exact(name):
    z = load("gen_codec")
    p, s = O.quantize_fp4(z[f"{name}_x"])
    assert np.array_equal(s, z[f"{name}_scales"])
    assert np.array_equal(p, z[f"{name}_packed"])
    assert np.array_equal(O.dequantize_fp4(p, s).view(np.uint32), z[f"{name}_deq"].view(np.uint32))


def test_decoder_every_code_and_scale():
    z = load("gen_codec")
    d = O.dequantize_fp4(z["all_packed"], z["all_scales"])
    assert np.array_equal(d.view(np.uint32), z["all_deq"].view(np.uint32))


def test_encoder_reference_unit_cases():
    # exact grid round trip with scale bytes 127 / 130 (reference tests/test_attn.py:23-34)
    grid = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float32)
    x = np.concatenate([grid, -grid, grid, -grid]).reshape(1, 32)
    for mul, byte in ((1.0, 127), (8.0, 130)):
        p, s = O.quantize_fp4(x * mul)
        assert s.item() == byte
        assert np.array_equal(O.dequantize_fp4(p, s), x * mul)
    # all-zero group -> scale byte 25, codes 0; ties go to the smaller magnitude
    p, s = O.quantize_fp4(np.zeros((1, 32), np.float32))
    assert s.item() == 25 and not p.any()
    t = np.zeros((1, 32), np.float32)
    t[0, :4] = [0.75, 2.5, 5.0, 6.0]
    p, s = O.quantize_fp4(t)
    assert s.item() == 127 and p[0, 0] == (1 | (4 << 4)) and p[0, 1] == (6 | (7 << 4))
    # negative values that round to magnitude zero keep their sign bit; -0.0 does not
    t = np.zeros((1, 32), np.float32)
    t[0, :3] = [-1e-9, -0.0, 6.0]
    p, _ = O.quantize_fp4(t)
    assert p[0, 0] == 0x08 and (p[0, 1] & 0xF) == 7
    assert O.dequantize_fp4(p, np.array([[127]], np.uint8))[0, 0] == 0.0


def test_cache_bytes_of_cfg0_reproduced_from_raw():
    z = load("gen_cfg0")
    kc, ks = O.quantize_fp4(z["raw_k"])
    vc, vs = O.quantize_fp4(z["raw_v"])
    pg = z["raw_pages"]
    assert np.array_equal(kc, z["kc"][pg]) and np.array_equal(ks, z["ks"][pg])
    assert np.array_equal(vc, z["vc"][pg]) and np.array_equal(vs, z["vs"][pg])


def test_append_kv_matches_reference():
    z = load("gen_append")
    kc, ks, vc, vs = (z[n].copy() for n in ("kc0", "ks0", "vc0", "vs0"))
    O.append_kv(kc, ks, vc, vs, O.bf16_to_f32(z["key"]), O.bf16_to_f32(z["value"]), z["slots"])
    for got, name in ((kc, "kc1"), (ks, "ks1"), (vc, "vc1"), (vs, "vs1")):
        assert np.array_equal(got, z[name]), name


@pytest.mark.parametrize("R", [1, 2, 4, 8])
def test_context_split_partials_merge_to_unsplit(R):
    """Page-range shards with a position offset, merged by log-sum-exp, equal the unsplit answer."""
    c = [x for x in load_cases("gen_d256")][0]
    full = O.reference(c.q, c.kc, c.ks, c.vc, c.vs, c.bt, c.sl)
    npg = c.max_pages
    per = -(-npg // R)
    os_, ls_ = [], []
    for r in range(R):
        lo, hi = min(r * per, npg), min((r + 1) * per, npg)
        bt = np.zeros((c.B, max(per, 1)), np.int32)
        bt[:, : hi - lo] = c.bt[:, lo:hi]
        off = np.full(c.B, lo * c.PAGE, np.int32)
        nloc = np.clip(c.sl - lo * c.PAGE, 0, (hi - lo) * c.PAGE).astype(np.int32)
        o, lse = O.reference(c.q, c.kc, c.ks, c.vc, c.vs, bt, c.sl, pos_offset=off, n_local=nloc, return_lse=True)
        os_.append(o)
        ls_.append(lse)
    merged = O.merge(np.stack(os_), np.stack(ls_))
    assert np.abs(merged - full).max() <= 2e-6
    assert np.abs(full - c.ref).max() <= 2e-5
