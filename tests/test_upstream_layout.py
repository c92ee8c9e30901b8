"""The byte permute to and from the upstream engines' slot layout, with the two representation details of the upstream
encoder (minus-zero codes, the zero-group scale byte): the oracle's numpy restatement against the fixture written with the
reference's converter formulas, its canon_negzero and the upstream encoder it vendors (tests/golden/make_golden.py
gen_upstream), then the CUDA kernels against the same fixture, byte for byte."""
import numpy as np
import pytest
import torch

from oracle import uq_oracle as O
from tests.cases import load

Z = load("gen_upstream")
DS = (64, 128, 256)


def arrays(D):
    return tuple(Z[f"d{D}_{n}"] for n in ("kc", "ks", "vc", "vs"))


@pytest.mark.parametrize("D", DS)
def test_oracle_layout_matches_the_references_converter(D):
    kc, ks, vc, vs = arrays(D)
    assert np.array_equal(O.to_upstream(kc, ks, vc, vs), Z[f"d{D}_aos"])
    assert np.array_equal(O.to_upstream(kc, ks, vc, vs, slot_bytes=D + D // 16 + 8), Z[f"d{D}_aos_pad8"])
    for a, b in zip(O.from_upstream(Z[f"d{D}_aos_pad8"], D), (kc, ks, vc, vs)):
        assert np.array_equal(a, b)
    assert np.array_equal(O.canon_negzero(kc), Z[f"d{D}_canon_kc"]) and np.array_equal(O.canon_negzero(vc), Z[f"d{D}_canon_vc"])


@pytest.mark.parametrize("D", (128, 256))
def test_oracle_sentinel_gives_the_upstream_encoders_scale_bytes(D):
    """'paper'-rule bytes of the reference's quantiser + minus-zero canonicalisation + zero-group scale byte = the bytes of the
    upstream encoder on the same values (a fifth of the groups are all zero in the fixture)."""
    kc, ks, vc, vs = arrays(D)
    assert (Z[f"d{D}_up_ks"] == 0).any() and not np.array_equal(ks, Z[f"d{D}_up_ks"])
    assert np.array_equal(O.zero_sentinel(kc, ks), Z[f"d{D}_up_ks"]) and np.array_equal(O.zero_sentinel(vc, vs), Z[f"d{D}_up_vs"])


@pytest.mark.gpu
@pytest.mark.parametrize("D", DS)
def test_layout_kernels_match_the_fixture_byte_for_byte(D):
    from all_quant_b200 import uq_cuda
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    kc, ks, vc, vs = arrays(D)
    d = tuple(dev(a) for a in (kc, ks, vc, vs))
    assert np.array_equal(uq_cuda.to_upstream_layout(*d).cpu().numpy(), Z[f"d{D}_aos"])
    out = torch.full((kc.shape[0], kc.shape[2], kc.shape[1], D + D // 16 + 8), 0xAB, dtype=torch.uint8, device="cuda")
    assert np.array_equal(uq_cuda.to_upstream_layout(*d, slot_bytes=D + D // 16 + 8, out=out).cpu().numpy(), Z[f"d{D}_aos_pad8"])
    for a, b in zip(uq_cuda.from_upstream_layout(dev(Z[f"d{D}_aos_pad8"]), D), (kc, ks, vc, vs)):
        assert np.array_equal(a.cpu().numpy(), b)
    # both details applied: the oracle's answer, which for head_dim 128 / 256 is the upstream encoder's bytes
    got = uq_cuda.to_upstream_layout(*d, canon_negzero=True, zero_sentinel=True).cpu().numpy()
    assert np.array_equal(got, O.to_upstream(kc, ks, vc, vs, canon=True, sentinel=True))
    if D != 64:
        up = O.to_upstream(Z[f"d{D}_canon_kc"], Z[f"d{D}_up_ks"], Z[f"d{D}_canon_vc"], Z[f"d{D}_up_vs"])
        assert np.array_equal(got, up)
    # a cache that came in from upstream decodes as it is: round trip through both kernels
    back = uq_cuda.from_upstream_layout(dev(got), D)
    assert np.array_equal(back[0].cpu().numpy(), Z[f"d{D}_canon_kc"])


@pytest.mark.gpu
@pytest.mark.parametrize("D,HKV,PAGE,pages,pad", [(128, 8, 64, 5, 0), (128, 3, 16, 7, 8), (128, 5, 48, 3, 1), (128, 2, 16, 9, 2),
                                                    (64, 1, 16, 5, 0), (64, 7, 32, 3, 3), (256, 4, 16, 3, 0), (256, 3, 80, 2, 5),
                                                    (128, 1, 16, 1, 0), (128, 2, 64, 1, 700)])
def test_layout_kernels_on_sizes_that_do_not_line_up(D, HKV, PAGE, pages, pad):
    """Slot counts that are not a multiple of a block's 64, slot sizes whose pieces are only 2- or 1-byte aligned inside the
    slot, head counts and page sizes that are not powers of two, a slot too large for the staged kernel: against the numpy
    restatement, both directions, with a fifth of the groups all zero and minus-zero codes in the data."""
    from all_quant_b200 import uq_cuda
    rng = np.random.default_rng(D + HKV + PAGE + pad)
    G = D // 32
    kc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
    vc = rng.integers(0, 256, (pages, HKV, PAGE, D // 2), dtype=np.uint8)
    for c in (kc, vc):
        z = rng.random((pages, HKV, PAGE, G)) < 0.2
        c.reshape(pages, HKV, PAGE, G, 16)[z] = 0
        c.reshape(pages, HKV, PAGE, G, 16)[rng.random((pages, HKV, PAGE, G)) < 0.1] = 0x88
    ks = rng.integers(1, 255, (pages, HKV, PAGE, G), dtype=np.uint8)
    vs = rng.integers(1, 255, (pages, HKV, PAGE, G), dtype=np.uint8)
    slot = D + 2 * G + pad
    dev = lambda a: torch.from_numpy(a).cuda()
    d = tuple(dev(a) for a in (kc, ks, vc, vs))
    for canon, sentinel in ((False, False), (True, True)):
        out = torch.full((pages, PAGE, HKV, slot), 0xCD, dtype=torch.uint8, device="cuda")
        got = uq_cuda.to_upstream_layout(*d, slot_bytes=slot, canon_negzero=canon, zero_sentinel=sentinel, out=out).cpu().numpy()
        assert np.array_equal(got, O.to_upstream(kc, ks, vc, vs, slot_bytes=slot, canon=canon, sentinel=sentinel))
    plain = O.to_upstream(kc, ks, vc, vs, slot_bytes=slot)
    plain[..., D + 2 * G:] = 0x5A                       # whatever the allocator left in the padding is ignored on the way in
    for a, b in zip(uq_cuda.from_upstream_layout(dev(plain), D), (kc, ks, vc, vs)):
        assert np.array_equal(a.cpu().numpy(), b)
