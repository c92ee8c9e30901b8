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
