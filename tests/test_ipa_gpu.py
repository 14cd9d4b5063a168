"""Invariant point attention against the fp32 oracle: the golden fixture made from the reference's own
function, the reference test's shape (tests/test_ipa.py:141-157) with its tolerance
(`assert_close(..., atol=1e-2, rtol=1e-2)`, test_ipa.py:197), and AlphaFold-sized residues counts."""
from pathlib import Path

import pytest
import torch

import flashlight_b200
from flashlight_b200 import attention_variants as av
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def inputs(B, H, N, C, Pqk, Pv, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, device="cuda").to(torch.bfloat16)
    return (r(B, H, N, C), r(B, H, N, C), r(B, H, N, C), r(B, H, N, Pqk, 4), r(B, H, N, Pqk, 4), r(B, H, N, Pv, 4),
            r(B, H, N, N))


def check(out, ref):
    """The reference test's own tolerance (test_ipa.py:197)."""
    flashlight_b200.check_status()
    for o, r in zip(out, ref):
        assert o.dtype == torch.bfloat16 and o.shape == r.shape
        torch.testing.assert_close(o.float(), r.float(), atol=1e-2, rtol=1e-2)


def test_golden_fixture_of_the_reference_function():
    c = torch.load(GOLDEN / "ipa.pt", weights_only=True)
    t = lambda n: c[n].cuda()
    out = av.invariant_point_attention(t("q"), t("k"), t("v"), t("q_points"), t("k_points"), t("v_points"),
                                       t("pair_bias"), None, None, c_hidden=c["c_hidden"],
                                       no_qk_points=c["no_qk_points"])
    check(out, (c["out"].cuda(), c["out_points"].cuda()))


@pytest.mark.parametrize("B,H,N,C,Pqk,Pv", [(2, 8, 64, 16, 4, 8),      # tests/test_ipa.py:141-146
                                            (1, 12, 384, 16, 4, 8),    # a structure module's sizes
                                            (2, 4, 200, 32, 8, 12),    # operands of 98 and 80 columns
                                            (1, 2, 1, 16, 4, 8)])      # one residue
def test_against_the_oracle(B, H, N, C, Pqk, Pv):
    args = inputs(B, H, N, C, Pqk, Pv, 11)
    out = av.invariant_point_attention(*args, None, None, c_hidden=C, no_qk_points=Pqk)
    assert out[0].shape == (B, H, N, C) and out[1].shape == (B, N, H, Pv, 4)
    check(out, ao.invariant_point_attention(*args, c_hidden=C, no_qk_points=Pqk))


def test_distance_term_survives_an_offset_of_the_points():
    """Points away from the origin: |q_p - k_p|^2 is a small difference of large squares (here about 300
    against a spread of 4), which the split of the key-side products into two bf16 terms has to carry."""
    B, H, N, C, Pqk, Pv = 1, 2, 128, 16, 4, 8
    qs, ks, vs, qp, kp, vp, pb = inputs(B, H, N, C, Pqk, Pv, 12)
    qp, kp = (qp.float() * 0.5 + 4.0).to(torch.bfloat16), (kp.float() * 0.5 + 4.0).to(torch.bfloat16)
    out = av.invariant_point_attention(qs, ks, vs, qp, kp, vp, pb, None, None, c_hidden=C, no_qk_points=Pqk)
    check(out, ao.invariant_point_attention(qs, ks, vs, qp, kp, vp, pb, c_hidden=C, no_qk_points=Pqk))


def test_rejects_other_dtypes_and_shapes():
    args = list(inputs(1, 2, 32, 16, 4, 8, 13))
    with pytest.raises(NotImplementedError):
        av.invariant_point_attention(*[a.float() for a in args], None, None, c_hidden=16, no_qk_points=4)
    with pytest.raises(ValueError):
        av.invariant_point_attention(*args, None, None, c_hidden=16, no_qk_points=8)


def test_three_dimensional_points_and_other_key_count():
    """Points with three coordinates (the reference's test stores four), and more keys than queries."""
    g = torch.Generator(device="cuda").manual_seed(14)
    r = lambda *s: torch.randn(*s, generator=g, device="cuda").to(torch.bfloat16)
    B, H, N, Nk, C, Pqk, Pv = 2, 4, 100, 260, 16, 4, 8
    args = (r(B, H, N, C), r(B, H, Nk, C), r(B, H, Nk, C), r(B, H, N, Pqk, 3), r(B, H, Nk, Pqk, 3), r(B, H, Nk, Pv, 3),
            r(B, H, N, Nk))
    out = av.invariant_point_attention(*args, None, None, c_hidden=C, no_qk_points=Pqk)
    assert out[0].shape == (B, H, N, C) and out[1].shape == (B, N, H, Pv, 3)
    check(out, ao.invariant_point_attention(*args, c_hidden=C, no_qk_points=Pqk))
