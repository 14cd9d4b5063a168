"""The CPU oracle must reproduce the reference's own eager outputs (tests/golden/*.pt, made by
tests/golden/make_golden.py from the unmodified reference)."""
from pathlib import Path

import pytest
import torch

from oracle import attention_oracle as ao

GOLDEN = Path(__file__).resolve().parent / "golden"


def load(name):
    return torch.load(GOLDEN / f"{name}.pt", weights_only=True)


def close(a, b):
    torch.testing.assert_close(a, b, atol=2e-5, rtol=2e-5)


def test_vanilla():
    c = load("vanilla_nogqa")
    close(ao.vanilla(c["q"], c["k"], c["v"]), c["out"])
    c = load("vanilla_gqa")
    close(ao.vanilla(c["q"], c["k"], c["v"], enable_gqa=True), c["out"])


def test_causal():
    c = load("causal")
    close(ao.causal(c["q"], c["k"], c["v"]), c["out"])
    c = load("causal_gqa")
    out = ao.causal(c["q"], c["k"], c["v"], enable_gqa=True)
    assert out.dim() == 5  # the reference keeps (N, Hkv, G, L, Ev)
    close(out, c["out"])


def test_alibi():
    c = load("alibi")
    close(ao.alibi(c["q"], c["k"], c["v"], nheads=c["nheads"]), c["out"])
    c = load("alibi_gqa")
    close(ao.alibi(c["q"], c["k"], c["v"], nheads=c["nheads"], enable_gqa=True), c["out"])


def test_alibi_check_values():
    # H = 4 -> slope_0 = 0.25; bias row 0 = [0, 0.25, 0.5]
    s = ao.alibi_slopes(4, "cpu")
    assert abs(float(s[0]) - 0.25) < 1e-7 and abs(float(s[3]) - 2.0 ** -8) < 1e-9


def test_softcap():
    c = load("softcap")
    close(ao.softcap(c["q"], c["k"], c["v"], c["cap"]), c["out"])


def test_sliding():
    c = load("sliding")
    close(ao.sliding_window(c["q"], c["k"], c["v"], window_size=c["window"]), c["out"])


@pytest.mark.parametrize("name", ["document", "document_unsorted"])
def test_document(name):
    c = load(name)
    close(ao.document_mask(c["q"], c["k"], c["v"], c["document_id"]), c["out"])


def test_prefix():
    c = load("prefix")
    close(ao.prefix_lm(c["q"], c["k"], c["v"], prefix_lengths=c["prefix"]), c["out"])
    # a per-sequence tensor holding the same length must agree with the int form
    pl = torch.full((c["q"].size(0),), c["prefix"], dtype=torch.long)
    close(ao.prefix_lm(c["q"], c["k"], c["v"], prefix_lengths=pl), c["out"])


@pytest.mark.parametrize("name", ["diff", "diff_l08", "diff_d128"])
def test_diff(name):
    c = load(name)
    close(ao.diffattn(c["q"], c["k"], c["v"], lambda_full=c["lam"]), c["out"])


@pytest.mark.parametrize("name", ["evoformer", "evoformer_mask"])
def test_evoformer(name):
    c = load(name)
    close(ao.evoformer(c["q"], c["k"], c["v"], [c["bias1"], c["bias2"]]), c["out"])


def test_invariant_point_attention():
    """Both aggregates, read out of the unmodified reference function at a shape where its final sum
    broadcasts (tests/golden/make_golden.py says how)."""
    c = load("ipa")
    scalar, points = ao.invariant_point_attention(c["q"], c["k"], c["v"], c["q_points"], c["k_points"], c["v_points"],
                                                  c["pair_bias"], c_hidden=c["c_hidden"], no_qk_points=c["no_qk_points"])
    close(scalar, c["out"])
    close(points, c["out_points"])


def test_extensions_reduce_to_reference_when_off():
    """Extension flags default to the reference's behaviour; causal composition equals the
    causal oracle when the score modifier is the identity (cap -> infinity)."""
    c = load("causal")
    big = ao.softcap(c["q"], c["k"], c["v"], 1e9, is_causal=True)
    torch.testing.assert_close(big, c["out"], atol=1e-4, rtol=1e-4)
    c = load("prefix")
    zero = ao.prefix_lm(c["q"], c["k"], c["v"], prefix_lengths=0)
    torch.testing.assert_close(zero, ao.causal(c["q"], c["k"], c["v"]), atol=1e-5, rtol=1e-5)


def test_diff_rms_norm_definition():
    c = load("diff")
    base = ao.diffattn(c["q"], c["k"], c["v"], lambda_full=0.8, is_causal=True)
    normed = ao.diffattn(c["q"], c["k"], c["v"], lambda_full=0.8, is_causal=True, rms_norm=True, rms_eps=1e-5)
    ref = base * torch.rsqrt((base * base).mean(-1, keepdim=True) + 1e-5)
    torch.testing.assert_close(normed, ref)
    rms = normed.pow(2).mean(-1).sqrt()
    assert torch.allclose(rms, torch.ones_like(rms), atol=2e-2)


def test_log_sum_exp_output_is_the_logsumexp_of_the_scaled_masked_scores():
    """`return_lse` (an extension of this library: the reference returns only the output) must be
    `logsumexp(q k^T * scale + mask)` over the keys, and must not change the output."""
    c = load("causal")
    q, k, v = c["q"].float(), c["k"].float(), c["v"].float()
    out, lse = ao.causal(c["q"], c["k"], c["v"], return_lse=True)
    close(out, c["out"])
    L, S = q.size(-2), k.size(-2)
    s = q @ k.transpose(-1, -2) / q.size(-1) ** 0.5
    s = s.masked_fill(torch.triu(torch.ones(L, S, dtype=torch.bool), 1), float("-inf"))
    close(lse, torch.logsumexp(s, dim=-1))
    c = load("vanilla_nogqa")
    q, k = c["q"].float(), c["k"].float()
    out, lse = ao.vanilla(c["q"], c["k"], c["v"], return_lse=True)
    close(out, c["out"])
    close(lse, torch.logsumexp(q @ k.transpose(-1, -2) / q.size(-1) ** 0.5, dim=-1))


@pytest.mark.parametrize("name", ["vanilla", "causal_gqa", "sliding_window", "evoformer"])
def test_oracle_equals_the_compiled_reference_modules(name):
    """Where `oracle/_ref/` holds the reference's own byte-compiled modules (built by
    `oracle/build_ref.py`), the restatement and the reference give the same fp32 result on a
    shortened benchmark workload, bit for bit."""
    from flashlight_b200.workloads import WORKLOADS, make_inputs
    from oracle.run_config import reference_runner, run_oracle
    w = WORKLOADS[name]
    w = w.scaled(N=min(w.N, 3), S=200)
    fn = reference_runner(w)
    if fn is None:
        pytest.skip("oracle/_ref has not been built here")
    t = make_inputs(w, seed=9)
    assert torch.equal(fn(w, t), run_oracle(w, t))
