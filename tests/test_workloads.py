"""Effective-FLOP numerators: closed-form pair counts against brute-force masks, and the
full-size values the benchmark reports."""
import pytest
import torch

from flashlight_b200.workloads import WORKLOADS, effective_flops, make_inputs, unmasked_pairs


def brute_pairs(w, t):
    S = w.S
    i = torch.arange(S).view(-1, 1)
    j = torch.arange(S).view(1, -1)
    total = 0
    heads = w.Hq // 2 if w.variant == "diff" else w.Hq
    for n in range(w.N):
        if w.variant == "vanilla":
            keep = torch.ones(S, S, dtype=torch.bool)
        elif w.variant in ("causal", "alibi", "softcap", "diff"):
            keep = (j <= i) if w.causal else torch.ones(S, S, dtype=torch.bool)
        elif w.variant == "sliding":
            keep = (j <= i) & ((i - j) <= w.extra["window"])
        elif w.variant == "document":
            d = t["document_id"][n]
            keep = d.view(-1, 1) == d.view(1, -1)
            if w.causal:
                keep &= j <= i
        elif w.variant == "prefix":
            keep = j <= torch.maximum(t["prefix_len"][n] - 1, i)
        elif w.variant == "evoformer":
            keep = torch.isfinite(t["mask_bias"][0, n, 0, 0].float()).view(1, -1).expand(S, S)
        total += int(keep.sum()) * heads
    return total


@pytest.mark.parametrize("name", list(WORKLOADS))
def test_pair_counts_small(name):
    w = WORKLOADS[name]
    small = w.scaled(N=min(w.N, 3), Hq=4, Hkv=2 if w.Hq != w.Hkv else 4, S=200)
    if small.variant == "sliding":
        small = small.scaled(extra={"window": 37})
    if small.variant == "document":
        small = small.scaled(extra={"doc_min": 10, "doc_max": 60})
    t = make_inputs(small, seed=3)
    assert unmasked_pairs(small, t) == brute_pairs(small, t)


def test_full_size_flops():
    w = WORKLOADS["causal_gqa"]
    assert unmasked_pairs(w, {}) == 256 * 8390656
    assert effective_flops(w, {}) == pytest.approx(1.0998e12, rel=1e-4)
    w = WORKLOADS["sliding_window"]
    assert unmasked_pairs(w, {}) == 64 * 7872000
    w = WORKLOADS["alibi_causal"]
    assert effective_flops(w, {}) == pytest.approx(1.0996e12, rel=1e-4)
    w = WORKLOADS["diff_attn"]
    assert effective_flops(w, {}) == pytest.approx(4.1242e11, rel=1e-4)
    w = WORKLOADS["vanilla"]
    assert effective_flops(w, {}) == pytest.approx(4.295e9, rel=1e-3)


def test_inputs_are_seeded_and_bf16():
    w = WORKLOADS["prefix_lm"].scaled(N=2, Hq=2, Hkv=2, S=64)
    a, b = make_inputs(w, seed=5), make_inputs(w, seed=5)
    for k in a:
        assert torch.equal(a[k], b[k])
    assert a["q"].dtype == torch.bfloat16 and a["prefix_len"].dtype == torch.int64
    assert int(a["prefix_len"].max()) <= w.S // 2
    c = make_inputs(w, seed=6)
    assert not torch.equal(a["q"], c["q"])


# ---------------------------------------------------------------- slices for several GPUs
def _small(name):
    w = WORKLOADS[name]
    kw = dict(S=96)
    if w.variant == "evoformer":
        kw.update(N=8, Hq=2, Hkv=2)
    elif w.variant == "document":
        kw.update(N=1, Hq=8, Hkv=8, extra={"doc_min": 10, "doc_max": 40})
    elif w.variant == "diff":
        kw.update(N=2, Hq=16, Hkv=16)
    elif w.variant == "sliding":
        kw.update(N=2, Hq=8, Hkv=8, extra={"window": 20})
    else:
        kw.update(N=2, Hq=16 if w.Hq != w.Hkv else 8, Hkv=4 if w.Hq != w.Hkv else 8)
    return w.scaled(**kw)


@pytest.mark.parametrize("name", [n for n in WORKLOADS if n != "vanilla"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_slices_are_disjoint_cover_everything_and_reproduce_the_whole(name, world):
    """Every rank's slice through the oracle, put back together, is the oracle on the whole
    workload: the slices cover every (batch, head) unit once, per-sequence inputs and the ALiBi
    slopes travel with them, and the work adds up."""
    from flashlight_b200.workloads import shard
    from oracle.run_config import run_oracle
    w = _small(name)
    t = make_inputs(w, seed=5)
    whole = run_oracle(w, t)
    parts, flops = [], 0.0
    for rank in range(world):
        ws, ts = shard(w, t, rank, world)
        flops += effective_flops(ws, ts)
        parts.append(run_oracle(ws, ts))
    assert flops == pytest.approx(effective_flops(w, t), rel=1e-12)
    if w.variant == "evoformer":
        got = torch.cat(parts, dim=1)
    elif w.N % world == 0:
        got = torch.cat(parts, dim=0)
    else:
        c = world // w.N                              # ranks per sequence: head groups of one sequence
        got = torch.cat([torch.cat(parts[b * c:(b + 1) * c], dim=1) for b in range(w.N)], dim=0)
    assert got.shape == whole.shape
    assert torch.equal(got, whole)


def test_full_size_slices_carry_equal_work():
    from flashlight_b200.workloads import shard
    for name in ("causal_gqa", "alibi_causal", "sliding_window", "diff_attn"):
        w = WORKLOADS[name]
        shapes = {k: torch.empty(0) for k in ()}
        # only shapes matter for these variants' pair counts: use meta tensors
        t = {"q": torch.empty(w.N, w.Hq, w.S, w.E, device="meta"),
             "k": torch.empty(w.N, w.Hkv, w.S, w.E, device="meta"),
             "v": torch.empty(w.N, w.Hq // 2 if w.variant == "diff" else w.Hkv, w.S, w.Ev, device="meta")}
        for world in (2, 4, 8):
            per = {effective_flops(*shard(w, t, r, world)) for r in range(world)}
            assert len(per) == 1 and per.pop() * world == pytest.approx(effective_flops(w, t), rel=1e-12)
