"""GPU parity: the sm_100a kernels (called through the variant API -> custom op -> C ABI)
against the reference's golden outputs and the fp32 oracle.

Tolerances (bf16 output vs fp32 oracle on the same bf16-rounded inputs):
  N(0,1) inputs:  max-abs <= 2e-2 and mean-abs <= 2e-3 (flat; see tests/_parity.py for the
                  handling of the rare reference values of magnitude 4 and more)
  U[-9,9) inputs (the reference tests' distribution, tests/test_causal.py:28-30):
                  |a-b| <= 2e-2 + 1e-2 |b|   (tests/test_vanilla.py:36)
"""
from pathlib import Path

import pytest
import torch

import flashlight_b200
from flashlight_b200 import attention_variants as av
from flashlight_b200.workloads import WORKLOADS, make_inputs, run as run_product
from oracle import attention_oracle as ao
from oracle.run_config import run_oracle
from _parity import check, report

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(params=[2, 1], ids=["two_stage", "one_stage"])
def stages(request, monkeypatch):
    """Run a test with both kernel layouts (two query tiles per CTA, or one and two CTAs per SM)
    instead of the layout the library would pick for the shape."""
    monkeypatch.setenv("FLB200_STAGES", str(request.param))
    return request.param


def dev(t):
    return t.cuda() if torch.is_tensor(t) else t


def load(name):
    return {k: dev(v) for k, v in torch.load(GOLDEN / f"{name}.pt", weights_only=True).items()}


# ---------------------------------------------------------------- golden vectors
def test_golden_vanilla(stages):
    c = load("vanilla_nogqa")
    check(av.attention_pytorch_nogqa(c["q"], c["k"], c["v"]), c["out"])
    c = load("vanilla_gqa")
    check(av.attention_pytorch(c["q"], c["k"], c["v"], enable_gqa=True), c["out"])


def test_golden_causal(stages):
    c = load("causal")
    check(av.attention_pytorch_causal(c["q"], c["k"], c["v"]), c["out"])
    c = load("causal_gqa")
    check(av.attention_pytorch_causal(c["q"], c["k"], c["v"], enable_gqa=True), c["out"])


def test_golden_alibi(stages):
    c = load("alibi")
    check(av.attention_pytorch_alibi(c["q"], c["k"], c["v"], score_mod=av.generate_alibi_bias_pytorch(c["nheads"])),
          c["out"])
    c = load("alibi_gqa")
    check(av.attention_pytorch_alibi(c["q"], c["k"], c["v"], score_mod=av.generate_alibi_bias_pytorch(c["nheads"]),
                                     enable_gqa=True), c["out"])


def test_golden_softcap(stages):
    c = load("softcap")
    check(av.attention_softcapped(c["q"], c["k"], c["v"], av.generate_tanh_softcap(c["cap"])), c["out"])


def test_golden_sliding(stages):
    c = load("sliding")
    check(av.attention_pytorch_sliding_window(c["q"], c["k"], c["v"], window_size=c["window"]), c["out"])


@pytest.mark.parametrize("name", ["document", "document_unsorted"])
def test_golden_document(name, stages):
    c = load(name)
    check(av.attention_pytorch_document_mask(c["q"], c["k"], c["v"], c["document_id"]), c["out"])


def test_golden_prefix(stages):
    c = load("prefix")
    check(av.attention_pytorch_prefix_lm(c["q"], c["k"], c["v"], prefix_lengths=c["prefix"]), c["out"])


@pytest.mark.parametrize("name", ["diff", "diff_l08", "diff_d128"])
def test_golden_diff(name):
    c = load(name)
    check(av.diffattn(c["q"], c["k"], c["v"], lambda_full=c["lam"]), c["out"])


@pytest.mark.parametrize("name", ["evoformer", "evoformer_mask"])
def test_golden_evoformer(name, stages):
    c = load(name)
    check(av.attention_reference(c["q"], c["k"], c["v"], [c["bias1"], c["bias2"]]), c["out"])


# ---------------------------------------------------------------- shape matrix vs oracle
def rnd(shape, seed, uniform=False):
    g = torch.Generator().manual_seed(seed)
    if uniform:
        return (torch.rand(*shape, generator=g) * 18 - 9).to(torch.bfloat16).cuda()
    return torch.randn(*shape, generator=g).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("S", [1, 17, 127, 128, 129, 384, 1000])
@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_shapes_vanilla_causal(S, D, causal, stages):
    q, k, v = rnd((2, 3, S, D), 1), rnd((2, 3, S, D), 2), rnd((2, 3, S, D), 3)
    if causal:
        check(av.attention_pytorch_causal(q, k, v), ao.causal(q, k, v), (S, D))
    else:
        check(av.attention_pytorch(q, k, v), ao.vanilla(q, k, v), (S, D))


@pytest.mark.parametrize("G", [4, 8])
@pytest.mark.parametrize("D", [64, 128])
def test_gqa(G, D, stages):
    q, k, v = rnd((2, 2 * G, 333, D), 4), rnd((2, 2, 333, D), 5), rnd((2, 2, 333, D), 6)
    out = av.attention_pytorch_causal(q, k, v, enable_gqa=True)
    assert out.shape == (2, 2, G, 333, D)
    check(out, ao.causal(q, k, v, enable_gqa=True))
    check(av.attention_pytorch(q, k, v, enable_gqa=True), ao.vanilla(q, k, v, enable_gqa=True))


def test_cross_attention_lengths():
    """L != S: vanilla on any lengths, causal aligned top-left as triu(ones(L, S), 1)."""
    q, k, v = rnd((1, 2, 200, 64), 7), rnd((1, 2, 520, 64), 8), rnd((1, 2, 520, 64), 9)
    check(av.attention_pytorch(q, k, v), ao.vanilla(q, k, v))
    check(av.attention_pytorch_causal(q, k, v), ao.causal(q, k, v))
    q = rnd((1, 2, 520, 64), 10)
    k, v = rnd((1, 2, 200, 64), 11), rnd((1, 2, 200, 64), 12)
    check(av.attention_pytorch_causal(q, k, v), ao.causal(q, k, v))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("is_causal", [False, True])
def test_alibi_softcap(D, is_causal, stages):
    q, k, v = rnd((2, 8, 700, D), 13), rnd((2, 2, 700, D), 14), rnd((2, 2, 700, D), 15)
    check(av.attention_pytorch_alibi(q, k, v, score_mod=av.generate_alibi_bias_pytorch(8), is_causal=is_causal,
                                     enable_gqa=True),
          ao.alibi(q, k, v, nheads=8, is_causal=is_causal, enable_gqa=True))
    for cap in (50.0, 2.0):
        check(av.attention_softcapped(q, k, v, av.generate_tanh_softcap(cap), is_causal=is_causal, enable_gqa=True),
              ao.softcap(q, k, v, cap, is_causal=is_causal, enable_gqa=True), cap)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("shape", ["ramp", "step", "spikes"])
def test_row_maximum_that_grows_along_the_keys(D, shape, stages):
    """Later key tiles beat the running maximum by a little (absorbed), by a lot (accumulator
    rescaled) or in single keys: the tile is first tried with the old maximum and must be redone."""
    S = 1280
    q, k, v = rnd((1, 4, S, D), 61), rnd((1, 4, S, D), 62), rnd((1, 4, S, D), 63)
    j = torch.arange(S, device="cuda", dtype=torch.float32)
    if shape == "ramp":
        gain = 0.25 + 5.0 * j / S
    elif shape == "step":
        gain = torch.where(j < 700, 0.2, 6.0)
    else:
        gain = torch.where((j % 131) == 130, 7.0, 0.5)
    k = (k.float() * gain[None, None, :, None]).to(torch.bfloat16)
    check(av.attention_pytorch(q, k, v), ao.vanilla(q, k, v), shape)
    check(av.attention_pytorch_causal(q, k, v), ao.causal(q, k, v), shape)
    check(av.attention_pytorch_alibi(q, k, v, score_mod=av.generate_alibi_bias_pytorch(4), is_causal=False),
          ao.alibi(q, k, v, nheads=4, is_causal=False), shape)
    check(av.attention_pytorch_alibi(q, k, v, score_mod=av.generate_alibi_bias_pytorch(4), is_causal=True),
          ao.alibi(q, k, v, nheads=4, is_causal=True), shape)


@pytest.mark.parametrize("S,window", [(1024, 256), (1000, 1), (777, 0), (640, 5000), (1536, 128), (2048, 1024)])
def test_sliding_window(S, window, stages):
    q, k, v = rnd((1, 2, S, 64), 16), rnd((1, 2, S, 64), 17), rnd((1, 2, S, 64), 18)
    check(av.attention_pytorch_sliding_window(q, k, v, window_size=window),
          ao.sliding_window(q, k, v, window_size=window), (S, window))


@pytest.mark.parametrize("S,D", [(300, 128), (1024, 128), (2500, 128), (1024, 64), (700, 64)])
@pytest.mark.parametrize("is_causal", [False, True])
def test_document_mask(S, D, is_causal, stages):
    q, k, v = rnd((2, 2, S, D), 19), rnd((2, 2, S, D), 20), rnd((2, 2, S, D), 21)
    g = torch.Generator().manual_seed(S)
    lens = []
    while sum(lens) < S:
        lens.append(min(int(torch.randint(1, 400, (1,), generator=g)), S - sum(lens)))
    ids = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens))
    doc = torch.stack([ids, ids.flip(0)]).cuda()          # second row: descending ids
    check(av.attention_pytorch_document_mask(q, k, v, doc, is_causal=is_causal),
          ao.document_mask(q, k, v, doc, is_causal=is_causal), (S, is_causal))
    # the reference's generator: one row expanded over the batch (document_mask.py:64-67)
    doc_e = av.create_document_id(2, S, num_docs=7, device=torch.device("cuda"))
    check(av.attention_pytorch_document_mask(q, k, v, doc_e, is_causal=is_causal),
          ao.document_mask(q, k, v, doc_e, is_causal=is_causal))


@pytest.mark.parametrize("S", [256, 1000])
def test_prefix_lm(S, stages):
    q, k, v = rnd((3, 2, S, 64), 22), rnd((3, 2, S, 64), 23), rnd((3, 2, S, 64), 24)
    for p in (0, 1, 256, S):
        check(av.attention_pytorch_prefix_lm(q, k, v, prefix_lengths=p), ao.prefix_lm(q, k, v, prefix_lengths=p), p)
    pl = torch.tensor([0, S // 3, S // 2])
    check(av.attention_pytorch_prefix_lm(q, k, v, prefix_lengths=pl), ao.prefix_lm(q, k, v, prefix_lengths=pl))
    check(av.attention_pytorch_prefix_lm(q, k, v, prefix_lengths=pl.cuda()), ao.prefix_lm(q, k, v, prefix_lengths=pl))


@pytest.mark.parametrize("d", [32, 64])
@pytest.mark.parametrize("S", [128, 700])
def test_diff_attention(d, S):
    q, k = rnd((2, 6, S, d), 25), rnd((2, 6, S, d), 26)
    v = rnd((2, 3, S, 2 * d), 27)
    check(av.diffattn(q, k, v), ao.diffattn(q, k, v))
    check(av.diffattn(q, k, v, lambda_full=0.8, is_causal=True), ao.diffattn(q, k, v, lambda_full=0.8, is_causal=True))
    check(av.diffattn(q, k, v, lambda_full=0.8, is_causal=True, rms_norm=True, rms_eps=1e-5),
          ao.diffattn(q, k, v, lambda_full=0.8, is_causal=True, rms_norm=True, rms_eps=1e-5))


@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("S", [256, 384, 200])
def test_evoformer(D, S, stages):
    B, N, H = 1, 5, 4
    q, k, v = rnd((B, N, S, H, D), 28), rnd((B, N, S, H, D), 29), rnd((B, N, S, H, D), 30)
    pair = rnd((B, 1, H, S, S), 31)
    g = torch.Generator().manual_seed(32)
    keep = torch.rand(B, N, 1, 1, S, generator=g) < 0.9
    keep[..., 0] = True
    mask = torch.where(keep, 0.0, float("-inf")).to(torch.bfloat16).cuda()
    out = av.attention_reference(q, k, v, [mask, pair])
    assert out.shape == q.shape and out.is_contiguous()
    check(out, ao.evoformer(q, k, v, [mask, pair]), (D, S))
    check(av.attention_reference(q, k, v, [pair]), ao.evoformer(q, k, v, [pair]))
    check(av.attention_reference(q, k, v, []), ao.evoformer(q, k, v, []))


@pytest.mark.parametrize("D,S", [(32, 328), (64, 256), (64, 200)])
def test_evoformer_key_vector_added_by_the_tensor_cores(D, S, monkeypatch):
    """Resident pair-bias kernel (four or more rows share a pair bias, narrow heads, enough work to pay for
    one more launch): the per-row key vector, with its -inf entries, is added by one more k-step of the
    score product when the caller gives scratch memory (the second launch lays the vector out), by the
    softmax threads otherwise.  Heads of 64 run it on a ring of two slots per stage."""
    B, N, H = 2, 200, 4   # enough rows to pay for the extra launch; bias rows start on 16-byte boundaries (TMA)
    q, k, v = rnd((B, N, S, H, D), 60), rnd((B, N, S, H, D), 61), rnd((B, N, S, H, D), 62)
    pair = rnd((B, 1, H, S, S), 63)
    g = torch.Generator().manual_seed(64)
    keep = torch.rand(B, N, 1, 1, S, generator=g) < 0.8
    keep[..., 5] = True
    vec = (torch.randn(B, N, 1, 1, S, generator=g) * 3).masked_fill(~keep, float("-inf")).to(torch.bfloat16).cuda()
    ref = ao.evoformer(q, k, v, [vec, pair])
    outs = {}
    for flag, launches in (("1", 2), ("0", 1)):
        monkeypatch.setenv("FLB200_KEYVEC_MMA", flag)
        n0 = flashlight_b200.launch_count()
        outs[flag] = av.attention_reference(q, k, v, [vec, pair])
        assert flashlight_b200.launch_count() - n0 == launches
        check(outs[flag], ref, flag)
    # the two paths round independently: up to one bf16 step apart on top of the flat band
    a, b = outs["1"].float(), outs["0"].float()
    assert bool(((a - b).abs() <= 2e-2 + 2.0 ** -7 * b.abs()).all())


# ---------------------------------------------------------------- the reference tests' own inputs
def close_ref(out, ref):
    """assert_close(atol=2e-2, rtol=1e-2) as in the reference's tests (tests/test_vanilla.py:36).

    With |values| up to 9 and P rounded to bf16 before the PV product (as the reference's compiled
    kernel does, monkeypatch/fusion/block_reduction.py:86-103) an element lands a hair outside
    that band about once in a few million; the reference's tests draw unseeded inputs and live
    with that.  Here: at most 2 elements per million outside, and none beyond twice the band.
    """
    flashlight_b200.check_status()
    o, r = out.float().cpu(), ref.float().cpu()
    assert o.shape == r.shape
    excess = (o - r).abs() - (2e-2 + 1e-2 * r.abs())
    bad = int((excess > 0).sum())
    assert bad <= max(1, 2 * o.numel() // 1_000_000), (bad, excess.max().item())
    assert ((o - r).abs() <= 2 * (2e-2 + 1e-2 * r.abs())).all(), excess.max().item()


def test_uniform_inputs_like_reference_tests():
    # tests/test_vanilla.py:21-36 shape family (B2 H1 D128), scaled to S=2048
    q, k, v = (rnd((2, 1, 2048, 128), s, uniform=True) for s in (40, 41, 42))
    close_ref(av.attention_pytorch(q, k, v), ao.vanilla(q, k, v))
    close_ref(av.attention_pytorch_causal(q, k, v), ao.causal(q, k, v))
    # tests/test_alibi.py / test_sliding_window.py: B4 H16 G8 S1024 D64, window 256
    q = rnd((2, 16, 1024, 64), 43, uniform=True)
    k, v = rnd((2, 2, 1024, 64), 44, uniform=True), rnd((2, 2, 1024, 64), 45, uniform=True)
    close_ref(av.attention_pytorch_alibi(q, k, v, score_mod=av.generate_alibi_bias_pytorch(16), enable_gqa=True),
              ao.alibi(q, k, v, nheads=16, enable_gqa=True))
    close_ref(av.attention_pytorch_sliding_window(q, k, v, window_size=256, enable_gqa=True),
              ao.sliding_window(q, k, v, window_size=256, enable_gqa=True))
    close_ref(av.attention_pytorch_prefix_lm(q, k, v, prefix_lengths=256, enable_gqa=True),
              ao.prefix_lm(q, k, v, prefix_lengths=256, enable_gqa=True))
    close_ref(av.attention_softcapped(q, k, v, av.generate_tanh_softcap(30.0), enable_gqa=True),
              ao.softcap(q, k, v, 30.0, enable_gqa=True))


# ---------------------------------------------------------------- properties
@pytest.mark.parametrize("D", [64, 128])
def test_a_row_with_one_key_returns_its_value_row_exactly(D, stages):
    """softmax over a single visible key is exactly 1: the row maximum is exact, so P = 1, l = 1 and
    the output row is the bf16 value row, bit for bit (S = 1, and row 0 under a causal mask)."""
    q, k, v = rnd((2, 4, 1, D), 70), rnd((2, 2, 1, D), 71), rnd((2, 2, 1, D), 72)
    want = v.repeat_interleave(2, dim=1)
    assert torch.equal(av.attention_pytorch(q, k, v, enable_gqa=True), want)
    assert torch.equal(av.attention_pytorch_alibi(q, k, v, score_mod=av.generate_alibi_bias_pytorch(4),
                                                  enable_gqa=True).reshape(want.shape), want)
    assert torch.equal(av.attention_softcapped(q, k, v, av.generate_tanh_softcap(30.0),
                                               enable_gqa=True).reshape(want.shape), want)
    q, k, v = rnd((1, 2, 300, D), 73), rnd((1, 2, 300, D), 74), rnd((1, 2, 300, D), 75)
    for out in (av.attention_pytorch_causal(q, k, v),
                av.attention_pytorch_alibi(q, k, v, score_mod=av.generate_alibi_bias_pytorch(2), is_causal=True),
                av.attention_pytorch_sliding_window(q, k, v, window_size=0)):
        assert torch.equal(out[:, :, 0], v[:, :, 0])
    # window 0 keeps only the diagonal: every row returns its own value row
    assert torch.equal(av.attention_pytorch_sliding_window(q, k, v, window_size=0), v)
    flashlight_b200.check_status()


def test_deterministic():
    q, k, v = rnd((2, 4, 1500, 128), 50), rnd((2, 4, 1500, 128), 51), rnd((2, 4, 1500, 128), 52)
    first = av.attention_pytorch_causal(q, k, v)
    for _ in range(5):
        assert torch.equal(av.attention_pytorch_causal(q, k, v), first)


def test_strided_inputs_and_layouts(stages):
    """Head-major and row-major storage give the same result (no copies are made)."""
    base = rnd((2, 500, 3, 3 * 64), 53)                   # packed [N, L, H, 3*D]
    q, k, v = (base[..., i * 64:(i + 1) * 64].transpose(1, 2) for i in range(3))
    out = av.attention_pytorch_causal(q, k, v)
    check(out, ao.causal(q, k, v))


def test_host_tensors_are_staged_through_the_device():
    g = torch.Generator().manual_seed(54)
    q, k, v = (torch.randn(1, 2, 300, 64, generator=g).to(torch.bfloat16).pin_memory() for _ in range(3))
    out = av.attention_pytorch_causal(q, k, v)
    assert out.device.type == "cpu"
    check(out, ao.causal(q, k, v))


def test_pinned_host_batches_are_pipelined_and_identical():
    """Large pinned host inputs go through the chunked three-stream path (copy-in, kernel and
    copy-out of successive batch chunks overlap); the result is the one the device path gives."""
    g = torch.Generator().manual_seed(60)
    N, Hq, Hkv, S, D = 5, 8, 2, 1024, 128
    q = torch.randn(N, Hq, S, D, generator=g).to(torch.bfloat16).pin_memory()
    k = torch.randn(N, Hkv, S, D, generator=g).to(torch.bfloat16).pin_memory()
    v = torch.randn(N, Hkv, S, D, generator=g).to(torch.bfloat16).pin_memory()
    assert q.numel() * 2 >= 8 << 20
    out = av.attention_pytorch_causal(q, k, v, enable_gqa=True)
    assert out.device.type == "cpu" and out.shape == (N, Hkv, Hq // Hkv, S, D)
    dev_out = av.attention_pytorch_causal(q.cuda(), k.cuda(), v.cuda(), enable_gqa=True)
    assert torch.equal(out, dev_out.cpu())
    # per-sequence arguments are sliced with the batch
    pl = torch.tensor([0, 100, 1024, 513, 7])
    out = av.attention_pytorch_prefix_lm(q, k, v, prefix_lengths=pl, enable_gqa=True)
    dev_out = av.attention_pytorch_prefix_lm(q.cuda(), k.cuda(), v.cuda(), prefix_lengths=pl.cuda(), enable_gqa=True)
    assert torch.equal(out, dev_out.cpu())
    ids = torch.stack([torch.repeat_interleave(torch.arange(4), torch.tensor([100 + 10 * n, 300, 400, 224 - 10 * n]))
                       for n in range(N)])
    out = av.attention_pytorch_document_mask(q, k, v, ids, enable_gqa=True)
    dev_out = av.attention_pytorch_document_mask(q.cuda(), k.cuda(), v.cuda(), ids.cuda(), enable_gqa=True)
    assert torch.equal(out, dev_out.cpu())
    flashlight_b200.check_status()


def test_unsupported_raises_instead_of_falling_back():
    q = rnd((1, 2, 128, 264), 55)                     # head dims above 256 have no kernel
    with pytest.raises(NotImplementedError):
        av.attention_pytorch(q, q, q)
    q = rnd((1, 2, 128, 64), 55)
    with pytest.raises(NotImplementedError):
        av.attention_pytorch(q.float(), q.float(), q.float())
    before = flashlight_b200.launch_count()
    q = rnd((1, 2, 128, 64), 56)
    av.attention_pytorch(q, q, q)
    assert flashlight_b200.launch_count() == before + 1


def test_torch_compile_wraps_the_op():
    q, k, v = rnd((1, 2, 512, 64), 57), rnd((1, 2, 512, 64), 58), rnd((1, 2, 512, 64), 59)
    fn = torch.compile(av.attention_pytorch_causal, dynamic=False)
    check(fn(q, k, v), ao.causal(q, k, v))


# ---------------------------------------------------------------- benchmark configurations, full size
@pytest.mark.parametrize("name", [n for n in WORKLOADS if n != "vanilla"])
def test_full_size_workloads(name):
    """Full benchmark shapes against the fp32 oracle evaluated on the device (the CPU would
    need minutes); the oracle code is the same, only its tensors live in HBM.  The whole batch
    is computed; the first two sequences (MSA rows) of it are compared, which is the whole
    batch for the document workload (one sequence)."""
    w = WORKLOADS[name]
    t = {k: v.cuda() for k, v in make_inputs(w, seed=0).items()}
    out = run_product(w, t)
    flashlight_b200.check_status()
    # compare a slice of the batch to bound oracle time and memory
    ws = w.scaled(N=min(w.N, 2))
    ts = {k: (v[:, :ws.N] if w.variant == "evoformer" and v.size(1) == w.N else
              v[:ws.N] if w.variant != "evoformer" else v) for k, v in t.items()}
    ref = run_oracle(ws, ts)
    got = out[:, :ws.N] if w.variant == "evoformer" else out[:ws.N]
    s = check(got, ref, name)
    report(name, s)
    # the flat figure of the stated tolerance: nothing above 2e-2 except next to a reference value
    # of 4 or more, whose bf16 rounding alone takes most of that band
    assert s["n_above_2e-2"] == 0 or s["largest_ref_above_2e-2"] >= 4.0, s


def test_vanilla_workload_against_cpu_oracle():
    w = WORKLOADS["vanilla"]
    t = make_inputs(w, seed=0)
    ref = run_oracle(w, t)                                   # fp32 on the host, as configured
    out = run_product(w, {k: v.cuda() for k, v in t.items()})
    check(out, ref)


# ---------------------------------------------------------------- differential attention, wide heads
@pytest.mark.parametrize("S", [128, 700])
@pytest.mark.parametrize("d", [128, 96])
def test_diff_attention_with_value_heads_of_256(d, S):
    """q/k heads of 128 with value heads of 256, the reference's own test shape family
    (tests/test_diffattn.py:25-34: B16 H16 S1024 d128): two CTAs per work item take one half of the
    value columns each; with the RMS normalisation they run as a cluster and swap row sums."""
    q, k = rnd((2, 4, S, d), 80), rnd((2, 4, S, d), 81)
    v = rnd((2, 2, S, 2 * d), 82)
    check(av.diffattn(q, k, v), ao.diffattn(q, k, v))
    check(av.diffattn(q, k, v, lambda_full=0.8, is_causal=True), ao.diffattn(q, k, v, lambda_full=0.8, is_causal=True))
    check(av.diffattn(q, k, v, lambda_full=0.8, is_causal=True, rms_norm=True, rms_eps=1e-5),
          ao.diffattn(q, k, v, lambda_full=0.8, is_causal=True, rms_norm=True, rms_eps=1e-5))


def test_diff_attention_reference_test_shape():
    q, k = rnd((16, 16, 1024, 128), 83), rnd((16, 16, 1024, 128), 84)
    v = rnd((16, 8, 1024, 256), 85)
    out = av.diffattn(q, k, v)
    ref = torch.cat([ao.diffattn(q[n:n + 4], k[n:n + 4], v[n:n + 4]) for n in range(0, 16, 4)])
    check(out, ref)


@pytest.mark.parametrize("d", [32, 64])
@pytest.mark.parametrize("v_exp", [0, -10, 8, -30])
def test_diff_rms_product_in_fp16_whatever_the_scale_of_v(d, v_exp, monkeypatch):
    """RMS-normalised differential attention with value heads up to 128 runs P.V in fp16 when the caller
    gives scratch (one launch more: the pass that finds max |v|): V is rewritten as fp16 in shared memory
    after a multiplication by the power of two that centres its range, and eps is scaled alike, so the
    result follows the oracle for V of any magnitude (2^-10: eps dominates the mean square; 2^-30: below
    the fp16 range before the scaling).  Switched off, P goes as two bf16 terms."""
    q, k = rnd((1, 6, 520, d), 90), rnd((1, 6, 520, d), 91)
    v = (rnd((1, 3, 520, 2 * d), 92).float() * 2.0 ** v_exp).to(torch.bfloat16)
    # with eps = 0 the result is of order one whatever the scale, so the smallest V really tests the scaling
    kw = dict(lambda_full=0.8, is_causal=True, rms_norm=True, rms_eps=0.0 if v_exp == -30 else 1e-5)
    ref = ao.diffattn(q, k, v, **kw)
    assert ref.abs().mean().item() > 0.1 or v_exp == -10
    for flag, launches in (("1", 2), ("0", 1)):
        monkeypatch.setenv("FLB200_DIFF_PV_F16", flag)
        n0 = flashlight_b200.launch_count()
        out = av.diffattn(q, k, v, **kw)
        assert flashlight_b200.launch_count() - n0 == launches
        check(out, ref, (flag, v_exp))


def test_diff_rms_norm_divides_by_the_true_width():
    q, k, v = rnd((1, 4, 300, 48), 86), rnd((1, 4, 300, 48), 87), rnd((1, 2, 300, 96), 88)
    check(av.diffattn(q, k, v, lambda_full=0.5, rms_norm=True), ao.diffattn(q, k, v, lambda_full=0.5, rms_norm=True))
