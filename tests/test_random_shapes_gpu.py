"""Seeded random shapes and variants against the fp32 oracle: odd lengths, GQA groups, head dims,
sorted / reversed / shuffled document ids, tensor prefix lengths, cross attention, biases."""
import random

import pytest
import torch

import flashlight_b200
from flashlight_b200 import attention_variants as av
from oracle import attention_oracle as ao
from _parity import check

pytestmark = pytest.mark.gpu
LENGTHS = [1, 2, 17, 100, 128, 129, 255, 256, 257, 383, 500, 640, 777, 1024, 1500]
VARIANTS = ["vanilla", "cross", "causal", "alibi", "alibi_c", "softcap", "softcap_c", "sliding", "prefix",
            "doc", "doc_c", "diff", "evo"]


def _rnd(shape, g):
    return torch.randn(shape, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)


def _close(out, ref):
    try:
        check(out, ref)
    except AssertionError:
        return False
    return True


def _case(rng, g):
    D = rng.choice([32, 64, 128])
    N, Hkv, G = rng.randint(1, 3), rng.randint(1, 3), rng.choice([1, 1, 2, 4])
    Hq, S, variant = Hkv * G, rng.choice(LENGTHS), rng.choice(VARIANTS)
    gqa = G > 1
    if D == 32 and variant not in ("vanilla", "cross", "causal", "diff", "evo"):
        return None
    q, k, v = _rnd((N, Hq, S, D), g), _rnd((N, Hkv, S, D), g), _rnd((N, Hkv, S, D), g)
    what = (variant, N, Hq, Hkv, S, D)
    if variant == "vanilla":
        return what, av.attention_pytorch(q, k, v, enable_gqa=gqa), ao.vanilla(q, k, v, enable_gqa=gqa)
    if variant == "cross":
        q = _rnd((N, Hq, rng.choice([1, 64, 130, 300]), D), g)
        return what, av.attention_pytorch(q, k, v, enable_gqa=gqa), ao.vanilla(q, k, v, enable_gqa=gqa)
    if variant == "causal":
        return what, av.attention_pytorch_causal(q, k, v, enable_gqa=gqa), ao.causal(q, k, v, enable_gqa=gqa)
    if variant in ("alibi", "alibi_c"):
        c = variant.endswith("_c")
        return (what, av.attention_pytorch_alibi(q, k, v, score_mod=av.generate_alibi_bias_pytorch(Hq),
                                                 is_causal=c, enable_gqa=gqa),
                ao.alibi(q, k, v, nheads=Hq, is_causal=c, enable_gqa=gqa))
    if variant in ("softcap", "softcap_c"):
        c, cap = variant.endswith("_c"), rng.choice([2.0, 30.0, 50.0])
        return (what + (cap,), av.attention_softcapped(q, k, v, av.generate_tanh_softcap(cap), is_causal=c,
                                                       enable_gqa=gqa),
                ao.softcap(q, k, v, cap, is_causal=c, enable_gqa=gqa))
    if variant == "sliding":
        w = rng.choice([0, 1, 63, 128, 300, 5000])
        return (what + (w,), av.attention_pytorch_sliding_window(q, k, v, window_size=w, enable_gqa=gqa),
                ao.sliding_window(q, k, v, window_size=w, enable_gqa=gqa))
    if variant == "prefix":
        pl = torch.tensor([rng.randint(0, S) for _ in range(N)])
        return (what, av.attention_pytorch_prefix_lm(q, k, v, prefix_lengths=pl, enable_gqa=gqa),
                ao.prefix_lm(q, k, v, prefix_lengths=pl, enable_gqa=gqa))
    if variant in ("doc", "doc_c"):
        c, rows = variant.endswith("_c"), []
        for _ in range(N):
            lens = []
            while sum(lens) < S:
                lens.append(min(rng.randint(1, 300), S - sum(lens)))
            ids = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens))
            kind = rng.random()
            if kind < 0.15:
                ids = ids.flip(0)                                   # descending
            elif kind < 0.3:
                ids = ids[torch.randperm(S, generator=torch.Generator().manual_seed(rng.randint(0, 999)))]
            rows.append(ids)
        doc = torch.stack(rows).cuda()
        return (what, av.attention_pytorch_document_mask(q, k, v, doc, is_causal=c, enable_gqa=gqa),
                ao.document_mask(q, k, v, doc, is_causal=c, enable_gqa=gqa))
    if variant == "diff":
        if D == 128:
            return None
        H = 2 * Hkv
        q, k, v = _rnd((N, H, S, D), g), _rnd((N, H, S, D), g), _rnd((N, H // 2, S, 2 * D), g)
        c, rms = rng.random() < 0.5, rng.random() < 0.5
        return (what + (c, rms), av.diffattn(q, k, v, lambda_full=0.8, is_causal=c, rms_norm=rms, rms_eps=1e-5),
                ao.diffattn(q, k, v, lambda_full=0.8, is_causal=c, rms_norm=rms, rms_eps=1e-5))
    B, R, H = 1, rng.randint(1, 4), rng.randint(1, 3)
    q, k, v = _rnd((B, R, S, H, D), g), _rnd((B, R, S, H, D), g), _rnd((B, R, S, H, D), g)
    pair = _rnd((B, 1, H, S, S), g)
    keep = torch.rand(B, R, 1, 1, S, generator=g, device="cuda") < 0.9
    keep[..., 0] = True
    mask = torch.where(keep, 0.0, float("-inf")).to(torch.bfloat16)
    return what + (R, H), av.attention_reference(q, k, v, [mask, pair]), ao.evoformer(q, k, v, [mask, pair])


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_cases_match_the_oracle(seed):
    rng = random.Random(seed)
    g = torch.Generator(device="cuda").manual_seed(seed)
    done, bad = 0, []
    while done < 150:
        case = _case(rng, g)
        if case is None:
            continue
        what, out, ref = case
        done += 1
        if not _close(out, ref):
            bad.append(what)
    assert not bad, bad
