"""Named attention workloads: seeded synthetic inputs, effective-FLOP counts and the call
into the variant API for each of them.

The shapes are those of the benchmark configurations this library is measured on
(vanilla 2x8x1024x64; causal GQA 8x32/8x4096x128; ALiBi / softcap / sliding window at
4x16x8192x128; document mask 1x32x16384x128; prefix-LM 4x32x8192x128; Evoformer
1x256x384x8x32; differential attention 4x32x4096x64 with 128-wide values).  Inputs are
N(0,1) draws from a seeded CPU generator, rounded to bf16; q, k, v are drawn in that order.
They stand in for the public benchmark sweeps the reference takes its shapes from.

Effective FLOPs count only unmasked (query, key) pairs: pairs * (2 E + 2 Ev) per query head
(both branches for differential attention).  Mask evaluation, exp, biases, rescaling and
normalisation count as zero.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Dict

import torch

from . import attention_variants as av


@dataclass(frozen=True)
class Workload:
    name: str
    variant: str          # vanilla | causal | alibi | softcap | sliding | document | prefix | evoformer | diff
    N: int                # batch (Evoformer: number of MSA rows per batch element)
    Hq: int
    Hkv: int
    S: int                # sequence length (queries and keys)
    E: int
    Ev: int
    causal: bool = False
    extra: Dict[str, Any] = field(default_factory=dict)

    def scaled(self, **kw) -> "Workload":
        return replace(self, **kw)


WORKLOADS: Dict[str, Workload] = {
    w.name: w for w in [
        Workload("vanilla", "vanilla", 2, 8, 8, 1024, 64, 64),
        Workload("causal_gqa", "causal", 8, 32, 8, 4096, 128, 128, causal=True),
        Workload("alibi_causal", "alibi", 4, 16, 16, 8192, 128, 128, causal=True),
        Workload("softcap_causal", "softcap", 4, 16, 16, 8192, 128, 128, causal=True, extra={"cap": 50.0}),
        Workload("sliding_window", "sliding", 4, 16, 16, 8192, 128, 128, causal=True, extra={"window": 1024}),
        Workload("document_causal", "document", 1, 32, 32, 16384, 128, 128, causal=True,
                 extra={"doc_min": 256, "doc_max": 2048}),
        Workload("prefix_lm", "prefix", 4, 32, 32, 8192, 128, 128, causal=True),
        Workload("evoformer", "evoformer", 256, 8, 8, 384, 32, 32, extra={"keep": 0.95}),
        Workload("diff_attn", "diff", 4, 32, 32, 4096, 64, 128, causal=True,
                 extra={"lambda": 0.8, "rms_eps": 1e-5}),
    ]
}


def _randn_bf16(gen: torch.Generator, *shape) -> torch.Tensor:
    return torch.randn(*shape, generator=gen, dtype=torch.float32).to(torch.bfloat16)


def make_inputs(w: Workload, seed: int = 0, pin: bool = False) -> Dict[str, torch.Tensor]:
    """Seeded host tensors for a workload (bf16 data, int64 ids / lengths)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    t: Dict[str, torch.Tensor] = {}
    if w.variant == "evoformer":
        # [1, N_seq, N_res, H, D]; pair bias shared across rows; residue mask as 0 / -inf key bias
        shape = (1, w.N, w.S, w.Hq, w.E)
        t["q"], t["k"], t["v"] = (_randn_bf16(g, *shape) for _ in range(3))
        t["pair_bias"] = _randn_bf16(g, 1, 1, w.Hq, w.S, w.S)
        keep = torch.rand(1, w.N, 1, 1, w.S, generator=g) < w.extra["keep"]
        keep[..., 0] = True  # no row may lose every key
        t["mask_bias"] = torch.where(keep, 0.0, float("-inf")).to(torch.bfloat16)
    elif w.variant == "diff":
        t["q"] = _randn_bf16(g, w.N, w.Hq, w.S, w.E)
        t["k"] = _randn_bf16(g, w.N, w.Hkv, w.S, w.E)
        t["v"] = _randn_bf16(g, w.N, w.Hq // 2, w.S, w.Ev)
    else:
        t["q"] = _randn_bf16(g, w.N, w.Hq, w.S, w.E)
        t["k"] = _randn_bf16(g, w.N, w.Hkv, w.S, w.E)
        t["v"] = _randn_bf16(g, w.N, w.Hkv, w.S, w.Ev)
    if w.variant == "document":
        lens, total = [], 0
        while total < w.S:
            n = int(torch.randint(w.extra["doc_min"], w.extra["doc_max"] + 1, (1,), generator=g))
            n = min(n, w.S - total)
            lens.append(n)
            total += n
        ids = torch.repeat_interleave(torch.arange(len(lens), dtype=torch.int64), torch.tensor(lens))
        t["document_id"] = ids.unsqueeze(0).repeat(w.N, 1)
    if w.variant == "prefix":
        t["prefix_len"] = torch.randint(0, w.S // 2 + 1, (w.N,), generator=g, dtype=torch.int64)
    if pin and torch.cuda.is_available():
        t = {k: v.pin_memory() for k, v in t.items()}
    return t


def unmasked_pairs(w: Workload, t: Dict[str, torch.Tensor]) -> int:
    """Kept (query, key) pairs summed over batch and query heads (output heads for diff)."""
    S = w.S
    tri = S * (S + 1) // 2
    if w.variant == "vanilla":
        return w.N * w.Hq * S * S
    if w.variant in ("causal", "alibi", "softcap"):
        return w.N * w.Hq * (tri if w.causal else S * S)
    if w.variant == "sliding":
        win = w.extra["window"]
        per = sum(min(i + 1, win + 1) for i in range(S))
        return w.N * w.Hq * per
    if w.variant == "document":
        total = 0
        for n in range(w.N):
            cnt = torch.bincount(t["document_id"][n] - t["document_id"][n].min())
            cnt = cnt[cnt > 0].to(torch.int64)
            total += int((cnt * (cnt + 1) // 2).sum()) if w.causal else int((cnt * cnt).sum())
        return total * w.Hq
    if w.variant == "prefix":
        total = 0
        for p in t["prefix_len"].tolist():
            total += tri + (p * (p - 1) // 2 if p > 0 else 0)
        return total * w.Hq
    if w.variant == "evoformer":
        kept = torch.isfinite(t["mask_bias"].float()).sum(dim=-1).reshape(-1)  # per MSA row
        return int(kept.sum()) * S * w.Hq
    if w.variant == "diff":
        return w.N * (w.Hq // 2) * (tri if w.causal else S * S)
    raise KeyError(w.variant)


def effective_flops(w: Workload, t: Dict[str, torch.Tensor]) -> float:
    per_pair = 2 * w.E + 2 * w.Ev
    if w.variant == "diff":
        per_pair *= 2
    return float(unmasked_pairs(w, t)) * per_pair


def io_bytes(w: Workload, t: Dict[str, torch.Tensor]) -> int:
    """Bytes of q, k, v and every auxiliary input (the host->device traffic of one step)."""
    return sum(v.numel() * v.element_size() for v in t.values())


def hbm_bytes(w: Workload, t: Dict[str, torch.Tensor]) -> int:
    """Compulsory HBM traffic of one forward: every input read once, the result written once."""
    return io_bytes(w, t) + output_bytes(w)


def shard(w: Workload, t: Dict[str, torch.Tensor], rank: int, world: int):
    """Rank `rank`'s contiguous slice of the workload's independent units, as (workload, tensors).

    Units are the (batch, kv head) pairs in row-major order (MSA rows for Evoformer, (batch, output
    head) for differential attention): whole sequences when the batch divides over the ranks,
    otherwise a group of heads of one sequence.  Per-sequence inputs (document ids, prefix
    lengths, the pair bias) are replicated; ALiBi keeps its slopes through the head offset.  The
    slices are disjoint, cover every unit, and carry equal work for the benchmark configurations.
    """
    if world == 1:
        return w, t
    if w.variant == "evoformer":
        if w.N % world:
            raise ValueError(f"{w.N} MSA rows do not divide over {world} ranks")
        r0, r1 = rank * w.N // world, (rank + 1) * w.N // world
        out = {k: (v[:, r0:r1].contiguous() if v.size(1) == w.N else v) for k, v in t.items()}
        return w.scaled(N=r1 - r0), out
    if w.N % world == 0:
        n0, n1 = rank * w.N // world, (rank + 1) * w.N // world
        return w.scaled(N=n1 - n0), {k: v[n0:n1].contiguous() for k, v in t.items()}
    if world % w.N:
        raise ValueError(f"batch {w.N} and {world} ranks: neither divides the other")
    c = world // w.N                        # ranks per sequence
    b, j = rank // c, rank % c
    H_out = w.Hq // 2 if w.variant == "diff" else w.Hkv
    if H_out % c:
        raise ValueError(f"{H_out} heads do not divide over {c} ranks per sequence")
    hk = H_out // c                         # kv (or output) heads of this rank
    out: Dict[str, torch.Tensor] = {}
    if w.variant == "diff":
        H = w.Hq // 2
        sel = list(range(j * hk, (j + 1) * hk)) + list(range(H + j * hk, H + (j + 1) * hk))
        out["q"] = t["q"][b:b + 1, sel].contiguous()
        out["k"] = t["k"][b:b + 1, sel].contiguous()
        out["v"] = t["v"][b:b + 1, j * hk:(j + 1) * hk].contiguous()
        return w.scaled(N=1, Hq=2 * hk, Hkv=2 * hk), out
    G = w.Hq // w.Hkv
    out["q"] = t["q"][b:b + 1, j * hk * G:(j + 1) * hk * G].contiguous()
    out["k"] = t["k"][b:b + 1, j * hk:(j + 1) * hk].contiguous()
    out["v"] = t["v"][b:b + 1, j * hk:(j + 1) * hk].contiguous()
    for name in ("document_id", "prefix_len"):
        if name in t:
            out[name] = t[name][b:b + 1].contiguous()
    extra = dict(w.extra)
    if w.variant == "alibi":
        extra.update(alibi_heads=w.extra.get("alibi_heads", w.Hq),
                     alibi_head0=w.extra.get("alibi_head0", 0) + j * hk * G)
    return w.scaled(N=1, Hq=hk * G, Hkv=hk, extra=extra), out


def output_bytes(w: Workload) -> int:
    heads = w.Hq // 2 if w.variant == "diff" else w.Hq
    return w.N * heads * w.S * w.Ev * 2


def run(w: Workload, t: Dict[str, torch.Tensor]) -> torch.Tensor:
    """Call the variant API the way a user of the reference would."""
    q, k, v = t["q"], t["k"], t["v"]
    gqa = w.Hq != w.Hkv
    if w.variant == "vanilla":
        return av.attention_pytorch(q, k, v, enable_gqa=gqa)
    if w.variant == "causal":
        return av.attention_pytorch_causal(q, k, v, enable_gqa=gqa)
    if w.variant == "alibi":
        sm = av.AlibiScoreMod(w.extra.get("alibi_heads", w.Hq), head_offset=w.extra.get("alibi_head0", 0),
                              head_count=w.Hq)
        return av.attention_pytorch_alibi(q, k, v, score_mod=sm, is_causal=w.causal, enable_gqa=gqa)
    if w.variant == "softcap":
        return av.attention_softcapped(q, k, v, av.generate_tanh_softcap(w.extra["cap"]),
                                       is_causal=w.causal, enable_gqa=gqa)
    if w.variant == "sliding":
        return av.attention_pytorch_sliding_window(q, k, v, window_size=w.extra["window"], enable_gqa=gqa)
    if w.variant == "document":
        return av.attention_pytorch_document_mask(q, k, v, t["document_id"], enable_gqa=gqa,
                                                  is_causal=w.causal)
    if w.variant == "prefix":
        return av.attention_pytorch_prefix_lm(q, k, v, prefix_lengths=t["prefix_len"], enable_gqa=gqa)
    if w.variant == "evoformer":
        return av.attention_reference(q, k, v, [t["mask_bias"], t["pair_bias"]])
    if w.variant == "diff":
        return av.diffattn(q, k, v, lambda_full=w.extra["lambda"], is_causal=w.causal,
                           rms_norm=True, rms_eps=w.extra["rms_eps"])
    raise KeyError(w.variant)
