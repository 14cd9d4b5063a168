"""CPU oracle: fp32 restatement of the reference's eager attention variants.

TEST INFRASTRUCTURE ONLY.  Nothing in the product path (`flashlight_b200/`) may import
this module; it is used by `tests/`, by `__graft_entry__.smoke()` as the checker and by
`bench.py` for the CPU baseline legs.

Every function follows the eager PyTorch code of bozhiyou/flashlight
(`attention_variants/*.py`, cited per function) and is pinned against outputs of that
code: `tests/golden/make_golden.py` imports the reference itself, runs it on seeded
inputs and stores the results, and `tests/test_oracle_golden.py` checks this module
against those files.  Where the benchmark configurations extend the reference (causal
ALiBi / softcap / document mask, per-sequence prefix lengths, causal + RMS-normalised
differential attention) the extension is restated here and marked as such; those parts
have no reference output to pin against.

All arithmetic is fp32 (or fp64 with `dtype=torch.float64`) on whatever device the
inputs live on; scores are processed per (batch, kv head, row chunk) so the L x S score
block stays small.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Union

import torch

NEG_INF = float("-inf")
FILL_1E10 = -1e10  # the reference's fill value outside causal.py (sliding_window.py:40 etc.)


def _scale(q: torch.Tensor, scale) -> float:
    # vanilla.py:14: 1/sqrt(E) unless given
    return 1.0 / math.sqrt(q.size(-1)) if scale is None else float(scale)


def _attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
            score_mod: Optional[Callable] = None, mask: Optional[Callable] = None,
            fill: float = NEG_INF, row_chunk: int = 4096,
            dtype: torch.dtype = torch.float32, return_lse: bool = False):
    """softmax(where(mask, fill, score_mod(q k^T * scale))) v, chunked.

    q [N,Hq,L,E], k [N,Hkv,S,E], v [N,Hkv,S,Ev]; query head h reads kv head h // G, the
    grouping of `query.view(N, Hkv, -1, L, E)` (causal.py:28).
    score_mod(s, n, h0, h1, l0, l1) gets scores [h1-h0, l1-l0, S] of query heads h0..h1.
    mask(n, l0, l1) returns bool [l1-l0, S], True = masked out.
    Returns [N, Hq, L, Ev]; with `return_lse` also the natural-log sum of exp over the keys of
    every row, [N, Hq, L] (what a backward pass would take from the forward).
    """
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    N, Hq, L, E = q.shape
    Hkv, S, Ev = k.size(1), k.size(2), v.size(3)
    G = Hq // Hkv
    out = torch.empty((N, Hq, L, Ev), dtype=dtype, device=q.device)
    lse = torch.empty((N, Hq, L), dtype=dtype, device=q.device) if return_lse else None
    # all heads of one sequence at a time; rows chunked so a score block stays below ~1 GiB
    budget = (1 << 30) // (q.element_size() * Hq * S)
    row_chunk = max(16, min(row_chunk if row_chunk else L, L, budget))
    for n in range(N):
        kt = k[n].transpose(1, 2).unsqueeze(1)          # [Hkv, 1, E, S]
        vn = v[n].unsqueeze(1)                           # [Hkv, 1, S, Ev]
        for l0 in range(0, L, row_chunk):
            l1 = min(L, l0 + row_chunk)
            qs = q[n, :, l0:l1].view(Hkv, G, l1 - l0, E)
            s = (torch.matmul(qs, kt) * scale).view(Hq, l1 - l0, S)
            if score_mod is not None:
                s = score_mod(s, n, 0, Hq, l0, l1)
            if mask is not None:
                s = torch.where(mask(n, l0, l1), torch.tensor(fill, dtype=dtype, device=s.device), s)
            p = torch.softmax(s, dim=-1).view(Hkv, G, l1 - l0, S)
            out[n, :, l0:l1] = torch.matmul(p, vn).view(Hq, l1 - l0, Ev)
            if return_lse:
                lse[n, :, l0:l1] = torch.logsumexp(s, dim=-1)
    return (out, lse) if return_lse else out


def _gqa_view(out: torch.Tensor, Hkv: int, enable_gqa: bool) -> torch.Tensor:
    # every variant but vanilla keeps the grouped 5-D result (causal.py:28,36)
    if not enable_gqa:
        return out
    N, Hq, L, Ev = out.shape
    return out.view(N, Hkv, Hq // Hkv, L, Ev)


def _causal_mask_fn(L: int, S: int, device) -> Callable:
    # causal.py:32: triu(ones(L, S), diagonal=1) -> masked iff j > i
    j = torch.arange(S, device=device).view(1, S)

    def fn(n, l0, l1):
        i = torch.arange(l0, l1, device=device).view(-1, 1)
        return j > i
    return fn


def vanilla(query, key, value, scale=None, enable_gqa=False, **kw):
    """attention_pytorch / attention_pytorch_nogqa (vanilla.py:4-35); 4-D result."""
    return _attend(query, key, value, _scale(query, scale), **kw)


def causal(query, key, value, scale=None, enable_gqa=False, **kw):
    """attention_pytorch_causal (causal.py:25-36): -inf above the diagonal."""
    L, S = query.size(-2), key.size(-2)
    out = _attend(query, key, value, _scale(query, scale),
                  mask=_causal_mask_fn(L, S, query.device), fill=NEG_INF, **kw)
    return _gqa_view(out, key.size(1), enable_gqa)


def alibi_slopes(nheads: int, device, dtype=torch.float32) -> torch.Tensor:
    # alibi.py:6-7: exp2(-((arange(h) + 1) * 8.0 / h))
    return torch.exp2(-((torch.arange(nheads, dtype=torch.int32, device=device) + 1) * 8.0 / nheads)).to(dtype)


def alibi(query, key, value, nheads=None, is_causal=False, scale=None, enable_gqa=False, head_offset=0, **kw):
    """attention_pytorch_alibi (alibi.py:13-33): score * scale + slope_h * (j - i).

    The slope index is the query head (alibi.py:27-28 views the bias as (Hkv, G, L, S)).
    `is_causal=True` is an extension: the reference ignores the flag (alibi.py:15); here it
    composes the causal mask of causal.py:32-33.
    """
    L, S = query.size(-2), key.size(-2)
    H = query.size(1) if nheads is None else nheads
    dtype = kw.get("dtype", torch.float32)
    # `head_offset`: the query holds heads [head_offset, head_offset + Hq) of the H heads (a slice
    # of the reference's [H, L, S] bias, for workloads whose heads are split over several GPUs)
    slopes = alibi_slopes(H, query.device, dtype)[head_offset:]
    j = torch.arange(S, device=query.device, dtype=torch.int32).view(1, 1, S)

    def mod(s, n, h0, h1, l0, l1):
        i = torch.arange(l0, l1, device=s.device, dtype=torch.int32).view(1, -1, 1)
        return s + slopes[h0:h1].view(-1, 1, 1) * (j - i)

    out = _attend(query, key, value, _scale(query, scale), score_mod=mod,
                  mask=_causal_mask_fn(L, S, query.device) if is_causal else None, **kw)
    return _gqa_view(out, key.size(1), enable_gqa)


def softcap(query, key, value, cap: float, is_causal=False, scale=None, enable_gqa=False, **kw):
    """attention_softcapped (softcap.py:36-53) with score_mod = cap * tanh(score / cap), the
    formula of the callable the reference's benchmark passes (run_flex_variants.py:133;
    attn-gym itself is not available here, so this formula is the restatement).
    `is_causal=True` is an extension as for ALiBi.
    """
    L, S = query.size(-2), key.size(-2)

    def mod(s, n, h0, h1, l0, l1):
        return cap * torch.tanh(s / cap)

    out = _attend(query, key, value, _scale(query, scale), score_mod=mod,
                  mask=_causal_mask_fn(L, S, query.device) if is_causal else None, **kw)
    return _gqa_view(out, key.size(1), enable_gqa)


def sliding_window(query, key, value, window_size=1024, scale=None, enable_gqa=False, **kw):
    """attention_pytorch_sliding_window (sliding_window.py:4-44): masked iff i < j or
    i - j > window (so window + 1 keys are kept), fill -1e10."""
    L = query.size(-2)
    assert L == key.size(-2)
    j = torch.arange(L, device=query.device).view(1, L)

    def m(n, l0, l1):
        i = torch.arange(l0, l1, device=query.device).view(-1, 1)
        return (i < j) | ((i - j) > window_size)

    out = _attend(query, key, value, _scale(query, scale), mask=m, fill=FILL_1E10, **kw)
    return _gqa_view(out, key.size(1), enable_gqa)


def document_mask(query, key, value, document_id, is_causal=False, scale=None, enable_gqa=False, **kw):
    """attention_pytorch_document_mask (document_mask.py:22-41): masked iff the ids differ,
    fill -1e10.  `is_causal=True` (extension) also masks j > i."""
    L = query.size(-2)
    doc = document_id.to(query.device)
    j = torch.arange(L, device=query.device).view(1, L)

    def m(n, l0, l1):
        mm = doc[n, l0:l1].view(-1, 1) != doc[n].view(1, -1)
        if is_causal:
            mm = mm | (j > torch.arange(l0, l1, device=query.device).view(-1, 1))
        return mm

    out = _attend(query, key, value, _scale(query, scale), mask=m, fill=FILL_1E10, **kw)
    return _gqa_view(out, key.size(1), enable_gqa)


def prefix_lm(query, key, value, prefix_lengths: Union[int, torch.Tensor] = 256, scale=None,
              enable_gqa=False, **kw):
    """attention_pytorch_prefix_lm (prefix_lm.py:5-42): masked iff j > max(prefix - 1, i),
    fill -1e10.  The reference takes one int for the whole batch (prefix_lm.py:34); a tensor
    with one length per sequence is the extension the benchmark configuration needs."""
    B, L = query.size(0), query.size(-2)
    if torch.is_tensor(prefix_lengths):
        pl = prefix_lengths.to(device=query.device, dtype=torch.long).view(B)
    else:
        pl = torch.full((B,), int(prefix_lengths), dtype=torch.long, device=query.device)
    j = torch.arange(L, device=query.device).view(1, L)

    def m(n, l0, l1):
        i = torch.arange(l0, l1, device=query.device).view(-1, 1)
        return j > torch.maximum(pl[n] - 1, i)

    out = _attend(query, key, value, _scale(query, scale), mask=m, fill=FILL_1E10, **kw)
    return _gqa_view(out, key.size(1), enable_gqa)


def diffattn(q, k, v, scale=None, lambda_full=0.2, is_causal=False, rms_norm=False, rms_eps=1e-5, **kw):
    """diffattn (diff_attn.py:6-30): heads [0,H) and [H,2H) of q/k are the two branches;
    softmax(q0 k0^T s) v - lambda * softmax(q1 k1^T s) v.

    Extensions (the benchmark configuration, not in the reference): `is_causal` masks both
    branches as causal.py:32-33; `rms_norm` then applies x * rsqrt(mean(x^2, -1) + rms_eps)
    per head with no learnable weight.
    """
    H = q.size(1) // 2
    L, S = q.size(-2), k.size(-2)
    sc = _scale(q, scale)
    m = _causal_mask_fn(L, S, q.device) if is_causal else None
    a0 = _attend(q[:, :H], k[:, :H], v, sc, mask=m, **kw)
    a1 = _attend(q[:, H:], k[:, H:], v, sc, mask=m, **kw)
    out = a0 - lambda_full * a1
    if rms_norm:
        out = out * torch.rsqrt(out.pow(2).mean(dim=-1, keepdim=True) + rms_eps)
    return out


def evoformer(q_input, k_input, v_input, biases: Sequence[torch.Tensor], sm_scale=None,
              dtype=torch.float32, **kw):
    """attention_reference (evoformer.py:8-36): inputs [*, S, H, D]; scores get every bias
    added (broadcast to [*, H, S, S]); result [*, S, H, D]."""
    lead = q_input.shape[:-3]
    S, H, D = q_input.shape[-3:]
    Sk = k_input.size(-3)
    n = 1
    for d in lead:
        n *= d
    q = q_input.reshape(n, S, H, D).transpose(1, 2)
    k = k_input.reshape(n, Sk, H, D).transpose(1, 2)
    v = v_input.reshape(n, Sk, H, v_input.size(-1)).transpose(1, 2)
    # keep the biases as broadcast views; index them with the unravelled leading index
    bs = [b.to(dtype).expand(*lead, H, S, Sk) for b in biases]

    def mod(s, ni, h0, h1, l0, l1):
        idx = []
        for d in reversed(lead):
            idx.append(ni % d)
            ni //= d
        idx = tuple(reversed(idx))
        for b in bs:
            s = s + b[idx][h0:h1, l0:l1]
        return s

    out = _attend(q, k, v, _scale(q, sm_scale), score_mod=mod, dtype=dtype, **kw)
    return out.transpose(1, 2).reshape(*lead, S, H, out.size(-1))


def product_chain(a, b, c, pointwise: str = "identity", scale: float = 1.0, dtype=torch.float32):
    """(f((a @ b) * scale)) @ c with the intermediate rounded to bf16 before the second product, as the
    reference's fused template does (monkeypatch/template/fused_bmm.py:398-404: `acc_ab` through the
    pointwise subgraph, `.to(c.type.element_ty)`, second `tl.dot`); its own test is the identity case
    `torch.bmm(torch.bmm(a, b), c)` (fused_bmm.py:433-434).  Both products accumulate in `dtype`."""
    f = {"identity": lambda x: x, "relu": torch.relu, "tanh": torch.tanh, "sigmoid": torch.sigmoid}[pointwise]
    mid = f(torch.matmul(a.to(dtype), b.to(dtype)) * scale)
    mid = mid.to(torch.bfloat16).to(dtype)
    return torch.matmul(mid, c.to(dtype))


def invariant_point_attention(q_scalar, k_scalar, v_scalar, q_points, k_points, v_points, pair_bias,
                              c_hidden: int = 64, no_qk_points: int = 8, dtype=torch.float32):
    """Invariant point attention as the reference's fusion test states it (tests/test_ipa.py:57-125).

    Scalars are [B, H, N, C], points [B, H, N, P, 4], the pair bias [B, H, N, N].  The logits are
    q.k / sqrt(c_hidden) + w * sum_p |q_p - k_p|^2 + bias with w = -0.5 sqrt(9 / (2 no_qk_points))
    (test_ipa.py:83-108); the frame transforms and the residue mask are commented out there
    (test_ipa.py:86-88,110-111,124) and are therefore not applied here either.  Returns the two
    aggregates of test_ipa.py:118-124: the scalar output [B, H, N, C] and the point output in the
    einsum's order [B, N, H, P_v, 4].  The reference's last line adds the two, which broadcasts only
    for contrived shapes (C == 4, B == 1, N == P_v); the golden fixture uses such a shape with one of
    the two value operands zeroed to read each aggregate out of the unmodified function.
    """
    q, k, v = (t.to(dtype) for t in (q_scalar, k_scalar, v_scalar))
    qp, kp, vp = (t.to(dtype) for t in (q_points, k_points, v_points))
    content = (q / (c_hidden ** 0.5)) @ k.transpose(-1, -2)
    dist_sq = ((qp.unsqueeze(3) - kp.unsqueeze(2)) ** 2).sum(dim=-1)  # [B, H, N, N, P]
    w = -0.5 * (9.0 / (2 * no_qk_points)) ** 0.5
    logits = content + dist_sq.sum(dim=-1) * w + pair_bias.to(dtype)
    a = torch.softmax(logits, dim=-1)
    out_scalar = a @ v
    out_points = torch.einsum("...hij,...hjpv->...ihpv", a, vp)
    return out_scalar, out_points
