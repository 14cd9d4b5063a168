"""Run a named workload (see `flashlight_b200/workloads.py` for shapes and generators)
through the CPU oracle.  TEST INFRASTRUCTURE ONLY: imported by tests/, smoke() and the CPU
baseline legs of bench.py, never by the product path."""
from __future__ import annotations

import time
from typing import Dict

import torch

from . import attention_oracle as ao


def run_oracle(w, t: Dict[str, torch.Tensor], dtype=torch.float32) -> torch.Tensor:
    """fp32 oracle result for workload `w` on inputs `t`, in the shape the variant API returns."""
    q, k, v = t["q"], t["k"], t["v"]
    gqa = w.Hq != w.Hkv
    kw = dict(dtype=dtype)
    if w.variant == "vanilla":
        return ao.vanilla(q, k, v, enable_gqa=gqa, **kw)
    if w.variant == "causal":
        return ao.causal(q, k, v, enable_gqa=gqa, **kw)
    if w.variant == "alibi":
        return ao.alibi(q, k, v, nheads=w.extra.get("alibi_heads", w.Hq), is_causal=w.causal, enable_gqa=gqa,
                        head_offset=w.extra.get("alibi_head0", 0), **kw)
    if w.variant == "softcap":
        return ao.softcap(q, k, v, w.extra["cap"], is_causal=w.causal, enable_gqa=gqa, **kw)
    if w.variant == "sliding":
        return ao.sliding_window(q, k, v, window_size=w.extra["window"], enable_gqa=gqa, **kw)
    if w.variant == "document":
        return ao.document_mask(q, k, v, t["document_id"], is_causal=w.causal, enable_gqa=gqa, **kw)
    if w.variant == "prefix":
        return ao.prefix_lm(q, k, v, prefix_lengths=t["prefix_len"], enable_gqa=gqa, **kw)
    if w.variant == "evoformer":
        return ao.evoformer(q, k, v, [t["mask_bias"], t["pair_bias"]], **kw)
    if w.variant == "diff":
        return ao.diffattn(q, k, v, lambda_full=w.extra["lambda"], is_causal=w.causal, rms_norm=True,
                           rms_eps=w.extra["rms_eps"], **kw)
    raise KeyError(w.variant)


def reference_runner(w):
    """The reference's OWN eager function for workload `w`, or None.

    `oracle/build_ref.py` compiles the reference's `attention_variants/*.py` (where its checkout is
    mounted) into an archive of sourceless modules under `oracle/_ref/`; they are imported from it.  Only
    workloads the reference's functions compute as they stand qualify (fp32 on the host, as the
    reference's tests run them): the benchmark configurations that add a causal mask to ALiBi,
    softcap or the document mask, tensor prefix lengths, or RMS-normalised differential attention
    have no reference function, and the caller falls back to the restatement in this package.
    """
    import importlib
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent / "_ref" / "attention_variants.bin"
    if not root.exists():
        return None
    if w.variant not in ("vanilla", "causal", "sliding", "evoformer"):
        return None
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    try:
        mod = importlib.import_module("attention_variants." + {
            "vanilla": "vanilla", "causal": "causal", "sliding": "sliding_window", "evoformer": "evoformer"}[w.variant])
    except Exception:
        return None

    def run(w, t):
        q, k, v = (t[n].float() for n in ("q", "k", "v"))
        gqa = w.Hq != w.Hkv
        if w.variant == "vanilla":
            return mod.attention_pytorch(q, k, v, enable_gqa=gqa)
        if w.variant == "causal":
            return mod.attention_pytorch_causal(q, k, v, enable_gqa=gqa)
        if w.variant == "sliding":
            return mod.attention_pytorch_sliding_window(q, k, v, window_size=w.extra["window"], enable_gqa=gqa)
        return mod.attention_reference(q, k, v, [t["mask_bias"].float(), t["pair_bias"].float()])

    return run


def time_oracle(w, t: Dict[str, torch.Tensor], reps: int = 1) -> float:
    """Median wall seconds of the oracle on the host cores (all torch threads)."""
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        run_oracle(w, t)
        times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2]
