"""The parity gate of the GPU tests: a bf16 kernel result against the fp32 oracle on the same
bf16-rounded inputs.

Gate (N(0,1) inputs): max-abs <= 2e-2 and mean-abs <= 2e-3, flat, over every element whose
reference value is below 4 in magnitude.  A bf16 result cannot meet a flat 2e-2 for larger values:
writing an exact fp32 value v as bf16 alone costs up to 2**-8 * |v| (1.6e-2 at |v| = 4, 3.1e-2 at
|v| = 8).  Such values are rare (rows that copy a single value row, steep ALiBi heads); they are
counted and held to |out - ref| <= 2e-2 + 2**-8 * |ref|, which stays inside the reference tests'
own atol 2e-2 + rtol 1e-2 (tests/test_vanilla.py:36 of the reference).
"""
import json
import os

import torch

MAX_ABS, MEAN_ABS, BIG = 2e-2, 2e-3, 4.0
TOTALS = {"elements": 0, "big": 0}


def stats(out: torch.Tensor, ref: torch.Tensor) -> dict:
    """Flat error figures of `out` against `ref` (both on one device; fp32 arithmetic)."""
    o, r = out.float(), ref.float().to(out.device)
    d = (o - r).abs()
    big = r.abs() >= BIG
    above = d > MAX_ABS
    n_above = int(above.sum())
    return {
        "elements": o.numel(),
        "finite": bool(torch.isfinite(o).all()),
        "max_abs": d.max().item(),
        "mean_abs": d.mean().item(),
        "max_abs_small": d[~big].max().item() if (~big).any() else 0.0,   # over |ref| < 4
        "n_big": int(big.sum()),                                         # elements with |ref| >= 4
        "big_excess": (d[big] - (MAX_ABS + 2.0 ** -8 * r[big].abs())).max().item() if big.any() else -1.0,
        "n_above_2e-2": n_above,
        "largest_ref_above_2e-2": r[above].abs().max().item() if n_above else 0.0,
    }


def check(out: torch.Tensor, ref: torch.Tensor, what="") -> dict:
    import flashlight_b200
    flashlight_b200.check_status()
    assert out.shape == ref.shape, (what, out.shape, ref.shape)
    assert out.dtype == torch.bfloat16
    s = stats(out, ref)
    TOTALS["elements"] += s["elements"]
    TOTALS["big"] += s["n_big"]
    assert s["finite"], what
    assert s["max_abs_small"] <= MAX_ABS, (what, s)          # the flat gate
    assert s["mean_abs"] <= MEAN_ABS, (what, s)
    assert s["big_excess"] <= 0, (what, s)                   # |ref| >= 4: rounding-aware band
    assert s["n_big"] <= max(8, s["elements"] // 2000), (what, s)   # and such values stay rare
    return s


def report(name: str, s: dict) -> None:
    """Print one line per benchmark configuration; FLB200_PARITY_REPORT=<file> also appends JSON."""
    print(f"[parity] {name}: max-abs {s['max_abs']:.3e} (|ref|<4: {s['max_abs_small']:.3e}) "
          f"mean-abs {s['mean_abs']:.3e} above-2e-2 {s['n_above_2e-2']} "
          f"(largest |ref| among them {s['largest_ref_above_2e-2']:.2f}) of {s['elements']}")
    path = os.environ.get("FLB200_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(dict(s, name=name)) + "\n")
