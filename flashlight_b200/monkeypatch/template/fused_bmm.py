"""Back-to-back matrix product `(f(A @ B)) @ C` — the counterpart of the reference's Triton template
`monkeypatch/template/fused_bmm.py:332-422`, which Inductor substitutes for `bmm(subgraph(bmm(a, b)), c)`.

Here the fusion is explicit: one call runs both products in the attention kernel's pipeline with its
softmax replaced by the pointwise function; the intermediate `A @ B` never leaves tensor memory and is
rounded to bf16 before the second product, as the template does (`fused_bmm.py:404`).
"""
import torch

from ...ops import product_chain


def fused_bmm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, pointwise: str = "identity",
              scale: float = 1.0) -> torch.Tensor:
    """`f((a @ b) * scale) @ c` for bf16 a [*, M, N], b [*, N, O], c [*, O, P] with N, P <= 128.

    pointwise: "identity" (the reference's own test, `bmm(bmm(a, b), c)`), "relu", "tanh" or "sigmoid".
    Leading batch dimensions are flattened.  Raises NotImplementedError for shapes no kernel serves
    (inner widths above 128); there is no unfused fallback.
    """
    lead = a.shape[:-2]
    a3, b3, c3 = (t.reshape(-1, t.size(-2), t.size(-1)) if t.dim() != 3 else t for t in (a, b, c))
    out = product_chain(a3, b3, c3, float(scale), pointwise)
    return out.reshape(*lead, out.size(-2), out.size(-1))
