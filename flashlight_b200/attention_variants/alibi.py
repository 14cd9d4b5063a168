"""ALiBi attention — drop-in for `attention_variants/alibi.py`."""
import torch

from .. import _lib
from ._dispatch import default_scale, run


def alibi_bias(h, q_len, kv_len, device='cuda'):
    """bias[h, i, j] = 2^(-8 (h+1) / H) * (j - i), fp32 (attention_variants/alibi.py:5-9)."""
    slopes = torch.exp2(-((torch.arange(h, dtype=torch.int32, device=device) + 1) * 8.0 / h))
    rel = (torch.arange(kv_len, dtype=torch.int32, device=device)[None, :]
           - torch.arange(q_len, dtype=torch.int32, device=device)[:, None])
    return slopes[:, None, None] * rel


class AlibiScoreMod:
    """Callable with the reference's `score_mod(q_len, kv_len) -> [H, L, S]` contract
    (alibi.py:11,26) that also tells the kernel which closed form it stands for, so the
    bias tensor is never materialised on the fused path."""

    kind = "alibi"

    def __init__(self, nheads: int, device='cuda', head_offset: int = 0, head_count=None):
        self.nheads = int(nheads)
        self.device = device
        # a slice [head_offset, head_offset + head_count) of the heads, for callers that split the
        # heads of one model over several calls (or GPUs); the default is all of them
        self.head_offset = int(head_offset)
        self.head_count = self.nheads if head_count is None else int(head_count)

    def __call__(self, q_len, kv_len):
        bias = alibi_bias(self.nheads, q_len, kv_len, device=self.device)
        return bias[self.head_offset:self.head_offset + self.head_count]


def generate_alibi_bias_pytorch(nheads):
    return AlibiScoreMod(nheads)


def attention_pytorch_alibi(
        query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, score_mod=None,
        attn_mask=None, dropout_p=0.0, is_causal: bool = False, scale=None,
        enable_gqa=False) -> torch.Tensor:
    r"""softmax(Q K^T * scale + alibi) V (attention_variants/alibi.py:13-33).

    `score_mod` must come from :func:`generate_alibi_bias_pytorch`; an arbitrary callable
    cannot be compiled into the kernel and raises NotImplementedError.  None selects the
    standard slopes for the query head count.  The reference ignores `is_causal`
    (alibi.py:15); here True additionally applies the causal mask, False reproduces the
    reference.  `attn_mask` and `dropout_p` are ignored as in the reference.
    """
    if score_mod is None:
        score_mod = AlibiScoreMod(query.size(1))
    if getattr(score_mod, "kind", None) != "alibi":
        raise NotImplementedError(
            "score_mod must be built by generate_alibi_bias_pytorch(); arbitrary callables "
            "cannot run inside the fused kernel and there is no fallback")
    if score_mod.head_count != query.size(1):
        # the reference adds a [nheads, L, S] bias to [N, Hq, L, S] scores (alibi.py:27-29): any
        # other head count fails to broadcast there
        raise ValueError(f"ALiBi bias built for {score_mod.head_count} heads, query has {query.size(1)}")
    return run(query, key, value, scale=default_scale(query, scale), enable_gqa=enable_gqa,
               gqa_5d=True, score_mod=_lib.SCORE_ALIBI, alibi_heads=score_mod.nheads, alibi_head0=score_mod.head_offset,
               mask=_lib.MASK_CAUSAL if is_causal else _lib.MASK_NONE)
