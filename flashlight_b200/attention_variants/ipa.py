"""Invariant point attention — the reference's fusion stress test (tests/test_ipa.py:57-125) lowered
onto the fused pair-bias kernel."""
from typing import Optional, Tuple

import torch

from .. import _lib
from ..ops import ipa_pack
from ._dispatch import run


def invariant_point_attention(
    q_scalar: torch.Tensor,  # [B, H, N, C]
    k_scalar: torch.Tensor,
    v_scalar: torch.Tensor,
    q_points: torch.Tensor,  # [B, H, N, P_qk, 4]
    k_points: torch.Tensor,
    v_points: torch.Tensor,  # [B, H, N, P_v, 4]
    pair_bias: torch.Tensor,  # [B, H, N, N]
    frames=None,
    mask: Optional[torch.Tensor] = None,
    c_hidden: int = 64,
    no_qk_points: int = 8,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax(q.k / sqrt(c_hidden) + w * sum_p |q_p - k_p|^2 + pair_bias) applied to the scalar and the
    point values, w = -0.5 sqrt(9 / (2 no_qk_points)) (tests/test_ipa.py:83-124).

    One launch of the pair-bias kernel behind one that assembles its operands (`flb200_ipa_pack`).  With
    a = w sqrt(c_hidden) the logits are
    (q.k + a |k_p|^2 - 2 a q_p.k_p) / sqrt(c_hidden) + bias + a row constant (w |q_p|^2, which the
    softmax cancels), so the squared distances become extra columns of the q/k operands:

        Q' = [ q | q_p | q_p | 1 | 1 ]      K' = [ k | hi(-2a k_p) | lo(-2a k_p) | hi(a |k_p|^2) | lo(a |k_p|^2) ]

    The key-side products are formed in fp32 and split into two bf16 terms, so the tensor cores see the
    fp32 value of every logit term to about 16 bits; the value operand is [ v | v_p ].  As in the
    reference function, `frames` and `mask` are accepted and not applied (test_ipa.py:86-88,110-111,124).
    Returns (scalar output [B, H, N, C], point output [B, N, H, P_v, 4]): the two aggregates of
    test_ipa.py:118-124, whose final sum does not broadcast for the test's own shapes.
    """
    if q_scalar.dim() != 4 or q_points.dim() != 5 or v_points.dim() != 5:
        raise ValueError("expected scalars [B, H, N, C] and points [B, H, N, P, 4]")
    B, H, N, C = q_scalar.shape
    Nk = k_scalar.size(2)
    if pair_bias.shape != (B, H, N, Nk):
        raise ValueError("pair_bias must be [B, H, N, N]")
    if q_points.shape[-2] != no_qk_points or k_points.shape[-2] != no_qk_points:
        raise ValueError("q_points / k_points must hold no_qk_points points")
    dt = torch.bfloat16
    if any(t.dtype != dt for t in (q_scalar, k_scalar, v_scalar, q_points, k_points, v_points, pair_bias)):
        raise NotImplementedError("invariant_point_attention: bfloat16 inputs only")
    if not q_scalar.is_cuda:
        raise NotImplementedError("invariant_point_attention: CUDA tensors only")
    scale = 1.0 / (c_hidden ** 0.5)
    a = -0.5 * (9.0 / (2 * no_qk_points)) ** 0.5 / scale
    q_aug, k_aug, v_aug = ipa_pack(q_scalar, k_scalar, v_scalar, q_points, k_points, v_points, a)
    Ev_real = C + v_points.size(-2) * v_points.size(-1)
    if max(q_aug.size(-1), v_aug.size(-1)) > 128:
        raise NotImplementedError("invariant_point_attention: operand width above 128 columns")
    bias = pair_bias if pair_bias.stride(-1) == 1 else pair_bias.contiguous()
    out = run(q_aug, k_aug, v_aug, scale=scale, score_mod=_lib.SCORE_BIAS, biases=[bias.unsqueeze(1), None],
              bias_inner=1)
    out_scalar = out[..., :C]
    out_points = out[..., C:Ev_real].reshape(B, H, N, v_points.size(-2), v_points.size(-1)).transpose(1, 2)
    return out_scalar, out_points
