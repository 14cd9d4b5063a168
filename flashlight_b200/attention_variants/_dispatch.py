"""Shared plumbing of the variant functions: argument normalisation, GQA shape
conventions and staging of host tensors through the device.

Tensors that live in host memory are copied to the current CUDA device, the
kernel runs there, and the result is copied back: the arithmetic never runs on
the CPU.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from .. import _lib
from ..ops import attn_fwd


def default_scale(query: torch.Tensor, scale) -> float:
    return 1.0 / math.sqrt(query.size(-1)) if scale is None else float(scale)


def _dev(t: Optional[torch.Tensor], device: torch.device) -> Optional[torch.Tensor]:
    if t is None or t.device == device:
        return t
    return t.to(device, non_blocking=t.is_pinned() if t.device.type == "cpu" else False)


_SIDE_STREAMS: dict = {}


def _side_streams(device: torch.device):
    key = device.index
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = [torch.cuda.Stream(device=device) for _ in range(3)]
    return _SIDE_STREAMS[key]


def _run_host_pipelined(query, key, value, device, args_for, n_chunks: int) -> torch.Tensor:
    """Host tensors in pinned memory: split the batch into chunks and run copy-in, kernel and
    copy-out of successive chunks on three streams, so that the two PCIe directions and the
    kernel overlap.  `args_for(n0, n1)` yields the per-chunk arguments after q, k, v."""
    N = query.size(0)
    bounds = [N * c // n_chunks for c in range(n_chunks + 1)]
    streams = _side_streams(device)
    ready = torch.cuda.Event()
    ready.record(torch.cuda.current_stream(device))
    host = None
    for c in range(n_chunks):
        n0, n1 = bounds[c], bounds[c + 1]
        if n1 == n0:
            continue
        st = streams[c % len(streams)]
        with torch.cuda.stream(st):
            st.wait_event(ready)
            q = query[n0:n1].to(device, non_blocking=True)
            k = key[n0:n1].to(device, non_blocking=True)
            v = value[n0:n1].to(device, non_blocking=True)
            out = attn_fwd(q, k, v, *args_for(n0, n1))
            if host is None:
                host = torch.empty((N,) + tuple(out.shape[1:]), dtype=out.dtype, device="cpu", pin_memory=True)
            host[n0:n1].copy_(out, non_blocking=True)
    for st in streams:
        st.synchronize()
    return host


def run(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, *, scale: float,
        enable_gqa: bool = False, gqa_5d: bool = False,
        score_mod: int = _lib.SCORE_NONE, alibi_heads: int = 0, alibi_head0: int = 0, softcap: float = 0.0,
        mask: int = _lib.MASK_NONE, causal: bool = False, window: int = 0,
        prefix_len: Optional[torch.Tensor] = None, prefix_scalar: int = 0,
        document_id: Optional[torch.Tensor] = None,
        biases: Sequence[Optional[torch.Tensor]] = (None, None), bias_inner: int = 1,
        diff: bool = False, diff_lambda: float = 0.0, diff_rms_norm: bool = False,
        diff_rms_eps: float = 0.0, rows_major_out: bool = False) -> torch.Tensor:
    """Run one fused forward; q/k/v are 4-D [N, H, L, E] views."""
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
        raise ValueError("expected 4-D query/key/value of shape (N, H, L, E)")
    Hq, Hkv = query.size(1), key.size(1)
    if not diff:
        if enable_gqa:
            if Hq % Hkv != 0:
                raise ValueError("enable_gqa: the number of query heads must be a multiple of the kv heads")
        elif Hq != Hkv:
            raise ValueError("query and key/value head counts differ; pass enable_gqa=True")
    home = query.device
    if home.type == "cuda":
        device = home
    else:
        if not torch.cuda.is_available():
            raise RuntimeError("flashlight_b200 needs a CUDA device (sm_100); there is no CPU implementation")
        device = torch.device("cuda", torch.cuda.current_device())
    b0, b1 = (_dev(b, device) for b in biases)
    N = query.size(0)
    if (home.type != "cuda" and N >= 2 and b0 is None and b1 is None and not rows_major_out
            and query.is_pinned() and key.is_pinned() and value.is_pinned()
            and query.numel() * query.element_size() >= (8 << 20)):
        pl_dev, doc_dev = _dev(prefix_len, device), _dev(document_id, device)

        def args_for(n0, n1):
            return (float(scale), int(score_mod), int(alibi_heads), int(alibi_head0), float(softcap), int(mask),
                    bool(causal),
                    int(window), None if pl_dev is None else pl_dev[n0:n1], int(prefix_scalar),
                    None if doc_dev is None else doc_dev[n0:n1], None, None, int(bias_inner),
                    bool(diff), float(diff_lambda), bool(diff_rms_norm), float(diff_rms_eps), False)

        out = _run_host_pipelined(query, key, value, device, args_for, min(N, 8))
        if enable_gqa and gqa_5d and not diff:
            out = out.view(out.size(0), Hkv, Hq // Hkv, out.size(2), out.size(3))
        return out
    q, k, v = _dev(query, device), _dev(key, device), _dev(value, device)
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        # gradients: plain and causal attention have backward kernels (the reference stubs its backward)
        plain = (score_mod == _lib.SCORE_NONE and mask in (_lib.MASK_NONE, _lib.MASK_CAUSAL) and not diff
                 and b0 is None and b1 is None and not rows_major_out and home.type == "cuda"
                 and q.size(3) == v.size(3) and q.size(3) <= 128)
        if not plain:
            raise NotImplementedError("flashlight_b200: gradients are implemented for plain and causal attention "
                                      "(equal q/k and v head dims up to 128); no other variant has a backward kernel")
        from ..ops import attention_with_grad
        out = attention_with_grad(q, k, v, float(scale), mask == _lib.MASK_CAUSAL)
        if enable_gqa and gqa_5d:
            out = out.view(out.size(0), Hkv, Hq // Hkv, out.size(2), out.size(3))
        return out
    out = attn_fwd(q, k, v, float(scale), int(score_mod), int(alibi_heads), int(alibi_head0), float(softcap),
                   int(mask), bool(causal), int(window), _dev(prefix_len, device),
                   int(prefix_scalar), _dev(document_id, device), b0, b1, int(bias_inner),
                   bool(diff), float(diff_lambda), bool(diff_rms_norm), float(diff_rms_eps),
                   bool(rows_major_out))
    if enable_gqa and gqa_5d and not diff:
        # the eager functions keep the (kv head, group) split in their result (causal.py:28,36)
        out = out.view(out.size(0), Hkv, Hq // Hkv, out.size(2), out.size(3))
    if home.type != "cuda":
        # result goes back through pinned memory (cached by torch's host allocator)
        host = torch.empty(out.shape, dtype=out.dtype, device="cpu", pin_memory=True)
        host.copy_(out, non_blocking=True)
        torch.cuda.current_stream(device).synchronize()
        out = host
    return out
