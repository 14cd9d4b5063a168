"""`torch.ops.flb200.attn_fwd`: the one custom op every variant function lowers to.

The op takes the tensors exactly as the reference's eager functions see them
(any strides, no copies), fills the C parameter block and enqueues the sm_100a
kernel on the current CUDA stream through the C ABI.  It is registered with a
fake (meta) implementation so `torch.compile(fn)` around a variant function
traces it as a single opaque node, as `torch.compile` did for the reference's
generated Triton kernel (tests/test_causal.py:33).

There is no fallback: non-CUDA-resident work, other dtypes and shapes without a
kernel raise.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib

_STATUS: dict[int, torch.Tensor] = {}
_STATUS_HOST: dict[int, torch.Tensor] = {}
_MAP_CACHE: dict[tuple, tuple] = {}
_MAP_CACHE_MAX = 8


def _raise_for(code: int, what: str) -> None:
    msg = f"flb200 {what}: {_lib.strerror(code)}"
    if code == _lib.E_UNSUPPORTED:
        raise NotImplementedError(msg)
    if code in (_lib.E_BAD_ARG, _lib.E_MISALIGNED, _lib.E_WORKSPACE):
        raise ValueError(msg)
    raise RuntimeError(msg)


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _STATUS.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _STATUS[idx] = t
    return t


def _status_mirror(device: torch.device) -> torch.Tensor:
    """Pinned host copy of the status word: a kernel that gives up also stores the word here, so
    the next call on the device sees it without synchronising."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _STATUS_HOST.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32).pin_memory()
        _STATUS_HOST[idx] = t
    return t


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if a device-side bounded wait expired since the last check."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    t = _status_word(device)
    word = int(t.item())
    if word != 0:
        t.zero_()
        _status_mirror(device).zero_()
        bar, blk = C.c_int32(0), C.c_int32(0)
        code = _lib.load().flb200_decode_status(word, C.byref(bar), C.byref(blk))
        raise RuntimeError(
            f"flb200 kernel reported {_lib.strerror(code)} (barrier {bar.value}, block {blk.value})")


def launch_count() -> int:
    """Kernels launched by the library since it was loaded."""
    return int(_lib.load().flb200_launch_count())


def _strides3(t: torch.Tensor) -> tuple[int, int, int]:
    if t.stride(3) != 1:
        raise ValueError("flb200: the feature axis must be contiguous")
    return (t.stride(0), t.stride(1), t.stride(2))


def _fill_bias(p: _lib.AttnParams, slot: int, b: Optional[torch.Tensor], keep: list) -> None:
    if b is None:
        p.bias[slot] = None
        return
    if b.dim() != 5:
        raise ValueError("flb200: a bias must be 5-D [b, r, h, L, S] (broadcast by expand)")
    if b.dtype != torch.bfloat16:
        raise NotImplementedError("flb200: biases must be bfloat16")
    if b.size(4) > 1 and b.stride(4) == 0:
        # broadcast along the keys (evoformer.py:26-27 accepts it): write that axis out, keeping the
        # zero strides of every other broadcast axis
        core = b[tuple(slice(0, 1) if b.stride(i) == 0 else slice(None) for i in range(5))]
        b = core.expand(core.shape[:4] + (b.size(4),)).contiguous().expand(b.shape)
    if b.stride(4) != 1 and b.size(4) != 1:
        raise ValueError("flb200: the key axis of a bias must be contiguous")
    keep.append(b)
    p.bias[slot] = b.data_ptr()
    for i in range(4):
        p.bias_stride[slot][i] = b.stride(i) if b.size(i) > 1 else 0


@torch.library.custom_op("flb200::attn_fwd", mutates_args=())
def attn_fwd(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
    score_mod: int, alibi_heads: int, alibi_head0: int, softcap: float,
    mask: int, causal: bool, window: int,
    prefix_len: Optional[torch.Tensor], prefix_scalar: int,
    document_id: Optional[torch.Tensor],
    bias0: Optional[torch.Tensor], bias1: Optional[torch.Tensor], bias_inner: int,
    diff: bool, diff_lambda: float, diff_rms_norm: bool, diff_rms_eps: float,
    rows_major_out: bool,
) -> torch.Tensor:
    """q [N,Hq,L,E], k [N,Hkv,S,E], v [N,Hv,S,Ev] (views with any batch/head/row strides).

    Returns [N,Ho,L,Ev]; with `rows_major_out` the storage order is [N,L,Ho,Ev] (the
    Evoformer layout) and the returned tensor is the transposed view of it.
    """
    return _attn_fwd_impl(q, k, v, scale, score_mod, alibi_heads, alibi_head0, softcap, mask, causal, window,
                          prefix_len, prefix_scalar, document_id, bias0, bias1, bias_inner,
                          diff, diff_lambda, diff_rms_norm, diff_rms_eps, rows_major_out, None)


def attn_fwd_lse(q, k, v, scale, *, score_mod=_lib.SCORE_NONE, alibi_heads=0, alibi_head0=0, softcap=0.0,
                 mask=_lib.MASK_NONE, causal=False, window=0, prefix_len=None, prefix_scalar=0,
                 document_id=None, bias0=None, bias1=None, bias_inner=1):
    """Forward pass that also returns the log-sum-exp of every query row, fp32 [N, Hq, L] (what a
    backward pass needs from the forward; the reference stubs its backward).  Same arguments as
    the `flb200::attn_fwd` op without the differential / layout options; not traceable by
    `torch.compile`."""
    lse = torch.empty((q.size(0), q.size(1), q.size(2)), dtype=torch.float32, device=q.device)
    o = _attn_fwd_impl(q, k, v, scale, score_mod, alibi_heads, alibi_head0, softcap, mask, causal, window,
                       prefix_len, prefix_scalar, document_id, bias0, bias1, bias_inner,
                       False, 0.0, False, 0.0, False, lse)
    return o, lse


def _attn_fwd_impl(q, k, v, scale, score_mod, alibi_heads, alibi_head0, softcap, mask, causal, window,
                   prefix_len, prefix_scalar, document_id, bias0, bias1, bias_inner,
                   diff, diff_lambda, diff_rms_norm, diff_rms_eps, rows_major_out, lse):
    lib = _lib.load()
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("flb200: tensors must live on a CUDA device (there is no CPU path)")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise NotImplementedError("flb200: only bfloat16 inputs are supported")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("flb200: q, k, v must be 4-D [N, H, L, E]")
    N, Hq, L, E = q.shape
    Hkv, S = k.size(1), k.size(2)
    Ev = v.size(3)
    if k.size(0) != N or v.size(0) != N or k.size(3) != E or v.size(2) != S:
        raise ValueError("flb200: inconsistent q/k/v shapes")
    Ho = Hq // 2 if diff else Hq
    if v.size(1) != (Ho if diff else Hkv):
        raise ValueError("flb200: inconsistent number of value heads")

    if rows_major_out:
        o = torch.empty((N, L, Ho, Ev), dtype=q.dtype, device=q.device).transpose(1, 2)
    else:
        o = torch.empty((N, Ho, L, Ev), dtype=q.dtype, device=q.device)

    keep: list = []
    p = _lib.new_params()
    p.diff = int(diff)
    p.N, p.Hq, p.Hkv, p.L, p.S, p.E, p.Ev = N, Hq, Hkv, L, S, E, Ev
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("o_stride", o)):
        arr = getattr(p, name)
        arr[0], arr[1], arr[2] = _strides3(t)
    p.scale = float(scale)
    p.score_mod = int(score_mod)
    p.alibi_heads = int(alibi_heads)
    p.alibi_head0 = int(alibi_head0)
    p.softcap = float(softcap)
    _fill_bias(p, 0, bias0, keep)
    _fill_bias(p, 1, bias1, keep)
    p.bias_inner = int(bias_inner)
    p.mask = int(mask)
    p.causal = int(causal)
    p.window = int(window)
    if prefix_len is not None:
        pl = prefix_len.to(device=q.device, dtype=torch.int32).contiguous()
        if pl.numel() != N:
            raise ValueError("flb200: prefix_len must hold one length per sequence")
        keep.append(pl)
        p.prefix_len = pl.data_ptr()
    p.prefix_scalar = int(prefix_scalar)
    p.diff_lambda = float(diff_lambda)
    p.diff_rms_norm = int(diff_rms_norm)
    p.diff_rms_eps = float(diff_rms_eps)
    p.status = _status_word(q.device).data_ptr()
    mirror = _status_mirror(q.device)
    if int(mirror[0]) != 0:
        # an earlier launch on this device gave up on a wait; every launch after it ends at once
        # until the word is cleared, so say so now instead of returning undefined results
        check_status(q.device)
    p.status_host = mirror.data_ptr()
    if lse is not None:
        p.lse = lse.data_ptr()
        p.lse_stride[0], p.lse_stride[1] = lse.stride(0), lse.stride(1)

    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        if mask == _lib.MASK_DOCUMENT:
            if document_id is None:
                raise ValueError("flb200: document mask needs document_id")
            doc = document_id
            if doc.dtype != torch.int64 or not doc.is_cuda:
                doc = doc.to(device=q.device, dtype=torch.int64)
            if doc.dim() != 2 or doc.size(0) != N or doc.size(1) != L:
                raise ValueError("flb200: document_id must be [N, L]")
            if doc.stride(1) != 1:
                doc = doc.contiguous()
            keep.append(doc)
            p.document_id = doc.data_ptr()
            p.doc_stride_n = doc.stride(0) if N > 1 else 0
            nbytes = lib.flb200_attn_workspace_bytes(C.byref(p))
            # block map cache: same ids (storage, version, layout) and same causal flag
            key = (doc.data_ptr(), doc._version, tuple(doc.shape), tuple(doc.stride()),
                   bool(causal), q.device.index)
            hit = _MAP_CACHE.get(key)
            ws = hit[0] if hit is not None else None
            cur = torch.cuda.current_stream(q.device)
            if ws is None or ws.numel() < nbytes:
                ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=q.device)
                p.workspace, p.workspace_bytes, p.block_map_ready = ws.data_ptr(), ws.numel(), 0
                rc = lib.flb200_build_block_map(C.byref(p), C.c_void_p(stream))
                if rc != _lib.OK:
                    _raise_for(rc, "build_block_map")
                built = torch.cuda.Event()
                built.record(cur)
                if len(_MAP_CACHE) >= _MAP_CACHE_MAX:
                    _MAP_CACHE.pop(next(iter(_MAP_CACHE)))
                # the entry keeps `doc` alive, so its address cannot be handed to other ids
                _MAP_CACHE[key] = (ws, doc, built, cur)
            else:
                # the map may have been built on another stream: order this launch after the build
                if hit[3] != cur:
                    cur.wait_event(hit[2])
            # an evicted map must not return to the allocator while a kernel of this stream reads it
            ws.record_stream(cur)
            keep.append(ws)
            p.workspace, p.workspace_bytes, p.block_map_ready = ws.data_ptr(), ws.numel(), 1
        elif score_mod == _lib.SCORE_BIAS or diff:
            # optional scratch: key-vector rows of the resident pair-bias kernel, or the word that takes max |v|
            # for the fp16 P.V product of differential attention; stream-ordered
            # like every other temporary of this call
            nbytes = lib.flb200_attn_workspace_bytes(C.byref(p))
            if nbytes:
                ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
                keep.append(ws)
                p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        rc = lib.flb200_attn_fwd(C.byref(p), C.c_void_p(stream))
    if rc != _lib.OK:
        _raise_for(rc, "attn_fwd")
    return o


@attn_fwd.register_fake
def _attn_fwd_fake(q, k, v, scale, score_mod, alibi_heads, alibi_head0, softcap, mask, causal, window,
                   prefix_len, prefix_scalar, document_id, bias0, bias1, bias_inner,
                   diff, diff_lambda, diff_rms_norm, diff_rms_eps, rows_major_out):
    N, Hq, L, _ = q.shape
    Ho = Hq // 2 if diff else Hq
    Ev = v.size(3)
    if rows_major_out:
        return q.new_empty((N, L, Ho, Ev)).transpose(1, 2)
    return q.new_empty((N, Ho, L, Ev))


def attn_bwd(q, k, v, o, dout, lse, scale: float, causal: bool):
    """dq, dk, dv of plain / causal attention (GQA by head counts) from the forward's inputs, output and
    log-sum-exp and the output's gradient: q, o, dout [N, Hq, L, E]; k, v [N, Hkv, S, E]; lse fp32
    [N, Hq, L] as `attn_fwd_lse` returns it.  The reference stubs its backward
    (benchmarks/_utils.py:16-21); this is the derivative of its eager functions."""
    lib = _lib.load()
    for t in (q, k, v, o, dout):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 4:
            raise ValueError("flb200: attn_bwd takes 4-D bfloat16 CUDA tensors")
    N, Hq, L, E = q.shape
    Hkv, S = k.size(1), k.size(2)
    if v.shape != k.shape or o.shape != q.shape or dout.shape != q.shape:
        raise ValueError("flb200: attn_bwd needs equal q/k and v head dims and matching shapes")
    dout = dout if dout.stride(3) == 1 else dout.contiguous()
    o = o if o.stride(3) == 1 else o.contiguous()
    lse = lse.contiguous()
    dq, dk, dv = torch.empty_like(q, memory_format=torch.contiguous_format), \
        torch.empty_like(k, memory_format=torch.contiguous_format), torch.empty_like(v, memory_format=torch.contiguous_format)
    p = _lib.AttnBwdParams()
    p.struct_size = C.sizeof(_lib.AttnBwdParams)
    p.N, p.Hq, p.Hkv, p.L, p.S, p.E = N, Hq, Hkv, L, S, E
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o), ("dout", dout), ("dq", dq), ("dk", dk), ("dv", dv)):
        setattr(p, name, t.data_ptr())
    for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("o_stride", o), ("do_stride", dout),
                    ("dq_stride", dq), ("dk_stride", dk), ("dv_stride", dv)):
        arr = getattr(p, name)
        arr[0], arr[1], arr[2] = _strides3(t)
    p.lse = lse.data_ptr()
    p.lse_stride[0], p.lse_stride[1] = lse.stride(0), lse.stride(1)
    p.scale, p.causal = float(scale), int(causal)
    ws = torch.empty(max(lib.flb200_attn_bwd_workspace_bytes(C.byref(p)), 256), dtype=torch.uint8, device=q.device)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    p.status = _status_word(q.device).data_ptr()
    mirror = _status_mirror(q.device)
    if int(mirror[0]) != 0:
        check_status(q.device)
    p.status_host = mirror.data_ptr()
    with torch.cuda.device(q.device):
        rc = lib.flb200_attn_bwd(C.byref(p), C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
    if rc != _lib.OK:
        _raise_for(rc, "attn_bwd")
    return dq, dk, dv


class _AttentionWithGrad(torch.autograd.Function):
    """Plain / causal attention whose backward runs the library's backward kernels."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal):
        o, lse = attn_fwd_lse(q, k, v, scale, mask=_lib.MASK_CAUSAL if causal else _lib.MASK_NONE)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale, ctx.causal = scale, causal
        return o

    @staticmethod
    def backward(ctx, dout):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = attn_bwd(q, k, v, o, dout.to(torch.bfloat16), lse, ctx.scale, ctx.causal)
        return dq, dk, dv, None, None


def attention_with_grad(q, k, v, scale: float, causal: bool) -> torch.Tensor:
    """softmax(q k^T * scale [causal]) v, differentiable with respect to q, k and v."""
    return _AttentionWithGrad.apply(q, k, v, float(scale), bool(causal))


_POINTWISE = {"identity": _lib.PW_IDENTITY, "relu": _lib.PW_RELU, "tanh": _lib.PW_TANH, "sigmoid": _lib.PW_SIGMOID}


def ipa_pack(q_scalar, k_scalar, v_scalar, q_points, k_points, v_points, a: float):
    """Augmented operands of invariant point attention (`flb200_ipa_pack`): returns q', k' `[B, H, N, E]` and
    v' `[B, H, N_k, Ev]` for a pair-biased forward with scale 1 / sqrt(c_hidden)."""
    lib = _lib.load()
    B, H, N, Cw = q_scalar.shape
    Nk = k_scalar.size(2)
    P_qk, pd = q_points.shape[-2:]
    P_v = v_points.size(-2)
    E = -(-(Cw + 2 * P_qk * pd + 2) // 8) * 8
    Ev = -(-(Cw + P_v * pd) // 8) * 8
    ts = [t.contiguous() for t in (q_scalar, k_scalar, v_scalar, q_points, k_points, v_points)]
    dev, dt = q_scalar.device, torch.bfloat16
    qa = torch.empty(B, H, N, E, dtype=dt, device=dev)
    ka = torch.empty(B, H, Nk, E, dtype=dt, device=dev)
    va = torch.empty(B, H, Nk, Ev, dtype=dt, device=dev)
    p = _lib.IpaPackParams()
    p.struct_size = C.sizeof(_lib.IpaPackParams)
    p.rows_q, p.rows_k = B * H * N, B * H * Nk
    p.C, p.P_qk, p.P_v, p.point_dim = Cw, P_qk, P_v, pd
    (p.q_scalar, p.k_scalar, p.v_scalar, p.q_points, p.k_points, p.v_points) = (t.data_ptr() for t in ts)
    p.a, p.E, p.Ev = float(a), E, Ev
    p.q_aug, p.k_aug, p.v_aug = qa.data_ptr(), ka.data_ptr(), va.data_ptr()
    with torch.cuda.device(dev):
        rc = lib.flb200_ipa_pack(C.byref(p), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if rc != _lib.OK:
        _raise_for(rc, "ipa_pack")
    return qa, ka, va


@torch.library.custom_op("flb200::product_chain", mutates_args=())
def product_chain(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, scale: float, pointwise: str) -> torch.Tensor:
    """f((a @ b) * scale) @ c in one kernel, no softmax: a [B, M, N], b [B, N, O], c [B, O, P] bf16 with
    N, P <= 128 -> [B, M, P].  The counterpart of the reference's fused `bmm(f(bmm(a, b)), c)`
    template (monkeypatch/template/fused_bmm.py:332-422).  `b` is read where it lies: with its last
    axis contiguous (the natural [B, N, O] layout) or as a transposed view of a [B, O, N] tensor."""
    lib = _lib.load()
    if pointwise not in _POINTWISE:
        raise NotImplementedError(f"flb200: pointwise must be one of {sorted(_POINTWISE)}")
    if not (a.is_cuda and b.is_cuda and c.is_cuda):
        raise RuntimeError("flb200: tensors must live on a CUDA device (there is no CPU path)")
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or c.dtype != torch.bfloat16:
        raise NotImplementedError("flb200: only bfloat16 inputs are supported")
    if a.dim() != 3 or b.dim() != 3 or c.dim() != 3:
        raise ValueError("flb200: a, b, c must be 3-D [batch, rows, cols]")
    B, M, N = a.shape
    O, P = c.size(1), c.size(2)
    if b.shape != (B, N, O) or c.size(0) != B:
        raise ValueError("flb200: inconsistent shapes for (a @ b) @ c")
    if a.stride(2) != 1:
        a = a.contiguous()
    if c.stride(2) != 1:
        c = c.contiguous()
    keys_contiguous = b.stride(2) == 1
    if not keys_contiguous and b.stride(1) != 1:
        b = b.contiguous()
        keys_contiguous = True
    if keys_contiguous and b.stride(1) % 8 != 0 and N % 8 == 0:
        # rows of O keys that do not start on 16-byte boundaries cannot be fetched as tiles: lay b
        # out as O rows of N features instead
        b = b.transpose(1, 2).contiguous().transpose(1, 2)
        keys_contiguous = False
    o = torch.empty((B, M, P), dtype=a.dtype, device=a.device)
    p = _lib.new_params()
    p.product_chain, p.pointwise, p.k_keys_contiguous = 1, _POINTWISE[pointwise], int(keys_contiguous)
    p.N, p.Hq, p.Hkv, p.L, p.S, p.E, p.Ev = B, 1, 1, M, O, N, P
    p.q, p.k, p.v, p.o = a.data_ptr(), b.data_ptr(), c.data_ptr(), o.data_ptr()
    p.q_stride[0], p.q_stride[1], p.q_stride[2] = a.stride(0), 0, a.stride(1)
    # k: rows of features [O][N] (b given as a transposed view), or feature rows of keys [N][O]
    p.k_stride[0], p.k_stride[1] = b.stride(0), 0
    p.k_stride[2] = b.stride(1) if keys_contiguous else b.stride(2)
    p.v_stride[0], p.v_stride[1], p.v_stride[2] = c.stride(0), 0, c.stride(1)
    p.o_stride[0], p.o_stride[1], p.o_stride[2] = o.stride(0), 0, o.stride(1)
    p.scale = float(scale)
    p.status = _status_word(a.device).data_ptr()
    mirror = _status_mirror(a.device)
    if int(mirror[0]) != 0:
        check_status(a.device)
    p.status_host = mirror.data_ptr()
    with torch.cuda.device(a.device):
        rc = lib.flb200_attn_fwd(C.byref(p), C.c_void_p(torch.cuda.current_stream(a.device).cuda_stream))
    if rc != _lib.OK:
        _raise_for(rc, "product_chain")
    return o


@product_chain.register_fake
def _product_chain_fake(a, b, c, scale, pointwise):
    return a.new_empty((a.size(0), a.size(1), c.size(2)))


def clear_block_map_cache() -> None:
    _MAP_CACHE.clear()
