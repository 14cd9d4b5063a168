"""Backward kernels (dq, dk, dv of plain and causal attention, with grouped query heads) against torch
autograd through the fp32 oracle on the same bf16-rounded inputs.  The reference stubs its backward
(benchmarks/_utils.py:16-21), so the oracle's derivative is the definition.

Tolerance: gradients have no fixed scale (they grow with the upstream gradient and shrink with the
sequence length), so the band is relative to each gradient's own RMS (the larger of the whole tensor's
and the row's, since the first rows under a causal mask keep gradients of order one however long the
sequence): |d - ref| <= 2e-2 * rms + 1.6e-2 * |ref| elementwise (the bf16 rounding of P, dS and the
result), mean |d - ref| <= 4e-3 * rms(ref) (measured: 1.5e-3).  Under the causal mask the first few query rows see one to five keys: their
probabilities are of order one and the terms of their gradients cancel.  There the kernels' row sums
delta = sum(dO * O), taken as every fused backward takes them from the forward's bf16 OUTPUT, carry that
output's rounding (e.g. 9.787 for 9.821), which moves dS = P (dP - delta) scale of such a row by a few
per cent; a handful of elements per hundred thousand land outside the band (measured at most 62 per
million, the largest at 4.4 times the band, reproduced exactly by evaluating the formula with the
rounded output).  The test allows 2 per ten thousand outside the band and none beyond six times it.
"""
import pytest
import torch

import flashlight_b200
from flashlight_b200 import attention_variants as av
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu


def rnd(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(torch.bfloat16).cuda()


def grads(fn, q, k, v, dout):
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out = fn(q, k, v)
    out.backward(dout.reshape(out.shape).to(out.dtype))
    return out.detach(), q.grad, k.grad, v.grad


def close(d, ref, what):
    flashlight_b200.check_status()
    d, ref = d.float(), ref.float()
    rms = ref.pow(2).mean().sqrt().item()
    err = (d - ref).abs()
    # the scale of a row's rounding errors is the larger of the tensor's RMS and the row's own
    scale = torch.clamp(ref.pow(2).mean(dim=-1, keepdim=True).sqrt(), min=rms)
    band = 2e-2 * scale + 1.6e-2 * ref.abs()
    assert torch.isfinite(d).all(), what
    outside = int((err > band).sum())
    assert outside <= max(1, 2 * err.numel() // 10_000), (what, outside, err.numel())
    assert bool((err <= 6 * band).all()), (what, (err / band).max().item(), rms)
    assert err.mean().item() <= 4e-3 * rms, (what, err.mean().item(), rms)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", [128, 384, 1000])
def test_backward_matches_autograd_of_the_oracle(S, D, causal):
    N, Hq, Hkv = 2, 4, 2
    q, k, v = rnd((N, Hq, S, D), 1), rnd((N, Hkv, S, D), 2), rnd((N, Hkv, S, D), 3)
    dout = rnd((N, Hq, S, D), 4)
    if causal:
        fn = lambda a, b, c: av.attention_pytorch_causal(a, b, c, enable_gqa=True)
        fo = lambda a, b, c: ao.causal(a, b, c, enable_gqa=True)
    else:
        fn = lambda a, b, c: av.attention_pytorch(a, b, c, enable_gqa=True)
        fo = lambda a, b, c: ao.vanilla(a, b, c, enable_gqa=True)
    out, dq, dk, dv = grads(fn, q, k, v, dout)
    ref, rq, rk, rv = grads(fo, q.float(), k.float(), v.float(), dout.float())
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    close(dv, rv, ("dv", S, D, causal))
    close(dq, rq, ("dq", S, D, causal))
    close(dk, rk, ("dk", S, D, causal))


def test_backward_cross_lengths_and_narrow_heads():
    q, k, v = rnd((1, 2, 200, 48), 5), rnd((1, 2, 520, 48), 6), rnd((1, 2, 520, 48), 7)
    dout = rnd((1, 2, 200, 48), 8)
    _, dq, dk, dv = grads(lambda a, b, c: av.attention_pytorch(a, b, c), q, k, v, dout)
    _, rq, rk, rv = grads(lambda a, b, c: ao.vanilla(a, b, c), q.float(), k.float(), v.float(), dout.float())
    close(dq, rq, "dq")
    close(dk, rk, "dk")
    close(dv, rv, "dv")


def test_variants_without_a_backward_kernel_say_so():
    q = rnd((1, 2, 128, 64), 9).requires_grad_(True)
    with pytest.raises(NotImplementedError):
        av.attention_pytorch_sliding_window(q, q, q, window_size=16)


def test_backward_is_deterministic():
    q, k, v, dout = rnd((1, 4, 700, 128), 10), rnd((1, 1, 700, 128), 11), rnd((1, 1, 700, 128), 12), rnd((1, 4, 700, 128), 13)
    fn = lambda a, b, c: av.attention_pytorch_causal(a, b, c, enable_gqa=True)
    first = grads(fn, q, k, v, dout)
    for _ in range(3):
        again = grads(fn, q, k, v, dout)
        assert all(torch.equal(x, y) for x, y in zip(first, again))


def test_backward_long_causal_sequence_with_groups_of_four():
    """Sixteen key tiles per query head and four query heads per kv head: the rings of both kernels wrap
    several times and the dK/dV kernel walks 4 x 16 steps."""
    q, k, v, dout = rnd((1, 8, 2048, 128), 14), rnd((1, 2, 2048, 128), 15), rnd((1, 2, 2048, 128), 16), rnd((1, 8, 2048, 128), 17)
    fn = lambda a, b, c: av.attention_pytorch_causal(a, b, c, enable_gqa=True)
    fo = lambda a, b, c: ao.causal(a, b, c, enable_gqa=True)
    _, dq, dk, dv = grads(fn, q, k, v, dout)
    _, rq, rk, rv = grads(fo, q.float(), k.float(), v.float(), dout.float())
    close(dq, rq, "dq")
    close(dk, rk, "dk")
    close(dv, rv, "dv")


def test_backward_of_strided_views():
    """q, k, v as [N, L, H, D] storage seen as [N, H, L, D]: the tensor maps carry the strides."""
    base = [rnd((2, 300, 4, 64), 18 + i) for i in range(3)]
    q, k, v = (t.transpose(1, 2) for t in base)
    dout = rnd((2, 4, 300, 64), 21)
    _, dq, dk, dv = grads(lambda a, b, c: av.attention_pytorch_causal(a, b, c), q, k, v, dout)
    _, rq, rk, rv = grads(lambda a, b, c: ao.causal(a, b, c), q.float(), k.float(), v.float(), dout.float())
    close(dq, rq, "dq")
    close(dk, rk, "dk")
    close(dv, rv, "dv")


@pytest.mark.parametrize("D", [64, 128])
def test_a_backward_wait_that_runs_out_ends_the_launch_with_a_status(D):
    """The permitted form of a failure test, for the backward kernels: the self-test launch withholds
    their loads, the roles' first waits run into the one-millisecond limit, the CTAs leave through the
    common exit with E_TIMEOUT in the status word and its host mirror, the gradient buffers stay untouched,
    and the next normal backward gives the same bits as the one before."""
    import ctypes as C
    from flashlight_b200 import _lib, ops
    lib = _lib.load()
    q, k, v, dout = rnd((1, 4, 512, D), 30), rnd((1, 2, 512, D), 31), rnd((1, 2, 512, D), 32), rnd((1, 4, 512, D), 33)
    o, lse = ops.attn_fwd_lse(q, k, v, D ** -0.5, mask=_lib.MASK_CAUSAL)
    before = ops.attn_bwd(q, k, v, o, dout, lse, D ** -0.5, True)
    torch.cuda.synchronize()

    dq, dk, dv = torch.full_like(q, 7.0), torch.full_like(k, 7.0), torch.full_like(v, 7.0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    mirror = torch.zeros(1, dtype=torch.int32).pin_memory()
    p = _lib.AttnBwdParams()
    p.struct_size = C.sizeof(_lib.AttnBwdParams)
    p.N, p.Hq, p.Hkv, p.L, p.S, p.E = 1, 4, 2, 512, 512, D
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o), ("dout", dout), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        setattr(p, name, t.data_ptr())
    for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("o_stride", o), ("do_stride", dout),
                    ("dq_stride", dq), ("dk_stride", dk), ("dv_stride", dv)):
        a = getattr(p, name)
        a[0], a[1], a[2] = t.stride(0), t.stride(1), t.stride(2)
    p.lse_stride[0], p.lse_stride[1] = lse.stride(0), lse.stride(1)
    p.scale, p.causal = D ** -0.5, 1
    ws = torch.empty(lib.flb200_attn_bwd_workspace_bytes(C.byref(p)), dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    p.status, p.status_host, p.wait_limit_us = status.data_ptr(), mirror.data_ptr(), 1000
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.flb200_selftest_bwd_wait_timeout(C.byref(p), stream) == _lib.OK
    torch.cuda.synchronize()                        # returns: nothing hangs, nothing traps
    word = int(status.item())
    bar, blk = C.c_int32(-1), C.c_int32(-1)
    assert lib.flb200_decode_status(word, C.byref(bar), C.byref(blk)) == _lib.E_TIMEOUT
    assert 64 <= bar.value < 64 + 24                # the backward kernels number their barriers from 64
    assert int(mirror[0]) == word
    assert bool((dq == 7.0).all()) and bool((dk == 7.0).all()) and bool((dv == 7.0).all())

    status.zero_()
    mirror.zero_()
    p.wait_limit_us = 0
    assert lib.flb200_attn_bwd(C.byref(p), stream) == _lib.OK
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert all(torch.equal(a, b) for a, b in zip((dq, dk, dv), before))


@pytest.mark.parametrize("seed", range(24))
def test_backward_on_seeded_random_shapes(seed):
    """Random batch, group size, lengths (queries and keys alike under the causal mask, free otherwise) and
    head dims up to 128 in steps of 8."""
    g = torch.Generator().manual_seed(1000 + seed)
    ri = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g).item())
    causal = seed % 2 == 0
    N, Hkv, G = ri(1, 3), ri(1, 3), ri(1, 4)
    D = 8 * ri(1, 16)
    L = ri(1, 700)
    S = L if causal else ri(1, 700)
    q, k, v = rnd((N, Hkv * G, L, D), 40 + seed), rnd((N, Hkv, S, D), 140 + seed), rnd((N, Hkv, S, D), 240 + seed)
    dout = rnd((N, Hkv * G, L, D), 340 + seed)
    if causal:
        fn = lambda a, b, c: av.attention_pytorch_causal(a, b, c, enable_gqa=True)
        fo = lambda a, b, c: ao.causal(a, b, c, enable_gqa=True)
    else:
        fn = lambda a, b, c: av.attention_pytorch(a, b, c, enable_gqa=True)
        fo = lambda a, b, c: ao.vanilla(a, b, c, enable_gqa=True)
    _, dq, dk, dv = grads(fn, q, k, v, dout)
    _, rq, rk, rv = grads(fo, q.float(), k.float(), v.float(), dout.float())
    what = (N, Hkv, G, L, S, D, causal)
    close(dq, rq, ("dq",) + what)
    close(dk, rk, ("dk",) + what)
    close(dv, rv, ("dv",) + what)
