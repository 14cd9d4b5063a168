"""Head dims between the built kernel widths, unequal q/k and v widths, rows without a visible
key, biases that broadcast along the keys, and the bounded device-side wait."""
import ctypes as C

import pytest
import torch

import flashlight_b200
from flashlight_b200 import _lib, attention_variants as av
from flashlight_b200.ops import attn_fwd_lse
from oracle import attention_oracle as ao
from _parity import check

pytestmark = pytest.mark.gpu


def rnd(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("E,Ev", [(96, 96), (48, 48), (16, 16), (8, 8), (128, 64), (64, 128), (80, 32), (120, 104)])
@pytest.mark.parametrize("S", [200, 640])
def test_any_head_dim_up_to_128(E, Ev, S):
    """The reference takes any head dim up to 256 as a one-shot reduction range
    (monkeypatch/fusion/_common.py:4); here every width up to 128, equal or not for q/k and v,
    runs on the next wider kernel with the tensor maps zero-filling the missing columns."""
    q, k, v = rnd((2, 4, S, E), 1), rnd((2, 2, S, E), 2), rnd((2, 2, S, Ev), 3)
    check(av.attention_pytorch(q, k, v, enable_gqa=True), ao.vanilla(q, k, v, enable_gqa=True), (E, Ev))
    check(av.attention_pytorch_causal(q, k, v, enable_gqa=True), ao.causal(q, k, v, enable_gqa=True), (E, Ev))
    check(av.attention_pytorch_sliding_window(q, k, v, window_size=77, enable_gqa=True),
          ao.sliding_window(q, k, v, window_size=77, enable_gqa=True), (E, Ev))
    check(av.attention_pytorch_alibi(q, k, v, score_mod=av.generate_alibi_bias_pytorch(4), enable_gqa=True),
          ao.alibi(q, k, v, nheads=4, enable_gqa=True), (E, Ev))


@pytest.mark.parametrize("E,Ev", [(256, 256), (192, 192), (136, 64), (64, 256), (200, 160)])
@pytest.mark.parametrize("S", [200, 1000])
def test_head_dims_up_to_256(E, Ev, S):
    """Heads above 128 (the reference takes any width up to 256 as a one-shot reduction range,
    monkeypatch/fusion/_common.py:4) run plain and causal attention with one query tile per CTA."""
    q, k, v = rnd((2, 4, S, E), 31), rnd((2, 2, S, E), 32), rnd((2, 2, S, Ev), 33)
    check(av.attention_pytorch(q, k, v, enable_gqa=True), ao.vanilla(q, k, v, enable_gqa=True), (E, Ev))
    check(av.attention_pytorch_causal(q, k, v, enable_gqa=True), ao.causal(q, k, v, enable_gqa=True), (E, Ev))


def test_diff_attention_with_narrow_heads():
    q, k, v = rnd((1, 4, 300, 48), 4), rnd((1, 4, 300, 48), 5), rnd((1, 2, 300, 96), 6)
    check(av.diffattn(q, k, v, lambda_full=0.5), ao.diffattn(q, k, v, lambda_full=0.5))


@pytest.mark.parametrize("D", [32, 64])
def test_rows_without_a_visible_key_give_zeros_and_minus_inf(D, monkeypatch):
    """A -inf bias over every key of a row leaves that row without a visible key.  The reference
    returns NaN there (softmax of all -inf, evoformer.py:30); this library documents zeros and a
    log-sum-exp of -inf, for both kernel layouts, and the other rows are unaffected."""
    B, N, S, H = 1, 4, 384, 2
    q, k, v = rnd((B, N, S, H, D), 7), rnd((B, N, S, H, D), 8), rnd((B, N, S, H, D), 9)
    pair = rnd((B, 1, H, S, S), 10)
    g = torch.Generator().manual_seed(11)
    keep = torch.rand(B, N, 1, 1, S, generator=g) < 0.9
    keep[..., 0] = True
    mask = torch.where(keep, 0.0, float("-inf")).to(torch.bfloat16).cuda()
    mask[0, 2] = float("-inf")                      # MSA row 2: every key masked
    for st in ("1", "2"):
        monkeypatch.setenv("FLB200_STAGES", st)
        out = av.attention_reference(q, k, v, [mask, pair])
        flashlight_b200.check_status()
        assert torch.count_nonzero(out[0, 2]) == 0
        ref = ao.evoformer(q, k, v, [mask, pair])
        rows = [0, 1, 3]
        check(out[:, rows], ref[:, rows], st)
    # log-sum-exp of such rows through the 4-D entry
    q4, k4, v4 = rnd((1, 2, 300, D), 12), rnd((1, 2, 300, D), 13), rnd((1, 2, 300, D), 14)
    bias = torch.zeros(1, 1, 2, 300, 300, dtype=torch.bfloat16, device="cuda")
    bias[0, 0, 1, 5] = float("-inf")
    bias[0, 0, 0, 299] = float("-inf")
    o, lse = attn_fwd_lse(q4, k4, v4, D ** -0.5, score_mod=_lib.SCORE_BIAS, bias0=bias, bias_inner=1)
    flashlight_b200.check_status()
    assert torch.isinf(lse[0, 1, 5]) and lse[0, 1, 5] < 0 and torch.isinf(lse[0, 0, 299])
    assert torch.count_nonzero(o[0, 1, 5]) == 0 and torch.count_nonzero(o[0, 0, 299]) == 0
    assert torch.isfinite(lse[0, 1, :5]).all() and torch.isfinite(lse[0, 0, :299]).all()


def test_bias_that_broadcasts_along_the_keys():
    """`a += b` of the reference accepts a bias of key extent 1 (evoformer.py:26-27)."""
    B, N, S, H, D = 1, 3, 200, 2, 32
    q, k, v = rnd((B, N, S, H, D), 15), rnd((B, N, S, H, D), 16), rnd((B, N, S, H, D), 17)
    row_bias = rnd((B, 1, H, S, 1), 18)            # one value per query row: changes nothing after softmax
    pair = rnd((B, 1, H, S, S), 19)
    check(av.attention_reference(q, k, v, [row_bias, pair]), ao.evoformer(q, k, v, [row_bias, pair]))


def test_alibi_head_count_must_match():
    q = rnd((1, 4, 128, 64), 20)
    with pytest.raises(ValueError):
        av.attention_pytorch_alibi(q, q, q, score_mod=av.generate_alibi_bias_pytorch(8))


def _params(q, k, v, o, status, mirror):
    p = _lib.new_params()
    N, H, L, E = q.shape
    p.N, p.Hq, p.Hkv, p.L, p.S, p.E, p.Ev = N, H, H, L, L, E, E
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("o_stride", o)):
        a = getattr(p, name)
        a[0], a[1], a[2] = t.stride(0), t.stride(1), t.stride(2)
    p.scale = E ** -0.5
    p.mask = _lib.MASK_CAUSAL
    p.status = status.data_ptr()
    p.status_host = mirror.data_ptr()
    return p


@pytest.mark.parametrize("st", ["1", "2"])
def test_a_wait_that_runs_out_ends_the_launch_with_a_status(st, monkeypatch):
    """The permitted form of a failure test: the self-test launch withholds the kernel's loads, so
    the roles' first waits run into the one-millisecond limit; the CTAs leave through the common
    exit, the status word (and its host mirror) read E_TIMEOUT with a valid barrier id, the output
    buffer is untouched, and the next normal launch gives the same bits as the one before."""
    monkeypatch.setenv("FLB200_STAGES", st)
    lib = _lib.load()
    q, k, v = rnd((1, 2, 512, 128), 21), rnd((1, 2, 512, 128), 22), rnd((1, 2, 512, 128), 23)
    o = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    mirror = torch.zeros(1, dtype=torch.int32).pin_memory()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = _params(q, k, v, o, status, mirror)
    assert lib.flb200_attn_fwd(C.byref(p), stream) == _lib.OK
    torch.cuda.synchronize()
    before = o.clone()
    assert int(status.item()) == 0 and int(mirror[0]) == 0

    o.fill_(7.0)
    p.wait_limit_us = 1000
    assert lib.flb200_selftest_wait_timeout(C.byref(p), stream) == _lib.OK
    torch.cuda.synchronize()                        # returns: nothing hangs, nothing traps
    word = int(status.item())
    bar, blk = C.c_int32(-1), C.c_int32(-1)
    assert lib.flb200_decode_status(word, C.byref(bar), C.byref(blk)) == _lib.E_TIMEOUT
    assert 0 <= bar.value < 32 and 0 <= blk.value < 8
    assert int(mirror[0]) == word                   # the host sees it without reading device memory
    assert bool((o == 7.0).all())                   # no store happened

    # while the word is set, later launches end at once; cleared, the kernel is back to normal
    status.zero_()
    mirror.zero_()
    p.wait_limit_us = 0
    assert lib.flb200_attn_fwd(C.byref(p), stream) == _lib.OK
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(o, before)
