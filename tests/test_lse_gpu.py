"""Optional log-sum-exp output of the forward pass (what a backward pass takes from it)."""
import ctypes as C

import pytest
import torch

from flashlight_b200 import _lib, ops
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu


def rnd(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)


def check(o, lse, ref_o, ref_lse):
    ops.check_status()
    assert lse.dtype == torch.float32 and lse.shape == ref_lse.shape
    d = (lse - ref_lse).abs()
    finite = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), finite)
    assert d[finite].max().item() <= 2e-3, d[finite].max().item()
    assert (o.float() - ref_o).abs().max().item() <= 2e-2 + 2 ** -8 * ref_o.abs().max().item()


@pytest.mark.parametrize("S,D", [(384, 64), (1000, 128), (129, 32)])
def test_vanilla_and_causal(S, D):
    q, k, v = rnd((2, 8, S, D), 1), rnd((2, 2, S, D), 2), rnd((2, 2, S, D), 3)
    scale = D ** -0.5
    o, lse = ops.attn_fwd_lse(q, k, v, scale)
    check(o, lse, *ao.vanilla(q, k, v, return_lse=True))
    o, lse = ops.attn_fwd_lse(q, k, v, scale, mask=_lib.MASK_CAUSAL)
    check(o, lse, *ao.causal(q, k, v, return_lse=True))
    # the output is the one the plain op returns
    plain = torch.ops.flb200.attn_fwd(q, k, v, scale, 0, 0, 0, 0.0, _lib.MASK_CAUSAL, False, 0, None, 0, None,
                                      None, None, 1, False, 0.0, False, 0.0, False)
    assert torch.equal(plain, o)


def test_score_mods_and_masks():
    S, D, H = 900, 128, 4
    q, k, v = rnd((1, H, S, D), 4), rnd((1, H, S, D), 5), rnd((1, H, S, D), 6)
    scale = D ** -0.5
    o, lse = ops.attn_fwd_lse(q, k, v, scale, score_mod=_lib.SCORE_ALIBI, alibi_heads=H, mask=_lib.MASK_CAUSAL)
    check(o, lse, *ao.alibi(q, k, v, nheads=H, is_causal=True, return_lse=True))
    o, lse = ops.attn_fwd_lse(q, k, v, scale, score_mod=_lib.SCORE_ALIBI, alibi_heads=H)
    check(o, lse, *ao.alibi(q, k, v, nheads=H, return_lse=True))
    o, lse = ops.attn_fwd_lse(q, k, v, scale, score_mod=_lib.SCORE_SOFTCAP, softcap=20.0, mask=_lib.MASK_CAUSAL)
    check(o, lse, *ao.softcap(q, k, v, cap=20.0, is_causal=True, return_lse=True))
    o, lse = ops.attn_fwd_lse(q, k, v, scale, mask=_lib.MASK_SLIDING, window=100)
    check(o, lse, *ao.sliding_window(q, k, v, window_size=100, return_lse=True))
    o, lse = ops.attn_fwd_lse(q, k, v, scale, mask=_lib.MASK_PREFIX, prefix_scalar=300)
    check(o, lse, *ao.prefix_lm(q, k, v, prefix_lengths=300, return_lse=True))
    ids = torch.repeat_interleave(torch.arange(3), torch.tensor([200, 450, 250])).view(1, S).cuda()
    o, lse = ops.attn_fwd_lse(q, k, v, scale, mask=_lib.MASK_DOCUMENT, document_id=ids, causal=True)
    check(o, lse, *ao.document_mask(q, k, v, ids, is_causal=True, return_lse=True))


def test_lse_argument_checks():
    lib = _lib.load()
    q = rnd((1, 4, 256, 64), 7)
    v = rnd((1, 2, 256, 128), 8)
    lse = torch.empty(1, 4, 256, device="cuda")
    p = _lib.new_params()
    p.N, p.Hq, p.Hkv, p.L, p.S, p.E, p.Ev = 1, 4, 4, 256, 256, 64, 128
    p.diff = 1
    p.q = p.k = q.data_ptr()
    p.v = v.data_ptr()
    p.o = torch.empty(1, 2, 256, 128, dtype=torch.bfloat16, device="cuda").data_ptr()
    for name, t in (("q_stride", q), ("k_stride", q), ("v_stride", v), ("o_stride", v)):
        a = getattr(p, name)
        a[0], a[1], a[2] = t.stride(0), t.stride(1), t.stride(2)
    p.scale = 0.125
    p.diff_lambda = 0.5
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.OK
    p.lse = lse.data_ptr()
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.E_UNSUPPORTED   # no single LSE for two softmaxes
    p.diff, p.Hkv, p.Ev = 0, 4, 64
    p.v = q.data_ptr()
    for name in ("v_stride", "o_stride"):
        a = getattr(p, name)
        a[0], a[1], a[2] = q.stride(0), q.stride(1), q.stride(2)
    p.lse = lse.data_ptr() + 2
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.E_MISALIGNED
