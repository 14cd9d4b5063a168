"""Host-side behaviour of the C ABI: the library loads without a GPU, exports every symbol
the header declares, and rejects bad problem descriptions with distinct codes.  No compute
call is made here."""
import ctypes as C
import re
from pathlib import Path

import pytest

from flashlight_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "flb200_attn.h").read_text()

FAKE = 0x7F0000000000  # aligned, never dereferenced: validation is host-only


def good(**over):
    p = _lib.new_params()
    p.N, p.Hq, p.Hkv, p.L, p.S, p.E, p.Ev = 2, 4, 4, 256, 256, 128, 128
    p.q = p.k = p.v = p.o = FAKE
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        a = getattr(p, name)
        a[0], a[1], a[2] = 4 * 256 * 128, 256 * 128, 128
    p.scale = 0.088
    for k, v in over.items():
        if isinstance(v, tuple):
            arr = getattr(p, k)
            for i, x in enumerate(v):
                arr[i] = x
        else:
            setattr(p, k, v)
    return p


def test_header_symbols_are_exported(lib):
    declared = set(re.findall(r"\b(flb200_[a-z_]+)\s*\(", HEADER))
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_abi_version_and_struct_size(lib):
    assert lib.flb200_abi_version() == 3
    assert int(re.search(r"#define FLB200_ABI_VERSION (\d+)u", HEADER).group(1)) == 3
    p = good()
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.OK
    p.struct_size -= 4
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.E_BAD_ARG
    assert lib.flb200_attn_validate(None) == _lib.E_BAD_ARG


def test_strerror_distinct(lib):
    texts = {lib.flb200_strerror(c).decode() for c in range(0, -8, -1)}
    assert len(texts) == 8
    assert lib.flb200_strerror(-99).decode() == "unknown status"


@pytest.mark.parametrize("over,code", [
    (dict(N=0), _lib.E_BAD_ARG),
    (dict(q=None), _lib.E_BAD_ARG),
    (dict(scale=0.0), _lib.E_BAD_ARG),
    (dict(scale=float("nan")), _lib.E_BAD_ARG),
    (dict(Hq=6, Hkv=4), _lib.E_BAD_ARG),
    (dict(score_mod=9), _lib.E_BAD_ARG),
    (dict(mask=-1), _lib.E_BAD_ARG),
    (dict(score_mod=_lib.SCORE_ALIBI, alibi_heads=0), _lib.E_BAD_ARG),
    (dict(score_mod=_lib.SCORE_SOFTCAP, softcap=0.0), _lib.E_BAD_ARG),
    (dict(score_mod=_lib.SCORE_BIAS), _lib.E_BAD_ARG),               # no bias tensor
    (dict(mask=_lib.MASK_SLIDING, window=-1), _lib.E_BAD_ARG),
    (dict(mask=_lib.MASK_SLIDING, window=8, S=128), _lib.E_BAD_ARG),  # L != S
    (dict(mask=_lib.MASK_DOCUMENT), _lib.E_BAD_ARG),                 # no ids
    (dict(E=264, Ev=264), _lib.E_UNSUPPORTED),
    (dict(E=64, Ev=320), _lib.E_UNSUPPORTED),
    (dict(E=256, Ev=256, mask=_lib.MASK_SLIDING, window=8), _lib.E_UNSUPPORTED),   # wide heads: plain and causal only
    (dict(mask=_lib.MASK_DOCUMENT, document_id=FAKE + 4), _lib.E_MISALIGNED),
    (dict(mask=_lib.MASK_DOCUMENT, document_id=FAKE, N=70000), _lib.E_UNSUPPORTED),
    (dict(mask=_lib.MASK_DOCUMENT, document_id=FAKE, doc_stride_n=8), _lib.E_BAD_ARG),   # rows of L ids overlap
    (dict(lse=FAKE + 2), _lib.E_MISALIGNED),
    (dict(lse=FAKE, lse_stride=(16, 8)), _lib.E_BAD_ARG),                                # rows of L floats overlap
    (dict(score_mod=_lib.SCORE_ALIBI, alibi_heads=4, mask=_lib.MASK_SLIDING, window=4), _lib.E_UNSUPPORTED),
    (dict(q=FAKE + 2), _lib.E_MISALIGNED),
    (dict(mask=_lib.MASK_DOCUMENT, document_id=FAKE), _lib.E_WORKSPACE),
])
def test_validate_rejects(lib, over, code):
    assert lib.flb200_attn_validate(C.byref(good(**over))) == code


@pytest.mark.parametrize("E,Ev", [(96, 96), (128, 64), (64, 128), (48, 16), (8, 8), (120, 128)])
def test_narrow_and_unequal_head_dims_run_on_the_next_wider_kernel(lib, E, Ev):
    """Any head dims up to 128 are served by every variant: the tensor maps zero-fill the missing
    feature columns."""
    p = good(E=E, Ev=Ev)
    for name, w in (("q_stride", E), ("k_stride", E), ("v_stride", Ev), ("o_stride", Ev)):
        arr = getattr(p, name)
        arr[2], arr[1], arr[0] = w, w * 256, w * 256 * p.Hq
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.OK
    # ALiBi has no 32-wide kernel of its own: it runs on the 64-wide one
    p.score_mod, p.alibi_heads = _lib.SCORE_ALIBI, p.Hq
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.OK


@pytest.mark.parametrize("E,Ev", [(256, 256), (192, 192), (136, 64), (64, 256)])
def test_heads_up_to_256_for_plain_and_causal_attention(lib, E, Ev):
    p = good(E=E, Ev=Ev)
    for name, w in (("q_stride", E), ("k_stride", E), ("v_stride", Ev), ("o_stride", Ev)):
        arr = getattr(p, name)
        arr[2], arr[1], arr[0] = w, w * 256, w * 256 * p.Hq
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.OK
    p.mask = _lib.MASK_CAUSAL
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.OK
    p.score_mod, p.alibi_heads = _lib.SCORE_ALIBI, p.Hq
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.E_UNSUPPORTED


def test_stride_alignment(lib):
    p = good()
    p.q_stride[2] = 132  # not a multiple of 8 elements
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.E_MISALIGNED
    p = good()
    p.o_stride[2] = 64  # rows would overlap
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.E_BAD_ARG


def test_diff_shapes(lib):
    p = good(diff=1, E=64, Ev=128, Hq=8, Hkv=8)
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.OK
    p = good(diff=1, E=64, Ev=128, Hq=8, Hkv=4)
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.E_BAD_ARG
    p = good(diff=1, E=128, Ev=256, Hq=8, Hkv=8)   # the reference's d=128 test shape: two CTAs per item
    for name, w in (("v_stride", 256), ("o_stride", 256)):
        arr = getattr(p, name)
        arr[2], arr[1], arr[0] = w, w * 256, w * 256 * 4
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.OK
    p.Ev = 512
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.E_UNSUPPORTED


def test_workspace_bytes(lib):
    p = good(mask=_lib.MASK_DOCUMENT, document_id=FAKE, N=1, L=16384, S=16384)
    n = lib.flb200_attn_workspace_bytes(C.byref(p))
    # 128 q tiles x (2 int32 + 128 class bytes), one "sorted" flag per sequence, and two int32 run
    # bounds per position; each part rounded to 256 B
    assert n == 1024 + 128 * 128 + 256 + 16384 * 8
    p.workspace, p.workspace_bytes = FAKE, n - 1
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.E_WORKSPACE
    p.workspace_bytes = n
    assert lib.flb200_attn_validate(C.byref(p)) == _lib.OK
    assert lib.flb200_attn_workspace_bytes(C.byref(good())) == 0
    assert lib.flb200_attn_workspace_bytes(None) == 0


def test_decode_status(lib):
    bar, blk = C.c_int32(-1), C.c_int32(-1)
    assert lib.flb200_decode_status(0, C.byref(bar), C.byref(blk)) == _lib.OK
    word = (1 << 24) | (5 << 16) | 321
    assert lib.flb200_decode_status(word, C.byref(bar), C.byref(blk)) == _lib.E_TIMEOUT
    assert (bar.value, blk.value) == (5, 321)
    assert lib.flb200_decode_status(word, None, None) == _lib.E_TIMEOUT


def test_launch_without_device_fails_cleanly(lib):
    """On a box without a usable sm_100 device a launch returns an error code; it never
    falls back to another implementation and never aborts."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("needs a box without a GPU")
    before = lib.flb200_launch_count()
    rc = lib.flb200_attn_fwd(C.byref(good()), None)
    assert rc in (_lib.E_LAUNCH, _lib.E_ARCH)
    assert lib.flb200_launch_count() == before


def good_bwd(**over):
    p = _lib.AttnBwdParams()
    p.struct_size = C.sizeof(_lib.AttnBwdParams)
    p.N, p.Hq, p.Hkv, p.L, p.S, p.E = 2, 8, 2, 300, 300, 128
    for name in ("q", "k", "v", "o", "dout", "lse", "dq", "dk", "dv"):
        setattr(p, name, FAKE)
    for name, heads in (("q_stride", 8), ("o_stride", 8), ("do_stride", 8), ("dq_stride", 8),
                        ("k_stride", 2), ("v_stride", 2), ("dk_stride", 2), ("dv_stride", 2)):
        a = getattr(p, name)
        a[0], a[1], a[2] = heads * 300 * 128, 300 * 128, 128
    p.lse_stride[0], p.lse_stride[1] = 8 * 300, 300
    p.scale = 0.088
    p.workspace, p.workspace_bytes = FAKE, 1 << 30
    for k, v in over.items():
        if isinstance(v, tuple):
            arr = getattr(p, k)
            for i, x in enumerate(v):
                arr[i] = x
        else:
            setattr(p, k, v)
    return p


def test_backward_workspace_is_delta_plus_the_two_rows_of_the_extra_k_step(lib):
    lib.flb200_attn_bwd_workspace_bytes.restype = C.c_size_t
    # 300 query rows pad to 384; per padded row an fp32 delta and two rows of 16 bf16
    assert lib.flb200_attn_bwd_workspace_bytes(C.byref(good_bwd())) == 2 * 8 * 384 * (4 + 64)
    assert lib.flb200_attn_bwd_workspace_bytes(None) == 0


@pytest.mark.parametrize("over,code", [
    (dict(struct_size=8), _lib.E_BAD_ARG),
    (dict(Hkv=3), _lib.E_BAD_ARG),                       # query heads not a multiple of kv heads
    (dict(dq=None), _lib.E_BAD_ARG),
    (dict(scale=0.0), _lib.E_BAD_ARG),
    (dict(E=136), _lib.E_UNSUPPORTED),                   # backward kernels: head dims up to 128
    (dict(dk=FAKE + 8), _lib.E_MISALIGNED),
    (dict(q_stride=(8 * 300 * 128, 300 * 128, 132)), _lib.E_MISALIGNED),
    (dict(dv_stride=(2 * 300 * 128, 300 * 128, 64)), _lib.E_BAD_ARG),   # rows overlap
    (dict(lse_stride=(8 * 300, 100)), _lib.E_BAD_ARG),
    (dict(workspace_bytes=1024), _lib.E_WORKSPACE),
    (dict(workspace=FAKE + 64), _lib.E_MISALIGNED),
])
def test_backward_rejects_bad_problems_before_touching_the_device(lib, over, code):
    """Validation runs first and on the host: these calls return before any CUDA call."""
    lib.flb200_attn_bwd.restype = C.c_int
    assert lib.flb200_attn_bwd(C.byref(good_bwd(**over)), None) == code


def test_ipa_pack_rejects_bad_descriptions_on_the_host(lib):
    p = _lib.IpaPackParams()
    p.struct_size = C.sizeof(_lib.IpaPackParams)
    p.rows_q = p.rows_k = 64
    p.C, p.P_qk, p.P_v, p.point_dim = 16, 4, 8, 4
    for name in ("q_scalar", "k_scalar", "v_scalar", "q_points", "k_points", "v_points", "q_aug", "k_aug", "v_aug"):
        setattr(p, name, FAKE)
    p.a, p.E, p.Ev = -2.1, 48, 48          # E must hold 16 + 2 * 16 + 2 = 50 columns
    assert lib.flb200_ipa_pack(C.byref(p), None) == _lib.E_BAD_ARG
    p.E, p.Ev = 56, 44                     # widths are multiples of 8
    assert lib.flb200_ipa_pack(C.byref(p), None) == _lib.E_BAD_ARG
    p.Ev, p.k_points = 48, None
    assert lib.flb200_ipa_pack(C.byref(p), None) == _lib.E_BAD_ARG
    p.k_points, p.struct_size = FAKE, 12
    assert lib.flb200_ipa_pack(C.byref(p), None) == _lib.E_BAD_ARG


def _evo(D, S=384, rows=256, heads=8):
    """Evoformer-style description: bias 0 a key vector per row, bias 1 a pair bias shared by the rows."""
    p = good(N=rows, Hq=heads, Hkv=heads, L=S, S=S, E=D, Ev=D)
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        a = getattr(p, name)
        a[0], a[1], a[2] = S * heads * D, D, heads * D        # [rows, S, H, D] storage
    p.score_mod, p.bias_inner = _lib.SCORE_BIAS, rows
    p.bias[0] = p.bias[1] = FAKE
    for i, v in enumerate((0, S, 0, 0)):                        # strides {b, r, h, i}: one vector per row
        p.bias_stride[0][i] = v
    for i, v in enumerate((0, 0, S * S, S)):                    # one [S, S] matrix per head
        p.bias_stride[1][i] = v
    return p


def test_optional_scratch_of_the_resident_pair_bias_kernel(lib, monkeypatch):
    """4 KB of key-vector rows per (row, key tile) wherever an even number of ring slots fits beside them:
    heads of 32, heads of 64 with two bias tiles but not with three; the switch turns the path off."""
    monkeypatch.delenv("FLB200_KEYVEC_MMA", raising=False)
    assert lib.flb200_attn_validate(C.byref(_evo(32))) == _lib.OK
    assert lib.flb200_attn_workspace_bytes(C.byref(_evo(32))) == 256 * 3 * 4096
    assert lib.flb200_attn_workspace_bytes(C.byref(_evo(32, S=200))) == 256 * 2 * 4096
    assert lib.flb200_attn_workspace_bytes(C.byref(_evo(64))) == 0
    assert lib.flb200_attn_workspace_bytes(C.byref(_evo(64, S=256))) == 256 * 2 * 4096
    assert lib.flb200_attn_workspace_bytes(C.byref(_evo(32, rows=2))) == 0      # fewer than four rows share the pair bias
    assert lib.flb200_attn_workspace_bytes(C.byref(_evo(32, rows=16, heads=2))) == 0   # too little work for one more launch
    monkeypatch.setenv("FLB200_KEYVEC_MMA", "0")
    assert lib.flb200_attn_workspace_bytes(C.byref(_evo(32))) == 0


def test_optional_scratch_of_rms_normalised_differential_attention(lib, monkeypatch):
    """With the RMS normalisation and value heads up to 128 the P.V product can run in fp16: the call takes
    256 bytes of scratch for the word that receives max |v|; wider value heads (pairs of CTAs), no
    normalisation or the switch: none."""
    monkeypatch.delenv("FLB200_DIFF_PV_F16", raising=False)
    def diff(E, Ev, rms):
        p = good(Hq=8, Hkv=8, E=E, Ev=Ev, diff=1, diff_lambda=0.8, diff_rms_norm=rms, diff_rms_eps=1e-5)
        p.k_stride[0], p.k_stride[1], p.k_stride[2] = 8 * 256 * E, 256 * E, E
        p.q_stride[0], p.q_stride[1], p.q_stride[2] = 8 * 256 * E, 256 * E, E
        p.v_stride[0], p.v_stride[1], p.v_stride[2] = 4 * 256 * Ev, 256 * Ev, Ev
        p.o_stride[0], p.o_stride[1], p.o_stride[2] = 4 * 256 * Ev, 256 * Ev, Ev
        return p
    assert lib.flb200_attn_validate(C.byref(diff(64, 128, 1))) == _lib.OK
    assert lib.flb200_attn_workspace_bytes(C.byref(diff(64, 128, 1))) == 256
    assert lib.flb200_attn_workspace_bytes(C.byref(diff(32, 64, 1))) == 256
    assert lib.flb200_attn_workspace_bytes(C.byref(diff(64, 128, 0))) == 0
    assert lib.flb200_attn_workspace_bytes(C.byref(diff(128, 256, 1))) == 0
    monkeypatch.setenv("FLB200_DIFF_PV_F16", "0")
    assert lib.flb200_attn_workspace_bytes(C.byref(diff(64, 128, 1))) == 0
