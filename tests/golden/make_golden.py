"""Generate golden vectors from the reference's own eager implementation.

Run once in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/bozhiyou-flashlight

It imports the reference's `attention_variants` package unchanged, feeds it seeded bf16-rounded
inputs upcast to fp32 on the CPU (the reference tests' own oracle procedure,
tests/test_causal.py:32) and stores inputs and outputs in `tests/golden/*.pt`.  The files are
small (tens of KB each) and are what pins `oracle/attention_oracle.py`; the GPU parity tests
compare against them as well.
"""
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent


def rnd(g, *shape):
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(torch.bfloat16)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from attention_variants import vanilla, causal, alibi, softcap, sliding_window, document_mask, prefix_lm
    from attention_variants import diff_attn, evoformer

    g = torch.Generator().manual_seed(20240607)
    cases = {}

    def qkv(N, Hq, Hkv, L, E, Ev=None):
        Ev = E if Ev is None else Ev
        return rnd(g, N, Hq, L, E), rnd(g, N, Hkv, L, E), rnd(g, N, Hkv, L, Ev)

    def f32(*ts):
        return [t.float() for t in ts]

    # vanilla, no GQA and GQA (vanilla.py:4-35)
    q, k, v = qkv(2, 2, 2, 160, 64)
    cases["vanilla_nogqa"] = dict(q=q, k=k, v=v, out=vanilla.attention_pytorch_nogqa(*f32(q, k, v)))
    q, k, v = qkv(1, 4, 2, 200, 64)
    cases["vanilla_gqa"] = dict(q=q, k=k, v=v, out=vanilla.attention_pytorch(*f32(q, k, v), enable_gqa=True))
    # causal (causal.py:4-36)
    q, k, v = qkv(1, 2, 2, 300, 128)
    cases["causal"] = dict(q=q, k=k, v=v, out=causal.attention_pytorch_causal(*f32(q, k, v)))
    q, k, v = qkv(2, 4, 1, 130, 64)
    cases["causal_gqa"] = dict(q=q, k=k, v=v, out=causal.attention_pytorch_causal(*f32(q, k, v), enable_gqa=True))
    # ALiBi (alibi.py:13-33); the default generator hard-codes device='cuda' (alibi.py:5,11)
    q, k, v = qkv(1, 4, 4, 257, 64)
    sm = lambda ql, kl: alibi.alibi_bias(4, ql, kl, device="cpu")
    cases["alibi"] = dict(q=q, k=k, v=v, nheads=4, out=alibi.attention_pytorch_alibi(*f32(q, k, v), score_mod=sm))
    q, k, v = qkv(1, 8, 2, 129, 64)
    sm8 = lambda ql, kl: alibi.alibi_bias(8, ql, kl, device="cpu")
    cases["alibi_gqa"] = dict(q=q, k=k, v=v, nheads=8,
                              out=alibi.attention_pytorch_alibi(*f32(q, k, v), score_mod=sm8, enable_gqa=True))
    # softcap (softcap.py:4-53) with score_mod = cap * tanh(score / cap)
    q, k, v = qkv(1, 2, 2, 190, 128)
    cap = 5.0
    cases["softcap"] = dict(q=q, k=k, v=v, cap=cap, out=softcap.attention_softcapped(
        *f32(q, k, v), lambda s, b, h, qq, kk: cap * torch.tanh(s / cap)))
    # sliding window (sliding_window.py:14-44)
    q, k, v = qkv(1, 2, 2, 400, 64)
    cases["sliding"] = dict(q=q, k=k, v=v, window=100,
                            out=sliding_window.attention_pytorch_sliding_window(*f32(q, k, v), window_size=100))
    # document mask (document_mask.py:6-41): sorted ids and an unsorted id vector
    q, k, v = qkv(2, 2, 2, 384, 64)
    lens = torch.tensor([90, 7, 130, 157])
    doc = torch.repeat_interleave(torch.arange(4), lens).unsqueeze(0).expand(2, -1).contiguous()
    cases["document"] = dict(q=q, k=k, v=v, document_id=doc,
                             out=document_mask.attention_pytorch_document_mask(*f32(q, k, v), doc))
    doc_u = torch.randint(0, 3, (2, 384), generator=g)
    cases["document_unsorted"] = dict(q=q, k=k, v=v, document_id=doc_u,
                                      out=document_mask.attention_pytorch_document_mask(*f32(q, k, v), doc_u))
    # prefix-LM (prefix_lm.py:5-42), int prefix as the reference requires
    q, k, v = qkv(2, 2, 2, 300, 64)
    cases["prefix"] = dict(q=q, k=k, v=v, prefix=150,
                           out=prefix_lm.attention_pytorch_prefix_lm(*f32(q, k, v), prefix_lengths=150))
    # differential attention (diff_attn.py:6-30)
    q, k = rnd(g, 1, 4, 260, 64), rnd(g, 1, 4, 260, 64)
    v = rnd(g, 1, 2, 260, 128)
    cases["diff"] = dict(q=q, k=k, v=v, lam=0.2, out=diff_attn.diffattn(*f32(q, k, v)))
    cases["diff_l08"] = dict(q=q, k=k, v=v, lam=0.8, out=diff_attn.diffattn(*f32(q, k, v), lambda_full=0.8))
    # Evoformer (evoformer.py:8-36): [B, N, S, H, D], biases [B,N,1,1,S] and [B,1,H,S,S]
    B, N, S, H, D = 1, 3, 150, 2, 32
    q, k, v = rnd(g, B, N, S, H, D), rnd(g, B, N, S, H, D), rnd(g, B, N, S, H, D)
    b1, b2 = rnd(g, B, N, 1, 1, S), rnd(g, B, 1, H, S, S)
    cases["evoformer"] = dict(q=q, k=k, v=v, bias1=b1, bias2=b2,
                              out=evoformer.attention_reference(*f32(q, k, v), [b1.float(), b2.float()]))
    keep = torch.rand(B, N, 1, 1, S, generator=g) < 0.9
    bm = torch.where(keep, 0.0, float("-inf")).to(torch.bfloat16)
    cases["evoformer_mask"] = dict(q=q, k=k, v=v, bias1=bm, bias2=b2,
                                   out=evoformer.attention_reference(*f32(q, k, v), [bm.float(), b2.float()]))

    # differential attention at q/k width 128, value width 256: the reference's own test shape family
    # (tests/test_diffattn.py:25-34); drawn after every other case so that those keep their values
    q, k = rnd(g, 1, 4, 200, 128), rnd(g, 1, 4, 200, 128)
    v = rnd(g, 1, 2, 200, 256)
    cases["diff_d128"] = dict(q=q, k=k, v=v, lam=0.2, out=diff_attn.diffattn(*f32(q, k, v)))

    # invariant point attention: the function lives in the reference's test file (tests/test_ipa.py:57-125)
    # and ends by adding the scalar output [B, H, N, C] to the point output [B, N, H, P_v, 4], which
    # broadcasts only when C == 4, B == 1 and N == P_v.  At such a shape the unmodified function is run
    # twice, once per zeroed value operand, and each aggregate is read out of the sum.
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_test_ipa", str(Path(ref_root) / "tests" / "test_ipa.py"))
    ipa_mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ipa_mod)
    H, N, C, Pqk = 3, 24, 4, 4
    qs, ks, vs = rnd(g, 1, H, N, C), rnd(g, 1, H, N, C), rnd(g, 1, H, N, C)
    qp, kp, vp = rnd(g, 1, H, N, Pqk, 4), rnd(g, 1, H, N, Pqk, 4), rnd(g, 1, H, N, N, 4)
    pb = rnd(g, 1, H, N, N)
    # the function builds a per-head view of the frames and never uses it (test_ipa.py:77-88)
    frames = ipa_mod.Rigid(torch.nn.functional.normalize(rnd(g, 1, N, 4).float(), dim=-1), rnd(g, 1, N, 3).float())
    ipa = lambda v_s, v_p: ipa_mod.invariant_point_attention(
        *f32(qs, ks, v_s, qp, kp, v_p, pb), frames, torch.ones(1, N), c_hidden=C, no_qk_points=Pqk)
    points = ipa(torch.zeros_like(vs), vp)           # [1, N, H, P_v, 4]
    scalar = ipa(vs, torch.zeros_like(vp))[0, 0]     # [H, N(=P_v), C(=4)], the same for every query row
    cases["ipa"] = dict(q=qs, k=ks, v=vs, q_points=qp, k_points=kp, v_points=vp, pair_bias=pb, c_hidden=C,
                        no_qk_points=Pqk, out=scalar.unsqueeze(0), out_points=points)

    for name, c in cases.items():
        c["out"] = c["out"].contiguous()
        torch.save(c, HERE / f"{name}.pt")
        print(name, tuple(c["out"].shape), f"{(HERE / (name + '.pt')).stat().st_size / 1024:.0f} KB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/bozhiyou-flashlight")
    main(sys.argv[1])
