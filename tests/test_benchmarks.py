"""The benchmark sweeps that mirror the reference's `benchmarks/run_flex_variants.py` and
`benchmarks/run_diff_attn.py`: FLOP counting and CSV format on the CPU, a tiny sweep on the GPU."""
import csv

import pytest
import torch

from flashlight_b200.benchmarks import _utils as U
from flashlight_b200.benchmarks import run_diff_attn as RD
from flashlight_b200.benchmarks import run_evoformer as RE
from flashlight_b200.benchmarks import run_flex_variants as RF


def test_flop_formula_matches_reference_convention():
    # 4 * B * S^2 * H * D, halved when causal (reference benchmarks/_utils.py:16-21)
    assert U.attention_nflop(2, 1024, 64, 16) == 4 * 2 * 1024 ** 2 * 16 * 64
    assert U.attention_nflop(2, 1024, 64, 16, causal=True) == 2 * 2 * 1024 ** 2 * 16 * 64
    assert U.attention_nflop(1, 512, 64, 8, mode="bwd") == 2.5 * 4 * 512 ** 2 * 8 * 64


@pytest.mark.parametrize("seqlen", [512, 1000])
def test_block_sparsity_against_brute_force(seqlen):
    keep = lambda i, j: (j <= i) & (i - j <= 256)
    i = torch.arange(seqlen).view(-1, 1)
    j = torch.arange(seqlen).view(1, -1)
    full = keep(i, j)
    nb = (seqlen + 127) // 128
    empty = 0
    for a in range(nb):
        for b in range(nb):
            empty += int(not full[a * 128:(a + 1) * 128, b * 128:(b + 1) * 128].any())
    assert U.block_sparsity(keep, seqlen) == pytest.approx(100.0 * empty / nb ** 2)


def test_variant_flops():
    c = U.Config(2, 1024, 16, 64, 1, 0.0)
    dense = U.attention_nflop(2, 1024, 16, 64)
    assert RF.variant_flops("full", c) == dense
    assert RF.variant_flops("full_with_alibi", c) == dense
    assert RF.variant_flops("full_with_causal", c) == dense // 2
    # window 256 at S = 1024: the diagonal and two sub-diagonals of the 8 x 8 tile grid
    assert RF.variant_flops("full_with_sliding_window", c) == pytest.approx(dense * 21 / 64)
    assert 0 < RF.variant_flops("full_with_document_mask", c) < dense
    assert RF.variant_flops("full_with_prefix_lm", c) > dense / 2


def test_registry_names_and_cli_defaults():
    assert list(RF.registry()) == [
        "full", "full_with_alibi", "full_with_softcap", "full_with_causal",
        "full_with_sliding_window", "full_with_prefix_lm", "full_with_document_mask"]
    a = RF.parse_args([])
    assert (a.batch_size, a.seqlen) == ([32, 16, 8, 4, 2, 1], [512, 1024, 2048, 4096, 8192, 16384])
    assert (a.dim, a.headdim, a.group_size) == (1024, [64], [1, 8])
    f = RF.parse_args(["--grid", "flash"])
    assert (f.dim, f.headdim, f.group_size) == (2048, [64, 128], [1])
    d = RD.parse_args([])
    assert (d.dim, d.headdim) == (2048, [64, 128])
    e = RE.parse_args([])
    assert (e.seqlen, e.headdim, RE.N_ROWS) == ([256] * 6, [64, 128], 256)


def test_csv_columns(tmp_path):
    rows = [["full", 1.5, 100.0, 2, 1024, 16, 64, 1, 0.0]]
    U.write_results_csv(rows, str(tmp_path / "r.csv"))
    got = list(csv.reader(open(tmp_path / "r.csv")))
    assert got[0] == ["Implementation", "FW_Time_ms", "FW_TFLOPS", "batch_size", "seqlen", "nheads",
                      "headdim", "group_size", "dropout_p"]
    assert got[1][0] == "full" and float(got[1][2]) == 100.0
    with pytest.raises(ValueError):
        U.write_results_csv([["full", 1.0]], str(tmp_path / "bad.csv"))


@pytest.mark.gpu
def test_tiny_flex_sweep(tmp_path):
    args = RF.parse_args(["--batch_size", "2", "--seqlen", "512", "--group_size", "1", "8",
                          "--warmup", "1", "--repeat", "2", "--output", str(tmp_path / "b")])
    rows = RF.main(args)
    assert len(rows) == 14  # seven variants x two group sizes
    assert all(r[1] > 0 and r[2] > 0 for r in rows)
    assert len(list(csv.reader(open(tmp_path / "b.csv")))) == 15


@pytest.mark.gpu
def test_tiny_diff_sweep(tmp_path):
    args = RD.parse_args(["--batch_size", "1", "--seqlen", "512", "--warmup", "1", "--repeat", "2",
                          "--output", str(tmp_path / "d")])
    rows = RD.main(args)
    assert [r[6] for r in rows] == [64, 128]
    assert rows[0][1] > 0 and rows[1][1] > 0    # head dims 64 and 128 (value heads of 128 and 256) both run
    assert rows[0][-1] in ("B200", "unknown")


@pytest.mark.gpu
def test_tiny_evoformer_sweep(tmp_path):
    args = RE.parse_args(["--batch_size", "1", "--seqlen", "256", "--warmup", "1", "--repeat", "2",
                          "--output", str(tmp_path / "e")])
    rows = RE.main(args)
    assert [(r[4], r[5], r[6]) for r in rows] == [(256, 4, 64), (256, 4, 128)]   # seqlen, heads, head dim
    assert all(r[1] > 0 and r[2] > 0 for r in rows)
    # the call the sweep times gives the oracle's result
    from oracle import attention_oracle as ao
    q, k, v, biases = RE.make_input(RE.Config(1, 256, 4, 64, 1, 0.0))
    out = RE.av.attention_reference(q[:, :8], k[:, :8], v[:, :8], [biases[0][:, :8], biases[1]])
    ref = ao.evoformer(q[:, :8], k[:, :8], v[:, :8], [biases[0][:, :8], biases[1]])
    assert (out.float() - ref.float()).abs().max().item() <= 2e-2 + 2 ** -8 * ref.abs().max().item()
