"""Differential-attention sweep with the grid, FLOP estimate and CSV columns of the reference's
`benchmarks/run_diff_attn.py` (`:42-84` loop, `:93-103` grid): q, k [B, H, S, D], v [B, H/2, S, 2D],
H = dim // D, FLOPs counted as twice a vanilla attention (8 * B * S^2 * H * D).

    python -m flashlight_b200.benchmarks.run_diff_attn --output diff_attn

Head dimension 128 (value heads of 256) runs as pairs of CTAs that take one half of the value
columns each.  A shape without a kernel would be reported as `nan`, never computed some other way.
"""
from __future__ import annotations

import argparse
import os

import torch

from .. import attention_variants as av
from ._utils import Config, Result, do_bench, efficiency, print_results, write_results_csv

DEFAULT = {
    "batch_sizes": [32, 16, 8, 4, 2, 1],
    "seq_lengths": [512, 1024, 2048, 4096, 8192, 16384],
    "head_dims": [64, 128],
    "model_dim": 2048,
}


def make_input(config: Config, device="cuda", seed: int = 0):
    """As `attention_variants/diff_attn.py:33-38` of the reference, seeded."""
    batch_size, seqlen, nheads, headdim, _, _ = config
    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda *shape: torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    return (mk(batch_size, nheads, seqlen, headdim), mk(batch_size, nheads, seqlen, headdim),
            mk(batch_size, nheads // 2, seqlen, headdim * 2))


def main(args) -> list:
    name = torch.cuda.get_device_name(0).upper()
    gpu_label = next((tag for tag in ("B200", "H100", "A100") if tag in name), "unknown")
    all_results = []
    for headdim in args.headdim:
        for batch_size, seqlen in zip(args.batch_size, args.seqlen):
            nheads = args.dim // headdim
            config = Config(batch_size, seqlen, nheads, headdim, 1, args.dropout_p)
            print(f"### Config: {config} ###")
            flop_fwd = 8 * batch_size * seqlen ** 2 * nheads * headdim  # estimate as double vanilla
            q, k, v = make_input(config)
            try:
                time_ms = do_bench(lambda: av.diffattn(q, k, v), n_warmup=args.warmup, n_repeat=args.repeat)
                tflops = efficiency(flop_fwd, time_ms)
            except NotImplementedError as e:  # shape no kernel is built for: there is no fallback
                print(f"  unsupported: {e}")
                time_ms = tflops = float("nan")
            rows = [[*Result("diffattn", time_ms, tflops), *config, gpu_label]]
            print_results(rows)
            all_results.extend(rows)
            del q, k, v
    out = args.output if os.path.isabs(args.output) else os.path.join(os.getcwd(), args.output)
    write_results_csv(all_results, f"{out}.csv", extra_headers=["GPU"])
    print(f"wrote {out}.csv")
    return all_results


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Differential attention benchmark (flashlight_b200 kernels)")
    p.add_argument("--batch_size", type=int, nargs="+", default=DEFAULT["batch_sizes"], help="Batch size")
    p.add_argument("--seqlen", type=int, nargs="+", default=DEFAULT["seq_lengths"], help="Sequence length")
    p.add_argument("--dim", type=int, default=DEFAULT["model_dim"], help="Input dimension")
    p.add_argument("--headdim", type=int, nargs="+", default=DEFAULT["head_dims"], help="Head dimension")
    p.add_argument("--dropout_p", type=float, default=0.0, help="Dropout probability (must be 0)")
    p.add_argument("--skip_correctness", action="store_true",
                   help="accepted for compatibility; parity is the job of the test suite")
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--repeat", type=int, default=20)
    p.add_argument("--output", type=str, default="diff_attn", help="output file name, `.csv` is appended")
    return p.parse_args(argv)


if __name__ == "__main__":
    main(parse_args())
