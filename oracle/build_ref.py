"""Compile the reference's eager attention functions into `oracle/_ref/` (TEST INFRASTRUCTURE).

    python oracle/build_ref.py [/path/to/bozhiyou-flashlight]

The reference's hot path is pure Python (`attention_variants/*.py`), so "building" it means byte
compiling those files where they lie into sourceless modules, packed into one archive
`oracle/_ref/attention_variants.bin` (a zip of `attention_variants/*.pyc`, importable through
`sys.path` like any zip of modules).  No source is copied; the output directory is ignored by
git and travels with the built libraries.  `oracle/run_config.reference_runner` imports the modules
from there for the CPU baseline and the reference arm of `bench.py`, and
`tests/test_oracle_golden.py` checks the restatement in `attention_oracle.py` against them when
they are present.  The interpreter that compiled them must be the one that imports them (same
image on the build and the GPU box).
"""
import py_compile
import sys
import tempfile
import zipfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
ARCHIVE = "attention_variants.bin"
MODULES = ["__init__", "vanilla", "causal", "alibi", "softcap", "sliding_window", "document_mask", "prefix_lm",
           "diff_attn", "evoformer"]


def build(ref_root: str = "/root/reference") -> bool:
    src = Path(ref_root) / "attention_variants"
    if not src.is_dir():
        return False
    dst = HERE / "_ref"
    dst.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp, zipfile.ZipFile(dst / ARCHIVE, "w") as z:
        for name in MODULES:
            pyc = Path(tmp) / f"{name}.pyc"
            py_compile.compile(str(src / f"{name}.py"), cfile=str(pyc),
                               dfile=f"attention_variants/{name}.py", doraise=True)
            z.write(pyc, f"attention_variants/{name}.pyc")
    return True


if __name__ == "__main__":
    ok = build(*sys.argv[1:2])
    print("built oracle/_ref" if ok else "reference checkout not found: nothing built")
