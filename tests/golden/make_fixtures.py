"""Regenerate tests/golden/operator_fixtures/ from the reference's own generator.

Runs the reference repository's `crates/inferrous-qwen3/tools/operator_fixtures.py`
UNMODIFIED (PyTorch CPU, seed 824, 8 threads) into a scratch directory and keeps
the cases that exercise the W8A8 linear-layer path: `norm`, `quantize`, `linear`,
`swiglu`, `residual`.  The attention / rope / head / embedding cases are dropped
(they are not on this path and are 20 MB).  File format is the reference's:
raw little-endian tensors + `manifest.json` with shape and sha256 per tensor
(operator_fixtures.py:23-34,83).

Usage:  python tests/golden/make_fixtures.py /path/to/reference-checkout

The reference checkout is only needed to REGENERATE; tests read the committed files.
"""
import json
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

KEEP = {"norm", "quantize", "linear", "swiglu", "residual"}


def main() -> None:
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    gen = ref / "crates/inferrous-qwen3/tools/operator_fixtures.py"
    out = Path(__file__).resolve().parent / "operator_fixtures"
    with tempfile.TemporaryDirectory() as tmp:
        scratch = Path(tmp) / "fx"
        subprocess.run([sys.executable, str(gen), str(scratch)], check=True)
        manifest = json.loads((scratch / "manifest.json").read_text())
        cases = [c for c in manifest["cases"] if c["op"] in KEEP]
        if out.exists():
            shutil.rmtree(out)
        out.mkdir(parents=True)
        for c in cases:
            for t in c["tensors"].values():
                shutil.copy(scratch / t["file"], out / t["file"])
        manifest["cases"] = cases
        manifest["kept_ops"] = sorted(KEEP)
        (out / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n")
    print(f"wrote {len(cases)} cases to {out}")


if __name__ == "__main__":
    main()
