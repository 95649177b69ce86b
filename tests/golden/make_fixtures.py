"""Regenerate tests/golden/operator_fixtures/ from the reference's own generator.

Runs the reference repository's `crates/inferrous-qwen3/tools/operator_fixtures.py`
UNMODIFIED (PyTorch CPU, seed 824, 8 threads) into a scratch directory and keeps
the cases that exercise the W8A8 linear-layer path (`norm`, `quantize`, `linear`,
`swiglu`, `residual`) and the operators around it (`rope`, `attention`, `embedding`, `head`).
To keep the committed files small, the rope case's 2 MB table (4096 positions) is cut
to the rows the case reads (tensor `table_rows`, first row = `position`), and the
attention case at position 4095 (16 MB of keys and values) is dropped.  File format is the reference's:
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

import hashlib

import numpy as np

KEEP = {"norm", "quantize", "linear", "swiglu", "residual", "rope", "attention", "embedding", "head"}
MAX_ATTENTION_POSITION = 1024


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_fixtures.py /path/to/reference-checkout")
    ref = Path(sys.argv[1])
    gen = ref / "crates/inferrous-qwen3/tools/operator_fixtures.py"
    out = Path(__file__).resolve().parent / "operator_fixtures"
    with tempfile.TemporaryDirectory() as tmp:
        scratch = Path(tmp) / "fx"
        subprocess.run([sys.executable, str(gen), str(scratch)], check=True)
        manifest = json.loads((scratch / "manifest.json").read_text())
        cases = [c for c in manifest["cases"] if c["op"] in KEEP
                 and not (c["op"] == "attention" and c["position"] > MAX_ATTENTION_POSITION)]
        if out.exists():
            shutil.rmtree(out)
        out.mkdir(parents=True)
        for c in cases:
            if c["op"] == "rope":
                meta = c["tensors"].pop("table")
                rows = c["tensors"]["x"]["shape"][0]
                table = np.frombuffer((scratch / meta["file"]).read_bytes(), np.float32).reshape(meta["shape"])
                raw = table[c["position"]:c["position"] + rows].tobytes()
                name = meta["file"].replace("-table", "-table_rows")
                (out / name).write_bytes(raw)
                c["tensors"]["table_rows"] = dict(file=name, shape=[rows, meta["shape"][1]], sha256=hashlib.sha256(raw).hexdigest(),
                                                  full_table_sha256=meta["sha256"])
            for t in c["tensors"].values():
                if not (out / t["file"]).exists():
                    shutil.copy(scratch / t["file"], out / t["file"])
        manifest["cases"] = cases
        manifest["kept_ops"] = sorted(KEEP)
        (out / "manifest.json").write_text(json.dumps(manifest, indent=2) + "\n")
    print(f"wrote {len(cases)} cases to {out}")


if __name__ == "__main__":
    main()
