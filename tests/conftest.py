import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden" / "operator_fixtures"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


class Fixtures:
    """Reader for the reference's fixture format (tools/operator_fixtures.py:23-34,83):
    raw little-endian tensors, dtype implied by the key, shape and sha256 in manifest.json."""

    DTYPES = {"q": np.int8, "w": np.int8}
    # bf16 tensors are stored as their bit patterns (operator_fixtures.py:26-27)
    OP_DTYPES = {("attention", "q"): np.float32, ("attention", "k"): np.uint16, ("attention", "v"): np.uint16,
                 ("embedding", "ids"): np.uint32, ("embedding", "w"): np.uint16}

    def __init__(self, root: Path):
        self.root = root
        self.manifest = json.loads((root / "manifest.json").read_text())

    def cases(self, op: str):
        return [c for c in self.manifest["cases"] if c["op"] == op]

    def tensor(self, case, key: str) -> np.ndarray:
        import hashlib

        meta = case["tensors"][key]
        raw = (self.root / meta["file"]).read_bytes()
        assert hashlib.sha256(raw).hexdigest() == meta["sha256"], f"fixture hash: {meta['file']}"
        dtype = self.OP_DTYPES.get((case["op"], key), self.DTYPES.get(key, np.float32))
        return np.frombuffer(raw, dtype=dtype).reshape(meta["shape"]).copy()


@pytest.fixture(scope="session")
def fixtures() -> Fixtures:
    return Fixtures(GOLDEN)
