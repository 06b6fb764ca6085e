import json
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def load_golden(name: str):
    """Returns (tensors, metadata) of tests/golden/<name>.safetensors."""
    from safetensors import safe_open

    tensors = {}
    with safe_open(str(GOLDEN / f"{name}.safetensors"), framework="pt", device="cpu") as f:
        meta = {k: json.loads(v) for k, v in (f.metadata() or {}).items()}
        for key in f.keys():
            tensors[key] = f.get_tensor(key)
    return tensors, meta


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def sort_topk(vals: torch.Tensor, idx: torch.Tensor):
    """Canonical (descending value) order for unsorted top-k results."""
    order = torch.argsort(vals, dim=-1, descending=True, stable=True)
    return vals.gather(-1, order), idx.gather(-1, order)


@pytest.fixture(scope="session")
def cuda_lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from sparsify_b200 import _lib

    return _lib.lib()
