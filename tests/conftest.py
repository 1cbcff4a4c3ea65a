import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def mase_chop_dir() -> str | None:
    """`src/chop` of a MASE checkout for the tests that run the reference itself: $MASE_CHOP_DIR, else a checkout
    named `reference` next to this repository.  None when there is none (those tests are skipped)."""
    for cand in (os.environ.get("MASE_CHOP_DIR"), os.path.join(os.path.dirname(ROOT), "reference", "src", "chop")):
        if cand and os.path.isdir(cand):
            return cand
    return None


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """Fixtures produced by running the MASE reference (tests/golden/make_golden.py); bit patterns."""

    def __init__(self):
        self.arrays = np.load(os.path.join(GOLDEN_DIR, "reference_vectors.npz"))
        with open(os.path.join(GOLDEN_DIR, "reference_vectors.json")) as fh:
            self.meta = json.load(fh)
        self.cases = self.meta["cases"]

    def tensor(self, key: str, dtype_name: str | None = None) -> torch.Tensor:
        """Array `key` as a torch tensor; float bit patterns are reinterpreted per `dtype_name`."""
        a = self.arrays[key]
        if a.dtype == np.uint16 and dtype_name in ("bf16", None):
            return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
        if a.dtype == np.uint32:
            return torch.from_numpy(a.view(np.int32).copy()).view(torch.float32)
        return torch.from_numpy(a.copy())


@pytest.fixture(scope="session")
def golden():
    return Golden()


def bits_of(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    return t


def assert_bits_equal(a: torch.Tensor, b: torch.Tensor, what: str = "", signed_zero: bool = True):
    """Exact equality of two tensors; NaN equals NaN.  With signed_zero=False, -0 equals +0."""
    a, b = a.detach().cpu(), b.detach().cpu()
    assert a.dtype == b.dtype, f"{what}: dtype {a.dtype} vs {b.dtype}"
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    if a.is_floating_point():
        both_nan = torch.isnan(a) & torch.isnan(b)
        same = (bits_of(a) == bits_of(b)) if signed_zero else (a == b)
        ok = same | both_nan
    else:
        ok = a == b
    if not bool(ok.all()):
        bad = (~ok).nonzero()
        i = tuple(bad[0].tolist())
        raise AssertionError(f"{what}: {bad.shape[0]} of {a.numel()} elements differ; first at {i}: {a[i]} vs {b[i]}")
