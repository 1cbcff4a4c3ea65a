"""Stages the reference's own CPU implementation of the quantizer path for timing (test infrastructure, not product).

    python oracle/stage_reference.py /path/to/mase/src/chop

MASE's quantizers are pure Python/PyTorch, so "building" the reference means making its `chop/nn/quantizers` package
importable on a machine that has no MASE checkout (the GPU box): this script copies that package, unmodified, into the
git-ignored `oracle/_ref/chop/nn/quantizers`.  `bench.py --impl reference` and the `cpu_baseline` leg then time the
reference itself (`kind: "reference"`); where `oracle/_ref` is absent they time the restatement in `mx_oracle.py`
(`kind: "port"`).  Nothing under `oracle/_ref` is committed, and no product code imports it.
"""

from __future__ import annotations

import importlib
import os
import shutil
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")
PACKAGE = os.path.join("nn", "quantizers")


def stage(chop_dir: str) -> str:
    src = os.path.join(chop_dir, PACKAGE)
    if not os.path.isdir(src):
        raise SystemExit(f"{src} is not a directory: pass the src/chop directory of a MASE checkout")
    dst = os.path.join(REF_ROOT, "chop", PACKAGE)
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.md"))
    return dst


def staged() -> bool:
    return os.path.isfile(os.path.join(REF_ROOT, "chop", PACKAGE, "__init__.py"))


def import_staged_quantizers():
    """`chop.nn.quantizers` of the staged copy.  The parent packages are registered empty (their own `__init__`
    files pull in plotting and training dependencies that the quantizers do not need)."""
    if not staged():
        raise ImportError("oracle/_ref holds no staged reference (run oracle/stage_reference.py where MASE is available)")
    root = os.path.join(REF_ROOT, "chop")
    for name, path in (("chop", root), ("chop.nn", os.path.join(root, "nn"))):
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__path__ = [path]
            sys.modules[name] = mod
    return importlib.import_module("chop.nn.quantizers")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(stage(sys.argv[1]))
