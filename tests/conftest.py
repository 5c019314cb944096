"""Shared pytest set-up: the ``gpu`` marker, import path, golden fixtures."""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """Build the shared library if the tree does not hold it yet (seconds with nvcc)."""
    from ayla_b200 import _lib
    from ayla_b200.build import build

    if not _lib.library_path().exists():
        build()


_TD = {"float16": torch.float16, "bfloat16": torch.bfloat16}


class GoldenCase:
    def __init__(self, meta: dict, arrays):
        self.__dict__.update(meta)
        self.torch_dtype = _TD[meta["dtype"]]
        self._arrays = arrays

    def tensor(self, key: str) -> torch.Tensor:
        arr = self._arrays[f"{self.name}/{key}"]
        return torch.from_numpy(np.ascontiguousarray(arr)).view(self.torch_dtype)

    def operands(self) -> tuple[torch.Tensor, ...]:
        if self.operation == "addmm":
            return (self.tensor("bias"), self.tensor("a"), self.tensor("bt"))
        if self.operation == "swiglu":
            return (self.tensor("a"), self.tensor("bt"), self.tensor("wu"))
        return (self.tensor("a"), self.tensor("bt"))

    def expected(self) -> torch.Tensor:
        return self.tensor("out")

    def __repr__(self) -> str:
        return self.name


def load_golden_cases() -> list[GoldenCase]:
    arrays = np.load(GOLDEN / "gemm_vectors.npz")
    meta = json.loads(bytes(arrays["meta"]).decode())
    return [GoldenCase(m, arrays) for m in meta]


@pytest.fixture(scope="session")
def reference_api() -> dict:
    return json.loads((GOLDEN / "reference_api.json").read_text())
