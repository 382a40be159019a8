"""Shared pytest configuration: the ``gpu`` marker, import paths and golden-fixture loading."""

from __future__ import annotations

from pathlib import Path
import sys

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """Fixture file with typed accessors (bf16 / e4m3 are stored as integer views)."""

    def __init__(self, name: str):
        self._z = np.load(GOLDEN / name)

    def raw(self, key: str) -> torch.Tensor:
        return torch.from_numpy(np.array(self._z[key]))

    def bf16(self, key: str) -> torch.Tensor:
        return self.raw(key).view(torch.bfloat16)

    def f16(self, key: str) -> torch.Tensor:
        return self.raw(key).view(torch.float16)

    def typed(self, key: str, tag: str) -> torch.Tensor:
        """``tag`` in bf16 / f16 / f32."""
        return {"bf16": self.bf16, "f16": self.f16, "f32": self.raw}[tag](key)

    def e4m3(self, key: str) -> torch.Tensor:
        return self.raw(key).view(torch.float8_e4m3fn)

    def scalar(self, key: str):
        return self._z[key].item()


@pytest.fixture(scope="session")
def golden():
    return Golden
