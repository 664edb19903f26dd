"""Shared pytest set-up: marker registration, import paths, seeded inputs."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "flash-hob_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def make_inputs(bh, nq, nk, d, seed, dtype=torch.float32, device="cpu", cot_scale=1.0, on_device=False):
    """Seven seeded N(0,1) tensors with bf16-representable values.

    Layout (BH, N, D) like the reference entry point.  ``cot_scale`` scales dO
    and the three cotangents (one benchmark configuration uses 0.1).  ``on_device``
    draws the numbers with the device's generator (for the multi-gigabyte cases).
    """
    gen_dev = device if on_device else "cpu"
    g = torch.Generator(device=gen_dev).manual_seed(seed)
    shapes = dict(q=(bh, nq, d), k=(bh, nk, d), v=(bh, nk, d), do=(bh, nq, d),
                  ddq=(bh, nq, d), ddk=(bh, nk, d), ddv=(bh, nk, d))
    out = {}
    for n, s in shapes.items():
        t = torch.randn(s, generator=g, dtype=torch.float32, device=gen_dev)
        if n in ("do", "ddq", "ddk", "ddv"):
            t = t * cot_scale
        out[n] = t.bfloat16().to(dtype).to(device)
    return out
