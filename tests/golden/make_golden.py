"""Regenerates the committed golden fixtures in this folder.

Needs the reference checkout (pass its path as argv[1]); the fixtures
themselves are committed, so the test-suite never needs it.

1. ``fhog_test_data.npz`` — the reference's own known-answer vectors
   (``test_data.zip``: 9 inputs + 4 outputs, nq=128, nkv=256, D=64, non-causal,
   produced by fhog/jax_refs/jax_impl.py:422-505 with the LSE-based closed form
   and consumed by fhog/test_bwdbwd.py:27-82), repacked from torch ``.pt`` to
   one ``.npz`` with the values untouched (fp32).

2. ``ref_torch_closed_form.npz`` — outputs of the reference's torch
   restatement ``attn_bwd_bwd_torch`` (fhog/jax_refs/torch_impl.py:14-79),
   executed from the reference checkout on seeded inputs (fp64, non-causal:
   its causal branch is commented out there).  That file imports ``jax.numpy``
   at module level but the function uses torch only, so an empty stand-in
   module named ``jax`` is registered before the file is loaded by path.
"""
from __future__ import annotations

import importlib.util
import io
import sys
import types
import zipfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

# (name, nq, nk, d, seed) of the seeded cases run through the reference's torch code
TORCH_CASES = [
    ("nc_128x256_d64", 128, 256, 64, 11),
    ("nc_128x128_d128", 128, 128, 128, 13),
]


def seeded_inputs(nq, nk, d, seed, dtype=torch.float64):
    """Seven N(0,1) tensors rounded to bf16-representable values."""
    g = torch.Generator().manual_seed(seed)
    shapes = dict(q=(nq, d), k=(nk, d), v=(nk, d), do=(nq, d), ddq=(nq, d), ddk=(nk, d), ddv=(nk, d))
    return {n: torch.randn(s, generator=g, dtype=torch.float32).bfloat16().to(dtype)
            for n, s in shapes.items()}


def repack_test_data(ref_root: Path) -> None:
    out = {}
    with zipfile.ZipFile(ref_root / "test_data.zip") as z:
        for name in z.namelist():
            if name.endswith(".pt"):
                t = torch.load(io.BytesIO(z.read(name)), map_location="cpu")
                out[Path(name).stem] = t.numpy()
    np.savez_compressed(HERE / "fhog_test_data.npz", **out)
    print("fhog_test_data.npz:", {k: v.shape for k, v in out.items()})


def run_reference_torch(ref_root: Path) -> None:
    for stub in ("jax", "jax.numpy"):
        sys.modules.setdefault(stub, types.ModuleType(stub))
    spec = importlib.util.spec_from_file_location(
        "ref_torch_impl", ref_root / "fhog" / "jax_refs" / "torch_impl.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = {}
    for name, nq, nk, d, seed in TORCH_CASES:
        x = seeded_inputs(nq, nk, d, seed)
        scale = torch.tensor(1.0 / d ** 0.5, dtype=torch.float64)
        s = (x["q"] @ x["k"].T) * scale
        lse = torch.logsumexp(s, dim=-1)
        o = torch.softmax(s, dim=-1) @ x["v"]
        dq2, dk2, dv2, ddo = mod.attn_bwd_bwd_torch(
            stats=lse, q=x["q"], k=x["k"], v=x["v"], o=o, do=x["do"],
            ddq=x["ddq"], ddk=x["ddk"], ddv=x["ddv"], scale=scale, is_causal=False)
        for n, t in dict(dq2=dq2, dk2=dk2, dv2=dv2, ddo=ddo).items():
            out[f"{name}/{n}"] = t.numpy()
        out[f"{name}/meta"] = np.array([nq, nk, d, seed])
    np.savez_compressed(HERE / "ref_torch_closed_form.npz", **out)
    print("ref_torch_closed_form.npz:", sorted(out))


if __name__ == "__main__":
    root = Path(sys.argv[1])
    repack_test_data(root)
    run_reference_torch(root)
