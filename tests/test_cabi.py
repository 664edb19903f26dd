"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
header declares, and rejects bad problems before touching a GPU."""
from __future__ import annotations

import ctypes as C
import re

import pytest
import torch

from conftest import ROOT
from fhob import _lib


@pytest.fixture(scope="module")
def lib():
    import importlib.util
    spec = importlib.util.spec_from_file_location("fhob_build", ROOT / "flash-hob_b200" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    return _lib.load()


def test_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "fhob.h").read_text()
    declared = set(re.findall(r"\b(fhob_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.fhob_version() >= 100


def test_struct_matches_header(lib):
    header = (ROOT / "include" / "fhob.h").read_text()
    body = header.split("typedef struct FhobProblem {")[1].split("} FhobProblem;")[0]
    fields = re.findall(r"^\s*(?:const\s+)?(?:struct\s+)?[A-Za-z0-9_]+\*?\s+\*?([a-z0-9_]+);", body, flags=re.M)
    assert fields == [f[0] for f in _lib.FhobProblem._fields_]


def test_layout_struct_matches_header(lib):
    header = (ROOT / "include" / "fhob.h").read_text()
    body = header.split("typedef struct FhobLayout {")[1].split("} FhobLayout;")[0]
    fields = re.findall(r"^\s*[a-z0-9_]+\s+([a-z0-9_]+)(?:\[8\])?;", body, flags=re.M)
    assert fields == [f[0] for f in _lib.FhobLayout._fields_]
    assert C.sizeof(_lib.FhobLayout) == 8 + 3 * 8 * 8 + 16


def test_workspace_is_linear_in_rows(lib):
    w1 = lib.fhob_workspace_bytes(4, 1024)
    w2 = lib.fhob_workspace_bytes(4, 2048)
    w4 = lib.fhob_workspace_bytes(4, 4096)
    assert w2 - w1 == 4 * 1024 * 16 and w4 - w2 == 4 * 2048 * 16   # 4 fp32 row vectors
    assert lib.fhob_workspace_bytes(0, 5) == 0


def _problem(**over):
    """A well-formed problem over fake (never dereferenced) 256-byte aligned addresses."""
    p = _lib.FhobProblem()
    p.bh, p.n_q, p.n_k, p.d = 2, 128, 256, 64
    p.dtype, p.causal, p.impl, p.scale = _lib.FHOB_BF16, 0, 0, 0.125
    for i, name in enumerate(("q", "k", "v", "o", "d_o", "ddq", "ddk", "ddv", "lse", "dq2", "dk2", "dv2", "ddo")):
        setattr(p, name, 0x10000 + 0x1000 * i)
    p.workspace, p.workspace_bytes = 0x100000, 1 << 20
    for k, v in over.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("over,code", [
    (dict(q=None), 1), (dict(lse=None), 1), (dict(dq2=None), 1), (dict(bh=0), 1), (dict(dtype=7), 1),
    (dict(impl=9), 1), (dict(causal=2), 1),
    (dict(window=16), 1), (dict(causal=1, window=-1), 1), (dict(d_v=-8), 1),
    (dict(d=129), 2), (dict(d=4), 2), (dict(d=256), 2), (dict(d_v=4), 2), (dict(d_v=136), 2),
    (dict(impl=2, dtype=1, d=128), 2), (dict(impl=2, d=36), 2), (dict(impl=2, d_v=100), 2),
    (dict(impl=2, dtype=1, workspace_bytes=20000), 4),   # fp32 on the tensor cores needs room for the hi/lo copies
    (dict(k=0x10008), 3), (dict(ddo=0x20004), 3),
    (dict(workspace=None), 4), (dict(workspace_bytes=100), 4), (dict(workspace=0x100010), 4),
])
def test_bad_problems_are_rejected_before_launch(lib, over, code):
    p = _problem(**over)
    assert lib.fhob_bwdbwd(C.byref(p), None) == code
    assert lib.fhob_strerror(code) != b"unknown status"


def test_bad_layouts_are_rejected_before_launch(lib):
    def with_layout(**over):
        lay = _lib.FhobLayout()
        lay.heads = 2
        for i in range(8):
            lay.row[i], lay.head[i], lay.batch[i] = 128, 64, 128 * 256
        lay.lse_head, lay.lse_batch = 128, 256
        for k, v in over.items():
            if isinstance(v, tuple):
                getattr(lay, k)[v[0]] = v[1]
            else:
                setattr(lay, k, v)
        return lay
    cases = [(dict(heads=0), 1), (dict(heads=3), 1), (dict(reserved=1), 1), (dict(row=(1, 124)), 3), (dict(row=(0, 0)), 3),
             (dict(head=(2, 4)), 3), (dict(batch=(7, -8)), 3), (dict(lse_head=-1), 3)]
    for over, code in cases:
        lay = with_layout(**over)
        p = _problem()
        p.layout = C.pointer(lay)
        assert lib.fhob_bwdbwd(C.byref(p), None) == code, over
    lay = with_layout()
    p = _problem(impl=1)                    # views need the tensor-core kernels
    p.layout = C.pointer(lay)
    assert lib.fhob_bwdbwd(C.byref(p), None) == 2
    p = _problem(dtype=1, d=128)            # fp32 at head dim 128 runs on CUDA cores: no views
    p.layout = C.pointer(lay)
    assert lib.fhob_bwdbwd(C.byref(p), None) == 2


def test_null_problem(lib):
    assert lib.fhob_bwdbwd(None, None) == 1
    assert lib.fhob_pass3(None, None) == 1


def test_host_wrapper_validation():
    import fhob
    q = torch.zeros(2, 128, 64)
    with pytest.raises((RuntimeError, ValueError)):
        fhob.flash_bwdbwd(q, q, q, q, q, q, q, q, torch.zeros(2, 128), 0.125)  # CPU tensors, no GPU here
    if not torch.cuda.is_available():
        with pytest.raises(ValueError):
            fhob.ops._Problem(q, q, q, q, q, q, q, q, torch.zeros(2, 128), 0.125, False, "auto")
        with pytest.raises(ValueError):
            fhob.ops._Problem(q, q, q, q, q, q, q, q, torch.zeros(2, 128), 0.125, False, "fast")


def test_missing_library_is_loud(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libfhob.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_tile_range_rule_against_the_mask_definition(lib):
    """Exhaustive check of the streamed-tile range the kernels visit: it must contain every tile
    that holds a visible pair (otherwise results silently lose terms) and nothing beyond the
    first and last such tile (otherwise work is wasted)."""
    import itertools
    from oracle import attn_oracle as O
    import math
    tb, te = C.c_int(), C.c_int()
    checked = 0
    for n_q, n_k, window in itertools.product((5, 16, 37), (7, 16, 50), (0, 1, 6, 23)):
        for causal in ((1,) if window else (0, 1)):
            mask = O.bottom_right_mask(n_q, n_k, window if window else math.inf) if causal else None
            for rows, tile, q_stat in itertools.product((4, 16), (4, 8), (0, 1)):
                n_stat, n_strm = (n_q, n_k) if q_stat else (n_k, n_q)
                for m0 in range(0, n_stat, rows):
                    assert lib.fhob_visible_tiles(q_stat, m0, rows, tile, n_q, n_k, causal, window,
                                                  C.byref(tb), C.byref(te)) == 0
                    want = set()
                    for r in range(m0, min(m0 + rows, n_stat)):
                        for c in range(n_strm):
                            qi, kj = (r, c) if q_stat else (c, r)
                            if mask is None or bool(mask[qi, kj]):
                                want.add(c // tile)
                    n_tiles = -(-n_strm // tile)
                    assert 0 <= tb.value <= te.value <= n_tiles
                    if want:
                        assert tb.value <= min(want) and max(want) < te.value
                        # rows past the end of a ragged last stationary tile may widen the range, never shrink it
                        if m0 + rows <= n_stat:
                            assert (tb.value, te.value) == (min(want), max(want) + 1)
                    checked += 1
    assert checked > 1000


def test_custom_op_is_registered_and_infers_shapes_without_a_gpu():
    """torch.ops.fhob.bwdbwd exists and its shape-only implementation gives the four result shapes
    (this is what torch.compile traces; the reference relies on torch.compile, fhog/triton_bwdbwd.py:557)."""
    import torch
    import fhob  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        q = torch.empty(2, 3, 128, 64, dtype=torch.bfloat16)
        k = torch.empty(2, 3, 256, 64, dtype=torch.bfloat16)
        lse = torch.empty(2, 3, 128)
        out = torch.ops.fhob.bwdbwd(q, k, k, q, q, q, k, k, lse, 0.125, True, 0)
    assert [tuple(t.shape) for t in out] == [(2, 3, 128, 64), (2, 3, 256, 64), (2, 3, 256, 64), (2, 3, 128, 64)]
    assert all(t.dtype == torch.bfloat16 for t in out)
