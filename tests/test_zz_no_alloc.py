"""fhob_bwdbwd_static_scratch — the entry point for callers that cannot allocate.

Engines that own all device memory (one arena sized at start-up, another
framework's memory plan, latency-bound loops) may neither call cudaMalloc inside
an operator nor have a spare buffer to lend as workspace.  For them the library
keeps the operator's scratch in a fixed array of its own.  This file checks,
through the C ABI, that the variant gives the same four outputs as the regular
entry point on two calls in a row (the second call re-uses the array with the
first call's contents still in it), that it really ignores the workspace
fields, and that problems beyond the array's capacity are refused.

It sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
from __future__ import annotations

import ctypes as C

import pytest
import torch

from conftest import make_inputs
from fhob import _lib


@pytest.fixture(scope="module")
def lib():
    """The library, built first when the tree is fresh (same fixture as the C-ABI tests)."""
    import importlib.util
    from conftest import ROOT
    spec = importlib.util.spec_from_file_location("fhob_build", ROOT / "flash-hob_b200" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    return _lib.load()


def test_rows_beyond_capacity_are_refused(lib):
    p = _lib.FhobProblem()
    p.bh, p.n_q, p.n_k, p.d = 65, 4096, 4096, 128          # 266240 rows > 262144
    assert p.bh * p.n_q > _lib.STATIC_SCRATCH_MAX_ROWS
    assert lib.fhob_bwdbwd_static_scratch(C.byref(p), None) == 7
    assert b"FHOB_STATIC_SCRATCH_MAX_ROWS" in lib.fhob_strerror(7)
    assert lib.fhob_bwdbwd_static_scratch(None, None) == 1


@pytest.mark.gpu
def test_matches_regular_entry_point_on_two_calls_in_a_row(lib):
    import fhob
    from fhob.ops import _Problem
    from oracle import attn_oracle as O

    # The later problems are smaller than the first, causal, and have a ragged n_q (not a multiple
    # of 4 or 64): their padded row-vector slices and the tail the key-tiled pass reads past the
    # last head then hold the first call's values, which must not leak into the results.
    cases = [(4, 512, 768, 128, False, 101), (2, 256, 256, 64, True, 102), (3, 130, 131, 128, True, 103),
             (1, 99, 300, 64, True, 104)]
    for i, (bh, nq, nk, d, causal, seed) in enumerate(cases):
        x = make_inputs(bh, nq, nk, d, seed=seed, dtype=torch.bfloat16, device="cuda")
        scale = d ** -0.5
        o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], scale, is_causal=causal)
        args = (x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, scale)
        want = fhob.flash_bwdbwd(*args, is_causal=causal, check=True)

        prob = _Problem(*args, causal, "auto")           # fresh output tensors + the argument struct
        prob.p.workspace, prob.p.workspace_bytes = None, 0   # must not be needed
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        torch_before = torch.cuda.memory_allocated()
        st = lib.fhob_bwdbwd_static_scratch(C.byref(prob.p), C.c_void_p(prob.stream))
        assert st == 0, lib.fhob_strerror(st)
        assert lib.fhob_static_scratch_status(C.c_void_p(prob.stream)) == 0     # synchronises the stream
        if i > 0:
            # the claim itself: once the device has been set up by the first call, a call takes no
            # device memory, neither from the driver nor from torch's allocator
            assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.cuda.memory_allocated() == torch_before
        got = prob.outputs()
        for name, g, w in zip(("dq2", "dk2", "dv2", "ddo"), got, want):
            assert O.rel_err(g, w.float()) < 2e-2, name      # the tolerance of the bf16 parity tests
            assert torch.equal(g, w), name                    # same kernels, same order: bit-identical
