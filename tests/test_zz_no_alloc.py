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


def test_rows_beyond_capacity_are_refused():
    lib = _lib.load()
    p = _lib.FhobProblem()
    p.bh, p.n_q, p.n_k, p.d = 65, 4096, 4096, 128          # 266240 rows > 262144
    assert p.bh * p.n_q > _lib.STATIC_SCRATCH_MAX_ROWS
    assert lib.fhob_bwdbwd_static_scratch(C.byref(p), None) == 7
    assert b"FHOB_STATIC_SCRATCH_MAX_ROWS" in lib.fhob_strerror(7)
    assert lib.fhob_bwdbwd_static_scratch(None, None) == 1


@pytest.mark.gpu
def test_matches_regular_entry_point_on_two_calls_in_a_row():
    import fhob
    from fhob.ops import _Problem
    from oracle import attn_oracle as O

    lib = _lib.load()
    # second problem is smaller and causal, so stale row vectors of the first call would show
    cases = [(4, 512, 768, 128, False, 101), (2, 256, 256, 64, True, 102)]
    for bh, nq, nk, d, causal, seed in cases:
        x = make_inputs(bh, nq, nk, d, seed=seed, dtype=torch.bfloat16, device="cuda")
        scale = d ** -0.5
        o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], scale, is_causal=causal)
        args = (x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, scale)
        want = fhob.flash_bwdbwd(*args, is_causal=causal, check=True)

        prob = _Problem(*args, causal, "auto")           # fresh output tensors + the argument struct
        prob.p.workspace, prob.p.workspace_bytes = None, 0   # must not be needed
        st = lib.fhob_bwdbwd_static_scratch(C.byref(prob.p), C.c_void_p(prob.stream))
        assert st == 0, lib.fhob_strerror(st)
        torch.cuda.synchronize()
        got = prob.outputs()
        for name, g, w in zip(("dq2", "dk2", "dv2", "ddo"), got, want):
            assert O.rel_err(g, w.float()) < 2e-2, name      # the tolerance of the bf16 parity tests
            assert torch.equal(g, w), name                    # same kernels, same order: bit-identical
