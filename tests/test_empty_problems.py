"""Problems without any work (an empty batch, no queries, no keys) launch nothing and have defined
results: every result element is a sum over nothing, i.e. zero; the logsumexp of no scores is -inf.
No GPU needed: the entry points return before anything is loaded."""
from __future__ import annotations

import pytest
import torch

import fhob


@pytest.mark.parametrize("bh,nq,nk", [(0, 16, 8), (2, 0, 8), (2, 16, 0)])
def test_operator_on_empty_problems(bh, nq, nk):
    q, k = torch.ones(bh, nq, 64, dtype=torch.bfloat16), torch.ones(bh, nk, 64, dtype=torch.bfloat16)
    v, do = torch.ones(bh, nk, 32, dtype=torch.bfloat16), torch.ones(bh, nq, 32, dtype=torch.bfloat16)
    lse = torch.zeros(bh, nq)
    got = fhob.flash_bwdbwd(q, k, v, do, do, q, k, v, lse, 0.125)
    for g, like in zip(got, (q, k, v, do)):
        assert g.shape == like.shape and g.dtype == like.dtype and not g.any()
    out = tuple(torch.ones_like(t) for t in (q, k, v, do))
    again = fhob.flash_bwdbwd(q, k, v, do, do, q, k, v, lse, 0.125, out=out)
    for g, o in zip(again, out):
        assert g is o and not g.any()


def test_first_order_entry_points_on_empty_problems():
    q, k, v = torch.ones(2, 16, 64), torch.ones(2, 0, 64), torch.ones(2, 0, 32)
    dq, dk, dv = fhob.attention_backward(q, k, v, torch.zeros(2, 16, 32), torch.ones(2, 16, 32), torch.zeros(2, 16), 0.125)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape and not dq.any()
