"""Pins the CPU oracle: golden vectors of the reference and form A == form B."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN, make_inputs
from oracle import attn_oracle as O


def _t(a):
    return torch.from_numpy(np.asarray(a)).double()


def test_mask_is_bottom_right():
    # same picture as get_mask_bottom_right(10, 20, 5) in jax_refs/flash_impl.py:377
    m = O.bottom_right_mask(3, 5)
    assert m.int().tolist() == [[1, 1, 1, 0, 0], [1, 1, 1, 1, 0], [1, 1, 1, 1, 1]]
    w = O.bottom_right_mask(3, 5, sliding_window_length=2)
    assert w.int().tolist() == [[0, 1, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 1, 1]]
    assert torch.equal(O.bottom_right_mask(4, 4), torch.ones(4, 4).tril().bool())


def test_reference_fixture_closed_form():
    """test_data.zip of the reference (fhog/test_bwdbwd.py:27-82): all four outputs.

    The stored outputs carry bf16 matmul noise (they were produced with
    BF16_BF16_F32 dots), so they pin the oracle to 1e-2 of abs-max only.
    """
    z = np.load(GOLDEN / "fhog_test_data.npz")
    x = {k: _t(z[k]) for k in z.files}
    scale = 1.0 / 64 ** 0.5
    got = O.bwdbwd_closed_form(x["q"], x["k"], x["v"], x["do"], x["ddq"], x["ddk"], x["ddv"], scale)
    for name, g in zip(("dq2", "dk2", "dv2", "ddo"), got):
        assert O.rel_err(g, x[name]) < 1e-2, name
    # the LSE-based variant on the stored L and o (what the fixture generator ran)
    got = O.bwdbwd_closed_form(x["q"], x["k"], x["v"], x["do"], x["ddq"], x["ddk"], x["ddv"], scale,
                               lse=x["L"], o=x["o"])
    for name, g in zip(("dq2", "dk2", "dv2", "ddo"), got):
        assert O.rel_err(g, x[name]) < 1e-2, name
    # stored L and o are what they claim to be (to bf16 noise)
    assert O.rel_err(O.attn_lse(x["q"], x["k"], scale), x["L"]) < 2e-3
    assert O.rel_err(O.attn_fwd(x["q"], x["k"], x["v"], scale), x["o"]) < 1e-2
    # quirk of the generator: do was drawn with q's key (fhog/jax_refs/jax_impl.py:642-645)
    assert torch.equal(x["do"], x["q"])


def test_reference_torch_restatement_vectors():
    """Outputs of the reference's own torch code on seeded inputs (fp64): 1e-12."""
    from golden.make_golden import TORCH_CASES, seeded_inputs  # noqa: PLC0415
    z = np.load(GOLDEN / "ref_torch_closed_form.npz")
    for name, nq, nk, d, seed in TORCH_CASES:
        x = seeded_inputs(nq, nk, d, seed)
        scale = 1.0 / d ** 0.5
        for form in (O.bwdbwd_closed_form, O.bwdbwd_autograd):
            got = form(x["q"], x["k"], x["v"], x["do"], x["ddq"], x["ddk"], x["ddv"], scale)
            for n, g in zip(("dq2", "dk2", "dv2", "ddo"), got):
                assert O.rel_err(g, _t(z[f"{name}/{n}"])) < 1e-12, (name, n)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("nq,nk,d", [(128, 128, 64), (96, 160, 32), (128, 256, 128)])
def test_autograd_equals_closed_form(nq, nk, d, causal):
    x = make_inputs(2, nq, nk, d, seed=5, dtype=torch.float64)
    scale = 1.0 / d ** 0.5
    a = O.bwdbwd_autograd(*x.values(), scale, causal)
    b = O.bwdbwd_closed_form(*x.values(), scale, causal)
    lse = O.attn_lse(x["q"], x["k"], scale, causal)
    o = O.attn_fwd(x["q"], x["k"], x["v"], scale, causal)
    c = O.bwdbwd_closed_form(*x.values(), scale, causal, lse=lse, o=o)
    for ta, tb, tc in zip(a, b, c):
        assert O.rel_err(tb, ta) < 1e-12
        assert O.rel_err(tc, ta) < 1e-12


def test_first_backward_matches_autograd():
    """attn_bwd vs autograd of attn_fwd (check_backward_matched, jax_refs/flash_impl.py:364-374)."""
    x = make_inputs(1, 64, 96, 32, seed=9, dtype=torch.float64)
    q, k, v = (x[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
    o = O.attn_fwd(q, k, v, 0.2, True)
    ref = torch.autograd.grad(o, (q, k, v), x["do"])
    got = O.attn_bwd(x["q"], x["k"], x["v"], x["do"], 0.2, True)
    for g, r in zip(got, ref):
        assert O.rel_err(g, r) < 1e-12


def test_row_stats_linear_in_cotangents():
    """dd is linear in (ddq, ddk); b is linear in (ddq, ddk, ddv): a size-independent property."""
    x = make_inputs(1, 64, 64, 32, seed=3, dtype=torch.float64)
    base = O.bwdbwd_row_stats(*x.values(), 0.3)
    y = dict(x)
    for n in ("ddq", "ddk", "ddv"):
        y[n] = 2.5 * x[n]
    scaled = O.bwdbwd_row_stats(*y.values(), 0.3)
    assert O.rel_err(scaled[0], base[0]) < 1e-13
    assert O.rel_err(scaled[1], 2.5 * base[1]) < 1e-13
    assert O.rel_err(scaled[2], 2.5 * base[2]) < 1e-12


def test_sliding_window_mask_definition():
    """jax_refs/flash_impl.py:86-91: visible iff 0 <= (i + nk - nq) - j < sliding_window_length."""
    for nq, nk, w in [(5, 9, 3), (8, 8, 1), (7, 4, 2), (6, 10, 100)]:
        m = O.bottom_right_mask(nq, nk, w)
        for i in range(nq):
            for j in range(nk):
                dist = i + nk - nq - j
                assert bool(m[i, j]) == (0 <= dist < w)


@pytest.mark.parametrize("nq,nk,w", [(48, 48, 7), (40, 72, 16), (64, 64, 64)])
def test_sliding_window_autograd_equals_closed_form(nq, nk, w):
    x = make_inputs(2, nq, nk, 16, seed=5, dtype=torch.float64)
    a = O.bwdbwd_autograd(*x.values(), 0.25, True, sliding_window_length=w)
    b = O.bwdbwd_closed_form(*x.values(), 0.25, True, sliding_window_length=w)
    for u, v in zip(a, b):
        assert O.rel_err(u, v) < 1e-12
    if w >= nk:  # a window that covers every key is the plain causal mask
        c = O.bwdbwd_closed_form(*x.values(), 0.25, True)
        for u, v in zip(b, c):
            assert torch.equal(u, v)
    # the query-chunked form used at large sizes agrees too
    ch = O.bwdbwd_closed_form_chunked(*(t[0] for t in x.values()), 0.25, True, chunk=16, sliding_window_length=w)
    for u, v in zip(ch[:4], b):
        assert O.rel_err(u, v[0]) < 1e-12
