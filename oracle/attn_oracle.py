"""CPU oracle for the double backward of scaled-dot-product attention.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
module; it is the checker used by the test-suite, by the smoke test and by the
CPU-baseline leg of the benchmark.  It is a restatement, in torch on the CPU,
of the reference project's JAX maths:

* mask                       jax_refs/flash_impl.py:86-91   (bottom-right aligned causal)
* attention forward          jax_refs/flash_impl.py:94-121
* first backward             jax_refs/flash_impl.py:124-173  (the function that gets differentiated)
* grad-of-grad idiom         jax_refs/flash_impl.py:408-417, fhog/jax_refs/jax_impl.py:508-533
* closed-form double bwd     jax_refs/flash_impl.py:176-229
* LSE-based closed form      jax_refs/flash_impl.py:262-328  (what produced the golden fixture)

The reference evaluates these with jax 0.8.0 / jaxlib 0.8.0 (XLA), which is a
third-party dependency that is not installed in this environment, so the
arithmetic is restated here and pinned two ways:

1. against the reference's golden vectors (``test_data.zip``: nq=128, nkv=256,
   D=64, non-causal), which carry bf16 matmul noise and therefore pin the
   result to about 5e-3 of each tensor's abs-max;
2. against itself: the autograd-of-autograd form (A) and the closed form (B)
   are independent derivations and agree to ~1e-14 in fp64.

Causal masking, D=128 and the 1e-4 fp32 tolerance are pinned by no reference
test ("parity unpinned" for those); they rest on (2).

All functions take per-head 2-D tensors ``(N, D)`` like the reference maths,
or batched ``(..., N, D)`` tensors; the leading dims broadcast through.
"""
from __future__ import annotations

import math

import torch

__all__ = [
    "bottom_right_mask",
    "attn_fwd",
    "attn_lse",
    "attn_bwd",
    "bwdbwd_autograd",
    "bwdbwd_closed_form",
    "bwdbwd_row_stats",
    "rel_err",
]


def bottom_right_mask(nq: int, nk: int, sliding_window_length: float = math.inf,
                      device=None) -> torch.Tensor:
    """Boolean (nq, nk) mask, True where query i may attend key j.

    Follows jax_refs/flash_impl.py:86-91: the query index is shifted by
    ``nk - nq`` so the diagonal ends in the bottom-right corner.
    """
    qi = torch.arange(nq, device=device)[:, None] + (nk - nq)
    kj = torch.arange(nk, device=device)[None, :]
    mask = qi >= kj
    if sliding_window_length != math.inf:
        mask = mask & ((qi - kj) < sliding_window_length)
    return mask


def _scores(q, k, scale, is_causal, sliding_window_length=math.inf):
    s = torch.einsum("...qd,...kd->...qk", q, k) * scale
    if is_causal:
        m = bottom_right_mask(q.shape[-2], k.shape[-2], sliding_window_length, q.device)
        s = torch.where(m, s, torch.full_like(s, -math.inf))
    return s


def attn_fwd(q, k, v, scale, is_causal=False, sliding_window_length=math.inf):
    """O = softmax(QK^T scale) V   (jax_refs/flash_impl.py:94-121)."""
    p = torch.softmax(_scores(q, k, scale, is_causal, sliding_window_length), dim=-1)
    return p @ v


def attn_lse(q, k, scale, is_causal=False, sliding_window_length=math.inf):
    """Row-wise logsumexp of the (masked) scores; the ``stats``/``L`` input."""
    return torch.logsumexp(_scores(q, k, scale, is_causal, sliding_window_length), dim=-1)


def attn_bwd(q, k, v, do, scale, is_causal=False, sliding_window_length=math.inf):
    """First backward (dq, dk, dv), jax_refs/flash_impl.py:124-173."""
    p = torch.softmax(_scores(q, k, scale, is_causal, sliding_window_length), dim=-1)
    dp = do @ v.transpose(-1, -2)
    pdp = p * dp
    d = pdp.sum(dim=-1, keepdim=True)
    ds = scale * (pdp - p * d)
    dq = ds @ k
    dk = ds.transpose(-1, -2) @ q
    dv = p.transpose(-1, -2) @ do
    return dq, dk, dv


def bwdbwd_autograd(q, k, v, do, ddq, ddk, ddv, scale, is_causal=False, sliding_window_length=math.inf):
    """Form A: vector-Jacobian product of ``attn_bwd`` by reverse-mode autograd.

    Same idiom as ``jax.vjp(attn_bwd, q, k, v, do)`` applied to the cotangents
    ``(ddq, ddk, ddv)`` (jax_refs/flash_impl.py:408-417,
    fhog/jax_refs/jax_impl.py:522-532).  Returns (dq2, dk2, dv2, ddo).
    """
    q, k, v, do = (t.detach().clone().requires_grad_(True) for t in (q, k, v, do))
    dq, dk, dv = attn_bwd(q, k, v, do, scale, is_causal, sliding_window_length)
    dq2, dk2, dv2, ddo = torch.autograd.grad(
        (dq, dk, dv), (q, k, v, do), grad_outputs=(ddq, ddk, ddv))
    return dq2, dk2, dv2, ddo


def bwdbwd_closed_form(q, k, v, do, ddq, ddk, ddv, scale, is_causal=False, lse=None, o=None,
                       sliding_window_length=math.inf):
    """Form B: the closed-form equations of jax_refs/flash_impl.py:176-229.

    When ``lse`` (and ``o``) are given the LSE-based variant of
    jax_refs/flash_impl.py:262-328 is evaluated instead: P = exp(S - lse) and
    D = rowsum(o * do).  Masked pairs contribute exactly zero.
    """
    s = _scores(q, k, scale, is_causal, sliding_window_length)
    if lse is None:
        p = torch.softmax(s, dim=-1)
    else:
        p = torch.exp(s - lse[..., None])
    kt, vt = k.transpose(-1, -2), v.transpose(-1, -2)
    dp = do @ vt
    dds = scale * (ddq @ kt + q @ ddk.transpose(-1, -2))
    if o is None:
        d = (p * dp).sum(dim=-1, keepdim=True)
    else:
        d = (o * do).sum(dim=-1, keepdim=True)
    dd = (dds * p).sum(dim=-1, keepdim=True)
    dp2 = do @ ddv.transpose(-1, -2) - dp * dd - dds * d + dp * dds
    ddp = p * (dds - dd)
    b = (dp2 * p).sum(dim=-1, keepdim=True)
    ds2 = scale * p * (dp2 - b)
    ds = scale * p * (dp - d)
    dq2 = ds @ ddk + ds2 @ k
    dk2 = ds.transpose(-1, -2) @ ddq + ds2.transpose(-1, -2) @ q
    dv2 = ddp.transpose(-1, -2) @ do
    ddo = p @ ddv + ddp @ v
    return dq2, dk2, dv2, ddo


def bwdbwd_row_stats(q, k, v, do, ddq, ddk, ddv, scale, is_causal=False, sliding_window_length=math.inf):
    """The three per-query row statistics the four-pass algorithm stages:
    ``d = rowsum(P*dP)``, ``dd = rowsum(ddS*P)``, ``b = rowsum(dP2*P)``
    (jax_refs/flash_impl.py:232-259, ``precompute_values``)."""
    s = _scores(q, k, scale, is_causal, sliding_window_length)
    p = torch.softmax(s, dim=-1)
    dp = do @ v.transpose(-1, -2)
    dds = scale * (ddq @ k.transpose(-1, -2) + q @ ddk.transpose(-1, -2))
    d = (p * dp).sum(dim=-1)
    dd = (dds * p).sum(dim=-1)
    dp2 = do @ ddv.transpose(-1, -2) - dp * dd[..., None] - dds * d[..., None] + dp * dds
    b = (dp2 * p).sum(dim=-1)
    return d, dd, b


def rel_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max|x - ref| / max|ref| — the error metric every parity test uses."""
    ref = ref.double()
    return float((x.double().cpu() - ref.cpu()).abs().max() / ref.abs().max().clamp_min(1e-300))


def bwdbwd_closed_form_chunked(q, k, v, do, ddq, ddk, ddv, scale, is_causal=False, chunk=1024,
                               sliding_window_length=math.inf):
    """Form B evaluated over query-row chunks so that no (N_Q, N_K) matrix is
    ever held whole: memory is O(chunk * N_K).  Same equations as
    ``bwdbwd_closed_form``; works on any device/dtype torch supports (the
    large-shape parity tests run it in fp64 on the GPU).  2-D per-head inputs.
    Returns (dq2, dk2, dv2, ddo, lse, o) — the last two are the saved forward
    results the operator consumes, produced on the way.
    """
    nq, nk = q.shape[-2], k.shape[-2]
    off = nk - nq
    dq2 = torch.empty_like(q)
    ddo = torch.empty_like(q)
    o = torch.empty_like(q)
    lse = torch.empty(nq, dtype=q.dtype, device=q.device)
    dk2 = torch.zeros_like(k)
    dv2 = torch.zeros_like(k)
    kj = torch.arange(nk, device=q.device)[None, :]
    for r0 in range(0, nq, chunk):
        r1 = min(nq, r0 + chunk)
        qc, doc, ddqc = q[r0:r1], do[r0:r1], ddq[r0:r1]
        s = (qc @ k.T) * scale
        if is_causal:
            qi = torch.arange(r0, r1, device=q.device)[:, None] + off
            vis = qi >= kj
            if sliding_window_length != math.inf:
                vis = vis & ((qi - kj) < sliding_window_length)
            s = torch.where(vis, s, torch.full_like(s, -math.inf))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l[:, None])
        lse[r0:r1] = l
        o[r0:r1] = p @ v
        dp = doc @ v.T
        dds = scale * (ddqc @ k.T + qc @ ddk.T)
        d = (p * dp).sum(-1, keepdim=True)
        dd = (dds * p).sum(-1, keepdim=True)
        dp2 = doc @ ddv.T - dp * dd - dds * d + dp * dds
        ddp = p * (dds - dd)
        b = (dp2 * p).sum(-1, keepdim=True)
        ds2 = scale * p * (dp2 - b)
        ds = scale * p * (dp - d)
        dq2[r0:r1] = ds @ ddk + ds2 @ k
        ddo[r0:r1] = p @ ddv + ddp @ v
        dk2 += ds.T @ ddqc + ds2.T @ qc
        dv2 += ddp.T @ doc
    return dq2, dk2, dv2, ddo, lse, o
