"""Differentiable attention built on the library's three operators.

``attention(q, k, v, scale, is_causal)`` is an autograd function whose backward
is itself an autograd function, so ``torch.autograd.grad(..., create_graph=True)``
followed by a second ``grad`` runs

    forward          -> fhob_forward   (O and the fp32 logsumexp L, O(N) memory)
    first backward   -> fhob_backward  (dQ, dK, dV)
    double backward  -> fhob_bwdbwd    (dQ2, dK2, dV2, ddO)

This is the role the reference sketches but leaves commented out
(``class Bwd(torch.autograd.Function)``, fhog/triton_bwdbwd.py:538-554; its
forward/backward pair is FlashAttention2, fhog/triton_flash.py:136-198).
The derivative of the first backward is taken with O and L regarded as functions
of q, k, v, exactly like ``jax.vjp(attn_bwd)`` in jax_refs/flash_impl.py:408-417,
so no separate gradient flows into the saved O and L.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .ops import _fold, _Problem, attention_forward, flash_bwdbwd


def attention_backward(Q, K, V, O, dO, L, scale, *, is_causal: bool = False, sliding_window=None, impl: str = "auto"):
    """First backward from the saved forward results: returns ``(dQ, dK, dV)``.

    Same maths as ``attn_bwd`` (jax_refs/flash_impl.py:124-173) with
    ``P = exp(S - L)`` and ``D = rowsum(dO * O)``; O(N) memory.
    """
    if Q.numel() == 0 or K.numel() == 0 or V.numel() == 0:
        return tuple(torch.zeros_like(t) for t in (Q, K, V))   # no queries or no keys: nothing to launch
    # the problem struct wants three cotangent tensors of the right shapes; they are not read
    prob = _Problem(Q, K, V, O, dO, Q, K, V, L, scale, is_causal, impl, need_outputs=False, window=sliding_window)
    dq, dk, dv = (torch.empty(t.shape, dtype=t.dtype, device=t.device) for t in (Q, K, V))   # contiguous results
    lib = _lib.load()
    with torch.cuda.device(prob.device):
        call = lambda pr: lib.fhob_backward(C.byref(pr.p), C.c_void_p(dq.data_ptr()), C.c_void_p(dk.data_ptr()),
                                            C.c_void_p(dv.data_ptr()), C.c_void_p(pr.stream))
        rc = call(prob)
        if rc != 0 and prob.layout is not None:
            # a view the tensor-map encoder does not take: read copies instead
            prob = _Problem(Q, K, V, O, dO, Q, K, V, L, scale, is_causal, impl, need_outputs=False,
                            window=sliding_window, allow_views=False)
            rc = call(prob)
        _lib.check(rc, "fhob_backward")
    return dq, dk, dv


class _AttentionBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, o, lse, d_o, scale, is_causal, window):
        ctx.save_for_backward(q, k, v, o, lse, d_o)
        ctx.scale, ctx.is_causal, ctx.window = scale, is_causal, window
        return attention_backward(q, k, v, o, d_o, lse, scale, is_causal=is_causal, sliding_window=window)

    @staticmethod
    def backward(ctx, ddq, ddk, ddv):
        q, k, v, o, lse, d_o = ctx.saved_tensors
        dq2, dk2, dv2, ddo = flash_bwdbwd(q, k, v, o, d_o, ddq.contiguous(), ddk.contiguous(), ddv.contiguous(), lse,
                                          ctx.scale, is_causal=ctx.is_causal, sliding_window=ctx.window)
        return dq2, dk2, dv2, None, None, ddo, None, None, None


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, is_causal, window):
        o, lse = attention_forward(q, k, v, scale, is_causal=is_causal, sliding_window=window)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale, ctx.is_causal, ctx.window = scale, is_causal, window
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = _AttentionBackward.apply(q, k, v, o, lse, d_o.contiguous(), ctx.scale, ctx.is_causal,
                                              ctx.window)
        return dq, dk, dv, None, None, None


def attention(q, k, v, scale=None, *, is_causal: bool = False, sliding_window=None):
    """``softmax(q k^T scale) v`` for CUDA bfloat16/float32 tensors ``(BH, N, D)`` or ``(B, H, N, D)``,
    differentiable twice (``create_graph=True``)."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return _Attention.apply(q, k, v, float(scale), bool(is_causal), sliding_window)
