"""``torch.ops.fhob.bwdbwd``: the operator as a PyTorch custom op.

The reference wraps its entry point in ``torch.compile(fullgraph=True)``
(fhog/triton_bwdbwd.py:557).  A ctypes call cannot be traced, so for callers
that compile their step the operator is also registered as a custom op with a
shape-only ("fake") implementation: Dynamo and AOT autograd then treat it as
one opaque node and the compiled graph calls the same library entry point.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .ops import flash_bwdbwd


@torch.library.custom_op("fhob::bwdbwd", mutates_args=())
def bwdbwd(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, O: torch.Tensor, dO: torch.Tensor,
           ddQ: torch.Tensor, ddK: torch.Tensor, ddV: torch.Tensor, L: torch.Tensor, scale: float,
           is_causal: bool = False, sliding_window: int = 0
           ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dQ2, dK2, dV2, ddO); ``sliding_window`` 0 means none."""
    return flash_bwdbwd(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, is_causal=is_causal,
                        sliding_window=sliding_window if sliding_window > 0 else None)


@bwdbwd.register_fake
def _(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale, is_causal=False, sliding_window=0):
    return (torch.empty_like(Q, memory_format=torch.contiguous_format),
            torch.empty_like(K, memory_format=torch.contiguous_format),
            torch.empty_like(V, memory_format=torch.contiguous_format),
            torch.empty_like(dO, memory_format=torch.contiguous_format))
