"""B200-native double-backward flash attention behind the reference's entry
point (``from fhog import flash_bwdbwd`` becomes ``from fhob import flash_bwdbwd``)."""
from .autograd import attention, attention_backward
from .ops import attention_forward, flash_bwdbwd, produce_L, release_cached_memory, run_passes
from . import torch_op  # registers torch.ops.fhob.bwdbwd

__all__ = ["flash_bwdbwd", "produce_L", "attention_forward", "attention_backward", "attention", "run_passes",
           "release_cached_memory"]
