"""Universal Attention for NVIDIA B200 (sm_100a): hand-written CUDA kernels
behind the reference's autograd entry points."""
from . import _lib, ops  # noqa: F401
from .universal_attention_autograd import (  # noqa: F401
    SMVecMatMul,
    UniversalAttention,
    UniversalAttention2,
    UniversalAttentionMerged,
    set_merged_backward,
    set_merged_forward,
    set_output_layout,
    set_save_output,
    set_strict_masked_grads,
)

__all__ = ["UniversalAttention", "UniversalAttention2", "UniversalAttentionMerged", "SMVecMatMul", "set_output_layout", "set_merged_backward", "set_merged_forward",
           "set_save_output", "set_strict_masked_grads", "ops"]
