"""Import-path shim: ``from universal_attention_autograd import UniversalAttention, UniversalAttention2,
SMVecMatMul`` resolves to the CUDA-backed classes, as the reference's driver imports them (main.py:2-4)."""
from universal_attention_triton_b200.universal_attention_autograd import (  # noqa: F401
    SMVecMatMul,
    UniversalAttention,
    UniversalAttention2,
    UniversalAttentionMerged,
)
