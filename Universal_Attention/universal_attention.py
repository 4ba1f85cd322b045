"""Import-path shim: ``from Universal_Attention.universal_attention import UniversalAttention`` resolves to the
CUDA-backed kernel Function, as the reference's driver imports it (main.py:6)."""
from universal_attention_triton_b200.Universal_Attention.universal_attention import UniversalAttention  # noqa: F401
