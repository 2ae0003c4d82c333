"""B200-native Evoformer attention (pair-bias + residue-mask flash attention).

Public surface:
    EvoformerAttention            autograd.Function, drop-in for the reference class
    EvoformerAttentionTrueLayout  same op with genuine head-axis semantics
    evoformer_attention           DS4Sci-style ``attn(Q, K, V, [mask, pair_bias])``
"""
from .attention import (EvoformerAttention, EvoformerAttentionTrueLayout, check_device_status,
                        evoformer_attention, force_generic)

__all__ = ["EvoformerAttention", "EvoformerAttentionTrueLayout", "evoformer_attention",
           "check_device_status", "force_generic"]
