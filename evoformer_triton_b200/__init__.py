"""B200-native Evoformer attention (pair-bias + residue-mask flash attention).

Public surface:
    EvoformerAttention            autograd.Function, drop-in for the reference class
    EvoformerAttentionTrueLayout  same op with genuine head-axis semantics
    GatedEvoformerAttention       the op followed by ``sigmoid(gate) *``, fused into the kernel
    evoformer_attention           DS4Sci-style ``attn(Q, K, V, [mask, pair_bias])``; options for the
                                  ``[B, R, R, H]`` bias layout, the gate and the mask-bias gradient
"""
from .attention import (EvoformerAttention, EvoformerAttentionTrueLayout, GatedEvoformerAttention,
                        check_device_status, evoformer_attention, force_generic)

__all__ = ["EvoformerAttention", "EvoformerAttentionTrueLayout", "GatedEvoformerAttention",
           "evoformer_attention", "check_device_status", "force_generic"]
