"""``DS4Sci_EvoformerAttention(q, k, v, [mask_bias, pair_bias])`` call shape
(speed_benchmark.py:24,84) served by the B200 op with true head semantics."""
from evoformer_triton_b200 import evoformer_attention


def DS4Sci_EvoformerAttention(Q, K, V, biases):
    return evoformer_attention(Q, K, V, biases, layout="true")
