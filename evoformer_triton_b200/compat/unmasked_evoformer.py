"""Module-name shim for the reference's second module (unmasked_evoformer.py:585): the
same op; the "unmasked" fast path is simply N_res being a multiple of the tile."""
from evoformer_triton_b200 import EvoformerAttention  # noqa: F401
