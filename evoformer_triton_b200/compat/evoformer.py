"""Module-name shim: ``from evoformer import EvoformerAttention`` (test.py:2,
speed_benchmark.py:4, memory_benchmark.py:3 of the reference) resolves to the B200 op
when this folder is on PYTHONPATH."""
from evoformer_triton_b200 import EvoformerAttention  # noqa: F401
