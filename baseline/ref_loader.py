"""Import the reference's own Triton ``EvoformerAttention`` from ``baseline/_ref/kernels``.

The reference's ``evoformer.py`` imports ``deepspeed.utils.timer`` at module top
(evoformer.py:8) and never uses it (every use is commented out, :639-640); DeepSpeed is not
installed here, so an empty stand-in module with that one name is registered first.  The kernel
file itself is loaded unmodified, under the module name ``reference_evoformer`` so that it cannot
be confused with this project's ``evoformer`` shim.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "kernels", "evoformer.py"))


def _stub_deepspeed() -> None:
    if "deepspeed" in sys.modules:
        return
    ds = types.ModuleType("deepspeed")
    utils = types.ModuleType("deepspeed.utils")
    timer = types.ModuleType("deepspeed.utils.timer")

    class SynchronizedWallClockTimer:  # evoformer.py:8 imports the name only
        @staticmethod
        def memory_usage() -> str:
            return ""

    timer.SynchronizedWallClockTimer = SynchronizedWallClockTimer
    ds.utils, utils.timer = utils, timer
    sys.modules.update({"deepspeed": ds, "deepspeed.utils": utils, "deepspeed.utils.timer": timer})


def load_reference_attention(which: str = "evoformer"):
    """Returns the reference's ``EvoformerAttention`` class (needs a GPU: the file asks Triton
    for the active driver at import, evoformer.py:112)."""
    _stub_deepspeed()
    path = os.path.join(REF_DIR, "kernels", which + ".py")
    spec = importlib.util.spec_from_file_location("reference_" + which, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["reference_" + which] = mod
    spec.loader.exec_module(mod)
    return mod.EvoformerAttention
