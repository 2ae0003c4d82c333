"""Put an unmodified copy of the reference's five Python files where a GPU run can reach them.

    python baseline/prepare_ref.py [reference_dir]

The reference (``dsevoformer-triton/`` of lvhoaa/evoformer_triton) is a flat folder of scripts
with no package metadata, so there is nothing to ``pip install``; its files are copied as they
are into ``baseline/_ref/`` (ignored by git: the copy is a measurement aid, not part of this
project's source):

    baseline/_ref/kernels/   evoformer.py, unmasked_evoformer.py   (the Triton kernels)
    baseline/_ref/scripts/   test.py, speed_benchmark.py, memory_benchmark.py

The two folders are separate so that the scripts can be run against either implementation of
``evoformer.EvoformerAttention``: with ``kernels/`` on PYTHONPATH they drive the reference's
Triton kernels, with ``evoformer_triton_b200/compat/`` they drive this project's op.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
KERNELS = ("evoformer.py", "unmasked_evoformer.py")
SCRIPTS = ("test.py", "speed_benchmark.py", "memory_benchmark.py")


def prepare(src: str) -> bool:
    if not os.path.isdir(src):
        return False
    for sub, names in (("kernels", KERNELS), ("scripts", SCRIPTS)):
        os.makedirs(os.path.join(DEST, sub), exist_ok=True)
        for n in names:
            shutil.copyfile(os.path.join(src, n), os.path.join(DEST, sub, n))
    return True


if __name__ == "__main__":
    default = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference", "dsevoformer-triton")
    src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("EVOFORMER_REFERENCE_DIR", default)
    print("copied" if prepare(src) else f"reference not found at {src}")
