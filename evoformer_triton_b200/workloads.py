"""Seeded synthetic inputs for the five benchmark/parity configurations.

The reference only ever measures on ``randn`` tensors
(dsevoformer-triton/speed_benchmark.py:64-68, test.py:14-45), so these are the
real distributions, not stand-ins for a dataset.  Everything is drawn on the CPU
generator in fp32 in the fixed order Q, K, V, mask, dO (pair_bias on its own stream) and then cast,
so a CPU checker and a GPU run see identical bits.

Shapes are the reference's label shapes: Q/K/V/dO ``[B, N_seq, N_res, H, D]``,
res_mask ``[B, N_seq, 1, 1, N_res]`` (bool keep-mask), pair_bias
``[B, 1, H, N_res, N_res]`` (fp32, as in test.py:36-42).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    S: int  # N_seq (MSA rows)
    R: int  # N_res
    H: int
    D: int
    dtype: torch.dtype
    qkv_std: float
    bias_std: float
    mask: str  # "bernoulli:<keep>", "tail:<frac>", "randpad:<maxfrac>", "none"
    what: str

    @property
    def flops_fwd(self) -> float:
        """2 matmuls of 2*B*H*S*R*R*D flops (speed_benchmark.py:109-110, times N_seq)."""
        return 2.0 * 2.0 * self.B * self.H * self.S * self.R * self.R * self.D

    @property
    def flops_fwd_bwd(self) -> float:
        """Forward + 2.5x forward for backward (speed_benchmark.py:111-114)."""
        return 3.5 * self.flops_fwd

    def with_rows(self, S: int) -> "Workload":
        return Workload(self.name, self.B, S, self.R, self.H, self.D, self.dtype,
                        self.qkv_std, self.bias_std, self.mask, self.what)


WORKLOADS: Dict[str, Workload] = {
    "C1": Workload("C1", 1, 16, 64, 4, 32, torch.float32, 1.0, 1.0, "bernoulli:0.9",
                   "tiny CPU-runnable MSA-row attention, fp32"),
    "C2": Workload("C2", 1, 128, 384, 8, 32, torch.bfloat16, 0.5, 1.0, "tail:0.10",
                   "AlphaFold MSA row-wise gated-attention core, bf16"),
    "C3": Workload("C3", 1, 384, 384, 4, 32, torch.bfloat16, 0.5, 1.0, "randpad:0.15",
                   "triangle (starting-node) attention on the pair representation, bf16"),
    "C4": Workload("C4", 1, 1024, 384, 8, 8, torch.float16, 0.5, 2.0, "bernoulli:0.95",
                   "extra-MSA stack attention, many rows, small head dim, fp16"),
    "C5": Workload("C5", 2, 512, 768, 8, 64, torch.bfloat16, 0.5, 1.0, "randpad:0.20",
                   "large-crop MSA row attention, bf16"),
}


def make_keep_mask(w: Workload, gen: torch.Generator) -> Optional[torch.Tensor]:
    """Boolean keep-mask ``[B, S, 1, 1, R]`` (True = attend to that residue)."""
    kind, _, arg = w.mask.partition(":")
    if kind == "none":
        return None
    if kind == "bernoulli":
        keep = torch.rand((w.B, w.S, w.R), generator=gen) < float(arg)
    elif kind == "tail":
        n_drop = int(float(arg) * w.R)
        keep = (torch.arange(w.R) < w.R - n_drop).expand(w.B, w.S, w.R).clone()
    elif kind == "randpad":
        hi = int(float(arg) * w.R)
        pad = torch.randint(0, hi + 1, (w.B,), generator=gen)
        keep = (torch.arange(w.R)[None, :] < (w.R - pad)[:, None])
        keep = keep[:, None, :].expand(w.B, w.S, w.R).clone()
    else:
        raise ValueError(w.mask)
    return keep.reshape(w.B, w.S, 1, 1, w.R)


def make_inputs(w: Workload, seed: int = 0, device="cpu", rows: Optional[int] = None,
                row_offset: int = 0) -> Dict[str, Optional[torch.Tensor]]:
    """Draw Q, K, V, res_mask, pair_bias, dO for a workload.

    ``rows``/``row_offset`` draw only a shard of the MSA rows (its own seeded
    stream ``seed + 1000003*row_offset``); pair_bias has a stream of its own that
    depends on ``seed`` alone, so every shard of one job sees the same bias.
    """
    if rows is not None:
        w = w.with_rows(rows)
    gen_bias = torch.Generator().manual_seed(seed + 7919)
    gen = torch.Generator().manual_seed(seed + 1000003 * row_offset)
    shape = (w.B, w.S, w.R, w.H, w.D)

    def draw(std, shp, g):
        return (torch.randn(shp, generator=g, dtype=torch.float32) * std)

    Q = draw(w.qkv_std, shape, gen).to(w.dtype)
    K = draw(w.qkv_std, shape, gen).to(w.dtype)
    V = draw(w.qkv_std, shape, gen).to(w.dtype)
    mask = make_keep_mask(w, gen)
    bias = draw(w.bias_std, (w.B, 1, w.H, w.R, w.R), gen_bias)
    dO = draw(1.0, shape, gen).to(w.dtype)
    out = dict(Q=Q, K=K, V=V, res_mask=mask, pair_bias=bias, dO=dO)
    if str(device) != "cpu":
        out = {k: (None if t is None else t.to(device)) for k, t in out.items()}
    return out


def additive_mask(keep: torch.Tensor, dtype=torch.float32, value: float = -1e9) -> torch.Tensor:
    """DS4Sci-style additive form of a keep-mask: 0 where kept, ``value`` where dropped."""
    return torch.where(keep, torch.zeros((), dtype=dtype), torch.full((), value, dtype=dtype))
