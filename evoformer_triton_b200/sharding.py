"""Sharding of the MSA-row axis (N_seq) across the GPUs of one node.

Every (b, h, s) slab is an independent attention problem; only the pair-bias gradient
couples the N_seq rows (it is their sum, dsevoformer-triton/evoformer.py:458).  So each rank
runs the unchanged local op on its rows and the job needs exactly one collective: a sum
all-reduce of d(pair_bias), over NCCL or, for the GPUs of one node, by this package's own
peer-memory kernel (:class:`PeerReducer`).

The reference views ``[B, N_seq, N_res, H, D]`` buffers as ``[B, H, N_seq, N_res, D]``
(evoformer.py:648-650), so "row s" means row s of that *attention view*; slicing axis 1 of
the label shape would hand out something else.  The helpers below slice in the view.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def row_range(n_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block of rows owned by ``rank`` (sizes differ by at most one)."""
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(x: torch.Tensor, rank: int, world: int, layout: str = "reinterpret") -> torch.Tensor:
    """Local shard of a ``[B, N_seq, N_res, H, D]`` tensor, again in label shape
    ``[B, rows, N_res, H, D]``, such that the local op sees rows ``row_range(...)`` of
    the global attention view."""
    B, S, R, H, D = x.shape
    s0, s1 = row_range(S, rank, world)
    if layout == "reinterpret":
        return x.reshape(B, H, S, R, D)[:, :, s0:s1].contiguous().reshape(B, s1 - s0, R, H, D)
    return x[:, s0:s1].contiguous()


def unshard_rows(parts: List[torch.Tensor], layout: str = "reinterpret") -> torch.Tensor:
    """Inverse of :func:`shard_rows` over all ranks' results."""
    B, _, R, H, D = parts[0].shape
    if layout == "reinterpret":
        views = [p.reshape(B, H, p.shape[1], R, D) for p in parts]
        full = torch.cat(views, dim=2)
        return full.reshape(B, full.shape[2], R, H, D)
    return torch.cat(parts, dim=1)


def shard_mask(res_mask: Optional[torch.Tensor], rank: int, world: int) -> Optional[torch.Tensor]:
    """Rows of a ``[B, N_seq, 1, 1, N_res]`` mask that belong to ``rank``."""
    if res_mask is None:
        return None
    s0, s1 = row_range(res_mask.shape[1], rank, world)
    return res_mask[:, s0:s1].contiguous()


class _SumGradAcrossRanks(torch.autograd.Function):
    """Identity in forward; sum all-reduce of the gradient in backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if g.dtype in (torch.bfloat16, torch.float16):  # sum in fp32, never in a 16-bit type
            g32 = g.float()
            dist.all_reduce(g32, op=dist.ReduceOp.SUM, group=ctx.group)
            return g32.to(g.dtype), None
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


def replicate_pair_bias(pair_bias: torch.Tensor, group=None) -> torch.Tensor:
    """Mark a pair bias that every rank holds in full: its gradient is summed over ranks."""
    return _SumGradAcrossRanks.apply(pair_bias, group)


class _DeviceBuffer:
    """A raw device allocation presented to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerReducer:
    """Sum of the fp32 d(pair_bias) over the GPUs of one node through peer memory.

    The reference runs on one GPU and has no such step (its d_pair_bias is complete after
    dsevoformer-triton/evoformer.py:458,860).  With the MSA rows sharded, the local partial sums
    are a few megabytes, for which a library all-reduce is mostly launch and protocol latency.
    Here every rank maps every other rank's buffer (CUDA IPC over NVLink) and
    ``evoattn_peer_allreduce_f32`` sums in place with one kernel per rank: every rank stores its
    part of slice q into rank q's staging area, rank r adds up slice r in rank order and stores it
    into every rank's buffer; two flag barriers with bounded waits separate the phases.  Only
    stores cross NVLink, and all ranks end with the same bits.

    Set up once per (group, size); the op's backward writes its local d(pair_bias) straight into
    ``buffer(numel)`` and calls ``allreduce_``.  Construction is collective over ``group``.
    """

    def __init__(self, numel: int, device, group=None):
        from . import _lib
        self.lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise RuntimeError("PeerReducer serves the (at most 8) GPUs of one node")
        self.device = torch.device(device)
        self.numel = int(numel)
        self._own = []
        self._opened = []
        self._params = {}
        err = None
        bufs, flags = [], []
        with torch.cuda.device(self.device):
            try:
                data_ptr, data_h = self._create(int(self.lib.evoattn_peer_data_bytes(C.c_uint64(self.numel), self.world)))
                flag_ptr, flag_h = self._create(int(self.lib.evoattn_peer_flag_bytes()))
            except RuntimeError as e:
                err, data_ptr, flag_ptr, data_h, flag_h = e, 0, 0, None, None
            handles = [None] * self.world
            dist.all_gather_object(handles, (data_h, flag_h), group=group)
            if all(h[0] is not None for h in handles):
                try:
                    for q, (dh, fh) in enumerate(handles):
                        if q == self.rank:
                            bufs.append(data_ptr); flags.append(flag_ptr)
                        else:
                            bufs.append(self._open(dh)); flags.append(self._open(fh))
                except RuntimeError as e:
                    err = e
            elif err is None:
                err = RuntimeError("another rank could not create its exchange buffer")
        # every rank learns whether all of them succeeded, so that all take the same path
        ok = torch.tensor([0.0 if err is not None else 1.0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if ok.item() == 0:
            for ptr in self._opened:
                self.lib.evoattn_peer_buffer_close(C.c_void_p(ptr))
            dist.barrier(group=group)
            for ptr in self._own:
                self.lib.evoattn_peer_buffer_destroy(C.c_void_p(ptr))
            self._opened, self._own = [], []
            raise RuntimeError(f"peer-memory exchange buffers could not be set up on every rank: {err}")
        self._bufs = (C.c_void_p * self.world)(*bufs)
        self._flags = (C.c_void_p * self.world)(*flags)
        self._tensor = torch.as_tensor(_DeviceBuffer(data_ptr, self.numel * 4), device=self.device).view(torch.float32)
        dist.barrier(group=group)  # nobody starts before every rank has mapped every buffer

    def _create(self, nbytes):
        from . import _lib
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        _lib.check(self.lib.evoattn_peer_buffer_create(C.c_size_t(nbytes), C.byref(ptr), handle), "evoattn_peer_buffer_create")
        self._own.append(ptr.value)
        return ptr.value, handle.raw

    def _open(self, handle: bytes):
        from . import _lib
        ptr = C.c_void_p()
        _lib.check(self.lib.evoattn_peer_buffer_open(handle, C.byref(ptr)), "evoattn_peer_buffer_open")
        self._opened.append(ptr.value)
        return ptr.value

    def buffer(self, numel: int) -> torch.Tensor:
        """This rank's part of the exchange buffer (fp32, ``numel`` elements)."""
        if numel > self.numel:
            raise ValueError(f"PeerReducer was set up for {self.numel} elements, asked for {numel}")
        return self._tensor[:numel]

    def exchange_params(self, numel: int):
        """The parameters with which ``evoattn_bwd`` sums the first ``numel`` floats of the buffers
        over the ranks as part of the call (the structure stays alive with this object)."""
        from . import _lib, attention
        if numel > self.numel:
            raise ValueError(f"PeerReducer was set up for {self.numel} elements, asked for {numel}")
        p = self._params.get(numel)
        if p is None:
            p = _lib.PeerAllReduceParams()
            p.world, p.rank = self.world, self.rank
            p.bufs, p.flags = self._bufs, self._flags
            p.count, p.epoch = int(numel), 0
            p.status = attention._status_word(self.device).data_ptr()
            self._params[numel] = p
        return p

    def allreduce_(self, numel: int) -> None:
        """In-place sum over the ranks of the first ``numel`` floats of every rank's buffer, on the
        current stream.  Collective: every rank calls it with the same ``numel``."""
        from . import _lib, attention
        p = _lib.PeerAllReduceParams()
        p.world, p.rank = self.world, self.rank
        p.bufs, p.flags = self._bufs, self._flags
        p.count, p.epoch = int(numel), 0  # the library counts the calls itself: the launch may be replayed from a CUDA graph
        p.status = attention._status_word(self.device).data_ptr()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            _lib.check(self.lib.evoattn_peer_allreduce_f32(C.byref(p), C.c_void_p(stream)), "evoattn_peer_allreduce_f32")

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for ptr in self._opened:
            self.lib.evoattn_peer_buffer_close(C.c_void_p(ptr))
        dist.barrier(group=self.group)
        for ptr in self._own:
            self.lib.evoattn_peer_buffer_destroy(C.c_void_p(ptr))
        self._opened, self._own = [], []


def sharded_evoformer_attention(attn_fn, Q, K, V, res_mask, pair_bias, group=None, peer_reducer=None):
    """Run ``attn_fn`` (``EvoformerAttention.apply`` or a stand-in) on this rank's rows.

    Q, K, V, res_mask are already local shards; pair_bias is the full bias.  Forward needs
    no communication; backward sums d(pair_bias) over the ranks: with ``peer_reducer`` (a
    :class:`PeerReducer` of this group) through peer memory, otherwise with an NCCL all-reduce.
    """
    if pair_bias is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        owner = getattr(attn_fn, "__self__", None)
        from . import attention
        if isinstance(owner, type) and issubclass(owner, attention._EvoformerAttentionBase):
            # this package's op: its backward all-reduces the fp32 d(pair_bias) as it leaves the
            # kernel, before the cast to the bias dtype (one collective, no extra conversions, and
            # the local partial sums are never rounded to 16 bits)
            with attention.pair_bias_grad_summed_over(group, peer_reducer):
                return attn_fn(Q, K, V, res_mask, pair_bias)
        pair_bias = replicate_pair_bias(pair_bias, group)
    return attn_fn(Q, K, V, res_mask, pair_bias)
