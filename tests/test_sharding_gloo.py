"""CPU, two gloo ranks: sharding the MSA rows + one all-reduce of d(pair_bias) reproduces the
unsharded result.  The local op on each rank is the CPU oracle (the CUDA op needs a GPU);
what is under test is the partition algebra and the collective wiring of
evoformer_triton_b200.sharding."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_attn(Q, K, V, mask, bias):
    from oracle import evo_oracle as oc
    return oc.attention(Q, K, V, mask, bias)


def _worker(rank, world, port, layout, fail_rank, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from evoformer_triton_b200 import sharding
        from oracle import evo_oracle as oc
        g = torch.Generator().manual_seed(7)
        B, S, R, H, D = 2, 5, 24, 3, 8  # 5 rows over 2 ranks: uneven split
        shp = (B, S, R, H, D)
        Q, K, V, dO = (torch.randn(shp, generator=g, dtype=torch.float64) for _ in range(4))
        mask = torch.rand((B, S, 1, 1, R), generator=g) < 0.8
        mask[..., 0] = True
        bias = torch.randn((B, 1, H, R, R), generator=g, dtype=torch.float64)
        full = oc.attention_fwd_bwd(Q, K, V, mask, bias, dO, layout=layout)

        if rank == fail_rank:
            raise RuntimeError("injected host-side failure before the collective")

        loc = [sharding.shard_rows(t, rank, world, layout).requires_grad_() for t in (Q, K, V)]
        dO_loc = sharding.shard_rows(dO, rank, world, layout)
        if layout == "reinterpret":
            s0, s1 = sharding.row_range(S, rank, world)
            m_loc = mask[:, s0:s1].contiguous()
        else:
            m_loc = sharding.shard_mask(mask, rank, world)
        b = bias.clone().requires_grad_()
        attn = (lambda q, k, v, m, bb: oc.attention(q, k, v, m, bb, layout=layout))
        o = sharding.sharded_evoformer_attention(attn, loc[0], loc[1], loc[2], m_loc, b)
        o.backward(dO_loc)
        # d(pair_bias) is complete on every rank after the all-reduce
        err = {"dbias": oc.rel_err(b.grad, full[4])}
        for name, got, ref in (("O", o.detach(), full[0]), ("dQ", loc[0].grad, full[1]),
                               ("dK", loc[1].grad, full[2]), ("dV", loc[2].grad, full[3])):
            gathered = [None] * world  # shards differ in size: gather as objects
            dist.all_gather_object(gathered, got.contiguous())
            err[name] = oc.rel_err(sharding.unshard_rows(gathered, layout), ref)
        out.put((rank, "ok", err))
    except Exception as e:  # noqa: BLE001
        out.put((rank, "error", repr(e)))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(layout, fail_rank=-1):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, layout, fail_rank, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    return sorted(res)


@pytest.mark.parametrize("layout", ["reinterpret", "true"])
def test_sharded_equals_unsharded(layout):
    for rank, status, err in _run(layout):
        assert status == "ok", err
        for name, e in err.items():
            assert e < 1e-12, (rank, name, e)


def test_row_range_partitions_every_row_once():
    from evoformer_triton_b200.sharding import row_range
    for n in (1, 5, 128, 1000):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                a, b = row_range(n, r, world)
                seen += list(range(a, b))
            assert seen == list(range(n))


def test_label_axis_slice_is_not_the_row_shard():
    """Under the reference's reinterpretation, slicing axis 1 of the label shape is a
    different partition from slicing MSA rows of the attention view."""
    from evoformer_triton_b200.sharding import shard_rows
    x = torch.arange(1 * 4 * 3 * 2 * 2, dtype=torch.float32).reshape(1, 4, 3, 2, 2)
    assert not torch.equal(shard_rows(x, 0, 2, "reinterpret"), x[:, :2])
    assert torch.equal(shard_rows(x, 0, 2, "true"), x[:, :2])


def test_rank_failure_is_reported_not_hung():
    """A rank that raises on the host before the collective: the other rank's all-reduce
    ends with an error inside the process-group timeout instead of hanging."""
    res = _run("reinterpret", fail_rank=1)
    status = {r: s for r, s, _ in res}
    assert status[1] == "error"
    assert status[0] == "error"  # timed out / connection closed, reported as an exception
