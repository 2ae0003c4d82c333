#!/usr/bin/env python
"""Benchmark of the Evoformer attention hot path (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C2] [--impl ours|reference]

One "step" = one forward + one backward of the op over one batch of seeded synthetic
input (the workload's own distribution; the reference measures on randn as well).  With
N > 1 (launched by torchrun, one rank per GPU) every rank processes its own block of
MSA rows of the same size (weak scaling) and the d(pair_bias) all-reduce over NCCL is
inside the timed step.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from evoformer_triton_b200.workloads import WORKLOADS, make_inputs  # noqa: E402

METRIC = "evoformer_attn_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def ncu_dram_bytes(workload: str, kernel: str):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the named kernel, as recorded
    from an Nsight Compute capture of this benchmark (profiles/ncu_dram_bytes.json: workload ->
    kernel -> bytes and the capture it came from); None where no capture has been recorded."""
    path = os.path.join(ROOT, "profiles", "ncu_dram_bytes.json")
    try:
        with open(path) as f:
            rec = json.load(f).get(workload, {}).get(kernel)
    except (OSError, ValueError):
        return None, None
    if not rec:
        return None, None
    return int(rec["bytes"]), rec.get("source")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", 0)),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def oracle_step_seconds(w, rows: int, repeats: int, threads: int):
    """Time the CPU oracle (the reference's naive PyTorch path, restated) on `rows` MSA rows."""
    from oracle import evo_oracle as oc
    torch.set_num_threads(threads)
    x = make_inputs(w, rows=rows)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        oc.attention_fwd_bwd(x["Q"], x["K"], x["V"], x["res_mask"], x["pair_bias"], x["dO"], chunk=min(rows, 16))
        times.append(time.perf_counter() - t0)
    return times


def run_reference(args, rank, world):
    """--impl reference: the reference's own CPU implementation of the path (its naive
    PyTorch attention, dsevoformer-triton/test.py:47-62, restated in oracle/) on host cores."""
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    threads = os.cpu_count() or 1
    rows = max(1, min(w.S, args.ref_rows))
    wsub = w.with_rows(rows)
    oracle_step_seconds(w, rows, args.warmup, threads)
    times = oracle_step_seconds(w, rows, args.steps, threads)
    sec = sum(times) / len(times)
    val = wsub.flops_fwd_bwd / sec / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": dtype_name(w.dtype), "data": "synthetic",
        "config": {"workload": describe(w), "sample": f"{rows} of {w.S} MSA rows per step"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{rows} of {w.S} MSA rows, fwd+bwd, torch CPU {torch.get_num_threads()} threads"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def dtype_name(dt):
    return {"bfloat16": "bf16", "float16": "fp16", "float32": "fp32"}[str(dt).split(".")[-1]]


def algorithmic_bytes(w, backward: bool) -> int:
    """Bytes one call has to move: forward reads Q,K,V,bias,mask and writes O,LSE; backward reads
    Q,K,V,O,dO,LSE,bias,mask and writes dQ,dK,dV,dBias (bias and dBias fp32, counted once)."""
    es = 4 if w.dtype == torch.float32 else 2
    t = w.B * w.H * w.S * w.R * w.D * es
    lse = w.B * w.H * w.S * w.R * 4
    bias = w.B * w.H * w.R * w.R * 4
    mask = w.B * w.S * w.R
    return (8 * t + lse + 2 * bias + mask) if backward else (4 * t + lse + bias + mask)


def describe(w):
    return (f"{w.name}: {w.what}; B={w.B} N_seq={w.S} N_res={w.R} H={w.H} D={w.D} "
            f"{dtype_name(w.dtype)} fwd+bwd")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="C2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-rows", type=int, default=128, help="MSA rows per step of the CPU reference arm (capped at the workload's)")
    ap.add_argument("--cpu-baseline-rows", type=int, default=128)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every rank holds the workload's N_seq rows of its own; strong: the workload's rows are split over the ranks")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="sum of d(pair_bias) over the ranks: this package's peer-memory kernel (falls back to NCCL "
                         "if peer mapping is unavailable) or an NCCL all-reduce")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every step's kernels from Python instead of replaying a CUDA graph of one step")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    import evoformer_triton_b200 as evo
    from evoformer_triton_b200 import _lib, attention
    from evoformer_triton_b200.sharding import sharded_evoformer_attention

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the op has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    w = WORKLOADS[args.workload]
    if args.scaling == "strong":
        # strong scaling: one job of w.S MSA rows, split over the ranks (kernel-view rows)
        if w.S % world:
            raise SystemExit(f"--scaling strong needs N_seq={w.S} divisible by the number of GPUs")
        w_job, w = w, w.with_rows(w.S // world)
    else:
        # weak scaling: every rank holds w.S MSA rows of its own; the job has w.S * world rows
        w_job = w.with_rows(w.S * world)
    x = make_inputs(w, rows=w.S, row_offset=rank, device=dev)
    Q, K, V, dO = x["Q"], x["K"], x["V"], x["dO"]
    mask, bias = x["res_mask"], x["pair_bias"]
    Q.requires_grad_(); K.requires_grad_(); V.requires_grad_(); bias.requires_grad_()
    reducer, collective = None, "none"
    if world > 1:
        collective = "NCCL all-reduce of d(pair_bias) inside the step"
        if args.collective == "peer":
            from evoformer_triton_b200.sharding import PeerReducer
            ok = torch.ones(1, device=dev)
            try:
                reducer = PeerReducer(bias.numel(), dev)
            except RuntimeError as e:  # no peer mapping on this box: every rank must agree on the fallback
                ok.zero_()
                if rank == 0:
                    print(f"peer-memory reducer unavailable ({e}); using NCCL", file=sys.stderr)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                reducer = None
            else:
                collective = "peer-memory all-reduce of d(pair_bias) (own kernel over NVLink) inside the step"
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB of L2

    def zero_grads():
        Q.grad = K.grad = V.grad = bias.grad = None

    def step(q=Q, k=K, v=V, m=mask, b=bias, g=dO):
        out = sharded_evoformer_attention(evo.EvoformerAttention.apply, q, k, v, m, b, peer_reducer=reducer)
        out.backward(g)
        return out

    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    for _ in range(max(args.warmup, 3)):
        zero_grads()
        step()
    torch.cuda.synchronize()
    evo.check_device_status()
    launches_per_step = attention.launches["fwd"] + attention.launches["bwd"]
    paths = dict(attention.last_path)

    # ---- one step (forward, backward, exchange) captured in a CUDA graph: the host then issues one
    # launch per step instead of a dozen from Python (about 0.24 ms of host time per step, which
    # eight ranks sharing one host do not always have).  Any failure to capture falls back to
    # launching from Python; all ranks take the same path.
    graph = None
    # (not with the NCCL exchange: a process whose CUDA graph holds NCCL's kernels did not exit)
    if not args.no_graph and (world == 1 or reducer is not None):
        ok = torch.ones(1, device=dev)
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    zero_grads()
                    step()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize()
            zero_grads()
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_):
                step()
            torch.cuda.synchronize()
            g_.replay()
            torch.cuda.synchronize()
            evo.check_device_status()
            graph = g_
        except Exception as e:  # noqa: BLE001
            ok.zero_()
            print(f"[rank {rank}] CUDA graph capture of the step failed ({type(e).__name__}: {e}); launching from Python", file=sys.stderr)
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            graph = None
            torch.cuda.synchronize()
            zero_grads()

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            zero_grads()
            step()

    # ---- timed region: device-resident inputs, L2 flushed between steps
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    pairs = []
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = ev(), ev()
        e0.record()
        run_step()
        e1.record()
        pairs.append((e0, e1))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    step_ms = [a.elapsed_time(b) for a, b in pairs]
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(total_ms.item()) / args.steps
    med = torch.tensor([statistics.median(step_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(med, op=dist.ReduceOp.MAX)
    ms_per_step_median = float(med.item())
    flops_job = w.flops_fwd_bwd * world
    value = flops_job / (ms_per_step * 1e-3) / 1e12

    # ---- peak device memory of one forward + backward of the op, over what was allocated before it
    # (inputs, gradients of earlier steps dropped, the flush buffer): what memory_benchmark.py:38 reports
    zero_grads()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats(dev)
    mem_before = torch.cuda.memory_allocated(dev)
    step()
    torch.cuda.synchronize()
    op_peak_mem = torch.cuda.max_memory_allocated(dev) - mem_before
    zero_grads()

    # ---- per-kernel split (forward kernel, backward call), same flush discipline
    with torch.no_grad():
        qv, kv, vv, dov = (attention._view_dims(t.detach(), "reinterpret") for t in (Q, K, V, dO))
        mk = mask.reshape(w.B, w.S, w.R)
        bs = bias.detach().reshape(w.B, w.H, w.R, w.R)
        f_ms, b_ms = [], []
        for i in range(3 + 10):
            flush.zero_()
            e0, e1, e2 = ev(), ev(), ev()
            e0.record()
            o, lse = attention.attention_forward(qv, kv, vv, mk, bs, w.D ** -0.5)
            e1.record()
            attention.attention_backward(qv, kv, vv, o, lse, mk, bs, w.D ** -0.5, dov)
            e2.record()
            torch.cuda.synchronize()
            if i >= 3:
                f_ms.append(e0.elapsed_time(e1))
                b_ms.append(e1.elapsed_time(e2))
        fwd_ms, bwd_ms = statistics.mean(f_ms), statistics.mean(b_ms)
        bwd_launches = attention.launches["bwd"]
    peaks = measured_peaks()
    dom_bwd = bwd_ms >= fwd_ms
    dom_flops = (w.flops_fwd_bwd - w.flops_fwd) if dom_bwd else w.flops_fwd
    dom_ms = bwd_ms if dom_bwd else fwd_ms
    achieved = dom_flops / (dom_ms * 1e-3) / 1e12
    traffic, traffic_src = ncu_dram_bytes(w.name if args.scaling == "weak" else "", "backward kernel" if dom_bwd else "forward kernel")
    roofline = {
        "bound": "tensor", "kernel": "backward call" if dom_bwd else "forward kernel",
        "launches_in_call": bwd_launches if dom_bwd else attention.launches["fwd"],
        "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
        "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
        "traffic": traffic,
        "traffic_unit": "bytes per launch of the call's main kernel (ncu dram__bytes_read.sum + dram__bytes_write.sum)",
        "traffic_source": traffic_src,
        "algorithmic_bytes": algorithmic_bytes(w, backward=dom_bwd),
        "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
        "fwd_tflops": w.flops_fwd / (fwd_ms * 1e-3) / 1e12,
        "bwd_tflops": (w.flops_fwd_bwd - w.flops_fwd) / (bwd_ms * 1e-3) / 1e12,
    }

    # ---- end to end: host (pinned) inputs in, results back to the host, every step.
    # Every step copies its own inputs from pinned host memory and its five results back.  The
    # copies of neighbouring steps overlap with the compute (three streams, two sets of device
    # input buffers): the value is the sustained rate over K such steps, which is what a caller
    # streaming batches through the op sees; the latency of one isolated step is reported too.
    e2e = None
    if not args.no_e2e:
        host_in = {n: t.detach().cpu().pin_memory() for n, t in
                   dict(Q=Q, K=K, V=V, dO=dO, mask=mask, bias=bias).items()}
        h2d = sum(t.numel() * t.element_size() for t in host_in.values())
        s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        dev_in = [{n: torch.empty_like(t, device=dev) for n, t in host_in.items()} for _ in range(2)]
        host_out = None

        def run(k_steps):
            nonlocal host_out
            torch.cuda.synchronize()
            start, end = ev(), ev()
            freed = [None, None]   # compute of the step that last read an input set
            start.record(s_in)
            for i in range(k_steps):
                buf = i & 1
                with torch.cuda.stream(s_in):
                    if freed[buf] is not None:
                        s_in.wait_event(freed[buf])
                    for n, t in host_in.items():
                        dev_in[buf][n].copy_(t, non_blocking=True)
                    landed = ev()
                    landed.record(s_in)
                with torch.cuda.stream(s_cmp):
                    s_cmp.wait_event(landed)
                    d = dev_in[buf]
                    q, k, v, b = (d[n].detach().requires_grad_() for n in ("Q", "K", "V", "bias"))
                    out = step(q, k, v, d["mask"], b, d["dO"])
                    res = [out.detach(), q.grad, k.grad, v.grad, b.grad]
                    done = ev()
                    done.record(s_cmp)
                    freed[buf] = done
                if host_out is None:
                    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in res]
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done)
                    for hbuf, t in zip(host_out, res):
                        hbuf.copy_(t, non_blocking=True)
                        t.record_stream(s_out)
            end.record(s_out)
            end.synchronize()
            torch.cuda.synchronize()
            return start.elapsed_time(end) / k_steps

        run(2)
        latency_ms = run(1)
        k_e2e = max(8, args.steps)
        e2e_ms = run(k_e2e)
        d2h = sum(t.numel() * t.element_size() for t in host_out)
        t_e2e = torch.tensor([e2e_ms, latency_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
        e2e = {"value": flops_job / (float(t_e2e[0].item()) * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": float(t_e2e[0].item()),
               "steps": k_e2e, "single_step_latency_ms": float(t_e2e[1].item()),
               "how": "copies of neighbouring steps overlap the compute (3 streams, 2 input sets)"}
    evo.check_device_status()

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            rows = min(w.S, args.cpu_baseline_rows)
            oracle_step_seconds(w, rows, 1, threads)
            ts = oracle_step_seconds(w, rows, 3, threads)
            sec = sum(ts) / len(ts)
            cpu = {"value": w.with_rows(rows).flops_fwd_bwd / sec / 1e12, "unit": UNIT, "cores": threads,
                   "kind": "port", "sample": f"{rows} of {w.S} MSA rows, fwd+bwd, 3 runs, torch CPU"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": dtype_name(w.dtype), "data": "synthetic",
            "ms_per_step_median": ms_per_step_median,
            "config": {"workload": describe(w_job if args.scaling == "strong" else w), "rows_per_gpu": w.S,
                       "global_rows": w.S * world,
                       "l2": "256 MB buffer written between timed steps",
                       "collective": collective,
                       "launch": ("one CUDA graph replay per step (forward, backward and the exchange captured once)"
                                  if graph is not None else "every kernel launched from Python"),
                       "paths": {k: {0: "none", 1: "cuda-core", 2: "tcgen05"}[v] for k, v in paths.items()}},
            "frac_of_bf16_peak": value / (peaks["tflops"] * world),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "op_peak_mem_bytes": op_peak_mem, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    graph = None  # the captured step goes before the process group does
    torch.cuda.synchronize()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
