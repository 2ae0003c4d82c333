#!/usr/bin/env python
"""Time the reference's own Triton kernels and this project's op on one GPU, side by side, and
run the reference's three scripts, unmodified, against this project's drop-in modules.

    python baseline/run_reference.py triton  [--out FILE]   # reference Triton vs ours: ms, TFLOP/s
    python baseline/run_reference.py scripts [--out DIR]    # test.py, memory_benchmark.py, the sweep
                                                            # of speed_benchmark.py with compat/

Needs ``baseline/_ref`` (see prepare_ref.py) and a GPU.  Values are checked elsewhere (the
parity tests); this script only measures time and peak memory.  Every case runs in a child
process, so a case the Triton compiler rejects (head dimension 8: evoformer.py:176) is recorded
and the rest still runs.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
COMPAT = os.path.join(ROOT, "evoformer_triton_b200", "compat")
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)

# (label, B, S, R, H, D, dtype): the reference's own smallest test shape (test.py:84), the
# benchmark workloads the Triton kernel can run (D >= 16), a slice of C5, and the reference's
# published sweep shape (speed_benchmark.py:37,43: B=4, H=32, D=64, N_seq=1).
CASES = [
    ("test.py:84", 1, 128, 128, 4, 32, "bf16"),
    ("C2", 1, 128, 384, 8, 32, "bf16"),
    ("C3", 1, 384, 384, 4, 32, "bf16"),
    ("C4 (D=8)", 1, 64, 384, 8, 8, "fp16"),
    ("C5 rows 0-63", 2, 64, 768, 8, 64, "bf16"),
] + [("sweep N_CTX=%d" % n, 4, 1, n, 32, 64, "bf16") for n in (128, 256, 384, 512, 768, 1024, 2048)]


def one_case(label, B, S, R, H, D, dt, impl):
    import statistics
    import torch
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16}[dt]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1234)
    shp = (B, S, R, H, D)
    mk = lambda: (torch.randn(shp, generator=g, device=dev) * 0.5).to(dtype).requires_grad_()  # noqa: E731
    Q, K, V = mk(), mk(), mk()
    res_mask = torch.rand((B, S, 1, 1, R), generator=g, device=dev) < 0.9
    res_mask[..., 0] = True
    pair_bias = torch.randn((B, 1, H, R, R), generator=g, device=dev).requires_grad_()
    dO = torch.randn(shp, generator=g, device=dev).to(dtype)
    if impl == "triton":
        import ref_loader
        fn = ref_loader.load_reference_attention().apply
    else:
        import evoformer_triton_b200 as evo
        fn = evo.EvoformerAttention.apply
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def fwd():
        return fn(Q, K, V, res_mask, pair_bias)

    def full():
        Q.grad = K.grad = V.grad = pair_bias.grad = None
        fwd().backward(dO)

    out = {}
    legs = [("fwd", fwd), ("fwd_bwd", full)]
    for name, f in list(legs):  # two untimed calls absorb the Triton autotune sweep (evoformer.py:103-116)
        try:
            for _ in range(2):
                f()
            torch.cuda.synchronize()
        except Exception as e:  # e.g. a kernel the installed Triton refuses to compile
            out[name + "_error"] = f"{type(e).__name__}: {str(e).strip().splitlines()[-1] if str(e).strip() else ''}"[:300]
            legs.remove((name, f))
    torch.cuda.reset_peak_memory_stats()
    base_mem = torch.cuda.memory_allocated()
    for name, f in legs:
        ts = []
        for _ in range(3 + 10):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = f()
            e1.record()
            torch.cuda.synchronize()
            del r
            ts.append(e0.elapsed_time(e1))
        out[name + "_ms"] = statistics.median(ts[3:])
    fm = 2.0 * B * H * S * R * R * D
    if "fwd_ms" in out:
        out["fwd_tflops"] = 2 * fm / out["fwd_ms"] / 1e9
    if "fwd_bwd_ms" in out:
        out["fwd_bwd_tflops"] = 7 * fm / out["fwd_bwd_ms"] / 1e9
    out["peak_mem_over_inputs_gb"] = (torch.cuda.max_memory_allocated() - base_mem) / 2 ** 30
    return out


def run_triton(args):
    lines = []
    for case in CASES:
        for impl in ("triton", "ours"):
            cmd = [sys.executable, os.path.abspath(__file__), "_case", json.dumps(case), impl]
            try:
                r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
                tail = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
                rec = json.loads(tail[-1]) if (r.returncode == 0 and tail) else {
                    "error": (r.stderr.strip().splitlines() or ["exit %d" % r.returncode])[-1][:300]}
            except subprocess.TimeoutExpired:
                rec = {"error": "timed out after 900 s"}
            rec.update({"case": case[0], "shape": dict(zip("BSRHD", case[1:6])), "dtype": case[6], "impl": impl})
            print(json.dumps(rec), flush=True)
            lines.append(rec)
    if args.out:
        with open(args.out, "w") as f:
            for rec in lines:
                f.write(json.dumps(rec) + "\n")


def run_scripts(args):
    """The reference's scripts, as they are, with this project's modules in place of
    ``evoformer`` and ``deepspeed`` (PYTHONPATH = compat/)."""
    out_dir = args.out or "."
    os.makedirs(out_dir, exist_ok=True)
    scripts = os.path.join(HERE, "_ref", "scripts")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([COMPAT, ROOT, os.environ.get("PYTHONPATH", "")]))
    status = {}
    for name in ("test.py", "memory_benchmark.py"):
        r = subprocess.run([sys.executable, os.path.join(scripts, name)], env=env, capture_output=True, text=True,
                           timeout=1800, cwd=out_dir)
        with open(os.path.join(out_dir, name.replace(".py", "_with_compat.log")), "w") as f:
            f.write(r.stdout[-20000:] + "\n--- stderr ---\n" + r.stderr[-5000:] + f"\nexit code {r.returncode}\n")
        status[name] = r.returncode
    # speed_benchmark.py's own driver needs matplotlib (triton.testing.perf_report plots), which is
    # not installed: its benchmark function is called directly instead, for the same sweep.
    code = (
        "import json, speed_benchmark as sb\n"
        "for mode in ('fwd', 'bwd', 'full'):\n"
        "    for n in (128, 256, 384, 512, 768, 1024, 2048):\n"
        "        row = {'mode': mode, 'N_CTX': n}\n"
        "        for prov in ('triton-fp16', 'deepspeed', 'torch'):\n"
        "            row[prov] = sb.bench_flash_attention.fn(sb.BATCH, sb.N_HEADS, n, sb.HEAD_DIM, sb.N_SEQ, mode, prov)\n"
        "        print(json.dumps(row), flush=True)\n")
    r = subprocess.run([sys.executable, "-c", code], env=dict(env, PYTHONPATH=scripts + os.pathsep + env["PYTHONPATH"]),
                       capture_output=True, text=True, timeout=1800, cwd=out_dir)
    with open(os.path.join(out_dir, "speed_benchmark_with_compat.log"), "w") as f:
        f.write("# provider columns: 'triton-fp16' = this project's op through compat/evoformer.py, 'deepspeed' = this\n"
                "# project's op with true head semantics through the compat DS4Sci shim, 'torch' = the naive path\n")
        f.write(r.stdout[-20000:] + "\n--- stderr ---\n" + r.stderr[-5000:] + f"\nexit code {r.returncode}\n")
    status["speed_benchmark.py (sweep function)"] = r.returncode
    print(json.dumps(status))


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "_case":
        case = json.loads(sys.argv[2])
        print(json.dumps(one_case(*case, sys.argv[3])))
        sys.exit(0)
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["triton", "scripts"])
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    (run_triton if a.what == "triton" else run_scripts)(a)
