"""Benchmark of the WKV-7 hot path: forward + backward of the recurrence at the headline
shape (H*N = 2048, T = 4096, bf16), batch-sharded over N GPUs with no collective on the path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

One "step" is one forward (saving the backward's residual) plus one backward over one
batch of synthetic inputs.  Prints ONE JSON line (rank 0).  Keys beyond the usual ones:

* ``value``      tokens/s over all GPUs with inputs resident in HBM (CUDA-event timed).
* ``e2e``        same metric through the C ABI with HOST buffers: pinned host -> device copies
                 of all inputs and device -> host copies of all outputs inside the timed region.
* ``roofline``   dominant kernel's algorithmic bytes / its event-timed duration vs the measured
                 HBM copy bandwidth.
* ``cpu_baseline`` the AssociativeScan formulation of the reference restated in torch-CPU fp32,
                 timed on a bounded sample on the host cores (rank 0, N=1 only).

``--impl reference`` times only that CPU restatement (jaxrwkv itself needs JAX, which is
not installable here) and prints the same line shape with ``"impl": "reference"``.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, N, T = 32, 64, 4096
METRIC = "wkv7_fwd_bwd_tokens_per_s"


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_tokens_per_s(steps, warmup, fwd_bwd=True):
    """AssociativeScanRWKV (src/jaxrwkv/rwkv7.py:319-346) restated in torch-CPU fp32 with all
    host threads, on a bounded sample of the workload: one sequence of 512 tokens at H=32, N=64."""
    import numpy as np
    import torch
    from oracle import make_wkv7_inputs
    from oracle.torch_ref import wkv7_assoc_torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Ts = 512
    d = make_wkv7_inputs(1, Ts, H, N, seed=1237)
    ts = [torch.tensor(d[n][0], requires_grad=fwd_bwd) for n in ("r", "w", "k", "v", "a", "b", "s0")]
    ns = torch.tensor(d["new_starts"][0])
    gy = torch.randn(Ts, H, N)
    gs = torch.randn(H, N, N)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        s, y = wkv7_assoc_torch(*ts, Ts, ns)
        if fwd_bwd:
            for x in ts:
                x.grad = None
            ((y * gy).sum() + (s * gs).sum()).backward()
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    return Ts / (ms / 1e3), ms, cores, f"1 sequence x {Ts} tokens, H={H}, N={N}, fp32, fwd+bwd via autograd"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    val, ms, cores, sample = cpu_reference_tokens_per_s(args.steps, min(args.warmup, 1))
    line = {"metric": METRIC, "value": val, "unit": "tokens/s", "impl": "reference", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"wkv7 fwd+bwd, T={T}, H={H}, N={N}; bounded CPU sample: {sample}"},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def make_device_inputs(torch, B, dtype, device, seed):
    """Seeded synthetic operands at the headline shape (see jaxrwkv_b200.synthetic)."""
    from jaxrwkv_b200.synthetic import make_wkv7_device_inputs
    return make_wkv7_device_inputs(B, T, H, N, dtype, device, seed)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8, help="sequences per GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from jaxrwkv_b200 import rwkv7, _lib
    from jaxrwkv_b200.shard import max_over_ranks

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the WKV operators have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    B = args.batch
    dtype = torch.bfloat16
    x = make_device_inputs(torch, B, dtype, dev, 1237 + rank)
    order = ("r", "w", "k", "v", "a", "b", "s0")

    def step(ev=None):
        if ev:
            ev[0].record()
        (s, y), res = rwkv7.batched_wkv7_fwd(*[x[n] for n in order], x["length"], x["new_starts"], B)
        if ev:
            ev[1].record()
        g = rwkv7.batched_wkv7_bwd(res, (x["ds"], x["dy"]), B)
        if ev:
            ev[2].record()
        return s, y, g

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(args.steps):
        step(evs[i])
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = t_begin.elapsed_time(t_end)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
    ms_step = max_over_ranks(ms_total, dev) / args.steps
    tokens = B * T * world
    value = tokens / (ms_step / 1e3)

    # ---- end to end through the public host API: pinned host buffers in, pinned host buffers out ----
    e2e = None
    if not args.no_e2e:
        from jaxrwkv_b200.host import wkv7_fwd_bwd_host, alloc_host_outputs
        names_in = order + ("dy", "ds")
        host_in = {n: torch.empty(x[n].shape, dtype=x[n].dtype).pin_memory() for n in names_in}
        for n in names_in:
            host_in[n].copy_(x[n])
        host_out = alloc_host_outputs(host_in)
        e_steps = max(3, min(args.steps, 5))
        for _ in range(2):
            wkv7_fwd_bwd_host(host_in, x["length"], x["new_starts"], host_out)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e_steps):
            wkv7_fwd_bwd_host(host_in, x["length"], x["new_starts"], host_out)   # returns after the last D2H copy
        e1.record()
        barrier()
        te_ms = max_over_ranks(e0.elapsed_time(e1), dev)
        h2d = sum(host_in[n].numel() * host_in[n].element_size() for n in names_in)
        d2h = sum(h.numel() * h.element_size() for h in host_out.values())
        e2e = {"value": tokens / (te_ms / e_steps / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e_steps,
               "api": "jaxrwkv_b200.host.wkv7_fwd_bwd_host (batch sliced over copy-in / compute / copy-out streams)"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    e = 2  # bf16 bytes
    fwd_bytes = B * (T * 7 * H * N * e + 2 * H * N * N * e)
    bwd_bytes = B * (T * 13 * H * N * e + 3 * H * N * N * e)
    peak, which = measured_peak_gbs()
    dom, dom_ms, dom_bytes = ("wkv7_bwd", bwd_ms, bwd_bytes) if bwd_ms >= fwd_ms else ("wkv7_fwd", fwd_ms, fwd_bytes)
    achieved = dom_bytes / (dom_ms / 1e3) / 1e9
    # DRAM bytes per launch from the ncu capture at B=2 (summaries of both kernels are kept under profiles/:
    # dram__bytes_read.sum + dram__bytes_write.sum), scaled by B/2 because traffic is proportional to B
    traffic = {"wkv7_bwd": 612.4e6, "wkv7_fwd": 397.4e6}[dom] * B / 2
    roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "peak_source": which,
                "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                "traffic_source": "ncu capture at B=2 scaled by B/2",
                "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                "fwd_bwd_frac": (fwd_bytes + bwd_bytes) / ((fwd_ms + bwd_ms) / 1e3) / 1e9 / peak}
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        val, ms, cores, sample = cpu_reference_tokens_per_s(2, 1)
        cpu = {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample, "ms_per_sample": ms}
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"wkv7 fwd+bwd, B={B}/GPU, T={T}, H={H}, N={N}, bf16 (H*N=2048)",
                       "global_batch": B * world, "seq_len": T, "parallelism": f"dp{world} (batch-sharded, no collective)",
                       "l2": "inputs (0.94 GB per step) exceed the 126 MB L2"},
            "value_per_gpu": value / world, "e2e": e2e, "roofline": roofline, "cpu_baseline": cpu,
            "clocks": clocks, "gpu_launches": 2 * args.steps * world}
    # two launches per step and rank inside the device-timed region: wkv7_chunk_fwd_kernel, wkv7_chunk_bwd_kernel
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
