"""Benchmark of the WKV hot path.  Headline: forward + backward of the RWKV-7 recurrence at
H*N = 2048, T = 4096, bf16, batch-sharded over N GPUs with no collective on the path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]
    python bench.py --case {wkv7,wkv7-fwd,wkv6,decode,decode-packed,token-shift,mix,config2} [--batch B --seq T --heads H --iters I]
    torchrun --nproc-per-node N bench.py --case fsdp      (the train-step configuration's collectives)

One "step" is one forward (saving the backward's residual) plus one backward over one batch of
synthetic inputs; results and the residual are preallocated outside the timed region, as a framework
that hands a custom call its result buffers does.  Prints ONE JSON line (rank 0):

* ``value``        tokens/s over all GPUs with inputs resident in HBM (CUDA-event timed).
* ``e2e``          same metric through the host API with HOST buffers: pinned host -> device copies of
                   all inputs and device -> host copies of all outputs inside the timed region.
* ``roofline``     dominant kernel's algorithmic bytes / its event-timed duration vs the measured HBM
                   copy bandwidth; ``traffic`` is the DRAM bytes of one launch from an ncu capture of the
                   kernels whose source hash is recorded beside it (null when the sources changed since).
* ``configs``      the other benchmark configurations, operator slice only: config 1 (fp32 forward,
                   B=2, T=256, H=4), config 2 (bf16 forward, B=8, T=1024, H=12, Bernoulli(1/256)
                   starts, ragged lengths; per layer and x12 layers), config 3 (RWKV-6 fwd+bwd, B=16,
                   T=4096, H=32), config 5 (recurrent decoding, 256 sequences over the GPUs, H=40,
                   32 layers of packed state updated in place, 512 steps after a 1024-token prefill).
* ``strong``       the headline with the GLOBAL batch fixed at 64 sequences (64/N per GPU).
* ``sustained``    the headline step repeated for >= 2 s with its own clock samples.
* ``cpu_baseline`` the AssociativeScan formulation of the reference restated in torch-CPU fp32 on the
                   host cores (rank 0, N=1 only): a bounded sample of the headline (1 sequence x 512
                   tokens, fwd+bwd), config 1 exactly (fwd, fwd+bwd) and the headline shape at B=1
                   forward-only when memory allows.

``--impl reference`` times only that CPU restatement (jaxrwkv itself needs JAX, which is not
installable here) and prints the same line shape with ``"impl": "reference"``.  ``--case`` runs one
small workload a few times and prints its time: the command the ncu summaries under profiles/ use.
"""
import argparse
import hashlib
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

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch at B=8, T=4096, H=32 from the
# ncu captures summarised under profiles/, with the hash of the kernel sources they were taken from.
# Traffic is proportional to B; the figure is dropped (null) when the sources no longer match.
NCU_TRAFFIC = {"sources": "20d31d569af8", "B": 8, "wkv7_fwd": 1974.2e6, "wkv7_bwd": 521.5e6 + 2670.7e6}
# The backward call is timed as a whole (CUDA events around the call): its device time is the sequential
# state-gradient carry followed by the block-parallel gradient kernel; the launch list under profiles/
# gives each kernel's share.  Traffic of the backward is the sum over both kernels.
KERNELS = {"wkv7_fwd": ["wkv7_chunk_fwd_kernel"], "wkv7_bwd": ["wkv7_carry_bwd_kernel<3>", "wkv7_grad_bwd_kernel"]}


def kernel_source_hash():
    h = hashlib.sha1()
    d = os.path.join(ROOT, "jaxrwkv_b200", "csrc")
    for fn in sorted(os.listdir(d)):
        if fn.startswith(("wkv7_chunk", "wkv7_carry", "wkv7_grad", "chunk_common", "tc05", "tmap")):
            h.update(open(os.path.join(d, fn), "rb").read())
    return h.hexdigest()[:12]


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index, period_ms=20):
        self.index, self.rows, self.proc, self.period = index, [], None, period_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            time.sleep(0.3)      # the first sample takes a moment: have it before the region starts
        except Exception:
            self.proc = None
        self.mark = len(self.rows)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        rows = self.rows[max(self.mark - 1, 0):]
        num = lambda x: x.replace(".", "").isdigit()
        sm = [float(r[1]) for r in rows if len(r) >= 9 and num(r[1])]
        mx = [float(r[2]) for r in rows if len(r) >= 9 and num(r[2])]
        pw = [float(r[3]) for r in rows if len(r) >= 9 and num(r[3])]
        reasons = set()
        for r in rows:
            if len(r) >= 9:
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------ CPU arm
def _cpu_assoc(Bc, Tc, Hc, fwd_bwd, reps, warmup, seed):
    """AssociativeScanRWKV (src/jaxrwkv/rwkv7.py:319-346) restated in torch-CPU fp32, all host threads,
    on Bc sequences of Tc tokens.  Returns (tokens/s, ms per repetition)."""
    import torch
    from oracle import make_wkv7_inputs
    from oracle.torch_ref import wkv7_assoc_torch
    d = make_wkv7_inputs(Bc, Tc, Hc, N, seed=seed)
    seqs = []
    for i in range(Bc):
        ts = [torch.tensor(d[n][i], requires_grad=fwd_bwd) for n in ("r", "w", "k", "v", "a", "b", "s0")]
        seqs.append((ts, torch.tensor(d["new_starts"][i])))
    gy, gs = torch.randn(Tc, Hc, N), torch.randn(Hc, N, N)
    times = []
    for it in range(warmup + reps):
        t0 = time.perf_counter()
        for ts, ns in seqs:           # the reference vmaps over the batch; rows are independent
            with torch.set_grad_enabled(fwd_bwd):
                s, y = wkv7_assoc_torch(*ts, Tc, ns)
            if fwd_bwd:
                for x in ts:
                    x.grad = None
                ((y * gy).sum() + (s * gs).sum()).backward()
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    return Bc * Tc / (ms / 1e3), ms


def cpu_reference(steps, warmup, full=True):
    """The CPU baseline: a bounded sample of the headline (1 sequence x 512 tokens at H=32, fwd+bwd through
    autograd), plus - when ``full`` - config 1 exactly and the headline shape at B=1 forward-only."""
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample = f"1 sequence x 512 tokens, H={H}, N={N}, fp32, fwd+bwd via autograd"
    val, ms = _cpu_assoc(1, 512, H, True, steps, warmup, 1237)
    out = {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample, "ms_per_sample": ms,
           "repetitions": steps}
    if full:
        f_val, f_ms = _cpu_assoc(2, 256, 4, False, 5, 1, 1234)
        fb_val, fb_ms = _cpu_assoc(2, 256, 4, True, 5, 1, 1234)
        out["config1"] = {"workload": "config 1 exactly: fp32, B=2, T=256, H=4, N=64", "fwd_tokens_per_s": f_val, "fwd_ms": f_ms,
                          "fwd_bwd_tokens_per_s": fb_val, "fwd_bwd_ms": fb_ms, "repetitions": 5}
        try:
            avail = int(open("/proc/meminfo").read().split("MemAvailable:")[1].split()[0]) * 1024
        except Exception:
            avail = 0
        need = 12 * (T + 1) * H * N * N * 4     # the two (T+1,H,N,N) operands, their masked copies and the scan's levels
        est_s = ms / 1e3 * (T / 512) / 3.0      # forward only, from the fwd+bwd sample (a floor: the big case is memory-bound)
        if est_s > 20.0:
            out["headline_b1_fwd"] = {"skipped": f"estimated at more than {est_s:.0f} s on these {cores} cores: outside the bounded sample"}
        elif avail > need:
            try:
                h_val, h_ms = _cpu_assoc(1, T, H, False, 1, 0, 1237)
                out["headline_b1_fwd"] = {"workload": f"B=1, T={T}, H={H}, N={N}, fp32, forward only", "tokens_per_s": h_val, "ms": h_ms}
            except (MemoryError, RuntimeError) as e:
                out["headline_b1_fwd"] = {"skipped": f"allocation failed: {str(e)[:120]}"}
        else:
            out["headline_b1_fwd"] = {"skipped": f"needs about {need >> 30} GiB of host memory for the materialised (T+1,H,N,N) "
                                                 f"operands and scan levels, {avail >> 30} GiB available"}
    return out


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cpu = cpu_reference(max(args.steps, 1), max(args.warmup, 1), full=True)
    line = {"metric": METRIC, "value": cpu["value"], "unit": "tokens/s", "impl": "reference", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": cpu["ms_per_sample"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"wkv7 fwd+bwd, T={T}, H={H}, N={N}; each step is a bounded CPU sample: {cpu['sample']}"},
            "cpu_baseline": cpu,
            "e2e": {"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ GPU arm
def cuda_ms(torch, fn, warmup, iters):
    """Mean CUDA-event time of ``fn`` over ``iters`` calls after ``warmup`` calls, on the current stream."""
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


class Headline:
    """Inputs, preallocated results and the step function of the headline workload on one GPU."""

    def __init__(self, torch, B, dev, seed, Tn=T, Hn=H):
        from jaxrwkv_b200 import rwkv7, _lib
        from jaxrwkv_b200.synthetic import make_wkv7_device_inputs
        self.torch, self.rwkv7, self.B, self.T, self.H = torch, rwkv7, B, Tn, Hn
        self.x = x = make_wkv7_device_inputs(B, Tn, Hn, N, torch.bfloat16, dev, seed)
        rbytes = _lib.load().b200wkv7_residual_bytes(_lib.BF16, B, Tn, Hn, N)
        self.fb = {"out": torch.empty_like(x["k"]), "new_s": torch.empty_like(x["s0"]),
                   "residual": torch.empty(rbytes, dtype=torch.uint8, device=dev)}
        self.bb = {n: torch.empty_like(x["k"]) for n in ("gw", "gr", "gk", "gv", "ga", "gb")}
        self.bb["gs"] = torch.empty_like(x["s0"])
        self.order = ("r", "w", "k", "v", "a", "b", "s0")

    def fwd(self, need_residual=True):
        x = self.x
        return self.rwkv7.batched_wkv7_fwd(*[x[n] for n in self.order], x["length"], x["new_starts"], self.B,
                                           need_residual=need_residual, buffers=self.fb)

    def step(self, ev=None):
        x = self.x
        if ev:
            ev[0].record()
        (s, y), res = self.fwd()
        if ev:
            ev[1].record()
        g = self.rwkv7.batched_wkv7_bwd(res, (x["ds"], x["dy"]), self.B, buffers=self.bb)
        if ev:
            ev[2].record()
        return s, y, g


def wkv7_bytes(B, Tn, Hn, e=2):
    """Algorithmic bytes of one forward and one backward call: 7 (13) streams per token, 2 (3) states per sequence."""
    return B * (Tn * 7 * Hn * N * e + 2 * Hn * N * N * e), B * (Tn * 13 * Hn * N * e + 3 * Hn * N * N * e)


def bench_configs(torch, dev, world, rank, peak):
    """Operator slices of the other benchmark configurations (CUDA-event times; inputs of configs 2, 3 and 5
    exceed the 126 MB L2, config 1 is 3.7 MB and runs from L2 by its nature)."""
    from jaxrwkv_b200 import rwkv7, rwkv6
    from jaxrwkv_b200.synthetic import make_wkv7_device_inputs, make_wkv6_device_inputs
    out = {}
    order = ("r", "w", "k", "v", "a", "b", "s0")
    gb = lambda nbytes, ms: nbytes / (ms / 1e3) / 1e9
    if world == 1:
        # ---- config 1: fp32 forward, B=2, T=256, H=4, zero state, start only at t=0
        x = make_wkv7_device_inputs(2, 256, 4, N, torch.float32, dev, 1234, s0_scale=0.0, grads=False)
        ms = cuda_ms(torch, lambda: rwkv7.batched_wkv7_fwd(*[x[n] for n in order], x["length"], x["new_starts"], 2, need_residual=False), 3, 20)
        nb = 2 * (256 * 7 * 4 * N * 4 + 2 * 4 * N * N * 4)
        out["config1"] = {"workload": "wkv7 forward, fp32, B=2, T=256, H=4 (sequential fp32 kernel; 8 sequences on 148 SMs)",
                          "ms": ms, "tokens_per_s": 2 * 256 / (ms / 1e3), "algorithmic_bytes": nb, "roofline_frac": gb(nb, ms) / peak}
        # ---- config 2: bf16 forward, B=8, T=1024, H=12, Bernoulli(1/256) starts, ragged lengths
        xs = [make_wkv7_device_inputs(8, 1024, 12, N, torch.bfloat16, dev, 1235 + i, p_start=1 / 256, random_length=True,
                                      s0_scale=0.0, grads=False) for i in range(3)]   # 3 x 76 MB of inputs: rotated, so not L2-resident
        it = [0]

        def c2():
            x = xs[it[0] % 3]
            it[0] += 1
            rwkv7.batched_wkv7_fwd(*[x[n] for n in order], x["length"], x["new_starts"], 8, need_residual=False)
        ms = cuda_ms(torch, c2, 3, 24)
        nb = 8 * (1024 * 7 * 12 * N * 2 + 2 * 12 * N * N * 2)
        out["config2"] = {"workload": "wkv7 forward, bf16, B=8, T=1024, H=12, starts p=1/256, lengths U[T/2,T]; one layer's call",
                          "ms_per_layer": ms, "ms_12_layers": 12 * ms, "tokens_per_s_per_layer": 8 * 1024 / (ms / 1e3),
                          "tokens_per_s_12_layers": 8 * 1024 / (12 * ms / 1e3), "algorithmic_bytes": nb, "roofline_frac": gb(nb, ms) / peak}
        del xs
        # ---- config 3: RWKV-6 fwd+bwd, bf16, B=16, T=4096, H=32, starts p=1/512, s0 ~ N(0, 0.1), dy, dstate ~ N(0,1)
        x = make_wkv6_device_inputs(16, 4096, 32, N, torch.bfloat16, dev, 1236)
        leaves = [x[n].clone().requires_grad_(True) for n in ("r", "k", "v", "w", "u", "s0")]

        def c3():
            for leaf in leaves:
                leaf.grad = None
            s, y = rwkv6.CudaRWKV.inner_loop(*leaves, x["length"], x["new_starts"])
            torch.autograd.backward((y, s), (x["dy"], x["ds"]))
        ms = cuda_ms(torch, c3, 2, 5)
        nb = 16 * (4096 * 14 * 32 * N * 2 + 5 * 32 * N * N * 2)
        out["config3"] = {"workload": "wkv6 fwd+bwd, bf16, B=16, T=4096, H=32, starts p=1/512 (through the operator's autograd hooks)",
                          "ms": ms, "tokens_per_s": 16 * 4096 / (ms / 1e3), "algorithmic_bytes": nb, "roofline_frac": gb(nb, ms) / peak}
        del x, leaves
        torch.cuda.empty_cache()
    # ---- config 5: recurrent decoding, 256 sequences over the GPUs, H=40, L=32 layers of packed state
    Hd, L, steps = 40, 32, 512
    Bd = 256 // world
    D = Hd * N
    state = torch.zeros(Bd, L, 2 + N, D, dtype=torch.bfloat16, device=dev)      # jaxrwkv's container (rwkv7.py:175-180)
    # the carried state comes from a 1024-token prefill through the forward kernel (one layer's worth of
    # streams, in batch slices; every layer gets the same block: the values do not affect the timing)
    for lo in range(0, Bd, 32):
        hi = min(lo + 32, Bd)
        xp = make_wkv7_device_inputs(hi - lo, 1024, Hd, N, torch.bfloat16, dev, 1238 + rank * 64 + lo, s0_scale=0.0, grads=False)
        (s, _), _ = rwkv7.batched_wkv7_fwd(*[xp[n] for n in order], xp["length"], xp["new_starts"], hi - lo, need_residual=False)
        state[lo:hi, :, 2:] = s.reshape(hi - lo, 1, N, D)
        del xp, s
    xd = make_wkv7_device_inputs(Bd, 8, Hd, N, torch.bfloat16, dev, 1239 + rank, grads=False)   # 8 distinct tokens, cycled
    toks = [[xd[n][:, j:j + 1].contiguous() for n in ("r", "w", "k", "v", "a", "b")] for j in range(8)]

    def decode(nsteps):
        for i in range(nsteps):
            a = toks[i % 8]
            for layer in range(L):
                rwkv7.wkv7_step_packed(*a, state, layer)
    decode(2)
    torch.cuda.synchronize()
    # 8 tokens x 32 layers captured once and replayed: the launches come from a CUDA graph, as they would inside a
    # compiled decoding loop, so the host's per-call Python overhead is not what is timed
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            decode(8)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps // 8):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    nb = Bd * Hd * (2 * N * N + 7 * N) * 2
    us_layer = 1e3 * ms / (steps * L)
    out["config5"] = {"workload": f"wkv7 decode step in place on the packed state, bf16, B={Bd}/GPU, H=40, {L} layers x {steps} steps "
                                  f"(2.7 GB of state per 256 sequences cycles through HBM every token)",
                      "us_per_layer_step": us_layer, "ms_per_token_32_layers": ms / steps,
                      "tokens_per_s_per_gpu": Bd * steps / (ms / 1e3), "algorithmic_bytes_per_layer_step": nb,
                      "roofline_frac": nb / (us_layer / 1e6) / 1e9 / peak, "launches": steps * L}
    del state, graph
    torch.cuda.empty_cache()
    if world == 1:
        # the same step at 1024 sequences (8 layers, 2.8 GB of state): a launch moves 708 MB instead of 177 MB, so the
        # fixed cost of a launch (first loads in flight, last stores drained) weighs a quarter as much
        Bw, Lw = 1024, 8
        state = torch.zeros(Bw, Lw, 2 + N, D, dtype=torch.bfloat16, device=dev)
        xw = make_wkv7_device_inputs(Bw, 1, Hd, N, torch.bfloat16, dev, 1240, grads=False)
        aw = [xw[n] for n in ("r", "w", "k", "v", "a", "b")]

        def wide():
            for layer in range(Lw):
                rwkv7.wkv7_step_packed(*aw, state, layer)
        wide()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                wide()
        torch.cuda.current_stream().wait_stream(side)
        ms = cuda_ms(torch, graph.replay, 2, 20)
        nbw = Bw * Hd * (2 * N * N + 7 * N) * 2
        out["config5"]["at_1024_sequences"] = {"us_per_layer_step": 1e3 * ms / Lw, "algorithmic_bytes_per_layer_step": nbw,
                                               "roofline_frac": nbw / (ms / Lw / 1e3) / 1e9 / peak}
        del state, graph
        torch.cuda.empty_cache()
    return out


def run_fsdp_case(args):
    """The collectives of the train-step configuration (config 4: L=24, d_model=2048, vocab 65536, bf16) timed
    on their own under torchrun: every large weight all-gathered on use (twice per step: forward and the
    rematerialised forward of the backward pass) and its gradient reduce-scattered once, through
    jaxrwkv_b200.utils.fsdp (src/jaxrwkv/utils/fsdp.py:42-55).  One JSON line from rank 0."""
    import torch
    import torch.distributed as dist
    from jaxrwkv_b200.utils import fsdp
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    d, L, V = 2048, 24, 65536
    shapes = [(V, d), (V, d)] + [(d, d)] * (4 * L) + [(d, 4 * d), (4 * d, d)] * L      # emb, head, r/k/v/o, ffn key/value
    params = [fsdp.shard_param(torch.empty(s, dtype=torch.bfloat16, device=dev).normal_()) for s in shapes]
    total = sum(a * b for a, b in shapes)
    grads = {}

    def gather_all():
        with torch.no_grad():
            for p in params:
                w = fsdp.gather_param(p)
                del w

    def scatter_all():
        for p in params:
            full = grads.setdefault(tuple(p.v.shape), torch.ones((p.v.shape[0] * world if p.idx == -2 else p.v.shape[0],
                                                                   p.v.shape[1] * world if p.idx == -1 else p.v.shape[1]),
                                                                  dtype=torch.bfloat16, device=dev))
            fsdp._GatherMeanGrads.backward(type("C", (), {"axis": p.v.dim() + p.idx, "group": None})(), full)
    ag = cuda_ms(torch, gather_all, 2, args.iters)
    rs = cuda_ms(torch, scatter_all, 2, args.iters)
    t = torch.tensor([ag, rs], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        nbytes = total * 2
        bus = lambda ms: nbytes * (world - 1) / world / (ms / 1e3) / 1e9
        print(json.dumps({"case": "fsdp", "n_gpus": world, "params": total, "bytes": nbytes, "all_gather_ms": t[0].item(),
                          "reduce_scatter_ms": t[1].item(), "all_gather_bus_gbs": bus(t[0].item()),
                          "reduce_scatter_bus_gbs": bus(t[1].item()),
                          "per_train_step_ms": 2 * t[0].item() + t[1].item()}), flush=True)
    dist.destroy_process_group()


def run_mix_case(torch, dev, B, Tn, Hn, iters):
    """Times b200wkv7_mix_{pre,post}_{fwd,bwd} through the C ABI on (B*T, H*64) bf16 streams and prints, per kernel,
    the time and the algorithmic GB/s (streams read + streams written, 2 bytes per element)."""
    from jaxrwkv_b200 import _lib
    lib = _lib.load()
    C, rows = Hn * N, B * Tn
    g = torch.Generator(device=dev).manual_seed(5)
    stream = lambda: torch.randn(rows, C, device=dev, generator=g).to(torch.bfloat16)
    param = lambda: torch.rand(C, device=dev, generator=g).add_(0.5).to(torch.bfloat16)
    ins = [stream() for _ in range(6)]          # k, wl, al, v, v_first, vl  /  y, r, k, v, g, (gx)
    grads = [stream() for _ in range(5)]
    outs = [torch.empty(rows, C, dtype=torch.bfloat16, device=dev) for _ in range(6)]
    pars = [param() for _ in range(5)]
    n_part = lib.b200wkv7_mix_partial_rows(rows, Hn, N)
    partial = torch.empty(n_part, 5, C, dtype=torch.float32, device=dev)
    st = lambda: torch.cuda.current_stream().cuda_stream
    p = lambda ts: [t.data_ptr() for t in ts]
    calls = {
        "mix_pre_fwd": (11, lambda: lib.b200wkv7_mix_pre_fwd(st(), _lib.BF16, rows, Hn, N, 1, *p(ins), *p(pars), *p(outs[:5]))),
        "mix_pre_bwd": (17, lambda: lib.b200wkv7_mix_pre_bwd(st(), _lib.BF16, rows, Hn, N, 1, *p(ins), *p(pars), *p(grads), *p(outs),
                                                             partial.data_ptr())),
        "mix_post_fwd": (6, lambda: lib.b200wkv7_mix_post_fwd(st(), _lib.BF16, rows, Hn, N, 64e-5, *p(ins[:5]), *p(pars[:3]), outs[0].data_ptr())),
        "mix_post_bwd": (11, lambda: lib.b200wkv7_mix_post_bwd(st(), _lib.BF16, rows, Hn, N, 64e-5, *p(ins[:5]), *p(pars[:3]), ins[5].data_ptr(),
                                                               *p(outs[:5]), partial.data_ptr())),
    }
    for name, (n_streams, fn) in calls.items():
        assert fn() == 0, name
        ms = cuda_ms(torch, fn, 2, iters)
        nbytes = n_streams * rows * C * 2
        print(f"case mix {name} rows={rows} C={C}: {ms * 1e3:.1f} us, {n_streams} streams, {nbytes / ms / 1e6:.0f} GB/s algorithmic")
    # the same forward arithmetic as one framework op after another (what runs without these kernels when nothing fuses)
    k, wl, al, v, vf, vl = ins
    w0, a0, v0, k_k, k_a = pars

    def eager_pre():
        w = -torch.nn.functional.softplus(-(w0 + wl)) - 0.5
        vp = v + (vf - v) * torch.sigmoid(v0 + vl)
        a = torch.sigmoid(a0 + al)
        kk = (k * k_k).view(rows, Hn, N)
        kk = (kk / torch.clamp(torch.linalg.norm(kk, dim=-1, keepdim=True), min=1e-12)).view(rows, C)
        return w, k * (1 + (a - 1) * k_a), vp, -kk, kk * a

    def eager_post():
        y, r, kp, vp, g_ = ins[:5]
        x = torch.nn.functional.group_norm(y, Hn, pars[0], pars[1], 64e-5)
        bonus = (r.view(rows, Hn, N) * kp.view(rows, Hn, N) * pars[2].view(Hn, N)).sum(-1, keepdim=True)
        return (x + (bonus * vp.view(rows, Hn, N)).view(rows, C)) * g_
    for name, fn in (("eager torch, before the operator (forward)", eager_pre), ("eager torch, after the operator (forward)", eager_post)):
        print(f"case mix {name}: {cuda_ms(torch, fn, 2, iters) * 1e3:.1f} us")


def run_case(args):
    """One small workload a few times, its last iteration timed: for profilers and quick checks."""
    if args.case == "fsdp":
        return run_fsdp_case(args)
    import torch
    from jaxrwkv_b200 import rwkv7, rwkv6
    from jaxrwkv_b200.synthetic import make_wkv7_device_inputs, make_wkv6_device_inputs
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    B, Tn, Hn = args.batch, args.seq, args.heads
    if args.case in ("wkv7", "wkv7-fwd"):
        hd = Headline(torch, B, dev, 1, Tn, Hn)
        fn = hd.step if args.case == "wkv7" else (lambda: hd.fwd(need_residual=False))
    elif args.case == "config2":
        x = make_wkv7_device_inputs(B, Tn, Hn, N, torch.bfloat16, dev, 1235, p_start=1 / 256, random_length=True, s0_scale=0.0, grads=False)
        fn = lambda: rwkv7.batched_wkv7_fwd(*[x[n] for n in ("r", "w", "k", "v", "a", "b", "s0")], x["length"], x["new_starts"], B, need_residual=False)
    elif args.case == "wkv6":
        x = make_wkv6_device_inputs(B, Tn, Hn, N, torch.bfloat16, dev, 1236)
        leaves = [x[n].clone().requires_grad_(True) for n in ("r", "k", "v", "w", "u", "s0")]

        def fn():
            for leaf in leaves:
                leaf.grad = None
            s, y = rwkv6.CudaRWKV.inner_loop(*leaves, x["length"], x["new_starts"])
            torch.autograd.backward((y, s), (x["dy"], x["ds"]))
    elif args.case == "decode-packed":   # config 5's step: one layer's block of the packed container, in place, 4 layers
        x = make_wkv7_device_inputs(B, 1, Hn, N, torch.bfloat16, dev, 1, grads=False)
        state = torch.zeros(B, 4, 2 + N, Hn * N, dtype=torch.bfloat16, device=dev)
        state[:, :, 2:] = x["s0"].reshape(B, 1, N, Hn * N)
        a = [x[n] for n in ("r", "w", "k", "v", "a", "b")]

        def fn():
            for layer in range(4):
                rwkv7.wkv7_step_packed(*a, state, layer)
    elif args.case == "token-shift":     # forward + backward of the six-way token shift over (B, T, H*N)
        from jaxrwkv_b200.token_shift import token_shift
        g = torch.Generator(device=dev).manual_seed(3)
        D = Hn * N
        xs = torch.randn(B, Tn, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        prev = torch.randn(B, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        mix = torch.rand(6, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
        length = torch.full((B,), Tn, dtype=torch.int32, device=dev)
        starts = torch.zeros(B, Tn, dtype=torch.uint8, device=dev)
        gout = torch.randn(6, B, Tn, D, device=dev, generator=g).to(torch.bfloat16)

        def fn():
            for leaf in (xs, prev, mix):
                leaf.grad = None
            mixed, new_prev = token_shift(xs, prev, mix, length, starts)
            torch.autograd.backward((mixed,), (gout,))
    elif args.case == "mix":             # the elementwise stages on both sides of the operator, forward and backward
        return run_mix_case(torch, dev, B, Tn, Hn, args.iters)
    else:   # decode: chained single-token steps on a carried state
        x = make_wkv7_device_inputs(B, 1, Hn, N, torch.bfloat16, dev, 1, grads=False)
        st = [x["s0"]]
        a = [x[n] for n in ("r", "w", "k", "v", "a", "b")]

        def fn():
            st[0], _ = rwkv7.wkv7_step(*a, st[0])
    for it in range(args.iters):
        if it == args.iters - 1:
            e0.record()
        fn()
    e1.record()
    torch.cuda.synchronize()
    print(f"case {args.case} B={B} T={Tn} H={Hn}: last iteration {e0.elapsed_time(e1):.3f} ms")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="sequences per GPU (default 8; --case: 2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the configs / strong / sustained blocks")
    ap.add_argument("--case", default=None, choices=["wkv7", "wkv7-fwd", "wkv6", "decode", "decode-packed", "token-shift", "mix", "config2", "fsdp"])
    ap.add_argument("--seq", type=int, default=T)
    ap.add_argument("--heads", type=int, default=H)
    ap.add_argument("--iters", type=int, default=2)
    args = ap.parse_args()
    if args.case is not None:
        args.batch = 2 if args.batch is None else args.batch
        return run_case(args)
    args.batch = 8 if args.batch is None else args.batch
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from jaxrwkv_b200 import _lib
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
    lib = _lib.load()
    B = args.batch
    hd = Headline(torch, B, dev, 1237 + rank)
    x = hd.x

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        hd.step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(args.steps):
        hd.step(evs[i])
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = t_begin.elapsed_time(t_end)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
    ms_step = max_over_ranks(ms_total, dev) / args.steps
    tokens = B * T * world
    value = tokens / (ms_step / 1e3)
    status = lib.b200wkv_device_status()

    # ---- end to end through the public host API: pinned host buffers in, pinned host buffers out ----
    e2e = None
    if not args.no_e2e:
        from jaxrwkv_b200.host import wkv7_fwd_bwd_host, alloc_host_outputs
        names_in = hd.order + ("dy", "ds")
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
        del host_in, host_out

    peak, which = measured_peak_gbs()
    sustained = strong = configs = None
    if not args.no_configs:
        # ---- sustained: the same step for at least 2 s, with its own clock samples
        n_sus = max(int(2200.0 / ms_step), args.steps)
        barrier()
        s2 = ClockSampler(local, period_ms=100)
        if rank == 0:
            s2.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_sus):
            hd.step()
        e1.record()
        barrier()
        sus_ms = max_over_ranks(e0.elapsed_time(e1), dev)
        sustained = {"value": tokens * n_sus / (sus_ms / 1e3), "unit": "tokens/s", "steps": n_sus, "seconds": sus_ms / 1e3,
                     "ms_per_step": sus_ms / n_sus, "clocks": s2.stop() if rank == 0 else None}
        del hd, x
        torch.cuda.empty_cache()
        # ---- strong scaling: the global batch fixed at 64 sequences
        if 64 % world == 0:
            hs = Headline(torch, 64 // world, dev, 1337 + rank)
            for _ in range(2):
                hs.step()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                hs.step()
            e1.record()
            barrier()
            st_ms = max_over_ranks(e0.elapsed_time(e1), dev) / 5
            strong = {"value": 64 * T / (st_ms / 1e3), "unit": "tokens/s", "global_batch": 64, "per_gpu_batch": 64 // world,
                      "ms_per_step": st_ms, "steps": 5, "scaling": "strong"}
            del hs
            torch.cuda.empty_cache()
        configs = bench_configs(torch, dev, world, rank, peak)
        if world > 1:      # config 5 shards its 256 sequences: whole-job tokens/s = sum over ranks (slowest rank's time)
            c5 = configs["config5"]
            slow = max_over_ranks(c5["ms_per_token_32_layers"], dev)
            c5["tokens_per_s_all_gpus"] = 256 / (slow / 1e3)
        status = status or lib.b200wkv_device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    fwd_bytes, bwd_bytes = wkv7_bytes(B, T, H)
    dom, dom_ms, dom_bytes = ("wkv7_bwd", bwd_ms, bwd_bytes) if bwd_ms >= fwd_ms else ("wkv7_fwd", fwd_ms, fwd_bytes)
    achieved = dom_bytes / (dom_ms / 1e3) / 1e9
    src = kernel_source_hash()
    traffic = NCU_TRAFFIC[dom] * B / NCU_TRAFFIC["B"] if (NCU_TRAFFIC[dom] and NCU_TRAFFIC["sources"] == src) else None
    roofline = {"bound": "hbm", "kernel": dom, "kernels": KERNELS[dom], "achieved": achieved, "peak": peak, "peak_source": which,
                "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                "traffic_source": (f"ncu capture at B={NCU_TRAFFIC['B']} of kernel sources {NCU_TRAFFIC['sources']}, scaled by B"
                                   if traffic else f"none for kernel sources {src} (the committed capture is of {NCU_TRAFFIC['sources'] or 'no build'})"),
                "algorithmic_bytes": dom_bytes, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                "fwd_bwd_frac": (fwd_bytes + bwd_bytes) / ((fwd_ms + bwd_ms) / 1e3) / 1e9 / peak}
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_reference(5, 1, full=True)
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"wkv7 fwd+bwd, B={B}/GPU, T={T}, H={H}, N={N}, bf16 (H*N=2048)",
                       "global_batch": B * world, "seq_len": T, "parallelism": f"dp{world} (batch-sharded, no collective)",
                       "l2": "inputs (0.94 GB per step) exceed the 126 MB L2",
                       "buffers": "results and residual preallocated outside the timed region"},
            "value_per_gpu": value / world, "e2e": e2e, "roofline": roofline, "cpu_baseline": cpu,
            "clocks": clocks, "sustained": sustained, "strong": strong, "configs": configs,
            "device_status": status,
            # launches of this library's kernels per step and rank inside the device-timed region.  Forward call:
            # the chunked kernel and the sequential kernel that redoes the call when a decay left the chunked
            # kernel's range (it returns at once otherwise).  Backward call: state-gradient carry, gradient kernel,
            # the one-kernel backward for sequences the forward did not mark as fast (none here: it returns at
            # once) and the sequential backward under the same condition as the forward's; plus one memset node
            # clearing the one-kernel backward's hand-over flags.
            "gpu_launches": 6 * args.steps * world, "memset_nodes": args.steps * world}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
