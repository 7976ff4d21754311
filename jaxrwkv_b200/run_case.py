"""Run the RWKV-7 WKV forward + backward a few times on one synthetic case (for profilers and quick
timing):  python -m jaxrwkv_b200.run_case --batch 2 --seq 4096 --heads 32 --iters 2 [--fp32]"""
import argparse

import torch

from . import rwkv7
from .synthetic import make_wkv7_device_inputs


def decode(a):
    """Recurrent decoding: one token per step, the state carried from step to step."""
    dtype = torch.float32 if a.fp32 else torch.bfloat16
    x = make_wkv7_device_inputs(a.batch, 1, a.heads, 64, dtype, torch.device("cuda"), 1)
    st = x["s0"]
    args = [x[n] for n in ("r", "w", "k", "v", "a", "b")]
    for _ in range(3):
        st, y = rwkv7.wkv7_step(*args, st)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        st, y = rwkv7.wkv7_step(*args, st)
    e1.record()
    torch.cuda.synchronize()
    us = 1e3 * e0.elapsed_time(e1) / a.iters
    nbytes = a.batch * a.heads * (2 * 64 * 64 + 7 * 64) * st.element_size()
    print(f"decode B={a.batch} H={a.heads} {dtype}: {us:.1f} us/step, {a.batch / us:.2f} M tokens/s per layer, "
          f"{nbytes / us / 1e3:.0f} GB/s of state+vector traffic")
    # the same chain replayed from a CUDA graph: launch overhead of the host loop taken out
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        g_st = st.clone()
        with torch.cuda.graph(graph, stream=side):
            cur = g_st
            for _ in range(a.iters):
                cur, y = rwkv7.wkv7_step(*args, cur)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = 1e3 * e0.elapsed_time(e1) / a.iters
    print(f"decode B={a.batch} H={a.heads} {dtype} (CUDA graph of {a.iters} steps): {us:.1f} us/step, "
          f"{a.batch / us:.2f} M tokens/s per layer, {nbytes / us / 1e3:.0f} GB/s of state+vector traffic")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--fp32", action="store_true")
    ap.add_argument("--forward-only", action="store_true")
    ap.add_argument("--decode", action="store_true", help="time --iters chained single-token steps (T = 1)")
    a = ap.parse_args()
    if a.decode:
        return decode(a)
    dtype = torch.float32 if a.fp32 else torch.bfloat16
    x = make_wkv7_device_inputs(a.batch, a.seq, a.heads, 64, dtype, torch.device("cuda"), 1)
    order = ("r", "w", "k", "v", "a", "b", "s0")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for it in range(a.iters):
        if it == a.iters - 1:
            e0.record()
        (s, y), res = rwkv7.batched_wkv7_fwd(*[x[n] for n in order], x["length"], x["new_starts"], a.batch,
                                             need_residual=not a.forward_only)
        if not a.forward_only:
            rwkv7.batched_wkv7_bwd(res, (x["ds"], x["dy"]), a.batch)
    e1.record()
    torch.cuda.synchronize()
    print(f"B={a.batch} T={a.seq} H={a.heads} {dtype}: last iteration {e0.elapsed_time(e1):.3f} ms, "
          f"mean|y| {float(y.float().abs().mean()):.4f}")


if __name__ == "__main__":
    main()
