"""Forward + backward of the RWKV-7 recurrence for callers whose tensors live in HOST memory.

``wkv7_fwd_bwd_host`` takes pinned host tensors, runs the two kernels on the GPU and leaves every
result in pinned host tensors.  The batch is cut into slices that flow through three streams
(host->device copy, compute, device->host copy), so the two PCIe directions and the kernels
overlap; the recurrence is independent per sequence, so slicing the batch changes nothing in the
results.
"""
import torch

from . import rwkv7

_IN = ("r", "w", "k", "v", "a", "b", "s0", "dy", "ds")
_OUT = ("y", "s_out", "dr", "dw", "dk", "dv", "da", "db", "ds0")


def alloc_host_outputs(host_in):
    """Pinned result tensors matching ``host_in`` (y and the six stream gradients like k; states like s0)."""
    like_k, like_s = host_in["k"], host_in["s0"]
    out = {n: torch.empty(like_k.shape, dtype=like_k.dtype).pin_memory() for n in ("y", "dr", "dw", "dk", "dv", "da", "db")}
    out.update({n: torch.empty(like_s.shape, dtype=like_s.dtype).pin_memory() for n in ("s_out", "ds0")})
    return out


class _Pipe:
    def __init__(self, device):
        self.s_in, self.s_c, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))
        self.bufs = {}


_PIPES = {}


def wkv7_fwd_bwd_host(host_in, length, new_starts, host_out=None, device=None, slice_rows=1):
    """host_in: dict of pinned tensors r,w,k,v,a,b,dy (B,T,H,N) and s0,ds (B,H,N,N); ``length`` (B,)
    and ``new_starts`` (B,T) may be host or device tensors.  Returns ``host_out`` (allocated when None)
    holding y, s_out and the seven gradients.  The call returns after the last copy has completed."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B = host_in["k"].shape[0]
    if host_out is None:
        host_out = alloc_host_outputs(host_in)
    pipe = _PIPES.setdefault(device, _Pipe(device))
    length = length.to(device)
    new_starts = new_starts.to(device)
    key = (tuple(host_in["k"].shape[1:]), host_in["k"].dtype, slice_rows)
    if key not in pipe.bufs:
        pipe.bufs[key] = [{n: torch.empty((slice_rows,) + tuple(host_in[n].shape[1:]), dtype=host_in[n].dtype, device=device)
                           for n in _IN} for _ in range(2)]
    bufs = pipe.bufs[key]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_c = [torch.cuda.Event() for _ in range(2)]
    start = torch.cuda.Event()
    start.record(torch.cuda.current_stream(device))
    for s in (pipe.s_in, pipe.s_c, pipe.s_out):
        s.wait_event(start)
    n_slices = (B + slice_rows - 1) // slice_rows
    for i in range(n_slices):
        lo, hi = i * slice_rows, min((i + 1) * slice_rows, B)
        b = bufs[i & 1]
        with torch.cuda.stream(pipe.s_in):
            if i >= 2:
                pipe.s_in.wait_event(ev_c[i & 1])          # the kernels of slice i-2 have read this buffer
            for n in _IN:
                b[n][: hi - lo].copy_(host_in[n][lo:hi], non_blocking=True)
            ev_in[i & 1].record(pipe.s_in)
        with torch.cuda.stream(pipe.s_c):
            pipe.s_c.wait_event(ev_in[i & 1])
            args = [b[n][: hi - lo] for n in ("r", "w", "k", "v", "a", "b", "s0")]
            (s_out, y), res = rwkv7.batched_wkv7_fwd(*args, length[lo:hi], new_starts[lo:hi], hi - lo)
            g = rwkv7.batched_wkv7_bwd(res, (b["ds"][: hi - lo], b["dy"][: hi - lo]), hi - lo)
            ev_c[i & 1] = torch.cuda.Event()
            ev_c[i & 1].record(pipe.s_c)
            outs = dict(zip(_OUT, (y, s_out) + tuple(g)))
        with torch.cuda.stream(pipe.s_out):
            pipe.s_out.wait_event(ev_c[i & 1])
            for n, t in outs.items():
                t.record_stream(pipe.s_out)
                host_out[n][lo:hi].copy_(t, non_blocking=True)
    done = torch.cuda.Event()
    done.record(pipe.s_out)
    torch.cuda.current_stream(device).wait_event(done)
    done.synchronize()
    return host_out
