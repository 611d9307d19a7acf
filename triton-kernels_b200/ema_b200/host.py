"""EMA forward + backward for tensors that live in host memory.

The scan rows of different batch entries are independent, so a host-resident problem is cut into batch
slices that flow through three CUDA streams: host-to-device copies of x and dy, the fused forward and
backward kernels, device-to-host copies of y and dx.  PCIe carries both directions at once, so a step
costs about max(bytes in, bytes out) / link bandwidth instead of their sum, and the kernels hide behind
the copies.  Device memory holds `depth` slices of each tensor, whatever the batch size.

    pipe = HostPipeline(x_host.shape, x_host.dtype, per_head=True, device="cuda:0")
    pipe.run(x_host, a_host, dy_host, y_host, dx_host, da_host)      # host tensors, ideally pinned

`run` orders everything after the caller's current stream and, unless told otherwise, returns once the last
copy has landed in the output tensors.  With sync=False it only queues the work: consecutive runs then overlap (the
next run's first copies travel while the previous run's last results are still on their way back), and `wait()`
makes the caller's stream wait for everything queued so far.
"""
import ctypes

import torch

from . import ops
from ._lib import lib


def bind_to_gpu_numa_node(device=None):
    """Restricts the calling process to the CPUs of the NUMA node the GPU hangs off, so that pinned host buffers
    allocated afterwards are local to the GPU's PCIe root.  On a two-socket host with one process per GPU this keeps the
    copies of half of the GPUs off the inter-socket link.  Returns the node number, or None when the platform does not
    tell (no sysfs entry, node -1, not Linux): then nothing is changed.  Call it before allocating pinned memory."""
    import os
    try:
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        props = torch.cuda.get_device_properties(dev)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            spec = f.read().strip()
        cpus = set()
        for part in spec.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


class HostPipeline:
    def __init__(self, shape, dtype, per_head, device="cuda", slices=8, depth=3, prescaled_log=False):
        b, L, h, d = shape
        if b < 1:
            raise ValueError("batch must not be empty")
        self.shape, self.dtype, self.per_head = (b, L, h, d), dtype, per_head
        self.prescaled_log = prescaled_log
        self.device = torch.device(device)
        slices = max(1, min(slices, b))
        self.bounds = [(i * b) // slices for i in range(slices + 1)]        # batch rows of slice i: bounds[i]:bounds[i+1]
        bs = max(self.bounds[i + 1] - self.bounds[i] for i in range(slices))
        self.depth = depth = max(1, min(depth, slices))
        dev = self.device
        mk = lambda: [torch.empty((bs, L, h, d), dtype=dtype, device=dev) for _ in range(depth)]
        self.x, self.dy, self.y, self.dx = mk(), mk(), mk(), mk()
        probe_a = torch.empty((h,) if per_head else (bs, L, h), dtype=torch.float32, device=dev)
        _, nt = ops.n_tiles_of(self.x[0], probe_a)
        self.tile_states = [torch.empty((bs * h, nt, d), dtype=torch.float32, device=dev) for _ in range(depth)]
        # the backward's workspace, sized for the largest slice
        prob = ops._problem(self.x[0], probe_a, self.dx[0], dy=self.dy[0],
                            convention=ops.CONV_PRESCALED_LOG if prescaled_log else ops.CONV_NORTH_STAR)
        ws_floats = (lib().ema_b200_bwd_workspace_bytes(ctypes.byref(prob)) + 3) // 4
        self.workspace = [torch.empty((ws_floats,), dtype=torch.float32, device=dev) for _ in range(depth)]
        fws_floats = (lib().ema_b200_fwd_workspace_bytes(ctypes.byref(prob)) + 3) // 4
        self.fwd_workspace = [torch.empty((max(fws_floats, 1),), dtype=torch.float32, device=dev) for _ in range(depth)]
        # the decay lives in two device buffers used by alternate runs, so that a run's copy of it need not wait for
        # the kernels of the run before
        self.a2 = [torch.empty((h,) if per_head else (b, L, h), dtype=torch.float32, device=dev) for _ in range(2)]
        self.a = self.a2[0]
        self.ev_a_free = [torch.cuda.Event() for _ in range(2)]
        self.n_runs = 0
        # per-head decay: one partial gradient per slice, summed in slice order at the end (deterministic)
        self.da = torch.empty((slices, h) if per_head else (b, L, h), dtype=torch.float32, device=dev)
        self.da_sum = torch.empty((h,), dtype=torch.float32, device=dev) if per_head else None
        self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        ev = lambda: [torch.cuda.Event() for _ in range(depth)]
        self.ev_in, self.ev_comp, self.ev_out = ev(), ev(), ev()
        self.n_launches = 0   # library kernel launches of the last run

    def run(self, x, a, dy, y, dx, da, sync=True):
        """x, dy -> y, dx (host tensors shaped like the problem); a -> da (host, fp32).

        With sync=False the call only queues the work on the pipeline's streams; call wait() (or a run with
        sync=True) before touching the outputs."""
        b, L, h, d = self.shape
        for t in (x, dy, y, dx):
            if tuple(t.shape) != (b, L, h, d) or t.dtype != self.dtype or t.is_cuda:
                raise ValueError("x, dy, y, dx must be host tensors of the pipeline's shape and dtype")
        if tuple(a.shape) != tuple(self.a.shape) or tuple(da.shape) != tuple(self.a.shape):
            raise ValueError("a and da must have the decay's shape")
        n = len(self.bounds) - 1
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_event(start)
        again = self.n_runs > 0          # the ring slots and events carry state from the previous run
        a_dev = self.a2[self.n_runs % 2]
        with torch.cuda.stream(self.s_in):
            if self.n_runs >= 2:
                self.s_in.wait_event(self.ev_a_free[self.n_runs % 2])   # the run before last has read this buffer
            a_dev.copy_(a, non_blocking=True)
            ev_a = torch.cuda.Event()
            ev_a.record(self.s_in)
        self.s_comp.wait_event(ev_a)
        launches = 0
        for i in range(n):
            lo, hi = self.bounds[i], self.bounds[i + 1]
            k, slot = hi - lo, i % self.depth
            xs, dys, ys, dxs = self.x[slot][:k], self.dy[slot][:k], self.y[slot][:k], self.dx[slot][:k]
            with torch.cuda.stream(self.s_in):
                if i >= self.depth or again:
                    self.s_in.wait_event(self.ev_comp[slot])     # the kernels that last used this slot have read x, dy
                xs.copy_(x[lo:hi], non_blocking=True)
                dys.copy_(dy[lo:hi], non_blocking=True)
                self.ev_in[slot].record(self.s_in)
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(self.ev_in[slot])
                if i >= self.depth or again:
                    self.s_comp.wait_event(self.ev_out[slot])    # y, dx of the slice that last used this slot have left
                a_i = a_dev if self.per_head else a_dev[lo:hi]
                da_i = self.da[i] if self.per_head else self.da[lo:hi]
                ts = self.tile_states[slot][: k * h]
                ops.ema_fwd(xs, a_i, out=ys, tile_states=ts, prescaled_log=self.prescaled_log,
                            workspace=self.fwd_workspace[slot])
                ops.ema_bwd(xs, a_i, dys, ts, dx=dxs, ddecay=da_i, workspace=self.workspace[slot],
                            prescaled_log=self.prescaled_log)
                launches += 3   # forward scan, backward scan, decay-gradient reduction
                self.ev_comp[slot].record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_comp[slot])
                y[lo:hi].copy_(ys, non_blocking=True)
                dx[lo:hi].copy_(dxs, non_blocking=True)
                self.ev_out[slot].record(self.s_out)
        with torch.cuda.stream(self.s_comp):
            if self.per_head:
                torch.sum(self.da, dim=0, out=self.da_sum)
                da.copy_(self.da_sum, non_blocking=True)
            else:
                da.copy_(self.da, non_blocking=True)
            self.ev_a_free[self.n_runs % 2].record(self.s_comp)
        self.n_runs += 1
        self.n_launches = launches
        if sync:
            self.wait()
            cur.synchronize()
        return y, dx, da

    def wait(self):
        """Makes the caller's current stream wait for every run queued so far."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_comp, self.s_out):
            cur.wait_stream(s)


def ema_fwd_bwd_host(x, a, dy, y=None, dx=None, da=None, device="cuda", slices=8, depth=3, prescaled_log=False):
    """One-shot form: builds a pipeline for this problem, runs it, synchronises, returns (y, dx, da) on the host."""
    pin = torch.cuda.is_available()
    y = torch.empty_like(x, pin_memory=pin) if y is None else y
    dx = torch.empty_like(x, pin_memory=pin) if dx is None else dx
    da = torch.empty_like(a, pin_memory=pin) if da is None else da
    pipe = HostPipeline(tuple(x.shape), x.dtype, per_head=a.dim() == 1, device=device, slices=slices, depth=depth,
                        prescaled_log=prescaled_log)
    return pipe.run(x, a, dy, y, dx, da)
