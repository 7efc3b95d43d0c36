"""Benchmark of the RAM-Net sparse slot-memory hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One pass of the hot path runs one batch of seeded synthetic input of the benchmark shape (random
logits / values of the stated distributions; no dataset is involved):

  prefill (headline)  B8 T16384 H16 U2 P64 K16 C128 bf16, zero fp32 state: joined address decode
                      + gated sparse update/read.  tokens = B*T per pass.
  decode              B256 H16 U2 P64 K16 C128, fp32 state 8.6 GB, 1024 one-token steps.
  addr                B8 T8192 H16 U3 P32 K8 bf16 address decode alone.

A timed region has to last a couple of seconds to be a measurement, so one "step" of the K timed
steps is ``passes_per_step`` passes (stated in ``config``); five regions of K steps are timed and the
median region is reported.  At N > 1 (torchrun, one rank per GPU) every rank runs the full
single-GPU shape on its own batch shard (weak scaling, no collective on the data path); the regions
are bracketed by a barrier and a device synchronise and the slowest rank's device time counts.
``strong`` holds the same kernels on the benchmark batch SPLIT over the ranks (prefill B = 8 / N,
decode batch 256 / N per rank).

Prints ONE JSON line.  ``value`` is whole-job tokens/s with inputs resident in HBM; ``e2e`` is the
same metric through ``ramnet_ops.random_access_memory_attention`` with pinned HOST inputs, the
host->device copies and the device->host copy of y inside the timed region; ``roofline`` is for the
dominant kernel, timed with CUDA events recorded on the launch stream inside the library;
``cpu_baseline`` is the CPU oracle (a port of the reference's algorithm) on a bounded sample of the
same inputs, whose outputs also serve as the parity check of the timed outputs.
``--impl reference`` times that CPU port alone with all host threads.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "ram-net_b200"))
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

SHAPES = {
    "prefill": dict(B=8, T=16384, H=16, U=2, P=64, K=16, C=128, E=8),
    "decode": dict(B=256, T=1024, H=16, U=2, P=64, K=16, C=128, E=8),
    "addr": dict(B=8, T=8192, H=16, U=3, P=32, K=8, C=0, E=8),
}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------------------------
# clocks sampling during the timed region
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = max(mx, float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------------------------
def make_prefill_inputs(s, device, seed, pinned_host=False):
    g = torch.Generator().manual_seed(seed)
    B, T, H, U, P, C = s["B"], s["T"], s["H"], s["U"], s["P"], s["C"]

    def mk(shape, fn=None):
        out = torch.empty(shape, dtype=torch.bfloat16, pin_memory=pinned_host)
        step = max(1, shape[0] // 8)
        for lo in range(0, shape[0], step):  # bounded fp32 scratch
            blk = torch.randn((min(step, shape[0] - lo),) + tuple(shape[1:]), generator=g)
            out[lo:lo + blk.shape[0]] = (fn(blk) if fn else blk).to(torch.bfloat16)
        return out

    q = mk((B, T, H, U, P))
    k = mk((B, T, H, U, P))
    v = mk((B, T, H, C))
    gamma = mk((B, T, H), lambda z: torch.sigmoid(z + 1.0))
    host = dict(q=q, k=k, v=v, gamma=gamma)
    if pinned_host:
        return host
    return {n: t.to(device) for n, t in host.items()}


def lib():
    import ramnet_ops._C as C
    return C.lib


def kernel_times(n):
    buf = (ctypes.c_float * n)()
    got = lib().rn_prof_read(buf, n)
    return [buf[i] for i in range(max(got, 0))]


# ---------------------------------------------------------------------------------------------
# workloads (each returns a dict of measurements for this rank)
# ---------------------------------------------------------------------------------------------
REGIONS = 5            # timed regions per measurement; the median region is reported
REGION_SECONDS = 2.0   # a region is stretched to at least this long by repeating the pass inside a step
PARITY_HEADS = (6, 10)  # heads of batch row 0 that the CPU sample recomputes: two with the CAPE shift, two without
PARITY_TOKENS = 4096


def median(v):
    v = sorted(v)
    return v[len(v) // 2]


def timed_regions(fn, passes, barrier, max_over_ranks):
    """REGIONS regions of `passes` back-to-back calls of fn, each bracketed by barrier + synchronise and CUDA events
    on the current stream; returns the list of region times in ms (max over ranks)."""
    out = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(REGIONS):
        barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(passes):
            fn()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        out.append(max_over_ranks(e0.elapsed_time(e1)))
    return out


def run_prefill(args, device, rank, barrier, max_over_ranks, batch=None, full=True):
    """full=False: only the device-resident timing (used for the strong-scaling shard)."""
    import ramnet_ops  # noqa: F401
    s = dict(SHAPES["prefill"])
    if batch is not None:
        s["B"] = batch
    B, T, H, U, P, K, C, E = (s[k] for k in ("B", "T", "H", "U", "P", "K", "C", "E"))
    A = P ** U
    host = make_prefill_inputs(s, device, seed=rank, pinned_host=True)
    dev = {n: t.to(device) for n, t in host.items()}
    sample = None
    if full and rank == 0:  # the slice of the inputs that the CPU baseline recomputes
        h0, h1 = PARITY_HEADS
        sample = {n: host[n][0:1, :PARITY_TOKENS, h0:h1].clone() for n in ("q", "k", "v", "gamma")}
    w_view = dev["k"].permute(0, 2, 3, 4, 1)
    r_view = dev["q"].permute(0, 2, 3, 4, 1)
    x_view = dev["v"].permute(0, 2, 1, 3)
    g_view = dev["gamma"].permute(0, 2, 1)
    pos = torch.arange(T, device=device, dtype=torch.int32).view(1, T).expand(B, T).contiguous()
    slot0 = torch.zeros(B, H, A, C, device=device)
    mass0 = torch.full((B, H, A), 1.0 / A, device=device)
    ops = torch.ops.ramnet_ops
    keep = {}

    def step():
        idx, val = ops.topk_addr_forward(w_view, r_view, E, A, pos, K, K, 0.0, 0.0)
        keep["out"] = ops.gsu_forward(idx, val, x_view, g_view, slot0, mass0, None, K, K, False, 1e-12)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    # per-kernel device times (events on the launch stream, recorded inside the library)
    lib().rn_prof_enable(1)
    t_addr, t_gsu = [], []
    for _ in range(5):
        idx, val = ops.topk_addr_forward(w_view, r_view, E, A, pos, K, K, 0.0, 0.0)
        t_addr.append(sum(kernel_times(4)))
        ops.gsu_forward(idx, val, x_view, g_view, slot0, mass0, None, K, K, False, 1e-12)
        t_gsu.append(kernel_times(4))
    del idx, val
    lib().rn_prof_enable(0)
    torch.cuda.synchronize()
    est_ms = median(t_addr) + median([sum(t) for t in t_gsu])
    passes_per_step = max(1, int(REGION_SECONDS * 1e3 / max(est_ms * args.steps, 1e-3) + 0.999))
    for _ in range(3):  # the allocator's pool reaches the steady state of the timed loop
        step()
    torch.cuda.synchronize()

    allocs0 = torch.cuda.memory_stats(device).get("num_device_alloc", 0)
    with ClockSampler(torch.cuda.current_device()) as clocks:
        regions = timed_regions(step, args.steps * passes_per_step, barrier, max_over_ranks)
    # cudaMalloc calls inside the timed loops (0 when the caching allocator served every tensor from its pool)
    device_allocs = torch.cuda.memory_stats(device).get("num_device_alloc", 0) - allocs0
    y_dev = keep["out"][0]
    y_sample = None
    if sample is not None:
        h0, h1 = PARITY_HEADS
        y_sample = y_dev.permute(0, 2, 1, 3)[0:1, :PARITY_TOKENS, h0:h1].float().cpu()   # (1, T', 4, C)
    keep.clear()
    names = ["rn_addr_fast_kernel"] + (["rn_gsu_owner_kernel"] if len(t_gsu[0]) == 1 else
                                       ["rn_gsu_schedule_kernel", "rn_gsu_apply_fast_kernel"])
    kms = [median(t_addr)] + [median([t[i] for t in t_gsu]) for i in range(len(t_gsu[0]))]
    result = dict(tokens_per_pass=B * T, regions_ms=regions, passes=args.steps * passes_per_step,
                  passes_per_step=passes_per_step, clocks=clocks.summary(), kernels=dict(zip(names, kms)),
                  launches_per_pass=len(names), device_allocs=device_allocs, batch=B)
    if not full:
        return result

    # ---- end to end through the public API with pinned host inputs -----------------------------------------
    import ramnet_ops as ro
    y_host = torch.empty((B, T, H, C), dtype=torch.bfloat16, pin_memory=True)
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = y_host.numel() * y_host.element_size()
    # Every step copies its inputs from pinned host memory and its output back; the copies of step i+1 /
    # i-1 run on their own streams next to the compute of step i (double-buffered device tensors).
    copy_in, copy_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    main = torch.cuda.current_stream(device)
    dev_in = [dev, {n: torch.empty_like(t, device=device) for n, t in host.items()}]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = torch.cuda.Event()

    def stage_inputs(i):
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(in_free[i & 1])  # the compute that last read this buffer has finished
            for n, t in host.items():
                dev_in[i & 1][n].copy_(t, non_blocking=True)
            in_ready[i & 1].record(copy_in)

    def run_e2e(nsteps):
        for ev in in_free:
            ev.record(main)
        stage_inputs(0)
        for i in range(nsteps):
            if i + 1 < nsteps:
                stage_inputs(i + 1)
            main.wait_event(in_ready[i & 1])
            d = dev_in[i & 1]
            y, _state = ro.random_access_memory_attention(d["k"], d["q"], d["v"], d["gamma"], embed_num=E, top_k=K,
                                                          impl_backend="cuda")
            in_free[i & 1].record(main)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                y_host.copy_(y, non_blocking=True)
                y.record_stream(copy_out)
                out_done.record(copy_out)
        main.wait_event(out_done)  # the timed region ends when the last output is on the host

    e2e_steps = max(4, min(args.steps, 8))
    run_e2e(2)
    torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_e2e(e2e_steps)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    del y_host, dev_in

    # ---- backward of the same pass (address backward + update/read backward), timed per kernel -------------
    bwd = None
    if not args.no_extra:
        idx, val = ops.topk_addr_forward(w_view, r_view, E, A, pos, K, K, 0.0, 0.0)
        d_y = torch.randn(B, T, H, C, device=device, dtype=torch.bfloat16).permute(0, 2, 1, 3)
        d_slot = torch.zeros_like(slot0)
        d_mass = torch.zeros_like(mass0)
        shape6 = [B, H, U, P, A, T]
        tb = {"schedule": [], "replay": [], "reverse": [], "scalar": [], "addr_bwd": []}
        lib().rn_prof_enable(1)
        for i in range(3):
            d_val, d_x, d_g, d_s, d_m = ops.gsu_backward(idx, val, x_view, g_view, slot0, mass0, None, d_y, d_slot, d_mass,
                                                         K, K, False, 1e-12)
            ts = kernel_times(6)
            dw, dr = ops.topk_addr_backward(idx, val, w_view, r_view, d_val, E, pos, K, K, 0.0, 0.0, shape6, torch.bfloat16)
            ta = kernel_times(2)
            if i > 0:
                for n, v in zip(("schedule", "replay", "reverse", "scalar"), ts):
                    tb[n].append(v)
                tb["addr_bwd"] += ta
        lib().rn_prof_enable(0)
        torch.cuda.synchronize()
        bwd = {n: sum(v) / max(len(v), 1) for n, v in tb.items()}
        bwd["total_ms"] = sum(bwd.values())
        del d_val, d_x, d_g, d_s, d_m, dw, dr, d_y, d_slot, d_mass, idx, val
        torch.cuda.empty_cache()

    gsu_name = names[-1]
    per_bh = T * (C * 2 + C * 2) + 2 * A * C * 4  # update/read kernel: x once, y once, slot state in and out
    if gsu_name == "rn_gsu_owner_kernel":
        per_bh += T * 2 * K * 8 + T * 2 + 2 * A * 4  # it also reads idx / val and gamma and moves the mass
    step_bytes = B * H * (T * (2 * U * P * 2 + C * 2 + 2 + C * 2) + 2 * A * C * 4 + 2 * A * 4)
    result.update(
        e2e_ms_total=e2e_ms, e2e_steps=e2e_steps, h2d=h2d, d2h=d2h, bwd=bwd, step_bytes=step_bytes,
        dominant=(gsu_name, B * H * per_bh, kms[-1]), sample=sample, y_sample=y_sample,
        plan=__import__("ramnet_ops._C", fromlist=["x"]).gsu_plan_info(B, H, T, A, C, K, K),
        workload="prefill_fwd B8 T16384 H16 U2 P64(A4096) Kw16 Kr16 C128 bf16, CAPE on 8 heads, zero fp32 state")
    return result


def run_decode(args, device, rank, barrier, max_over_ranks, steps=None, batch=None, check=False):
    import ramnet_ops  # noqa: F401
    s = SHAPES["decode"]
    B, H, U, P, K, C, E = (s[k] for k in ("B", "H", "U", "P", "K", "C", "E"))
    if batch is not None:
        B = batch
    A = P ** U
    nsteps = steps or s["T"]
    g = torch.Generator(device=device).manual_seed(100 + rank)
    slot = torch.empty(B, H, A, C, device=device)
    for b in range(0, B, 16):
        nb = min(16, B - b)
        slot[b:b + nb] = torch.randn(nb, H, A, C, device=device, generator=g) * 0.1
    mass = torch.rand(B, H, A, device=device, generator=g) + 0.1
    nbuf = 16  # rotate through a few input sets; the state is the traffic that matters
    q = torch.randn(nbuf, B, H, U, P, device=device, generator=g).bfloat16()
    k = torch.randn(nbuf, B, H, U, P, device=device, generator=g).bfloat16()
    v = torch.randn(nbuf, B, H, C, device=device, generator=g).bfloat16()
    gm = torch.sigmoid(torch.randn(nbuf, B, H, device=device, generator=g)).bfloat16()
    pos = torch.zeros(B, device=device, dtype=torch.int32)
    nomask = torch.empty(0, dtype=torch.bool, device=device)
    ops = torch.ops.ramnet_ops

    def one(i):
        j = i % nbuf
        pos.fill_(i)
        return ops.topk_autoregressive_(k[j], q[j], v[j], gm[j], slot, mass, nomask, E, pos, K, K, 0.0, 0.0, False, 1e-12)

    for i in range(8):
        one(i)
    torch.cuda.synchronize()
    lib().rn_prof_enable(1)
    tk = []
    for i in range(16):
        one(i)
        tk += kernel_times(2)
    lib().rn_prof_enable(0)
    # eager loop: one operator call per step from Python, events around the loop
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(64):
        one(i)
    e1.record()
    torch.cuda.synchronize()
    eager_ms = e0.elapsed_time(e1) / 64
    # the timed loop replays a CUDA graph of nbuf steps (the operator plus the on-device position increment):
    # launched step by step from Python the loop is bound by the host, not by the kernel
    from ramnet_ops import DecodeGraph
    pos.zero_()
    graph = DecodeGraph(k, q, v, gm, slot, mass, pos, embed_num=E, top_k=K)
    replays = max(1, nsteps // nbuf)
    nsteps = replays * nbuf
    graph.replay()
    regions = timed_regions(graph.replay, replays, barrier, max_over_ranks)
    ms = median(regions)
    per_bh = 2 * U * P * 2 + C * 2 + 2 + 2 * K * C * 4 + 2 * K * 4 + K * C * 4 + C * 2
    kt = median(tk)
    out = dict(tokens_per_s=B * nsteps / (ms / 1e3), ms_per_step=ms / nsteps, kernel_ms=kt, eager_ms_per_step=eager_ms,
               bytes_per_step=B * H * per_bh, steps=nsteps, regions_ms=regions, batch=B)
    if check:
        # one more step on known inputs: batch row 0 before and after, for the CPU oracle
        row_slot, row_mass = slot[0:1].cpu(), mass[0:1].cpu()
        pos.fill_(7)
        y = ops.topk_autoregressive_(k[3], q[3], v[3], gm[3], slot, mass, nomask, E, pos, K, K, 0.0, 0.0, False, 1e-12)
        out["check"] = dict(w=k[3][0:1].float().cpu(), r=q[3][0:1].float().cpu(), x=v[3][0:1].float().cpu(),
                            g=gm[3][0:1].float().cpu(), slot=row_slot, mass=row_mass, y=y[0:1].float().cpu(),
                            slot_after=slot[0:1].cpu(), mass_after=mass[0:1].cpu())
    return out


def run_addr(args, device, rank, barrier, max_over_ranks):
    import ramnet_ops  # noqa: F401
    s = SHAPES["addr"]
    B, T, H, U, P, K, E = (s[k] for k in ("B", "T", "H", "U", "P", "K", "E"))
    A = P ** U
    g = torch.Generator(device=device).manual_seed(200 + rank)
    q = (torch.randn(B, T, H, U, P, device=device, generator=g) * 1.5).bfloat16()
    k = (torch.randn(B, T, H, U, P, device=device, generator=g) * 1.5).bfloat16()
    pos = torch.arange(T, device=device, dtype=torch.int32).view(1, T).expand(B, T).contiguous()
    ops = torch.ops.ramnet_ops
    wv, rv = k.permute(0, 2, 3, 4, 1), q.permute(0, 2, 3, 4, 1)
    for _ in range(3):
        ops.topk_addr_forward(wv, rv, E, A, pos, K, K, 0.0, 0.0)
    torch.cuda.synchronize()
    lib().rn_prof_enable(1)
    tk = []
    for _ in range(5):
        ops.topk_addr_forward(wv, rv, E, A, pos, K, K, 0.0, 0.0)
        tk += kernel_times(2)
    lib().rn_prof_enable(0)
    kt = sum(tk) / len(tk)
    nbytes = B * T * H * (2 * U * P * 2 + 2 * K * 4 + 2 * K * 4)
    return dict(tokens_per_s=B * T / (kt / 1e3), kernel_ms=kt, kernel_gbs=nbytes / (kt / 1e3) / 1e9, bytes=nbytes)


# ---------------------------------------------------------------------------------------------
# twin shapes: the reference's own CUDA kernels only take radix P <= 8, so they cannot run the benchmark shapes;
# shapes with the same slot count and P <= 8 are timed on both implementations through the same public API
# (random_access_memory_attention / topk_addr).  The reference package (its Python files plus its extension built
# for sm_100 from the unmodified sources) is looked for under baseline/_ref/ops_pkg and runs in a subprocess,
# because both packages are called `ramnet_ops`.
# ---------------------------------------------------------------------------------------------
TWIN_SHAPES = {
    # name: (kind, B, T, H, U, P, K, C, dtype)
    "addr_U5P8_K8 (config-2 twin, 32768 slots)": ("addr", 8, 8192, 16, 5, 8, 8, 0, "bfloat16"),
    "prefill_U4P8_K16_C128 (config-3 twin, 4096 slots)": ("prefill", 4, 8192, 16, 4, 8, 16, 128, "bfloat16"),
    "prefill_fwd_bwd_U4P8_K16_C128 (config-3 twin, forward + backward)": ("train", 4, 8192, 16, 4, 8, 16, 128, "bfloat16"),
    "prefill_U4P8_K16_C128 at config-3 size (B8 T16384)": ("prefill", 8, 16384, 16, 4, 8, 16, 128, "bfloat16"),
    "prefill_fwd_bwd_U4P8_K16_C128 at config-3 size (B8 T16384)": ("train", 8, 16384, 16, 4, 8, 16, 128, "bfloat16"),
    "decode_U4P8_K16_C128 (config-4 twin, 4096 slots)": ("decode", 64, 1, 16, 4, 8, 16, 128, "bfloat16"),
    "prefill_U4P4_K4_C64 (config-1 twin, 256 slots)": ("prefill", 1, 512, 4, 4, 4, 4, 64, "float32"),
}
TWIN_REF_DIR = ROOT / "baseline" / "_ref" / "ops_pkg"


def twin_times(tag):
    """Time every twin shape with whichever `ramnet_ops` is first on the import path; returns {name: ms}."""
    import ramnet_ops as ro
    device = torch.device("cuda", 0)
    out = {"package": str(Path(ro.__file__).parent), "impl": tag}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, (kind, B, T, H, U, P, K, C, dt) in TWIN_SHAPES.items():
        dtype = getattr(torch, dt)
        g = torch.Generator(device=device).manual_seed(7)
        A = P ** U
        q = torch.randn(B, T, H, U, P, device=device, generator=g).to(dtype)
        k = torch.randn(B, T, H, U, P, device=device, generator=g).to(dtype)
        E = H // 2
        if kind == "addr":
            pos = torch.arange(T, device=device).view(1, T).expand(B, T).contiguous()
            view = k.permute(0, 2, 3, 4, 1)  # (B,H,U,P,T) view of token-major storage, as the attention layer has it

            def call():
                return ro.topk_addr(view, E, pos, K, 0.0, impl_backend="cuda")
        else:
            v = torch.randn(B, T, H, C, device=device, generator=g).to(dtype)
            gm = torch.sigmoid(torch.randn(B, T, H, device=device, generator=g)).to(dtype)
            if kind == "prefill":
                def call():
                    return ro.random_access_memory_attention(k, q, v, gm, embed_num=E, top_k=K, impl_backend="cuda")
            elif kind == "train":
                leaves = [t.requires_grad_() for t in (q, k, v, gm)]
                dy = torch.randn(B, T, H, C, device=device, generator=g).to(dtype)

                def call():
                    out = ro.random_access_memory_attention(k, q, v, gm, embed_num=E, top_k=K, impl_backend="cuda")
                    (out[0] if isinstance(out, (tuple, list)) else out).backward(dy)
                    for t in leaves:
                        t.grad = None
            else:
                slot = torch.randn(B, H, A, C, device=device, generator=g) * 0.1
                mass = torch.rand(B, H, A, device=device, generator=g) + 0.1
                pos = torch.full((B, 1), 5, device=device)

                def call():
                    return ro.random_access_memory_attention(k, q, v, gm, (slot, mass), embed_num=E, position_ids=pos,
                                                             top_k=K, inplace=True, impl_backend="cuda")
        try:
            for _ in range(3):
                call()
            torch.cuda.synchronize()
            reps = 20 if kind not in ("prefill", "train") or B * T < 10000 else (5 if B * T < 100000 else 2)
            run, how = None, "eager"
            if kind != "train":
                # forward-only shapes are replayed from a CUDA graph of `reps` calls: the small ones (one decode
                # step, config 1) would otherwise measure the host's launch overhead, not the kernels
                try:
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        call()
                    torch.cuda.current_stream().wait_stream(side)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        for _ in range(reps):
                            call()
                    run, how = graph.replay, "cuda_graph"
                    run()
                    torch.cuda.synchronize()
                except Exception:  # noqa: BLE001
                    torch.cuda.synchronize()
                    run, how = None, "eager"
            times = []
            for _ in range(3):
                e0.record()
                if run is not None:
                    run()
                else:
                    for _ in range(reps):
                        call()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1) / reps)
            out[name] = median(times)
            out[name + " timing"] = how
        except Exception as exc:  # noqa: BLE001
            out[name] = f"failed: {type(exc).__name__}: {exc}"[:160]
        del q, k
        torch.cuda.empty_cache()
    return out


def run_twin():
    """ours in this process, the reference in a subprocess; returns the `twin` object of the JSON line."""
    if not (TWIN_REF_DIR / "ramnet_ops").exists():
        return {"unavailable": "reference ops package (with its built extension) not found under baseline/_ref/ops_pkg"}
    ours = twin_times("ours")
    env = dict(os.environ)
    res = subprocess.run([sys.executable, str(Path(__file__).resolve()), "--twin-ref-worker"], capture_output=True, text=True,
                         env=env, timeout=900)
    try:
        ref = json.loads(res.stdout.strip().splitlines()[-1])
    except Exception:  # noqa: BLE001
        return {"unavailable": "reference worker failed: " + (res.stderr or res.stdout)[-300:]}
    twin = {"api": "ramnet_ops.random_access_memory_attention / topk_addr, impl_backend='cuda', CUDA events, median of 3; "
                   "forward-only shapes replayed from a CUDA graph where the package allows capture, else eager",
            "reference_package": ref.get("package"), "our_package": ours.get("package")}
    for name in TWIN_SHAPES:
        a, b = ref.get(name), ours.get(name)
        twin[name] = {"reference_ms": a, "ours_ms": b,
                      "speedup": (a / b) if isinstance(a, float) and isinstance(b, float) and b > 0 else None,
                      "timing": {"reference": ref.get(name + " timing"), "ours": ours.get(name + " timing")}}
    return twin


# ---------------------------------------------------------------------------------------------
# full language model (24 blocks, d_model 2048, 16 heads, U2 P64 K16 C128, SwiGLU 5632, vocab 32000), batch 64
# sharded over the ranks: 2048-token prompt, then 512 greedy tokens.  The model classes are the reference's
# (package `ramnet`, looked for on the import path and under baseline/_ref); the operators are this package's.
# ---------------------------------------------------------------------------------------------
def run_full_model(args, device, rank, world, barrier, max_over_ranks, dist):
    ref_dir = ROOT / "baseline" / "_ref"
    if ref_dir.exists() and str(ref_dir) not in sys.path:
        sys.path.append(str(ref_dir))
    try:
        from ramnet.models import RAMNetConfig, RAMNetForCausalLM
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": f"reference model package `ramnet` not importable: {type(exc).__name__}: {exc}"[:200]}
    from ramnet_ops.layers import GreedyGraphDecoder, use_fused_attention
    B_total, T_prompt, n_new = 64, 2048, 512
    B = max(1, B_total // world)
    cfg = RAMNetConfig(hidden_size=2048, num_attention_heads=16, num_hidden_layers=24, addr_order=2, addr_radix=64,
                       value_chs=128, embed_num=8, addr_top_k=16, hidden_act="SwiGLU", intermediate_size=5632,
                       fuse_norm=False, fuse_cross_entropy=False, vocab_size=32000)
    torch.manual_seed(1234)  # the same random-init weights on every rank
    with torch.device(device):
        model = RAMNetForCausalLM(cfg)
    model = model.to(torch.bfloat16).eval()
    g = torch.Generator(device=device).manual_seed(500 + rank)
    ids = torch.randint(3, 32000, (B, T_prompt), device=device, generator=g)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def prompt(tokens):
        with torch.no_grad():
            out = model.model(input_ids=tokens, use_cache=True)
            first = model.lm_head(out.last_hidden_state[:, -1]).argmax(-1, keepdim=True)
        return out.past_key_values, first

    prompt(ids[:1, :128])  # warm-up of kernels and GEMM heuristics
    torch.cuda.synchronize()
    barrier()
    e0.record()
    cache, first = prompt(ids)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1))

    # decode, the reference's own layer code step by step from Python, for a few tokens (the graph-replayed
    # generation below continues from where these steps leave the state)
    eager_steps = 16
    tok = first
    with torch.no_grad():
        for i in range(eager_steps + 2):
            if i == 2:
                torch.cuda.synchronize()
                e0.record()
            out = model.model(input_ids=tok, past_key_values=cache, use_cache=True)
            tok = model.lm_head(out.last_hidden_state[:, -1]).argmax(-1, keepdim=True)
    e1.record()
    torch.cuda.synchronize()
    eager_ms = e0.elapsed_time(e1) / eager_steps
    first = tok

    # decode, fused one-token step replayed from a CUDA graph; the generated ids of all ranks are gathered (NCCL)
    decoder = GreedyGraphDecoder(model, cache, first)
    barrier()
    torch.cuda.synchronize()
    e0.record()
    new_ids = decoder.generate(n_new)
    if dist is not None:
        gathered = [torch.empty_like(new_ids) for _ in range(world)]
        dist.all_gather(gathered, new_ids)
        new_ids = torch.cat(gathered, dim=0)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    decode_ms = max_over_ranks(e0.elapsed_time(e1))
    state_gb = sum(l.state.slot.numel() * 4 for l in (cache.get_layer(i) for i in range(len(cache)))) / 1e9
    res = {"workload": f"full LM 24 x (d2048, H16, C128, U2 P64 K16, CAPE on 8 heads, SwiGLU 5632), vocab 32000, bf16 random init, "
                       f"batch {B_total} sharded {B} per rank, {T_prompt}-token prompt + {n_new} greedy tokens",
           "prefill_tokens_per_s": world * B * T_prompt / (prefill_ms / 1e3), "prefill_ms": prefill_ms,
           "decode_tokens_per_s": world * B * n_new / (decode_ms / 1e3), "decode_ms_per_token_step": decode_ms / n_new,
           "decode_ms_per_token_step_reference_layer_eager": eager_ms,
           "state_gb_per_rank": state_gb, "gathered_ids_shape": list(new_ids.shape),
           "collective": "all_gather of the generated ids (NCCL)" if dist is not None else "none (one rank)",
           "model_classes": "reference `ramnet` package, attention switched to the fused one-token step for generation"}
    del decoder, cache, model
    torch.cuda.empty_cache()
    return res


# ---------------------------------------------------------------------------------------------
# CPU baseline: the oracle port on a bounded sample of the prefill workload (and the parity check)
# ---------------------------------------------------------------------------------------------
def close_enough(got, want, atol, rtol, max_bad):
    err = (got.double() - want.double()).abs() / (atol + rtol * want.double().abs())
    return bool(torch.isfinite(got).all()) and float((err > 1).double().mean()) <= max_bad


def cpu_baseline(reps=1, sample=None, y_sample=None, decode_check=None):
    """Times the oracle on B1 x 4 heads x 4096 tokens of the prefill workload.  With `sample` (that slice of the
    inputs the GPU ran) the oracle's output is also compared with the GPU's y for the same tokens; with
    `decode_check` one decode step of one batch row is compared as well."""
    from oracle import ramnet_oracle as orc
    s = SHAPES["prefill"]
    B, H, T = 1, PARITY_HEADS[1] - PARITY_HEADS[0], PARITY_TOKENS
    U, P, K, C = s["U"], s["P"], s["K"], s["C"]
    E = max(0, min(PARITY_HEADS[1], s["E"]) - PARITY_HEADS[0])
    A = P ** U
    if sample is None:
        g = torch.Generator().manual_seed(0)
        sample = dict(k=torch.randn(B, T, H, U, P, generator=g).bfloat16(), q=torch.randn(B, T, H, U, P, generator=g).bfloat16(),
                      v=torch.randn(B, T, H, C, generator=g).bfloat16(),
                      gamma=torch.sigmoid(torch.randn(B, T, H, generator=g) + 1).bfloat16())
    w = sample["k"].float().permute(0, 2, 3, 4, 1)
    r = sample["q"].float().permute(0, 2, 3, 4, 1)
    x = sample["v"].float().permute(0, 2, 1, 3)
    gm = sample["gamma"].float().permute(0, 2, 1)
    slot, mass = torch.zeros(B, H, A, C), torch.full((B, H, A), 1.0 / A)
    pos = torch.arange(T).view(1, T)
    best, y = float("inf"), None
    for _ in range(reps + 1):
        t0 = time.perf_counter()
        y, _, _ = orc.ram_attn(w, r, x, gm, slot, mass, None, E, pos, (K, K))
        best = min(best, time.perf_counter() - t0)
    # tokens carry all 16 heads in the metric; the sample ran H=4 of them
    tokens = B * T * H / s["H"]
    out = dict(value=tokens / best, unit="tokens/s", cores=torch.get_num_threads(), kind="port",
               sample=f"oracle.ram_attn on batch row 0, heads {PARITY_HEADS[0]}-{PARITY_HEADS[1] - 1}, first {T} tokens of the "
                      f"prefill inputs (U{U} P{P} K{K} C{C}, bf16-quantised values in fp32), scaled to {s['H']}-head tokens; "
                      f"{best:.2f} s")
    parity = None
    if y_sample is not None:
        ok = close_enough(y_sample, y.permute(0, 2, 1, 3), 7.5e-2, 7.5e-2, 0.02)
        parity = {"prefill_y": "ok" if ok else "MISMATCH"}
        if decode_check is not None:
            d = decode_check
            dec = SHAPES["decode"]
            ry, rs, rm = orc.decode_step(d["w"], d["r"], d["x"], d["g"], d["slot"], d["mass"], None, dec["E"],
                                         torch.full((1,), 7), (dec["K"], dec["K"]))
            ok_d = (close_enough(d["y"], ry, 7.5e-2, 7.5e-2, 0.02) and close_enough(d["slot_after"], rs, 5e-4, 5e-4, 0.01)
                    and close_enough(d["mass_after"], rm, 5e-4, 5e-4, 0.01))
            parity["decode_row"] = "ok" if ok_d else "MISMATCH"
    return out, parity


def run_ncu_case(name):
    """Small single-GPU cases of the same kernels for profiler captures (a few GB at most, inputs
    larger than L2): prints a short JSON and exits."""
    import ramnet_ops  # noqa: F401
    device = torch.device("cuda", 0)
    ops = torch.ops.ramnet_ops
    g = torch.Generator(device=device).manual_seed(0)
    if name in ("prefill_small", "prefill_full"):
        # prefill_full: the benchmark shape itself, three passes (for the one-pass launch list only)
        B, T, H, U, P, K, C, E = (2, 4096, 16, 2, 64, 16, 128, 8) if name == "prefill_small" else (8, 16384, 16, 2, 64, 16, 128, 8)
        A = P ** U
        q = torch.randn(B, T, H, U, P, device=device, generator=g).bfloat16()
        k = torch.randn(B, T, H, U, P, device=device, generator=g).bfloat16()
        v = torch.randn(B, T, H, C, device=device, generator=g).bfloat16()
        gm = torch.sigmoid(torch.randn(B, T, H, device=device, generator=g) + 1).bfloat16()
        pos = torch.arange(T, device=device, dtype=torch.int32).view(1, T).expand(B, T).contiguous()
        slot0, mass0 = torch.zeros(B, H, A, C, device=device), torch.full((B, H, A), 1.0 / A, device=device)
        for _ in range(3):
            idx, val = ops.topk_addr_forward(k.permute(0, 2, 3, 4, 1), q.permute(0, 2, 3, 4, 1), E, A, pos, K, K, 0.0, 0.0)
            y, s1, m1 = ops.gsu_forward(idx, val, v.permute(0, 2, 1, 3), gm.permute(0, 2, 1), slot0, mass0, None, K, K, False, 1e-12)
        out = float(y.float().abs().mean())
    elif name == "prefill_bwd_small":
        # forward + backward of the model shape at B2 T4096 (3.3 GB of backward workspace), two passes
        B, T, H, U, P, K, C, E = 2, 4096, 16, 2, 64, 16, 128, 8
        A = P ** U
        q = torch.randn(B, T, H, U, P, device=device, generator=g).bfloat16().requires_grad_()
        k = torch.randn(B, T, H, U, P, device=device, generator=g).bfloat16().requires_grad_()
        v = torch.randn(B, T, H, C, device=device, generator=g).bfloat16().requires_grad_()
        gm = torch.sigmoid(torch.randn(B, T, H, device=device, generator=g) + 1).bfloat16().requires_grad_()
        dy = torch.randn(B, T, H, C, device=device, generator=g).bfloat16()
        for _ in range(2):
            y = ramnet_ops.random_access_memory_attention(k, q, v, gm, embed_num=E, top_k=K, impl_backend="cuda")
            (y[0] if isinstance(y, (tuple, list)) else y).backward(dy)
        out = float(v.grad.float().abs().mean())
    elif name == "decode_small":
        B, H, U, P, K, C, E = 64, 16, 2, 64, 16, 128, 8
        A = P ** U
        slot = torch.randn(B, H, A, C, device=device, generator=g) * 0.1
        mass = torch.rand(B, H, A, device=device, generator=g) + 0.1
        nomask = torch.empty(0, dtype=torch.bool, device=device)
        pos = torch.zeros(B, device=device, dtype=torch.int32)
        for _ in range(6):
            q = torch.randn(B, H, U, P, device=device, generator=g).bfloat16()
            k = torch.randn(B, H, U, P, device=device, generator=g).bfloat16()
            v = torch.randn(B, H, C, device=device, generator=g).bfloat16()
            gm = torch.sigmoid(torch.randn(B, H, device=device, generator=g)).bfloat16()
            y = ops.topk_autoregressive_(k, q, v, gm, slot, mass, nomask, E, pos, K, K, 0.0, 0.0, False, 1e-12)
        out = float(y.float().abs().mean())
    else:
        B, T, H, U, P, K, E = 2, 8192, 16, 3, 32, 8, 8
        A = P ** U
        q = (torch.randn(B, T, H, U, P, device=device, generator=g) * 1.5).bfloat16()
        k = (torch.randn(B, T, H, U, P, device=device, generator=g) * 1.5).bfloat16()
        pos = torch.arange(T, device=device, dtype=torch.int32).view(1, T).expand(B, T).contiguous()
        for _ in range(3):
            idx, val = ops.topk_addr_forward(k.permute(0, 2, 3, 4, 1), q.permute(0, 2, 3, 4, 1), E, A, pos, K, K, 0.0, 0.0)
        out = float(val.abs().mean())
    torch.cuda.synchronize()
    emit({"ncu_case": name, "checksum": out})


_RESULT_FD = None


def emit(line: dict) -> None:
    """The one JSON line of this run, on the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    # Everything else that libraries write to stdout (NCCL's version banner, for one) goes to stderr, so that
    # stdout carries the JSON line and nothing else.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill", choices=["prefill"])
    ap.add_argument("--no-extra", action="store_true", help="skip the decode and address-only measurements")
    ap.add_argument("--no-full-model", action="store_true", help="skip the full language-model run")
    ap.add_argument("--no-twin", action="store_true", help="skip the twin-shape comparison with the reference's CUDA kernels")
    ap.add_argument("--twin-ref-worker", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--ncu-case", default=None, choices=["prefill_small", "prefill_full", "prefill_bwd_small", "decode_small", "addr_small"],
                    help="run one small case of the kernels (for profiler captures) and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.ncu_case:
        run_ncu_case(args.ncu_case)
        return
    if args.twin_ref_worker:  # subprocess of run_twin(): the REFERENCE package has to win the import
        sys.path.insert(0, str(TWIN_REF_DIR))
        emit(twin_times("reference"))
        return

    if args.impl == "reference":
        if rank != 0:
            return
        torch.set_num_threads(os.cpu_count() or 1)
        vals = []
        for _ in range(max(args.warmup, 0)):
            cpu_baseline(0)
        for _ in range(max(1, min(args.steps, 5))):
            vals.append(cpu_baseline(0)[0])
        v = sorted(x["value"] for x in vals)[len(vals) // 2]
        base = vals[0]
        base["value"] = v
        line = {"impl": "reference", "metric": "prefill_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "prefill_fwd sample on host cores: " + base["sample"]},
                "cpu_baseline": base,
                "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        emit(line)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the hot path has no CPU fallback)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        tns = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(tns, op=dist.ReduceOp.MAX)
        return float(tns.item())

    m = run_prefill(args, device, rank, barrier, max_over_ranks)
    extra = {}
    if not args.no_extra:
        torch.cuda.empty_cache()
        d = run_decode(args, device, rank, barrier, max_over_ranks, check=(rank == 0 and world == 1))
        torch.cuda.empty_cache()
        a = run_addr(args, device, rank, barrier, max_over_ranks)
        extra = {"decode": d, "addr": a}
        torch.cuda.empty_cache()
        if not args.no_full_model:
            extra["full_model"] = run_full_model(args, device, rank, world, barrier, max_over_ranks, dist)
            torch.cuda.empty_cache()
        if world > 1:
            # the benchmark batch split over the ranks (strong scaling): prefill B = 8 / N, decode batch 256 / N
            sp = run_prefill(args, device, rank, barrier, max_over_ranks, batch=max(1, SHAPES["prefill"]["B"] // world), full=False)
            torch.cuda.empty_cache()
            sd = run_decode(args, device, rank, barrier, max_over_ranks, batch=max(1, SHAPES["decode"]["B"] // world))
            torch.cuda.empty_cache()
            extra["strong"] = (sp, sd)

    peak, peak_kind = peaks()
    name, alg_bytes, kms = m["dominant"]
    achieved = alg_bytes / (kms / 1e3) / 1e9
    region_ms = median(m["regions_ms"])
    ms_per_pass = region_ms / m["passes"]
    ms_per_step = region_ms / args.steps
    value = world * m["tokens_per_pass"] / (ms_per_pass / 1e3)
    e2e_value = world * m["tokens_per_pass"] / (m["e2e_ms_total"] / m["e2e_steps"] / 1e3)
    line = {
        "metric": "prefill_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": m["workload"], "io_dtype": "bf16", "state_dtype": "f32", "per_gpu_batch": SHAPES["prefill"]["B"],
                   "passes_per_step": m["passes_per_step"], "ms_per_pass": ms_per_pass,
                   "timing": f"median of {REGIONS} regions of steps x passes_per_step passes each",
                   "l2": "inputs_exceed_l2 (1.3 GB per pass)", "sharding": "batch, no data-path collective", "plan": m["plan"]},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": m["h2d"], "d2h_bytes_per_step": m["d2h"],
                "steps": m["e2e_steps"], "passes_per_step": 1},
        "gpu_launches": m["launches_per_pass"] * m["passes"] * REGIONS, "device_allocs_in_timed_loop": m["device_allocs"],
        "regions_ms": m["regions_ms"], "clocks": m["clocks"],
        "roofline": {"bound": "hbm", "kernel": name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic_of(name, m),
                     "traffic_scaled_from": TRAFFIC.get(name, {}).get("capture"),
                     "algorithmic_bytes_per_launch": alg_bytes, "kernel_ms": kms},
        "roofline_step": {"algorithmic_bytes": m["step_bytes"], "achieved": m["step_bytes"] / (ms_per_pass / 1e3) / 1e9,
                          "frac": m["step_bytes"] / (ms_per_pass / 1e3) / 1e9 / peak},
        "kernel_ms": m["kernels"],
    }
    if m.get("bwd"):
        bw = m["bwd"]
        bwd_bytes = SHAPES["prefill"]["B"] * SHAPES["prefill"]["H"] * 35.7e6
        fb = world * m["tokens_per_pass"] / ((ms_per_pass + bw["total_ms"]) / 1e3)
        line["prefill_bwd"] = {"kernel_ms": bw, "fwd_plus_bwd_tokens_per_s": fb, "algorithmic_bytes": bwd_bytes,
                               "frac": bwd_bytes / (bw["total_ms"] / 1e3) / 1e9 / peak}
        line["fwd_bwd_tokens_per_s"] = fb   # second headline: the benchmark config is forward plus backward
    if extra:
        d, a = extra["decode"], extra["addr"]
        # achieved bandwidth from the graph-replayed step time (kernel plus position increment, back to back);
        # kernel_ms is the same kernel bracketed by events in eager mode, event overhead included
        dec_gbs = d["bytes_per_step"] / (d["ms_per_step"] / 1e3) / 1e9
        line["decode"] = {"tokens_per_s": world * d["tokens_per_s"], "ms_per_step": d["ms_per_step"], "kernel_ms": d["kernel_ms"],
                          "eager_ms_per_step": d["eager_ms_per_step"],
                          "achieved_gbs": dec_gbs, "frac": dec_gbs / peak, "timing": "cuda_graph_replay, median of 5 regions",
                          "algorithmic_bytes_per_step": d["bytes_per_step"], "steps": d["steps"],
                          "workload": "decode B256 H16 U2 P64 K16 C128, fp32 state 8.6 GB"}
        line["addr"] = {"tokens_per_s": world * a["tokens_per_s"], "kernel_ms": a["kernel_ms"], "achieved_gbs": a["kernel_gbs"],
                        "frac": a["kernel_gbs"] / peak, "algorithmic_bytes": a["bytes"],
                        "workload": "addr B8 T8192 H16 U3 P32 K8 bf16"}
        if "full_model" in extra:
            line["full_model"] = extra["full_model"]
        if rank == 0 and world == 1 and not args.no_twin:
            line["twin"] = run_twin()
        if "strong" in extra:
            sp, sd = extra["strong"]
            sp_ms = median(sp["regions_ms"]) / sp["passes"]
            line["strong"] = {
                "prefill_tokens_per_s": world * sp["tokens_per_pass"] / (sp_ms / 1e3), "prefill_ms_per_pass": sp_ms,
                "prefill_batch_per_rank": sp["batch"], "decode_tokens_per_s": world * sd["tokens_per_s"],
                "decode_ms_per_step": sd["ms_per_step"], "decode_batch_per_rank": sd["batch"],
                "note": "total work fixed: the benchmark batch split over the ranks, no data-path collective"}
        else:
            line["strong"] = {"prefill_tokens_per_s": value, "prefill_batch_per_rank": SHAPES["prefill"]["B"],
                              "decode_tokens_per_s": d["tokens_per_s"], "decode_batch_per_rank": d["batch"],
                              "note": "one rank: the split batch is the whole batch"}
    if rank == 0:
        if world == 1:
            torch.set_num_threads(os.cpu_count() or 1)
            base, parity = cpu_baseline(1, m["sample"], m["y_sample"], extra.get("decode", {}).get("check") if extra else None)
            line["cpu_baseline"] = base
            line["parity_check"] = parity
            if parity and any(v != "ok" for v in parity.values()):
                line["parity_check"]["verdict"] = "FAILED: the timed outputs do not match the oracle"
        else:
            line["parity_check"] = "not run at N > 1 (the CPU sample runs at N = 1)"
        emit(line)
    if dist is not None:
        dist.destroy_process_group()


# DRAM traffic of the dominant kernel from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum) of a SMALL
# case, per (b,t,h), to be scaled to the benchmark shape by the token-heads processed (the traffic is x / y rows,
# decoded addresses and the state round trip, all proportional to them at fixed T).  None: no capture yet.
TRAFFIC = {
    "rn_gsu_apply_fast_kernel": {"bytes_per_bth": (139.20384e6 + 63.06048e6) / (2 * 4096 * 16),
                                 "capture": "ncu, --ncu-case prefill_small (B2 T4096 H16), scaled by token-heads"},
}


def traffic_of(name, m):
    t = TRAFFIC.get(name)
    if t is None:
        return None
    s = SHAPES["prefill"]
    return t["bytes_per_bth"] * s["B"] * s["T"] * s["H"]


if __name__ == "__main__":
    main()
