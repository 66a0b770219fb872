"""Benchmark of the ISSM scan hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c3|c3s|c2|c1|c0] [--dtype bf16|f32]

Prints ONE JSON line (rank 0).  Workloads (the benchmark definition's configurations):
  c3 (default)  one bidirectional ISSM layer forward+backward at the large-scene size: forward scan + reversed
                scan per sample, both with D skip, in-kernel softplus(dt + bias) and clamp, silu(z) gate, initial
                states, final states and their gradients; on more than one GPU followed by the single all-reduce
                of the packed per-head parameter gradients.  c3s is the same with a 10x shorter sequence (the
                small case used for profiler captures).
  c1            the detector-sized layer forward+backward as the detector calls it: bidirectional scan with
                z = None, then the z-gated RMSNorm over all 288 features; the norm kernels are inside the step.
  c2            six stacked bidirectional layers, forward only, dstate 512 / chunk 128, each layer's final states
                seeding the next layer's initial states; --dtype f32 and --dtype bf16 give the two lines.
metric = batch * seqlen * dstate [* layers] / time (points x states per second, whole job); each point-state is
visited by two scan directions.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

if hasattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch"):
    torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: per-GPU batch at N=1, global batch at N>1, sizes, kind of step
    "c3": dict(batch1=16, global_multi=64, L=40000, H=8, P=36, N=256, Q=256, kind="layer",
               desc="large-scene ISSM fwd+bwd, bidirectional (b16 at 1 GPU; global b64 at 2/4/8 GPUs)"),
    "c3s": dict(batch1=16, global_multi=64, L=4096, H=8, P=36, N=256, Q=256, kind="layer",
                desc="c3 with a 10x shorter sequence: the small case used for profiler captures"),
    "c1": dict(batch1=8, global_multi=64, L=1024, H=8, P=36, N=256, Q=256, kind="layer_norm",
               desc="DEST decoder ISSM layer fwd+bwd: bidirectional scan (z = None, as the detector calls it) followed by the "
                    "z-gated RMSNorm over all 288 features (eps 1e-5, weight ~ N(1, 0.02))"),
    "c2": dict(batch1=16, global_multi=64, L=4096, H=8, P=36, N=512, Q=128, kind="stack_fwd", layers=6,
               desc="6 stacked bidirectional ISSM layers, forward only, final states of a layer are the next layer's "
                    "initial states (the six layers share x, B, C, dt and differ in A, D and the incoming states)"),
    "scene": dict(batch1=1, global_multi=8, L=40000, H=8, P=36, N=256, Q=256, kind="layer",
                  desc="ONE large scene per GPU, fwd+bwd, bidirectional: 8 (sample, head) streams for 148 SMs unless the "
                       "sequence is cut into slices (--slices)"),
    "scene16": dict(batch1=1, global_multi=8, L=640000, H=8, P=36, N=256, Q=256, kind="layer",
                    desc="one sequence of 640000 points (16 scenes' worth), fwd+bwd, bidirectional; meant for --slices / "
                         "--sequence-parallel"),
    "c0": dict(batch1=2, global_multi=2, L=1024, H=8, P=36, N=256, Q=256, kind="layer", desc="CPU-runnable reference case"),
}
METRIC, UNIT = "issm_fwd_bwd_points_states_per_s", "points*states/s"
DTYPES = {"bf16": torch.bfloat16, "f32": torch.float32}


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def scan_bytes(b, L, H, P, N, e=2, with_z=True):
    """Algorithmic bytes of ONE scan direction (each input read once, each output written once; e = activation
    element size): fwd  dt + (x, [z,] out) + (B, C) + initial/final states;  bwd  (dt, ddt) +
    (x, dout, dx [, z, out_x, dz]) + (B, C, dB, dC) + state gradients."""
    nz = 1 if with_z else 0
    fwd = L * H * N * e + (2 + nz) * L * H * P * e + 2 * L * N * e + H * P * N * (e + 4)
    bwd = 2 * L * H * N * e + (3 + 3 * nz) * L * H * P * e + 4 * L * N * e + H * P * N * (2 * e + 4)
    return b * fwd, b * bwd


def norm_bytes(rows, hidden, e=2):
    """Gated RMSNorm: fwd reads x, z and writes y (+ rstd); bwd reads x, z, dy (+ rstd) and writes dx, dz."""
    return rows * (3 * hidden * e + 4), rows * (5 * hidden * e + 4)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.lines, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True).start()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for l in self.lines:
            f = [c.strip() for c in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def make_batch(w, batch, sample0, pin=False, dtype=torch.bfloat16):
    """Seeded synthetic inputs of the benchmark's distributions for samples [sample0, sample0+batch):
    x, z ~ N(0,1); B, C ~ N(0,1)/sqrt(N); dt_raw ~ N(0,1) with bias -4 (softplus, clamp [1e-3, 1e-1]);
    A = -exp(U(log 1, log 16)) per head (one draw per layer); D ~ N(0,1); initial states ~ N(0,1)/16;
    dout ~ N(0,1); norm weight ~ N(1, 0.02).  Per-sample seeds, so any GPU count reproduces the same global batch."""
    L, H, P, N = w["L"], w["H"], w["P"], w["N"]
    names = dict(x_f=(L, H, P), x_b=(L, H, P), z=(L, H, P), B_f=(L, 1, N), C_f=(L, 1, N), B_b=(L, 1, N), C_b=(L, 1, N),
                 dt=(L, H, N), init=(H, P, N), dout=(L, H, P))
    if w["kind"] == "stack_fwd":
        del names["dout"], names["z"]
    host = {k: torch.empty((batch,) + s, dtype=dtype, pin_memory=pin) for k, s in names.items()}
    for i in range(batch):
        g = torch.Generator().manual_seed(1000 + sample0 + i)
        for k, s in names.items():
            t = torch.randn(s, generator=g)
            if k[0] in "BC":
                t /= math.sqrt(N)
            if k == "init":
                t /= 16.0
            host[k][i] = t.to(dtype)
    g = torch.Generator().manual_seed(7)
    nl = w.get("layers", 1)
    A = (-torch.exp(torch.rand(nl, H, generator=g) * math.log(16.0)))[:, :, None].repeat(1, 1, N).contiguous()
    par = dict(A=A if nl > 1 else A[0], D=torch.randn(nl, H, generator=g) if nl > 1 else torch.randn(H, generator=g),
               dt_bias=torch.full((H, N), -4.0), norm_w=1 + 0.02 * torch.randn(H * P, generator=g))
    dfinal = torch.randn(batch, H, P, N, generator=torch.Generator().manual_seed(11 + sample0)) / 16.0
    return host, par, dfinal


_SIDE = {}


def _streams():
    key = torch.cuda.current_device()
    if key not in _SIDE:
        _SIDE[key] = (torch.cuda.Stream(), torch.cuda.Stream())
    return _SIDE[key]


def _two_directions(call_f, call_b):
    """The two scan directions are independent, so they are enqueued on two CUDA streams (autograd runs each
    scan's backward on the stream of its forward): with few samples per GPU one direction alone does not fill the
    148 SMs (one CTA per (sample, head))."""
    main = torch.cuda.current_stream()
    s1, s2 = _streams()
    s1.wait_stream(main)
    s2.wait_stream(main)
    with torch.cuda.stream(s1):
        yf, sf = call_f()
    with torch.cuda.stream(s2):
        yb, sb = call_b()
    main.wait_stream(s1)
    main.wait_stream(s2)
    for t in (yf, sf, yb, sb):
        t.record_stream(main)
    return yf, sf, yb, sb


SEQPAR = False  # --sequence-parallel: the ranks hold consecutive parts of ONE sequence (dest3d_b200.seqpar)
SLICES = 1      # --slices: cut every sequence into this many slices run as extra batch entries (0 = chosen from the sizes)


def layer_step(dev, par, dfinal, w, path):
    """One step of the workload through the public interface.  Returns (out, final states, parameter gradients)."""
    from dest3d_b200 import ISSM_chunk_scan_combined, rmsnorm_fn
    if SEQPAR:
        from dest3d_b200.seqpar import issm_scan_sequence_parallel

        def ISSM_chunk_scan_combined(*a, return_final_states=True, **k):   # noqa: F811
            return issm_scan_sequence_parallel(*a, slices=SLICES or None, **k)
    elif SLICES != 1:
        from dest3d_b200.seqpar import issm_scan_chunk_parallel
        plain = ISSM_chunk_scan_combined

        def ISSM_chunk_scan_combined(*a, **k):             # noqa: F811  (same signature plus the slice count)
            if w["kind"] == "stack_fwd":
                return plain(*a, **k)
            return issm_scan_chunk_parallel(*a, slices=SLICES or None, **k)
    main = torch.cuda.current_stream()
    s1, s2 = _streams()
    kind = w["kind"]
    if kind == "stack_fwd":
        init, out = dev["init"], None
        with torch.no_grad():
            for k in range(w["layers"]):
                kw = dict(D=par["D"][k], dt_bias=par["dt_bias"], initial_states=init, dt_softplus=True, dt_limit=(1e-3, 1e-1),
                          return_final_states=True, path=path)
                yf, sf, yb, sb = _two_directions(
                    lambda: ISSM_chunk_scan_combined(dev["x_f"], dev["dt"], par["A"][k], dev["B_f"], dev["C_f"], w["Q"], **kw),
                    lambda: ISSM_chunk_scan_combined(dev["x_b"], dev["dt"], par["A"][k], dev["B_b"], dev["C_b"], w["Q"], reverse=True, **kw))
                out = (yf + yb) * 0.5
                init = ((sf + sb) * 0.5).to(dev["init"].dtype)        # next layer's initial states
        return out, init, {}
    leaves = {k: v.detach().requires_grad_() for k, v in dev.items() if k not in ("dout",)}
    P_ = {k: v.detach().requires_grad_() for k, v in par.items()}
    with_norm = kind == "layer_norm"
    kw = dict(D=P_["D"], z=None if with_norm else leaves["z"], dt_bias=P_["dt_bias"], initial_states=leaves["init"],
              dt_softplus=True, dt_limit=(1e-3, 1e-1), return_final_states=True, path=path)
    yf, sf, yb, sb = _two_directions(
        lambda: ISSM_chunk_scan_combined(leaves["x_f"], leaves["dt"], P_["A"], leaves["B_f"], leaves["C_f"], w["Q"], **kw),
        lambda: ISSM_chunk_scan_combined(leaves["x_b"], leaves["dt"], P_["A"], leaves["B_b"], leaves["C_b"], w["Q"], reverse=True, **kw))
    out = (yf + yb) * 0.5                       # the reference's combine (models/dest_module.py:574)
    fin = (sf + sb) * 0.5
    if with_norm:                               # models/dest_module.py:578-579
        b, L, H, P = out.shape
        out = rmsnorm_fn(out.reshape(b, L, H * P), P_["norm_w"], None, leaves["z"].reshape(b, L, H * P), eps=1e-5,
                         norm_before_gate=False).reshape(b, L, H, P)
    torch.autograd.backward([out, fin], [dev["dout"], dfinal])
    main.wait_stream(s1)
    main.wait_stream(s2)
    grads = {"dA": P_["A"].grad, "ddt_bias": P_["dt_bias"].grad, "dD": P_["D"].grad}
    if with_norm:
        grads["dW"] = P_["norm_w"].grad
    return out, fin, grads


def run_mine(args):
    from dest3d_b200 import _lib, issm_combined
    from dest3d_b200.dist import PackedParamGrads, max_over_ranks, shard_samples
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    w = WORKLOADS[args.workload]
    dtype = DTYPES[args.dtype]
    gbatch = w["batch1"] if world == 1 else w["global_multi"]
    mine = shard_samples(gbatch, world, rank)
    seqpar = SEQPAR and world > 1
    if seqpar:                                             # every rank: all samples, 1 / world of the points
        gbatch = w["batch1"]
        mine = range(0, gbatch)
    batch = len(mine)
    L_total = w["L"]
    # With several ranks pulling their inputs from host memory at once, pin each rank's buffers on its GPU's NUMA
    # node (skipped at one GPU, where the CPU baseline leg wants every core; ISSM_BENCH_NUMA=0 switches it off).
    numa_cpus = 0
    if world > 1 and os.environ.get("ISSM_BENCH_NUMA", "1") != "0":
        from dest3d_b200.dist import bind_to_gpu_numa_node
        numa_cpus = bind_to_gpu_numa_node(local)
    host, par, dfinal = make_batch(w, batch, mine.start, pin=not seqpar, dtype=dtype)
    if seqpar:
        lo, hi = L_total * rank // world, L_total * (rank + 1) // world
        host = {k: (v if k == "init" else v[:, lo:hi].contiguous()).pin_memory() for k, v in host.items()}
        w = dict(w, L=hi - lo)
    dev = {k: v.to(device, non_blocking=True) for k, v in host.items()}
    par = {k: v.to(device) for k, v in par.items()}
    dfinal = dfinal.to(device)
    shapes = {"dA": par["A"].shape, "ddt_bias": par["dt_bias"].shape, "dD": par["D"].shape}
    if w["kind"] == "layer_norm":
        shapes["dW"] = par["norm_w"].shape
    packed = PackedParamGrads(shapes, device) if w["kind"] != "stack_fwd" else None
    path = args.path
    nl = w.get("layers", 1)

    def step(inputs=None):
        out, fin, grads = layer_step(inputs if inputs is not None else dev, par, dfinal, w, path)
        if packed is not None:
            packed.load(grads).all_reduce()
        return out, fin

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def status_or_die(where):
        """A bounded device-side wait that expired makes the kernels leave early: such a step must not be
        reported as a (fast) throughput."""
        st = issm_combined.device_status(device)
        if st & 1:
            raise SystemExit(f"bench: device status {st} after {where}: a bounded wait expired, results invalid")
        return st

    for _ in range(args.warmup):
        step()
    sync_all()
    status_or_die("warm-up")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync_all()
    launches = _lib.launch_count() - l0
    ms = max_over_ranks(e0.elapsed_time(e1), device)
    clocks = sampler.stop() if rank == 0 else None
    status = status_or_die("the timed region")
    L, H, P, N = w["L"], w["H"], w["P"], w["N"]
    value = gbatch * L_total * N * nl * args.steps / (ms * 1e-3)

    # The same step replayed from a CUDA graph (one GPU, --graph): at the detector's size a step is ~20 short launches
    # and the eager number is bound by launch latency; a training loop with static shapes can capture it once.
    graph_info = None
    if args.graph and world == 1:
        try:
            torch.cuda.synchronize()
            gstream = torch.cuda.Stream()
            with torch.cuda.stream(gstream):
                for _ in range(2):
                    step()                                  # warm the allocator's pools on the capture stream
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=gstream):
                step()
            for _ in range(args.warmup):
                graph.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(args.steps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            gms = e0.elapsed_time(e1) / args.steps
            status_or_die("the graph replay")
            graph_info = {"ms_per_step": gms, "value": gbatch * L_total * N * nl / (gms * 1e-3), "unit": UNIT}
            del graph
        except Exception as exc:                            # a capture that is refused is reported, not fatal
            graph_info = {"error": f"{type(exc).__name__}: {str(exc)[:200]}"}

    # end to end through the public call with HOST buffers: H2D of the step's inputs from pinned memory,
    # the layer, D2H of the combined output, final states and packed parameter gradients.  The steps are
    # pipelined the way a training loop with a prefetching loader runs them: the H2D copy of step i+1 (copy
    # stream, second set of device buffers) overlaps the layer of step i.  Every step's inputs are copied and
    # every step's results are read back inside the timed region; the first copy is not overlapped.
    out_h = torch.empty((batch, L, H, P), dtype=dtype, pin_memory=True)
    fin_h = torch.empty((batch, H, P, N), dtype=torch.float32 if w["kind"] != "stack_fwd" else dtype, pin_memory=True)
    pg_h = torch.empty(packed.flat.shape, dtype=torch.float32, pin_memory=True) if packed is not None else None
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_h.numel() * out_h.element_size() + fin_h.numel() * fin_h.element_size() + (pg_h.numel() * 4 if pg_h is not None else 0)

    bufs = (dev, {k: torch.empty_like(v) for k, v in dev.items()})
    copy_stream = torch.cuda.Stream()
    ready = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(nsteps):
        main = torch.cuda.current_stream()
        copy_stream.wait_stream(main)
        for i in range(nsteps):
            j = i & 1
            with torch.cuda.stream(copy_stream):
                if i >= 2:
                    copy_stream.wait_event(freed[j])       # the layer of step i-2 is done with this buffer set
                for k, v in host.items():
                    bufs[j][k].copy_(v, non_blocking=True)
                ready[j].record(copy_stream)
            main.wait_event(ready[j])
            out, fin = step(bufs[j])
            freed[j].record(main)
            out_h.copy_(out, non_blocking=True)
            fin_h.copy_(fin, non_blocking=True)
            if pg_h is not None:
                pg_h.copy_(packed.flat, non_blocking=True)

    e2e_steps = max(2, min(args.steps, 6))
    e2e_run(2)
    sync_all()
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    sync_all()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1), device)
    e2e_value = gbatch * L_total * N * nl * e2e_steps / (ms_e2e * 1e-3)
    status_or_die("the end-to-end region")

    # roofline of the dominant kernel, timed live with CUDA events on the launching stream
    roof, cpu = None, None
    if rank == 0:
        roof = kernel_roofline(dev, par, dfinal, w, batch, path, dtype)
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(w)
    if rank == 0:
        line = {"metric": METRIC if w["kind"] != "stack_fwd" else "issm_fwd_points_states_per_s", "value": value, "unit": UNIT,
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if seqpar else "weak",
                "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
                "config": {"workload": f"{args.workload}: {w['desc']}", "global_batch": gbatch, "per_gpu_batch": batch,
                           "seqlen": L_total, "points_per_gpu": L if seqpar else None, "nheads": H, "headdim": P, "dstate": N, "chunk_size": w["Q"], "directions": 2,
                           "layers": nl, "path": path, "slices_per_sequence": SLICES, "resolved_path": roof.get("resolved_path") if roof else None,
                           "l2": "inputs larger than L2 (no flush needed)",
                           "scaling_note": "N = 1 runs batch 16, N > 1 a global batch of 64 split over the ranks: compare "
                                           "points*states/s across N, not step times",
                           "parallelism": (f"sp{world}: every rank holds 1/{world} of the points of every sequence" if seqpar
                                           else f"dp{world} by sample, both directions on one GPU")},
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps,
                        "pipelining": "H2D of step i+1 overlaps the layer of step i (two device buffer sets)",
                        "host_numa_bound_cpus": numa_cpus},
                "gpu_launches": int(launches), "cuda_graph": graph_info, "device_status": status, "clocks": clocks, "roofline": roof, "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch on the small profiling case c3s
# (batch 16, L = 4096) from the ncu captures summarised in profiles/k_fwd_tensor_c3s.md and
# profiles/k_bwd_tensor_c3s.md; traffic grows in proportion to batch x L
NCU_C3S_TRAFFIC = {"fwd": 413.6e6 + 247.9e6, "bwd": 698.3e6 + 835.9e6}
NCU_C3S_SOURCE = "ncu capture of the c3s case (profiles/k_fwd_tensor_c3s.md, profiles/k_bwd_tensor_c3s.md), scaled by batch x L"


def _median_ms(fn, warm=2, reps=5):
    e = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ts = []
    for i in range(warm + reps):
        e[0].record()
        r = fn()
        e[1].record()
        torch.cuda.synchronize()
        if i >= warm:
            ts.append(e[0].elapsed_time(e[1]))
    # median of the repetitions: a call that has to grow the caching allocator's pool is not a kernel time
    return sorted(ts)[reps // 2], [round(t, 3) for t in ts], r


def kernel_roofline(dev, par, dfinal, w, batch, path, dtype):
    """Time the forward call and the backward call of one direction separately (CUDA events on the current
    stream), plus the two norm calls where the workload has them; report the roofline of the slowest one."""
    from dest3d_b200 import issm_bwd, issm_fwd, _lib, issm_combined
    import ctypes as ct
    hbm, src = peaks()
    e = dtype.itemsize
    kind = w["kind"]
    A = par["A"][0] if kind == "stack_fwd" else par["A"]
    D = par["D"][0] if kind == "stack_fwd" else par["D"]
    z = dev.get("z") if kind == "layer" else None
    kw = dict(D=D, z=z, dt_bias=par["dt_bias"], initial_states=dev["init"], dt_softplus=True, dt_limit=(1e-3, 1e-1), path=path)
    need_bwd = kind != "stack_fwd"
    tf, tfs, res = _median_ms(lambda: issm_fwd(dev["x_f"], dev["dt"], A, dev["B_f"], dev["C_f"], w["Q"], save_states=need_bwd, **kw))
    fb, bb = scan_bytes(batch, w["L"], w["H"], w["P"], w["N"], e=e, with_z=z is not None)
    stages = {"forward call (k_fwd_tensor)": (tf, fb, "fwd")}
    out = {"fwd_ms_one_direction": tf, "fwd_ms_reps": tfs, "fwd_frac": fb / (tf * 1e-3) / 1e9 / hbm}
    if need_bwd:
        out_x, saved = res[1], res[3]
        tb, tbs, _ = _median_ms(lambda: issm_bwd(dev["dout"], dev["x_f"], dev["dt"], A, dev["B_f"], dev["C_f"], out_x, w["Q"],
                                                 dfinal_states=dfinal, saved_states=saved, **kw))
        stages["backward call (k_bwd_tensor + head/batch reductions)"] = (tb, bb, "bwd")
        out.update({"bwd_ms_one_direction": tb, "bwd_ms_reps": tbs, "bwd_frac": bb / (tb * 1e-3) / 1e9 / hbm})
    if kind == "layer_norm":
        from dest3d_b200 import rmsnorm_fn
        b, L, H, P = dev["x_f"].shape
        xk = dev["x_f"].reshape(b * L, H * P).detach().requires_grad_()
        zk = dev["z"].reshape(b * L, H * P).detach().requires_grad_()
        wk = par["norm_w"].detach().requires_grad_()
        nf, nb = norm_bytes(b * L, H * P, e)
        tnf, _, y = _median_ms(lambda: rmsnorm_fn(xk, wk, None, zk, eps=1e-5, norm_before_gate=False))
        dy = dev["dout"].reshape(b * L, H * P)
        tnb, _, _ = _median_ms(lambda: torch.autograd.grad(y, (xk, zk, wk), dy, retain_graph=True))
        out.update({"norm_fwd_ms": tnf, "norm_bwd_ms": tnb, "norm_fwd_frac": nf / (tnf * 1e-3) / 1e9 / hbm,
                    "norm_bwd_frac": nb / (tnb * 1e-3) / 1e9 / hbm})
        # the same two kernels on 2^18 rows (151 MB per tensor, larger than L2): at the detector's 8192 rows a call
        # moves 14 MB and is bound by launch latency, not by HBM
        rows = 1 << 18
        g = torch.Generator(device="cuda").manual_seed(3)
        xl = torch.randn(rows, H * P, device="cuda", generator=g).to(dtype).requires_grad_()
        zl = torch.randn(rows, H * P, device="cuda", generator=g).to(dtype).requires_grad_()
        dyl = torch.randn(rows, H * P, device="cuda", generator=g).to(dtype)
        nfl, nbl = norm_bytes(rows, H * P, e)
        tl_f, _, yl = _median_ms(lambda: rmsnorm_fn(xl, wk, None, zl, eps=1e-5, norm_before_gate=False))
        tl_b, _, _ = _median_ms(lambda: torch.autograd.grad(yl, (xl, zl, wk), dyl, retain_graph=True))
        out.update({"norm_large_rows": rows, "norm_large_fwd_ms": tl_f, "norm_large_bwd_ms": tl_b,
                    "norm_large_fwd_frac": nfl / (tl_f * 1e-3) / 1e9 / hbm, "norm_large_bwd_frac": nbl / (tl_b * 1e-3) / 1e9 / hbm})
        del xl, zl, dyl, yl
    which = max(stages, key=lambda k: stages[k][0])
    t, nbytes, tag = stages[which]
    ach = nbytes / (t * 1e-3) / 1e9
    traffic, traffic_src = None, None
    if (w["H"], w["P"], w["N"]) == (8, 36, 256) and dtype == torch.bfloat16 and kind == "layer":
        traffic = NCU_C3S_TRAFFIC[tag] * (batch * w["L"]) / (16 * 4096)
        traffic_src = NCU_C3S_SOURCE
    p = _lib.IssmParams()
    p.batch, p.seqlen, p.nheads, p.headdim, p.dstate, p.ngroups, p.chunk_size = batch, w["L"], w["H"], w["P"], w["N"], 1, w["Q"]
    p.io_dtype = p.dt_dtype = _lib.dtype_code(dtype)
    p.path = issm_combined._PATHS[path]
    p.dt_max = 1.0
    s = w["H"] * w["P"]
    p.x_sb, p.x_sl, p.x_sh = w["L"] * s, s, w["P"]
    p.out_sb, p.out_sl, p.out_sh = p.x_sb, p.x_sl, p.x_sh
    p.dout_sb, p.dout_sl, p.dout_sh = p.x_sb, p.x_sl, p.x_sh
    p.dt_sb, p.dt_sl, p.dt_sh = w["L"] * w["H"] * w["N"], w["H"] * w["N"], w["N"]
    p.B_sb, p.B_sl, p.B_sg = w["L"] * w["N"], w["N"], w["N"]
    p.C_sb, p.C_sl, p.C_sg = p.B_sb, p.B_sl, p.B_sg
    resolved = {1: "simt", 2: "tensor"}.get(_lib.lib().issm_b200_resolve_path(ct.byref(p)), "?")
    out.update({"bound": "hbm", "kernel": which, "achieved": ach, "peak": hbm, "peak_source": src, "unit": "GB/s",
                "frac": ach / hbm, "traffic": traffic, "traffic_source": traffic_src, "algorithmic_bytes_per_launch": nbytes,
                "ms_per_launch": t, "resolved_path": resolved})
    return out


# ---- CPU arms ---------------------------------------------------------------------------------------------
def _reference_scan():
    """The reference's own pure-PyTorch scan (`ISSM_minimal_discrete`, test_issm.py:18-67), imported unmodified from
    the copy under baseline/_ref when that copy travelled with the tree; None otherwise."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref, "test_issm.py")):
        return None
    if ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        from test_issm import ISSM_minimal_discrete
        return ISSM_minimal_discrete
    except Exception:
        return None


def cpu_sample(w, L_sample, scan):
    """Forward + backward of one scan direction on the CPU, float32, batch 1, the first L_sample points of the
    workload's shape.  `scan` is the reference's ISSM_minimal_discrete (wrapped with the dt transform, D skip and
    gate the reference applies around it: issm_chunk_state.py:84-99, issm_chunk_scan.py:196-210) or, without a
    copy of the reference, the oracle's restatement of it.  Returns seconds."""
    from oracle import issm_oracle as O
    from tests import parity
    inp = O.make_inputs(1, L_sample, w["H"], w["P"], w["N"], seed=0, dtype=torch.float32)
    opts = dict(dt_softplus=True, dt_limit=(1e-3, 1e-1))
    t0 = time.perf_counter()
    if scan is None:
        parity.oracle_run(inp, w["Q"], opts, compute_dtype=torch.float32)
        return time.perf_counter() - t0
    leaves = {k: inp[k].clone().requires_grad_() for k in ("x", "dt", "A", "B", "C", "D", "z", "dt_bias", "initial_states")}
    H, N, Q = w["H"], w["N"], min(w["Q"], L_sample)
    dtv = torch.clamp(O.softplus_ref(leaves["dt"] + leaves["dt_bias"]), 1e-3, 1e-1)
    b, L = 1, L_sample
    y, fin = scan(leaves["x"], dtv, leaves["A"] * dtv, leaves["B"].expand(b, L, H, N), leaves["C"].expand(b, L, H, N), Q,
                  initial_states=leaves["initial_states"])
    y = (y + leaves["x"] * leaves["D"][None, None, :, None]) * torch.nn.functional.silu(leaves["z"])
    ((y * inp["dout"]).sum() + (fin * inp["dfinal"]).sum()).backward()
    return time.perf_counter() - t0


def cpu_baseline(w):
    scan = _reference_scan()
    Ls = min(1024, w["L"]) // w["Q"] * w["Q"] or w["Q"]
    cpu_sample(w, w["Q"], scan)
    t = cpu_sample(w, Ls, scan)
    what = "the reference's ISSM_minimal_discrete (baseline/_ref/test_issm.py)" if scan else "oracle restatement of the reference's pure-PyTorch scan"
    return {"value": Ls * w["N"] / t, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "reference" if scan else "port",
            "sample": f"{what} fwd+bwd, fp32, batch 1, L={Ls}, H={w['H']}, P={w['P']}, N={w['N']}, Q={w['Q']}, "
                      f"one direction, {t:.2f} s; host has {os.cpu_count()} logical cores"}


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path - its only CPU code is the pure-PyTorch
    scan of its test script - on all host threads, on a bounded sample of the same workload per step."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 for multi-process launches; this arm runs on rank 0 alone and is meant to
    # use every host core
    torch.set_num_threads(os.cpu_count() or 1)
    w = WORKLOADS[args.workload]
    scan = _reference_scan()
    Ls = max(w["Q"], min(512, w["L"]) // w["Q"] * w["Q"])
    for _ in range(min(args.warmup, 1)):
        cpu_sample(w, Ls, scan)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_sample(w, Ls, scan)
    t = time.perf_counter() - t0
    value = Ls * w["N"] * args.steps / t
    what = "the reference's ISSM_minimal_discrete (unmodified copy under baseline/_ref)" if scan else "oracle restatement (no copy of the reference on this machine)"
    sample = (f"{what}: fwd+bwd fp32, batch 1, first {Ls} points of the {args.workload} shape (H={w['H']}, P={w['P']}, "
              f"N={w['N']}, Q={w['Q']}), one direction per step")
    kind = "reference" if scan else "port"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": int(os.environ.get("WORLD_SIZE", 1)),
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['desc']}", "sample": sample},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="mine", choices=["mine", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--dtype", default="bf16", choices=sorted(DTYPES))
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "tensor"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--sequence-parallel", action="store_true",
                    help="N > 1: the ranks hold consecutive parts of the same sequences instead of different samples")
    ap.add_argument("--slices", type=int, default=1, help="slices per sequence run as extra batch entries (0 = automatic)")
    ap.add_argument("--graph", action="store_true", help="also time the step replayed from a CUDA graph (one GPU)")
    args = ap.parse_args()
    global SLICES, SEQPAR
    SLICES, SEQPAR = args.slices, args.sequence_parallel
    if args.impl == "reference":
        run_reference(args)
    else:
        run_mine(args)


if __name__ == "__main__":
    main()
