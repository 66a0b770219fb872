"""Benchmark of the ISSM scan hot path: fused forward+backward, bidirectional, bf16 activations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c3|c1|c0]

Prints ONE JSON line (rank 0).  A "step" is one bidirectional ISSM layer forward+backward over one
batch of seeded synthetic inputs (forward scan + reversed scan per sample, both with D skip,
in-kernel softplus(dt + bias) clamp, silu(z) gate, initial states, final states and their
gradients), followed - on more than one GPU - by the single all-reduce of the packed per-head
parameter gradients.  metric = batch * seqlen * dstate / time (points x states per second, whole
job); each point-state is visited by two scan directions.
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

torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False) if hasattr(torch.autograd.graph, 'set_warn_on_accumulate_grad_stream_mismatch') else None

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (per-GPU batch at N=1, global batch at N>1, L, H, P, N, Q)
    "c3": dict(batch1=16, global_multi=64, L=40000, H=8, P=36, N=256, Q=256,
               desc="large-scene ISSM fwd+bwd, bidirectional (b16 at 1 GPU; global b64 at 2/4/8 GPUs)"),
    "c3s": dict(batch1=16, global_multi=64, L=4096, H=8, P=36, N=256, Q=256,
                desc="c3 with a 10x shorter sequence: the small case used for profiler captures"),
    "c1": dict(batch1=8, global_multi=64, L=1024, H=8, P=36, N=256, Q=256, desc="DEST decoder layer size"),
    "c0": dict(batch1=2, global_multi=2, L=1024, H=8, P=36, N=256, Q=256, desc="CPU-runnable reference case"),
}
METRIC, UNIT = "issm_fwd_bwd_points_states_per_s", "points*states/s"


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def algorithmic_bytes(b, L, H, P, N, e=2, dirs=2):
    """Each input read once, each output written once (e = activation element size), per direction:
    fwd  dt + (x, z, out) + (B, C) + initial/final states;  bwd  (dt, ddt) + (x, z, out_x, dout, dx, dz)
    + (B, C, dB, dC) + state gradients."""
    fwd = L * H * N * e + 3 * L * H * P * e + 2 * L * N * e + H * P * N * (e + 4)
    bwd = 2 * L * H * N * e + 6 * L * H * P * e + 4 * L * N * e + H * P * N * (2 * e + 4)
    return b * dirs * fwd, b * dirs * bwd


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


def make_batch(w, batch, sample0, device=None, pin=False):
    """Seeded synthetic inputs of the benchmark's distributions for samples [sample0, sample0+batch):
    x, z ~ N(0,1); B, C ~ N(0,1)/sqrt(N); dt_raw ~ N(0,1) with bias -4 (softplus, clamp [1e-3, 1e-1]);
    A = -exp(U(log 1, log 16)) per head; D ~ N(0,1); initial states ~ N(0,1)/16; dout ~ N(0,1).
    Per-sample seeds, so any GPU count reproduces the same global batch."""
    L, H, P, N = w["L"], w["H"], w["P"], w["N"]
    bf = torch.bfloat16
    names = dict(x_f=(L, H, P), x_b=(L, H, P), z=(L, H, P), B_f=(L, 1, N), C_f=(L, 1, N), B_b=(L, 1, N), C_b=(L, 1, N),
                 dt=(L, H, N), init=(H, P, N), dout=(L, H, P))
    host = {k: torch.empty((batch,) + s, dtype=bf, pin_memory=pin) for k, s in names.items()}
    for i in range(batch):
        g = torch.Generator().manual_seed(1000 + sample0 + i)
        for k, s in names.items():
            t = torch.randn(s, generator=g)
            if k[0] in "BC":
                t /= math.sqrt(N)
            if k == "init":
                t /= 16.0
            host[k][i] = t.to(bf)
    g = torch.Generator().manual_seed(7)
    A = (-torch.exp(torch.rand(H, generator=g) * math.log(16.0)))[:, None].repeat(1, N).contiguous()
    par = dict(A=A, D=torch.randn(H, generator=g), dt_bias=torch.full((H, N), -4.0))
    dfinal = torch.randn(batch, H, P, N, generator=torch.Generator().manual_seed(11 + sample0)) / 16.0
    return host, par, dfinal


_SIDE = {}


def layer_step(dev, par, dfinal, w, path):
    """One bidirectional ISSM layer forward+backward through the public interface.  The two scan
    directions are independent, so they are enqueued on two CUDA streams (autograd runs each scan's
    backward on the stream of its forward): with few samples per GPU one direction alone does not
    fill the 148 SMs (one CTA per (sample, head))."""
    from dest3d_b200 import ISSM_chunk_scan_combined
    main = torch.cuda.current_stream()
    key = torch.cuda.current_device()
    if key not in _SIDE:
        _SIDE[key] = (torch.cuda.Stream(), torch.cuda.Stream())
    s1, s2 = _SIDE[key]
    leaves = {k: v.detach().requires_grad_() for k, v in dev.items() if k not in ("dout",)}
    P_ = {k: v.detach().requires_grad_() for k, v in par.items()}
    kw = dict(D=P_["D"], z=leaves["z"], dt_bias=P_["dt_bias"], initial_states=leaves["init"], dt_softplus=True,
              dt_limit=(1e-3, 1e-1), return_final_states=True, path=path)
    s1.wait_stream(main)
    s2.wait_stream(main)
    with torch.cuda.stream(s1):
        yf, sf = ISSM_chunk_scan_combined(leaves["x_f"], leaves["dt"], P_["A"], leaves["B_f"], leaves["C_f"], w["Q"], **kw)
    with torch.cuda.stream(s2):
        yb, sb = ISSM_chunk_scan_combined(leaves["x_b"], leaves["dt"], P_["A"], leaves["B_b"], leaves["C_b"], w["Q"],
                                          reverse=True, **kw)
    main.wait_stream(s1)
    main.wait_stream(s2)
    for t in (yf, sf, yb, sb):
        t.record_stream(main)
    out = (yf + yb) * 0.5                       # the reference's combine (models/dest_module.py:574)
    fin = (sf + sb) * 0.5
    torch.autograd.backward([out, fin], [dev["dout"], dfinal])
    main.wait_stream(s1)
    main.wait_stream(s2)
    return out, fin, {"dA": P_["A"].grad, "ddt_bias": P_["dt_bias"].grad, "dD": P_["D"].grad}


def run_mine(args):
    from dest3d_b200 import _lib
    from dest3d_b200.dist import PackedParamGrads, max_over_ranks, shard_samples
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    w = WORKLOADS[args.workload]
    gbatch = w["batch1"] if world == 1 else w["global_multi"]
    mine = shard_samples(gbatch, world, rank)
    batch = len(mine)
    host, par, dfinal = make_batch(w, batch, mine.start, pin=True)
    dev = {k: v.to(device, non_blocking=True) for k, v in host.items()}
    par = {k: v.to(device) for k, v in par.items()}
    dfinal = dfinal.to(device)
    packed = PackedParamGrads({"dA": par["A"].shape, "ddt_bias": par["dt_bias"].shape, "dD": par["D"].shape}, device)
    path = args.path

    def step(inputs=None):
        out, fin, grads = layer_step(inputs if inputs is not None else dev, par, dfinal, w, path)
        packed.load(grads).all_reduce()
        return out, fin

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()
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
    L, H, P, N = w["L"], w["H"], w["P"], w["N"]
    value = gbatch * L * N * args.steps / (ms * 1e-3)

    # end to end through the public call with HOST buffers: H2D of the step's inputs from pinned memory,
    # the layer, D2H of the combined output, final states and packed parameter gradients.  The steps are
    # pipelined the way a training loop with a prefetching loader runs them: the H2D copy of step i+1 (copy
    # stream, second set of device buffers) overlaps the layer of step i.  Every step's inputs are copied and
    # every step's results are read back inside the timed region; the first copy is not overlapped.
    out_h = torch.empty((batch, L, H, P), dtype=torch.bfloat16, pin_memory=True)
    fin_h = torch.empty((batch, H, P, N), dtype=torch.float32, pin_memory=True)
    pg_h = torch.empty(packed.flat.shape, dtype=torch.float32, pin_memory=True)
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_h.numel() * 2 + fin_h.numel() * 4 + pg_h.numel() * 4

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
            pg_h.copy_(packed.flat, non_blocking=True)

    e2e_steps = max(2, min(args.steps, 6))
    e2e_run(2)
    sync_all()
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    sync_all()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1), device)
    e2e_value = gbatch * L * N * e2e_steps / (ms_e2e * 1e-3)

    # roofline of the dominant kernel, timed live with CUDA events on the launching stream
    roof, cpu = None, None
    if rank == 0:
        roof = kernel_roofline(dev, par, dfinal, w, batch, path)
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(w)
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak" if world == 1 else "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"{args.workload}: {w['desc']}", "global_batch": gbatch, "per_gpu_batch": batch,
                           "seqlen": L, "nheads": H, "headdim": P, "dstate": N, "chunk_size": w["Q"], "directions": 2,
                           "path": path, "l2": "inputs larger than L2 (no flush needed)",
                           "parallelism": f"dp{world} by sample, both directions on one GPU"},
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps,
                        "pipelining": "H2D of step i+1 overlaps the layer of step i (two device buffer sets)"},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch on the small profiling case c3s
# (batch 16, L = 4096), from the ncu captures summarised in profiles/; traffic grows in proportion to batch x L
NCU_C3S_TRAFFIC = {"fwd": 413.5e6 + 248.0e6, "bwd": 698.5e6 + 839.5e6}


def kernel_roofline(dev, par, dfinal, w, batch, path):
    """Time the forward call and the backward call of one direction separately (CUDA events on
    the current stream); report the roofline of the slower one's main kernel."""
    from dest3d_b200 import issm_bwd, issm_fwd
    hbm, src = peaks()
    kw = dict(D=par["D"], z=dev["z"], dt_bias=par["dt_bias"], initial_states=dev["init"], dt_softplus=True,
              dt_limit=(1e-3, 1e-1), path=path)
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    warm, reps, tfs, tbs = 2, 5, [], []
    for i in range(warm + reps):
        e[0].record()
        out, out_x, fin, saved = issm_fwd(dev["x_f"], dev["dt"], par["A"], dev["B_f"], dev["C_f"], w["Q"],
                                          save_states=True, **kw)
        e[1].record()
        issm_bwd(dev["dout"], dev["x_f"], dev["dt"], par["A"], dev["B_f"], dev["C_f"], out_x, w["Q"],
                 dfinal_states=dfinal, saved_states=saved, **kw)
        e[2].record()
        torch.cuda.synchronize()
        if i >= warm:
            tfs.append(e[0].elapsed_time(e[1]))
            tbs.append(e[1].elapsed_time(e[2]))
    # median of the repetitions: a call that has to grow the caching allocator's pool is not a kernel time
    tf, tb = sorted(tfs)[reps // 2], sorted(tbs)[reps // 2]
    fb, bb = algorithmic_bytes(batch, w["L"], w["H"], w["P"], w["N"], dirs=1)
    which, t, nbytes = (("forward call (k_fwd_tensor)", tf, fb) if tf >= tb else
                        ("backward call (k_bwd_tensor + head/batch reductions)", tb, bb))
    ach = nbytes / (t * 1e-3) / 1e9
    traffic = None
    if (w["H"], w["P"], w["N"]) == (8, 36, 256):
        traffic = NCU_C3S_TRAFFIC["fwd" if tf >= tb else "bwd"] * (batch * w["L"]) / (16 * 4096)
    return {"bound": "hbm", "kernel": which, "achieved": ach, "peak": hbm, "peak_source": src, "unit": "GB/s",
            "frac": ach / hbm, "traffic": traffic, "algorithmic_bytes_per_launch": nbytes, "ms_per_launch": t,
            "fwd_ms_one_direction": tf, "bwd_ms_one_direction": tb, "fwd_ms_reps": [round(t, 3) for t in tfs], "bwd_ms_reps": [round(t, 3) for t in tbs],
            "fwd_frac": fb / (tf * 1e-3) / 1e9 / hbm, "bwd_frac": bb / (tb * 1e-3) / 1e9 / hbm}


def oracle_sample(w, L_sample):
    """The CPU oracle (a restatement of the reference's pure-PyTorch scan) forward+backward on a
    bounded sample of the workload: batch 1, the first L_sample points, one direction, float32."""
    from oracle import issm_oracle as O
    from tests import parity
    inp = O.make_inputs(1, L_sample, w["H"], w["P"], w["N"], seed=0, dtype=torch.float32)
    opts = dict(dt_softplus=True, dt_limit=(1e-3, 1e-1))
    t0 = time.perf_counter()
    parity.oracle_run(inp, w["Q"], opts, compute_dtype=torch.float32)
    return time.perf_counter() - t0


def cpu_baseline(w):
    Ls = min(1024, w["L"])
    oracle_sample(w, 256)
    t = oracle_sample(w, Ls)
    return {"value": Ls * w["N"] / t, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"oracle (reference's pure-PyTorch chunked scan restated) fwd+bwd, fp32, batch 1, L={Ls}, "
                      f"H={w['H']}, P={w['P']}, N={w['N']}, Q={w['Q']}, one direction, {t:.2f} s; "
                      f"host has {os.cpu_count()} logical cores"}


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path.  Its only CPU code is the
    pure-PyTorch scan in its test script, which the oracle restates (the GPU box has no copy of the
    reference tree), timed with all host threads on a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 for multi-process launches; this arm runs on rank 0 alone and is meant to
    # use every host core
    torch.set_num_threads(os.cpu_count() or 1)
    w = WORKLOADS[args.workload]
    Ls = min(512, w["L"])
    for _ in range(min(args.warmup, 1)):
        oracle_sample(w, Ls)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle_sample(w, Ls)
    t = time.perf_counter() - t0
    value = Ls * w["N"] * args.steps / t
    sample = (f"oracle fwd+bwd fp32, batch 1, first {Ls} points of the {args.workload} shape (H={w['H']}, P={w['P']}, "
              f"N={w['N']}, Q={w['Q']}), one direction per step")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": int(os.environ.get("WORLD_SIZE", 1)),
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['desc']}", "sample": sample},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="mine", choices=["mine", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "tensor"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_mine(args)


if __name__ == "__main__":
    main()
