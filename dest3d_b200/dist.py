"""Data-parallel sharding of the ISSM scan: one process per GPU, (sample x direction) units.

A scan is independent per (sample, direction); both directions of a sample stay on one rank so the
bidirectional combine (models/dest_module.py:574-575) is local and dt is read from one copy.  The
only exchange is ONE all-reduce of the packed per-head parameter gradients
[dA (H*N) | ddt_bias (H*N) | dD (H or H*P) | dW_norm (hidden)] - about 17.6 KB for the detector's
sizes.  The reference has no multi-GPU code at all; this module is new.
"""
import torch
import torch.distributed as dist


def shard_samples(global_batch, world_size, rank):
    """Contiguous block of sample indices owned by `rank`; the first (global_batch % world_size)
    ranks take one extra sample.  Returns range(start, stop)."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank / world_size")
    base, extra = divmod(global_batch, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


class PackedParamGrads:
    """Flat float32 buffer holding every parameter gradient of one ISSM layer, so that a single
    all-reduce covers them all.  `views` are zero-copy windows with the parameters' shapes."""

    def __init__(self, shapes, device):
        self.names = list(shapes.keys())
        self.shapes = {k: tuple(v) for k, v in shapes.items()}
        sizes = [int(torch.Size(self.shapes[k]).numel()) for k in self.names]
        self.flat = torch.zeros(sum(sizes), dtype=torch.float32, device=device)
        self.views, off = {}, 0
        for k, n in zip(self.names, sizes):
            self.views[k] = self.flat[off:off + n].view(self.shapes[k])
            off += n

    def load(self, grads):
        """Copy (and cast to float32) the given gradients into the flat buffer; missing names are zeroed.
        All present gradients go in ONE multi-tensor copy launch."""
        dst, src, absent = [], [], []
        for k in self.names:
            g = grads.get(k)
            if g is None:
                absent.append(self.views[k])
            else:
                dst.append(self.views[k])
                src.append(g.detach().reshape(self.shapes[k]))
        if absent:
            torch._foreach_zero_(absent)
        if dst:
            torch._foreach_copy_(dst, src)
        return self

    def all_reduce(self, group=None, average=False):
        """Sum (or average) over ranks with ONE collective; no-op without an initialised group."""
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
            if average:
                self.flat.div_(dist.get_world_size(group))
        return self


def max_over_ranks(value, device):
    """Max of a python float over all ranks (used for device-timed step durations)."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bind_to_gpu_numa_node(device_index):
    """Restrict this process to the CPUs NVML reports as local to the GPU, so that host memory pinned afterwards
    (first touch by this thread) lies on the GPU's NUMA node.  Returns the number of CPUs bound to, or 0 when NVML,
    the affinity query or an overlap with the CPUs this process may use is missing (nothing is changed then)."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
    except Exception:
        return 0
    local = {64 * i + bit for i, word in enumerate(words) for bit in range(64) if (int(word) >> bit) & 1}
    usable = local & os.sched_getaffinity(0)
    if not usable:
        return 0
    os.sched_setaffinity(0, usable)
    return len(usable)
