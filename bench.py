#!/usr/bin/env python
"""fwd+bwd lattice-nodes/sec of the compact RNN-T loss on B200, with its HBM roofline and the host-CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--cfg 2]

A step is one pass of the hot path over one synthetic batch: forward (row offsets, fused log-softmax + gather,
alpha/beta wavefront, costs, loss) and backward (dense gradient w.r.t. the logits), called through the C ABI.

N = 1: the Conformer-shape workload (B=32, T~U[150,250], U~U[20,80], V=1024, float32 logits), 1.3 GB of logits, larger
than the 126 MB L2, so every step streams from HBM. N > 1 (launched by torch.distributed.run, one rank per GPU): weak
scaling - the global batch is 32*N sequences of the same distribution, sharded by lattice size; the only collective
is the all-reduce of the [B_global+1] cost vector.

One JSON line comes out of rank 0:
  value / ms_per_step   lattice nodes of all ranks / max-over-ranks device time, inputs resident in HBM. The timed
                        region is `--repeats` blocks of exactly K steps, each block between barrier + synchronise and
                        two CUDA events; the MEDIAN block is reported, with the fastest and slowest beside it.
  e2e                   the same metric through the host-buffer entry point (pinned host logits in, host gradients out,
                        PCIe copies inside the timed region), with each direction's bandwidth alone per rank.
  roofline              the gradient kernel (the dominant launch) against the measured copy bandwidth.
  cpu_baseline          the CPU checker (oracle/) timed on a bounded sample of the same workload; its costs also give
                        `loss_check` (the run exits non-zero when the device loss is more than 1e-5 off).
  python_api            the step through `cwarp_rnnt.transducer_loss(..., fused_log_softmax=True)` + `.backward()`.
  configs               the other benchmark workloads (1, 3, 4, 5), device-timed the same way, with the recursion's
                        latency per lattice diagonal.
  strong_cfg5           the ragged workload (B = 256 fixed) sharded over the N ranks: strong scaling.
`--impl reference` times the path's CPU implementation alone (the reference project has no CPU path of its own: its
three source files are CUDA only).
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

import torch  # noqa: E402

from compactwarprnntloss_b200 import synth  # noqa: E402

METRIC = "fwd+bwd lattice-nodes/sec"
UNIT = "nodes/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the gradient kernel, per lattice node, from the ncu
# captures summarised under profiles/ (the algorithmic figure is 2 * V * sizeof(element)); a run scales it by its rows.
GRAD_KERNEL_DRAM_BYTES_PER_NODE = {2: (8047.0, "profiles/grad_rows_kernel_conformer_v1024.md")}
DTYPE_NAME = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=21, help="timed blocks of --steps steps; the median block is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_cuda"],
                    help="ours: this engine; reference: the path's CPU implementation on the host cores; "
                         "reference_cuda: the reference project's own CUDA kernels rebuilt for sm_100a (oracle/_ref)")
    ap.add_argument("--cfg", type=int, default=2, help="workload (1-5); the headline metric is quoted on 2")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: B*N sequences over N GPUs (default); strong: the workload's B sequences sharded over N")
    ap.add_argument("--groups", type=int, default=0,
                    help="sequence groups of the pipelined step (0 = chosen by the library, 1 = no overlap)")
    ap.add_argument("--order", default="pipeline", choices=["longest_first", "pipeline", "ascending"],
                    help="row order of a rank's sequences (sharding.plan_shards)")
    ap.add_argument("--sequences", type=int, default=0,
                    help="use only the first N sequences of the workload (0 = all): a smaller case of the same "
                         "kernels for a profiler capture, not a benchmark configuration")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the other workloads (N = 1 only)")
    ap.add_argument("--no-python-api", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="skip the ragged strong-scaling block")
    ap.add_argument("--cpu-sample-seqs", type=int, default=32,
                    help="sequences of the workload the CPU baseline runs per repetition")
    return ap.parse_args()


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, polled through NVML (read-only queries) from a thread every
    few milliseconds while the timed region runs; falls back to `nvidia-smi -lms` when NVML is unavailable."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device_index, period_s=0.003):
        self.rows, self.stop_flag, self.mode, self.proc = [], False, None, None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.mode = "nvml"
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self._start_smi(device_index)

    def _poll(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                sm = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    why = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    why = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                pw = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                self.rows.append((float(sm), int(why), pw))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def _start_smi(self, device_index):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            sel = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            self.proc = subprocess.Popen(["nvidia-smi", "-i", sel, "--query-gpu=" + q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.mode = "smi"
            self.thread = threading.Thread(target=self._read_smi, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self.mode = None

    def _read_smi(self):
        names = [0x8, 0x40, 0x20, 0x4]
        for line in self.proc.stdout:
            c = [v.strip() for v in line.split(",")]
            if len(c) >= 7 and c[0].replace(".", "").isdigit():
                why = sum(bit for i, bit in enumerate(names) if c[3 + i].lower().startswith("active"))
                self.sm_max = float(c[1])
                self.rows.append((float(c[0]), why, float(c[2]) if c[2].replace(".", "").isdigit() else 0.0))

    def mark(self):
        return len(self.rows)

    def stop(self, start=0):
        if self.mode is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML and no nvidia-smi"]}
        if self.mode == "smi":
            time.sleep(0.12)
            self.proc.terminate()
        self.stop_flag = True
        rows = self.rows[start:] or self.rows[-1:]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        why = 0
        for r in rows:
            why |= r[1]
        return {"sm_mhz": statistics.median(r[0] for r in rows), "sm_max_mhz": self.sm_max,
                "power_w_max": max(r[2] for r in rows), "samples": len(rows), "source": self.mode,
                "reasons": [n for bit, n in self.REASONS.items() if why & bit]}


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def workload_config(cfg, world, scaling, order, sequences=0):
    """The `config` object of the JSON line, from the lengths alone - the same for this engine's arm and for the CPU
    reference arm, so that the two lines name one workload."""
    from compactwarprnntloss_b200 import sharding
    wl = synth.WORKLOADS[cfg]
    B_global = (sequences or wl.B) * (world if scaling == "weak" else 1)
    lx, ly, _ = synth.lengths_and_labels(cfg, B=B_global)
    plan = sharding.plan_shards(lx.tolist(), ly.tolist(), world, order=order)
    elt = torch.empty((), dtype=wl.dtype).element_size()
    per_gpu = int(synth.lattice_nodes(lx, ly, plan[0]) * wl.V * elt)
    return {"workload": wl.name, "global_sequences": B_global, "lattice_nodes": synth.lattice_nodes(lx, ly),
            "logits_bytes_per_gpu": per_gpu,
            "sharding": f"lattice-size LPT over {world} rank(s)", "row_order": order,
            "l2": "inputs larger than L2 (no flush needed)" if per_gpu > (126 << 20) else
                  "inputs fit in L2 and are not flushed: a launch-bound, correctness-sized workload",
            "reduction": wl.reduction,
            "shard_imbalance": round(sharding.shard_imbalance(lx, ly, plan), 4)}


def cpu_reference_time(cfg, lx, ly, y, n_seqs, budget_s=12.0):
    """The CPU checker's fused float32 pipeline (all host threads) on the first n_seqs sequences, repeated until
    about budget_s seconds of wall time are spent; nodes/s of the best repetition, and the costs it computed."""
    from oracle import oracle
    oracle.build()
    oracle.set_num_threads(host_threads())
    import numpy as np
    ids = list(range(min(n_seqs, len(lx))))
    x = synth.compact_logits(cfg, lx, ly, ids).float().numpy()
    lxs, lys, ys = lx[ids].numpy(), ly[ids].numpy(), y[ids].numpy()
    out = np.empty_like(x)
    w = np.full(len(ids), 1.0 / len(lx))
    oracle.fused_f32io(x[: int(lxs[0]) * (int(lys[0]) + 1)], lxs[:1], lys[:1], ys[:1], 0)  # touch the library
    times, costs = [], None
    while sum(times) < budget_s and len(times) < 200:
        t0 = time.perf_counter()
        costs, _ = oracle.fused_f32io(x, lxs, lys, ys, 0, weights=w, dense_out=out)
        times.append(time.perf_counter() - t0)
    nodes = x.shape[0]
    return nodes / min(times), oracle.num_threads(), nodes, sum(times), len(times), costs


def run_reference(args):
    """--impl reference: the path's CPU implementation on the box's host cores. The reference project itself is CUDA
    only, so this is the CPU checker (oracle/rnnt_oracle.c, OpenMP over rows and sequences)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = args.cfg
    world = int(os.environ.get("WORLD_SIZE", "1"))
    lx, ly, y = synth.lengths_and_labels(cfg)
    n_seqs = args.cpu_sample_seqs
    from oracle import oracle
    oracle.build()
    oracle.set_num_threads(host_threads())  # torch.distributed.run exports OMP_NUM_THREADS=1: use the cores anyway
    import numpy as np
    ids = list(range(min(n_seqs, len(lx))))
    x = synth.compact_logits(cfg, lx, ly, ids).float().numpy()
    lxs, lys, ys = lx[ids].numpy(), ly[ids].numpy(), y[ids].numpy()
    out = np.empty_like(x)
    w = np.full(len(ids), 1.0 / len(lx))
    for _ in range(max(args.warmup, 1)):
        oracle.fused_f32io(x[: int(lxs[0]) * (int(lys[0]) + 1)], lxs[:1], lys[:1], ys[:1], 0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.fused_f32io(x, lxs, lys, ys, 0, weights=w, dense_out=out)
    dt = time.perf_counter() - t0
    nodes = x.shape[0]
    value = nodes * args.steps / dt
    wl = synth.WORKLOADS[cfg]
    sample = f"first {len(ids)} of {wl.B} sequences of the workload ({nodes} lattice nodes) per step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": DTYPE_NAME[wl.dtype], "data": "synthetic",
        "config": workload_config(cfg, world, args.scaling, args.order, args.sequences),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_reference_cuda(args):
    """The reference's own pipeline on one GPU: torch.log_softmax -> its _cwarp_rnnt_forward -> its
    _cwarp_rnnt_backward -> log_softmax backward, float32, device-resident inputs, CUDA events. Extra comparator
    (not the CPU reference arm); needs oracle/_ref/cwarp_rnnt_ref_C.so, built by oracle/build_ref.py."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle.build_ref import load_ref
    ref = load_ref()
    if ref is None or not torch.cuda.is_available():
        print(json.dumps({"impl": "reference_cuda", "unavailable": "oracle/_ref/cwarp_rnnt_ref_C.so not built or no GPU"}))
        return
    cfg = args.cfg
    wl = synth.WORKLOADS[cfg]
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    lx, ly, y = synth.lengths_and_labels(cfg)
    x = synth.compact_logits(cfg, lx, ly).float().to(dev).requires_grad_(True)
    lxd, lyd, yd = lx.to(dev), ly.to(dev), y.to(dev).contiguous()
    gc = torch.full((len(lx),), 1.0 / len(lx), device=dev)
    nodes = x.shape[0]

    def step():
        x.grad = None
        lp = torch.log_softmax(x, -1)
        costs, grads, _, _ = ref._cwarp_rnnt_forward(lp, lxd, yd, lyd, 0)
        dense = ref._cwarp_rnnt_backward(grads, gc, yd, lxd, lyd, 0, wl.V)
        lp.backward(dense)
        return costs

    for _ in range(max(args.warmup, 3)):
        costs = step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        costs = step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({
        "impl": "reference_cuda", "metric": METRIC, "value": nodes / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "dtype": "f32", "data": "synthetic", "loss": float(costs.mean()),
        "config": {"workload": wl.name, "lattice_nodes": nodes,
                   "pipeline": "torch.log_softmax + reference _cwarp_rnnt_forward/_backward (sm_100a rebuild of its "
                               "unmodified sources) + log_softmax backward"}}))


# ------------------------------------------------------------------------------------------------ this engine's arm

def device_logits(cfg, lx, ly, ids, dev):
    """Compact logits of the listed sequences drawn ON the device (a CUDA generator seeded per sequence with
    1000*cfg + 1 + i, N(0, sigma) in float32, then cast): the same shapes and distribution as synth.compact_logits
    without the minutes a host generator takes for several GB. Used for the workloads that are timed only."""
    wl = synth.WORKLOADS[cfg]
    rows = [int(lx[i]) * (int(ly[i]) + 1) for i in ids]
    x = torch.empty(sum(rows), wl.V, dtype=wl.dtype, device=dev)
    g = torch.Generator(device=dev)
    at = 0
    for i, r in zip(ids, rows):
        g.manual_seed(1000 * cfg + 1 + i)
        if wl.dtype == torch.float32:
            x[at:at + r].normal_(0.0, wl.sigma, generator=g)
        else:
            x[at:at + r].copy_(torch.empty(r, wl.V, dtype=torch.float32, device=dev).normal_(0.0, wl.sigma, generator=g))
        at += r
    return x


class Job:
    """One rank's share of a workload, resident on the device, with everything a step needs."""

    def __init__(self, cfg, lx, ly, y, ids, B_global, dev, x, world, groups):
        from compactwarprnntloss_b200 import capi
        self.capi, self.cfg, self.dev, self.world, self.groups = capi, cfg, dev, world, groups
        wl = synth.WORKLOADS[cfg]
        self.wl, self.ids, self.B_global = wl, ids, B_global
        self.x = x
        self.lx, self.ly = lx[ids].contiguous().to(dev), ly[ids].contiguous().to(dev)
        self.y = y[ids].contiguous().to(dev)
        self.flags = capi.FUSED_LOG_SOFTMAX | (capi.REDUCE_MEAN if wl.reduction == "mean" else capi.REDUCE_SUM)
        self.p = capi.make_problem(x, self.lx, self.y, 0, self.flags, mean_denominator=B_global)
        self.ws = capi.alloc_workspace(self.p, dev)
        ct = capi.cost_dtype(x.dtype)
        self.costs = torch.empty(self.p.B, dtype=ct, device=dev)
        self.loss = torch.zeros((), dtype=ct, device=dev)
        self.gx = torch.empty_like(x)
        self.one = torch.ones(1, dtype=ct, device=dev)
        self.vec = torch.empty(B_global + 1, dtype=ct, device=dev)
        self.ids_dev = torch.tensor(ids, dtype=torch.int32, device=dev)
        self.pipe = capi.Pipe(dev)
        self.n_groups = capi.pipeline_groups(self.p, groups)
        self.launches = 1 + 3 * self.n_groups
        self.nodes = x.shape[0]
        self.elt = x.element_size()
        self.longest = max((int(lx[i]) + int(ly[i]) for i in ids), default=0)
        self.main, self.comm = torch.cuda.current_stream(dev), torch.cuda.Stream(dev)

    def step(self):
        """One pipelined call: K0, then per sequence group gather -> wavefront (side stream) -> gradient. Sharded:
        the wavefront epilogue fills the global cost vector; one all-reduce is the whole exchange and it runs on a
        second stream as soon as the wavefronts are done, underneath the gradient kernels."""
        capi = self.capi
        if self.world == 1:
            capi.loss_grad(self.p, self.x, self.lx, self.ly, self.y, self.ws, self.costs, self.loss, self.one, 0,
                           self.gx, pipe=self.pipe, groups=self.groups)
        else:
            import torch.distributed as dist
            capi.loss_grad(self.p, self.x, self.lx, self.ly, self.y, self.ws, self.costs, self.loss, self.one, 0,
                           self.gx, pipe=self.pipe, groups=self.groups, global_ids=self.ids_dev,
                           n_global=self.B_global, cost_vector=self.vec)
            with torch.cuda.stream(self.comm):
                self.pipe.wait_costs(self.comm)
                dist.all_reduce(self.vec, op=dist.ReduceOp.SUM)
            self.main.wait_stream(self.comm)

    def forward(self):
        self.capi.forward(self.p, self.x, self.lx, self.ly, self.y, self.ws, self.costs, self.loss)

    def backward(self):
        self.capi.backward(self.p, self.x, self.lx, self.ly, self.y, self.ws, self.one, 0, self.gx)

    def recursion(self):
        self.capi.recursion(self.p, self.lx, self.ly, self.ws, self.costs, self.loss)

    def loss_value(self):
        return float(self.vec[self.B_global] if self.world > 1 else self.loss)

    def close(self):
        self.pipe.close()


def make_fence(world, dev):
    def fence():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize(dev)
    return fence


def max_over_ranks(values, world, dev):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.cpu()]


def timed_blocks(step, K, repeats, fence, world, dev):
    """`repeats` blocks of exactly K steps; a block is bracketed by barrier + synchronise on both sides and timed with
    CUDA events on the launching stream. Returns the per-block milliseconds, each the max over ranks."""
    ms = []
    for _ in range(repeats):
        b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fence()
        b.record()
        for _k in range(K):
            step()
        e.record()
        fence()
        ms.append(b.elapsed_time(e))
    return max_over_ranks(ms, world, dev)


def per_call_ms(fn, n, dev, before=None):
    """Median, min and max over n calls of fn, each between its own pair of CUDA events."""
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for a, b in ev:
        if before is not None:
            before()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize(dev)
    t = [a.elapsed_time(b) for a, b in ev]
    return statistics.median(t), min(t), max(t)


def spread(ms_blocks, K):
    return {"median": statistics.median(ms_blocks) / K, "min": min(ms_blocks) / K, "max": max(ms_blocks) / K,
            "blocks": len(ms_blocks), "steps_per_block": K}


def measure_job(job, K, repeats, fence, peak, want_breakdown=True):
    """Device-timed figures of one workload on this rank's share: the pipelined step, the same work as two plain
    calls, the gradient kernel alone, the recursion alone (latency per diagonal)."""
    for _ in range(3):
        job.step()
    fence()
    st = job.capi.read_status(job.ws)
    if st[0] & 0x3:
        raise SystemExit(f"device status reports invalid inputs: {st}")
    blocks = timed_blocks(job.step, K, repeats, fence, job.world, job.dev)
    loss = job.loss_value()
    out = {"blocks_ms": blocks, "loss": loss}
    if want_breakdown:
        job.forward()
        fwd = per_call_ms(job.forward, K, job.dev)
        bwd = per_call_ms(job.backward, K, job.dev)
        k2 = per_call_ms(job.recursion, K, job.dev)
        out.update(fwd=fwd, bwd=bwd, k2=k2)
    return out


def config_block(job, m, K, peak, peak_kind):
    """JSON object of one extra workload (configs[...] / strong_cfg5) from measure_job's figures."""
    wl = job.wl
    sp = spread(m["blocks_ms"], K)
    ms = sp["median"]
    step_gbs = 3.0 * job.nodes * wl.V * job.elt / (ms * 1e-3) / 1e9
    out = {"workload": wl.name, "dtype": DTYPE_NAME[wl.dtype], "lattice_nodes": job.nodes,
           "logits_bytes": int(job.nodes * wl.V * job.elt), "sequence_groups": job.n_groups,
           "gpu_launches_per_step": job.launches,
           "ms_per_step": ms, "ms_per_step_min": sp["min"], "ms_per_step_max": sp["max"], "steps": K,
           "blocks": sp["blocks"], "value": job.nodes / (ms * 1e-3), "unit": UNIT,
           "step_roofline": {"achieved": step_gbs, "peak": peak, "unit": "GB/s", "frac": step_gbs / peak,
                             "peak_kind": f"of {peak_kind}", "bytes_per_node": 3 * wl.V * job.elt},
           "loss": m["loss"]}
    if "bwd" in m:
        grad_gbs = 2.0 * job.nodes * wl.V * job.elt / (m["bwd"][0] * 1e-3) / 1e9
        out.update({
            "unpipelined_ms_per_step": m["fwd"][0] + m["bwd"][0],
            "grad_kernel": {"launch_ms": m["bwd"][0], "achieved": grad_gbs, "frac": grad_gbs / peak, "unit": "GB/s"},
            "recursion": {"kernel_ms": m["k2"][0], "longest_diagonals": job.longest,
                          "us_per_diagonal": m["k2"][0] * 1e3 / max(job.longest, 1),
                          "what": "cwrnnt_recursion alone (alpha and beta of every sequence in one launch) / longest "
                                  "T+U of the batch"}})
    return out


def python_api_ms(job, K, repeats, fence):
    """The metric as the reference's user measures it: one `transducer_loss(...)` + `.backward()` per step through the
    Python entry point, CUDA events around blocks of K steps, median block; with and without the input check."""
    import cwarp_rnnt
    x = job.x.detach().requires_grad_(True)
    out = {}
    for name, check in (("check_true_ms", True), ("check_false_ms", False)):
        def step():
            x.grad = None
            loss = cwarp_rnnt.transducer_loss(x, job.lx, job.y, job.ly, 0, job.wl.reduction, fused_log_softmax=True,
                                              check=check)
            loss.backward()
            return loss
        for _ in range(3):
            loss = step()
        blocks = timed_blocks(step, K, repeats, fence, 1, job.dev)
        out[name] = statistics.median(blocks) / K
        out[name.replace("_ms", "_min_ms")] = min(blocks) / K
        out[name.replace("_ms", "_max_ms")] = max(blocks) / K
        out["loss"] = float(loss)
    x.grad = None
    out["what"] = ("cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, reduction, fused_log_softmax=True) + loss.backward(), "
                   f"median of {repeats} blocks of {K} steps (CUDA events)")
    return out


def numa_of(ptr):
    """NUMA placement of the mapping that holds `ptr`, from /proc/self/numa_maps ({'N0': pages, ...}); None when the
    kernel does not show it."""
    try:
        best, where = -1, None
        with open("/proc/self/numa_maps") as f:
            for line in f:
                parts = line.split()
                start = int(parts[0], 16)
                if best < start <= ptr:
                    best, where = start, {k: int(v) for k, v in (q.split("=") for q in parts[2:] if q[0] == "N" and "=" in q)}
        return where
    except Exception:  # noqa: BLE001
        return None


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "reference_cuda":
        return run_reference_cuda(args)

    from compactwarprnntloss_b200 import capi, sharding
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback of the product path)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    fence = make_fence(world, dev)
    cfg = args.cfg
    wl = synth.WORKLOADS[cfg]
    K, repeats = args.steps, max(args.repeats, 1)
    peak, peak_kind = measured_peak()

    # ---- headline workload: weak scaling, B = wl.B * world sequences sharded by lattice size, host-generated (the
    # e2e leg and the CPU baseline need the same logits in host memory)
    B_global = (args.sequences or wl.B) * (world if args.scaling == "weak" else 1)
    lx, ly, y = synth.lengths_and_labels(cfg, B=B_global)
    plan = sharding.plan_shards(lx.tolist(), ly.tolist(), world, order=args.order)
    sharding.validate_plan(plan, B_global)
    ids = plan[rank]
    x_host = synth.compact_logits(cfg, lx, ly, ids, pin=True)
    nodes_global = synth.lattice_nodes(lx, ly)
    job = Job(cfg, lx, ly, y, ids, B_global, dev, x_host.to(dev), world, args.groups)
    elt, nodes_local = job.elt, job.nodes

    for _ in range(max(args.warmup, 3)):
        job.step()
    fence()
    st = capi.read_status(job.ws)
    if st[0] & 0x3:
        raise SystemExit(f"device status reports invalid inputs: {st}")

    # ---- timed region: `repeats` blocks of K pipelined steps (every side stream is joined back into the launching
    # stream inside the call); clocks sampled over all of them
    sampler = ClockSampler(local) if rank == 0 else None
    fence()
    mark = sampler.mark() if sampler else 0
    blocks = timed_blocks(job.step, K, repeats, fence, world, dev)
    clocks = sampler.stop(mark) if sampler else None
    loss_value = job.loss_value()
    sp = spread(blocks, K)
    ms_per_step = sp["median"]
    value = nodes_global / (ms_per_step * 1e-3)

    # ---- kernel breakdown: the same work as two plain calls (no overlap), so that the gradient kernel - one launch
    # over the whole matrix - can be timed by itself for the roofline; and the recursion by itself
    job.forward()
    n_break = max(K, 20)
    fwd = per_call_ms(job.forward, n_break, dev)
    bwd = per_call_ms(job.backward, n_break, dev)
    k2 = per_call_ms(job.recursion, n_break, dev)
    fwd_ms, bwd_ms, bwd_min, bwd_max, k2_ms = max_over_ranks([fwd[0], bwd[0], bwd[1], bwd[2], k2[0]], world, dev)

    # ---- the step through the Python entry point (N = 1: one process, the whole batch)
    py_api = None
    if world == 1 and not args.no_python_api:
        py_api = python_api_ms(job, K, min(repeats, 9), fence)

    # ---- the other workloads, device-generated, one after the other (the largest last), each freed before the next
    configs = {}
    strong = None
    x_keep = job.x
    if world == 1 and not args.no_configs:
        job.gx = None  # room for the 6.4 GB workload: the headline job's gradient buffer is re-made for nothing below
        for c in (1, 4, 5, 3):
            if c == cfg:
                continue
            lxc, lyc, yc = synth.lengths_and_labels(c)
            idc = sharding.plan_shards(lxc.tolist(), lyc.tolist(), 1, order=args.order)[0]
            jc = Job(c, lxc, lyc, yc, idc, len(lxc), dev, device_logits(c, lxc, lyc, idc, dev), 1, 0)
            m = measure_job(jc, K, 5, fence, peak)
            configs[str(c)] = config_block(jc, m, K, peak, peak_kind)
            if c == 1:
                configs["1"]["l2"] = "0.4 MB of logits: resident in L2, launch-bound (correctness-sized workload)"
            if c == 5:
                strong = dict(configs["5"], n_gpus=1, shard_imbalance=1.0, longest_diagonals_per_rank=[jc.longest])
            jc.close()
            del jc, m
            torch.cuda.empty_cache()
    if world > 1 and not args.no_strong:
        # the ragged workload, B = 256 FIXED, sharded over the ranks: strong scaling, bounded by the longest T+U chain
        lx5, ly5, y5 = synth.lengths_and_labels(5)
        plan5 = sharding.plan_shards(lx5.tolist(), ly5.tolist(), world, order=args.order)
        sharding.validate_plan(plan5, len(lx5))
        j5 = Job(5, lx5, ly5, y5, plan5[rank], len(lx5), dev, device_logits(5, lx5, ly5, plan5[rank], dev), world, 0)
        m5 = measure_job(j5, K, 7, fence, peak, want_breakdown=False)
        sp5 = spread(m5["blocks_ms"], K)
        nodes5 = synth.lattice_nodes(lx5, ly5)
        longest = [0] * world
        longest[rank] = j5.longest
        longest = [int(v) for v in max_over_ranks(longest, world, dev)]
        strong = {"workload": synth.WORKLOADS[5].name, "n_gpus": world, "global_sequences": len(lx5),
                  "lattice_nodes": nodes5, "ms_per_step": sp5["median"], "ms_per_step_min": sp5["min"],
                  "ms_per_step_max": sp5["max"], "steps": K, "blocks": sp5["blocks"],
                  "value": nodes5 / (sp5["median"] * 1e-3), "unit": UNIT,
                  "shard_imbalance": round(sharding.shard_imbalance(lx5, ly5, plan5), 4),
                  "longest_diagonals_per_rank": longest, "sequence_groups": j5.n_groups, "loss": m5["loss"],
                  "step_roofline_frac": 3.0 * nodes5 * 128 * 2 / (sp5["median"] * 1e-3) / 1e9 / (peak * world)}
        j5.close()
        del j5
        torch.cuda.empty_cache()

    # ---- end to end through the host-buffer entry point: pinned host logits in, host gradients + costs out
    e2e = None
    job.close()
    flags = job.flags
    lx_l, ly_l, y_l = lx[ids].contiguous(), ly[ids].contiguous(), y[ids].contiguous()
    ct = capi.cost_dtype(x_host.dtype)
    if not args.no_e2e:
        hp = capi.HostPipeline(dev)
        g_host = torch.empty_like(x_host).pin_memory()
        gc = torch.ones(1, dtype=ct)
        vec = job.vec
        e2e_steps = max(2, min(K, 5))

        def e2e_step():
            c, l, s = hp.run(x_host, lx_l, ly_l, y_l, blank=0, flags=flags, grad_costs=gc, grad_x=g_host,
                             mean_denominator=B_global)
            if world > 1:
                sharding.exchange_costs(c.to(dev), ids, B_global, local_loss=l.to(dev), out=vec)
                vec.cpu()
            return l

        e2e_step()
        fence()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            l_host = e2e_step()
        fence()
        e2e_s = max_over_ranks([time.perf_counter() - t0], world, dev)[0] / e2e_steps
        # each direction by itself, all ranks at once: what the link (and the host side it shares) gives one rank
        nbytes = x_host.numel() * elt
        fence()
        up = per_call_ms(lambda: x_keep.copy_(x_host, non_blocking=True), 3, dev)[0]
        fence()
        down = per_call_ms(lambda: g_host.copy_(x_keep, non_blocking=True), 3, dev)[0]
        gbs = [nbytes / (up * 1e-3) / 1e9, nbytes / (down * 1e-3) / 1e9]
        hi = max_over_ranks(gbs, world, dev)
        lo = [-v for v in max_over_ranks([-v for v in gbs], world, dev)]
        small = (lx_l.numel() * 2 + y_l.numel()) * 4
        e2e = {"value": nodes_global / e2e_s, "unit": UNIT,
               "h2d_bytes_per_step": int(nbytes + small + 4),
               "d2h_bytes_per_step": int(g_host.numel() * elt + job.p.B * 4 + 16),
               "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
               "what": "cwrnnt_loss_grad_host: pinned host logits -> device (chunked, 3 streams) -> host gradients "
                       "and costs; per-rank bytes",
               "both_directions_gbs_per_rank": 2.0 * nbytes / e2e_s / 1e9,
               "all_ranks_host_traffic_gbs": 2.0 * nbytes * world / e2e_s / 1e9,
               "h2d_alone_gbs": {"max": hi[0], "min": lo[0]}, "d2h_alone_gbs": {"max": hi[1], "min": lo[1]},
               "alone_means": "one direction at a time, all ranks copying at once (1 plain cudaMemcpyAsync of the "
                              "whole buffer per rank)",
               "pinned_numa_pages_rank0": {"logits": numa_of(x_host.data_ptr()), "gradients": numa_of(g_host.data_ptr())},
               "cpus_allowed_rank0": host_threads(),
               "loss": float(vec[B_global]) if world > 1 else float(l_host)}
        hp.close()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    grad_bytes = 2.0 * nodes_local * wl.V * elt  # one launch: every row read once and written once
    achieved = grad_bytes / (bwd_ms * 1e-3) / 1e9
    traffic = GRAD_KERNEL_DRAM_BYTES_PER_NODE.get(cfg)
    n_groups = job.n_groups
    step_gbs = 3.0 * nodes_local * wl.V * elt / (ms_per_step * 1e-3) / 1e9
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": DTYPE_NAME[wl.dtype], "data": "synthetic",
        "config": workload_config(cfg, world, args.scaling, args.order, args.sequences),
        "timing": {"blocks": repeats, "steps_per_block": K, "ms_per_step_median": sp["median"],
                   "ms_per_step_min": sp["min"], "ms_per_step_max": sp["max"],
                   "timed_region_ms": sum(blocks),
                   "what": "each block: barrier + synchronize, CUDA event, K steps, CUDA event, barrier + synchronize; "
                           "max over ranks per block; ms_per_step and value are the median block"},
        "gpu_launches": job.launches * K * repeats,
        "gpu_launches_per_step": job.launches,
        "kernels_per_step": ["prep_kernel"] + ["gather_rows_kernel", "wavefront_split_kernel",
                                               "grad_rows_kernel"] * n_groups,
        "pipeline": {"entry": "cwrnnt_loss_grad", "sequence_groups": n_groups,
                     "unpipelined_ms_per_step": fwd_ms + bwd_ms, "unpipelined_fwd_ms": fwd_ms,
                     "unpipelined_bwd_ms": bwd_ms},
        "recursion": {"kernel_ms": k2_ms, "longest_diagonals": job.longest,
                      "us_per_diagonal": k2_ms * 1e3 / max(job.longest, 1),
                      "what": "cwrnnt_recursion alone (alpha and beta of every sequence in one launch) / longest T+U"},
        "loss": loss_value,
        "roofline": {"bound": "hbm", "kernel": "grad_rows_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                     "traffic": traffic[0] * nodes_local if traffic else None,
                     "traffic_scaled_from": (f"{traffic[1]}: DRAM bytes per lattice node of one captured launch, "
                                             "times this run's rows") if traffic else None,
                     "algorithmic_bytes": grad_bytes, "launch_ms": bwd_ms, "launch_ms_min": bwd_min,
                     "launch_ms_max": bwd_max, "launches_timed": n_break,
                     "timed": "one launch over the whole matrix (cwrnnt_backward), each between its own CUDA events, "
                              "median of the breakdown loop that follows the timed region"},
        "step_roofline": {"achieved": step_gbs, "peak": peak, "unit": "GB/s", "frac": step_gbs / peak,
                          "bytes_per_node": 3 * wl.V * elt},
        "clocks": clocks,
    }
    if py_api:
        out["python_api"] = py_api
    if configs:
        out["configs"] = configs
    if strong:
        out["strong_cfg5"] = strong
    if e2e:
        out["e2e"] = e2e
    failed = None
    if world == 1 and not args.no_cpu_baseline:
        v, cores, nodes, spent, reps, oc = cpu_reference_time(cfg, lx, ly, y, args.cpu_sample_seqs)
        out["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                               "sample": f"first {min(args.cpu_sample_seqs, wl.B)} of {wl.B} sequences ({nodes} "
                                         f"lattice nodes) per repetition, best of {reps}, {spent:.1f} s of wall time"}
        if len(oc) == B_global:
            want = float(oc.mean() if wl.reduction == "mean" else oc.sum())
            rel = abs(loss_value - want) / abs(want)
            out["loss_check"] = {"oracle": want, "device": loss_value, "rel_err": rel, "tolerance": 1e-5,
                                 "what": "loss of the timed steps against the CPU checker's costs on all sequences"}
            if e2e:
                out["loss_check"]["e2e_rel_err"] = abs(e2e["loss"] - want) / abs(want)
            if not rel <= 1e-5:
                failed = f"loss check failed: device {loss_value} vs oracle {want} (rel {rel:.2e})"
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    if failed:
        raise SystemExit(failed)


if __name__ == "__main__":
    main()
