#!/usr/bin/env python
"""fwd+bwd lattice-nodes/sec of the compact RNN-T loss on B200, with its HBM roofline and the host-CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--cfg 2]

A step is one pass of the hot path over one synthetic batch: forward (row offsets, fused log-softmax + gather,
alpha/beta wavefront, costs, loss) and backward (dense gradient w.r.t. the logits), called through the C ABI.

N = 1: the Conformer-shape workload (B=32, T~U[150,250], U~U[20,80], V=1024, float32 logits), 1.3 GB of logits, larger
than the 126 MB L2, so every step streams from HBM. N > 1 (launched by torch.distributed.run, one rank per GPU): weak
scaling - the global batch is 32*N sequences of the same distribution, sharded by lattice size; the only collective
is the all-reduce of the [B_global+1] cost vector.

One JSON line comes out of rank 0: `value` = lattice nodes of all ranks / max-over-ranks device time with inputs
resident in HBM; `e2e` = the same through the host-buffer entry point (pinned host logits in, host gradients out,
PCIe copies inside the timed region); `roofline` = the gradient kernel (the dominant launch) against the measured copy
bandwidth; `cpu_baseline` = the CPU checker (oracle/) timed on a bounded sample of the same workload.
`--impl reference` times that CPU implementation alone (the reference project has no CPU path of its own: its three
source files are CUDA only).
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
# capture summarised in profiles/grad_rows_kernel_conformer_v1024.md (V=1024 float32; algorithmic figure is 8192).
GRAD_KERNEL_DRAM_BYTES_PER_NODE = {2: 8047.0}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_cuda"],
                    help="ours: this engine; reference: the path's CPU implementation on the host cores; "
                         "reference_cuda: the reference project's own CUDA kernels rebuilt for sm_100a (oracle/_ref)")
    ap.add_argument("--cfg", type=int, default=2, help="workload (1-5); the headline metric is quoted on 2")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: B*N sequences over N GPUs (default); strong: the workload's B sequences sharded over N")
    ap.add_argument("--groups", type=int, default=0,
                    help="sequence groups of the pipelined step (0 = chosen by the library, 1 = no overlap)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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


def cpu_reference_time(cfg, lx, ly, y, n_seqs, budget_s=12.0):
    """The CPU checker's fused float32 pipeline (all host threads) on the first n_seqs sequences, repeated until
    about budget_s seconds of wall time are spent; nodes/s of the best repetition."""
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
    times = []
    while sum(times) < budget_s and len(times) < 200:
        t0 = time.perf_counter()
        oracle.fused_f32io(x, lxs, lys, ys, 0, weights=w, dense_out=out)
        times.append(time.perf_counter() - t0)
    nodes = x.shape[0]
    return nodes / min(times), oracle.num_threads(), nodes, sum(times), len(times)


def run_reference(args):
    """--impl reference: the path's CPU implementation on the box's host cores. The reference project itself is CUDA
    only, so this is the CPU checker (oracle/rnnt_oracle.c, OpenMP over rows and sequences)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = args.cfg
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
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl.name, "sample": sample, "host_threads": oracle.num_threads()},
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
    cfg = args.cfg
    wl = synth.WORKLOADS[cfg]

    # ---- workload: weak scaling, B = wl.B * world sequences sharded by lattice size
    B_global = wl.B * world if args.scaling == "weak" else wl.B
    lx, ly, y = synth.lengths_and_labels(cfg, B=B_global)
    plan = sharding.plan_shards(lx.tolist(), ly.tolist(), world)
    sharding.validate_plan(plan, B_global)
    ids = plan[rank]
    x_host = synth.compact_logits(cfg, lx, ly, ids, pin=True)
    lx_l, ly_l, y_l = lx[ids].contiguous(), ly[ids].contiguous(), y[ids].contiguous()
    nodes_local = x_host.shape[0]
    nodes_global = synth.lattice_nodes(lx, ly)
    elt = x_host.element_size()

    x = x_host.to(dev)
    lxd, lyd, yd = lx_l.to(dev), ly_l.to(dev), y_l.to(dev)
    flags = capi.FUSED_LOG_SOFTMAX | (capi.REDUCE_MEAN if wl.reduction == "mean" else capi.REDUCE_SUM)
    p = capi.make_problem(x, lxd, yd, 0, flags, mean_denominator=B_global)
    ws = capi.alloc_workspace(p, dev)
    ct = capi.cost_dtype(x.dtype)
    costs = torch.empty(p.B, dtype=ct, device=dev)
    loss = torch.zeros((), dtype=ct, device=dev)
    gx = torch.empty_like(x)
    one = torch.ones(1, dtype=ct, device=dev)
    vec = torch.empty(B_global + 1, dtype=ct, device=dev)
    ids_dev = torch.tensor(ids, dtype=torch.int32, device=dev)

    pipe = capi.Pipe(dev)
    n_groups = capi.pipeline_groups(p, args.groups)
    main, comm = torch.cuda.current_stream(dev), torch.cuda.Stream(dev)

    def forward():
        if world == 1:
            capi.forward(p, x, lxd, lyd, yd, ws, costs, loss)
        else:
            capi.forward_sharded(p, x, lxd, lyd, yd, ws, costs, loss, ids_dev, B_global, vec)

    def step():
        # one pipelined call: K0, then per sequence group gather -> wavefront (side stream) -> gradient
        if world == 1:
            capi.loss_grad(p, x, lxd, lyd, yd, ws, costs, loss, one, 0, gx, pipe=pipe, groups=args.groups)
        else:
            # the wavefront epilogue fills the global cost vector; one all-reduce is the whole exchange
            # and it runs on a second stream as soon as the wavefronts are done, underneath the gradient kernels
            capi.loss_grad(p, x, lxd, lyd, yd, ws, costs, loss, one, 0, gx, pipe=pipe, groups=args.groups,
                           global_ids=ids_dev, n_global=B_global, cost_vector=vec)
            with torch.cuda.stream(comm):
                pipe.wait_costs(comm)
                dist.all_reduce(vec, op=dist.ReduceOp.SUM)
            main.wait_stream(comm)

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    fence()
    st = capi.read_status(ws)
    if st[0] & 0x3:
        raise SystemExit(f"device status reports invalid inputs: {st}")

    # ---- timed region: K pipelined steps between two CUDA events on the launching stream (every side stream is
    # joined back into it inside the call)
    K = args.steps
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local) if rank == 0 else None
    fence()
    mark = sampler.mark() if sampler else 0
    begin.record()
    for k in range(K):
        step()
    end.record()
    fence()
    clocks = sampler.stop(mark) if sampler else None
    total_ms = begin.elapsed_time(end)
    loss_value = float(vec[B_global] if world > 1 else loss)

    # ---- kernel breakdown: the same work as two plain calls (no overlap), so that the gradient kernel - one launch
    # over the whole matrix - can be timed by itself for the roofline
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    for k in range(K):
        ev[k][0].record()
        forward()
        ev[k][1].record()
        capi.backward(p, x, lxd, lyd, yd, ws, one, 0, gx)
        ev[k][2].record()
    fence()
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / K
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / K
    t = torch.tensor([total_ms, fwd_ms, bwd_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, fwd_ms, bwd_ms = [float(v) for v in t.cpu()]
    ms_per_step = total_ms / K
    value = nodes_global / (ms_per_step * 1e-3)

    # ---- end to end through the host-buffer entry point: pinned host logits in, host gradients + costs out
    e2e = None
    if not args.no_e2e:
        pipe = capi.HostPipeline(dev)
        g_host = torch.empty_like(x_host).pin_memory()
        gc = torch.ones(1, dtype=ct)
        e2e_steps = max(2, min(K, 5))

        def e2e_step():
            c, l, s = pipe.run(x_host, lx_l, ly_l, y_l, blank=0, flags=flags, grad_costs=gc, grad_x=g_host,
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
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e_s = float(dt.cpu()) / e2e_steps
        small = (lx_l.numel() * 2 + y_l.numel()) * 4
        e2e = {"value": nodes_global / e2e_s, "unit": UNIT,
               "h2d_bytes_per_step": int(x_host.numel() * elt + small + 4),
               "d2h_bytes_per_step": int(g_host.numel() * elt + p.B * 4 + 16),
               "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
               "what": "cwrnnt_loss_grad_host: pinned host logits -> device (chunked, 3 streams) -> host gradients "
                       "and costs; per-rank bytes",
               "loss": float(vec[B_global]) if world > 1 else float(l_host)}
        pipe.close()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    grad_bytes = 2.0 * nodes_local * wl.V * elt  # one launch: every row read once and written once
    achieved = grad_bytes / (bwd_ms * 1e-3) / 1e9
    traffic = GRAD_KERNEL_DRAM_BYTES_PER_NODE.get(cfg)
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[wl.dtype],
        "data": "synthetic",
        "config": {"workload": wl.name, "global_sequences": B_global, "lattice_nodes": nodes_global,
                   "logits_bytes_per_gpu": int(x_host.numel() * elt), "sharding": f"lattice-size LPT over {world} rank(s)",
                   "l2": "inputs larger than L2 (no flush needed)", "reduction": wl.reduction,
                   "shard_imbalance": round(sharding.shard_imbalance(lx, ly, plan), 4)},
        "gpu_launches": (1 + 3 * n_groups) * K,
        "kernels_per_step": ["prep_kernel"] + ["gather_rows_kernel", "wavefront_split_kernel",
                                               "grad_rows_kernel"] * n_groups,
        "pipeline": {"entry": "cwrnnt_loss_grad", "sequence_groups": n_groups,
                     "unpipelined_ms_per_step": fwd_ms + bwd_ms, "unpipelined_fwd_ms": fwd_ms,
                     "unpipelined_bwd_ms": bwd_ms},
        "loss": loss_value,
        "roofline": {"bound": "hbm", "kernel": "grad_rows_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                     "traffic": traffic * nodes_local if traffic else None,
                     "algorithmic_bytes": grad_bytes, "launch_ms": bwd_ms,
                     "timed": "one launch over the whole matrix (cwrnnt_backward), CUDA events, mean of the "
                              "breakdown loop that follows the timed region"},
        "step_roofline": {"achieved": 3.0 * nodes_local * wl.V * elt / (ms_per_step * 1e-3) / 1e9, "peak": peak,
                          "unit": "GB/s", "frac": 3.0 * nodes_local * wl.V * elt / (ms_per_step * 1e-3) / 1e9 / peak,
                          "bytes_per_node": 3 * wl.V * elt},
        "clocks": clocks,
    }
    if e2e:
        out["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        v, cores, nodes, spent, reps = cpu_reference_time(cfg, lx, ly, y, args.cpu_sample_seqs)
        out["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                               "sample": f"first {min(args.cpu_sample_seqs, wl.B)} of {wl.B} sequences ({nodes} "
                                         f"lattice nodes) per repetition, best of {reps}, {spent:.1f} s of wall time"}
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
