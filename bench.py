#!/usr/bin/env python
"""Benchmark of the recurrent hot path: forward + backward of one compiled step
function over a batch of synthetic sequences.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--op NAME]

A "step" is one forward + backward pass (upstream gradients for the output and
the final state given) over B=8, T=1024, H=32, 128x128 bf16 Delta Rule inputs
per GPU (seeded synthetic data with the benchmark's distributions).  With
N > 1 (launched by torch.distributed.run) every rank runs the same per-GPU
workload on its own batch shard: the (b,h) recurrences are independent, so
there is no collective in the timed region ("weak" scaling); the only NCCL
calls are the barriers and the max-reduction of the timings.

Printed JSON (rank 0): tokens/s of the whole job with inputs resident in HBM
(`value`), the same through the public API with pinned host buffers and
host<->device copies in the timed region (`e2e`), the roofline record of the
dominant kernel (the backward scan; bound = FP32 CUDA-core pipe, peak measured
in-run by an FMA-only probe kernel), and the CPU oracle timed on a bounded
sample (`cpu_baseline`).

`--impl reference` times the CPU oracle (the restatement of the reference's
`jit.naive` + autograd, which is the reference's only CPU implementation of
this path) on a bounded sample of the same workload, on all host threads.

`--impl reference_cuda` times the unmodified reference package's own generated
CUDA kernels (through its `jit` object) on the same GPU, workload and inputs,
when an install of it is present under `baseline/_ref` (not part of this
repository); otherwise it prints an `unavailable` line.  It is the GPU kernel
this backend replaces, reported beside the CPU baseline.
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

WORKLOADS = {
    # name: (oracle step name, B, T, H, M, N)
    "delta_rule": ("delta_rule", 8, 1024, 32, 128, 128),
    "rwkv7": ("rwkv7", 8, 1024, 32, 128, 128),
    "mamba2": ("mamba2", 8, 1024, 32, 64, 128),
    "gated_delta_rule": ("gated_delta_rule", 8, 1024, 32, 128, 128),
    # the scaling configuration: a global batch of 64 sequences of 4096 steps split over the GPUs ("strong" scaling;
    # 8 sequences per GPU at 8 GPUs, all 64 on one: about 90 GB of checkpoints, row sums and I/O)
    "gated_delta_rule_c4": ("gated_delta_rule", 64, 4096, 32, 128, 128),
}
STRONG = ("gated_delta_rule_c4",)
# DRAM bytes (read + write) of one backward launch per (batch, head) pair, from the ncu capture summarised in
# profiles/*_b2_frnn_fw_bw_ncu_full.md (B=2, 64 pairs; Delta Rule 204.0 MB); traffic grows with the pair count
NCU_BW_DRAM_BYTES_PER_BH = {"delta_rule": 204.03e6 / 64, "rwkv7": 782.1e6 / 64, "mamba2": 355.5e6 / 64,
                            "gated_delta_rule": 690.5e6 / 64}
METRIC = "fwd+bwd tokens/s"
UNIT = "tokens/s"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                    if r[col].lower().startswith("active"):
                        reasons.add(name)
            except (IndexError, ValueError):
                pass
        busy = [s for s in sm if s > 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def bytes_io(tensors):
    return sum(t.numel() * t.element_size() for t in tensors)


def cpu_sample(opname, B, T, H, M, N, heads=None):
    """Times the CPU oracle (fwd + autograd bwd) on a (b,h) sub-slice of the
    workload and scales to whole-workload tokens/s (the slices are independent
    recurrences of equal cost).  ``heads``: heads of one batch element in the
    sample (default: all of them, about ten seconds of CPU work)."""
    import torch
    from oracle import naive_oracle as O
    # all the host threads this process may use (a launcher such as torch.distributed.run pins OMP_NUM_THREADS to 1)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    sb, sh = 1, min(H, heads or H)
    xs, dy, dS = O.make_case(opname, sb, T, sh, M, N, torch.bfloat16)
    t0 = time.perf_counter()
    O.fwd_bwd(O.STEPS[opname], xs[:-1], xs[-1:], [dy], [dS])
    dt = time.perf_counter() - t0
    frac = (sb * sh) / (B * H)
    return {"value": B * T * frac / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"oracle naive fwd+autograd bwd on B={sb},H={sh} of the B={B},H={H} workload "
                      f"(T={T}, {M}x{N}, bf16 inputs, fp32 math), {dt:.2f} s, scaled by {1 / frac:.0f}x"}, dt


def run_reference(args, rank, world):
    if rank != 0:
        return
    import torch
    opname, B, T, H, M, N = WORKLOADS[args.op]
    # size the per-step sample so that the whole run stays within a few minutes (about 0.25 s per head)
    n = max(1, args.warmup + args.steps)
    heads = next((h for h in (32, 16, 8, 4, 2, 1) if h <= H and 0.25 * h * n <= 150), 1)
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        base, dt = cpu_sample(opname, B, T, H, M, N, heads)
        if i >= args.warmup:
            times.append(dt)
    frac = (1 * min(H, heads)) / (B * H)
    ms = 1e3 * sum(times) / len(times)
    value = B * T * frac / (ms / 1e3)
    base["value"] = value
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp32", "data": "synthetic",
            "config": {"workload": f"{args.op} B{B} T{T} H{H} {M}x{N} bf16 I/O (bounded CPU sample per step)"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_reference_cuda(args, rank, world, local):
    """fwd+bwd of the reference package's own compiled path, timed like the main arm (device events, max over ranks)."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    opname, B, T, H, M, N = WORKLOADS[args.op]
    try:
        if not os.path.isdir(os.path.join(ref_dir, "flex_rnn")):
            raise RuntimeError("no reference install under baseline/_ref")
        sys.path.insert(0, ref_dir)
        import torch
        import torch.distributed as dist
        import flex_rnn
        from flex_rnn_b200 import workloads as W
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=dev)
        xs, dy, dS = W.synthetic(opname, B, T, H, M, N, torch.bfloat16, seed=rank)
        leaves = [x.to(dev).requires_grad_() for x in xs]
        dy, dS = dy.to(dev), dS.to(dev)
        op = flex_rnn.jit(W.STEPS[opname])

        def step():
            y, ST = op(*leaves)
            return torch.autograd.grad([y, ST], leaves, [dy.to(y.dtype), dS])
        # the reference builds its extension in a fixed directory: let rank 0 build, then the others load it
        for turn in range(2 if world > 1 else 1):
            if world == 1 or (rank == 0) == (turn == 0):
                step()
            if world > 1:
                dist.barrier()
        for _ in range(max(args.warmup, 3)):
            step()
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        times = []
        for _ in range(args.steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            torch.cuda.synchronize(dev)
            times.append(e0.elapsed_time(e1))
        ms = torch.tensor([sum(times) / len(times)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.destroy_process_group()
        ms = float(ms)
        if rank == 0:
            print(json.dumps({"impl": "reference_cuda", "metric": METRIC, "value": world * B * T / (ms / 1e3), "unit": UNIT,
                              "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
                              "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
                              "config": {"workload": f"{args.op} B{B} T{T} H{H} {M}x{N} bf16 I/O, fp32 math, per GPU",
                                         "l2": "256 MiB flush write between timed steps"}}), flush=True)
    except Exception as e:  # the reference is not part of this repository: report, do not fail
        if rank == 0:
            print(json.dumps({"impl": "reference_cuda", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_cuda"])
    ap.add_argument("--op", default="delta_rule", choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch (default: the benchmark's 8); smaller = profiling case")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    args = ap.parse_args()
    if args.batch:
        for k, w in list(WORKLOADS.items()):
            WORKLOADS[k] = (w[0], args.batch) + w[2:]
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.impl == "reference_cuda":
        run_reference_cuda(args, rank, world, local)
        return

    import torch
    import torch.distributed as dist
    import flex_rnn_b200
    from flex_rnn_b200 import runtime
    from flex_rnn_b200 import workloads as W

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    opname, B, T, H, M, N = WORKLOADS[args.op]
    strong = args.op in STRONG and not args.batch
    if strong:
        assert B % world == 0, "the global batch must divide over the GPUs"
        B //= world
    if B * T * H * N * 2 * 3 > 2e9:
        args.no_e2e = True          # the host-buffer leg would pin several GB per buffer set: kept to the headline sizes
    step_fn = W.STEPS[opname]
    # each rank draws its own shard of the global batch (seed offset by the rank)
    xs_host, dy_host, dS_host = W.synthetic(opname, B, T, H, M, N, torch.bfloat16, seed=rank)
    xs = [x.to(dev) for x in xs_host]
    dy, dS = dy_host.to(dev), dS_host.to(dev)
    op = flex_rnn_b200.jit(step_fn)
    leaves = [x.requires_grad_() for x in xs]

    stream = torch.cuda.current_stream(dev)
    fw_ms, bw_ms = [], []

    def one_step(record):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if record else None
        if record:
            ev[0].record(stream)
        y, ST = op(*leaves)
        if record:
            ev[1].record(stream)
        grads = torch.autograd.grad([y, ST], leaves, [dy, dS])
        if record:
            ev[2].record(stream)
        return ev, grads

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        one_step(False)
    sync_all()
    assert op.forward_func.kernel_status(dev) == 0, "a kernel reported a timed-out wait"

    # FP32 CUDA-core peak, measured now with the library's FMA-only probe kernel
    sink = torch.zeros(4, device=dev)
    probe = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fl = runtime.fp32_peak_probe(sink.data_ptr(), 20000, stream.cuda_stream)
        e1.record(stream)
        torch.cuda.synchronize(dev)
        probe.append(fl / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    fp32_peak = max(probe[1:])
    sms = torch.cuda.get_device_properties(dev).multi_processor_count

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sync_all()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    evs = []
    for _ in range(args.steps):
        ev, _ = one_step(True)
        evs.append(ev)
    t_end.record(stream)
    sync_all()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_start.elapsed_time(t_end)
    for ev in evs:
        fw_ms.append(ev[0].elapsed_time(ev[1]))
        bw_ms.append(ev[1].elapsed_time(ev[2]))
    tms = torch.tensor([total_ms], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    total_ms = float(tms.item())
    ms_per_step = total_ms / args.steps
    value = world * B * T / (ms_per_step * 1e-3)

    # end to end through the public API with host buffers (pinned), copies in the timed region
    if args.no_e2e:
        pin, pdy, pdS = [], dy_host, dS_host
    else:
        pin = [x.detach().cpu().pin_memory() for x in xs_host]
        pdy, pdS = dy_host.pin_memory(), dS_host.pin_memory()
    out_host = None

    # Three streams, two buffer sets: the host->device copy of step i+1 and the device->host copy of step
    # i-1 run beside the kernels of step i (all of them inside the timed region).
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    host_in = pin + [pdy, pdS]
    dev_in = [[] if args.no_e2e else [torch.empty_like(p, device=dev) for p in host_in] for _ in range(2)]
    dev_out = [None, None]
    ev_in = [torch.cuda.Event() for _ in range(2)]       # inputs of the slot are on the device
    ev_used = [torch.cuda.Event() for _ in range(2)]     # the kernels are done with the slot's inputs
    ev_done = [torch.cuda.Event() for _ in range(2)]     # results of the slot are staged
    ev_out = [torch.cuda.Event() for _ in range(2)]      # results of the slot have reached the host

    def e2e_step(i):
        nonlocal out_host
        k = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_used[k])
            for d_, h_ in zip(dev_in[k], host_in):
                d_.copy_(h_, non_blocking=True)
            ev_in[k].record(s_in)
        stream.wait_event(ev_in[k])
        stream.wait_event(ev_out[k])
        d = [t.detach().requires_grad_() for t in dev_in[k][:-2]]
        y, ST = op(*d)
        grads = torch.autograd.grad([y, ST], d, [dev_in[k][-2], dev_in[k][-1]])
        res = [y, ST, *grads]
        if dev_out[k] is None:
            dev_out[k] = [torch.empty_like(r) for r in res]
        if out_host is None:
            out_host = [torch.empty(r.shape, dtype=r.dtype, pin_memory=True) for r in res]
        for o_, r in zip(dev_out[k], res):
            o_.copy_(r.detach())
        ev_used[k].record(stream)
        ev_done[k].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[k])
            for h, o_ in zip(out_host, dev_out[k]):
                h.copy_(o_, non_blocking=True)
            ev_out[k].record(s_out)

    n_e2e = 0 if args.no_e2e else max(4, min(args.steps, 20))
    for i in range(0 if args.no_e2e else 4):
        e2e_step(i)
    torch.cuda.synchronize(dev)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(n_e2e):
        e2e_step(i)
    stream.wait_stream(s_out)          # the last results must have reached the host
    stream.wait_stream(s_in)
    e1.record(stream)
    torch.cuda.synchronize(dev)
    sync_all()
    e2e_ms = torch.tensor([e0.elapsed_time(e1) / max(1, n_e2e)], device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms.item())
    h2d = 0 if args.no_e2e else sum(p.numel() * p.element_size() for p in host_in)
    d2h = sum(h.numel() * h.element_size() for h in out_host) if out_host else 0

    if rank == 0:
        plan = op.forward_func.plan
        fw_src, bw_src = op.forward_func.sources
        stream_mb = (bytes_io(xs) * 3 + 2 * B * T * H * M * 2 + plan.nck * B * H * M * N * 4 * 2
                     + len(plan.aux) * B * T * H * M * 4 * 2) / 1e6
        k_bw = plan.k_joint - plan.k_fwd
        elems = B * T * H * M * N
        bw_avg, fw_avg = statistics.mean(bw_ms), statistics.mean(fw_ms)
        achieved = elems * k_bw / (bw_avg * 1e-3) / 1e12
        flops_all = elems * plan.k_joint
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        hbm = peaks.get("hbm_gbs", 6650.0)
        elt = 2
        bytes_alg = sum(x.numel() * x.element_size() for x in xs) * 2 + (B * T * H * M * elt) * 2 + 2 * B * H * M * N * elt \
            + sum(x.numel() * x.element_size() for x in xs[:-1])
        t_fp32 = flops_all / (fp32_peak * 1e12)
        t_hbm = bytes_alg / (hbm * 1e9)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "fp32", "data": "synthetic",
            "config": {"workload": f"{args.op} fwd+bwd, B{B} T{T} H{H} {M}x{N} per GPU, bf16 I/O, fp32 state and math",
                       "io_dtype": "bf16", "global_batch": B * world, "seq_len": T, "parallelism": f"batch shards x{world}, no collective",
                       "l2": f"no flush: each step streams {stream_mb:.0f} MB of inputs, outputs, checkpoints and row sums "
                             "through HBM (L2 is 126 MB)",
                       "checkpoint_every": plan.D, "backward": "reverse re-step" if plan.reverse else "recompute from slots",
                       "fw_kernel": {"grid": list(fw_src.grid), "block": fw_src.block, "smem": fw_src.smem_bytes,
                                     "tile": fw_src.info["tile"][:2], "packed_fp32x2": fw_src.info["packed"]},
                       "bw_kernel": {"grid": list(bw_src.grid), "block": bw_src.block, "smem": bw_src.smem_bytes,
                                     "tile": bw_src.info["tile"][:2], "packed_fp32x2": bw_src.info["packed"]}},
            "fw_ms": fw_avg, "bw_ms": bw_avg,
            # spread of the per-step device time (forward + backward events of each timed step), rank 0
            "step_ms_p20_p50_p80": [round(sorted(f + b for f, b in zip(fw_ms, bw_ms))[int(q * (len(fw_ms) - 1))], 4)
                                    for q in (0.2, 0.5, 0.8)],
            "roofline_fraction_step": max(t_fp32, t_hbm) / (ms_per_step * 1e-3),
            "roofline": {"bound": "fp32", "kernel": bw_src.name, "achieved": achieved, "peak": fp32_peak, "unit": "TFLOP/s",
                         "frac": achieved / fp32_peak,
                         "traffic": NCU_BW_DRAM_BYTES_PER_BH[args.op] * B * H if args.op in NCU_BW_DRAM_BYTES_PER_BH else None,
                         "algorithmic_bytes": bytes_io(xs) * 2 + B * T * H * M * 2,
                         "peak_source": f"measured in this run by the FMA probe kernel ({sms} SMs); HBM copy peak {hbm} GB/s "
                                        + ("of measured" if peaks else "of fallback"),
                         "flops_per_launch": elems * k_bw, "k_joint": plan.k_joint, "k_fwd": plan.k_fwd,
                         "hbm_bound_ms": t_hbm * 1e3, "fp32_bound_ms": t_fp32 * 1e3},
            "e2e": {"value": (world * B * T / (e2e_ms * 1e-3)) if n_e2e else None, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms},
            "gpu_launches": 2 * args.steps,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            # one cold pass, then the mean of three (about ten seconds of CPU work on all host threads)
            heads = H if T <= 1024 else 4          # bounds the autograd graph's memory for long sequences
            cpu_sample(opname, B, T, H, M, N, heads)
            runs = [cpu_sample(opname, B, T, H, M, N, heads) for _ in range(3)]
            base = runs[-1][0]
            mean_dt = sum(dt for _, dt in runs) / len(runs)
            base["value"] = base["value"] * runs[-1][1] / mean_dt
            base["sample"] += f"; mean of 3 passes after one cold pass ({mean_dt:.2f} s each)"
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
