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

Printed JSON (rank 0), one line:
  value / ms_per_step   tokens/s of the whole job with inputs resident in HBM
  e2e                   the same through the public API with pinned host buffers
                        and host<->device copies in the timed region
  roofline              the dominant kernel (the backward scan): bound = FP32
                        CUDA-core pipe, peak measured in-run by an FMA-only probe
  cpu_baseline          the reference's CPU path (its jit.naive + autograd) on a
                        bounded sample, on the host cores (one GPU only)
  workloads             (one GPU) the other benchmark configurations - RWKV-7,
                        Mamba-2, Gated Delta Rule at B8 T1024 - timed the same way
  scaling_c4            the scaling configuration: Gated Delta Rule, global batch
                        64, T4096, split over the N GPUs by ``shard.shard_args``
                        ("strong" scaling: total work fixed)
  reference_cuda        (one GPU) the unmodified reference package's own generated
                        CUDA kernels on the same GPU and inputs, when an install
                        of it is present under baseline/_ref

`--impl reference` times the reference's CPU implementation of the path on the
host cores: `jit.naive` of the reference package itself when an install of it is
importable from `baseline/_ref` (kind "reference"), else the restatement in
`oracle/` (kind "port"); one batch element, all heads, per step.

`--impl reference_cuda` is the arm behind the `reference_cuda` record.
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
    # name: (step name, B, T, H, M, N)
    "delta_rule": ("delta_rule", 8, 1024, 32, 128, 128),
    "rwkv7": ("rwkv7", 8, 1024, 32, 128, 128),
    "mamba2": ("mamba2", 8, 1024, 32, 64, 128),
    "gated_delta_rule": ("gated_delta_rule", 8, 1024, 32, 128, 128),
    # the scaling configuration: a global batch of 64 sequences of 4096 steps split over the GPUs
    "gated_delta_rule_c4": ("gated_delta_rule", 64, 4096, 32, 128, 128),
}
STRONG = ("gated_delta_rule_c4",)
# per-element op counts of the joint graphs as the reference's tracer yields them (scalars expanded to rows);
# this backend keeps scalars as scalars, which makes Mamba-2's executed graph three ops shorter
K_JOINT_REFERENCE_TRACER = {"delta_rule": 18, "rwkv7": 28, "mamba2": 19, "gated_delta_rule": 22}
METRIC = "fwd+bwd tokens/s"
UNIT = "tokens/s"


def workload_text(op, B, T, H, M, N):
    return f"{op} fwd+bwd, B{B} T{T} H{H} {M}x{N} per GPU, bf16 I/O, fp32 state and math"


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


# ---------------------------------------------------------------------------------------------------------------
# CPU legs: the reference's jit.naive + autograd on the host cores
# ---------------------------------------------------------------------------------------------------------------

_REF_JIT = {}


def reference_naive(step_fn):
    """(callable running the reference's own ``jit.naive`` for ``step_fn``, "reference"), from an install of the
    reference package under baseline/_ref; or (None, why) when there is none."""
    if "mod" not in _REF_JIT:
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        try:
            if not os.path.isdir(os.path.join(ref_dir, "flex_rnn")):
                raise ImportError("no reference install under baseline/_ref")
            sys.path.insert(0, ref_dir)
            import flex_rnn
            _REF_JIT["mod"] = flex_rnn
        except Exception as e:      # not part of this repository: fall back to the port
            _REF_JIT["mod"] = None
            _REF_JIT["why"] = f"{type(e).__name__}: {str(e)[:120]}"
    if _REF_JIT["mod"] is None:
        return None, _REF_JIT["why"]
    return _REF_JIT["mod"].jit(step_fn).naive, "reference"


def cpu_sample(opname, B, T, H, M, N, heads=None):
    """Times the reference's CPU path (fwd + autograd bwd) on a (b,h) sub-slice of the workload and scales to
    whole-workload tokens/s (the slices are independent recurrences of equal cost).  ``heads``: heads of one batch
    element in the sample (default: all of them, under a second to a few seconds of CPU work)."""
    import torch
    from oracle import naive_oracle as O
    # all the host threads this process may use (a launcher such as torch.distributed.run pins OMP_NUM_THREADS to 1)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    sb, sh = 1, min(H, heads or H)
    xs, dy, dS = O.make_case(opname, sb, T, sh, M, N, torch.bfloat16)
    naive, kind = reference_naive(O.STEPS[opname])
    t0 = time.perf_counter()
    if naive is not None:
        leaves = [x.detach().clone().requires_grad_() for x in xs]
        y, ST = naive(*leaves)
        torch.autograd.grad([y, ST], leaves, [dy.to(y.dtype), dS.to(ST.dtype)], allow_unused=True)
        what = "the reference's jit.naive (baseline/_ref)"
    else:
        O.fwd_bwd(O.STEPS[opname], xs[:-1], xs[-1:], [dy], [dS])
        kind, what = "port", "oracle restatement of jit.naive"
    dt = time.perf_counter() - t0
    frac = (sb * sh) / (B * H)
    return {"value": B * T * frac / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{what} fwd + autograd bwd on B={sb},H={sh} of the B={B},H={H} workload "
                      f"(T={T}, {M}x{N}, bf16 inputs, fp32 math), {dt:.2f} s, scaled by {1 / frac:.0f}x"}, dt


def cpu_heads(H, T, n_passes):
    """Heads of one batch element per pass: all of them for the headline sizes (the same sample in the
    `cpu_baseline` record and in the reference arm), fewer only when many passes or long sequences are asked for."""
    per_head = 0.03 * T / 1024
    return next((h for h in (H, 16, 8, 4, 2, 1) if h <= H and per_head * h * n_passes <= 240), 1)


def run_reference(args, rank, world):
    if rank != 0:
        return
    opname, B, T, H, M, N = WORKLOADS[args.op]
    n = max(1, args.warmup + args.steps)
    heads = cpu_heads(H, T, n)
    times, base = [], None
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
            "config": {"workload": workload_text(args.op, B, T, H, M, N)},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# the reference's own CUDA path (third arm)
# ---------------------------------------------------------------------------------------------------------------

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
        torch.cuda.synchronize(dev)
        torch.cuda.reset_peak_memory_stats(dev)
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
        peak_gib = (torch.cuda.max_memory_allocated(dev) - flush.numel()) / 2 ** 30
        ms = torch.tensor([sum(times) / len(times)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.destroy_process_group()
        ms = float(ms)
        if rank == 0:
            print(json.dumps({"impl": "reference_cuda", "metric": METRIC, "value": world * B * T / (ms / 1e3), "unit": UNIT,
                              "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
                              "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
                              "peak_memory_gib": round(peak_gib, 3),
                              "config": {"workload": workload_text(args.op, B, T, H, M, N),
                                         "l2": "256 MiB flush write between timed steps"}}), flush=True)
    except Exception as e:  # the reference is not part of this repository: report, do not fail
        if rank == 0:
            print(json.dumps({"impl": "reference_cuda", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}), flush=True)


def reference_cuda_record(op, steps):
    """Runs the `--impl reference_cuda` arm in a process of its own (the reference compiles an extension with nvcc
    and ninja on first use) and returns its JSON record."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference_cuda", "--op", op, "--steps", str(steps), "--warmup", "3"]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        for ln in reversed(r.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)
        return {"impl": "reference_cuda", "unavailable": f"no record (exit {r.returncode}): {r.stderr[-200:]}"}
    except Exception as e:
        return {"impl": "reference_cuda", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


# ---------------------------------------------------------------------------------------------------------------
# this backend
# ---------------------------------------------------------------------------------------------------------------

class Bench:
    def __init__(self, args, rank, world, local):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.args, self.rank, self.world, self.local = args, rank, world, local
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
        torch.cuda.set_device(local)
        self.dev = torch.device("cuda", local)
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
        self.stream = torch.cuda.current_stream(self.dev)
        self.sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
        self.peaks = {}
        try:
            self.peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        self.hbm = self.peaks.get("hbm_gbs", 6650.0)
        self.fp32_peak = None

    def sync_all(self):
        self.torch.cuda.synchronize(self.dev)
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, x):
        t = self.torch.tensor([float(x)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def probe_fp32_peak(self):
        """FP32 CUDA-core peak, measured now with the library's FMA-only probe kernel."""
        from flex_rnn_b200 import runtime
        torch = self.torch
        sink = torch.zeros(4, device=self.dev)
        probe = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            fl = runtime.fp32_peak_probe(sink.data_ptr(), 20000, self.stream.cuda_stream)
            e1.record(self.stream)
            torch.cuda.synchronize(self.dev)
            probe.append(fl / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        self.fp32_peak = max(probe[1:])
        return self.fp32_peak

    def probe_fma_kinds(self):
        """Share of the measured FP32 peak that register-only loops of the scan kernels' kinds of FMA reach (the
        library's probe kernels: all operands distinct registers, one operand kept, the Delta Rule step mixes)."""
        from flex_rnn_b200 import runtime
        torch = self.torch
        sink = torch.zeros(4, device=self.dev)
        src = torch.rand(4096, device=self.dev) * 1e-3
        out = {}
        for kind, name in runtime.MIX_PROBES.items():
            best = 0.0
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                fl = runtime.fp32_mix_probe(kind, sink.data_ptr(), src.data_ptr(), 2000, self.stream.cuda_stream)
                e1.record(self.stream)
                torch.cuda.synchronize(self.dev)
                best = max(best, fl / (e0.elapsed_time(e1) * 1e-3) / 1e12)
            out[name] = round(best / self.fp32_peak, 4)
        return out

    # ---- one workload, inputs resident in HBM -------------------------------------------------------------
    def measure(self, opname, xs, dy, dS, steps, warmup, sample_clocks=False):
        """Forward + backward of ``jit(step)`` on device-resident arguments: ``warmup`` untimed steps (the first
        compiles and autotunes), then ``steps`` timed ones between barriers; device events; max over ranks."""
        import flex_rnn_b200
        from flex_rnn_b200 import workloads as W
        torch = self.torch
        op = flex_rnn_b200.jit(W.STEPS[opname])
        leaves = [x.requires_grad_() for x in xs]
        stream = self.stream

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

        for _ in range(warmup):
            one_step(False)
        self.sync_all()
        assert op.forward_func.kernel_status(self.dev) == 0, "a kernel reported a timed-out wait"
        torch.cuda.reset_peak_memory_stats(self.dev)
        sampler = ClockSampler(self.local) if (sample_clocks and self.rank == 0) else None
        if sampler:
            sampler.start()
        self.sync_all()
        t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_start.record(stream)
        evs = [one_step(True)[0] for _ in range(steps)]
        t_end.record(stream)
        self.sync_all()
        clocks = sampler.stop() if sampler else None
        total_ms = self.max_over_ranks(t_start.elapsed_time(t_end))
        fw_ms = [ev[0].elapsed_time(ev[1]) for ev in evs]
        bw_ms = [ev[1].elapsed_time(ev[2]) for ev in evs]
        return {"op": op, "ms_per_step": total_ms / steps, "fw_ms": fw_ms, "bw_ms": bw_ms, "clocks": clocks,
                "peak_memory_gib": torch.cuda.max_memory_allocated(self.dev) / 2 ** 30}

    def analyse(self, opname, m, xs, B, T, H, M, N):
        """Roofline arithmetic of one measured workload (per GPU)."""
        plan = m["op"].forward_func.plan
        fw_src, bw_src = m["op"].forward_func.sources
        tuned = m["op"].forward_func.tuned
        elems = B * T * H * M * N
        elt = xs[0].element_size()
        in_bytes = bytes_io(xs[:-1])
        st_bytes = bytes_io(xs[-1:])
        y_bytes = B * T * H * M * elt
        # compulsory traffic (no checkpoints, no saved row sums): fwd reads inputs + S0, writes y + S_T;
        # bwd reads inputs + dy + dS_T, writes the gradients + dS0
        bytes_fw_alg = in_bytes + st_bytes + y_bytes + st_bytes
        bytes_bw_alg = in_bytes + y_bytes + st_bytes + in_bytes + st_bytes
        # what the backward launch actually moves, from the plan: plus saved row sums and fp32 checkpoints read
        aux_bytes = len(plan.aux) * B * H * T * M * 4
        ck_bytes = plan.nck * B * H * M * N * 4 * plan.n_st
        traffic_bw = bytes_bw_alg + aux_bytes + ck_bytes
        traffic_fw = bytes_fw_alg + aux_bytes + ck_bytes
        fw_avg, bw_avg = statistics.mean(m["fw_ms"]), statistics.mean(m["bw_ms"])
        k_bw = plan.k_joint - plan.k_fwd
        peak = self.fp32_peak
        t_fp32 = elems * plan.k_joint / (peak * 1e12)
        t_hbm = (bytes_fw_alg + bytes_bw_alg) / (self.hbm * 1e9)
        step_s = m["ms_per_step"] * 1e-3
        rec = {
            "fw_ms": round(fw_avg, 4), "bw_ms": round(bw_avg, 4), "ms_per_step": round(m["ms_per_step"], 4),
            "tokens_per_s": self.world * B * T / step_s,
            "roofline_fraction_step": max(t_fp32, t_hbm) / step_s,
            "roofline_fraction_fw": elems * plan.k_fwd / (fw_avg * 1e-3) / 1e12 / peak,
            "roofline_fraction_bw": elems * k_bw / (bw_avg * 1e-3) / 1e12 / peak,
            "k_joint": plan.k_joint, "k_fwd": plan.k_fwd,
            "fp32_bound_ms": t_fp32 * 1e3, "hbm_bound_ms": t_hbm * 1e3,
            "peak_memory_gib": round(m["peak_memory_gib"], 3),
            "checkpoint_every": plan.D, "backward": "reverse re-step" if plan.reverse else "recompute from slots",
            "fw_kernel": {"grid": list(fw_src.grid), "block": fw_src.block, "smem": fw_src.smem_bytes,
                          "tile": fw_src.info["tile"][:2], "packed_fp32x2": fw_src.info["packed"],
                          "variant": tuned["fw_choice"], "timed_variants": len(tuned["fw_log"])},
            "bw_kernel": {"grid": list(bw_src.grid), "block": bw_src.block, "smem": bw_src.smem_bytes,
                          "tile": bw_src.info["tile"][:2], "packed_fp32x2": bw_src.info["packed"],
                          "variant": tuned["bw_choice"], "timed_variants": len(tuned["bw_log"])},
        }
        kref = K_JOINT_REFERENCE_TRACER.get(opname)
        if kref and kref != plan.k_joint:
            rec["roofline_fraction_step_reference_tracer_k"] = elems * kref / (peak * 1e12) / step_s
            rec["k_joint_reference_tracer"] = kref
        units = B * H * (M // bw_src.info["tile"][2])
        per_wave = self.sms * max(1, plan.tuning.bw_min_blocks)
        issued = (plan.k_joint - plan.k_fwd) / 2 + (plan.n_st if plan.reverse else 0)
        extra = {"counted_per_issued": ((plan.k_joint - plan.k_fwd) / 2) / issued if plan.reverse else None,
                 "sm_fill": units / (-(-units // per_wave) * per_wave),
                 "bytes_fw_alg": bytes_fw_alg, "bytes_bw_alg": bytes_bw_alg, "traffic_bw": traffic_bw, "traffic_fw": traffic_fw,
                 "achieved_bw": elems * k_bw / (bw_avg * 1e-3) / 1e12, "flops_bw": elems * k_bw, "bw_name": bw_src.name,
                 "stream_mb": (traffic_fw + traffic_bw) / 1e6}
        return rec, extra

    # ---- end to end through the public API with host buffers ---------------------------------------------------
    def measure_e2e(self, op, xs_host, dy_host, dS_host, n_steps):
        """Pinned host buffers in, pinned host buffers out, copies inside the timed region.  Three streams, two
        buffer sets: the host->device copy of step i+1 and the device->host copy of step i-1 run beside the
        kernels of step i."""
        torch, dev, stream = self.torch, self.dev, self.stream
        pin = [x.detach().cpu().pin_memory() for x in xs_host]
        host_in = pin + [dy_host.pin_memory(), dS_host.pin_memory()]
        out_host = None
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        dev_in = [[torch.empty_like(p, device=dev) for p in host_in] for _ in range(2)]
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

        for i in range(4):
            e2e_step(i)
        self.sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(n_steps):
            e2e_step(i)
        stream.wait_stream(s_out)          # the last results must have reached the host
        stream.wait_stream(s_in)
        e1.record(stream)
        self.sync_all()
        ms = self.max_over_ranks(e0.elapsed_time(e1) / max(1, n_steps))
        h2d = sum(p.numel() * p.element_size() for p in host_in)
        d2h = sum(h.numel() * h.element_size() for h in out_host)
        return ms, h2d, d2h

    # ---- the scaling configuration ---------------------------------------------------------------------------------
    def scaling_c4(self, steps):
        """Gated Delta Rule, global batch 64, T4096 ("strong" scaling): every rank draws the same global batch on its
        GPU, keeps the rows ``shard.shard_args`` assigns to it and runs the single-GPU op on them; no collective."""
        from flex_rnn_b200 import shard
        from flex_rnn_b200 import workloads as W
        torch = self.torch
        opname, GB, T, H, M, N = WORKLOADS["gated_delta_rule_c4"]
        # the global batch, drawn on the device (same seed, hence the same values, on every rank), then cut
        xs_g, dy_g, dS_g = W.synthetic(opname, GB, T, H, M, N, torch.bfloat16, seed=1000, device=self.dev)
        ins, sts, (lo, hi) = shard.shard_args(xs_g[:-1], xs_g[-1:], self.rank, self.world)
        own = (lambda t: t) if self.world == 1 else (lambda t: t.contiguous().clone())
        xs = [own(t) for t in list(ins) + list(sts)]
        dy, dS = own(dy_g[lo:hi]), own(dS_g[lo:hi])
        del xs_g, dy_g, dS_g, ins, sts
        torch.cuda.empty_cache()
        B = hi - lo
        m = self.measure(opname, xs, dy, dS, steps, 2)
        rec, _ = self.analyse(opname, m, xs, B, T, H, M, N)
        rec["tokens_per_s"] = GB * T / (m["ms_per_step"] * 1e-3)
        rec.update({"workload": f"gated_delta_rule fwd+bwd, global B{GB} T{T} H{H} {M}x{N} bf16 I/O, {B} sequences per GPU",
                    "scaling": "strong", "n_gpus": self.world, "steps": steps, "global_batch": GB,
                    "sharding": "flex_rnn_b200.shard: contiguous batch rows per rank, no collective"})
        del m["op"]
        return rec


def run_ours(args, rank, world, local):
    import torch
    from flex_rnn_b200 import workloads as W
    bench = Bench(args, rank, world, local)
    dev = bench.dev
    opname, B, T, H, M, N = WORKLOADS[args.op]
    strong = args.op in STRONG and not args.batch
    if strong:
        assert B % world == 0, "the global batch must divide over the GPUs"
        B //= world
    big = B * T * H * N * 2 * 3 > 2e9
    no_e2e = args.no_e2e or big      # the host-buffer leg would pin several GB per buffer set: kept to the headline sizes
    # each rank draws its own shard of the global batch (seed offset by the rank)
    xs_host, dy_host, dS_host = W.synthetic(args.op if args.op in W.STEPS else opname, B, T, H, M, N, torch.bfloat16, seed=rank,
                                            device=dev if big else "cpu")
    xs = [x.to(dev) for x in xs_host]
    dy, dS = dy_host.to(dev), dS_host.to(dev)
    bench.probe_fp32_peak()
    fma_kinds = bench.probe_fma_kinds() if rank == 0 else {}
    m = bench.measure(opname, xs, dy, dS, args.steps, args.warmup, sample_clocks=True)
    rec, extra = bench.analyse(opname, m, xs, B, T, H, M, N)
    ms_per_step = m["ms_per_step"]
    value = world * B * T / (ms_per_step * 1e-3)

    e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    if not no_e2e:
        n_e2e = max(4, min(args.steps, 20))
        e2e_ms, h2d, d2h = bench.measure_e2e(m["op"], xs_host, dy_host, dS_host, n_e2e)
        e2e = {"value": world * B * T / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms, "steps": n_e2e,
               # per rank; all ranks copy through the same host at once, so this is what one GPU got of the host path
               "h2d_gbs_per_rank": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (e2e_ms * 1e-3) / 1e9,
               "host_path_gbs_all_ranks": world * (h2d + d2h) / (e2e_ms * 1e-3) / 1e9}

    fw_ms, bw_ms = m["fw_ms"], m["bw_ms"]
    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "fp32", "data": "synthetic",
            "config": {"workload": workload_text(args.op, B, T, H, M, N),
                       "io_dtype": "bf16", "math_dtype": "fp32", "global_batch": B * world, "seq_len": T,
                       "parallelism": f"batch shards x{world}, no collective",
                       "l2": f"no flush: each step streams {extra['stream_mb']:.0f} MB of inputs, outputs, checkpoints and row sums "
                             "through HBM (L2 is 126 MB)",
                       "checkpoint_every": rec["checkpoint_every"], "backward": rec["backward"],
                       "fw_kernel": rec["fw_kernel"], "bw_kernel": rec["bw_kernel"]},
            "fw_ms": rec["fw_ms"], "bw_ms": rec["bw_ms"],
            # spread of the per-step device time (forward + backward events of each timed step), rank 0
            "step_ms_p20_p50_p80": [round(sorted(f + b for f, b in zip(fw_ms, bw_ms))[int(q * (len(fw_ms) - 1))], 4)
                                    for q in (0.2, 0.5, 0.8)],
            "roofline_fraction_step": rec["roofline_fraction_step"],
            "roofline_fraction_fw": rec["roofline_fraction_fw"],
            "peak_memory_gib": rec["peak_memory_gib"],
            "roofline": {"bound": "fp32", "kernel": extra["bw_name"], "achieved": extra["achieved_bw"], "peak": bench.fp32_peak,
                         "unit": "TFLOP/s", "frac": extra["achieved_bw"] / bench.fp32_peak,
                         "traffic": extra["traffic_bw"],
                         "traffic_source": "computed from the plan (inputs, dy, dS_T, saved row sums and fp32 checkpoints read; "
                                           "gradients and dS0 written)",
                         "algorithmic_bytes": extra["bytes_bw_alg"],
                         "peak_source": f"measured in this run by the FMA probe kernel ({bench.sms} SMs); HBM copy peak {bench.hbm} GB/s "
                                        + ("of measured" if bench.peaks else "of fallback"),
                         "flops_per_launch": extra["flops_bw"], "k_joint": rec["k_joint"], "k_fwd": rec["k_fwd"],
                         "hbm_bound_ms": rec["hbm_bound_ms"], "fp32_bound_ms": rec["fp32_bound_ms"],
                         # what bounds `frac` below 1: the share of the FP32 peak that FMAs of the kernels' kinds reach in
                         # register-only loops (probe kernels of the library, measured now), the FMAs the kernel issues per
                         # counted one, and how evenly the (b,h) recurrences fill the SMs
                         "fp32_pipe_share_by_fma_kind": fma_kinds,
                         "counted_per_issued_fma": extra["counted_per_issued"],
                         "sm_fill": extra["sm_fill"],
                         "ceiling_frac": (fma_kinds.get("delta_rule_backward_mix_packed", 1.0) * extra["counted_per_issued"]
                                          * extra["sm_fill"]) if (args.op == "delta_rule" and fma_kinds) else None},
            "e2e": e2e,
            "gpu_launches": 2 * args.steps,
            "clocks": m["clocks"],
        }
    # release the headline workload before the further records allocate theirs
    del m, xs, dy, dS
    torch.cuda.empty_cache()

    if not args.no_extras:
        n_extra = max(3, min(args.steps, 20))
        if world == 1:
            others = {}
            for name in ("rwkv7", "mamba2", "gated_delta_rule"):
                if name == args.op:
                    continue
                o, b2, t2, h2, m2, n2 = WORKLOADS[name]
                xs2, dy2, dS2 = W.synthetic(o, b2, t2, h2, m2, n2, torch.bfloat16, seed=0)
                xs2 = [x.to(dev) for x in xs2]
                mm = bench.measure(o, xs2, dy2.to(dev), dS2.to(dev), n_extra, 3)
                r2, _ = bench.analyse(o, mm, xs2, b2, t2, h2, m2, n2)
                r2["workload"] = workload_text(name, b2, t2, h2, m2, n2)
                r2["steps"] = n_extra
                others[name] = r2
                del mm, xs2, dy2, dS2
                torch.cuda.empty_cache()
            line["workloads"] = others
        if args.op == "delta_rule" and not args.batch:
            c4 = bench.scaling_c4(max(2, min(args.steps, 5)))
            torch.cuda.empty_cache()
            if rank == 0:
                line["scaling_c4"] = c4
        if world == 1:
            line["reference_cuda"] = reference_cuda_record(args.op, n_extra)

    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            # one cold pass, then the mean of three; the same sample as one step of the reference arm
            heads = cpu_heads(H, T, 4)
            cpu_sample(opname, B, T, H, M, N, heads)
            runs = [cpu_sample(opname, B, T, H, M, N, heads) for _ in range(3)]
            base = runs[-1][0]
            mean_dt = sum(dt for _, dt in runs) / len(runs)
            base["value"] = base["value"] * runs[-1][1] / mean_dt
            base["sample"] = base["sample"].replace(f", {runs[-1][1]:.2f} s, scaled",
                                                    f", {mean_dt:.2f} s per pass (mean of 3 after one cold pass), scaled")
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if world > 1:
        bench.dist.barrier()
        bench.dist.destroy_process_group()


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
    ap.add_argument("--probe-only", action="store_true",
                    help="only run the library's FP32 probe kernels (peak and the scan kernels' kinds of FMA) and print their rates")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the records beside the headline (other workloads, scaling configuration, reference CUDA)")
    args = ap.parse_args()
    if args.batch:
        for k, w in list(WORKLOADS.items()):
            WORKLOADS[k] = (w[0], args.batch) + w[2:]
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.gpus != world:
        sys.exit(f"bench.py: --gpus {args.gpus} but {world} process(es) were launched; for N > 1 start it with "
                 f"`python -m torch.distributed.run --nnodes=1 --nproc-per-node {args.gpus} bench.py --gpus {args.gpus} ...`")
    if args.probe_only:
        b = Bench(args, rank, world, local)
        peak = b.probe_fp32_peak()
        print(json.dumps({"fp32_peak_tflops": peak, "sms": b.sms, "fp32_pipe_share_by_fma_kind": b.probe_fma_kinds()}), flush=True)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    elif args.impl == "reference_cuda":
        run_reference_cuda(args, rank, world, local)
    else:
        run_ours(args, rank, world, local)


if __name__ == "__main__":
    main()
