#!/usr/bin/env python
"""Benchmark of the attention forward + tangent (JVP) hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload C3|C2]

A step is one fused forward+tangent pass over one batch of seeded synthetic
tensors with the shapes of the named configuration (default C3: SiT-XL/2 512px,
B=64, H=16, N=1024, D=72, q/k RMS-normalised, tangents N(0,1)*0.1).  One process
per GPU; with N > 1 (launched by torch.distributed.run) every rank runs the same
per-GPU workload on its own batch shard - the op has no collective - and the
reported value is the units all ranks processed divided by the slowest rank's
device time ("weak" scaling).

Rank 0 prints ONE JSON line.  `value` is kernel throughput with inputs resident in
HBM; `e2e` is the same metric through the public API (flash_attn_func under
torch.func.jvp) with pinned host buffers, host<->device copies inside the timed
region; `roofline` relates the kernel to the measured bf16 peak; `cpu_baseline`
is the CPU oracle (the reference's 'base' attention under torch.func.jvp, fp32)
timed on this host on a bounded sample.

The default line carries more than the headline, all measured in the same process:
`roofline.sustained` (the same launch looped for about two seconds, with the SM clock it ran at),
`secondary` (plain forward, primal backward, the C2 shapes, the q/k norm and adaLN ops), `c4` and
`c5` (DMFT-XL/2 training step and 4-step sampling on all N GPUs: the data-parallel path with its
gradient all-reduce) and `gpu_comparator` (the reference's own GPU kernels - its Triton dual kernel
and the FlashAttention-2 forward / backward it calls - timed in a child process on the same GPU).

--impl reference times the reference's CPU path alone (all host threads), on the same metric and
config, each step a bounded sample of the workload.  --impl reference-gpu is the child process
behind `gpu_comparator`: it needs the reference's three attention files under baseline/_ref/models
(put there by __graft_entry__.build() where the reference tree is present) and prints
{"impl": "reference-gpu", "unavailable": ...} when they, Triton or flash_attn cannot be used.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "attn_jvp_fwd_tangent_tflops"
UNIT = "TFLOP/s"

WORKLOADS = {
    # name: (B, L, H, D, tangent_scale, qk_norm, description)
    "C3": (64, 1024, 16, 72, 0.1, True, "attention JVP fwd+tangent, SiT-XL/2 512px: B=64 H=16 N=1024 D=72, qk-norm"),
    "C2": (256, 256, 16, 72, 0.1, False, "attention JVP fwd+tangent, SiT-XL/2 256px: B=256 H=16 N=256 D=72"),
}
CPU_SAMPLE_BATCH = 2  # batch slice of the workload one CPU step computes
CPU_SAMPLE_SECONDS = 12.0  # CPU work the cpu_baseline leg aims for


def _flops(B, L, H, D):
    return 12.0 * B * H * L * L * D


def _algo_bytes(B, L, H, D):
    return 16.0 * B * L * H * D + 4.0 * B * H * L


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def _kernel_name(op, D, L):
    """The kernel instance the library's launcher picks for this shape, asked of the library itself."""
    from dmf_b200 import _lib
    return _lib.kernel_name(op, L, L, D)


def _traffic(workload):
    """DRAM bytes per launch from the committed ncu capture of this kernel (not measured by this run), or None."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if p.exists():
        d = json.loads(p.read_text()).get(workload, {})
        return (d.get("dram_bytes_per_launch"),
                f"profiles/dram_traffic.json: ncu capture at batch {d.get('captured_at_batch')} x {d.get('scale')}, "
                "not measured by this run")
    return None, None


def _nvml_handle(nv, dev_index):
    """NVML handle of torch's CUDA device ``dev_index``: NVML numbers all GPUs of the machine and ignores
    CUDA_VISIBLE_DEVICES, so the device is looked up by its UUID."""
    import torch
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev_index).uuid)
        return nv.nvmlDeviceGetHandleByUUID(uuid), uuid
    except Exception:
        return nv.nvmlDeviceGetHandleByIndex(dev_index), None


def _pin_to_gpu_numa_node(dev_index):
    """Run this process (and place its pinned host buffers) on the CPUs NVML lists as local to the GPU.  Read-only
    query; returns the number of CPUs in the set, or None when it cannot be had."""
    try:
        import pynvml as nv
        nv.nvmlInit()
        h, _ = _nvml_handle(nv, dev_index)
        words = nv.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


class ClockSampler(threading.Thread):
    """Reads (never sets) SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.001):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz, self.uuid = [], set(), None, None
        self._stop_evt = threading.Event()
        self.active = threading.Event()
        self.ready = threading.Event()
        self.error = None

    def start(self):
        """Start the thread and wait until NVML answers (its first call can take longer than a short timed region)."""
        super().start()
        self.ready.wait(timeout=15)

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h, self.uuid = _nvml_handle(nv, self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)  # the first read is the slow one
            self.ready.set()
            names = {
                "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
                "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
            }
            def read_reasons():
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)

            n, was_active = 0, False
            while not self._stop_evt.is_set():
                if self.active.is_set():
                    # the clock every time round (one NVML call: a short timed region still gets several samples),
                    # the throttle reasons every fourth time and once more when the window closes
                    self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                    if n % 4 == 0:
                        read_reasons()
                    n, was_active = n + 1, True
                elif was_active:
                    read_reasons()
                    n, was_active = 0, False
                time.sleep(self.period)
        except Exception as e:  # NVML missing: report, do not fail the bench
            self.error = repr(e)
        finally:
            self.ready.set()

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s), "gpu_uuid": self.uuid,
                **({"error": self.error} if self.error else {})}

    def window(self):
        """Start a fresh measurement window (the thread keeps running)."""
        self.samples, self.reasons = [], set()


def _cpu_step_fn(workload, batch):
    """The CPU oracle on a batch slice of the workload; returns (callable, flops per call)."""
    import torch
    from oracle import attn_jvp_oracle as orc
    B, L, H, D, ts, qkn, _ = WORKLOADS[workload]
    ins = orc.make_inputs(batch, L, H, D, seed=0, tangent_scale=ts, qk_norm=qkn)

    def step():
        with torch.no_grad():
            return orc.attn_jvp_base(*ins)

    return step, _flops(batch, L, H, D)


def _time_cpu(step, n_steps, warmup):
    for _ in range(warmup):
        step()
    ts = []
    for _ in range(n_steps):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    return ts


def run_reference(args):
    """The reference's CPU implementation of the path (oracle port), all host threads, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    B, L, H, D, ts, qkn, desc = WORKLOADS[args.workload]
    step, fl = _cpu_step_fn(args.workload, CPU_SAMPLE_BATCH)
    times = _time_cpu(step, args.steps, args.warmup)
    total = sum(times)
    value = fl * len(times) / total / 1e12
    sample = (f"batch slice B={CPU_SAMPLE_BATCH} of {args.workload} per step ({fl / 1e9:.1f} GFLOP), fp32, "
              f"'base' attention under torch.func.jvp")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {desc}", "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _make_attn_inputs(workload, batch, dev, seed):
    """Seeded synthetic inputs of a workload on the device: (q, k, v, tq, tk, tv), in the layout the model's
    attention block produces (strided views of the packed projection; q, k contiguous after a qk-norm)."""
    import torch
    B, L, H, D, ts, qkn, _ = WORKLOADS[workload]
    B = batch or B
    gen = torch.Generator(device=dev).manual_seed(seed)
    qkv = torch.randn(B, L, 3, H, D, device=dev, dtype=torch.float32, generator=gen)
    tqkv = torch.randn(B, L, 3, H, D, device=dev, dtype=torch.float32, generator=gen) * ts
    if qkn:
        # per-head RMSNorm of q, k and the matching tangents (weight = 1, eps = 1e-6)
        def norm_jvp(x, tx):
            r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
            return x * r, tx * r - x * r.pow(3) * (x * tx).mean(-1, keepdim=True)
        q, tq = norm_jvp(qkv[:, :, 0], tqkv[:, :, 0])
        k, tk = norm_jvp(qkv[:, :, 1], tqkv[:, :, 1])
        q, k, tq, tk = (x.to(torch.bfloat16).contiguous() for x in (q, k, tq, tk))
    else:
        qkv16, tqkv16 = qkv.to(torch.bfloat16), tqkv.to(torch.bfloat16)
        q, k, tq, tk = qkv16[:, :, 0], qkv16[:, :, 1], tqkv16[:, :, 0], tqkv16[:, :, 1]
    v = qkv.to(torch.bfloat16)[:, :, 2]
    tv = tqkv.to(torch.bfloat16)[:, :, 2]
    return (q, k, v, tq, tk, tv), gen


def _time_launches(fn, steps, warmup=3):
    """Milliseconds per call of ``fn`` on torch's current stream: CUDA events around ``steps`` back-to-back calls."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _attn_roofline(op, B, L, H, D, ms, peaks):
    """The bound of an attention op at this shape (the higher of its tensor-time and HBM-time floors at the measured
    peaks) and the fraction of it that ``ms`` per launch reaches."""
    fl = {"dual": 12.0, "fwd": 4.0, "bwd": 10.0}[op] * B * H * L * L * D
    # dual: read 6 tensors, write 2 (+ lse); fwd: read 3, write 1 (+ lse); bwd: read 5 (+ lse), write 3
    nbytes = {"dual": 16.0, "fwd": 8.0, "bwd": 16.0}[op] * B * L * H * D + 4.0 * B * H * L
    tf, gbs = fl / (ms * 1e-3) / 1e12, nbytes / (ms * 1e-3) / 1e9
    hbm_bound = nbytes / (peaks["hbm_gbs"] * 1e9) > fl / (peaks["tflops"] * 1e12)
    return {"bound": "hbm" if hbm_bound else "tensor", "flops": fl, "bytes": nbytes, "tflops": tf, "gbs": gbs,
            "frac": gbs / peaks["hbm_gbs"] if hbm_bound else tf / peaks["tflops"]}


def _launches_per_call(op: str, L: int, D: int) -> int:
    """Kernels of this library that one call of the op launches (a memset of the one-pass backward is not counted)."""
    if op != "bwd":
        return 1
    return _kernel_name("bwd", D, L).count(" + ") + 1      # the entry point names its kernels joined by " + "


def _secondary(dev, peaks, steps):
    """The other kernels of the path at the shapes the model runs them at, a second or so each: value and fraction of
    the roofline that bounds each (of the measured peaks)."""
    import torch
    from dmf_b200 import adaln, ops
    out = {}
    for wl in ("C3", "C2"):
        B, L, H, D, ts, _, _ = WORKLOADS[wl]
        (q, k, v, tq, tk, tv), gen = _make_attn_inputs(wl, None, dev, 7)
        scale = D ** -0.5
        o, lse = ops.fwd_raw(q, k, v, scale)
        dout = torch.randn(B, L, H, D, device=dev, generator=gen).to(torch.bfloat16)
        runs = {"fwd": lambda: ops.fwd_raw(q, k, v, scale), "bwd": lambda: ops.bwd_raw(dout, q, k, v, o, lse, scale)}
        if wl != "C3":
            runs["dual"] = lambda: ops.fwd_dual_raw(q, k, v, tq, tk, tv, scale)
        for op, fn in runs.items():
            ms = _time_launches(fn, steps)
            r = _attn_roofline(op, B, L, H, D, ms, peaks)
            out[f"{wl}_{op}"] = {"ms": ms, "tflops": r["tflops"], "gbs": r["gbs"], "bound": r["bound"], "frac": r["frac"],
                                 "kernel": _kernel_name(op, D, L)}
        if wl == "C3":
            # q / k RMS norm with tangents on the packed projection, and the adaLN ops of one block with tangents
            qkv = torch.randn(B, L, 3, H, D, device=dev, generator=gen).to(torch.bfloat16)
            tqkv = (torch.randn(B, L, 3, H, D, device=dev, generator=gen) * ts).to(torch.bfloat16)
            w = torch.ones(D, device=dev)

            def rms():
                ops.rmsnorm_fwd_raw(qkv[:, :, 0], tqkv[:, :, 0], w, 1e-6)
                ops.rmsnorm_fwd_raw(qkv[:, :, 1], tqkv[:, :, 1], w, 1e-6)

            ms = _time_launches(rms, steps)
            nbytes = 2 * 4 * B * L * H * D * 2.0
            out["C3_qk_rmsnorm_dual"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "bound": "hbm",
                                         "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"]}
            del qkv, tqkv
            Cn = H * D
            rn = lambda *sh: torch.randn(*sh, device=dev, generator=gen)
            x, tx = rn(B, L, Cn), rn(B, L, Cn) * ts
            h, th = rn(B, L, Cn).to(torch.bfloat16), (rn(B, L, Cn) * ts).to(torch.bfloat16)
            mods, tmods = (0.3 * rn(B, 1, 6 * Cn)).to(torch.bfloat16), (0.03 * rn(B, 1, 6 * Cn)).to(torch.bfloat16)
            sh_a, sc_a, g_a, sh_m, sc_m, g_m = mods.chunk(6, dim=-1)
            tsh_a, tsc_a, tg_a, tsh_m, tsc_m, tg_m = tmods.chunk(6, dim=-1)

            def block():
                adaln.ln_modulate_fwd_raw(x, tx, sh_a, sc_a, tsh_a, tsc_a, 1e-6, torch.bfloat16)
                adaln.gate_residual_fwd_raw(x, tx, h, th, g_a, tg_a)
                adaln.ln_modulate_fwd_raw(x, tx, sh_m, sc_m, tsh_m, tsc_m, 1e-6, torch.bfloat16)
                adaln.gate_residual_fwd_raw(x, tx, h, th, g_m, tg_m)

            ms = _time_launches(block, steps)
            nbytes = 2.0 * B * L * Cn * (12 + 20)
            out["C3_adaln_block_dual"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "bound": "hbm",
                                          "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"]}
            del x, tx, h, th
        del q, k, v, tq, tk, tv, o, lse, dout
        torch.cuda.empty_cache()
    return out


class _E2EPipeline:
    """The op through the public API from pinned host buffers, as a user streaming a batch would run it: the batch is
    cut into chunks along B; chunk i+1 is copied in (one stream) while chunk i computes (second stream) and chunk i-1
    is copied out (third stream), with two sets of device buffers.  One copy_ per tensor per chunk."""

    def __init__(self, ins, dev, chunks):
        import torch
        self.torch, self.dev = torch, dev
        B = ins[0].shape[0]
        self.chunks = max(1, min(chunks, B))
        while B % self.chunks:
            self.chunks -= 1
        self.bc = B // self.chunks
        self.host_in = [x.contiguous().cpu().pin_memory() for x in ins]
        shape = tuple(ins[0].shape)
        self.host_out = [torch.empty(shape, dtype=ins[0].dtype).pin_memory() for _ in range(2)]
        cshape = (self.bc,) + shape[1:]
        self.dev_in = [[torch.empty(cshape, dtype=ins[0].dtype, device=dev) for _ in range(6)] for _ in range(2)]
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        self.h2d = sum(x.numel() * x.element_size() for x in self.host_in)
        self.d2h = sum(x.numel() * x.element_size() for x in self.host_out)

    def step(self):
        torch = self.torch
        from dmf_b200 import flash_attn_func
        cur = torch.cuda.current_stream(self.dev)
        for st in (self.s_in, self.s_cmp, self.s_out):
            st.wait_stream(cur)
        computed = [None, None]     # per buffer set: event "the op that read this set has run"
        keep = []
        for c in range(self.chunks):
            slot, lo = c % 2, c * self.bc
            with torch.cuda.stream(self.s_in):
                if computed[slot] is not None:
                    self.s_in.wait_event(computed[slot])
                for h, d in zip(self.host_in, self.dev_in[slot]):
                    d.copy_(h[lo:lo + self.bc], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(ready)
                d = self.dev_in[slot]
                o, do = torch.func.jvp(lambda a, b, cc: flash_attn_func(a, b, cc), tuple(d[:3]), tuple(d[3:]))
                done = torch.cuda.Event()
                done.record(self.s_cmp)
                computed[slot] = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                self.host_out[0][lo:lo + self.bc].copy_(o, non_blocking=True)
                self.host_out[1][lo:lo + self.bc].copy_(do, non_blocking=True)
                o.record_stream(self.s_out)
                do.record_stream(self.s_out)
            keep.append((o, do))
        for st in (self.s_in, self.s_cmp, self.s_out):
            cur.wait_stream(st)


def _run_comparator(args):
    """The reference's own GPU kernels on this GPU, in a child process (Triton and flash_attn never load into this
    one).  Returns the child's record, or why there is none."""
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference-gpu", "--steps", str(min(args.steps, 20))]
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the comparator child process did not finish within 600 s"}
    for line in reversed(res.stdout.strip().splitlines()):
        try:
            rec = json.loads(line)
        except ValueError:
            continue
        if rec.get("impl") == "reference-gpu":
            rec.pop("impl")
            return rec
    return {"unavailable": f"child exited {res.returncode}: {(res.stderr or res.stdout).strip()[-400:]}"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the sm_100a kernels have no CPU path "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa_cpus = _pin_to_gpu_numa_node(local_rank)     # before any pinned host buffer is allocated
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev, timeout=__import__("datetime").timedelta(seconds=900))

    from dmf_b200 import ops

    B, L, H, D, ts, qkn, desc = WORKLOADS[args.workload]
    if args.batch is not None:
        B, desc = args.batch, desc + f" [batch overridden to {args.batch}: not a bench line]"
    scale = D ** -0.5
    # seeded synthetic inputs, per-rank shard of the data-parallel batch (seed = rank)
    ins, gen = _make_attn_inputs(args.workload, B, dev, rank)
    q, k, v, tq, tk, tv = ins
    in_bytes = sum(x.numel() * x.element_size() for x in ins)

    # --op selects the entry point: the fused forward+tangent (the bench line), the plain forward, or the
    # primal backward (both launches); flops and bytes follow the op
    op = args.op
    if op == "bwd":
        o_saved, lse_saved = ops.fwd_raw(q, k, v, scale)
        dout = torch.randn(B, L, H, D, device=dev, dtype=torch.float32, generator=gen).to(torch.bfloat16)

    def step():
        if op == "dual":
            return ops.fwd_dual_raw(*ins, scale)
        if op == "fwd":
            return ops.fwd_raw(q, k, v, scale)
        return ops.bwd_raw(dout, q, k, v, o_saved, lse_saved, scale)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(args.warmup, 3)):
        out = step()
    sync_all()

    sampler = ClockSampler(local_rank)
    sampler.start()
    stream = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    sampler.active.set()
    e0.record(stream)
    for _ in range(args.steps):
        out = step()
    e1.record(stream)
    sync_all()
    sampler.active.clear()
    clocks = sampler.summary()
    ms_step = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    ops.check_device_status(dev)
    peaks = _peaks()
    roof = _attn_roofline(op, B, L, H, D, ms_step, peaks)
    fl = roof["flops"]
    value = world * fl / (ms_step * 1e-3) / 1e12

    # ---- the same launch back to back for about two seconds: what the power cap leaves of the burst figure ----
    sustained = None
    if not args.no_sustained and world == 1:
        n_sus = int(min(20000, max(args.steps, 2000.0 / ms_step)))
        sampler.window()
        sampler.active.set()
        e0.record(stream)
        for _ in range(n_sus):
            step()
        e1.record(stream)
        torch.cuda.synchronize()
        sampler.active.clear()
        sc = sampler.summary()
        ms_sus = e0.elapsed_time(e1) / n_sus
        tf_sus = fl / (ms_sus * 1e-3) / 1e12
        sustained = {"launches": n_sus, "seconds": ms_sus * n_sus / 1e3, "ms_per_launch": ms_sus, "tflops": tf_sus,
                     "frac_of_sustained_peak": tf_sus / peaks["tflops_sustained"] if peaks["tflops_sustained"] else None,
                     "frac_of_burst_peak": tf_sus / peaks["tflops"],
                     "sm_mhz_median": sc["sm_mhz"], "reasons": sc["reasons"],
                     "cycles_per_launch": (ms_sus * 1e-3 * sc["sm_mhz"] * 1e6) if sc["sm_mhz"] else None,
                     "burst_cycles_per_launch": (ms_step * 1e-3 * clocks["sm_mhz"] * 1e6) if clocks["sm_mhz"] else None}
        ops.check_device_status(dev)

    # ---- end to end through the public API, host buffers, copies inside the timed region ----
    e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    if not args.no_e2e and op == "dual":
        e2e_steps = max(3, min(args.steps, 10))
        pipe = _E2EPipeline(ins, dev, args.e2e_chunks)
        for _ in range(2):
            pipe.step()
        sync_all()
        e0.record(stream)
        for _ in range(e2e_steps):
            pipe.step()
        e1.record(stream)
        sync_all()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
        e2e = {"value": world * fl / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": pipe.h2d,
               "d2h_bytes_per_step": pipe.d2h, "steps": e2e_steps, "ms_per_step": e2e_ms,
               "h2d_gbs_per_gpu": pipe.h2d / e2e_ms / 1e6, "d2h_gbs_per_gpu": pipe.d2h / e2e_ms / 1e6,
               "api": "torch.func.jvp(dmf_b200.flash_attn_func) on pinned host tensors",
               "pipeline": f"{pipe.chunks} chunks of {pipe.bc} along the batch; host-to-device copy, op and "
                           "device-to-host copy on three streams, two sets of device buffers",
               "numa_local_cpus": numa_cpus}
        del pipe
        ops.check_device_status(dev)
    sampler.stop()

    traffic, traffic_src = _traffic(args.workload) if (op == "dual" and args.batch is None) else (None, None)
    roofline = {
        "bound": roof["bound"],
        "achieved": roof["gbs"] if roof["bound"] == "hbm" else roof["tflops"],
        "peak": peaks["hbm_gbs"] if roof["bound"] == "hbm" else peaks["tflops"],
        "unit": "GB/s" if roof["bound"] == "hbm" else "TFLOP/s",
        "frac": roof["frac"],
        "traffic": traffic, "traffic_source": traffic_src,
        "peak_source": f"{'HBM copy' if roof['bound'] == 'hbm' else 'bf16 burst'}, of {peaks['source']}",
        "tflops_achieved": roof["tflops"], "frac_of_burst_tflops": roof["tflops"] / peaks["tflops"],
        "frac_of_sustained": (roof["tflops"] / peaks["tflops_sustained"]) if peaks["tflops_sustained"] else None,
        "frac_of_nominal_2250": roof["tflops"] / 2250.0,
        "algorithmic_flops_per_launch": fl, "algorithmic_bytes_per_launch": roof["bytes"],
        "hbm_gbs_achieved": roof["gbs"], "frac_of_hbm": roof["gbs"] / peaks["hbm_gbs"],
        "kernel": _kernel_name(op, D, L),
        "sustained": sustained,
    }
    del ins, q, k, v, tq, tk, tv, out
    if op == "bwd":
        del o_saved, lse_saved, dout
    gc.collect()
    torch.cuda.empty_cache()

    secondary = comparator = None
    if world == 1 and op == "dual" and args.batch is None:
        if not args.no_secondary:
            secondary = _secondary(dev, peaks, min(args.steps, 30))
            ops.check_device_status(dev)
        if not args.no_comparator:
            comparator = _run_comparator(args)

    # ---- the whole-model configurations on all N GPUs: C5 (sampling, no collective), C4 (training, all-reduce) ----
    c4 = c5 = None
    if op == "dual" and args.batch is None and not args.no_model:
        c5 = _model_record_in_children(args, "C5", world, rank, local_rank, 1)
        sync_all()
        c4 = _model_record_in_children(args, "C4", world, rank, local_rank, 2)
        sync_all()

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and op == "dual":
        cores = os.cpu_count() or 1
        try:
            os.sched_setaffinity(0, range(cores))     # the CPU leg may use every core again
        except OSError:
            pass
        torch.set_num_threads(cores)
        cstep, cfl = _cpu_step_fn(args.workload, CPU_SAMPLE_BATCH)
        t0 = time.perf_counter()
        first = _time_cpu(cstep, 1, 1)[0]
        n_cpu = int(min(5000, max(5, round(CPU_SAMPLE_SECONDS / max(first, 1e-3)))))
        times = _time_cpu(cstep, n_cpu, 0)
        cpu_base = {
            "value": cfl * len(times) / sum(times) / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"{n_cpu} runs of a B={CPU_SAMPLE_BATCH} batch slice of {args.workload} ({cfl / 1e9:.1f} GFLOP each), "
                      f"fp32 'base' attention under torch.func.jvp, {time.perf_counter() - t0:.1f} s of CPU work",
        }

    if rank == 0:
        line = {
            "metric": METRIC if op == "dual" else f"attn_{op}_tflops", "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {desc}", "per_gpu_batch": B,
                       "l2": f"inputs ({in_bytes / 1e6:.0f} MB per GPU) are larger than the 126 MB L2; no flush between steps",
                       "layout": "q,k contiguous after qk-norm; v and tangents strided views of packed qkv"
                                 if qkn else "strided views of packed qkv"},
            "roofline": roofline,
            "op": op,
            "cpu_baseline": cpu_base,
            "e2e": e2e,
            "gpu_launches": args.steps * _launches_per_call(op, L, D),
            "clocks": clocks,
            "secondary": secondary,
            "gpu_comparator": comparator,
            "c4": c4, "c5": c5,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_reference_gpu(args):
    """Bench-only comparator: the reference's own GPU path for this op on this GPU - its Triton kernel
    _attn_fwd_dual(_split) (models/triton_utils.py:258-500) behind FlashAttnFunc.forward's dual branch, and the
    FlashAttention-2 forward / backward it calls for the plain forward and the primal backward
    (models/flash_attention_2_jvp.py:47-61, 119-139) - driven through the reference's stock FlashAttnFunc and
    _flash_attn_backward, on the same inputs and with the same CUDA-event protocol as this package's kernels.
    Nothing of this package runs here, and nothing of this runs in the product process."""
    def bail(why):
        print(json.dumps({"impl": "reference-gpu", "unavailable": why[:600]}), flush=True)

    ref = ROOT / "baseline" / "_ref"
    if not (ref / "models" / "flash_attention_2_jvp.py").exists():
        return bail("baseline/_ref/models/flash_attention_2_jvp.py is missing (the reference tree was not present when "
                    "the package was built)")
    try:
        import torch
        if not torch.cuda.is_available():
            return bail("no CUDA device")
        sys.path.insert(0, str(ref))
        import models.flash_attention_2_jvp as R
    except Exception as e:
        return bail(f"import of the reference module failed: {type(e).__name__}: {e}")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    from importlib import metadata

    def version(pkg):
        try:
            return metadata.version(pkg)
        except Exception:
            return None

    rec = {"impl": "reference-gpu", "triton": version("triton"), "flash_attn": version("flash_attn"),
           "api": "models.flash_attention_2_jvp.FlashAttnFunc / _flash_attn_backward (unmodified copy of the reference files)"}
    peaks = _peaks()
    for wl in ("C3", "C2"):
        B, L, H, D, ts, _, _ = WORKLOADS[wl]
        (q, k, v, tq, tk, tv), gen = _make_attn_inputs(wl, None, dev, 0)
        dout = torch.randn(B, L, H, D, device=dev, generator=gen).to(torch.bfloat16)
        scale = D ** -0.5
        legs = {}

        def timed(name, op, fn):
            try:
                with torch.no_grad():
                    ms = _time_launches(fn, args.steps, 3)
                r = _attn_roofline(op, B, L, H, D, ms, peaks)
                legs[name] = {"ms": ms, "tflops": r["tflops"], "gbs": r["gbs"]}
            except Exception as e:
                legs[name] = {"unavailable": f"{type(e).__name__}: {e}"[:400]}
                try:
                    torch.cuda.synchronize()
                except Exception:
                    pass

        timed("triton_dual", "dual", lambda: R.FlashAttnFunc.apply(q, k, v, tq, tk, tv, None))
        timed("fa2_fwd", "fwd", lambda: R.FlashAttnFunc.apply(q, k, v, None, None, None, None))
        try:
            with torch.no_grad():
                o, m, _ = R.FlashAttnFunc.apply(q, k, v, None, None, None, None)
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            timed("fa2_bwd", "bwd", lambda: R._flash_attn_backward(dout, q, k, v, o, m, dq, dk, dv, 0.0, scale, False,
                                                                   -1, -1, 0.0, None, False))
        except Exception as e:
            legs["fa2_bwd"] = {"unavailable": f"{type(e).__name__}: {e}"[:400]}
        rec[wl] = legs
        del q, k, v, tq, tk, tv, dout
        torch.cuda.empty_cache()
    print(json.dumps(rec), flush=True)


def _cpu_port_gbs(fn, nbytes, what, seconds=6.0):
    """cpu_baseline of a memory-bound op: ``fn`` (the reference formulas under torch.func.jvp, fp32, all host threads)
    timed for about ``seconds``; GB/s of the same algorithmic bytes the GPU figure counts."""
    import torch
    torch.set_num_threads(os.cpu_count() or 1)
    first = _time_cpu(fn, 1, 1)[0]
    n = int(min(2000, max(3, round(seconds / max(first, 1e-3)))))
    times = _time_cpu(fn, n, 0)
    return {"value": nbytes * len(times) / sum(times) / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
            "kind": "port", "sample": f"{n} runs of {what}, {sum(times):.1f} s of CPU work"}


def _e2e_gbs(host_in, run, n_out_bytes, nbytes, steps, dev):
    """The same op from pinned host buffers: host-to-device copies of the inputs, the op, device-to-host copies of
    the results, all inside the timed region."""
    import torch
    outs_host = None

    def step():
        nonlocal outs_host
        outs = run([t.to(dev, non_blocking=True) for t in host_in])
        if outs_host is None:
            outs_host = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        for h, o in zip(outs_host, outs):
            h.copy_(o, non_blocking=True)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms,
            "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host_in), "d2h_bytes_per_step": n_out_bytes}


def run_rmsnorm(args):
    """The fused per-head RMS norm of q and k with tangents (one of the callers either side of the attention op):
    a step normalises q and k of a packed qkv projection of the workload's shape, with their tangents."""
    import torch
    from dmf_b200 import ops
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, L, H, D, ts, _, desc = WORKLOADS[args.workload]
    if args.batch is not None:
        B = args.batch
    gen = torch.Generator(device=dev).manual_seed(rank)
    qkv = torch.randn(B, L, 3, H, D, device=dev, generator=gen).to(torch.bfloat16)
    tqkv = (torch.randn(B, L, 3, H, D, device=dev, generator=gen) * ts).to(torch.bfloat16)
    w = torch.ones(D, device=dev)

    def step():
        ops.rmsnorm_fwd_raw(qkv[:, :, 0], tqkv[:, :, 0], w, 1e-6)
        return ops.rmsnorm_fwd_raw(qkv[:, :, 1], tqkv[:, :, 1], w, 1e-6)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(dev.index)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.active.set()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    sampler.active.clear()
    sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    nbytes = 2 * 4 * B * L * H * D * 2.0  # q and k: read x, tx; write y, ty
    gbs = nbytes / (ms * 1e-3) / 1e9
    peaks = _peaks()
    cpu_base = e2e = None
    if not args.no_e2e:
        host = [t.contiguous().cpu().pin_memory() for t in (qkv[:, :, 0], qkv[:, :, 1], tqkv[:, :, 0], tqkv[:, :, 1])]

        def run(d):
            y0, t0 = ops.rmsnorm_fwd_raw(d[0], d[2], w, 1e-6)
            y1, t1 = ops.rmsnorm_fwd_raw(d[1], d[3], w, 1e-6)
            return [y0, t0, y1, t1]

        e2e = _e2e_gbs(host, run, int(nbytes // 2), nbytes, min(args.steps, 10), dev)
    if not args.no_cpu_baseline:
        from oracle import attn_jvp_oracle as orc  # cpu_baseline leg only
        cq, ctq = torch.randn(2, L, H, D), ts * torch.randn(2, L, H, D)
        ck, ctk = torch.randn(2, L, H, D), ts * torch.randn(2, L, H, D)
        cw = torch.ones(D)

        def cstep():
            with torch.no_grad():
                torch.func.jvp(lambda a: orc.rms_norm(a, cw), (cq,), (ctq,))
                return torch.func.jvp(lambda a: orc.rms_norm(a, cw), (ck,), (ctk,))

        cpu_base = _cpu_port_gbs(cstep, nbytes * 2 / B, f"a B=2 batch slice of {args.workload}: the reference's RMSNorm "
                                 "form (models/layers.py:39-42) under torch.func.jvp, fp32")
    if rank == 0:
        print(json.dumps({
            "metric": "qk_rmsnorm_dual_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload} shapes: per-head RMS norm of q and k with tangents, strided views "
                                   f"of packed (B={B}, L={L}, 3, H={H}, D={D}) projections",
                       "l2": "inputs are larger than the 126 MB L2; no flush between steps"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                         "peak_source": f"HBM copy, of {peaks['source']}", "algorithmic_bytes_per_step": nbytes,
                         "kernel": "rmsnorm_fwd_kernel<bf16, dual> x 2"},
            "cpu_baseline": cpu_base, "e2e": e2e,
            "op": "rmsnorm", "gpu_launches": 2 * args.steps, "clocks": sampler.summary()}))


def run_adaln(args):
    """The adaLN-Zero elementwise ops of one DiT block with tangents, at the workload's token count and the model
    width H*D: a step is the block's two LayerNorm-modulates and two gate-residuals (fp32 stream, bf16 matmul side,
    as in training under bf16 autocast)."""
    import torch
    from dmf_b200 import adaln
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, L, H, D, ts, _, desc = WORKLOADS[args.workload]
    if args.batch is not None:
        B = args.batch
    Cn = H * D
    gen = torch.Generator(device=dev).manual_seed(rank)
    rn = lambda *s: torch.randn(*s, device=dev, generator=gen)
    x, tx = rn(B, L, Cn), rn(B, L, Cn) * ts
    h, th = rn(B, L, Cn).to(torch.bfloat16), (rn(B, L, Cn) * ts).to(torch.bfloat16)
    mods, tmods = (0.3 * rn(B, 1, 6 * Cn)).to(torch.bfloat16), (0.03 * rn(B, 1, 6 * Cn)).to(torch.bfloat16)
    sh_a, sc_a, g_a, sh_m, sc_m, g_m = mods.chunk(6, dim=-1)
    tsh_a, tsc_a, tg_a, tsh_m, tsc_m, tg_m = tmods.chunk(6, dim=-1)
    per = {}

    def ln(sh, sc, tsh, tsc):
        return adaln.ln_modulate_fwd_raw(x, tx, sh, sc, tsh, tsc, 1e-6, torch.bfloat16)

    def gate(g, tg):
        return adaln.gate_residual_fwd_raw(x, tx, h, th, g, tg)

    def step():
        ln(sh_a, sc_a, tsh_a, tsc_a)
        gate(g_a, tg_a)
        ln(sh_m, sc_m, tsh_m, tsc_m)
        return gate(g_m, tg_m)

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    n_el = B * L * Cn
    ln_bytes = n_el * (4 + 4 + 2 + 2.0)        # x, tx fp32 in; y, ty bf16 out
    gate_bytes = n_el * (4 + 4 + 2 + 2 + 4 + 4.0)  # x, tx fp32, h, th bf16 in; out, tout fp32 out
    for _ in range(max(args.warmup, 3)):
        step()
    per["ln_modulate_dual_gbs"] = ln_bytes / (timed(lambda: ln(sh_a, sc_a, tsh_a, tsc_a), args.steps) * 1e-3) / 1e9
    per["gate_residual_dual_gbs"] = gate_bytes / (timed(lambda: gate(g_a, tg_a), args.steps) * 1e-3) / 1e9
    # the primal backwards (not part of the timed step): dy bf16, x fp32 in, dx fp32 out / dout fp32, h bf16 in, dh bf16 out
    dy = rn(B, L, Cn).to(torch.bfloat16)
    per["ln_modulate_bwd_gbs"] = n_el * 10.0 / (timed(lambda: adaln.ln_modulate_bwd_raw(dy, x, sc_a, 1e-6), args.steps) * 1e-3) / 1e9
    per["gate_residual_bwd_gbs"] = n_el * 8.0 / (timed(lambda: adaln.gate_residual_bwd_raw(x, h, g_a), args.steps) * 1e-3) / 1e9
    sampler = ClockSampler(dev.index)
    sampler.start()
    sampler.active.set()
    ms = timed(step, args.steps)
    sampler.active.clear()
    sampler.stop()
    nbytes = 2 * (ln_bytes + gate_bytes)
    gbs = nbytes / (ms * 1e-3) / 1e9
    peaks = _peaks()
    cpu_base = e2e = None
    if not args.no_e2e:
        host = [t.cpu().pin_memory() for t in (x, tx, h, th)]

        def run(d):
            y, ty = adaln.ln_modulate_fwd_raw(d[0], d[1], sh_a, sc_a, tsh_a, tsc_a, 1e-6, torch.bfloat16)
            o, to = adaln.gate_residual_fwd_raw(d[0], d[1], d[2], d[3], g_a, tg_a)
            return [y, ty, o, to]

        half = ln_bytes + gate_bytes   # one LayerNorm-modulate and one gate-residual from host buffers
        e2e = _e2e_gbs(host, run, int(n_el * 12), half, min(args.steps, 10), dev)
        e2e["note"] = "one LayerNorm-modulate + one gate-residual per step (half a block), modulation rows resident"
    if not args.no_cpu_baseline:
        from oracle import adaln_oracle as ada  # cpu_baseline leg only
        cx, ctx_, ch, cth = (torch.randn(2, L, Cn) for _ in range(4))
        cm, ctm = 0.3 * torch.randn(2, 1, 6 * Cn), 0.03 * torch.randn(2, 1, 6 * Cn)
        c_sh, c_sc, c_g = cm.chunk(6, dim=-1)[:3]
        c_tsh, c_tsc, c_tg = ctm.chunk(6, dim=-1)[:3]

        def cstep():
            with torch.no_grad():
                for _ in range(2):
                    torch.func.jvp(ada.ln_modulate, (cx, c_sh, c_sc), (ctx_, c_tsh, c_tsc))
                    torch.func.jvp(ada.gate_residual, (cx, c_g, ch), (ctx_, c_tg, cth))

        cpu_base = _cpu_port_gbs(cstep, nbytes * 2 / B, f"a B=2 batch slice of {args.workload} tokens: the reference's "
                                 "modulate(norm(x)) and x + gate * h (models/layers.py:28-29, 195-201) under "
                                 "torch.func.jvp, fp32")
    if rank == 0:
        print(json.dumps({
            "metric": "adaln_block_dual_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload} tokens (B={B}, L={L}), width {Cn}: the adaLN ops of one DiT block with "
                                   "tangents (2 LayerNorm-modulate, 2 gate-residual), fp32 stream, bf16 matmul side",
                       "l2": "every tensor is larger than the 126 MB L2; no flush between steps"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                         "peak_source": f"HBM copy, of {peaks['source']}", "algorithmic_bytes_per_step": nbytes,
                         "kernel": "ln_modulate_fwd_kernel<f32, bf16, dual> x 2 + gate_residual_fwd_kernel<f32, bf16, dual> x 2",
                         "per_kernel_gbs": per},
            "cpu_baseline": cpu_base, "e2e": e2e,
            "op": "adaln", "gpu_launches": 4 * args.steps, "clocks": sampler.summary()}))


def _model_record(args, workload, world, rank, dev, steps=None, warm=None):
    """One whole-model configuration on all ranks of an initialised job: C4 (training step, data parallel with an NCCL
    gradient all-reduce) or C5 (4-step Euler sampling, sharded per rank, no collective).  Returns the record (the
    same on every rank for the timing fields).  Frees what it built before it returns."""
    import torch
    import torch.distributed as dist
    from dmf_b200 import ops
    from dmf_b200.harness import train as T
    from dmf_b200.harness.model import build_dmft
    from dmf_b200.harness.sampler import GraphedSampler, euler_sampler

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(dev.index)
    sampler.start()
    warm = 3 if warm is None else max(warm, 3)
    steps = steps or (5 if workload == "C4" else 10)
    torch.cuda.reset_peak_memory_stats(dev)
    extra = {}

    if workload == "C4":
        global_batch = 256
        mb = args.micro_batch or next(m for m in (128, 64, 32, 16, 8, 4, 2, 1) if (global_batch // world) % m == 0)
        assert global_batch % (mb * world) == 0, "256 must be divisible by micro_batch * n_gpus"
        n_micro = global_batch // (mb * world)
        st = T.build_train_state(dev, name=args.model, input_size=32, dmf_depth=20, attn_func="fa3", seed=0,
                                 graphs=not args.no_graphs, overlap=not args.no_overlap, n_buckets=args.buckets)
        gen = torch.Generator(device="cpu").manual_seed(1000 + rank)
        # the step's inputs start in pinned host memory: latents N(0,1), labels uniform
        host = [(torch.randn(mb, 4, 32, 32, generator=gen).pin_memory(),
                 torch.randint(0, 1000, (mb,), generator=gen).pin_memory()) for _ in range(n_micro)]
        torch.manual_seed(rank)

        def step():
            batches = [(x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)) for x, y in host]
            return T.train_step(st, batches)

        units, metric, unit, scaling = global_batch, "dmft_xl2_train_images_per_s", "images/s", "strong"
        reduce_how = ("no collective (one GPU)" if world == 1 else
                      f"NCCL all-reduce of the flat fp32 gradient buffer in {len(st.bucket_bounds)} buckets inside the last "
                      "micro-batch's graph, under its backward pass" if (st.graphs and st.overlap) else
                      "one NCCL all-reduce of the flat fp32 gradient buffer after the last micro-batch" if st.graphs else
                      "DistributedDataParallel bucketed all-reduce")
        desc = (f"{args.model} training step: FM forward + JVP forward + backward, bf16 autocast, global batch 256 = "
                f"{world} GPU x {n_micro} micro-batches x {mb}, "
                + ("micro-batch forward+backward replayed as a CUDA graph, " if st.graphs else "eager launches, ")
                + reduce_how + ", clip 1.0, fused AdamW, EMA")
        h2d = sum(x.numel() * x.element_size() + y.numel() * y.element_size() for x, y in host)
        d2h = 4
        extra = {"micro_batch": mb, "n_micro": n_micro, "global_batch": global_batch,
                 "grad_bytes": int(st.flat_grad.numel() * 4) if st.graphs else None}
    else:
        per_gpu = 64
        torch.manual_seed(0)
        model = build_dmft(args.model, input_size=64, dmf_depth=20, use_logvar=False, num_classes=1000,
                           attn_func="fa3", qk_norm=True).to(dev).to(torch.bfloat16).eval()
        gen = torch.Generator(device="cpu").manual_seed(rank)   # per-rank seed, as generate.py:43
        z_host = torch.randn(per_gpu, 4, 64, 64, generator=gen).to(torch.bfloat16).pin_memory()
        y_host = torch.randint(0, 1000, (per_gpu,), generator=gen).pin_memory()
        out_host = torch.empty(per_gpu, 4, 64, 64, dtype=torch.float64).pin_memory()

        graphed = None if args.no_graphs else GraphedSampler(model, per_gpu, (4, 64, 64), torch.bfloat16, dev,
                                                              num_steps=4, shift=1.5, cfg_scale=1.0)

        def step():
            if graphed is not None:      # the pinned host buffers are copied straight into the graph's inputs
                x = graphed(z_host, y_host)
            else:
                z, y = z_host.to(dev, non_blocking=True), y_host.to(dev, non_blocking=True)
                x = euler_sampler(model, z, y, num_steps=4, shift=1.5, cfg_scale=1.0)
            out_host.copy_(x, non_blocking=True)
            return x

        units, metric, unit, scaling = per_gpu * world, "dmft_xl2_sample_images_per_s", "images/s", "weak"
        desc = (f"{args.model} 4-step Euler sampling at 512px (latent 4x64x64, shift 1.5, qk-norm, bf16 weights), "
                f"{per_gpu} images per GPU, no VAE decode, no collective"
                + ("" if args.no_graphs else ", the 4-step loop replayed as one CUDA graph"))
        h2d = z_host.numel() * 2 + y_host.numel() * 8
        d2h = out_host.numel() * 8
        extra = {"per_gpu_batch": per_gpu}

    for _ in range(warm):
        out = step()
    sync_all()
    if workload == "C4":
        st.timing = {}                       # CUDA events around the phases of the timed steps
    sampler.active.set()
    launches0 = ops.launch_count
    e0.record(stream)
    for _ in range(steps):
        out = step()
    e1.record(stream)
    sync_all()
    launches = ops.launch_count - launches0
    sampler.active.clear()
    sampler.stop()
    ms_total = e0.elapsed_time(e1)
    ops.check_device_status(dev)
    phase = {}
    if workload == "C4" and st.timing:
        tm = st.timing
        n = len(tm["tail_done"])
        fwd_bwd = sum(a.elapsed_time(b) for a, b in zip(tm["step_start"], tm["backward_done"])) / n
        phase = {"fwd_bwd_ms": fwd_bwd,
                 "allreduce_exposed_ms": sum(a.elapsed_time(b) for a, b in zip(tm["backward_done"], tm["allreduce_done"])) / n,
                 "tail_ms": sum(a.elapsed_time(b) for a, b in zip(tm["allreduce_done"], tm["tail_done"])) / n}
        st.timing = None
    if world > 1:
        t = torch.tensor([ms_total] + [phase.get(k, 0.0) for k in ("fwd_bwd_ms", "allreduce_exposed_ms", "tail_ms")],
                         device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t[0])
        if phase:
            phase = {k: float(t[i + 1]) for i, k in enumerate(("fwd_bwd_ms", "allreduce_exposed_ms", "tail_ms"))}
    ms_step = ms_total / steps
    value = units / (ms_step * 1e-3)
    loss_val = float(out.float().mean().item()) if workload == "C4" else None
    rec = {
        "metric": metric, "images_per_s": value, "value": value, "unit": unit, "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": ms_step, "scaling": scaling, **extra, **phase,
        "workload": f"{workload}: {desc}", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
        "gpu_launches": launches, "clocks": sampler.summary(),
        "mem_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
        **({"last_loss": loss_val} if loss_val is not None else {}),
    }
    # free the model, its optimiser state and the graphs' memory pools before the caller goes on
    if workload == "C4":
        del st, host
    else:
        del model, graphed
    del out, step
    gc.collect()
    torch.cuda.empty_cache()
    return rec


def _model_record_in_children(args, workload, world, rank, local_rank, port_offset, limit_s=300):
    """A whole-model configuration for the default line, run as a job of its own: every rank of this job starts one
    child process (`bench.py --workload C4|C5 --record-only`), the children form their own process group on another
    port, and rank 0's child prints the record.  A failure or a stall in there costs the sub-record (the child is
    ended when its time limit runs out), never the headline of this process."""
    cmd = [sys.executable, str(ROOT / "bench.py"), "--workload", workload, "--gpus", str(world), "--record-only",
           "--model", args.model, "--buckets", str(args.buckets)]
    if args.no_graphs:
        cmd.append("--no-graphs")
    if args.no_overlap:
        cmd.append("--no-overlap")
    if args.micro_batch:
        cmd += ["--micro-batch", str(args.micro_batch)]
    env = dict(os.environ)
    env["MASTER_ADDR"] = "127.0.0.1"
    env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + 16 + port_offset)
    env["RANK"], env["LOCAL_RANK"], env["WORLD_SIZE"] = str(rank), str(local_rank), str(world)
    for k in ("TORCHELASTIC_RUN_ID", "TORCHELASTIC_RESTART_COUNT", "TORCHELASTIC_MAX_RESTARTS", "GROUP_RANK",
              "ROLE_RANK", "TORCHELASTIC_USE_AGENT_STORE"):
        env.pop(k, None)
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=limit_s, env=env)
    except subprocess.TimeoutExpired:     # subprocess.run has ended the child it started
        return {"error": f"the {workload} child process did not finish within {limit_s} s"}
    if rank != 0:
        return None
    for line in reversed(res.stdout.strip().splitlines()):
        try:
            rec = json.loads(line)
        except ValueError:
            continue
        if isinstance(rec, dict) and "metric" in rec:
            return rec
    return {"error": f"child exited {res.returncode}: {(res.stderr or res.stdout).strip()[-600:]}"}


def run_model(args):
    """--workload C4 / C5 as the bench line itself."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _pin_to_gpu_numa_node(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # a collective that cannot complete ends the job with an error after two minutes instead of blocking it
        dist.init_process_group("nccl", device_id=dev, timeout=__import__("datetime").timedelta(seconds=120))
    rec = _model_record(args, args.workload, world, rank, dev,
                        steps=None if args.steps == 50 else args.steps, warm=None if args.warmup == 10 else args.warmup)
    if rank == 0 and args.record_only:
        print(json.dumps(rec), flush=True)
    elif rank == 0:
        line = {
            "metric": rec["metric"], "value": rec["value"], "unit": rec["unit"], "n_gpus": world, "steps": rec["steps"],
            "warmup": rec["warmup"], "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
            "scaling": rec["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": rec["workload"], "weights": "random init (reference initialisation)",
                       "attn_func": "fa3 -> dmf_b200 sm_100a kernels",
                       "l2": "activations and weights far exceed the 126 MB L2"},
            "roofline": None, "cpu_baseline": None,
            # every step already starts from pinned host inputs and ends with a device-to-host read
            "e2e": {"value": rec["value"], "unit": rec["unit"], "h2d_bytes_per_step": rec["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": rec["d2h_bytes_per_step"], "api": "dmf_b200.harness train_step / euler_sampler"},
            "gpu_launches": rec["gpu_launches"], "clocks": rec["clocks"], "mem_gb": rec["mem_gb"],
            **{k: rec[k] for k in ("micro_batch", "n_micro", "fwd_bwd_ms", "allreduce_exposed_ms", "tail_ms", "last_loss",
                                   "grad_bytes", "per_gpu_batch") if k in rec},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference", "reference-gpu"], default="ours")
    ap.add_argument("--workload", choices=list(WORKLOADS) + ["C4", "C5"], default="C3",
                    help="C3/C2: attention JVP op (default C3, the bench line); C4: DMFT-XL/2 training step, "
                         "global batch 256; C5: DMFT-XL/2 4-step Euler sampling at 512px, 64 images per GPU")
    ap.add_argument("--micro-batch", type=int, default=0,
                    help="C4: images per forward/backward pass; 0 = the largest of 128, 64, 32 that divides the per-GPU "
                         "share of the global batch (128 images keep 123 GB of the 180 GB HBM in use)")
    ap.add_argument("--model", default="DMFT-XL/2", help="C4/C5: harness model name (smaller ones for smoke runs)")
    ap.add_argument("--no-graphs", action="store_true", help="C4 / C5: eager launches (and DDP) instead of the CUDA-graphed micro-step / sampler loop")
    ap.add_argument("--op", choices=["dual", "fwd", "bwd", "rmsnorm", "adaln"], default="dual",
                    help="C2/C3: entry point to time (default: the fused forward+tangent, which is the bench line)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second back-to-back loop")
    ap.add_argument("--no-secondary", action="store_true", help="skip the other kernels of the path")
    ap.add_argument("--no-comparator", action="store_true", help="skip the reference's GPU kernels (child process)")
    ap.add_argument("--no-model", action="store_true", help="skip the C4 / C5 sub-records of the default line")
    ap.add_argument("--op-only", action="store_true",
                    help="only the timed op and its roofline: no sustained loop, host-buffer leg, CPU baseline, secondary "
                         "kernels, comparator or whole-model records (profiling runs)")
    ap.add_argument("--record-only", action="store_true",
                    help="C4 / C5: print the bare record (what the default line embeds as its c4 / c5 entry)")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="chunks along the batch of the pipelined host-buffer leg")
    ap.add_argument("--no-overlap", action="store_true",
                    help="C4: one all-reduce after the last micro-batch instead of bucketed all-reduces inside its graph")
    ap.add_argument("--buckets", type=int, default=8, help="C4: gradient buckets of the overlapped all-reduce")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--batch", type=int, default=None,
                    help="override the per-GPU batch of the workload (profiling runs only; the bench line needs the default)")
    args = ap.parse_args()
    if args.op_only:
        args.no_sustained = args.no_e2e = args.no_cpu_baseline = args.no_secondary = True
        args.no_comparator = args.no_model = True
    if args.impl == "reference-gpu":
        run_reference_gpu(args)
        return
    if args.workload in ("C4", "C5"):
        if args.impl == "reference":
            # whole-model CPU runs of DMFT-XL/2 take minutes per step; the CPU arm exists for the op (C2/C3)
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "whole-model CPU baseline not provided; use --workload C3 for the op"}))
            return
        run_model(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.op == "rmsnorm":
        run_rmsnorm(args)
    elif args.op == "adaln":
        run_adaln(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
