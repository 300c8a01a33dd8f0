#!/usr/bin/env python3
"""Benchmark of the attention-forward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config cfg5] [--impl reference]

One step = one forward pass of the workload, through the library's C ABI.  The default workload is
the sharded benchmark configuration: bf16 SDPA with the additive sinusoidal encoding fused into
the Q/K load, B=16 H=32 L=4096 head_d=512, one such problem per GPU (weak scaling; the (batch,
head) slices are independent, so there is no collective on the data path).  Prints ONE JSON line.

  value      whole-job TFLOP/s (4*B*H*Lq*Lk*D flops per problem) with inputs resident in HBM
  e2e        the same through b200attn_forward_host with pinned HOST buffers, copies in the timed region
  roofline   the dominant kernel against the measured peak of MEASURED_PEAKS.json
  cpu_baseline  the reference project's own CPU attention (oracle/_ref) on a bounded sample, on
             this box's host cores (rank 0, N=1 only)

`--impl reference` times only that CPU implementation, with all host threads, on bounded samples.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PE = {"none": 0, "rope_half": 2, "sinusoidal": 3, "rope_half_q_only": 5}
CONFIGS = {
    # name: (dtype, pe, B, H, Lq, Lk, D, dist, bound)
    "cfg1": ("f32", "none", 1, 4, 64, 64, 2048, "uniform", "hbm"),
    "cfg2a": ("f32", "none", 1, 4, 64, 64, 512, "uniform", "hbm"),
    "cfg2b": ("f32", "none", 1, 4, 64, 64, 4096, "uniform", "hbm"),
    "cfg2c": ("f32", "none", 1, 4, 64, 64, 8192, "uniform", "hbm"),
    "cfg2d": ("f32", "none", 1, 4, 32, 64, 4096, "uniform", "hbm"),
    "cfg3": ("bf16", "none", 8, 16, 1024, 1024, 512, "normal", "tensor"),
    "cfg4": ("bf16", "rope_half", 4, 32, 2048, 2048, 1024, "normal", "tensor"),
    "cfg5": ("bf16", "sinusoidal", 16, 32, 4096, 4096, 512, "normal", "tensor"),
    # the decode regime (few queries against a long key cache): K rotated beforehand (KV-cache use) / in the load
    "decode": ("bf16", "rope_half_q_only", 1, 32, 4, 32768, 128, "normal", "hbm"),
    "decode_rope": ("bf16", "rope_half", 1, 32, 4, 32768, 128, "normal", "hbm"),
    # narrow heads (what most transformer models use): the one-kernel path
    "narrow128": ("bf16", "none", 4, 16, 4096, 4096, 128, "normal", "tensor"),
    "narrow64": ("bf16", "none", 4, 16, 4096, 4096, 64, "normal", "tensor"),
    "narrow256": ("bf16", "none", 4, 16, 4096, 4096, 256, "normal", "tensor"),
    # profiling-size variants of cfg4 and cfg5 (16 heads): small enough for a multi-pass ncu capture
    "cfg4p": ("bf16", "rope_half", 1, 16, 2048, 2048, 1024, "normal", "tensor"),
    "cfg5p": ("bf16", "sinusoidal", 1, 16, 4096, 4096, 512, "normal", "tensor"),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum from ncu captures of the kernels in use, per STEP (a
# step of the two-kernel bf16 path is several launches; `achieved` is per step as well); null until a
# capture exists for the kernel in use
NCU_TRAFFIC_BYTES = {
    ("cfg5", "tc_wide"): 48.9e9,        # a 16-head capture (1526.5 MB over the three launches) x 32
    ("cfg4", "tc_wide"): 5.68e9,        # a 16-head capture (709.9 MB) x 8
    ("cfg3", "tc_bf16"): 514.8e6,       # 402.8 MB read + 112.0 MB written
    ("cfg5", "tc_bf16"): 8 * 2.0**30 + 2 * 2.0**30,   # scaled from the cfg 3 capture by input/output bytes plus the encoded-K scratch
    ("cfg1", "splitd_tc"): 6.42e6 + 2.10e6,           # 6.42 MB read inside the kernel; the 2 MiB output leaves the L2 after it
    ("cfg2c", "splitd_tc"): 25.29e6 + 8.39e6,         # 25.29 MB read; 8 MiB output
    ("decode", "tc_decode"): 537.0e6 + 3.75e6,
    ("narrow128", "tc_fused"): 201.7e6 + 44.5e6,      # (part of the 67 MB output is still in L2 when the kernel ends)
    ("narrow256", "tc_fused"): 403.1e6 + 112.5e6,
}
# nominal fp32 FMA rate of the CUDA cores: 148 SMs x 128 lanes x 2 flops x 1.965 GHz (the fp32 path now
# does its products on the tensor cores as tf32 MMAs on split operands; the figure is reported as the
# "compute roof" the task statement asks for next to the HBM roof)
FFMA_ROOF_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12


def flops_of(cfg):
    _, _, B, H, Lq, Lk, D, _, _ = CONFIGS[cfg]
    return 4.0 * B * H * Lq * Lk * D


def bytes_of(cfg):
    dt, _, B, H, Lq, Lk, D, _, _ = CONFIGS[cfg]
    return (4 if dt == "f32" else 2) * B * H * D * (2 * Lq + 2 * Lk)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {k: float(d[k]) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained")}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "50"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [r.split(", ") for r in open(self.f.name).read().strip().splitlines() if r.strip()]
        os.unlink(self.f.name)
        sm = sorted(float(r[1]) for r in rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.strip().lower() == "active":
                        reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def torch_dtype(torch, dt):
    return torch.float32 if dt == "f32" else torch.bfloat16


def make_inputs(pkg, torch, cfg, dev, seed):
    dt, _, B, H, Lq, Lk, D, dist, _ = CONFIGS[cfg]
    td = torch_dtype(torch, dt)
    Q = torch.empty((B, H, Lq, D), dtype=td, device=dev)
    K = torch.empty((B, H, Lk, D), dtype=td, device=dev)
    V = torch.empty((B, H, Lk, D), dtype=td, device=dev)
    for t, tid in ((Q, 0), (K, 1), (V, 2)):
        pkg.synth_fill(t, seed, tid, dist)
    return Q, K, V, torch.empty_like(Q)


def time_steps(pkg, torch, sets, pe, steps, warmup, barrier=None, flags=0, kernel_events=False):
    """Times `steps` forwards (cycling through `sets` of (Q,K,V,out)) with CUDA events on the
    stream the kernels are launched on; returns ms per step.  The steps are enqueued by one
    b200attn_forward_many call so that no interpreter time sits between launches.  With kernel_events the
    library also brackets every launch of its two-kernel bf16 path with an event pair (time_steps.kernels):
    that costs a few microseconds per launch - a quarter of a cfg 3 step -, so the step time that is reported is
    always taken without it."""
    n = len(sets)
    mk = lambda i: pkg.args_for(*sets[i % n][:3], sets[i % n][3], pe=pe, flags=pkg.FLAG_ASYNC | flags)
    if warmup:
        pkg.forward_many([mk(i) for i in range(warmup)])
    torch.cuda.synchronize()
    pkg.kernel_times(bool(kernel_events), collect=True)   # per-kernel events of the two-kernel bf16 path; record cleared
    if barrier:
        barrier()
    torch.cuda.synchronize()
    batch = [mk(i) for i in range(steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = pkg.launch_count()
    e0.record()
    pkg.forward_many(batch)
    e1.record()
    torch.cuda.synchronize()
    time_steps.launches = pkg.launch_count() - n0
    time_steps.kernels = pkg.kernel_times(False, collect=True)
    if barrier:
        barrier()
    return e0.elapsed_time(e1) / steps


SETTLE_S = 3.0   # idle time before each side measurement of a default run


def settle(torch):
    """The side measurements follow the long, power-capped steps of the main configuration; the board's power
    controller averages over seconds, so a short configuration measured right after them runs at the clocks the
    main one left behind (decode: 0.57 of the HBM peak against 0.72 on its own).  A few idle seconds put each side
    measurement in the state a run of that configuration alone starts from; the rows carry `settle_s`."""
    torch.cuda.synchronize()
    time.sleep(SETTLE_S)


def narrow_sweep(pkg, torch, dev, pk):
    """bf16 at the head widths most models use (64, 128, 256), where the scores stay on the SM in one kernel: the default
    path and, for comparison, the two-kernel path of the wide heads on the same inputs."""
    out = []
    for cfg in ("narrow256", "narrow128", "narrow64"):
        _, _, B, H, Lq, Lk, D, _, _ = CONFIGS[cfg]
        sets = [make_inputs(pkg, torch, cfg, dev, 42 + i) for i in range(2)]
        settle(torch)
        t = time_steps(pkg, torch, sets, 0, 20, 5)
        path = pkg.last_path()
        t2 = time_steps(pkg, torch, sets, 0, 10, 3, flags=pkg.FLAG_TWO_KERNELS)
        fl = flops_of(cfg)
        out.append({"config": cfg, "shape": [B, H, Lq, Lk, D], "path": path, "ms": round(t, 4), "tflops": round(fl / t / 1e9, 1),
                    "frac_of_sustained_bf16_peak": round(fl / t / 1e9 / pk["bf16_tflops_sustained"], 4),
                    "two_kernel_path_ms": round(t2, 4), "two_kernel_path_tflops": round(fl / t2 / 1e9, 1), "settle_s": SETTLE_S})
        del sets
        torch.cuda.empty_cache()
    return out


def bf16_sweep(pkg, torch, dev, pk, skip):
    """The other bf16 benchmark configurations (cfg 3: no encoding; cfg 4: rotate-half RoPE, head_d 1024) and the
    decode regime (K rotated beforehand, and rotated in the load), one short measurement each, so that a default run
    reports them all."""
    out = []
    for cfg in ("cfg3", "cfg4", "decode", "decode_rope"):
        if cfg == skip:
            continue
        dt, pe_name, B, H, Lq, Lk, D, _, bound = CONFIGS[cfg]
        sets = [make_inputs(pkg, torch, cfg, dev, 42 + i) for i in range(2)]
        settle(torch)
        t = time_steps(pkg, torch, sets, PE[pe_name], 20, 5)
        row = {"config": cfg, "shape": [B, H, Lq, Lk, D], "pe": pe_name, "path": pkg.last_path(), "ms": round(t, 4), "settle_s": SETTLE_S}
        if bound == "tensor":
            row["tflops"] = round(flops_of(cfg) / t / 1e9, 1)
            row["frac_of_sustained_bf16_peak"] = round(flops_of(cfg) / t / 1e9 / pk["bf16_tflops_sustained"], 4)
        else:
            row["gbs_algorithmic"] = round(bytes_of(cfg) / t / 1e6, 1)
            row["frac_of_hbm_peak"] = round(bytes_of(cfg) / t / 1e6 / pk["hbm_gbs"], 4)
        out.append(row)
        del sets
        pkg.lib().b200attn_release_workspace()
        torch.cuda.empty_cache()
    return out


def bind_to_gpu_numa_node(torch, dev_index):
    """Pins this process to the CPUs of the NUMA node its GPU hangs off (read from sysfs), so that the pinned host
    buffers allocated afterwards are node-local (first touch).  Returns what it found; does nothing where the
    information is missing or the box has one node."""
    info = {"gpu_numa_node": None, "numa_nodes": None, "bound": False}
    try:
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        info["numa_nodes"] = len(nodes)
        props = torch.cuda.get_device_properties(dev_index)
        bus = "%04x:%02x:%02x.0" % (getattr(props, "pci_domain_id", 0), props.pci_bus_id, props.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        info["gpu_numa_node"] = node
        if node < 0 or len(nodes) < 2:
            return info
        cpus = set()
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            info["bound"] = True
    except (OSError, ValueError, AttributeError):
        pass
    return info


def cpu_full(cfg, threads):
    """The reference's attention_cpu on the WHOLE problem of an fp32 configuration: with one thread exactly
    as written, or with the (b,h) slices fanned over `threads` host threads.  Returns seconds."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    _, _, B, H, Lq, Lk, D, _, _ = CONFIGS[cfg]
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 42, "uniform")
    out = np.empty_like(Q)
    f, ref = ol._f, ol.ref()

    def run(bh0, n):
        q, k, v, o = (x.reshape(B * H, -1, D)[bh0:bh0 + n] for x in (Q, K, V, out))
        if ref is not None:
            ref.ref_attention_cpu(f(q), f(k), f(v), f(o), 1, n, Lq, Lk, D)
        else:
            ol.oracle().oracle_attention_pe_f32(f(q), f(k), f(v), f(o), 1, n, Lq, Lk, D, ol.PE_NONE, D, 10000.0, 0, 1)
    t0 = time.perf_counter()
    if threads <= 1:
        run(0, B * H)
    else:
        th = [threading.Thread(target=run, args=(i, 1)) for i in range(B * H)]
        for t in th:
            t.start()
        for t in th:
            t.join()
    return time.perf_counter() - t0


def fp32_sweep(pkg, torch, dev, pk, with_cpu=True):
    """The fp32 small-sequence configurations.  Per configuration: step time of back-to-back asynchronous
    launches through b200attn_forward_many, L2-cold (rotation through >= 512 MiB of distinct inputs) and
    L2-warm (one set re-used); the same launches without overlap between consecutive calls; a blocking
    call's host latency; the HBM and compute rooflines; and the reference's CPU attention on the whole problem."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    out = []
    for cfg in ("cfg1", "cfg2a", "cfg2b", "cfg2c", "cfg2d"):
        nbytes = bytes_of(cfg)
        nsets = max(2, min(256, (512 << 20) // nbytes))
        sets = [make_inputs(pkg, torch, cfg, dev, 42 + i) for i in range(nsets)]
        settle(torch)
        cold = min(time_steps(pkg, torch, sets, 0, nsets, nsets if r == 0 else 0) for r in range(3))
        warm = time_steps(pkg, torch, sets[:1], 0, 200, 20)
        serial = min(time_steps(pkg, torch, sets, 0, nsets, 0, flags=pkg.FLAG_NO_OVERLAP) for r in range(2))
        Q, K, V, O = sets[0]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(50):
            pkg.forward(Q, K, V, out=O)
        lat = (time.perf_counter() - t0) / 50 * 1e3
        _, _, B, H, Lq, Lk, D, _, _ = CONFIGS[cfg]
        tfl = flops_of(cfg) / cold / 1e9
        row = {"config": cfg, "shape": [B, H, Lq, Lk, D], "path": pkg.last_path(), "cold_ms": round(cold, 5),
               "warm_ms": round(warm, 5), "blocking_call_ms": round(lat, 5),
               # the same launches with each one started only after the previous has completed: kernel + launch gap
               "serial_step_us": round(serial * 1e3, 2), "overlap_gain_us": round((serial - cold) * 1e3, 2),
               "cold_gbs": round(nbytes / cold / 1e6, 1), "cold_tflops": round(tfl, 2),
               "cold_frac_of_hbm_peak": round(nbytes / cold / 1e6 / pk["hbm_gbs"], 4),
               "hbm_floor_us": round(nbytes / pk["hbm_gbs"] / 1e3, 2),
               "frac_of_fp32_compute_roof": round(tfl / FFMA_ROOF_TFLOPS, 4), "fp32_compute_roof_tflops": round(FFMA_ROOF_TFLOPS, 1),
               "rotation_sets": nsets, "settle_s": SETTLE_S}
        if with_cpu:
            one = cpu_full(cfg, 1)
            fan = cpu_full(cfg, B * H)
            row["cpu_baseline"] = {"kind": "reference" if ol.ref() is not None else "port", "sample": "whole problem",
                                   "single_thread_ms": round(one * 1e3, 2), "fanned_ms": round(fan * 1e3, 2),
                                   "fanned_threads": B * H, "host_cores": os.cpu_count(),
                                   "single_thread_tflops": round(flops_of(cfg) / one / 1e12, 6)}
        out.append(row)
        del sets
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference project's own CPU attention (oracle/_ref), all host threads
# ------------------------------------------------------------------------------------------------
class CpuRef:
    def __init__(self, cfg):
        import numpy as np
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as ol
        self.np, self.ol = np, ol
        self.cfg = cfg
        self.kind = "reference" if ol.ref() is not None else "port"
        self.cores = os.cpu_count() or 1
        dt, pe, B, H, Lq, Lk, D, dist, _ = CONFIGS[cfg]
        self.pe, self.Lk, self.D, self.Lq = pe, Lk, D, Lq
        gen = ol.synth_uniform if dist == "uniform" else ol.synth_normal
        n = min(self.cores, B * H)
        self.nslices = n
        self.K = [gen((1, 1, Lk, D), 42, 1 + 3 * i) for i in range(n)]
        self.V = [gen((1, 1, Lk, D), 42, 2 + 3 * i) for i in range(n)]
        self.Qfull = [gen((1, 1, Lq, D), 42, 3 * i) for i in range(n)]
        if dt == "bf16":
            rnd = lambda x: ol.from_bf16_bits(ol.to_bf16_bits(x))
            self.K, self.V, self.Qfull = [rnd(x) for x in self.K], [rnd(x) for x in self.V], [rnd(x) for x in self.Qfull]
        L = max(Lq, Lk)
        if pe == "sinusoidal":
            self.t0, self.t1 = ol.sinusoidal_tables(L, D)
        elif pe in ("rope_half", "rope_half_q_only"):   # (q-only: the CPU code rotates K itself, the same mathematics)
            pe = self.pe = "rope_half"
            self.t0, self.t1 = ol.rope_cache(L, D)
            perm = np.empty(D, dtype=np.int64)   # rotate-half == interleaved under this column order
            perm[0::2] = np.arange(D // 2)
            perm[1::2] = np.arange(D // 2) + D // 2
            self.K = [np.ascontiguousarray(x[..., perm]) for x in self.K]
            self.Qfull = [np.ascontiguousarray(x[..., perm]) for x in self.Qfull]

    def _one(self, i, rows):
        np, ol = self.np, self.ol
        q = np.ascontiguousarray(self.Qfull[i][:, :, :rows])
        out = np.empty_like(q)
        f = ol._f
        ref = ol.ref()
        if ref is not None:
            if self.pe == "sinusoidal":
                ref.ref_attention_sinusoidal_cpu(f(q), f(self.K[i]), f(self.V[i]), f(self.t0), f(self.t1), f(out), 1, 1, rows, self.Lk, self.D)
            elif self.pe == "rope_half":
                ref.ref_attention_rope_cpu(f(q), f(self.K[i]), f(self.V[i]), f(out), f(self.t0), f(self.t1), 1, 1, rows, self.Lk, self.D)
            else:
                ref.ref_attention_cpu(f(q), f(self.K[i]), f(self.V[i]), f(out), 1, 1, rows, self.Lk, self.D)
        else:
            pe = {"none": ol.PE_NONE, "sinusoidal": ol.PE_SINUSOIDAL, "rope_half": ol.PE_ROPE_INTERLEAVED}[self.pe]
            ol.oracle().oracle_attention_pe_f32(f(q), f(self.K[i]), f(self.V[i]), f(out), 1, 1, rows, self.Lk, self.D, pe, self.D, 10000.0, 0, 1)

    def run(self, rows):
        """One sample: every host thread evaluates `rows` query rows of its own (b,h) slice.
        Returns (seconds, flops)."""
        th = [threading.Thread(target=self._one, args=(i, rows)) for i in range(self.nslices)]
        t0 = time.perf_counter()
        for t in th:
            t.start()
        for t in th:
            t.join()
        return time.perf_counter() - t0, 4.0 * self.nslices * rows * self.Lk * self.D

    def calibrate(self, target_s):
        rows = min(self.Lq, 4)
        sec, _ = self.run(rows)
        rows = int(max(1, min(self.Lq, rows * target_s / max(sec, 1e-4))))
        return rows


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = args.config
    cpu = CpuRef(cfg)
    total = args.steps + args.warmup
    rows = cpu.calibrate(min(6.0, 150.0 / max(total, 1)))
    for _ in range(args.warmup):
        cpu.run(rows)
    secs, fl = 0.0, 0.0
    for _ in range(args.steps):
        s, f = cpu.run(rows)
        secs += s
        fl += f
    v = fl / secs / 1e12
    dt, pe, B, H, Lq, Lk, D, _, _ = CONFIGS[cfg]
    sample = f"{cpu.nslices} (b,h) slices x {rows} of {Lq} query rows x all {Lk} keys per step, one slice per host thread"
    line = {"impl": "reference", "metric": "attn_fwd_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs / max(args.steps, 1) * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(cfg),
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cpu.nslices, "kind": cpu.kind, "sample": sample},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def torch_sdpa_arm(args):
    """A timed competitor, never on the product path: torch.nn.functional.scaled_dot_product_attention on
    the same shapes and dtype (what the reference's final/benchmark_pytorch_wrapper.cu:40-60 measured on
    its GPU).  The positional encoding of cfg 4 / cfg 5 is NOT applied (torch has no fused equivalent), so
    those lines time plain attention of the same shape.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    import torch.nn.functional as F
    dev = torch.device("cuda:0")
    names = [args.config] if args.config != "cfg5" or args.no_extras else ["cfg1", "cfg2a", "cfg2b", "cfg2c", "cfg2d", "cfg3", "cfg4", "narrow256", "narrow128", "narrow64", "cfg5"]
    rows = []
    for cfg in names:
        dt, pe, B, H, Lq, Lk, D, dist, _ = CONFIGS[cfg]
        td = torch_dtype(torch, dt)
        nbytes = bytes_of(cfg)
        nsets = 1 if nbytes > (200 << 20) else max(2, min(64, (512 << 20) // nbytes))
        sets = []
        for i in range(nsets):
            g = torch.Generator(device=dev).manual_seed(42 + i)
            mk = (lambda *sh: (torch.rand(*sh, device=dev, generator=g) * 2 - 1).to(td)) if dist == "uniform" else \
                 (lambda *sh: torch.randn(*sh, device=dev, generator=g).to(td))
            sets.append((mk(B, H, Lq, D), mk(B, H, Lk, D), mk(B, H, Lk, D)))
        steps = max(args.steps, nsets)
        for i in range(max(args.warmup, 3)):
            F.scaled_dot_product_attention(*sets[i % nsets])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            F.scaled_dot_product_attention(*sets[i % nsets])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        rows.append({"config": cfg, "shape": [B, H, Lq, Lk, D], "dtype": dt, "pe_applied": False, "ms_per_step": ms,
                     "tflops": flops_of(cfg) / (ms * 1e-3) / 1e12, "gbs_algorithmic": nbytes / (ms * 1e-3) / 1e9})
        del sets
        torch.cuda.empty_cache()
    main_row = next(r for r in rows if r["config"] == args.config)
    print(json.dumps({"impl": "torch_sdpa", "metric": "attn_fwd_tflops", "value": main_row["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": main_row["ms_per_step"], "higher_is_better": True,
                      "dtype": CONFIGS[args.config][0], "data": "synthetic", "config": workload_config(args.config),
                      "torch": torch.__version__, "note": "competitor timing only; no positional encoding applied", "configs": rows}))


def workload_config(cfg):
    dt, pe, B, H, Lq, Lk, D, dist, bound = CONFIGS[cfg]
    return {"workload": f"{cfg}: {dt} SDPA forward, pe={pe}, B={B} H={H} Lq={Lq} Lk={Lk} head_d={D} per GPU, non-causal",
            "inputs": f"iid {dist} from a counter-based generator", "l2": "inputs larger than L2 (126 MB)" if bytes_of(cfg) > (200 << 20)
            else "rotation through >= 512 MiB of distinct input sets", "parallelism": "one problem per GPU, sharded by (batch, head), no collective"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="cfg5", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "torch_sdpa"])
    ap.add_argument("--no-extras", action="store_true", help="skip the fp32 sweep, e2e and CPU baseline legs")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.impl == "torch_sdpa":
        torch_sdpa_arm(args)
        return

    import torch
    import __graft_entry__ as ge
    pkg = ge.load_package()
    pkg.lib()   # fails loudly when the CUDA library is missing: there is no fallback
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()

    cfg = args.config
    dt, pe_name, B, H, Lq, Lk, D, _, bound = CONFIGS[cfg]
    pe = PE[pe_name]
    pk, pk_src = peaks()
    nbytes, fl = bytes_of(cfg), flops_of(cfg)
    nsets = 1 if nbytes > (200 << 20) else max(2, min(256, (512 << 20) // nbytes))
    sets = [make_inputs(pkg, torch, cfg, dev, 42 + 1000 * rank + i) for i in range(nsets)]
    warm = max(args.warmup, 3)

    sampler = ClockSampler(local) if rank == 0 else None
    ms = time_steps(pkg, torch, sets, pe, args.steps, warm, barrier)
    launches = time_steps.launches
    clocks = sampler.stop() if sampler else None
    path = pkg.last_path()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = fl * world / (ms_max * 1e-3) / 1e12

    line = {"metric": "attn_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": workload_config(cfg), "kernel_path": path, "hbm_gbs_algorithmic": nbytes * world / (ms_max * 1e-3) / 1e9,
            "gpu_launches": int(launches)}
    launches_per_step = max(1, round(launches / max(args.steps, 1)))
    if bound == "tensor":
        peak = pk["bf16_tflops_sustained"]
        ach = fl / (ms * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                            "traffic": NCU_TRAFFIC_BYTES.get((cfg, path)), "peak_source": pk_src + " (sustained cuBLAS bf16)",
                            "kernel": path, "launches_per_step": launches_per_step,
                            "per": "step (all launches of the path; the per-kernel figures are in `kernels`)"}
        kt = None
        ksteps = args.steps   # as long as the timed region, so that the clocks settle the same way under the power cap
        if path == "tc_wide":
            # per kernel: a second, short pass with an event pair around every launch (the timed region above has none)
            time_steps(pkg, torch, sets, pe, ksteps, 1, barrier, kernel_events=True)
            kt = getattr(time_steps, "kernels", None)
        if path == "tc_wide" and kt and sum(v[1] for v in kt.values()) > 0:
            nqt, nkt = Lq // 128, (Lk + 255) // 256
            n_enc = max(nqt, nkt) if pe != 0 else 0
            tile_fl = 2.0 * 128 * 256 * D
            k_fl = {"scores_encode": B * H * n_enc * tile_fl, "scores": B * H * (nqt * nkt - n_enc) * tile_fl, "pv": fl / 2.0}
            names = {"scores_encode": "tcw_scores_kernel (encoding launch)",
                     "scores": "tcw_scores256_kernel (score GEMM; tcw_scores_kernel when the query tiles do not pair up)", "pv": "tcw_pv_kernel"}
            tot = sum(v[0] for v in kt.values())
            rows = []
            for k, (kms, cnt) in kt.items():
                if cnt:
                    rows.append({"kernel": names[k], "launches": cnt, "ms_per_step": kms / ksteps, "share": kms / tot,
                                 "tflops": k_fl[k] * ksteps / (kms * 1e-3) / 1e12})
            line["kernels"] = rows
            line["kernels_from"] = f"a separate pass of {ksteps} steps with a CUDA-event pair around every launch, same stream, same inputs"
            dom = max(rows, key=lambda r: r["ms_per_step"])
            line["roofline"].update({"dominant_kernel": dom["kernel"], "dominant_achieved": dom["tflops"],
                                     "dominant_frac": dom["tflops"] / peak, "dominant_share": dom["share"]})
    else:
        peak = pk["hbm_gbs"]
        ach = nbytes / (ms * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                            "traffic": NCU_TRAFFIC_BYTES.get((cfg, path)), "peak_source": pk_src + " (device copy)",
                            "kernel": path, "launches_per_step": launches_per_step}
    if clocks:
        line["clocks"] = clocks

    # ---- ONE problem of the configuration cut by (batch, head) over the ranks: rank r runs the contiguous
    # range of B*H/N flat slices b200attn_shard_ranges gives it (no collective on the data path) ----
    if world > 1:
        begin, count = pkg.shard_ranges(B * H, world)
        nh = count[rank]
        if nh > 0:
            shard = tuple(t.view(B * H, -1, D)[:nh].unsqueeze(0) for t in sets[0])   # the bytes differ per rank (seeded by rank); the work is that of the rank's slice range
            s_ms = time_steps(pkg, torch, [shard], pe, args.steps, warm, barrier)
        else:
            barrier(); barrier()
            s_ms = 0.0
        t = torch.tensor([s_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        s_max = float(t.item())
        line["strong"] = {"what": f"one {cfg} problem, its {B * H} (batch, head) slices cut into {world} contiguous ranges, one per GPU",
                          "slices_per_gpu": count, "ms_per_step": s_max, "value": fl / (s_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                          "one_gpu_ms_per_step": ms_max,
                          "speedup_over_one_gpu": ms_max / s_max, "efficiency": ms_max / s_max / world}

    # ---- host -> device copy rate of this rank's PCIe link (pinned memory, one cudaMemcpyAsync per copy) ----
    h2d_gbs = None
    numa = None
    affinity0 = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None
    if not args.no_extras:
        numa = bind_to_gpu_numa_node(torch, dev.index or 0)   # the host buffers below are allocated node-local
        try:
            nb = 1 << 30
            hsrc = torch.empty(nb, dtype=torch.uint8).pin_memory()
            ddst = torch.empty(nb, dtype=torch.uint8, device=dev)
            ddst.copy_(hsrc, non_blocking=True)
            torch.cuda.synchronize()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                ddst.copy_(hsrc, non_blocking=True)
            e1.record()
            torch.cuda.synchronize()
            h2d_gbs = 3 * nb / (e0.elapsed_time(e1) * 1e-3) / 1e9
            del hsrc, ddst
        except RuntimeError:
            h2d_gbs = None
        torch.cuda.empty_cache()

    # ---- end to end through the host-buffer entry point (pinned host memory, copies timed) ----
    if not args.no_extras:
        Q, K, V, O = sets[0]
        esz = 4 if dt == "f32" else 2
        e2e_steps = max(1, min(args.steps, 3 if nbytes > (1 << 30) else 20))
        e2e_ms, e2e_err = 0.0, None
        hq = hk = hv = ho = None
        try:   # a rank that cannot pin its host buffers still joins the reduction below, so the line is printed
            hq, hk, hv = (torch.empty(x.shape, dtype=x.dtype).pin_memory() for x in (Q, K, V))
            ho = torch.empty(O.shape, dtype=O.dtype).pin_memory()
            hq.copy_(Q); hk.copy_(K); hv.copy_(V)
        except RuntimeError as e:
            e2e_err = f"rank {rank}: {str(e).splitlines()[0][:160]}"
        del sets, Q, K, V, O
        torch.cuda.empty_cache()
        if e2e_err is None:
            pkg.forward_host(hq, hk, hv, ho, pe=pe)
            torch.cuda.synchronize()
        barrier()
        if e2e_err is None:
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                pkg.forward_host(hq, hk, hv, ho, pe=pe)
                _ = float(ho.view(-1)[0])   # the result is read on the host every step
            torch.cuda.synchronize()
            e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
        t = torch.tensor([e2e_ms, 0.0 if e2e_err is None else 1.0], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if float(t[1].item()) == 0.0:
            h2d_b, d2h_b = esz * B * H * D * (Lq + 2 * Lk), esz * B * H * D * Lq
            line["e2e"] = {"value": fl * world / (float(t[0].item()) * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": float(t[0].item()),
                           "steps": e2e_steps, "h2d_bytes_per_step": h2d_b, "d2h_bytes_per_step": d2h_b,
                           "api": "b200attn_forward_host (pinned host buffers)", "numa": numa}
            tg = torch.tensor([h2d_gbs if h2d_gbs else 0.0], dtype=torch.float64, device=dev)
            if dist is not None:
                dist.all_reduce(tg, op=dist.ReduceOp.MIN)
            if float(tg.item()) > 0:
                # the copies in (and out, on the other direction of the link) bound the step from below
                floor_ms = h2d_b / (float(tg.item()) * 1e9) * 1e3
                line["e2e"].update({"h2d_gbs_measured_min_over_ranks": float(tg.item()), "h2d_floor_ms": floor_ms,
                                    "frac_of_h2d_roof": floor_ms / float(t[0].item()),
                                    "bound": "host-to-device link (PCIe): the copies of a step take longer than its kernels"})
        else:
            line["e2e"] = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": esz * B * H * D * (Lq + 2 * Lk),
                           "d2h_bytes_per_step": esz * B * H * D * Lq, "error": e2e_err or "pinned host allocation failed on another rank"}
        del hq, hk, hv, ho
        pkg.lib().b200attn_release_workspace()
        torch.cuda.empty_cache()
    if affinity0 is not None and numa and numa.get("bound"):
        os.sched_setaffinity(0, affinity0)   # the CPU baseline below uses every host core again

    if rank == 0 and world == 1 and not args.no_extras:
        line["bf16_configs"] = bf16_sweep(pkg, torch, dev, pk, cfg)
        line["narrow_heads"] = narrow_sweep(pkg, torch, dev, pk)
        line["fp32_configs"] = fp32_sweep(pkg, torch, dev, pk)
        line["cpu_baseline_fp32"] = "per configuration in fp32_configs[].cpu_baseline: the reference's attention_cpu on the whole problem"
        cpu = CpuRef(cfg)
        rows = cpu.calibrate(15.0)
        sec, cfl = cpu.run(rows)
        line["cpu_baseline"] = {"value": cfl / sec / 1e12, "unit": "TFLOP/s", "cores": cpu.nslices, "kind": cpu.kind, "seconds": round(sec, 2),
                                "sample": f"{cpu.nslices} (b,h) slices x {rows} of {Lq} query rows x all {Lk} keys, one slice per host thread"}
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
