#!/usr/bin/env python
"""Benchmark of the transformer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--quick]

Headline (the JSON line's metric/value): causal bf16 scaled-dot-product attention forward
on the Llama-style configuration  B=8 Hq=Hkv=32 S=2048 D=128  in TFLOP/s, algorithmic
FLOPs = 4*B*H*Lq*Lk*D/2 (causal).  One step = one attention forward over one batch that is
already resident in HBM; K steps are timed with CUDA events on the launching stream, after W
warm-up steps, between barrier + synchronize on both sides, max over ranks.  q,k,v,out are
537 MB per step, larger than the 126 MB L2, so no explicit L2 flush is needed.

Beside it, in "extra": RMSNorm [16384,4096] and SwiGLU [32768,14336] in HBM GB/s, the GQA
long-sequence attention (B=4 Hq=64 Hkv=8 S=8192) in TFLOP/s and the decode step
(B=64 q_len=1 kv_len=32768 Hq=32 Hkv=8) in HBM GB/s, each with its roofline fraction.

"e2e" is the same attention with HOST buffers, copies inside the timed region, through
torch_paras.nn.attention_host (C ABI paras_b200_sdpa_fwd_host): pinned host q,k,v stream through
the GPU in batch chunks (copy in, attention, copy out overlap) into a pinned host result.
"e2e.device_api" is the unpipelined route: pinned host q,k,v -> paras:N,
F.scaled_dot_product_attention, .cpu().

N > 1 (one process per GPU under torchrun): every rank runs the same per-GPU workload on its
own batch shard (weak scaling, no collective on the forward path); value = total FLOPs of all
ranks / max-over-ranks time.

`--impl reference` times the reference's own CPU implementation (its paras:0 host engine,
built into oracle/_ref by oracle/Makefile; the oracle restatement if that build is absent) on
a bounded sample of the same workload, with all the host threads torch gives it.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "framework-torch-paras_b200", "python"), ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

WORKLOAD = "config2: bf16 causal SDPA B=8 Hq=Hkv=32 S=2048 D=128 (Llama-style)"
C2 = dict(B=8, Hq=32, Hkv=32, S=2048, D=128)
# bounded CPU sample of config 2: one batch element, 16 of its 32 heads, full sequence
CPU_SAMPLE = dict(B=1, H=16, S=2048, D=128)   # used where the whole workload does not fit the time


def sdpa_flops(B, Hq, Lq, Lk, D, causal):
    f = 4.0 * B * Hq * Lq * Lk * D
    return f / 2 if causal else f


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while a timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    _NAMES = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
              0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
              0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def _poll(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self._NAMES.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


TRAFFIC_FILE = os.path.join(ROOT, "profiles", "sdpa_tc_kernel_config2_dram_traffic.txt")


def read_ncu_traffic():
    """DRAM bytes of one launch of the headline kernel, from the text file `--ingest-ncu` wrote out
    of an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum); None when there is none."""
    try:
        vals = dict(line.split("=", 1) for line in open(TRAFFIC_FILE).read().split() if "=" in line)
        return float(vals["dram_bytes_read"]) + float(vals["dram_bytes_write"])
    except (OSError, KeyError, ValueError):
        return None


def ingest_ncu(csv_path: str):
    """`ncu -i X.ncu-rep --page raw --csv > X.csv` of a capture of this bench's headline kernel ->
    profiles/sdpa_tc_kernel_config2_dram_traffic.txt (key=value lines; mean over captured launches)."""
    import csv
    rows = list(csv.reader(open(csv_path)))
    hdr = next(i for i, r in enumerate(rows) if "Kernel Name" in r)
    names, units = rows[hdr], rows[hdr + 1]
    col = {n: i for i, n in enumerate(names)}
    mult = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "ns": 1.0, "us": 1e3, "usecond": 1e3,
            "ms": 1e6, "msecond": 1e6, "nsecond": 1.0, "%": 1.0, "": 1.0}
    launches = [r for r in rows[hdr + 2:] if len(r) == len(names) and "sdpa_tc_kernel" in r[col["Kernel Name"]]]
    if not launches:
        raise SystemExit("no sdpa_tc_kernel launch in " + csv_path)

    def mean(metric):
        i = col[metric]
        return sum(float(r[i].replace(",", "")) * mult.get(units[i], 1.0) for r in launches) / len(launches)

    name = launches[0][col["Kernel Name"]]
    out = {"kernel": name[name.index("sdpa_tc_kernel"):].split("(")[0].replace(" ", ""), "launches": len(launches),
           "dram_bytes_read": mean("dram__bytes_read.sum"), "dram_bytes_write": mean("dram__bytes_write.sum"),
           "gpu_time_ns": mean("gpu__time_duration.sum")}
    for extra_metric, key in (("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed", "tensor_pipe_pct"),
                              ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "dram_throughput_pct")):
        if extra_metric in col:
            out[key] = mean(extra_metric)
    with open(TRAFFIC_FILE, "w") as f:
        for k_, v_ in out.items():
            f.write(f"{k_}={v_}\n")
    print(open(TRAFFIC_FILE).read())


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# --------------------------------------------------------------------------------------
# reference arm: the reference's CPU implementation on the host cores
# --------------------------------------------------------------------------------------
def host_cores() -> int:
    """Cores this process may run on (torchrun sets OMP_NUM_THREADS=1 for its children: the CPU
    arm must not inherit that, so the count is taken from the affinity mask)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_inputs(shape):
    g = torch.Generator().manual_seed(1001)
    mk = lambda: torch.randn(shape["B"], shape["H"], shape["S"], shape["D"], generator=g).bfloat16()  # noqa: E731
    return mk(), mk(), mk()


def time_cpu_reference(shape, repeat: int, warmup: int):
    """Times causal bf16 attention of `shape` on the host.  Returns (seconds per pass list, kind,
    threads).  kind = "reference" when the unmodified reference build is present (run in a child
    process with every core this process may use), else "port" (the oracle restatement)."""
    q, k, v = cpu_inputs(shape)
    cores = host_cores()
    ref_so = os.path.join(ROOT, "oracle", "_ref", "_C.so")
    if os.path.exists(ref_so):
        jobs = [{"op": "sdpa", "args": {"q": q, "k": k, "v": v, "is_causal": True},
                 "repeat": 1, "keep_out": False} for _ in range(warmup + repeat)]
        env = dict(os.environ)
        for key in ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "PARAS_REF_THREADS"):
            env[key] = str(cores)
        with tempfile.TemporaryDirectory() as td:
            torch.save(jobs, os.path.join(td, "j.pt"))
            subprocess.check_call([sys.executable, os.path.join(ROOT, "oracle", "ref_run.py"),
                                   os.path.join(td, "j.pt"), os.path.join(td, "r.pt")], env=env)
            res = torch.load(os.path.join(td, "r.pt"))
        return [r["seconds"] for r in res[warmup:]], "reference", res[0]["threads"]
    from oracle import oracle as O
    torch.set_num_threads(cores)
    times = []
    for i in range(warmup + repeat):
        t0 = time.perf_counter()
        O.sdpa(q, k, v, is_causal=True)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return times, "port", torch.get_num_threads()


FULL = dict(B=C2["B"], H=C2["Hq"], S=C2["S"], D=C2["D"])


def sample_desc(shape):
    if shape == FULL:
        return (f"B={shape['B']} H={shape['H']} S={shape['S']} D={shape['D']} causal bf16 = the whole workload "
                f"({shape['B'] * shape['H']}/{C2['B'] * C2['Hq']} (batch, head) units)")
    return (f"B={shape['B']} H={shape['H']} S={shape['S']} D={shape['D']} causal bf16 = "
            f"{shape['B'] * shape['H']}/{C2['B'] * C2['Hq']} of the workload's (batch, head) units")


def choose_cpu_shape(passes: int, budget_s: float):
    """The whole config-2 workload when `passes` passes of it fit `budget_s` on this box's cores
    (estimated from one pass of the 16/256 sample), else the sample.  Returns (shape, estimate)."""
    t, _, _ = time_cpu_reference(CPU_SAMPLE, 1, 0)
    scale = (FULL["B"] * FULL["H"]) / (CPU_SAMPLE["B"] * CPU_SAMPLE["H"])
    est_full = t[0] * scale
    try:
        mem_ok = os.sysconf("SC_PHYS_PAGES") * os.sysconf("SC_PAGE_SIZE") >= 24 << 30  # the reference peaks at about 9 GB on it
    except (ValueError, OSError):
        mem_ok = False
    if mem_ok and passes * est_full <= budget_s:
        return FULL, est_full
    return CPU_SAMPLE, t[0]


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    budget = float(os.environ.get("PARAS_REF_BUDGET_S", "600"))
    shape, _ = choose_cpu_shape(args.steps + args.warmup, budget)
    times, kind, threads = time_cpu_reference(shape, args.steps, args.warmup)
    fl = sdpa_flops(shape["B"], shape["H"], shape["S"], shape["S"], shape["D"], True)
    total = sum(times)
    val = fl * len(times) / total / 1e12
    step = "the whole workload per step" if shape == FULL else "bounded CPU sample: " + sample_desc(shape)
    line = {
        "impl": "reference", "metric": "sdpa_fwd_tflops", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "step": step, "per_gpu_batch": shape["B"]},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                         "sample": sample_desc(shape)},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
def timed_loop(fn, steps, warmup, barrier):
    """fn() launches one step on torch's current stream.  Returns total milliseconds for
    `steps` steps, measured with CUDA events on that stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(stop)


def run_ours(args):
    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no GPU visible; the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    import torch.nn.functional as F
    import torch_paras
    from torch_paras import nn as paras_nn
    from torch_paras import abi

    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # no device_id: with the `paras` backend registered torch reports it as the accelerator
        dist.init_process_group("nccl")

    def barrier():
        # an all-reduce of one CUDA scalar: dist.barrier() would pick the registered `paras`
        # accelerator, which NCCL does not serve
        if dist is not None:
            tok = torch.zeros(1, device=torch.device("cuda", local))
            dist.all_reduce(tok)
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dev = torch.device("cuda", local)
    peaks = measured_peaks()
    steps, warmup = args.steps, max(args.warmup, 3)

    def gen(shape, seed, mean=0.0, std=1.0):
        g = torch.Generator(device=dev).manual_seed(seed * 1000 + rank)
        return (mean + std * torch.randn(shape, generator=g, device=dev)).bfloat16()

    # ---------------- headline: config 2 attention ----------------
    c = C2
    q = gen((c["B"], c["Hq"], c["S"], c["D"]), 1)
    k = gen((c["B"], c["Hkv"], c["S"], c["D"]), 2)
    v = gen((c["B"], c["Hkv"], c["S"], c["D"]), 3)
    out = torch.empty_like(q)
    flops = sdpa_flops(c["B"], c["Hq"], c["S"], c["S"], c["D"], True)

    def step():
        abi.sdpa_fwd(q, k, v, causal=True, out=out, flags=abi.SDPA_REF_SCALE)

    step()
    kernel_name = abi.sdpa_last_kernel()
    with ClockSampler(local) as clk:
        ms = max_over_ranks(timed_loop(step, steps, warmup, barrier))
    ms_step = ms / steps
    tflops = world * flops / (ms_step * 1e-3) / 1e12
    per_gpu_tflops = tflops / world

    roofline = {"bound": "tensor", "kernel": f"sdpa_tc_kernel ({kernel_name})",
                "achieved": per_gpu_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": per_gpu_tflops / peaks["bf16_tflops"], "peak_source": peaks["source"] + " (burst)",
                "frac_of_nominal_2250": per_gpu_tflops / 2250.0,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload, read from
                # the file `bench.py --ingest-ncu` wrote out of an ncu capture (null without one);
                # algorithmic q+k+v+o = 536.9 MB
                "traffic": read_ncu_traffic(), "traffic_unit": "bytes per launch (ncu)",
                "algorithmic_bytes": 4 * c["B"] * c["Hq"] * c["S"] * c["D"] * 2}

    extra = {}
    only = args.only
    esteps = max(5, min(steps, 20))
    s3 = max(3, esteps // 4)

    def want(name):
        return only == name or (only is None and not args.quick)

    def loop_ms(fn, n, w=warmup):
        return max_over_ranks(timed_loop(fn, n, w, barrier)) / n

    if want("config1"):
        # config 1, the fp32 parity configuration (latency-bound): causal attention B=2 H=4 S=128 D=64
        # on the CUDA-core kernel (fp32 at tolerance 1e-4 rules out TF32) + RMSNorm on [256, 256]
        g1 = torch.Generator(device=dev).manual_seed(1000)
        q1, k1, v1 = (torch.randn(2, 4, 128, 64, generator=g1, device=dev) for _ in range(3))
        o1 = torch.empty_like(q1)
        x1 = torch.randn(256, 256, generator=g1, device=dev)
        w1 = 1 + 0.1 * torch.randn(256, generator=g1, device=dev)
        y1_ = torch.empty_like(x1)
        t_a = loop_ms(lambda: abi.sdpa_fwd(q1, k1, v1, causal=True, out=o1, flags=abi.SDPA_REF_SCALE), esteps)
        kname = abi.sdpa_last_kernel()
        t_n = loop_ms(lambda: abi.rmsnorm_fwd(x1, w1, 1e-6, out=y1_, mode=abi.ROUND_PER_OP), esteps)
        extra["config1_fp32_B2_H4_S128_D64"] = {"sdpa_ms": t_a, "sdpa_kernel": kname, "rmsnorm_256x256_ms": t_n,
                                                 "note": "launch-latency bound; parity at 1e-4 is checked by the tests and smoke()"}
        del q1, k1, v1, o1, x1, w1, y1_

    if want("rmsnorm"):
        # RMSNorm, config 2 shape: bytes = 2*rows*H*2 + H*2
        x = gen((16384, 4096), 4)
        w = gen((4096,), 5, mean=1.0, std=0.1)
        y = torch.empty_like(x)
        nbytes = 2 * x.numel() * 2 + w.numel() * 2
        for key, mode in (("rmsnorm_fused_16384x4096", abi.ROUND_ONCE), ("rmsnorm_aten_16384x4096", abi.ROUND_PER_OP)):
            t = loop_ms(lambda: abi.rmsnorm_fwd(x, w, 1e-6, out=y, mode=mode), esteps)
            gbs = nbytes / (t * 1e-3) / 1e9
            extra[key] = {"ms": t, "gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"], "bytes": nbytes}
        # its backward (grad_x and grad_weight in one pass over grad_out and x): bytes = 3*rows*H*2
        _, rstd_ = abi.rmsnorm_fwd(x, w, 1e-6, out=y, return_rstd=True)
        go_ = gen((16384, 4096), 26)
        t = loop_ms(lambda: abi.rmsnorm_bwd(go_, x, w, rstd_), esteps)
        nb = 3 * x.numel() * 2
        extra["rmsnorm_backward_16384x4096"] = {"ms": t, "gbs": nb / (t * 1e-3) / 1e9,
                                                "frac_of_hbm_peak": nb / (t * 1e-3) / 1e9 / peaks["hbm_gbs"], "bytes": nb}
        del x, y, go_, rstd_

    if want("swiglu"):
        # SwiGLU, config 3 shape: bytes = 3*n*2
        srows = 8192 if args.small else 32768
        gate, up = gen((srows, 14336), 6), gen((srows, 14336), 7)
        so = torch.empty_like(gate)
        t = loop_ms(lambda: abi.swiglu_fwd(gate, up, out=so), esteps)
        nbytes = 3 * gate.numel() * 2
        gbs = nbytes / (t * 1e-3) / 1e9
        extra[f"swiglu_{srows}x14336"] = {"ms": t, "gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
                                       "bytes": nbytes}
        # its backward: three tensors read, two written
        t = loop_ms(lambda: abi.swiglu_bwd(so, gate, up), esteps)
        nb = 5 * gate.numel() * 2
        extra[f"swiglu_backward_{srows}x14336"] = {"ms": t, "gbs": nb / (t * 1e-3) / 1e9,
                                                   "frac_of_hbm_peak": nb / (t * 1e-3) / 1e9 / peaks["hbm_gbs"], "bytes": nb}
        del gate, up, so

    if want("gqa"):
        # config 3 attention: B=4 Hq=64 Hkv=8 S=8192
        q3, k3, v3 = gen((4, 64, 8192, 128), 8), gen((4, 8, 8192, 128), 9), gen((4, 8, 8192, 128), 10)
        o3 = torch.empty_like(q3)
        t = loop_ms(lambda: abi.sdpa_fwd(q3, k3, v3, causal=True, out=o3), s3, 3)
        f3 = sdpa_flops(4, 64, 8192, 8192, 128, True)
        tf = f3 / (t * 1e-3) / 1e12
        extra["sdpa_gqa_B4_Hq64_Hkv8_S8192"] = {"ms": t, "tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"],
                                                 "kernel": abi.sdpa_last_kernel()}
        del q3, k3, v3, o3

    if want("variants"):
        # the other instantiations of the tcgen05 kernel at config 2's batch and sequence: head dim 64
        # (half the tensor work per exponential) and explicit masks (bool key padding [B,1,1,S];
        # additive [S,S] in the tensors' dtype, a row of which every softmax thread reads per kv tile)
        res = {}
        qv, kv_, vv = gen((8, 32, 2048, 128), 40), gen((8, 32, 2048, 128), 41), gen((8, 32, 2048, 128), 42)
        ov = torch.empty_like(qv)
        pad = torch.ones(8, 1, 1, 2048, dtype=torch.bool, device=dev)
        pad[:, :, :, 1900:] = False
        add = (0.5 * torch.randn(2048, 2048, device=dev, generator=torch.Generator(device=dev).manual_seed(43))).to(qv.dtype)
        for key, kw in (("full_nomask", {}), ("bool_padding_mask_B11S", {"mask": pad}), ("additive_mask_SS", {"mask": add})):
            t = loop_ms(lambda: abi.sdpa_fwd(qv, kv_, vv, out=ov, **kw), esteps)
            tf = sdpa_flops(8, 32, 2048, 2048, 128, False) / (t * 1e-3) / 1e12
            res[key] = {"ms": t, "tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"], "kernel": abi.sdpa_last_kernel()}
        del qv, kv_, vv, ov
        q6, k6, v6 = gen((8, 32, 2048, 64), 44), gen((8, 32, 2048, 64), 45), gen((8, 32, 2048, 64), 46)
        o6 = torch.empty_like(q6)
        for key, causal in (("d64_causal", True), ("d64_full", False)):
            t = loop_ms(lambda: abi.sdpa_fwd(q6, k6, v6, causal=causal, out=o6), esteps)
            tf = sdpa_flops(8, 32, 2048, 2048, 64, causal) / (t * 1e-3) / 1e12
            res[key] = {"ms": t, "tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"], "kernel": abi.sdpa_last_kernel()}
        del q6, k6, v6, o6
        extra["sdpa_variants_B8_H32_S2048"] = res
        # few query positions against a long key range (a prompt chunk, or the tokens a speculative step
        # verifies): too few (batch, head, query block) units to fill the GPU, so the key range runs in
        # pieces; with GQA the heads of a group share one pass over K/V.  HBM floor = K + V once per kv head.
        res = {}
        for key, (b_, lq_, lk_) in (("chunk_B1_Lq512_Lk32768", (1, 512, 32768)), ("verify_B8_Lq64_Lk16384", (8, 64, 16384)),
                                    ("verify_B8_Lq16_Lk16384", (8, 16, 16384))):
            qs_, ks_, vs_ = gen((b_, 32, lq_, 128), 47), gen((b_, 8, lk_, 128), 48), gen((b_, 8, lk_, 128), 49)
            os_ = torch.empty_like(qs_)
            t = loop_ms(lambda: abi.sdpa_fwd(qs_, ks_, vs_, out=os_, flags=abi.SDPA_FORCE_TENSOR), esteps)
            tf = sdpa_flops(b_, 32, lq_, lk_, 128, False) / (t * 1e-3) / 1e12
            gbs = (ks_.numel() + vs_.numel() + 2 * qs_.numel()) * 2 / (t * 1e-3) / 1e9
            res[key] = {"ms": t, "tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"], "gbs": gbs,
                        "frac_of_hbm_peak": gbs / peaks["hbm_gbs"], "kernel": abi.sdpa_last_kernel()}
            del qs_, ks_, vs_, os_
        extra["sdpa_short_queries_Hq32_Hkv8_D128"] = res

    if want("decode"):
        # config 4 decode: bytes = K + V (once per kv head) + q + o
        db = 8 if args.small else 64
        qd, kd, vd = gen((db, 32, 1, 128), 11), gen((db, 8, 32768, 128), 12), gen((db, 8, 32768, 128), 13)
        od = torch.empty_like(qd)
        ws_bytes = abi.sdpa_workspace_bytes(qd, kd, vd)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        t = loop_ms(lambda: abi.sdpa_fwd(qd, kd, vd, out=od, workspace=ws if ws_bytes else None), s3, 3)
        nbytes = (kd.numel() + vd.numel() + qd.numel() + od.numel()) * 2
        gbs = nbytes / (t * 1e-3) / 1e9
        extra[f"sdpa_decode_B{db}_kv32768"] = {"ms": t, "gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
                                            "bytes": nbytes, "kernel": abi.sdpa_last_kernel()}
        # the same step over caches of different lengths: a bool key-padding mask [B,1,1,kv]
        padm = torch.ones(db, 1, 1, 32768, dtype=torch.bool, device=dev)
        padm[:, :, :, 30000:] = False
        t = loop_ms(lambda: abi.sdpa_fwd(qd, kd, vd, out=od, mask=padm, workspace=ws if ws_bytes else None), s3, 3)
        # the kernel stops at the last valid key of each batch element: only the 30000 valid keys count as bytes
        vbytes = (kd.numel() + vd.numel()) * 2 * 30000 // 32768 + (qd.numel() + od.numel()) * 2
        gbs = vbytes / (t * 1e-3) / 1e9
        extra[f"sdpa_decode_padding_mask_B{db}_kv32768"] = {"ms": t, "gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
                                                         "bytes": vbytes, "valid_keys": 30000, "kernel": abi.sdpa_last_kernel()}
        # caches of 1000 .. 32000 valid keys in one batch
        lens = [1000 + (i * 499) % 31000 for i in range(db)]
        for i, n_ in enumerate(lens):
            padm[i, :, :, :n_] = True
            padm[i, :, :, n_:] = False
        t = loop_ms(lambda: abi.sdpa_fwd(qd, kd, vd, out=od, mask=padm, workspace=ws if ws_bytes else None), s3, 3)
        vbytes = sum(lens) * 8 * 128 * 2 * 2 + (qd.numel() + od.numel()) * 2
        gbs = vbytes / (t * 1e-3) / 1e9
        extra[f"sdpa_decode_ragged_B{db}_kv1000_to_32000"] = {"ms": t, "gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
                                                            "bytes": vbytes, "mean_valid_keys": sum(lens) / db,
                                                            "kernel": abi.sdpa_last_kernel()}
        del padm
        # One decoder layer of that step (hidden 4096, Hq=32, Hkv=8, D=128, FFN 14336, batch db): RMSNorm folded
        # into the QKV projection, decode attention, output projection, RMSNorm folded into the gate/up projection
        # with SwiGLU, down projection.  Bytes = the layer's weights (436 MB) + its KV cache + activations; the
        # launches queue behind a spin kernel so that the events see device time.
        hid, ffn = 4096, 14336
        xl = gen((db, hid), 70)
        wn1 = gen((hid,), 71, mean=1.0, std=0.1)
        w_qkv, w_o = gen((6144, hid), 72, std=0.02), gen((hid, hid), 73, std=0.02)
        w_g, w_u, w_d = gen((ffn, hid), 74, std=0.02), gen((ffn, hid), 75, std=0.02), gen((hid, ffn), 76, std=0.02)
        w_qkv_f = abi.scale_columns(w_qkv, wn1)
        qkv = torch.empty((db, 6144), dtype=torch.bfloat16, device=dev)
        att = torch.empty((db, 32, 1, 128), dtype=torch.bfloat16, device=dev)
        h1, ff, h2 = (torch.empty((db, n_), dtype=torch.bfloat16, device=dev) for n_ in (hid, ffn, hid))

        def layer():
            abi.gemm(xl, w_qkv_f, row_scale=abi.rms_rstd(xl, 1e-6), out=qkv)
            qv = qkv[:, :4096].view(db, 32, 1, 128)          # (the new token's k, v would be appended to the cache here)
            abi.sdpa_fwd(qv, kd, vd, out=att, workspace=ws if ws_bytes else None)
            abi.gemm(att.view(db, hid), w_o, out=h1)
            abi.gemm(h1, w_g, up_weight=w_u, out=ff)          # (a second norm would fold into w_g, w_u like the first)
            abi.gemm(ff, w_d, out=h2)

        for _ in range(3):
            layer()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(int(4e7))
        e0.record()
        for _ in range(5):
            layer()
        e1.record()
        torch.cuda.synchronize()
        t_layer = e0.elapsed_time(e1) / 5
        wbytes = (w_qkv.numel() + w_o.numel() + w_g.numel() + w_u.numel() + w_d.numel()) * 2
        lbytes = wbytes + (kd.numel() + vd.numel()) * 2
        extra[f"decode_layer_B{db}_kv32768"] = {
            "ms": t_layer, "ms_attention_alone": extra[f"sdpa_decode_B{db}_kv32768"]["ms"], "weight_bytes": wbytes,
            "gbs": lbytes / (t_layer * 1e-3) / 1e9, "frac_of_hbm_peak": lbytes / (t_layer * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "note": "rms_rstd + QKV projection (row-scale epilogue), decode attention, output projection, gate/up projection "
                    "with SwiGLU, down projection: five weight-streaming GEMM launches around the attention kernel"}
        del xl, wn1, w_qkv, w_o, w_g, w_u, w_d, w_qkv_f, qkv, att, h1, ff, h2
        del qd, kd, vd, od, ws
    if want("block"):
        # config 5, one GPU's share (B=64 over 8 GPUs -> 8 batch elements here): RMSNorm -> causal GQA
        # attention -> RMSNorm -> SwiGLU, hidden 4096 (Hq=32, Hkv=8, D=128), S=4096, FFN width 14336.
        # q/k/v and gate/up stand for the projections' outputs (the GEMMs are outside the path).
        Bp = 2 if args.small else 8
        rows = Bp * 4096
        xh = gen((rows, 4096), 14)
        wn = gen((4096,), 15, mean=1.0, std=0.1)
        qb, kb, vb = gen((Bp, 32, 4096, 128), 16), gen((Bp, 8, 4096, 128), 17), gen((Bp, 8, 4096, 128), 18)
        gb, ub = gen((rows, 14336), 19), gen((rows, 14336), 20)
        y1, ob, y2, sb = torch.empty_like(xh), torch.empty_like(qb), torch.empty_like(xh), torch.empty_like(gb)

        def block():
            abi.rmsnorm_fwd(xh, wn, 1e-6, out=y1, mode=abi.ROUND_PER_OP)
            abi.sdpa_fwd(qb, kb, vb, causal=True, out=ob, flags=abi.SDPA_REF_SCALE)
            abi.rmsnorm_fwd(ob.view(rows, 4096), wn, 1e-6, out=y2, mode=abi.ROUND_PER_OP)
            abi.swiglu_fwd(gb, ub, out=sb)

        stages = {
            "rmsnorm": lambda: abi.rmsnorm_fwd(xh, wn, 1e-6, out=y1, mode=abi.ROUND_PER_OP),
            "sdpa": lambda: abi.sdpa_fwd(qb, kb, vb, causal=True, out=ob, flags=abi.SDPA_REF_SCALE),
            "swiglu": lambda: abi.swiglu_fwd(gb, ub, out=sb),
        }
        res = {"per_gpu_batch": Bp, "ms_total": loop_ms(block, s3, 3)}
        for name, fn in stages.items():
            res["ms_" + name] = loop_ms(fn, s3, 3)
        fl = sdpa_flops(Bp, 32, 4096, 4096, 128, True)
        res["sdpa_tflops"] = fl / (res["ms_sdpa"] * 1e-3) / 1e12
        res["rmsnorm_gbs"] = (2 * rows * 4096 * 2 + 8192) / (res["ms_rmsnorm"] * 1e-3) / 1e9
        res["swiglu_gbs"] = 3 * rows * 14336 * 2 / (res["ms_swiglu"] * 1e-3) / 1e9
        res["global_batch_all_ranks"] = Bp * world
        extra["config5_decoder_block_share"] = res
        del xh, qb, kb, vb, gb, ub, y1, ob, y2, sb
    if want("bwd"):
        # Attention backward at the headline shape (config 2): forward with lse, then dq, dk, dv.
        # FLOPs counted as 2.5x the forward's algorithmic FLOPs (five products instead of two),
        # causal half only (the kernels skip the blocks a causal mask empties).
        Bb = 2 if args.small else c["B"]
        qb_, kb_, vb_ = q[:Bb].contiguous(), k[:Bb].contiguous(), v[:Bb].contiguous()
        dob = gen((Bb, c["Hq"], c["S"], c["D"]), 25)
        ob, lseb = abi.sdpa_fwd(qb_, kb_, vb_, causal=True, return_lse=True)
        t = loop_ms(lambda: abi.sdpa_bwd(dob, qb_, kb_, vb_, ob, lseb, causal=True), esteps, 3)
        t_c = loop_ms(lambda: abi.sdpa_bwd(dob, qb_, kb_, vb_, ob, lseb, causal=True, composite=True), s3, 3)
        fl = 2.5 * sdpa_flops(Bb, c["Hq"], c["S"], c["S"], c["D"], True)
        extra[f"sdpa_backward_B{Bb}_H{c['Hq']}_S{c['S']}"] = {
            "ms": t, "tflops": fl / (t * 1e-3) / 1e12, "frac_of_bf16_peak": fl / (t * 1e-3) / 1e12 / peaks["bf16_tflops"],
            "note": "fused tcgen05 kernels (dQ, which also forms delta, then dK/dV; S and dP recomputed in each: "
                    "7 tile products, counted as the 5 the gradient needs)",
            "composite_ms": t_c, "composite_tflops": fl / (t_c * 1e-3) / 1e12}
        del qb_, kb_, vb_, dob, ob, lseb
    if want("rope"):
        # Rotary embedding in front of the headline attention: two rotation passes + attention against the
        # one call that rotates the queries inside the attention kernel and the keys once on the way in
        pos = torch.arange(c["S"], device=dev, dtype=torch.float64)[:, None]
        inv = 1.0 / (10000.0 ** (torch.arange(0, c["D"], 2, device=dev, dtype=torch.float64) / c["D"]))
        ang = torch.cat((pos * inv, pos * inv), dim=-1)
        cos_t, sin_t = ang.cos().bfloat16().contiguous(), ang.sin().bfloat16().contiguous()
        t_sep = loop_ms(lambda: abi.sdpa_fwd(abi.rope(q, cos_t, sin_t), abi.rope(k, cos_t, sin_t), v, causal=True,
                                             out=out, flags=abi.SDPA_REF_SCALE), s3, 3)
        t_fus = loop_ms(lambda: abi.sdpa_rope_fwd(q, k, v, cos_t, sin_t, causal=True, out=out, flags=abi.SDPA_REF_SCALE), s3, 3)
        extra["rope_then_sdpa_config2"] = {
            "ms_separate": t_sep, "ms_fused": t_fus, "ms_attention_alone": ms_step, "kernel": abi.sdpa_last_kernel(),
            "hbm_bytes_saved": 2 * q.numel() * 2,
            "note": "fused = keys rotated once into scratch, queries rotated in shared memory inside the attention "
                    "kernel (no rotated copy of q is written or read)"}
        del cos_t, sin_t

    if want("gemm"):
        # The projections either side of the path at config 2 / 5 sizes (hidden 4096, FFN 14336):
        # fused QKV projection [rows,4096] x [6144,4096]^T (Hq=32, Hkv=8, D=128) and the gate/up
        # projection with SwiGLU in the epilogue; FLOPs = 2*M*N*K (x2 for the two FFN weights).
        rows = 4096 if args.small else 16384
        xg = gen((rows, 4096), 21)
        wqkv = gen((6144, 4096), 22, std=0.02)
        wgate, wup = gen((14336, 4096), 23, std=0.02), gen((14336, 4096), 24, std=0.02)
        oq = torch.empty((rows, 6144), dtype=torch.bfloat16, device=dev)
        of = torch.empty((rows, 14336), dtype=torch.bfloat16, device=dev)
        # The QKV projection in a decode step first (rows = the batch of config 4; measured before the large GEMMs,
        # which leave the GPU at its power cap for a while): a weight-streaming GEMM,
        # bytes = the weight once.  The weight rows sit on the MMA's M side, K is split inside a cluster.
        # Eight weights are cycled (400 MB, more than L2) so that every call streams its weight from HBM;
        # a call lasts less than the host needs to issue it, so the launches queue behind a spin kernel
        # and the events bracket device time only.
        xd = gen((64, 4096), 27)
        od = torch.empty((64, 6144), dtype=torch.bfloat16, device=dev)
        wcyc = [wqkv] + [gen((6144, 4096), 60 + i, std=0.02) for i in range(7)]
        for wc in wcyc:
            abi.gemm(xd, wc, out=od)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(int(4e7))
        e0.record()
        for _ in range(3):
            for wc in wcyc:
                abi.gemm(xd, wc, out=od)
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / 24
        gbs = (wqkv.numel() + xd.numel() + od.numel()) * 2 / (t * 1e-3) / 1e9
        extra["gemm_decode_qkv_64x6144x4096"] = {"ms": t, "gb_per_s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
                                                 "note": "weight-streaming kernel (gemm_skinny.cu), weights read from HBM; a 50 MB "
                                                         "weight is 7.7 us at the copy peak, the rest is launch and pipeline fill"}
        t = loop_ms(lambda: abi.gemm(xg, wqkv, out=oq), s3, 3)
        tf = 2.0 * rows * 6144 * 4096 / (t * 1e-3) / 1e12
        extra[f"gemm_qkv_{rows}x6144x4096"] = {"ms": t, "tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}
        t = loop_ms(lambda: abi.gemm(xg, wgate, up_weight=wup, out=of), s3, 3)
        tf = 4.0 * rows * 14336 * 4096 / (t * 1e-3) / 1e12
        extra[f"gemm_swiglu_{rows}x14336x4096"] = {"ms": t, "tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"]}
        # RMSNorm folded into the QKV projection (rstd pass + row-scale epilogue; the norm weight folded
        # into the projection weight beforehand) against the two separate kernels
        wn_ = gen((4096,), 26, mean=1.0, std=0.1)
        wfold = abi.scale_columns(wqkv, wn_)
        yn = torch.empty_like(xg)
        # the two forms alternate and each keeps its best pass: a GEMM of this size moves by a few per cent
        # with the power state the previous measurements left, more than the 20 us the fold saves
        sep = lambda: (abi.rmsnorm_fwd(xg, wn_, 1e-6, out=yn), abi.gemm(yn, wqkv, out=oq))  # noqa: E731
        fus = lambda: abi.gemm(xg, wfold, row_scale=abi.rms_rstd(xg, 1e-6), out=oq)          # noqa: E731
        t_sep = t_fus = float("inf")
        for _ in range(3):
            t_sep = min(t_sep, loop_ms(sep, esteps, 3))
            t_fus = min(t_fus, loop_ms(fus, esteps, 3))
        extra[f"rmsnorm_then_qkv_{rows}x6144x4096"] = {
            "ms_separate": t_sep, "ms_fused": t_fus,
            "hbm_bytes_saved": 2 * xg.numel() * 2,
            "note": "fused = one read of x for rstd + GEMM with rows scaled in the epilogue; the normalised "
                    "activations (one write, one read) never exist"}
        del xg, wqkv, wgate, wup, oq, of, wn_, wfold, yn, xd, od, wcyc
    torch.cuda.empty_cache()

    if only:
        if rank == 0:
            print(json.dumps({"only": only, "n_gpus": world, "headline_sdpa_tflops": tflops, "extra": extra}),
                  flush=True)
        if dist is not None:
            barrier()
            dist.destroy_process_group()
        return

    # ---------------- e2e: public operator on the paras device, host buffers ----------------
    pdev = f"paras:{local + 1}"
    # each rank feeds its GPU from host memory of the GPU's own NUMA node (buffers are pinned below,
    # after the binding, so their pages land there)
    from torch_paras import sharding as _sh
    numa_cpus = _sh.bind_host_to_gpu_node(local) if not args.no_numa_bind else []
    hq, hk, hv = (t_.cpu().pin_memory() for t_ in (q, k, v))
    h2d = (hq.numel() + hk.numel() + hv.numel()) * 2
    d2h = hq.numel() * 2

    def e2e_device_step():
        dq = hq.to(pdev, non_blocking=True)
        dk = hk.to(pdev, non_blocking=True)
        dv = hv.to(pdev, non_blocking=True)
        return F.scaled_dot_product_attention(dq, dk, dv, is_causal=True).cpu()

    hout = torch.empty(hq.shape, dtype=hq.dtype, pin_memory=True)

    def e2e_step():
        return paras_nn.attention_host(hq, hk, hv, is_causal=True, out=hout, device=local + 1)

    def time_host_loop(fn, n):
        for _ in range(2):
            fn()
        torch_paras.synchronize(local + 1)
        barrier()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        torch_paras.synchronize(local + 1)
        return max_over_ranks((time.perf_counter() - t0) / n * 1e3) * 1e-3

    def link_gbs():
        """Plain pinned copies of q to the GPU and of the result back, one direction at a time: the
        link's own rate on this box, beside which the pipelined figure can be read."""
        dq_ = torch.empty_like(q)
        res = {}
        for name, fn, nbytes in (("h2d", lambda: dq_.copy_(hq, non_blocking=True), hq.numel() * 2),
                                 ("d2h", lambda: hout.copy_(dq_, non_blocking=True), hq.numel() * 2)):
            fn()
            torch.cuda.synchronize()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                fn()
            e1.record()
            torch.cuda.synchronize()
            res[name] = 3 * nbytes / (max_over_ranks(e0.elapsed_time(e1)) * 1e-3) / 1e9
        return res

    e2e_steps = max(2, min(steps, 5))
    dev_s = time_host_loop(e2e_device_step, e2e_steps)
    e2e_s = time_host_loop(e2e_step, e2e_steps)
    e2e = {"value": world * flops / e2e_s / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_s * 1e3,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "api": "torch_paras.nn.attention_host: pinned host q/k/v in, pinned host result out, "
                  "batch chunks pipelined over three streams",
           "link_gbs_per_gpu_alone": link_gbs(), "numa_bound_cpus": len(numa_cpus),
           "achieved_h2d_gbs_per_gpu": h2d / e2e_s / 1e9,
           "device_api": {"value": world * flops / dev_s / 1e12, "ms_per_step": dev_s * 1e3,
                          "api": "pinned host q/k/v .to(paras:N), F.scaled_dot_product_attention, .cpu()"}}

    # The headline launch back to back for at least `--sustain-s` seconds: what the kernel holds once
    # the power cap and the clock have settled (the K-step headline loop is a few milliseconds: a
    # burst).  It runs last: the seconds under the power cap would otherwise colour every loop after it.
    sustained = None
    if args.sustain_s > 0 and not args.quick and not args.only:
        n_sus = max(steps, int(math.ceil(args.sustain_s * 1e3 / ms_step)))
        with ClockSampler(local, period_s=0.02) as clk_s:
            ms_s = max_over_ranks(timed_loop(step, n_sus, 1, barrier))
        cs = clk_s.summary()
        tf_s = flops / (ms_s / n_sus * 1e-3) / 1e12
        sustained = {"value": world * tf_s, "unit": "TFLOP/s", "per_gpu": tf_s, "launches": n_sus,
                     "seconds": ms_s * 1e-3, "ms_per_step": ms_s / n_sus,
                     "peak": peaks["bf16_tflops_sustained"],
                     "frac_of_sustained_peak": (tf_s / peaks["bf16_tflops_sustained"]) if peaks["bf16_tflops_sustained"] else None,
                     "clocks": cs,
                     # time x clock: comparable across runs whose clocks differ
                     "ms_x_mhz": (ms_s / n_sus * cs["sm_mhz"]) if cs["sm_mhz"] else None}
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        # about 10-30 s of CPU work: one pass of the whole workload where that fits, else the sample
        shape, _ = choose_cpu_shape(1, 30.0)
        rep = 1 if shape == FULL else args.cpu_repeat
        times, kind, threads = time_cpu_reference(shape, rep, 0 if shape == FULL else 1)
        fl = sdpa_flops(shape["B"], shape["H"], shape["S"], shape["S"], shape["D"], True)
        cpu_baseline = {"value": fl * len(times) / sum(times) / 1e12, "unit": "TFLOP/s", "cores": threads,
                        "kind": kind, "sample": sample_desc(shape), "seconds_per_pass": sum(times) / len(times)}

    gathered = None
    if dist is not None:
        # Optional re-assembly of the sharded outputs (outside every timed region): one head of
        # every rank's output, all-gathered over NCCL.
        from torch_paras import sharding
        piece = out[:, :1].contiguous()
        full = sharding.gather_shards(piece, [piece.shape[0]] * world, dim=0)
        torch.cuda.synchronize()
        gathered = list(full.shape)

    if rank == 0:
        line = {
            "metric": "sdpa_fwd_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_gpu_batch": c["B"], "global_batch": c["B"] * world,
                       "l2": "inputs (537 MB per step) larger than the 126 MB L2; no flush",
                       "sharding": "batch shards, one per rank, no collective on the forward path",
                       "gathered_output_shape": gathered},
            "value_sustained": sustained["value"] if sustained else None, "sustained": sustained,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": steps, "clocks": clk.summary(), "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--quick", action="store_true", help="headline + e2e only")
    ap.add_argument("--small", action="store_true",
                    help="shrink the extra workloads (SwiGLU 8192 rows, decode batch 8) so that a profiler "
                         "capture holds about 1 GB on the device; rates stay per-byte comparable")
    ap.add_argument("--sustain-s", type=float, default=2.0,
                    help="seconds of back-to-back headline launches for the sustained figure (0 = skip)")
    ap.add_argument("--ingest-ncu", metavar="CSV",
                    help="write profiles/sdpa_tc_kernel_config2_dram_traffic.txt from `ncu --page raw --csv` output and exit")
    ap.add_argument("--only", choices=["rope", "config1", "rmsnorm", "swiglu", "gqa", "variants", "decode", "block", "gemm", "bwd"],
                    help="after the headline loop run just this extra workload and print it (for profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-numa-bind", action="store_true",
                    help="leave the process where the launcher put it instead of binding it to the GPU's NUMA node for e2e")
    ap.add_argument("--cpu-repeat", type=int, default=3)
    args = ap.parse_args()
    if args.ingest_ncu:
        ingest_ncu(args.ingest_ncu)
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
