#!/usr/bin/env python
"""Benchmark of the Nystrom-attention forward + exact backward hot path.

    python bench.py --gpus N --steps K --warmup W            # this library, on N GPUs
    python bench.py --impl reference --steps K --warmup W    # the reference algorithm on host cores

A step is one forward + backward over one batch of synthetic input.  At every N each GPU runs
the north-star workload B=1, H=16, N=65536, D=64, fp16, num_landmarks=64, newton_iter=6,
kappa_star=0 (batch-parallel weak scaling: independent (b,h) slices, no collective on the data
path).  One JSON line is printed by rank 0:

  value      whole-job tokens/s (tokens = B*N per call, all heads) with inputs resident in HBM
  e2e        the same through the public Python API with pinned HOST buffers: the four input
             copies host->device and the four result copies device->host are inside the timing
  roofline   dominant kernel: algorithmic bytes per launch / its mean CUDA-event duration,
             against the measured copy bandwidth in MEASURED_PEAKS.json
  cpu_baseline  the CPU oracle port of reference.py timed on this box's cores on a bounded
             sample of the same workload
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = dict(B=1, H=16, N=65536, D=64, m=64, J=6, kappa_star=0.0)
WORKLOAD_NAME = "config3: B=1,H=16,N=65536,D=64 fp16, m=64, J=6, kappa*=0, fwd+bwd, dO~N(0,1)"
METRIC = "fwd+bwd tokens/s/GPU at N=64K,m=64,D=64 fp16; % of HBM roofline"
FALLBACK_HBM_GBS = 6650.0

# N*D-sized tensor passes each kernel must make (reads + writes), per (b,h) slice.
KERNEL_PASSES = {
    "landmark_partial": 2, "gen_fwd_b": 2, "gen_fwd_c": 2, "gen_bwd_a": 2, "gen_bwd_b": 4,
    "gen_bwd_c": 3,
    # tc_bwd_a also writes its dS1 tiles (into dq), tc_bwd_b writes dS3' tiles (into dk) and dV,
    # tc_bwd_c reads both sets of tiles and writes dQ and dK in place
    "tc_pool_q": 1, "tc_fwd_b": 2, "tc_fwd_c": 2, "tc_bwd_a": 3, "tc_bwd_b": 4, "tc_bwd_c": 4,
}


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback 6650 GB/s"


def ncu_traffic(kernel):
    """DRAM bytes per launch of `kernel` (dram__bytes_read.sum + dram__bytes_write.sum) from the
    table of the committed ncu summary of this workload, if it is there."""
    path = os.path.join(ROOT, "profiles", "step_config3_kernels.md")
    try:
        with open(path) as f:
            for line in f:
                cells = [c.strip() for c in line.strip().strip("|").split("|")]
                if len(cells) >= 6 and cells[0] == kernel:
                    return int(round((float(cells[4]) + float(cells[5])) * 1e6))
    except Exception:
        pass
    return None


class ClockSampler:
    """SM clock and throttle-reason samples taken WHILE the timed region runs.

    The timed region is tens of milliseconds, far shorter than nvidia-smi's polling interval, so the
    samples come from NVML in a thread of this process (about one per millisecond); the nvidia-smi
    query of the same fields is only the fallback when NVML cannot be loaded."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                   0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.file = None
        self.nvml = None
        self.handle = None
        self.thread = None
        self.stop = threading.Event()
        self.samples = []          # (sm_mhz, reasons bitmask)
        self.sm_max = None

    def _nvml_open(self):
        import pynvml
        import torch
        pynvml.nvmlInit()
        try:
            pr = torch.cuda.get_device_properties(self.index)
            bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
            self.handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        self.nvml = pynvml

    def sample_now(self):
        """One NVML sample from the calling thread (no-op without NVML)."""
        nv, h = self.nvml, self.handle
        if nv is None:
            time.sleep(0.001)
            return
        try:
            mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
            try:
                bits = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
            except Exception:
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
            self.samples.append((float(mhz), int(bits)))
        except Exception:
            pass

    def _poll(self):
        while not self.stop.is_set():
            self.sample_now()
            time.sleep(0.0005)

    def __enter__(self):
        try:
            self._nvml_open()
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.thread is not None:
            self.stop.set()
            self.thread.join(timeout=5)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.nvml is not None:
            sm = [x for x, _ in self.samples]
            bits = 0
            for _, b in self.samples:
                bits |= b
            out.update(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=self.sm_max,
                       reasons=sorted(n for bit, n in self.REASON_BITS.items() if bits & bit),
                       samples=len(sm), source="nvml")
            return out
        if self.file is None:
            return out
        try:
            self.file.flush()
            rows = [r.split(",") for r in open(self.file.name).read().strip().splitlines() if r.strip()]
            os.unlink(self.file.name)
            sm = [float(r[1]) for r in rows]
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            reasons = set()
            for r in rows:
                for name, cell in zip(names, r[5:9]):
                    if cell.strip().lower().startswith("active"):
                        reasons.add(name)
            out.update(sm_mhz=statistics.median(sm) if sm else None,
                       sm_max_mhz=float(rows[0][2]) if rows else None,
                       reasons=sorted(reasons), samples=len(rows))
        except Exception as e:  # clocks are evidence, not a reason to lose the measurement
            out["error"] = repr(e)
        return out


def cpu_reference_step(q, k, v, dO, w):
    from oracle import nystrom_oracle as O
    return O.forward_backward_autograd(q, k, v, dO, w["m"], w["J"], w["kappa_star"])


def cpu_sample_inputs(w, heads):
    import torch
    from oracle import nystrom_oracle as O
    q, k, v, dO = O.make_inputs(w["B"], heads, w["N"], w["D"], seed=0, dtype=torch.float16)
    return tuple(t.float() for t in (q, k, v, dO))


def time_cpu(w, heads, steps, warmup):
    """Mean seconds per step of the oracle port on `heads` of the workload's H heads."""
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    q, k, v, dO = cpu_sample_inputs(w, heads)
    for _ in range(warmup):
        cpu_reference_step(q, k, v, dO, w)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_reference_step(q, k, v, dO, w)
    dt = (time.perf_counter() - t0) / steps
    tokens_per_s = w["B"] * w["N"] / (dt * w["H"] / heads)
    return dt, tokens_per_s, cores, torch.get_num_threads()


def run_reference(args, rank):
    """The reference algorithm (CPU port of reference.py: oracle/nystrom_oracle.py, which the test
    suite pins bit-for-bit to reference.py in FP32) on the host cores."""
    if rank != 0:
        return
    w = WORKLOAD
    heads = 2
    dt, tps, cores, threads = time_cpu(w, heads, max(args.steps, 1), max(args.warmup, 0))
    sample = (f"{heads} of {w['H']} heads at full N={w['N']} per step, FP32, torch CPU "
              f"({threads} threads); tokens/s scaled by {w['H']}/{heads}")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3 * w["H"] / heads, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME, **w},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true",
                    help="skip the host-buffer end-to-end section (used for the ncu launch list, so that only\n"
                         "the device-resident steps are listed)")
    ap.add_argument("--heads", type=int, default=None, help="override H (debug only)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    from flashnystrom_b200 import _C, flash_nystrom_attention
    from oracle import nystrom_oracle as O  # only for seeded input generation and cpu_baseline

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    w = dict(WORKLOAD)
    if args.heads:
        w["H"] = args.heads
    B, H, N, D, m, J = w["B"], w["H"], w["N"], w["D"], w["m"], w["J"]
    steps, warmup = max(args.steps, 1), max(args.warmup, 3)

    # ---- inputs: pinned host originals + device-resident copies ------------------------------
    hq, hk, hv, hdO = (t.pin_memory() for t in O.make_inputs(B, H, N, D, seed=rank, dtype=torch.float16))
    q, k, v = (t.to(dev).requires_grad_(True) for t in (hq, hk, hv))
    dO = hdO.to(dev)
    elem_bytes = B * H * N * D * 2

    def step_resident():
        q.grad = k.grad = v.grad = None
        out = flash_nystrom_attention(q, k, v, num_landmarks=m, newton_iter=J)
        out.backward(dO)
        return out

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing --------------------------------------------------------------
    for _ in range(warmup):
        step_resident()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record()
        for _ in range(steps):
            step_resident()
        e1.record()
        # the launches above are asynchronous: while the GPU works through them, also sample
        # from this thread (the sampler thread competes with the launch loop for the interpreter)
        while not e1.query():
            clocks.sample_now()
        barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / steps
    tokens_per_s = world * B * N / (ms_step * 1e-3)
    clock_summary = clocks.summary()

    # ---- per-kernel durations (CUDA events around each launch, same stream) -------------------
    _C.set_profiling(True)
    per_kernel = {}
    launches_per_step = 0
    for it in range(steps):
        q.grad = k.grad = v.grad = None
        res = _C.forward(q.detach(), k.detach(), v.detach(), m, J, 0.0, False, True)
        pf = _C.last_profile()
        _C.backward(dO, *res[1:13], v.detach(), res[0], m, J, True, 0.0)
        pb = _C.last_profile()
        launches_per_step = len(pf) + len(pb)
        for name, ms in pf + pb:
            per_kernel.setdefault(name, []).append(ms)
    _C.set_profiling(False)
    torch.cuda.synchronize()
    # Outside profiling mode the backward column pass runs beside the pseudoinverse backward (side
    # stream) and takes its operands from one extra small kernel, bwd_mid1, that the one-by-one
    # profile does not launch.
    if "tc_bwd_b" in per_kernel and B * H * 4 <= torch.cuda.get_device_properties(dev).multi_processor_count:
        launches_per_step += 1
    kernel_ms = {n: sum(v_) / len(v_) for n, v_ in per_kernel.items()}
    total_kernel_ms = sum(kernel_ms.values())
    # The roofline is quoted for the HBM-streaming kernel with the longest launch (the pooling and
    # tensor-core passes move N-sized tensors); the Newton-Schulz and landmark-sized glue kernels
    # move kilobytes and are reported through kernel_ms / kernel_share and the whole-step figure.
    streaming = {n: t for n, t in kernel_ms.items() if KERNEL_PASSES.get(n, 0) > 0}
    top = max(streaming, key=streaming.get) if streaming else max(kernel_ms, key=kernel_ms.get)
    peak, peak_src = hbm_peak()
    top_bytes = KERNEL_PASSES.get(top, 0) * elem_bytes
    achieved = top_bytes / (kernel_ms[top] * 1e-3) / 1e9 if top_bytes else 0.0
    step_bytes = 11 * elem_bytes
    roofline = {
        "bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak, "traffic": ncu_traffic(top), "peak_source": peak_src,
        "algorithmic_bytes_per_launch": top_bytes,
        "kernel_ms": {n: round(t, 4) for n, t in kernel_ms.items()},
        "kernel_share": {n: round(t / total_kernel_ms, 4) for n, t in kernel_ms.items()},
        "step": {"algorithmic_bytes": step_bytes,
                 "achieved": step_bytes / (ms_step * 1e-3) / 1e9,
                 "frac": step_bytes / (ms_step * 1e-3) / 1e9 / peak},
    }

    e2e = None
    if not args.no_e2e:
        # ---- end to end through the public API with pinned host buffers ---------------------------
        hout, hdq, hdk, hdv = (torch.empty_like(hq).pin_memory() for _ in range(4))

        # A caller whose tensors live in host memory pipelines over the independent (b,h) slices:
        # groups of heads go through copy-in -> forward+backward -> copy-out on a few streams, so the
        # two PCIe directions and the kernels overlap.  Every step still moves all inputs in and all
        # results out, and the step ends only when the last result has landed in host memory.
        # measured on a B200 (ms per step): 16 groups / 4 streams 12.7, 8 / 4 13.7, 4 / 4 16.2, 8 / 8 17.8,
        # 16 / 16 17.2, unpipelined 19.7
        n_groups = int(os.environ.get("FNB_BENCH_E2E_GROUPS", "16")) if (B == 1 and H % 16 == 0) else 1
        hpg = H // n_groups
        n_streams = min(n_groups, int(os.environ.get("FNB_BENCH_E2E_STREAMS", "4")))
        streams = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]

        def group_e2e(g):
            h0, h1 = g * hpg, (g + 1) * hpg
            a, b_, c, go = (t[:, h0:h1].to(dev, non_blocking=True) for t in (hq, hk, hv, hdO))
            a.requires_grad_(True), b_.requires_grad_(True), c.requires_grad_(True)
            out = flash_nystrom_attention(a, b_, c, num_landmarks=m, newton_iter=J)
            out.backward(go)
            hout[:, h0:h1].copy_(out.detach(), non_blocking=True)
            hdq[:, h0:h1].copy_(a.grad, non_blocking=True)
            hdk[:, h0:h1].copy_(b_.grad, non_blocking=True)
            hdv[:, h0:h1].copy_(c.grad, non_blocking=True)

        def step_e2e():
            main = torch.cuda.current_stream(dev)
            for st_ in streams:
                st_.wait_stream(main)
            for g in range(n_groups):
                with torch.cuda.stream(streams[g % len(streams)]):
                    group_e2e(g)
            for st_ in streams:
                main.wait_stream(st_)

        for _ in range(3):
            step_e2e()
        barrier()
        e2e_steps = max(3, min(steps, 10))
        e0.record()
        for _ in range(e2e_steps):
            step_e2e()
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
        e2e = {"value": world * B * N / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 4 * elem_bytes, "d2h_bytes_per_step": 4 * elem_bytes,
               "pipeline": f"{n_groups} head groups on {len(streams)} streams"}

    # ---- CPU baseline (rank 0, N=1 only; bounded sample) ---------------------------------------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        heads = 2
        dt, tps, cores, threads = time_cpu(w, heads, 2, 1)
        cpu_baseline = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                        "sample": f"{heads} of {H} heads at full N={N}, FP32 torch CPU ({threads} threads), "
                                  f"1 warm-up + mean of 2; tokens/s scaled by {H}/{heads}",
                        "seconds_per_sample_step": dt}

    if rank == 0:
        line = {
            "metric": METRIC, "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, **w, "per_gpu": True,
                       "l2": "inputs (4 x 134 MB per GPU) exceed the 126 MB L2; no explicit flush"},
            "tokens_per_s_per_gpu": tokens_per_s / world,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": launches_per_step * steps, "launches_per_step": launches_per_step,
            "clocks": clock_summary,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
