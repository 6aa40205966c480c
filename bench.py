#!/usr/bin/env python
"""Benchmark of the Nystrom-attention forward + exact backward hot path.

    python bench.py --gpus N --steps K --warmup W            # this library, on N GPUs
    python bench.py --impl reference --steps K --warmup W    # the reference algorithm on host cores

A step is one forward + backward over one batch of synthetic input.  At every N each GPU runs
the north-star workload B=1, H=16, N=65536, D=64, fp16, num_landmarks=64, newton_iter=6,
kappa_star=0 (batch-parallel weak scaling: independent (b,h) slices, no collective on the data
path).  One JSON line is printed by rank 0:

  value      whole-job tokens/s (tokens = B*N per call, all heads) with inputs resident in HBM
  parity     rel_max of one head of this very workload against the float64 CPU oracle, checked
             before anything is timed
  e2e        the same through the public Python API with pinned HOST buffers: the four input
             copies host->device and the four result copies device->host are inside the timing
  roofline   dominant kernel: algorithmic bytes per launch / its mean CUDA-event duration,
             against the measured copy bandwidth in MEASURED_PEAKS.json; roofline.step is the
             11-pass figure of the whole step
  cpu_baseline  the CPU oracle port of reference.py timed on this box's cores
  sharded    (N > 1) the same 16 slices split over the N GPUs (16/N each): strong scaling
  seqpar     (N > 1) B=1, H=8, N=1048576 with the sequence split over the N GPUs
  extras     (N = 1) device-timed forward + backward of the other reference configurations
"""
import argparse
import ctypes
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
SEQPAR = dict(B=1, H=8, N=1048576, D=64, m=64, J=6, kappa_star=0.0)
METRIC = "fwd+bwd tokens/s/GPU at N=64K,m=64,D=64 fp16; % of HBM roofline"
FALLBACK_HBM_GBS = 6650.0
CONFIG = {"workload": WORKLOAD_NAME, **WORKLOAD}

# N*D-sized tensor passes each kernel makes (reads + writes), per (b,h) slice, as launched.
KERNEL_PASSES = {
    "landmark_partial": 2, "gen_fwd_b": 2, "gen_fwd_c": 2, "gen_bwd_a": 2, "gen_bwd_b": 4,
    "gen_bwd_c": 3,
    # tc_bwd_a also writes its dS1 tiles (into dq), tc_bwd_b writes dS3' tiles (into dk) and dV,
    # tc_bwd_c reads both sets of tiles and writes dQ and dK in place
    "tc_fwd_b": 2, "tc_fwd_c": 2, "tc_bwd_a": 3, "tc_bwd_b": 4, "tc_bwd_c": 4,
}
# The same kernels counted in the bytes the algorithm itself needs (reads of Q, K, V, dO once in each
# direction, writes of O, dQ, dK, dV once): the parked softmax-Jacobian tiles and the second
# reads of Q and K by the pooling pass are traffic this design adds, not algorithmic bytes.
ALGORITHMIC_PASSES = {
    "landmark_partial": 0, "tc_fwd_b": 2, "tc_fwd_c": 2, "tc_bwd_a": 2, "tc_bwd_b": 3, "tc_bwd_c": 2,
    "gen_fwd_b": 2, "gen_fwd_c": 2, "gen_bwd_a": 2, "gen_bwd_b": 4, "gen_bwd_c": 1,
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
    path = os.path.join(ROOT, "profiles", "step_config3_dram_traffic.md")
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
    """SM clock and throttle-reason samples of one GPU through NVML, taken by a thread of this
    process at a modest rate (one sample every 20 ms: NVML calls of several processes serialise in
    the driver, so a faster poll in every rank would itself slow the ranks down).  The timed
    region of a default run is shorter than that, so the caller keeps the GPU under the same load
    for a little longer right after the timed region and the samples cover both."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                   0x4: "sw_power_cap"}
    PERIOD_S = 0.02

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
        nv, h = self.nvml, self.handle
        if nv is None:
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
            self.stop.wait(self.PERIOD_S)

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
                       samples=len(sm), source="nvml",
                       window="timed region and 0.25 s of the same steps right after it, one sample per 20 ms")
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


# ---- CPU side ------------------------------------------------------------------------------------
def cpu_reference_step(q, k, v, dO, w):
    from oracle import nystrom_oracle as O
    return O.forward_backward_autograd(q, k, v, dO, w["m"], w["J"], w["kappa_star"])


def time_cpu(w, steps, warmup):
    """Mean seconds per step of the oracle port on the whole workload (all heads, full N), FP32,
    all host threads."""
    import torch
    from oracle import nystrom_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    q, k, v, dO = (t.float() for t in O.make_inputs(w["B"], w["H"], w["N"], w["D"], seed=0, dtype=torch.float16))
    for _ in range(warmup):
        cpu_reference_step(q, k, v, dO, w)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_reference_step(q, k, v, dO, w)
    dt = (time.perf_counter() - t0) / steps
    return dt, w["B"] * w["N"] / dt, cores, torch.get_num_threads()


def run_reference(args, rank):
    """The reference algorithm (CPU port of reference.py: oracle/nystrom_oracle.py, which the test
    suite pins bit-for-bit to reference.py in FP32) on the host cores: every step is the whole
    workload, all 16 heads at full N."""
    if rank != 0:
        return
    w = WORKLOAD
    steps, warmup = max(args.steps, 1), max(args.warmup, 0)
    dt, tps, cores, threads = time_cpu(w, steps, warmup)
    sample = f"the whole workload per step (all {w['H']} heads, N={w['N']}), FP32, torch CPU ({threads} threads)"
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": CONFIG,
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- host memory placement -----------------------------------------------------------------------
def prefer_gpu_numa_node(dev_index):
    """Ask the kernel to place this process's future host allocations (the pinned staging buffers
    of the end-to-end leg) on the NUMA node the GPU hangs off, so that N ranks do not all copy
    through one node's memory controllers.  Best effort; returns what happened."""
    info = {"gpu_node": None, "policy": "default"}
    try:
        import torch
        pr = torch.cuda.get_device_properties(dev_index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        info["gpu_node"] = node
        if node < 0:
            return info
        libc = ctypes.CDLL("libc.so.6", use_errno=True)
        mask = ctypes.c_ulong(1 << node)
        MPOL_PREFERRED, SYS_set_mempolicy = 1, 238          # x86-64
        rc = libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, ctypes.byref(mask), ctypes.c_ulong(64))
        info["policy"] = f"preferred node {node}" if rc == 0 else f"set_mempolicy failed (errno {ctypes.get_errno()})"
        try:
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                cpus = set()
                for part in f.read().strip().split(","):
                    a, _, b = part.partition("-")
                    cpus.update(range(int(a), int(b or a) + 1))
            allowed = os.sched_getaffinity(0) & cpus
            if allowed:
                os.sched_setaffinity(0, allowed)
                info["cpus"] = f"{len(allowed)} cores of node {node}"
        except Exception as e:
            info["cpus"] = f"affinity unchanged ({e!r})"
    except Exception as e:
        info["error"] = repr(e)
    return info


# ---- extra legs ----------------------------------------------------------------------------------
def _fwd_bwd_fn(q, k, v, dO, m, J, kappa):
    from flashnystrom_b200 import flash_nystrom_attention

    def fn():
        q.grad = k.grad = v.grad = None
        flash_nystrom_attention(q, k, v, num_landmarks=m, newton_iter=J, kappa_star=kappa).backward(dO)
    return fn


def _graph_replay_ms(fn, dev, timed, steps, warmup):
    """Device ms per call of fn replayed from a CUDA graph (the library allocates nothing and never
    synchronises, so a caller may capture it), or None where capture is not available."""
    import torch
    try:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(max(3, warmup)):
            g.replay()
        torch.cuda.synchronize()
        ms, _ = timed(g.replay, steps)
        del g
        return ms
    except Exception:
        torch.cuda.synchronize()
        return None


def _device_inputs(shape, dev, seed, dtype):
    import torch
    g = torch.Generator(device=dev).manual_seed(seed)
    q, k, v, dO = (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(4))
    return q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True), dO


def sharded_leg(dev, rank, world, w, steps, warmup, timed, peak, ms_full):
    """Config 3 with its 16 (b,h) slices split over the ranks (16 / world each), no collective on
    the data path: the strong-scaling curve of the same job."""
    import torch
    B, H, N, D, m, J = w["B"], w["H"], w["N"], w["D"], w["m"], w["J"]
    if H % world:
        return {"skipped": f"{H} heads do not split over {world} ranks"}
    hl = H // world
    q, k, v, dO = _device_inputs((B, hl, N, D), dev, 100 + rank, torch.float16)
    fn = _fwd_bwd_fn(q, k, v, dO, m, J, w["kappa_star"])
    for _ in range(warmup):
        fn()
    ms_eager, host_ms = timed(fn, steps)
    # every rank must take the same path through timed() (it holds collectives)
    ms_graph = _graph_replay_ms(fn, dev, timed, steps, warmup) if os.environ.get("FNB_BENCH_GRAPH", "1") == "1" else None
    ms = ms_graph if ms_graph is not None and ms_graph < ms_eager else ms_eager
    total_bytes = 11 * B * H * N * D * 2
    return {"heads_per_gpu": hl, "ms_per_step": ms, "tokens_per_s": B * N / (ms * 1e-3),
            "eager_ms_per_step": ms_eager, "graph_ms_per_step": ms_graph,
            "host_enqueue_ms_per_step": host_ms, "scaling": "strong",
            "frac_of_11_pass": total_bytes / world / (ms * 1e-3) / 1e9 / peak,
            "efficiency_vs_full_workload_on_one_gpu": (ms_full / world) / ms}


def seqpar_leg(dev, rank, world, w, steps, warmup, timed, peak):
    """B=1, H=8, N=1048576 with every slice's sequence cut into `world` shards
    (seq_parallel_nystrom_attention; four landmark-sized NCCL collectives per forward + backward).
    Head 0 is the same on every rank's view of the global sequence, so its rows are checked
    against the unsharded single-GPU call; a 65536-row case is checked against the CPU oracle."""
    import torch
    import torch.distributed as dist
    from flashnystrom_b200 import flash_nystrom_attention, _C
    from flashnystrom_b200.seqpar import seq_parallel_nystrom_attention
    from oracle import nystrom_oracle as O
    B, H, N, D, m, J, kap = w["B"], w["H"], w["N"], w["D"], w["m"], w["J"], w["kappa_star"]
    if m % world or N % world:
        return {"skipped": f"num_landmarks {m} / N {N} do not split over {world} ranks"}
    Nl = N // world
    rows = slice(rank * Nl, (rank + 1) * Nl)
    res = {"config": f"B={B},H={H},N={N},D={D},m={m},J={J} fp16, sequence split over {world} ranks", "world": world,
           "dO_loss_scale": 1024}

    # (a) small case against the CPU oracle (rank 0 checks its own rows)
    sq, sk, sv, sdO = O.make_inputs(1, 2, 65536, D, seed=5, dtype=torch.float16)
    srows = slice(rank * (65536 // world), (rank + 1) * (65536 // world))
    a, b_, c = (t[:, :, srows].contiguous().to(dev).requires_grad_(True) for t in (sq, sk, sv))
    o = seq_parallel_nystrom_attention(a, b_, c, m, J, kap)
    o.backward(sdO[:, :, srows].contiguous().to(dev))
    torch.cuda.synchronize()
    _C.check_device_status()
    if rank == 0:
        ref = O.forward_backward_autograd(sq.double(), sk.double(), sv.double(), sdO.double(), m, J, kap)
        res["rel_max_vs_oracle_N65536"] = {n_: O.rel_max(g.detach().cpu(), r[:, :, srows])
                                           for n_, g, r in zip(("out", "dq", "dk", "dv"), (o, a.grad, b_.grad, c.grad), ref)}
    del a, b_, c, o

    # (b) the full configuration: head 0 from a seed all ranks share, the others rank-private
    g0 = torch.Generator(device=dev).manual_seed(1234)
    # dO carries a loss scale of 1024, as fp16 training does: at N = 2^20 the gradients of unit-scale
    # dO are ~1e-6, where fp16 outputs are subnormal and two correct results differ by a quantum
    full = [torch.randn(1, 1, N, D, generator=g0, device=dev, dtype=torch.float32).mul_(sc).half()
            for sc in (1.0, 1.0, 1.0, 1024.0)]
    fq, fk, fv = (t.clone().requires_grad_(True) for t in full[:3])
    fo = flash_nystrom_attention(fq, fk, fv, num_landmarks=m, newton_iter=J, kappa_star=kap)
    fo.backward(full[3])
    want = [t[:, :, rows].clone() for t in (fo.detach(), fq.grad, fk.grad, fv.grad)]
    del fq, fk, fv, fo
    gr = torch.Generator(device=dev).manual_seed(4321 + rank)
    shard = []
    for t, sc in zip(full, (1.0, 1.0, 1.0, 1024.0)):
        rest = torch.randn(B, H - 1, Nl, D, generator=gr, device=dev, dtype=torch.float32).mul_(sc).half()
        shard.append(torch.cat([t[:, :, rows], rest], dim=1).contiguous())
    del full, rest
    q, k, v = (t.requires_grad_(True) for t in shard[:3])
    dO = shard[3]

    def fn():
        q.grad = k.grad = v.grad = None
        seq_parallel_nystrom_attention(q, k, v, m, J, kap).backward(dO)
        return None

    q.grad = k.grad = v.grad = None
    out = seq_parallel_nystrom_attention(q, k, v, m, J, kap)
    out.backward(dO)
    torch.cuda.synchronize()
    _C.check_device_status()
    errs = [O.rel_max(g[:, :1].float().cpu(), r.float().cpu()) for g, r in zip((out.detach(), q.grad, k.grad, v.grad), want)]
    t = torch.tensor(errs, device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res["rel_max_vs_unsharded_head0"] = dict(zip(("out", "dq", "dk", "dv"), (float(x) for x in t.tolist())))
    del out, want
    for _ in range(max(2, warmup // 2)):
        fn()
    n = max(3, min(steps, 10))
    ms, host_ms = timed(fn, n)
    # the four collectives alone, same payloads, back to back
    BH = B * H
    bufs = [torch.zeros(2 * BH * m * D, device=dev), torch.zeros(BH * m * (D + 2), device=dev),
            torch.zeros(2 * BH * m * D, device=dev), torch.zeros(BH * m * D, device=dev)]
    gathered = torch.zeros(world * BH * m * (D + 2), device=dev)

    def colls():
        dist.all_reduce(bufs[0])
        dist.all_gather_into_tensor(gathered, bufs[1])
        dist.all_reduce(bufs[2])
        dist.all_reduce(bufs[3])
    for _ in range(3):
        colls()
    cms, _ = timed(colls, 20)
    total_bytes = 11 * B * H * N * D * 2
    res.update(ms_per_step=ms, tokens_per_s=B * N / (ms * 1e-3), host_enqueue_ms_per_step=host_ms,
               frac_of_11_pass=total_bytes / world / (ms * 1e-3) / 1e9 / peak, collective_us=cms * 1e3,
               steps=n)
    return res


def extra_configs(dev, steps, warmup, timed, peak):
    """Device-timed forward + backward of the reference's other configurations on one GPU."""
    import torch
    from flashnystrom_b200 import FlashNystromAttention, NystromConfig
    out = {}
    n = max(3, min(steps, 10))
    cases = {
        "config2_op": ((4, 8, 4096, 64), 64, 6, 0.0),
        "config4": ((2, 8, 16384, 128), 128, 8, 5.0),
        # the two shapes of the reference's published B200 latency table, with its settings
        # (kappa* = 5): 6.15 / 18.32 ms and 1.46 ms there for forward + backward
        "reference_table_D128_N16384": ((4, 16, 16384, 128), 64, 6, 5.0),
        "reference_table_D128_N65536": ((4, 16, 65536, 128), 64, 6, 5.0),
        "reference_table_D64_m32_N65536": ((1, 4, 65536, 64), 32, 6, 5.0),
    }
    dtypes = {"config3_bf16": torch.bfloat16}
    cases["config3_bf16"] = ((1, 16, 65536, 64), 64, 6, 0.0)   # the bench workload with bf16 tensors
    for name, (shape, m, J, kap) in cases.items():
        q, k, v, dO = _device_inputs(shape, dev, 7, dtypes.get(name, torch.float16))
        fn = _fwd_bwd_fn(q, k, v, dO, m, J, kap)
        for _ in range(3):
            fn()
        ms_eager, host_ms = timed(fn, n)
        # small shapes are bound by the host's enqueue time when launched eagerly: the captured step too
        ms_graph = _graph_replay_ms(fn, dev, timed, n, 3) if os.environ.get("FNB_BENCH_GRAPH", "1") == "1" else None
        ms = ms_graph if ms_graph is not None and ms_graph < ms_eager else ms_eager
        B, H, N, D = shape
        out[name] = {"shape": f"B={B},H={H},N={N},D={D},m={m},J={J},kappa*={kap} " + ("bf16" if name in dtypes else "fp16"),
                     "ms_per_step": ms,
                     "eager_ms_per_step": ms_eager, "graph_ms_per_step": ms_graph,
                     "tokens_per_s": B * N / (ms * 1e-3), "host_enqueue_ms_per_step": host_ms,
                     "frac_of_11_pass": 11 * B * H * N * D * 2 / (ms * 1e-3) / 1e9 / peak,
                     "path": "tensor cores" if ((D == 64 and m <= 64) or (D == 128 and m <= 128)) else "CUDA cores"}
        del q, k, v, dO
    torch.manual_seed(0)
    mod = FlashNystromAttention(512, heads=8, config=NystromConfig(num_landmarks=64, newton_iter=6, conv_kernel_size=3))
    mod = mod.to(dev).half()
    x = torch.randn(4, 4096, 512, device=dev, dtype=torch.float16, requires_grad=True)

    def mod_fn():
        x.grad = None
        mod.zero_grad(set_to_none=True)
        mod(x).sum().backward()
    for _ in range(3):
        mod_fn()
    ms, host_ms = timed(mod_fn, n)
    out["config2_module"] = {"shape": "dim=512, heads=8, B=4, N=4096, m=64, J=6, conv k=3, fp16; y.sum().backward()",
                             "ms_per_step": ms, "tokens_per_s": 4 * 4096 / (ms * 1e-3), "host_enqueue_ms_per_step": host_ms}
    return out


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
    ap.add_argument("--no-extras", action="store_true", help="skip the parity check, the extra configurations,\n"
                    "the sharded and the sequence-parallel legs (quick A/B runs)")
    ap.add_argument("--heads", type=int, default=None, help="override H (debug only)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        # torchrun exports OMP_NUM_THREADS=1, and an OpenMP thread count set later from Python only
        # reaches the calling thread, not the autograd engine's: give the CPU arm every core before
        # the OpenMP runtime starts (torch is imported after this point)
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
        os.environ.pop("MKL_NUM_THREADS", None)
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    from flashnystrom_b200 import _C, flash_nystrom_attention
    from oracle import nystrom_oracle as O  # seeded input generation, the parity check and cpu_baseline

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = prefer_gpu_numa_node(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    w = dict(WORKLOAD)
    if args.heads:
        w["H"] = args.heads
    B, H, N, D, m, J = w["B"], w["H"], w["N"], w["D"], w["m"], w["J"]
    steps, warmup = max(args.steps, 1), max(args.warmup, 3)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count

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

    def timed(fn, n):
        """n calls of fn between two events on the current stream; (device ms per call, max over
        ranks; this rank's host enqueue ms per call)."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        host_ms = (time.perf_counter() - t0) * 1e3 / n
        e1.record()
        barrier()
        mine = e0.elapsed_time(e1) / n
        if world > 1:
            allr = torch.zeros(world, device=dev, dtype=torch.float64)
            dist.all_gather_into_tensor(allr, torch.tensor([mine], device=dev, dtype=torch.float64))
            timed.per_rank = [round(float(x), 4) for x in allr.tolist()]
        else:
            timed.per_rank = [round(mine, 4)]
        return max(timed.per_rank) if world > 1 else mine, host_ms

    # ---- parity of this very workload, before anything is timed --------------------------------
    parity = None
    out = step_resident()
    torch.cuda.synchronize()
    _C.check_device_status()
    if rank == 0 and not args.no_extras:
        h = H // 2
        ref = O.forward_backward_autograd(*(t[:, h:h + 1].double() for t in (hq, hk, hv, hdO)), m, J, w["kappa_star"])
        got = (out.detach(), q.grad, k.grad, v.grad)
        parity = {"head": h, "against": "float64 CPU oracle on the identical fp16 inputs",
                  "rel_max": {n_: O.rel_max(g[:, h:h + 1].cpu(), r) for n_, g, r in zip(("out", "dq", "dk", "dv"), got, ref)},
                  "bars": {"out": 2e-3, "grads": 1e-2}}
        e = parity["rel_max"]
        parity["ok"] = bool(e["out"] <= 2e-3 and max(e["dq"], e["dk"], e["dv"]) <= 1e-2)
        if not parity["ok"]:
            raise SystemExit(f"bench.py: the workload's own result fails parity: {parity}")
    del out

    # ---- device-resident timing --------------------------------------------------------------
    for _ in range(warmup):
        step_resident()
    with ClockSampler(local) as clocks:
        ms_eager, host_ms = timed(step_resident, steps)
        eager_per_rank = timed.per_rank
        # the same load a little longer, so that the 20 ms sampler sees the GPU under it
        t_end = time.perf_counter() + 0.25
        while time.perf_counter() < t_end:
            step_resident()
        torch.cuda.synchronize()
    clock_summary = clocks.summary()

    # The same step captured once into a CUDA graph and replayed (the library allocates nothing,
    # never synchronises and forks its side stream with events, so a caller may capture it): the
    # host then enqueues one graph launch per step instead of ~11 kernels and ~25 allocations.
    graph_ms, graph_note, graph_per_rank = None, None, None
    if os.environ.get("FNB_BENCH_GRAPH", "1") == "1":
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(3):
                    step_resident()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            q.grad = k.grad = v.grad = None
            with torch.cuda.graph(g):
                gout = flash_nystrom_attention(q, k, v, num_landmarks=m, newton_iter=J)
                gout.backward(dO)
            for _ in range(warmup):
                g.replay()
            torch.cuda.synchronize()
            _C.check_device_status()
            graph_ms, _ = timed(g.replay, steps)
            graph_per_rank = timed.per_rank
            if parity is not None:   # the replayed graph must reproduce the eager gradients
                h = parity["head"]
                graph_note = "replay matches the float64 oracle: " + str(
                    O.rel_max(q.grad[:, h:h + 1].cpu(), ref[1]) <= 1e-2 and O.rel_max(gout[:, h:h + 1].cpu(), ref[0]) <= 2e-3)
            del g, gout
        except Exception as exc:   # capture is an optimisation of the host side, not the product
            graph_note = f"CUDA-graph capture unavailable: {exc!r}"[:300]
            graph_ms = None
            torch.cuda.synchronize()
    use_graph = graph_ms is not None and graph_ms < ms_eager
    ms_step = graph_ms if use_graph else ms_eager
    tokens_per_s = world * B * N / (ms_step * 1e-3)

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
    # stream) and takes its operands from one extra small kernel that the one-by-one profile does
    # not launch.
    if "tc_bwd_b" in per_kernel and B * H * 4 <= sms:
        launches_per_step += 1
    kernel_ms = {n: sum(v_) / len(v_) for n, v_ in per_kernel.items()}
    total_kernel_ms = sum(kernel_ms.values())
    # The roofline is quoted for the HBM-streaming kernel with the longest launch (the pooling and
    # tensor-core passes move N-sized tensors); the Newton-Schulz and landmark-sized glue kernels
    # move kilobytes and are reported through kernel_ms / kernel_share and the whole-step figure.
    streaming = {n: t for n, t in kernel_ms.items() if KERNEL_PASSES.get(n, 0) > 0}
    top = max(streaming, key=streaming.get) if streaming else max(kernel_ms, key=kernel_ms.get)
    peak, peak_src = hbm_peak()
    alg_bytes = ALGORITHMIC_PASSES.get(top, 0) * elem_bytes
    moved_bytes = KERNEL_PASSES.get(top, 0) * elem_bytes
    achieved = alg_bytes / (kernel_ms[top] * 1e-3) / 1e9 if alg_bytes else 0.0
    step_bytes = 11 * elem_bytes
    roofline = {
        "bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak, "traffic": ncu_traffic(top), "peak_source": peak_src,
        "algorithmic_bytes_per_launch": alg_bytes,
        "as_launched": {"bytes_per_launch": moved_bytes, "note": "includes the parked softmax-Jacobian tiles",
                        "frac": moved_bytes / (kernel_ms[top] * 1e-3) / 1e9 / peak},
        "kernel_ms": {n: round(t, 4) for n, t in kernel_ms.items()},
        "kernel_share": {n: round(t / total_kernel_ms, 4) for n, t in kernel_ms.items()},
        "kernel_frac_as_launched": {n: round(KERNEL_PASSES[n] * elem_bytes / (t * 1e-3) / 1e9 / peak, 3)
                                    for n, t in kernel_ms.items() if KERNEL_PASSES.get(n, 0) > 0},
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
        n_groups = int(os.environ.get("FNB_BENCH_E2E_GROUPS", "16")) if (B == 1 and H % 16 == 0) else 1
        hpg = H // n_groups
        n_streams = min(n_groups, int(os.environ.get("FNB_BENCH_E2E_STREAMS", "4")))
        streams = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]

        def group_e2e(g):
            h0, h1 = g * hpg, (g + 1) * hpg
            a, b_, c, go = (t[:, h0:h1].to(dev, non_blocking=True) for t in (hq, hk, hv, hdO))
            a.requires_grad_(True), b_.requires_grad_(True), c.requires_grad_(True)
            o = flash_nystrom_attention(a, b_, c, num_landmarks=m, newton_iter=J)
            o.backward(go)
            hout[:, h0:h1].copy_(o.detach(), non_blocking=True)
            hdq[:, h0:h1].copy_(a.grad, non_blocking=True)
            hdk[:, h0:h1].copy_(b_.grad, non_blocking=True)
            hdv[:, h0:h1].copy_(c.grad, non_blocking=True)

        def step_e2e():
            main_s = torch.cuda.current_stream(dev)
            for st_ in streams:
                st_.wait_stream(main_s)
            for g in range(n_groups):
                with torch.cuda.stream(streams[g % len(streams)]):
                    group_e2e(g)
            for st_ in streams:
                main_s.wait_stream(st_)

        for _ in range(3):
            step_e2e()
        e2e_ms, _ = timed(step_e2e, max(3, min(steps, 10)))
        torch.cuda.synchronize()
        e2e_check = None
        if parity is not None:   # what landed in host memory is the result (same head, same oracle figures)
            h = parity["head"]
            e2e_check = {n_: O.rel_max(g[:, h:h + 1], r) for n_, g, r in zip(("out", "dq", "dk", "dv"), (hout, hdq, hdk, hdv), ref)}
            if not (e2e_check["out"] <= 2e-3 and max(e2e_check["dq"], e2e_check["dk"], e2e_check["dv"]) <= 1e-2):
                raise SystemExit(f"bench.py: the end-to-end pipeline's results fail parity: {e2e_check}")

        # the same bytes over two copy streams with no call in between: what the PCIe link allows
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

        def step_copies_only():
            main_s = torch.cuda.current_stream(dev)
            s_in.wait_stream(main_s), s_out.wait_stream(main_s)
            for g in range(n_groups):
                h0, h1 = g * hpg, (g + 1) * hpg
                with torch.cuda.stream(s_in):
                    for t in (hq, hk, hv, hdO):
                        t[:, h0:h1].to(dev, non_blocking=True)
                with torch.cuda.stream(s_out):
                    for dst, src in zip((hout, hdq, hdk, hdv), (q, k, v, dO)):
                        dst[:, h0:h1].copy_(src.detach()[:, h0:h1], non_blocking=True)
            main_s.wait_stream(s_in), main_s.wait_stream(s_out)
        step_copies_only()
        copies_ms, _ = timed(step_copies_only, 5)
        torch.cuda.synchronize()
        e2e = {"value": world * B * N / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 4 * elem_bytes, "d2h_bytes_per_step": 4 * elem_bytes,
               "pipeline": f"{n_groups} head groups on {len(streams)} streams", "host_numa": numa,
               "rel_max_vs_oracle": e2e_check, "copies_only_ms_per_step": copies_ms,
               "frac_of_copies_only": copies_ms / e2e_ms}
        del hout, hdq, hdk, hdv

    # ---- other legs ------------------------------------------------------------------------------
    sharded = seqpar = extras = None
    if not args.no_extras:
        del q, k, v, dO
        torch.cuda.empty_cache()
        if world > 1:
            sharded = sharded_leg(dev, rank, world, w, steps, warmup, timed, peak, ms_step)
            seqpar = seqpar_leg(dev, rank, world, SEQPAR, steps, warmup, timed, peak)
        else:
            extras = extra_configs(dev, steps, warmup, timed, peak)

    # ---- CPU baseline (rank 0, N=1 only) ----------------------------------------------------------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        dt, tps, cores, threads = time_cpu(w, 3, 1)
        cpu_baseline = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                        "sample": f"the whole workload (all {H} heads at full N={N}), FP32 torch CPU ({threads} threads), "
                                  f"1 warm-up + mean of 3 steps",
                        "seconds_per_step": dt}

    if rank == 0:
        line = {
            "metric": METRIC, "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": CONFIG if not args.heads else {**CONFIG, "H": H},
            "per_gpu_workload": True,
            "l2": "inputs (4 x 134 MB per GPU) exceed the 126 MB L2; no explicit flush",
            "launch_mode": "CUDA graph replay of the captured step" if use_graph else "eager (one API call per pass)",
            "eager": {"ms_per_step": ms_eager, "host_enqueue_ms_per_step": host_ms, "per_rank_ms": eager_per_rank},
            "graph": {"ms_per_step": graph_ms, "note": graph_note, "per_rank_ms": graph_per_rank},
            "tokens_per_s_per_gpu": tokens_per_s / world,
            "parity": parity, "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "sharded": sharded, "seqpar": seqpar, "extras": extras,
            "gpu_launches": launches_per_step * steps, "launches_per_step": launches_per_step,
            "clocks": clock_summary,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
