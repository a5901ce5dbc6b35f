#!/usr/bin/env python
"""Benchmark of the FP16 x FP16 -> FP32 GEMM path.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads (all synthetic, from the counter-based generator of the library):
    gemm8192  M=N=K=8192, A row-major, B column-major, alpha=2, beta=0.5, seed 2   (default at N=1)
    gemm4096  M=N=K=4096, A, B column-major, alpha=beta=1, seed 1
    skinny    M=16384, N=128, K=8192, A, B column-major, beta=0, seed 3              (HBM-bound)
    sharded   M=N=32768, K=16384, A, B column-major, alpha=beta=1, seed 4; B/C/D split into
              column slabs over the ranks; A travels from rank 0 to every rank in K panels over
              NVLink: copy-engine scatter + all-gather through the b200_sharded_* entry points
              (--transport p2p, default) or NCCL broadcast (--transport nccl)       (default at N>1)
Secondary workloads (1 GPU, device-resident timing only; no e2e / CPU leg):
    gemm8192_bf16  gemm8192 with bfloat16 A and B (b200_gemm_ex)
    batched64      64 products of 1024^3, Float16 in, Float32 C and D, alpha=beta=1, one launch
                   (b200_gemm_strided_batched); also timed as 64 launches of b200_gemm_f16f32

A "step" is one whole GEMM.  `value` is the whole job's TFLOP/s with operands resident in HBM,
timed with CUDA events on the launching stream (max over ranks); `e2e` is the same metric through
the host-buffer entry point, host<->device copies inside the timed region.  `--impl reference`
times the CPU statement of the same product (float32 sgemm on the Float16-rounded inputs -- the
stand-in for Julia's LinearAlgebra.mul!, which cannot run without Julia) on the host cores.

The default one-GPU line also carries, as extra keys, the other single-GPU configurations and the
denominator of the multi-GPU values: `sustained` (the 8192^3 product back to back for >= 2 s),
`skinny`, `gemm4096` and `scaling_baseline` (the sharded workload on one GPU).  Sharded runs check
sampled tiles of every rank's D slab against the CPU oracle after the timed region (`parity`) and
exit non-zero when they differ.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

import __graft_entry__ as entry  # noqa: E402

WORKLOADS = {
    # name: (M, N, K, transA, transB, alpha, beta, seed, a_scale_is_rsqrt_k, b_scale_is_rsqrt_k, c_dist)
    "gemm8192": dict(M=8192, N=8192, K=8192, transA=True, transB=False, alpha=2.0, beta=0.5, seed=2, b_rsqrt=True, c_dist="uniform"),
    "gemm4096": dict(M=4096, N=4096, K=4096, transA=False, transB=False, alpha=1.0, beta=1.0, seed=1, b_rsqrt=True, c_dist="normal"),
    "skinny": dict(M=16384, N=128, K=8192, transA=False, transB=False, alpha=1.0, beta=0.0, seed=3, b_rsqrt=False, c_dist="zeros"),
    "sharded": dict(M=32768, N=32768, K=16384, transA=False, transB=False, alpha=1.0, beta=1.0, seed=4, b_rsqrt=True, c_dist="normal"),
}
# device-resident timing of the bfloat16 and batched entry points (run_extra)
EXTRA_WORKLOADS = {
    "gemm8192_bf16": dict(M=8192, N=8192, K=8192, batch=1, transA=True, transB=False, alpha=2.0, beta=0.5, seed=2, bf16=True),
    "batched64": dict(M=1024, N=1024, K=1024, batch=64, transA=False, transB=False, alpha=1.0, beta=1.0, seed=5, bf16=False),
}
METRIC = "FP16->FP32 GEMM TFLOP/s (8192^3) & % of B200 tensor peak; 1/2/4/8-GPU scaling"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return dict(hbm_gbs=float(d["hbm_gbs"]), tf_burst=float(d["bf16_tflops"]),
                        tf_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


def algorithmic_bytes(w):
    M, N, K = w["M"], w["N"], w["K"]
    b = 2 * M * K + 2 * K * N + 4 * M * N
    if w["beta"] != 0.0:
        b += 4 * M * N
    return b


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """SM clock and throttle reasons while a timed region runs.  Reads NVML directly when the Python
    binding is there (a sample every ~2 ms, so that a region of a few milliseconds still gets
    several), else parses `nvidia-smi -lms`.  Only reads: no clock, power or mode setting is touched."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    # NVML clocks-event-reason bits
    NVML_REASONS = ((0x4, "sw_power_cap"), (0x8, "hw_slowdown"), (0x20, "sw_thermal_slowdown"), (0x40, "hw_thermal_slowdown"))

    def __init__(self, gpu_index: int, uuid: str | None = None):
        self.gpu_index = gpu_index
        self.uuid = uuid
        self.proc = None
        self.lines = []      # (t, nvidia-smi csv line)
        self.samples = []    # (t, sm_mhz, reasons bitmask) from NVML
        self.smax = None
        self._stop = False
        self._thread = None

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        if self.uuid:
            for cand in (self.uuid, "GPU-" + self.uuid):
                try:
                    return pynvml, pynvml.nvmlDeviceGetHandleByUUID(cand.encode() if isinstance(cand, str) else cand)
                except Exception:
                    try:
                        return pynvml, pynvml.nvmlDeviceGetHandleByUUID(cand)
                    except Exception:
                        continue
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)

    def start(self):
        try:
            nv, dev = self._nvml_handle()
            self.smax = float(nv.nvmlDeviceGetMaxClockInfo(dev, nv.NVML_CLOCK_SM))
            nv.nvmlDeviceGetClockInfo(dev, nv.NVML_CLOCK_SM)

            def pump():
                while not self._stop:
                    try:
                        mhz = float(nv.nvmlDeviceGetClockInfo(dev, nv.NVML_CLOCK_SM))
                        try:
                            why = int(nv.nvmlDeviceGetCurrentClocksEventReasons(dev))
                        except Exception:
                            why = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(dev))
                        self.samples.append((time.perf_counter(), mhz, why))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self._thread = threading.Thread(target=pump, daemon=True)
            self._thread.start()
            return
        except Exception:
            self._thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def window(self, t0: float, t1: float) -> dict:
        """Median clock and the reasons seen between two perf_counter times (sampling goes on)."""
        if self._thread is not None:
            got = [(m, w) for (t, m, w) in list(self.samples) if t0 <= t <= t1]
            reasons = sorted({name for (_, w) in got for (bit, name) in self.NVML_REASONS if w & bit})
            return {"sm_mhz": float(np.median([m for (m, _) in got])) if got else None, "sm_max_mhz": self.smax,
                    "reasons": reasons, "samples": len(got)}
        sm, smax, reasons = [], None, set()
        for (t, line) in list(self.lines):
            if t < t0 - 0.05 or t > t1 + 0.15:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}

    def stop(self, t0: float, t1: float) -> dict:
        if self._thread is not None:
            out = self.window(t0, t1)
            self._stop = True
            return out
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        return self.window(t0, t1)


# ---------------------------------------------------------------------------------------------
# CPU statement (oracle) legs
# ---------------------------------------------------------------------------------------------
def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1 to its ranks, which would turn the BLAS behind numpy into a
    one-thread library: raise the pool to every host core explicitly and report what it ended up with."""
    want = os.cpu_count() or 1
    try:
        import threadpoolctl

        threadpoolctl.threadpool_limits(limits=want)
        got = [int(i.get("num_threads", 0)) for i in threadpoolctl.threadpool_info() if i.get("user_api") == "blas"]
        if got:
            return max(got)
    except Exception:
        pass
    return int(os.environ.get("OMP_NUM_THREADS", want))


class CpuSample:
    """float32 sgemm on a bounded slab of the workload: rows 0..m_s-1 of op(A), full K, the first
    n_cols columns of B and C.  Operands are generated once; ``run()`` times one product."""

    def __init__(self, w, target_seconds=12.0):
        self.oracle = entry.load_oracle()
        rng = entry.load_package().rng
        self.w = w
        M, K, N = w["M"], w["K"], w["N"]
        self.cores = use_all_host_threads()
        m_s = min(M, 8192)
        a16 = rng.window(w["seed"], 0, (K if w["transA"] else M), 0, (K if w["transA"] else m_s), 0,
                         (m_s if w["transA"] else K), rng.NORMAL, K ** -0.5, np.float16)
        self.a32 = a16.astype(np.float32)  # the conversion is not part of mul!
        # a narrow probe learns the host's rate, then the slab is sized for ~target_seconds of work
        n_probe = min(N, 128)
        b_scale = K ** -0.5 if w["b_rsqrt"] else 1.0
        b32 = rng.window(w["seed"], 1, K, 0, K, 0, n_probe, rng.NORMAL, b_scale, np.float16).astype(np.float32)
        c = np.zeros((m_s, n_probe), np.float32, order="F")
        self._gemm(b32, c)  # warm-up (thread pool, pages)
        t0 = time.perf_counter()
        self._gemm(b32, c)
        rate = 2.0 * m_s * n_probe * K / max(time.perf_counter() - t0, 1e-6)
        n_cols = int(max(n_probe, min(N, target_seconds * rate / (2.0 * m_s * K))))
        self.b32 = rng.window(w["seed"], 1, K, 0, K, 0, n_cols, rng.NORMAL, b_scale, np.float16).astype(np.float32)
        self.c = np.zeros((m_s, n_cols), np.float32, order="F")
        self.flops = 2.0 * m_s * n_cols * K
        self.desc = (f"float32 sgemm (numpy/OpenBLAS, {self.cores} threads) on Float16-rounded inputs, rows 0..{m_s - 1} x cols 0..{n_cols - 1} "
                     f"x full K={K} of the workload")

    def _gemm(self, b32, c):
        w = self.w
        return self.oracle.gemm_ref_f32(w["transA"], False, w["alpha"], self.a32, b32, w["beta"], c)

    def run(self):
        """One timed product; returns (TFLOP/s, seconds)."""
        t0 = time.perf_counter()
        self._gemm(self.b32, self.c)
        dt = time.perf_counter() - t0
        return self.flops / dt / 1e12, dt


def cpu_sample(w, target_seconds=12.0):
    """Best of up to three products of a slab sized for ~target_seconds of CPU work.
    Returns (TFLOP/s, cores, description, seconds)."""
    smp = CpuSample(w, target_seconds)
    best = None
    for _ in range(3):
        v, dt = smp.run()
        if best is None or dt < best[1]:
            best = (v, dt)
        if dt > target_seconds / 2:
            break
    return best[0], smp.cores, smp.desc + ", best of up to 3", best[1]


# ---------------------------------------------------------------------------------------------
# parity of a sharded product (checker leg: the CPU oracle on sampled tiles)
# ---------------------------------------------------------------------------------------------
def check_slab_tiles(w, D, n0, ns, A=None, tiles=8, tile=128, seed=1234):
    """Compare sampled tile x tile blocks of a column slab of D (device tensor, column-major M x ns,
    columns [n0, n0+ns) of the workload) with the CPU oracle: `tiles` blocks at random places plus one
    on the slab's first and one on its last columns, each with the full K.  The operands of a block
    are regenerated from the counter-based generator, so no other rank is needed.  When `A` (device
    tensor, M x K column-major) is given, sampled columns of it are compared bit for bit with the
    generator as well (did A arrive intact on this rank?).  Returns a dict; never raises."""
    oracle = entry.load_oracle()
    rng = entry.load_package().rng
    M, K = w["M"], w["K"]
    out = {"tiles": 0, "rel_fro_max": 0.0, "elem_max": 0.0, "a_columns": 0, "ok": True, "why": None}
    if ns <= 0:
        return out
    rs = np.random.RandomState(seed + n0)
    tm, tn = min(tile, M), min(tile, ns)
    places = [(int(rs.randint(0, M - tm + 1)), 0), (int(rs.randint(0, M - tm + 1)), ns - tn)]
    places += [(int(rs.randint(0, M - tm + 1)), int(rs.randint(0, ns - tn + 1))) for _ in range(tiles)]
    b_scale = K ** -0.5 if w["b_rsqrt"] else 1.0
    d2 = D.view(ns, M)  # torch sees the column-major slab as its transpose
    for (r0, c0) in places:
        a = rng.window(w["seed"], 0, M, r0, r0 + tm, 0, K, rng.NORMAL, K ** -0.5, np.float16)
        b = rng.window(w["seed"], 1, K, 0, K, n0 + c0, n0 + c0 + tn, rng.NORMAL, b_scale, np.float16)
        c = None
        if w["beta"] != 0.0:
            c = rng.window(w["seed"], 2, M, r0, r0 + tm, n0 + c0, n0 + c0 + tn, dist_code(rng, w["c_dist"]), 1.0, np.float32)
        ref = oracle.gemm_ref(False, False, w["alpha"], a, b, w["beta"], c)
        got = d2[c0:c0 + tn, r0:r0 + tm].cpu().numpy().T
        out["tiles"] += 1
        if not np.all(np.isfinite(got)):
            out["ok"], out["why"] = False, f"non-finite values in rows {r0}.. cols {n0 + c0}.."
            continue
        rel, elem = oracle.errors(got, ref)
        out["rel_fro_max"] = max(out["rel_fro_max"], rel)
        out["elem_max"] = max(out["elem_max"], elem)
        if rel > oracle.REL_FRO_TOL or elem > oracle.ELEM_TOL:
            out["ok"], out["why"] = False, f"tile rows {r0}.. cols {n0 + c0}..: rel {rel:.3e}, elem {elem:.3e}"
    if A is not None:
        a2 = A.view(K, M)
        cols = sorted({0, K - 1, *[int(x) for x in rs.randint(0, K, size=14)]})
        for k in cols:
            want = rng.window(w["seed"], 0, M, 0, M, k, k + 1, rng.NORMAL, K ** -0.5, np.float16)[:, 0]
            got = a2[k].cpu().numpy()
            out["a_columns"] += 1
            if not np.array_equal(got.view(np.uint16), want.view(np.uint16)):
                out["ok"], out["why"] = False, f"column {k} of A differs from what rank 0 holds"
    out["rel_fro_max"] = float(f"{out['rel_fro_max']:.3e}")
    out["elem_max"] = float(f"{out['elem_max']:.3e}")
    return out


# ---------------------------------------------------------------------------------------------
# GPU legs
# ---------------------------------------------------------------------------------------------
def dist_code(rng, name):
    return {"uniform": rng.UNIFORM, "normal": rng.NORMAL, "zeros": rng.ZEROS}[name]


def event_timed(torch, fn, steps, warmup):
    """(total ms, perf_counter window) of `steps` calls of fn after `warmup` untimed ones, CUDA events
    on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    for _ in range(steps):
        fn()
    ev1.record()
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1), (t0, time.perf_counter())


def run_ours(args):
    import torch

    pkg = entry.load_package()
    from cudanative_jl_b200 import _lib, rng
    from cudanative_jl_b200.gemm import Handle, ShardedGemm
    from cudanative_jl_b200.nccl_broadcast import NcclBroadcastGemm, init_nccl_env

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N>1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        init_nccl_env(args.nccl_ctas)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    name = args.workload or ("gemm8192" if world == 1 else "sharded")
    w = WORKLOADS[name]
    M, N, K = w["M"], w["N"], w["K"]
    h = Handle(local_rank)
    stream = torch.cuda.current_stream().cuda_stream
    peaks = measured_peaks()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sharded = name == "sharded"
    p2p = sharded and (args.transport == "p2p" or world == 1)
    sg = None
    if sharded and p2p:
        def exchange(blob):
            blobs = [None] * world
            dist.all_gather_object(blobs, blob)
            return blobs
        sg = ShardedGemm(h, M, N, K, rank=rank, world=world, panels=args.panels, exchange=exchange if world > 1 else None)
        if world > 1:
            sg.set_option(_lib.SHARDED_OPT_SCATTER_LANES, args.scatter_lanes)
            sg.set_option(_lib.SHARDED_OPT_GATHER_LANES, args.gather_lanes)
            sg.set_option(_lib.SHARDED_OPT_FIRST_GROUP, args.first_group)
            if args.groups:
                sg.set_groups([int(x) for x in args.groups.split(",")])
        n0, ns = sg.n0, sg.slab_cols
        A = torch.as_tensor(sg.a_view(), device=torch.device("cuda", local_rank))
        n_launches = 1 if args.gated else sg.n_groups
        n_panels = sg.n_panels
    elif sharded:
        sg = NcclBroadcastGemm(h, M, N, K, panels=args.panels, reserve_ctas=args.nccl_ctas)
        n0, ns = sg.n0, sg.slab_cols
        A = torch.empty(M * K, dtype=torch.float16, device="cuda")
        n_launches = n_panels = len(sg.panels)
    else:
        n0, ns = 0, N
    a_rows, a_cols = (K, M) if w["transA"] else (M, K)
    if not sharded:
        A = torch.empty(a_rows * a_cols, dtype=torch.float16, device="cuda")
    B = torch.empty(K * max(ns, 1), dtype=torch.float16, device="cuda")
    Cm = torch.empty(M * max(ns, 1), dtype=torch.float32, device="cuda") if w["beta"] != 0.0 else None
    D = torch.empty(M * max(ns, 1), dtype=torch.float32, device="cuda")
    if (not sharded) or rank == 0:
        rng.fill_device(A.data_ptr(), a_rows, a_cols, a_rows, w["seed"], 0, rng.NORMAL, K ** -0.5, True, stream)
    else:
        A.zero_()
    rng.fill_device(B.data_ptr(), K, ns, K, w["seed"], 1, rng.NORMAL, K ** -0.5 if w["b_rsqrt"] else 1.0, True, stream, col0=n0)
    if Cm is not None:
        rng.fill_device(Cm.data_ptr(), M, ns, M, w["seed"], 2, dist_code(rng, w["c_dist"]), 1.0, False, stream, col0=n0)

    def step(no_transfer=False, no_compute=False):
        if sharded and p2p:
            sg.run(w["alpha"], B, w["beta"], Cm, D, stream=stream, gated=args.gated, no_transfer=no_transfer, no_compute=no_compute)
        elif sharded:
            sg.run(w["alpha"], A, B, w["beta"], Cm, D)
        else:
            h.gemm(w["transA"], w["transB"], M, N, K, w["alpha"], A.data_ptr(), a_rows, B.data_ptr(), K, w["beta"],
                   Cm.data_ptr() if Cm is not None else None, M, D.data_ptr(), M, stream=stream)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    code, block, _ = h.device_status()
    if code:
        raise SystemExit(f"device wait {code} ran out in block {block} during warm-up")
    launch = h.last_launch()

    sampler = None
    if rank == 0:
        uuid = None
        try:
            uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
        except Exception:
            pass
        sampler = ClockSampler(local_rank, uuid)
        sampler.start()
        time.sleep(0.25)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.perf_counter()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    t_wall1 = time.perf_counter()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    clocks = sampler.window(t_wall0, t_wall1) if sampler else None
    code, block, _ = h.device_status()
    if code:
        raise SystemExit(f"device wait {code} ran out in block {block} during the timed region")
    ms_step = ms_total / args.steps
    flops = 2.0 * M * N * K
    tflops = flops / (ms_step * 1e-3) / 1e12

    # ---- sharded runs: the result proves itself, and the exposed transfer becomes a number -------------
    parity = None
    compute_only_ms = transfer_only_ms = None
    if sharded:
        mine = check_slab_tiles(w, D, n0, ns, A=A if rank != 0 else None)
        if dist is not None:
            t = torch.tensor([mine["tiles"], mine["a_columns"], 0.0 if mine["ok"] else 1.0], dtype=torch.float64, device="cuda")
            dist.all_reduce(t)
            m = torch.tensor([mine["rel_fro_max"], mine["elem_max"]], dtype=torch.float64, device="cuda")
            dist.all_reduce(m, op=dist.ReduceOp.MAX)
            whys = [None] * world
            dist.all_gather_object(whys, mine["why"])
            parity = {"tiles": int(t[0].item()), "a_columns": int(t[1].item()), "rel_fro_max": float(m[0].item()),
                      "elem_max": float(m[1].item()), "ok": t[2].item() == 0.0, "ranks": world,
                      "why": next((f"rank {r}: {x}" for r, x in enumerate(whys) if x), None)}
        else:
            parity = dict(mine, ranks=1)
        parity["tolerance"] = {"rel_fro": 1e-3, "elem": 1e-2}
        if p2p and world > 1 and not args.gated:
            # the same launches with A already resident on every rank: what is left of ms_per_step is the
            # part of the transfer that the schedule does not hide
            k = max(3, min(args.steps, 10))
            barrier()
            ms, _ = event_timed(torch, lambda: step(no_transfer=True), k, 2)
            compute_only_ms = max_over_ranks(ms / k)
            barrier()
            # and the transfer alone (every copy, flag and wait, no launch): the floor the links set
            ms, _ = event_timed(torch, lambda: step(no_compute=True), k, 2)
            sg.wait(60000)
            transfer_only_ms = max_over_ranks(ms / k)
            barrier()

    # ---- end to end through the host-buffer API -------------------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    if args.no_e2e:
        e2e_steps = 0
    if sharded and args.no_e2e:
        h2d = d2h = 0

        def e2e_step():
            pass
    elif sharded:
        hA = torch.empty(M * K, dtype=torch.float16).pin_memory() if rank == 0 else None
        hB = torch.empty(K * max(ns, 1), dtype=torch.float16).pin_memory()
        hC = torch.empty(M * max(ns, 1), dtype=torch.float32).pin_memory()
        hD = torch.empty(M * max(ns, 1), dtype=torch.float32).pin_memory()
        if hA is not None:
            hA.copy_(A)
        hB.copy_(B)
        hC.copy_(Cm)
        barrier()

        def e2e_step():
            if hA is not None:
                A.copy_(hA, non_blocking=True)
            B.copy_(hB, non_blocking=True)
            Cm.copy_(hC, non_blocking=True)
            step()
            hD.copy_(D, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        h2d = (hA.numel() * 2 if hA is not None else 0) + hB.numel() * 2 + hC.numel() * 4
        d2h = hD.numel() * 4
        if dist is not None:
            t = torch.tensor([h2d, d2h], dtype=torch.float64, device="cuda")
            dist.all_reduce(t)
            h2d, d2h = int(t[0].item()), int(t[1].item())
    else:
        L = _lib.lib()
        import ctypes as C

        def pinned(nbytes):
            p = C.c_void_p()
            _lib.check(L.b200_host_alloc(C.byref(p), nbytes), "host_alloc")
            return p

        pA, pB, pD = pinned(A.numel() * 2), pinned(B.numel() * 2), pinned(D.numel() * 4)
        pC = pinned(Cm.numel() * 4) if Cm is not None else None
        _lib.check(L.b200_memcpy_d2h(pA, A.data_ptr(), A.numel() * 2, None), "d2h")
        _lib.check(L.b200_memcpy_d2h(pB, B.data_ptr(), B.numel() * 2, None), "d2h")
        if pC is not None:
            _lib.check(L.b200_memcpy_d2h(pC, Cm.data_ptr(), Cm.numel() * 4, None), "d2h")
        _lib.check(L.b200_stream_sync(None), "sync")

        def e2e_step():
            _lib.check(L.b200_gemm_f16f32_host(h._h, int(w["transA"]), int(w["transB"]), M, N, K, w["alpha"], pA, a_rows,
                                               pB, K, w["beta"], pC, M, pD, M), "gemm_host")
        h2d = A.numel() * 2 + B.numel() * 2 + (Cm.numel() * 4 if Cm is not None else 0)
        d2h = D.numel() * 4
    e2e_step()  # warm-up: workspace allocation, page faults
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = max_over_ranks((time.perf_counter() - t0) / max(e2e_steps, 1))
    e2e_tflops = flops / e2e_s / 1e12 if e2e_steps else 0.0
    if sharded and p2p:
        barrier()
        sg.close()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    launches_per_step = (n_launches if sharded else 1) * (2 if launch["split_k"] > 1 else 1)
    hbm_bound = name == "skinny"
    # kernel-level roofline: one launch == one step for the single-GPU workloads
    if hbm_bound:
        achieved = algorithmic_bytes(w) / (ms_step * 1e-3) / 1e9
        peak, unit = peaks["hbm_gbs"], "GB/s"
        peak_kind = "hbm_gbs"
    else:
        achieved = tflops / world
        long_run = (ms_total * 1e-3) > 1.0
        peak = peaks["tf_sustained"] if long_run else peaks["tf_burst"]
        peak_kind = "bf16_tflops_sustained" if long_run else "bf16_tflops"
        unit = "TFLOP/s"
    if sharded:
        how = (f"N-sharded x{world}, A sent in {n_panels} K-panels by " +
               ("NCCL broadcast, one GEMM launch per panel" if not p2p else
                "copy-engine scatter + all-gather over NVLink ordered by stream memory operations (b200_sharded_run)" +
                (", one gated GEMM launch" if args.gated else f", {n_launches} GEMM launches over growing K ranges")))
    else:
        how = "1 GPU"
    out = {
        "metric": METRIC, "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 5), "higher_is_better": True,
        "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "f16*f16->f32", "data": "synthetic",
        "config": {"workload": name, "M": M, "N": N, "K": K, "transA": w["transA"], "transB": w["transB"],
                   "alpha": w["alpha"], "beta": w["beta"], "seed": w["seed"],
                   "l2": f"inputs+outputs {algorithmic_bytes(w) / 1e6:.0f} MB per step exceed the 126 MB L2; no flush",
                   "kernel": launch, "parallelism": how},
        "clocks": clocks,
        "e2e": {"value": round(e2e_tflops, 3), "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "steps": e2e_steps, "api": "b200_sharded_run + pinned copies" if sharded else "b200_gemm_f16f32_host"},
        "gpu_launches": launches_per_step * args.steps * world,
        # traffic: DRAM bytes per launch come from an ncu capture; none is taken inside a bench run, so the line
        # does not claim one
        "roofline": {"bound": "hbm" if hbm_bound else "tensor", "achieved": round(achieved, 2), "peak": peak, "unit": unit,
                     "frac": round(achieved / peak, 4), "traffic": None, "peak_source": f"{peaks['source']} ({peak_kind})",
                     "nominal_frac": round(achieved / (8000.0 if hbm_bound else 2250.0), 4),
                     "algorithmic_bytes": algorithmic_bytes(w)},
    }
    if clocks and clocks.get("sm_mhz"):
        out["clocks"]["ms_x_mhz"] = round(ms_step * clocks["sm_mhz"], 1)
    if parity is not None:
        out["parity"] = parity
    if compute_only_ms is not None:
        out["compute_only_ms"] = round(compute_only_ms, 4)
        out["exposed_transfer_ms"] = round(ms_step - compute_only_ms, 4)
    if transfer_only_ms is not None:
        out["transfer_only_ms"] = round(transfer_only_ms, 4)
    if world == 1 and args.workload is None:
        # the other single-GPU configurations, each timed on its own: they share the line so that one
        # default run records every headline figure
        del A, B, Cm, D
        torch.cuda.empty_cache()
        if not args.no_extras:
            # short legs first, each after a pause: the power-capped clock needs a moment to recover from
            # the leg before it, and a leg that starts at the tail of another one's throttling measures that
            time.sleep(1.0)
            out["skinny"] = skinny_leg(h, stream, peaks, sampler)
            time.sleep(1.0)
            out["gemm4096"] = square_leg(h, stream, "gemm4096", peaks, sampler)
            time.sleep(1.0)
            out["sustained"] = sustained_loop(h, stream, peaks, sampler)
            time.sleep(1.0)
        if not args.no_scaling_baseline:
            # The multi-GPU lines (N > 1) time the sharded 32768 x 32768 x 16384 product; its one-GPU time is measured
            # here so that the N-GPU values have a like-for-like denominator next to the headline 8192^3 number.
            out["scaling_baseline"] = sharded_on_one_gpu(h, stream, sampler)
    if sampler:
        sampler.stop(0, 0)
    if world == 1 and not args.no_cpu:
        v, cores, desc, secs = cpu_sample(w)
        out["cpu_baseline"] = {"value": round(v, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc,
                               "seconds": round(secs, 2)}
    print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        raise SystemExit(f"parity check failed: {parity['why']}")
    sb = out.get("scaling_baseline")
    if sb and not sb["parity"]["ok"]:
        raise SystemExit(f"parity check of the one-GPU sharded run failed: {sb['parity']['why']}")


def _operands(torch, rng, w, stream, a_copies=1):
    """Device operands of a workload (column-major, filled from the generator); `a_copies` independent
    buffers of A so that an HBM-bound kernel never finds its stream in L2."""
    M, N, K = w["M"], w["N"], w["K"]
    a_rows, a_cols = (K, M) if w["transA"] else (M, K)
    As = []
    for i in range(a_copies):
        A = torch.empty(a_rows * a_cols, dtype=torch.float16, device="cuda")
        rng.fill_device(A.data_ptr(), a_rows, a_cols, a_rows, w["seed"] + 1000 * i, 0, rng.NORMAL, K ** -0.5, True, stream)
        As.append(A)
    B = torch.empty(K * N, dtype=torch.float16, device="cuda")
    rng.fill_device(B.data_ptr(), K, N, K, w["seed"], 1, rng.NORMAL, K ** -0.5 if w["b_rsqrt"] else 1.0, True, stream)
    Cm = None
    if w["beta"] != 0.0:
        Cm = torch.empty(M * N, dtype=torch.float32, device="cuda")
        rng.fill_device(Cm.data_ptr(), M, N, M, w["seed"], 2, dist_code(rng, w["c_dist"]), 1.0, False, stream)
    D = torch.empty(M * N, dtype=torch.float32, device="cuda")
    return As, B, Cm, D, a_rows


def _status_or_exit(h, what):
    code, block, _ = h.device_status()
    if code:
        raise SystemExit(f"device wait {code} ran out in block {block} in {what}")


def sustained_loop(h, stream, peaks, sampler, seconds=2.2):
    """The headline product back to back for at least two seconds: what the power cap leaves of the
    burst figure.  Compared with the measured sustained cuBLAS rate."""
    import torch
    from cudanative_jl_b200 import rng

    w = WORKLOADS["gemm8192"]
    M, N, K = w["M"], w["N"], w["K"]
    (A,), B, Cm, D, a_rows = _operands(torch, rng, w, stream)

    def step():
        h.gemm(w["transA"], w["transB"], M, N, K, w["alpha"], A.data_ptr(), a_rows, B.data_ptr(), K, w["beta"], Cm.data_ptr(), M,
               D.data_ptr(), M, stream=stream)
    ms, _ = event_timed(torch, step, 50, 3)
    launches = max(200, int(seconds * 1e3 / (ms / 50)))
    ms, (t0, t1) = event_timed(torch, step, launches, 0)
    _status_or_exit(h, "the sustained loop")
    tf = 2.0 * M * N * K / (ms / launches * 1e-3) / 1e12
    clocks = sampler.window(t0 + 0.2, t1) if sampler else None
    out = {"workload": "gemm8192", "launches": launches, "seconds": round(ms * 1e-3, 3), "ms_per_step": round(ms / launches, 5),
           "value": round(tf, 2), "unit": "TFLOP/s", "peak": peaks["tf_sustained"], "frac": round(tf / peaks["tf_sustained"], 4),
           "peak_source": f"{peaks['source']} (bf16_tflops_sustained)", "nominal_frac": round(tf / 2250.0, 4), "clocks": clocks}
    if clocks and clocks.get("sm_mhz"):
        out["clocks"]["ms_x_mhz"] = round(ms / launches * clocks["sm_mhz"], 1)
    return out


def skinny_leg(h, stream, peaks, sampler, launches=400):
    """Configuration 4 (HBM-bound): launches rotate over four independent copies of A (268 MB each, more
    than the L2), so every launch streams its A from HBM."""
    import torch
    from cudanative_jl_b200 import rng

    w = WORKLOADS["skinny"]
    M, N, K = w["M"], w["N"], w["K"]
    As, B, Cm, D, a_rows = _operands(torch, rng, w, stream, a_copies=4)
    i = [0]

    def step():
        A = As[i[0] & 3]
        i[0] += 1
        h.gemm(False, False, M, N, K, w["alpha"], A.data_ptr(), a_rows, B.data_ptr(), K, 0.0, None, M, D.data_ptr(), M, stream=stream)
    ms, (t0, t1) = event_timed(torch, step, launches, 8)
    _status_or_exit(h, "the skinny leg")
    us = ms / launches * 1e3
    gbs = algorithmic_bytes(w) / (us * 1e-6) / 1e9
    clocks = sampler.window(t0, t1) if sampler else None
    return {"workload": "skinny", "M": M, "N": N, "K": K, "launches": launches, "a_buffers": 4, "us_per_launch": round(us, 3),
            "achieved": round(gbs, 1), "unit": "GB/s", "algorithmic_bytes": algorithmic_bytes(w), "peak": peaks["hbm_gbs"],
            "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": f"{peaks['source']} (hbm_gbs)",
            "nominal_frac": round(gbs / 8000.0, 4), "value": round(2.0 * M * N * K / (us * 1e-6) / 1e12, 2), "kernel": h.last_launch(),
            "clocks": clocks}


def square_leg(h, stream, name, peaks, sampler, launches=400):
    """A tensor-bound single-GPU configuration, device-resident timing."""
    import torch
    from cudanative_jl_b200 import rng

    w = WORKLOADS[name]
    M, N, K = w["M"], w["N"], w["K"]
    (A,), B, Cm, D, a_rows = _operands(torch, rng, w, stream)

    def step():
        h.gemm(w["transA"], w["transB"], M, N, K, w["alpha"], A.data_ptr(), a_rows, B.data_ptr(), K, w["beta"],
               Cm.data_ptr() if Cm is not None else None, M, D.data_ptr(), M, stream=stream)
    ms, (t0, t1) = event_timed(torch, step, launches, 5)
    _status_or_exit(h, name)
    tf = 2.0 * M * N * K / (ms / launches * 1e-3) / 1e12
    return {"workload": name, "M": M, "N": N, "K": K, "launches": launches, "ms_per_step": round(ms / launches, 5),
            "value": round(tf, 2), "unit": "TFLOP/s", "peak": peaks["tf_burst"], "frac": round(tf / peaks["tf_burst"], 4),
            "peak_source": f"{peaks['source']} (bf16_tflops)", "nominal_frac": round(tf / 2250.0, 4), "kernel": h.last_launch(),
            "clocks": sampler.window(t0, t1) if sampler else None}


def sharded_on_one_gpu(h, stream, sampler=None, steps=10, warmup=3):
    """The sharded workload (config 5) on a single GPU: the denominator of the multi-GPU speed-up.
    Runs through the same entry point as the multi-GPU lines (b200_sharded_run with one rank) and
    checks sampled tiles of D against the CPU oracle."""
    import torch
    from cudanative_jl_b200 import rng
    from cudanative_jl_b200.gemm import ShardedGemm

    w = WORKLOADS["sharded"]
    M, N, K = w["M"], w["N"], w["K"]
    sg = ShardedGemm(h, M, N, K, rank=0, world=1)
    A = torch.as_tensor(sg.a_view(), device="cuda")
    B = torch.empty(K * N, dtype=torch.float16, device="cuda")
    Cm = torch.empty(M * N, dtype=torch.float32, device="cuda")
    D = torch.empty(M * N, dtype=torch.float32, device="cuda")
    rng.fill_device(A.data_ptr(), M, K, M, w["seed"], 0, rng.NORMAL, K ** -0.5, True, stream)
    rng.fill_device(B.data_ptr(), K, N, K, w["seed"], 1, rng.NORMAL, K ** -0.5, True, stream)
    rng.fill_device(Cm.data_ptr(), M, N, M, w["seed"], 2, rng.NORMAL, 1.0, False, stream)

    def step():
        sg.run(w["alpha"], B, w["beta"], Cm, D, stream=stream)
    ms, (t0, t1) = event_timed(torch, step, steps, warmup)
    ms /= steps
    _status_or_exit(h, "the one-GPU sharded run")
    parity = dict(check_slab_tiles(w, D, 0, N), ranks=1)
    del A
    sg.close()
    del B, Cm, D
    return {"workload": "sharded", "M": M, "N": N, "K": K, "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
            "value": round(2.0 * M * N * K / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "parity": parity,
            "clocks": sampler.window(t0, t1) if sampler else None}


def run_extra(args):
    """bfloat16 / batched entry points: operands resident in HBM, CUDA events on the launching stream."""
    import torch

    entry.load_package()
    from cudanative_jl_b200 import _lib, rng
    from cudanative_jl_b200.bfloat16 import BFloat16
    from cudanative_jl_b200.gemm import Handle

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit(f"workload {args.workload} runs on one GPU")
    w = EXTRA_WORKLOADS[args.workload]
    M, N, K, batch = w["M"], w["N"], w["K"], w["batch"]
    torch.cuda.set_device(0)
    h = Handle(0)
    stream = torch.cuda.current_stream().cuda_stream
    peaks = measured_peaks()
    L = _lib.lib()
    a_rows, a_cols = (K, M) if w["transA"] else (M, K)
    A = torch.empty(batch * M * K, dtype=torch.float16, device="cuda")  # 16-bit storage for either operand type
    B = torch.empty(batch * K * N, dtype=torch.float16, device="cuda")
    Cm = torch.empty(batch * M * N, dtype=torch.float32, device="cuda")
    D = torch.empty(batch * M * N, dtype=torch.float32, device="cuda")
    fill16 = L.b200_fill_bf16 if w["bf16"] else L.b200_fill_f16
    # a batch is laid out as one tall synthetic matrix per operand: matrix i = columns [i*cols, (i+1)*cols)
    _lib.check(fill16(stream, A.data_ptr(), a_rows, a_cols * batch, a_rows, w["seed"], 0, 0, rng.NORMAL, K ** -0.5), "fill")
    _lib.check(fill16(stream, B.data_ptr(), K, N * batch, K, w["seed"], 1, 0, rng.NORMAL, K ** -0.5), "fill")
    _lib.check(L.b200_fill_f32(stream, Cm.data_ptr(), M, N * batch, M, w["seed"], 2, 0, rng.UNIFORM, 1.0), "fill")
    ab = BFloat16 if w["bf16"] else np.float16

    def step():
        h.gemm_strided_batched(w["transA"], w["transB"], M, N, K, w["alpha"], A.data_ptr(), a_rows, M * K, B.data_ptr(), K,
                               K * N, ab, w["beta"], Cm.data_ptr(), M, M * N, np.float32, D.data_ptr(), M, M * N,
                               np.float32, batch, stream=stream)

    def loop_step():  # the same work as one launch per matrix
        for i in range(batch):
            h.gemm(w["transA"], w["transB"], M, N, K, w["alpha"], A.data_ptr() + 2 * i * M * K, a_rows,
                   B.data_ptr() + 2 * i * K * N, K, w["beta"], Cm.data_ptr() + 4 * i * M * N, M, D.data_ptr() + 4 * i * M * N,
                   M, stream=stream)

    def timed(fn, steps):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        torch.cuda.synchronize()
        code, block, _ = h.device_status()
        if code:
            raise SystemExit(f"device wait {code} ran out in block {block}")
        return ev0.elapsed_time(ev1), ev0.elapsed_time(ev1) / steps

    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.25)
    t0 = time.perf_counter()
    ms_total, ms_step = timed(step, args.steps)
    t1 = time.perf_counter()
    clocks = sampler.stop(t0, t1)
    launch = h.last_launch()
    flops = 2.0 * M * N * K * batch
    tflops = flops / (ms_step * 1e-3) / 1e12
    nbytes = batch * (2 * M * K + 2 * K * N + 8 * M * N)
    long_run = ms_total * 1e-3 > 1.0
    peak = peaks["tf_sustained"] if long_run else peaks["tf_burst"]
    out = {
        "metric": METRIC, "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16*bf16->f32" if w["bf16"] else "f16*f16->f32", "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "N": N, "K": K, "batch": batch, "transA": w["transA"],
                   "transB": w["transB"], "alpha": w["alpha"], "beta": w["beta"], "seed": w["seed"], "kernel": launch,
                   "l2": f"inputs+outputs {nbytes / 1e6:.0f} MB per step exceed the 126 MB L2; no flush"},
        "clocks": clocks, "e2e": None, "gpu_launches": args.steps,
        "roofline": {"bound": "tensor", "achieved": round(tflops, 2), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(tflops / peak, 4), "traffic": None,
                     "peak_source": f"{peaks['source']} ({'bf16_tflops_sustained' if long_run else 'bf16_tflops'})",
                     "hbm_gbs_algorithmic": round(nbytes / (ms_step * 1e-3) / 1e9, 1), "hbm_peak_gbs": peaks["hbm_gbs"]},
    }
    if batch > 1:
        _, loop_ms = timed(loop_step, max(1, args.steps // 4))
        out["one_launch_per_matrix"] = {"ms_per_step": round(loop_ms, 5), "value": round(flops / (loop_ms * 1e-3) / 1e12, 2),
                                        "unit": "TFLOP/s", "gpu_launches_per_step": batch}
    print(json.dumps(out), flush=True)


def run_reference(args):
    """CPU arm: the same product, float32 sgemm on the host cores, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    name = args.workload or ("gemm8192" if world == 1 else "sharded")
    w = WORKLOADS[name]
    total_budget = 120.0  # seconds for warm-up + steps
    n_runs = args.steps + max(args.warmup, 1)
    smp = CpuSample(w, target_seconds=max(0.5, min(12.0, total_budget / n_runs)))
    vals, secs, desc, cores = [], [], smp.desc, smp.cores
    for i in range(n_runs):
        v, dt = smp.run()
        if i >= max(args.warmup, 1):
            vals.append(v)
            secs.append(dt)
    v = float(np.mean(vals))
    M, N, K = w["M"], w["N"], w["K"]
    out = {
        "impl": "reference", "metric": METRIC, "value": round(v, 4), "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": max(args.warmup, 1), "ms_per_step": round(float(np.mean(secs)) * 1e3, 3), "higher_is_better": True,
        "scaling": "strong" if name == "sharded" else "weak", "vs_baseline": None, "dtype": "f32 (sgemm on f16-rounded inputs)",
        "data": "synthetic",
        "config": {"workload": name, "M": M, "N": N, "K": K, "transA": w["transA"], "transB": w["transB"], "alpha": w["alpha"],
                   "beta": w["beta"], "seed": w["seed"], "note": "each step is a bounded column-slab sample of the workload; "
                   "Julia (LinearAlgebra.mul!) is not installed, numpy/OpenBLAS sgemm stands in"},
        "cpu_baseline": {"value": round(v, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": round(v, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + sorted(EXTRA_WORKLOADS))
    ap.add_argument("--panels", type=int, default=16, help="K panels in which A travels (sharded)")
    ap.add_argument("--nccl-ctas", type=int, default=8, help="SMs left to NCCL while a broadcast is in flight (transport nccl)")
    ap.add_argument("--gated", action="store_true", help="p2p transport: one gated GEMM launch instead of a few launches over growing K ranges")
    ap.add_argument("--transport", default="p2p", choices=["p2p", "nccl"], help="how A reaches the other ranks (sharded)")
    ap.add_argument("--scatter-lanes", type=int, default=1, help="streams rank 0 spreads its copies over (sharded, p2p)")
    ap.add_argument("--gather-lanes", type=int, default=1, help="streams the other ranks spread their forwarding copies over (sharded, p2p)")
    ap.add_argument("--first-group", type=int, default=1, help="panels in the first GEMM launch (sharded, p2p)")
    ap.add_argument("--groups", default=None, help="panels per GEMM launch, e.g. 1,2,3,3,3,4 (sharded, p2p)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="sharded runs: skip the end-to-end leg (experiments; the line then has e2e.value 0)")
    ap.add_argument("--no-scaling-baseline", action="store_true", help="N=1: skip the one-GPU run of the sharded workload")
    ap.add_argument("--no-extras", action="store_true", help="N=1: skip the sustained / skinny / gemm4096 legs")
    args = ap.parse_args()
    if args.workload in EXTRA_WORKLOADS:
        if args.impl == "reference":
            raise SystemExit(f"workload {args.workload} has no CPU leg")
        run_extra(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
