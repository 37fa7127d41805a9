#!/usr/bin/env python
"""Benchmark of the Q4_K dequantize-matvec hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (``config.workload``): one Qwen2.5-7B-shaped decoder layer at batch 1 — the seven
Q4_K matvecs q/k/v/o/gate/up/down — on seeded synthetic super-blocks and N(0,1) f32
activations.  One "step" is one pass over the layer's seven projections.  Steps rotate
through several distinct copies of the layer's weights (> 1 GB in total, far above the
126 MB L2) so every step streams its weights from HBM.

``value`` is algorithmic GB/s (weights + x + y bytes of the seven matvecs / device time),
inputs resident in HBM, timed with CUDA events around CUDA-graph replays of the launch
sequence.  ``e2e`` is the same metric through the reference-facing host call
(``HipBuffer::matvec_q4k``: pinned host x in, host y out, copies and one sync per call).
At N > 1 the output rows of every projection are sharded across the ranks (no collective
on this path) and ``value`` is total bytes / max-over-ranks time: strong scaling.

``--impl reference`` times the CPU restatement of the reference's own Q4_K matvec
(row-parallel, AVX-512 when the host has it) on the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from modgrad_b200 import synth  # noqa: E402

WORKLOAD = "qwen2.5-7b decoder layer, 7 Q4_K matvecs, batch 1"
LAYER = synth.QWEN25_7B_LAYER
N_COPIES = 8  # distinct weight sets rotated through (8 x 131 MB = 1.05 GB >> L2)
FALLBACK_HBM_GBS = 6650.0


def layer_bytes(shard: int = 1) -> int:
    """Algorithmic bytes of one layer pass: weights + x + y per projection."""
    return sum((o // shard) * (i // 256) * 144 + 4 * i + 4 * (o // shard) for o, i in LAYER.values())


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def shard_rows(out_dim: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row range of rank `rank`: the unmodified row-major block array is cut at
    row boundaries, nothing is repacked."""
    base, rem = divmod(out_dim, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def host_layer(copy: int, rank: int, world: int):
    """Host bytes of this rank's row shard of every projection of weight copy `copy`."""
    out = {}
    for p, (name, (o, i)) in enumerate(LAYER.items()):
        lo, hi = shard_rows(o, rank, world)
        rng = np.random.Generator(np.random.PCG64([42, copy, p, rank]))
        out[name] = (synth.q4k_matrix(hi - lo, i, rng), hi - lo, i // 256)
    return out


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.period, self.samples, self.reasons, self.max_mhz = period_s, [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            pass

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, n in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---- the reference arm: the reference's CPU matvec on the host cores ---------------------------
def cpu_layer_pass(orc, layers, xs, mode):
    for name, (w, rows, bpr) in layers.items():
        orc.matvec(w, xs[name], rows, bpr, mode)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from oracle.loader import MODE_SELECT
    oracle.build()
    orc = oracle.lib()
    layers = [host_layer(c, 0, 1) for c in range(2)]  # 262 MB: above the host's last-level cache share per pass
    xs = {name: synth.activations(i, np.random.Generator(np.random.PCG64([43, p])))
          for p, (name, (o, i)) in enumerate(LAYER.items())}
    for s in range(args.warmup):
        cpu_layer_pass(orc, layers[s % 2], xs, MODE_SELECT)
    t0 = time.perf_counter()
    for s in range(args.steps):
        cpu_layer_pass(orc, layers[s % 2], xs, MODE_SELECT)
    dt = time.perf_counter() - t0
    gbs = layer_bytes() * args.steps / dt / 1e9
    cores = orc.max_threads()
    kind = "avx512" if orc.has_avx512() else "scalar"
    line = {
        "impl": "reference", "metric": "q4k_gemv_hbm_gbs", "value": round(gbs, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt / args.steps * 1e3, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "cpu_kernel": kind},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} full layer passes (7 matvecs, 131 MB each), "
                                   f"row-parallel {kind} dot on {cores} threads, rows split statically "
                                   f"(the reference's rayon splits them dynamically)"},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_sample(budget_s: float = 10.0):
    import oracle
    from oracle.loader import MODE_SELECT
    oracle.build()
    orc = oracle.lib()
    layers = [host_layer(c, 0, 1) for c in range(2)]
    xs = {name: synth.activations(i, np.random.Generator(np.random.PCG64([43, p])))
          for p, (name, (o, i)) in enumerate(LAYER.items())}
    cpu_layer_pass(orc, layers[0], xs, MODE_SELECT)
    n, t0 = 0, time.perf_counter()
    while True:
        cpu_layer_pass(orc, layers[n % 2], xs, MODE_SELECT)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or n >= 2000:
            break
    kind = "avx512" if orc.has_avx512() else "scalar"
    return {"value": round(layer_bytes() * n / dt / 1e9, 3), "unit": "GB/s", "cores": orc.max_threads(),
            "kind": "port",
            "sample": f"{n} layer passes in {dt:.1f} s, row-parallel {kind} dot (restated reference CPU matvec), rows "
                      f"split statically over the threads (the reference's rayon splits them dynamically)"}


# ---- our arm ------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5600)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=300)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the 7B-class decode tokens/s leg")
    ap.add_argument("--decode-only", action="store_true", help="run only the decode leg (profiling)")
    ap.add_argument("--no-matmul", action="store_true", help="skip the M>=16 tensor-core dequant-GEMM leg")
    ap.add_argument("--matmul-only", action="store_true", help="run only the tensor-core leg (profiling)")
    ap.add_argument("--matmul-reps", type=int, default=20)
    ap.add_argument("--no-layer70b", action="store_true", help="skip the 70B-class sharded layer leg")
    ap.add_argument("--no-kquant", action="store_true", help="skip the Q5_K / Q6_K matvec and mixed-checkpoint decode leg")
    ap.add_argument("--kquant-only", action="store_true", help="run only the K-quant leg (profiling)")
    ap.add_argument("--kquant-no-decode", action="store_true", help="K-quant leg without the mixed-checkpoint decode")
    ap.add_argument("--decode-tokens", type=int, default=256)
    ap.add_argument("--decode-prefill", type=int, default=2048)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist
    from modgrad_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the Q4_K path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = _lib.load()
    dev = torch.device("cuda", local_rank)
    warmup = max(args.warmup, 3)
    if args.decode_only:
        print(json.dumps({"decode": decode_leg(args)}), flush=True)
        return
    if args.matmul_only:
        print(json.dumps({"matmul_tc": matmul_leg(args, torch, lib, dev)}), flush=True)
        return
    if args.kquant_only:
        print(json.dumps({"kquant": kquant_leg(args, torch, lib, dev)}), flush=True)
        return

    # ---- inputs: generated on the host, uploaded verbatim, resident before timing ----------
    copies = []
    for c in range(N_COPIES):
        hl = host_layer(c, rank, world)
        copies.append({n: (torch.from_numpy(w).to(dev), rows, bpr) for n, (w, rows, bpr) in hl.items()})
    xs_host = {name: synth.activations(i, np.random.Generator(np.random.PCG64([43, p])))
               for p, (name, (o, i)) in enumerate(LAYER.items())}
    xs = {n: torch.from_numpy(v).to(dev) for n, v in xs_host.items()}
    ys = {n: torch.empty(copies[0][n][1], dtype=torch.float32, device=dev) for n in LAYER}
    torch.cuda.synchronize()

    stream = torch.cuda.Stream()

    def launch_step(c: int, s):
        for n, (w, rows, bpr) in copies[c].items():
            e = lib.launch_matvec_q4k_on_stream(w.data_ptr(), xs[n].data_ptr(), ys[n].data_ptr(), rows, bpr, s)
            if e:
                raise RuntimeError(f"launch_matvec_q4k({n}): {lib.mg_get_error_string(e).decode()}")

    with torch.cuda.stream(stream):
        for s in range(warmup):
            launch_step(s % N_COPIES, stream.cuda_stream)
        stream.synchronize()
        cycle = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cycle, stream=stream):
            for c in range(N_COPIES):
                launch_step(c, stream.cuda_stream)
        singles = []
        for c in range(args.steps % N_COPIES):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                launch_step(c, stream.cuda_stream)
            singles.append(g)
        cycle.replay()  # graph warm-up
        stream.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(args.steps // N_COPIES):
            cycle.replay()
        for g in singles:
            g.replay()
        end.record(stream)
    barrier()
    clocks = sampler.stop()
    ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    total_bytes = sum(layer_bytes_rank(r, world) for r in range(world)) * args.steps
    value = total_bytes / (ms * 1e-3) / 1e9

    # ---- per-projection device timing (explains `value`; not part of it) -------------------
    per_proj = {}
    if rank == 0:
        for n in LAYER:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(g, stream=stream):
                    for c in range(N_COPIES):
                        w, rows, bpr = copies[c][n]
                        lib.launch_matvec_q4k_on_stream(w.data_ptr(), xs[n].data_ptr(), ys[n].data_ptr(), rows, bpr,
                                                        stream.cuda_stream)
                g.replay()
                stream.synchronize()
                reps = 40
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(reps):
                    g.replay()
                b.record(stream)
                stream.synchronize()
            us = a.elapsed_time(b) * 1e3 / (reps * N_COPIES)
            w, rows, bpr = copies[0][n]
            nbytes = rows * bpr * 144 + 4 * bpr * 256 + 4 * rows
            per_proj[n] = {"us": round(us, 3), "gbs": round(nbytes / us / 1e3, 1)}

    # ---- the same layer with the matrices that share an input grouped (q/k/v, gate/up) ------
    # Not the headline: the reference's ABI has one launcher call per matrix.  This is what the
    # decode engine issues (mg_matvec_q4k_multi_on_stream): 4 matvec launches per layer.
    grouped = None
    if rank == 0:
        import ctypes as C

        def multi(c, names, s):
            n = len(names)
            w = (C.c_void_p * n)(*[copies[c][k][0].data_ptr() for k in names])
            y = (C.c_void_p * n)(*[ys[k].data_ptr() for k in names])
            dims = (C.c_int * n)(*[copies[c][k][1] for k in names])
            bpr = copies[c][names[0]][2]
            if bpr <= 32:
                return lib.mg_matvec_q4k_multi_on_stream(n, w, xs[names[0]].data_ptr(), 0, None, y, dims, bpr, s)
            return lib.launch_matvec_q4k_on_stream(w[0], xs[names[0]].data_ptr(), y[0], dims[0], bpr, s)

        def grouped_step(c, s):
            for names in (["q_proj", "k_proj", "v_proj"], ["o_proj"], ["gate_proj", "up_proj"], ["down_proj"]):
                e = multi(c, names, s)
                if e:
                    raise RuntimeError(f"grouped matvec {names}: {lib.mg_get_error_string(e).decode()}")

        with torch.cuda.stream(stream):
            grouped_step(0, stream.cuda_stream)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for c in range(N_COPIES):
                    grouped_step(c, stream.cuda_stream)
            g.replay()
            stream.synchronize()
            reps = 40
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(reps):
                g.replay()
            b.record(stream)
            stream.synchronize()
        us = a.elapsed_time(b) * 1e3 / (reps * N_COPIES)
        grouped = {"us_per_layer": round(us, 2), "gbs": round(layer_bytes_rank(0, world) / us / 1e3, 1),
                   "matvec_launches_per_layer": 4,
                   "note": "q/k/v and gate/up share their input: one launch each (mg_matvec_q4k_multi_on_stream)"}

    # ---- end to end: pinned host x in, host y out, through the host-facing call ------------
    xs_pin = {n: torch.from_numpy(v).pin_memory() for n, v in xs_host.items()}
    ys_pin = {n: torch.empty(copies[0][n][1], dtype=torch.float32).pin_memory() for n in LAYER}

    def e2e_step(c: int):
        for n, (w, rows, bpr) in copies[c].items():
            e = lib.mg_buffer_matvec_q4k(w.data_ptr(), w.numel(), xs_pin[n].data_ptr(), ys_pin[n].data_ptr(), rows, bpr)
            if e:
                raise RuntimeError(f"mg_buffer_matvec_q4k({n}): {lib.mg_get_error_string(e).decode()}")

    for s in range(3):
        e2e_step(s % N_COPIES)
    barrier()
    t0 = time.perf_counter()
    for s in range(args.e2e_steps):
        e2e_step(s % N_COPIES)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = sum(layer_bytes_rank(r, world) for r in range(world)) * args.e2e_steps / e2e_s / 1e9
    h2d = sum(4 * i for o, i in LAYER.values())
    d2h = sum(4 * copies[0][n][1] for n in LAYER)

    decode_sharded = None
    del copies, xs, ys
    torch.cuda.empty_cache()
    layer70b = None if args.no_layer70b else layer70b_leg(args, torch, lib, dev, rank, world)
    if layer70b is not None and "skipped" not in layer70b:
        eng = layer70b_engine_leg(args, rank, world)
        if rank == 0:
            layer70b["engine"] = eng
    if world > 1 and not args.no_decode:
        decode_sharded = decode_leg_sharded(args, rank, world)
    if rank == 0:
        peak, peak_kind = measured_peak()
        per_gpu = value / world
        dominant = None
        if "gate_proj" in per_proj and world == 1:
            gp = per_proj["gate_proj"]
            dominant = {"kernel": "matvec_q4k_mma_kernel", "projection": "gate_proj",
                        "bytes_per_launch": synth.gemv_bytes(*LAYER["gate_proj"]), "launch_us": gp["us"],
                        "achieved": gp["gbs"], "frac": round(gp["gbs"] / peak, 4),
                        "timing": "CUDA events around a graph of back-to-back launches of this projection "
                                  "(weight copies rotated), outside the headline region"}
        line = {
            "metric": "q4k_gemv_hbm_gbs", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms / args.steps, 6),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": f"rows sharded over {world} GPU(s), no collective",
                       "l2": f"inputs larger than L2: rotates {N_COPIES} weight copies, "
                             f"{N_COPIES * layer_bytes() / 1e9:.2f} GB", "launch": "CUDA graph replay"},
            "frac_of_8tbs_nominal": round(per_gpu / 8000.0, 4),
            "roofline": {"bound": "hbm", "achieved": round(per_gpu, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(per_gpu / peak, 4),
                         # NOT measured in this run: dram__bytes_read + write of one gate_proj launch of
                         # matvec_q4k_mma_kernel under ncu (38 459 648 B against 38 281 216 algorithmic
                         # bytes, 1.005x), scaled by bytes to the average launch of the layer
                         "traffic": round(layer_bytes_rank(0, world) / 7 * 38_459_648 / 38_281_216),
                         "traffic_source": "profiles/gemv_q4k_mma_qwen7b_layer.md (ncu capture of gate_proj), "
                                           "scaled by algorithmic bytes; not a per-run counter",
                         "peak_source": f"of {peak_kind}",
                         "kernel": "matvec_q4k_mma_kernel (gate/up, 73 % of the bytes) + matvec_q4k_ring_kernel "
                                   "(q/k/v/o/down): the timed region is the whole layer",
                         "bytes_per_launch": layer_bytes_rank(0, world) // 7,
                         "avg_launch_us": round(ms * 1e3 / (args.steps * 7), 4),
                         "dominant_kernel": dominant},
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": args.e2e_steps,
                    "call": "mg_buffer_matvec_q4k (HipBuffer::matvec_q4k): pinned host x, host y, 7 calls/step"},
            # six projections are one kernel each; down_proj (rows of 18944) is two
            "gpu_launches": args.steps * 8,
            "kernels_per_matvec": "matvec_q4k_mma_kernel for matrices of >= 4736 rows whose rows fit half an SM's "
                                  "shared memory (gate/up), else matvec_q4k_ring_kernel, with x_to_limbs_kernel in "
                                  "front of it for rows over 8192 weights (down)",
            "per_projection": per_proj,
            "grouped": grouped,
            "clocks": clocks,
        }
        if world == 1 and not args.no_matmul:
            line["matmul_tc"] = matmul_leg(args, torch, lib, dev)
        if world == 1 and not args.no_decode:
            torch.cuda.empty_cache()
            line["decode"] = decode_leg(args)
        if world == 1 and not args.no_kquant:
            torch.cuda.empty_cache()
            line["kquant"] = kquant_leg(args, torch, lib, dev)
        if world > 1 and decode_sharded is not None:
            line["decode"] = decode_sharded
        if layer70b is not None:
            line["layer70b"] = layer70b
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sample()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def matmul_leg(args, torch, lib, dev):
    """Multi-sequence dequant-GEMM on the tensor cores (tcgen05 + TMEM): M in {16, 32, 64}
    activation rows (N(0,1), f32 in, carried as two half limbs) times Q4_K W of 18944x3584 and 3584x18944.
    Weights rotate through 4 copies (153 MB > L2).  Device time per launch incl. the activation
    slab preparation kernels; GB/s counts the weight bytes, TFLOP/s counts 2*M*N*K."""
    peak_bw, kind = measured_peak()
    out = {}
    st = torch.cuda.Stream()
    ncopies = 4
    for (o, i) in [(18944, 3584), (3584, 18944)]:
        bpr = i // 256
        ws = [torch.from_numpy(synth.q4k_matrix(o, i, np.random.Generator(np.random.PCG64([44, c, o])))).to(dev)
              for c in range(ncopies)]
        for m in (16, 32, 64):
            x = torch.from_numpy(synth.activations(i, np.random.Generator(np.random.PCG64([45, m])), rows=m)).to(dev)
            y = torch.empty(m * o, device=dev)
            nb = lib.mg_matmul_q4k_scratch_bytes(m, bpr)
            scr = torch.empty(nb + 1024, dtype=torch.uint8, device=dev)
            sp = (scr.data_ptr() + 1023) & ~1023
            s = st.cuda_stream

            def launch(c):
                e = lib.launch_matmul_q4k_on_stream(ws[c].data_ptr(), x.data_ptr(), y.data_ptr(), m, o, bpr, sp, s)
                if e:
                    raise RuntimeError(f"launch_matmul_q4k: {lib.mg_get_error_string(e).decode()}")

            with torch.cuda.stream(st):
                for c in range(ncopies):
                    launch(c)
                st.synchronize()
                if lib.mg_matmul_q4k_status(sp, m, bpr) != 0:
                    raise RuntimeError("tensor-core matmul: a bounded wait expired")
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    for c in range(ncopies):
                        launch(c)
                g.replay()
                st.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(st)
                for _ in range(args.matmul_reps):
                    g.replay()
                b.record(st)
                st.synchronize()
            us = a.elapsed_time(b) * 1e3 / (args.matmul_reps * ncopies)
            wbytes = o * bpr * 144
            out[f"{o}x{i}_M{m}"] = {"us": round(us, 2), "weight_gbs": round(wbytes / us / 1e3, 1),
                                    "hbm_frac": round(wbytes / us / 1e3 / peak_bw, 4),
                                    "tflops": round(2.0 * m * o * i / us / 1e6, 1)}
        del ws
    out["peak_source"] = f"of {kind}"
    return out


def layer70b_leg(args, torch, lib, dev, rank, world):
    """A 70B-class decoder layer (hidden 8192, SwiGLU 28672, 64/8 heads of 128): every
    projection's rows sharded over the ranks, the output slices all-gathered at the four points of
    the layer where the decode engine exchanges them, the whole pass replayed as one CUDA graph.  At one GPU
    the same layer without the gathers.  Weight copies are rotated so that the per-rank working
    set exceeds L2."""
    import torch.distributed as dist
    layer = synth.LLAMA_70B_LAYER
    EXCHANGE_AFTER = ("v_proj", "o_proj", "up_proj", "down_proj")
    shard_bytes = sum((shard_rows(o, rank, world)[1] - shard_rows(o, rank, world)[0]) * (i // 256) * 144
                      for o, i in layer.values())
    n_copies = max(2, min(8, -(-400_000_000 // shard_bytes)))
    copies = []
    for c in range(n_copies):
        ws = {}
        for p, (name, (o, i)) in enumerate(layer.items()):
            lo, hi = shard_rows(o, rank, world)
            rng = np.random.Generator(np.random.PCG64([44, c, p, rank]))
            ws[name] = (torch.from_numpy(synth.q4k_matrix(hi - lo, i, rng)).to(dev), lo, hi, i // 256)
        copies.append(ws)
    xs = {n: torch.from_numpy(synth.activations(i, np.random.Generator(np.random.PCG64([45, p])))).to(dev)
          for p, (n, (o, i)) in enumerate(layer.items())}
    ys = {n: torch.zeros(o, dtype=torch.float32, device=dev) for n, (o, i) in layer.items()}
    even = all(o % world == 0 for o, i in layer.values())
    stream = torch.cuda.Stream()

    def step(c, s, only=None):
        for n, (w, lo, hi, bpr) in copies[c].items():
            if only is not None and n != only:
                continue
            e = lib.launch_matvec_q4k_on_stream(w.data_ptr(), xs[n].data_ptr(), ys[n].data_ptr() + 4 * lo, hi - lo,
                                                bpr, s)
            if e:
                raise RuntimeError(f"launch_matvec_q4k({n}): {lib.mg_get_error_string(e).decode()}")
            if world > 1 and n in EXCHANGE_AFTER:  # in place: this rank's slice already sits at its offset
                dist.all_gather_into_tensor(ys[n], ys[n][lo:hi])

    if world > 1 and not even:
        return {"skipped": "a projection's rows do not divide by the number of GPUs"}

    def timed(step_fn, only=None):
        with torch.cuda.stream(stream):
            for c in range(3):
                step_fn(c % n_copies, stream.cuda_stream, only)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for c in range(n_copies):
                    step_fn(c, stream.cuda_stream, only)
            graph.replay()
            stream.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        reps = 50
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            a.record(stream)
            for _ in range(reps):
                graph.replay()
            b.record(stream)
            stream.synchronize()
        ms = a.elapsed_time(b)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms * 1e3 / (reps * n_copies)

    # NCCL's kernels follow ours in the stream: ours must not let them launch before they finish
    trigger_before = lib.mg_pdl_early_trigger(0 if world > 1 else 1)
    us_nccl = timed(step)
    per_proj = {n: round(timed(step, n), 2) for n in layer} if world == 1 else None
    lib.mg_pdl_early_trigger(trigger_before)
    us, fused_note, max_diff = us_nccl, None, None
    final_o = ys["o_proj"].clone()  # gathered o_proj output of the last weight copy
    if world > 1:
        # the same layer with the all-gather done by the matvec kernels themselves: every result row
        # is stored into all peers' arenas over NVLink, the kernel ends with the flag handshake
        import ctypes as C
        names = list(layer)
        offs, off = {}, lib.mg_peer_arena_offset()
        for n in names:
            offs[n] = off
            off += (4 * layer[n][0] + 255) // 256 * 256
        handle = (C.c_ubyte * 64)()
        xh = C.c_void_p()
        e = lib.mg_peer_exchange_create(off, rank, world, handle, C.byref(xh))
        if e:
            fused_note = f"peer exchange unavailable: {lib.mg_get_error_string(e).decode()}"
        else:
            gathered = [None] * world
            dist.all_gather_object(gathered, bytes(handle))
            blob = (C.c_ubyte * (64 * world)).from_buffer_copy(b"".join(gathered))
            e = lib.mg_peer_exchange_open(xh, blob)
            ok = torch.tensor([0 if e else 1], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                fused_note = "peer exchange unavailable: a rank could not map its peers"
            else:
                arena = lib.mg_peer_arena(xh)

                def step_fused(c, s, only=None):
                    for site, (n, (w, lo, hi, bpr)) in enumerate(copies[c].items()):
                        if only is not None and n != only:
                            continue
                        if n in EXCHANGE_AFTER and lib.mg_peer_fuse_next(xh, site):
                            raise RuntimeError("mg_peer_fuse_next")
                        e2 = lib.launch_matvec_q4k_on_stream(w.data_ptr(), xs[n].data_ptr(), arena + offs[n] + 4 * lo,
                                                             hi - lo, bpr, s)
                        if e2:
                            raise RuntimeError(f"launch_matvec_q4k({n}): {lib.mg_get_error_string(e2).decode()}")

                us = timed(step_fused)
                per_proj = {n: round(timed(step_fused, n), 2) for n in layer}
                if lib.mg_peer_exchange_status(xh):
                    raise RuntimeError("peer exchange: a bounded wait expired")
                # both paths end on the same weight copy: the gathered vectors must be identical
                max_diff = 0.0
                for n in EXCHANGE_AFTER:
                    got = torch.empty_like(ys[n])
                    lib.mg_memcpy_d2d(got.data_ptr(), arena + offs[n], 4 * layer[n][0])
                    torch.cuda.synchronize()
                    max_diff = max(max_diff, float((got - ys[n]).abs().max().item()))
                    if n == "o_proj":
                        final_o = got.clone()
            dist.barrier()
            lib.mg_peer_exchange_destroy(xh)
    total = sum(o * (i // 256) * 144 + 4 * i + 4 * o for o, i in layer.values())
    peak, kind = measured_peak()
    gathered = sum(4 * layer[n][0] for n in EXCHANGE_AFTER) if world > 1 else 0
    # the gathered o_proj vector against the CPU oracle: 48 sampled rows of every rank's shard
    oracle_err = None
    if rank == 0:
        import oracle
        oracle.build()
        orc = oracle.lib()
        o, i = layer["o_proj"]
        y_host = final_o.cpu().numpy().astype(np.float64)
        x_host = xs["o_proj"].cpu().numpy()
        pidx = list(layer).index("o_proj")
        got_rows, ref_rows = [], []
        for r in range(world):
            lo, hi = shard_rows(o, r, world)
            wr = synth.q4k_matrix(hi - lo, i, np.random.Generator(np.random.PCG64([44, n_copies - 1, pidx, r])))
            pick = np.unique(np.random.Generator(np.random.PCG64([46, r])).integers(0, hi - lo, 48))
            sub = wr.reshape(hi - lo, -1)[pick].reshape(-1)
            ref_rows.append(orc.matvec_f64(sub, x_host, pick.size, i // 256))
            got_rows.append(y_host[lo + pick])
        ref, got_v = np.concatenate(ref_rows), np.concatenate(got_rows)
        oracle_err = float(np.max(np.abs(got_v - ref)) / np.sqrt(np.mean(ref * ref)))
    out = {"workload": "70B-class decoder layer (8192 / 28672, 64/8 heads), 7 Q4_K matvecs, batch 1",
           "n_gpus": world, "us_per_layer": round(us, 2), "gbs_total": round(total / us / 1e3, 1),
           "hbm_frac_per_gpu": round(total / us / 1e3 / world / peak, 4), "peak_source": f"of {kind}",
           "bytes_per_layer": total, "allgather_bytes_per_layer": gathered,
           "collective": ("4 all-gathers per layer, as the decode engine issues them (q/k stay rank-local under "
                          "head-parallel attention; the exchanges follow v_proj - standing in for the attention "
                          "output -, o_proj, up_proj - standing in for the SwiGLU slice - and down_proj), "
                          + ("fused into the producing matvec kernels (peer stores over NVLink)"
                             if fused_note is None else "NCCL all-gathers inside the graph")
                          if world > 1 else "none"),
           "oracle_check": {"projection": "o_proj", "rows": "48 sampled rows per shard", "max_err_over_rms": oracle_err,
                            "bound": 1e-5, "ok": None if oracle_err is None else bool(oracle_err <= 1e-5)},
           "us_per_layer_nccl": round(us_nccl, 2) if world > 1 else None,
           "fused_vs_nccl_max_abs_diff": max_diff, "note": fused_note, "per_projection_us": per_proj,
           "weight_copies_rotated": n_copies, "launch": "CUDA graph replay"}
    del copies
    torch.cuda.empty_cache()
    return out


def layer70b_engine_leg(args, rank, world):
    """The same 70B-class layer as the decode ENGINE runs it (grouped q/k/v and gate/up launches with the
    RMSNorm in front, one-launch attention over a short context, SwiGLU into limb records, the four
    exchanges per layer in the engine's default protocol): two random-init engines of 2 and 6 layers
    decode the same tokens; the difference of their times per token is four layers."""
    import torch
    import torch.distributed as dist
    from modgrad_b200 import decoder as dec, shard
    prefill, tokens = 64, 48
    ms_tok, mode, kpt = {}, None, {}
    for n_layers in (2, 6):
        cfg = dec.DecoderConfig(n_layers=n_layers, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128, d_ff=28672,
                                vocab=32768, max_seq=prefill + tokens + 16, rms_eps=1e-5, rope_base=5e5)
        nccl_id = shard.nccl_id_from_torch(rank) if world > 1 else None
        d = dec.Q4KDecoder(cfg, rank, world, nccl_id)
        d.load_random_shard(7, prefill=prefill)
        if world > 1:
            dist.barrier()
        d.generate(1, 4)
        d.set_position(prefill)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        _, ms = d.generate(1, tokens)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        ms_tok[n_layers] = ms / tokens
        kpt[n_layers] = d.kernels_per_token()
        mode = d.gather_mode() if world > 1 else "none"
        d.close()
        del d
        torch.cuda.empty_cache()
    us_layer = (ms_tok[6] - ms_tok[2]) * 1e3 / 4
    layer_bytes70 = sum(o * (i // 256) * 144 for o, i in synth.LLAMA_70B_LAYER.values())
    peak, kind = measured_peak()
    return {"us_per_layer": round(us_layer, 2), "gbs_total": round(layer_bytes70 / us_layer / 1e3, 1),
            "hbm_frac_per_gpu": round(layer_bytes70 / us_layer / 1e3 / world / peak, 4), "peak_source": f"of {kind}",
            "ms_per_token_2_layers": round(ms_tok[2], 4), "ms_per_token_6_layers": round(ms_tok[6], 4),
            "kernels_per_layer": (kpt[6] - kpt[2]) // 4, "exchange": mode, "exchanges_per_layer": 4 if world > 1 else 0,
            "context": f"{prefill} prefilled + {tokens} decoded positions",
            "method": "time per token of a 6-layer engine minus that of a 2-layer engine, over 4"}


def decode_leg_sharded(args, rank, world):
    """The same decode, rows sharded over `world` GPUs (one process each), NCCL all-gathers of the
    output slices inside the per-token graph.  Strong scaling: one model, one token stream."""
    import torch
    import torch.distributed as dist
    from modgrad_b200 import decoder as dec, shard
    cfg = dec.QWEN25_7B
    nccl_id = shard.nccl_id_from_torch(rank)
    d = dec.Q4KDecoder(cfg, rank, world, nccl_id)
    d.load_random_shard(42, prefill=args.decode_prefill)
    dist.barrier()
    d.generate(1, 4)
    d.set_position(args.decode_prefill)
    torch.cuda.synchronize()
    dist.barrier()
    toks, ms = d.generate(1, args.decode_tokens)
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    peak, kind = measured_peak()
    ctx0, ctx1 = args.decode_prefill, args.decode_prefill + args.decode_tokens
    bpt = (cfg.token_bytes(ctx0) + cfg.token_bytes(ctx1)) // 2
    ms_tok = ms / args.decode_tokens
    out = {"tok_s": round(1e3 / ms_tok, 2), "ms_per_token": round(ms_tok, 4), "tokens": args.decode_tokens,
           "n_gpus": world, "context": f"{ctx0} prefilled N(0,1) half KV + {args.decode_tokens} decoded",
           "bytes_per_token": bpt, "gbs_total": round(bpt / ms_tok / 1e6, 1),
           "hbm_frac_per_gpu": round(bpt / ms_tok / 1e6 / peak / world, 4), "peak_source": f"of {kind}",
           "kernels_per_token": d.kernels_per_token(), "collectives_per_token": 4 * cfg.n_layers + 1,
           "parallelism": f"rows sharded over {world} GPUs, head-parallel attention, all-gather of slices: "
                          + {"nccl": "NCCL collectives in the token graph",
                             "peer": "one peer-store gather kernel per collective (NVLink)",
                             "fused": "peer stores over NVLink fused into the producing kernels, flag handshake at their end",
                             "stamped": "peer stores over NVLink fused into the producing kernels, every word stamped "
                                        "with its epoch (no handshake; the consuming kernel polls)"}[d.gather_mode()],
           "gather": d.gather_mode(),
           "model": "qwen2.5-7b-shaped, random-init, Q4_K linears"}
    d.close()
    return out


def decode_leg(args):
    """7B-class random-init Q4_K decoder (28 layers, hidden 3584, SwiGLU 18944, 28/4 heads of 128,
    half embedding / LM head of vocab 152064): greedy decode after a prefilled half KV cache,
    one CUDA-graph launch per token, arg-max fed back on the device, one sync at the end."""
    from modgrad_b200 import decoder as dec
    cfg = dec.QWEN25_7B
    t0 = time.perf_counter()
    d = dec.Q4KDecoder(cfg)
    d.load_random(42, prefill=args.decode_prefill)
    load_s = time.perf_counter() - t0
    d.generate(1, 4)                       # graph capture + warm-up
    d.set_position(args.decode_prefill)
    toks, ms = d.generate(1, args.decode_tokens)
    peak, kind = measured_peak()
    ctx0, ctx1 = args.decode_prefill, args.decode_prefill + args.decode_tokens
    bpt = (cfg.token_bytes(ctx0) + cfg.token_bytes(ctx1)) // 2
    ms_tok = ms / args.decode_tokens
    out = {"tok_s": round(1e3 / ms_tok, 2), "ms_per_token": round(ms_tok, 4), "tokens": args.decode_tokens,
           "context": f"{ctx0} prefilled N(0,1) half KV + {args.decode_tokens} decoded",
           "bytes_per_token": bpt, "gbs": round(bpt / ms_tok / 1e6, 1),
           "hbm_frac": round(bpt / ms_tok / 1e6 / peak, 4), "peak_source": f"of {kind}",
           "kernels_per_token": d.kernels_per_token(), "load_s": round(load_s, 1),
           "model": "qwen2.5-7b-shaped, random-init, Q4_K linears"}
    d.close()
    return out


def kquant_leg(args, torch, lib, dev):
    """The other K-quants of a real checkpoint.  (1) Q5_K / Q6_K batch-1 matvecs on the 7B shapes where such
    tensors occur (attn_v, ffn_down, the LM head), weights rotated through > 400 MB of copies, CUDA events
    around back-to-back launches, from f32 activations and from limb records with the residual add folded in
    (as the typed engine calls them).  (2) Greedy decode of the 7B-class model with the tensor types of a Q4_K_M-style file:
    attn_v and ffn_down Q6_K in half of the layers, Q4_K token embedding, Q6_K LM head, the rest Q4_K."""
    from modgrad_b200 import decoder as dec
    rng = np.random.Generator(np.random.PCG64(77))
    stream = torch.cuda.current_stream().cuda_stream
    peak, kind = measured_peak()
    block_bytes = {5: 176, 6: 210}
    shapes = []
    for knd, name in ((5, "q5k"), (6, "q6k")):
        for label, rows, cols in (("attn_v", 512, 3584), ("ffn_down", 3584, 18944), ("lm_head", 152064, 3584)):
            one = synth.kquant_matrix(knd, rows, cols, rng)
            copies = max(2, int(400e6 // one.size) + 1)
            w = torch.empty(copies * one.size, dtype=torch.uint8, device=dev)
            w.view(copies, one.size)[:] = torch.from_numpy(one).to(dev)
            x = torch.randn(cols, device=dev)
            y = torch.zeros(rows, device=dev)
            rec = torch.empty(lib.mg_q4k_limb_record_bytes(cols), dtype=torch.uint8, device=dev)
            assert lib.mg_q4k_x_to_limbs_on_stream(x.data_ptr(), cols, rec.data_ptr(), stream) == 0
            variants = [("f32 x", lambda c: lib.mg_matvec_kquant_on_stream(8 + knd, w.data_ptr() + c * one.size, x.data_ptr(), 0,
                                                                           None, y.data_ptr(), rows, cols // 256, stream))]
            variants.append(("limb records + residual", lambda c: lib.mg_matvec_kquant_on_stream(
                8 + knd, w.data_ptr() + c * one.size, rec.data_ptr(), 1, y.data_ptr(), y.data_ptr(), rows, cols // 256, stream)))
            for vname, fn in variants:
                for i in range(5):
                    assert fn(i % copies) == 0
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 40
                a.record()
                for i in range(reps):
                    fn(i % copies)
                b.record()
                torch.cuda.synchronize()
                us = a.elapsed_time(b) / reps * 1e3
                nbytes = rows * (cols // 256) * block_bytes[knd] + 4 * cols + 4 * rows
                shapes.append({"type": name, "tensor": label, "rows": rows, "cols": cols, "input": vname,
                               "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
                               "hbm_frac": round(nbytes / us / 1e3 / peak, 4)})
            del w
    out = {"matvec": shapes, "peak_source": f"of {kind}", "gpu_launches": len(shapes) * 40}
    if args.kquant_no_decode:
        return out
    torch.cuda.empty_cache()
    cfg = dec.QWEN25_7B
    Q4, Q6, F16 = 12, 14, 1
    n = cfg.n_layers
    more_bits = lambda l: l < n // 8 or l >= 7 * n // 8 or (l - n // 8) % 3 == 2
    mix = [[Q4, Q4, Q6 if more_bits(l) else Q4, Q4, Q4, Q4, Q6 if more_bits(l) else Q4] for l in range(n)]
    d = dec.Q4KDecoder(cfg, types=(mix, Q4, Q6))
    D = cfg.d_model

    def mat(t, r, c):
        return synth.q4k_matrix(r, c, rng) if t == Q4 else synth.kquant_matrix(6, r, c, rng)

    total = 0
    for which, t in ((dec.W_EMBED, Q4), (dec.W_LM_HEAD, Q6)):
        m = mat(t, cfg.vocab, D)
        total += m.size if which == dec.W_LM_HEAD else D // 256 * 144
        d.upload(0, which, m)
    norm = (1.0 + 0.05 * rng.standard_normal(D, dtype=np.float32)).astype(np.float32)
    d.upload(0, dec.W_OUT_NORM, norm)
    for l in range(n):
        for idx, (o, i_) in enumerate(cfg.shapes().values()):
            m = mat(mix[l][idx], o, i_)
            total += m.size
            d.upload(l, idx, m)
        d.upload(l, dec.W_ATTN_NORM, norm)
        d.upload(l, dec.W_FFN_NORM, norm)
        k = rng.standard_normal(args.decode_prefill * cfg.kv_dim, dtype=np.float32).astype(np.float16)
        d.set_kv(l, k, k, args.decode_prefill)
    d.generate(1, 4)                       # graph capture + warm-up
    d.set_position(args.decode_prefill)
    tokens = min(args.decode_tokens, 128)
    _, ms = d.generate(1, tokens)
    ms_tok = ms / tokens
    kv = 2 * n * cfg.kv_dim * 2 * (args.decode_prefill + tokens // 2)
    out["decode_mixed"] = {"tok_s": round(1e3 / ms_tok, 2), "ms_per_token": round(ms_tok, 4), "tokens": tokens,
                           "weight_bytes_per_token": total, "gbs": round((total + kv) / ms_tok / 1e6, 1),
                           "hbm_frac": round((total + kv) / ms_tok / 1e6 / peak, 4),
                           "launches_per_token": d.kernels_per_token(),
                           "model": "qwen2.5-7b-shaped, random-init; attn_v and ffn_down Q6_K in %d of %d layers, "
                                    "Q4_K embedding, Q6_K LM head, other linears Q4_K" % (sum(map(more_bits, range(n))), n)}
    d.close()
    return out


def layer_bytes_rank(rank: int, world: int) -> int:
    tot = 0
    for o, i in LAYER.values():
        lo, hi = shard_rows(o, rank, world)
        tot += (hi - lo) * (i // 256) * 144 + 4 * i + 4 * (hi - lo)
    return tot


if __name__ == "__main__":
    main()
