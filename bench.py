#!/usr/bin/env python3
"""Benchmark of the SGEMM hot path: SGEMM TFLOPS (avg and min) + fraction of B200 FP32 peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one GEMM through the library's C ABI.  Workloads (all FP32, synthetic):
  c2  (default at 1 GPU)  4096^3 row-major, A ~ U[-1,1) seed 1 (mt19937, logical order), B = identity;
                          the identity-multiply methodology the reference's headline table uses.
  c5  (default at N > 1)  16384^3 row-major, A,B ~ N(0,1) seed 4 generated on the device; C is
                          partitioned by N-column blocks over the ranks (each rank holds all of A and its
                          K x N/G slice of B); no data-path collective.  An NCCL all-gather of C is timed
                          separately and reported as `allgather_ms`, outside `value`.
  c3:<abc>, c4:<MxNxK>    one layout of the 4096^3 all-layout configuration / one sweep shape.
At 1 GPU the line also carries `all_layouts` (the eight layout permutations at 4096^3, TFLOP/s and % of the FP32
peak each); at N > 1 rank 0 also times the unsharded workload on its own GPU (`single_gpu_same_workload_tflops`,
`speedup_vs_single_gpu`).

Prints ONE JSON line (rank 0).  `value` is whole-job TFLOPS with operands resident in HBM; `e2e` is the
same metric through the same C ABI call with pinned HOST buffers, the host<->device copies inside the
timed region.  `--impl reference` times the reference's own host GEMM loop (oracle/_ref, else the
oracle port) on the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sgemm_tflops"
UNIT = "TFLOP/s"
L2_BYTES = 126e6
FP32_LANES_PER_SM = 128


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
def parse_workload(name: str, n_gpus: int):
    if not name:
        name = "c2" if n_gpus == 1 else "c5"
    if name == "c2":
        return dict(name="c2", M=4096, N=4096, K=4096, la=0, lb=0, lc=0, init="identity", seed=1,
                    desc="4096^3 rrr, A~U[-1,1) seed 1, B=I (identity-multiply methodology)")
    if name == "c5":
        return dict(name="c5", M=16384, N=16384, K=16384, la=0, lb=0, lc=0, init="normal", seed=4,
                    desc="16384^3 rrr, A,B~N(0,1) seed 4 (device Philox), C column blocks over the ranks")
    if name.startswith("c3:"):
        la, lb, lc = ("rc".index(ch) for ch in name[3:])
        return dict(name=name, M=4096, N=4096, K=4096, la=la, lb=lb, lc=lc, init="uniform", seed=2,
                    desc=f"4096^3 layout {name[3:]} (A,B,C), A,B~U[-1,1) seed 2")
    if name.startswith("c4:"):
        M, N, K = (int(x) for x in name[3:].split("x"))
        return dict(name=name, M=M, N=N, K=K, la=0, lb=0, lc=0, init="uniform", seed=3,
                    desc=f"{M}x{N}x{K} rrr, A,B~U[-1,1) seed 3")
    raise SystemExit(f"unknown workload {name}")


def host_inputs(w):
    """Host A, B (packed float32 numpy) for the uniform / identity workloads, via the oracle's generator
    (the input generator is test infrastructure shared with the parity tests, not a compute path)."""
    import oracle
    M, N, K = w["M"], w["N"], w["K"]
    if w["init"] == "identity":
        A, _ = oracle.fill_ab(w["seed"], w["la"], w["lb"], M, N, K, with_b=False)
        return A, oracle.fill_identity(w["lb"], K, N)
    A, B = oracle.fill_ab(w["seed"], w["la"], w["lb"], M, N, K)
    return A, B


# ------------------------------------------------------------------------------------------------
# clocks during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], None, [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                smax = float(f[1])
                power.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": smax, "reasons": ["no samples"]}
        # "under load" = samples drawing at least 60 % of the highest power seen
        pmax = max(power)
        load = [c for c, p in zip(sm, power) if p >= 0.6 * pmax] or sm
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": smax, "reasons": sorted(reasons),
                "power_w_max": pmax, "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the reference's host GEMM loop on a bounded band of rows of C
# ------------------------------------------------------------------------------------------------
def cpu_reference_run(w, target_seconds: float = 12.0, repeats: int = 1):
    """Times the reference's sgemm_cpu (test/test.hpp:30-45) on a band of full rows of C of workload `w`,
    the band split over all host threads.  Uses the reference's own compiled code (oracle/_ref) when it
    has been built, else the oracle's restatement.  Returns (tflops, info)."""
    import numpy as np
    import oracle
    M, N, K, la, lb, lc = w["M"], w["N"], w["K"], w["la"], w["lb"], w["lc"]
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(1234)
    use_ref = oracle.have_ref() and la == 0 and lc == 0  # a band of rows is a packed sub-matrix only for row-major A, C
    B = (rng.random(K * N, dtype=np.float32) * 2 - 1) if w["init"] != "identity" else oracle.fill_identity(lb, K, N)

    def run(rows: int) -> float:
        A = rng.random(rows * K, dtype=np.float32) * 2 - 1
        t0 = time.perf_counter()
        if use_ref:
            # unmodified reference loop, one band of rows per thread (ctypes releases the GIL)
            per = max(1, math.ceil(rows / cores))
            outs, ths = [], []
            for r0 in range(0, rows, per):
                r1 = min(rows, r0 + per)
                a = np.ascontiguousarray(A[r0 * K:r1 * K])
                th = threading.Thread(target=lambda a=a, n=r1 - r0: outs.append(
                    oracle.ref_sgemm_cpu(lc, la, lb, a, B, n, N, K)))
                th.start()
                ths.append(th)
            for th in ths:
                th.join()
        else:
            Afull = A if la == 0 else np.ascontiguousarray(A.reshape(rows, K).T).ravel()
            oracle.sgemm_f32(lc, la, lb, Afull, B, rows, N, K, threads=cores)
        return time.perf_counter() - t0

    rows = min(M, max(cores, 8))
    t = run(rows)
    # grow the band towards the time budget
    want = int(min(M, max(rows, rows * target_seconds / max(t, 1e-3))))
    want = max(cores, want // cores * cores)
    times = [run(want) for _ in range(repeats)] if want > rows else [t]
    rows = want if want > rows else rows
    best = statistics.mean(times)
    tflops = 2.0 * rows * N * K / best / 1e12
    info = {"value": tflops, "unit": UNIT, "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"{rows} of {M} full rows of C ({rows}x{N}x{K}), {best:.2f} s, "
                      f"full problem extrapolates to {best * M / rows:.1f} s"}
    return tflops, info


def reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_all = []
    budget = max(2.0, min(15.0, 120.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_reference_run(w, target_seconds=budget)
    info = None
    for _ in range(args.steps):
        tf, info = cpu_reference_run(w, target_seconds=budget)
        t_all.append(tf)
    value = statistics.mean(t_all)
    info["value"] = value
    M, N, K = w["M"], w["N"], w["K"]
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 2.0 * M * N * K / (value * 1e12) * 1e3,
            "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "desc": w["desc"], "M": M, "N": N, "K": K,
                       "layout_abc": "".join("rc"[x] for x in (w["la"], w["lb"], w["lc"]))},
            "cpu_baseline": info,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def ours(args, w):
    import numpy as np
    import torch
    import torch.distributed as dist
    import rocm_sgemm_b200 as sg

    sg.lib()  # fail loudly if the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    M, N, K, la, lb, lc = w["M"], w["N"], w["K"], w["la"], w["lb"], w["lc"]
    G = world
    if N % G:
        raise SystemExit("N must divide over the ranks")
    Nl = N // G  # this rank's column block of B and C

    # ---- operands resident in HBM -------------------------------------------------------------------
    if w["init"] == "normal":
        g = torch.Generator(device=dev)
        g.manual_seed(w["seed"])
        dA = torch.randn(M * K, generator=g, dtype=torch.float32, device=dev)
        dBfull = torch.randn(K * N, generator=g, dtype=torch.float32, device=dev)
        hA = hB = None
    else:
        hA, hBfull = host_inputs(w)
        dA = torch.from_numpy(hA).to(dev)
        dBfull = torch.from_numpy(hBfull).to(dev)
    single_gpu = None
    if G > 1:
        from rocm_sgemm_b200 import sharded
        if rank == 0:
            # the same workload unsharded on one GPU, so that the N-GPU speed-up is formed on ONE workload in one run
            dCfull = torch.empty(M * N, dtype=torch.float32, device=dev)
            for _ in range(2):
                sg.gemm(lc, la, lb, dCfull, dA, dBfull, M, N, K)
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(3):
                sg.gemm(lc, la, lb, dCfull, dA, dBfull, M, N, K)
            s1.record()
            s1.synchronize()
            single_gpu = {"ms_per_step": s0.elapsed_time(s1) / 3}
            single_gpu["tflops"] = 2.0 * M * N * K / (single_gpu["ms_per_step"] * 1e-3) / 1e12
            del dCfull
        dB = sharded.local_b_slice(dBfull, lb, K, N, G, rank)  # packed K x Nl slice of this rank
        del dBfull
        torch.cuda.empty_cache()
    else:
        dB = dBfull
    dC = torch.empty(M * Nl, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream()
    params, variant = sg.select_config(M, Nl, K, lc, la, lb)
    # GEMM kernel + split-K reduction; the warp-specialised kernels transpose a pre-transposed operand themselves,
    # the others get one transposition kernel per such operand in front
    def kernels_per_call(p):
        return 1 + (1 if p.split_k > 1 else 0) + (0 if p.pipeline >= 1 else bin(p.pretranspose).count("1"))
    launches_per_step = kernels_per_call(params)
    launches_total = 0

    def step():
        sg.gemm(lc, la, lb, dC, dA, dB, M, Nl, K, stream=stream)

    flops_total = 2.0 * M * N * K
    flops_rank = 2.0 * M * Nl * K

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record()
    for e0, e1 in ev:
        e0.record()
        step()
        e1.record()
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_begin.elapsed_time(t_end)
    per = [e0.elapsed_time(e1) for e0, e1 in ev]
    tt = torch.tensor([total_ms, max(per), statistics.mean(per), min(per), statistics.median(per)], dtype=torch.float64,
                      device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    total_ms, max_ms, avg_ms, min_ms, median_ms = tt.tolist()
    ms_per_step = total_ms / args.steps
    value = flops_total / (ms_per_step * 1e-3) / 1e12

    # ---- correctness of what was just timed (cheap, on device) ---------------------------------------
    check = None
    if w["init"] == "identity" and G == 1:
        check = bool(torch.equal(dC.view(torch.int32), dA.view(torch.int32)))
        if not check:
            raise SystemExit("identity-multiply result differs from A: refusing to report a number")

    # ---- optional collective: all-gather of the C column blocks, timed separately ---------------------
    allgather_ms = None
    if world > 1:
        full = torch.empty(G * M * Nl, dtype=torch.float32, device=dev)
        for _ in range(2):
            dist.all_gather_into_tensor(full, dC)
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        dist.all_gather_into_tensor(full, dC)
        a1.record()
        barrier()
        ta = torch.tensor([a0.elapsed_time(a1)], dtype=torch.float64, device=dev)
        dist.all_reduce(ta, op=dist.ReduceOp.MAX)
        allgather_ms = ta.item()

    # ---- the same product with the all-gather folded into the GEMM epilogue (peer stores over NVLink) -------------
    fused = None
    if world > 1:
        from rocm_sgemm_b200 import sharded
        try:  # the constructor fails on all ranks or on none
            pc = sharded.PeerGatheredC(M, N, lc, G, rank)
        except RuntimeError as ex:
            pc, fused = None, {"unavailable": str(ex)}
        if pc is not None:
            for _ in range(2):
                sharded.fused_gather_gemm(sg, pc, lc, la, lb, dA, dB, M, N, K, stream=stream)
            barrier()
            fsteps = max(3, min(args.steps, 10))
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            for _ in range(fsteps):
                sharded.fused_gather_gemm(sg, pc, lc, la, lb, dA, dB, M, N, K, stream=stream)
            f1.record()
            barrier()
            tf = torch.tensor([f0.elapsed_time(f1) / fsteps], dtype=torch.float64, device=dev)
            dist.all_reduce(tf, op=dist.ReduceOp.MAX)
            # every rank now holds the whole C: it must equal the NCCL all-gather of the separately computed blocks
            same = torch.equal(pc.tensor().view(torch.int32), sharded.assemble_c(full, lc, M, N, G).view(torch.int32))
            ts = torch.tensor([1.0 if same else 0.0], dtype=torch.float64, device=dev)
            dist.all_reduce(ts, op=dist.ReduceOp.MIN)
            fused = {"ms_per_step": tf.item(), "tflops": flops_total / (tf.item() * 1e-3) / 1e12,
                     "gemm_then_nccl_allgather_ms": avg_ms + allgather_ms, "bit_identical_to_allgather": bool(ts.item()),
                     "note": "b200_sgemm_multi: each rank's epilogue stores its column block into every rank's C (CUDA IPC "
                             "peer mappings, plain stores); informational, not part of value"}
            pc.close()
        del full

    # ---- end to end: pinned host buffers -> device -> GEMM -> host, every step -------------------------
    e2e_steps = max(3, min(args.steps, 20))
    if hA is None:
        # device-generated workload: stage a host copy once (outside the timed region)
        hA_t = dA.cpu().pin_memory()
        hB_t = dB.cpu().pin_memory()
    else:
        hA_t = torch.from_numpy(hA).pin_memory()
        hB_t = dB.cpu().pin_memory()
    hC_t = torch.empty(M * Nl, dtype=torch.float32).pin_memory()

    hC2_t = torch.empty(M * Nl, dtype=torch.float32).pin_memory()

    # what this box's PCIe link gives a plain pinned copy (explains the end-to-end figure: the uploads bound it)
    def copy_gbs(dst, src):
        n = min(dst.numel(), src.numel(), 16 * 1024 * 1024)  # 64 MiB
        for _ in range(2):
            dst[:n].copy_(src[:n], non_blocking=True)
        torch.cuda.synchronize()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(4):
            dst[:n].copy_(src[:n], non_blocking=True)
        c1.record()
        c1.synchronize()
        return 4 * n * 4 / (c0.elapsed_time(c1) * 1e-3) / 1e9

    pcie_h2d_gbs = copy_gbs(dA, hA_t)
    pcie_d2h_gbs = copy_gbs(hC_t, dC)

    # both directions at once, on two streams: what the link gives the pipelined steps, whose uploads and downloads
    # overlap (on some hosts the two directions share about one direction's rate)
    def duplex_gbs():
        n = min(dA.numel(), hA_t.numel(), hC_t.numel(), dC.numel(), 16 * 1024 * 1024)
        s_up, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        torch.cuda.synchronize()
        c0, c1, c2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        c0.record()
        s_up.wait_event(c0)
        s_down.wait_event(c0)
        for _ in range(4):
            with torch.cuda.stream(s_up):
                dA[:n].copy_(hA_t[:n], non_blocking=True)
            with torch.cuda.stream(s_down):
                hC_t[:n].copy_(dC[:n], non_blocking=True)
        c1.record(s_up)
        c2.record(s_down)
        torch.cuda.synchronize()
        return 2 * 4 * n * 4 / (max(c0.elapsed_time(c1), c0.elapsed_time(c2)) * 1e-3) / 1e9

    pcie_duplex_gbs = duplex_gbs()

    submit_cpu_ms = []  # host time spent inside submit (it includes waiting for the slot of the job two steps back)

    def timed(fn, steps):
        barrier()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        fn(steps)
        b1.record()  # the host blocked until the last result was in host memory: the events bracket the whole loop
        barrier()
        t = torch.tensor([b0.elapsed_time(b1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() / steps

    if G == 1:
        def e2e_step():
            # one blocking call of the C ABI with HOST buffers: upload, GEMM and download overlapped inside the library
            sg.gemm_host(lc, la, lb, hC_t, hA_t, hB_t, M, Nl, K)

        def e2e_stream(steps):
            # the same call split into submit / wait, two jobs in flight: step i+1 is submitted before the result of
            # step i is awaited, so its uploads overlap the compute-bound tail and the downloads of step i.  Every
            # step uploads its A and B from pinned host memory and downloads its C (alternating host buffers).
            pending = []
            for i in range(steps):
                t0 = time.perf_counter()
                pending.append(sg.gemm_host_submit(lc, la, lb, hC_t if i % 2 == 0 else hC2_t, hA_t, hB_t, M, Nl, K))
                submit_cpu_ms.append((time.perf_counter() - t0) * 1e3)
                if len(pending) > 1:
                    sg.gemm_host_wait(pending.pop(0))
            for t in pending:
                sg.gemm_host_wait(t)

        for _ in range(2):
            e2e_step()
        e2e_stream(2)
        if w["init"] == "identity":
            if not (torch.equal(hC_t.view(torch.int32), hA_t.view(torch.int32))
                    and torch.equal(hC2_t.view(torch.int32), hA_t.view(torch.int32))):
                raise SystemExit("host-buffer entry: identity-multiply result differs from A")
        blocking_ms = timed(lambda n: [e2e_step() for _ in range(n)], max(3, e2e_steps // 2))
        e2e_ms = timed(e2e_stream, e2e_steps)
        h2d, d2h = (hA_t.numel() + hB_t.numel()) * 4, hC_t.numel() * 4
        mode = "b200_sgemm_host_submit / _wait, two steps in flight (every step uploads A, B and downloads C)"
        extra = {"blocking_call_ms": blocking_ms, "blocking_call_tflops": flops_total / (blocking_ms * 1e-3) / 1e12,
                 "submit_cpu_ms_median": statistics.median(submit_cpu_ms[-e2e_steps:])}
    else:
        # column-sharded job from host memory: each rank uploads 1/G of the replicated A and its own B slice, the
        # ranks all-gather A over NVLink, multiply, and download their C block; two steps in flight
        pipe = sharded.ShardedHostGemm(sg, lc, la, lb, M, N, K, G, rank)

        def e2e_stream(steps):
            for i in range(steps):
                pipe.submit(hC_t if i % 2 == 0 else hC2_t, hA_t, hB_t)
            pipe.wait_all()

        e2e_stream(2)
        # the pipeline's result must be the device-resident result bit for bit
        if not (torch.equal(hC_t.to(dev).view(torch.int32), dC.view(torch.int32))
                and torch.equal(hC2_t.to(dev).view(torch.int32), dC.view(torch.int32))):
            raise SystemExit("sharded host pipeline: result differs from the device-resident product")
        e2e_ms = timed(e2e_stream, e2e_steps)
        h2d, d2h = pipe.h2d_bytes * G, pipe.d2h_bytes * G
        mode = ("sharded.ShardedHostGemm: per rank upload of 1/G of A and of its B slice, NCCL all-gather of A over "
                "NVLink, b200_sgemm, download of the C block; two steps in flight")
        extra = {"allgather_of_a_bytes_per_rank": (G - 1) * pipe.a_len * 4}
        del pipe
    e2e = {"value": flops_total / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
           "steps": e2e_steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "mode": mode,
           "pcie_h2d_gbs": pcie_h2d_gbs, "pcie_d2h_gbs": pcie_d2h_gbs, "pcie_both_directions_gbs": pcie_duplex_gbs,
           "upload_bound_ms": h2d / G / (pcie_h2d_gbs * 1e9) * 1e3,
           "link_bound_ms": (h2d + d2h) / G / (pcie_duplex_gbs * 1e9) * 1e3}
    e2e.update(extra)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (FP32 FMA pipe) --------------------------------------------
    prop = torch.cuda.get_device_properties(local)
    sm_max = (clocks or {}).get("sm_max_mhz") or 1965.0
    peak_nominal = prop.multi_processor_count * FP32_LANES_PER_SM * 2 * sm_max * 1e6 / 1e12
    probe = max(sg.fma_peak(1, 8192)["tflops"] for _ in range(2))
    achieved = flops_rank / (avg_ms * 1e-3) / 1e12
    roofline = {"bound": "fp32_fma", "achieved": achieved, "peak": peak_nominal, "unit": "TFLOP/s",
                "frac": achieved / peak_nominal,
                "peak_source": f"nominal: {prop.multi_processor_count} SMs x 128 FP32 lanes x 2 x {sm_max:.0f} MHz "
                               "(clocks.max.sm); MEASURED_PEAKS.json has no FP32 non-tensor entry",
                "peak_measured_fma_probe": probe, "frac_of_measured_probe": achieved / probe,
                "achieved_at_min_time": flops_rank / (min_ms * 1e-3) / 1e12,
                # DRAM traffic is a profiler counter: this run does not measure it
                "traffic": None, "traffic_unit": "bytes per launch",
                "algorithmic_flops_per_launch": flops_rank,
                "algorithmic_bytes_per_launch": 4.0 * (M * K + K * Nl + M * Nl),
                "achieved_hbm_gbs": 4.0 * (M * K + K * Nl + M * Nl) / (avg_ms * 1e-3) / 1e9}

    _, cpu_info = cpu_reference_run(w, target_seconds=12.0)

    # ---- optional comparison column: the same problem on the tensor cores (3xTF32, not the graded arithmetic) ----
    tf32x3 = None
    if G == 1:
        for _ in range(3):
            sg.gemm_3xtf32(lc, la, lb, dC, dA, dB, M, Nl, K, stream=stream)
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        for _ in range(10):
            sg.gemm_3xtf32(lc, la, lb, dC, dA, dB, M, Nl, K, stream=stream)
        q1.record()
        q1.synchronize()
        t_ms = q0.elapsed_time(q1) / 10
        rows = slice(0, 256)
        a2 = dA.view(M, K) if la == 0 else dA.view(K, M).T
        b2 = dB.view(K, Nl) if lb == 0 else dB.view(Nl, K).T
        c2 = dC.view(M, Nl) if lc == 0 else dC.view(Nl, M).T
        ref = a2[rows].double() @ b2.double()
        rms = ref.pow(2).mean().sqrt()
        err = ((c2[rows].double() - ref).abs() / torch.maximum(ref.abs(), rms)).max().item()
        tf32x3 = {"tflops": flops_rank / (t_ms * 1e-3) / 1e12, "ms": t_ms, "max_rel_err_vs_f64_256_rows": err,
                  "status": sg.tf32x3_device_status(),
                  "note": "b200_sgemm_3xtf32: tcgen05 tensor-core path, FP32 split into two TF32 halves; "
                          "informational, not part of value/e2e"}

    # ---- every layout permutation of the 4096^3 configuration, outside `value` -----------------------------
    all_layouts = None
    if G == 1 and not args.no_layouts:
        Q = 4096
        xa = torch.rand(Q * Q, dtype=torch.float32, device=dev) * 2 - 1
        xb = torch.rand(Q * Q, dtype=torch.float32, device=dev) * 2 - 1
        xc = torch.empty(Q * Q, dtype=torch.float32, device=dev)
        fl, rows_l, worst = 2.0 * Q ** 3, {}, None
        for qa in (0, 1):
            for qb in (0, 1):
                for qc in (0, 1):
                    for _ in range(10):
                        sg.gemm(qc, qa, qb, xc, xa, xb, Q, Q, Q, stream=stream)
                    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(100)]
                    for e0, e1 in evs:
                        e0.record()
                        sg.gemm(qc, qa, qb, xc, xa, xb, Q, Q, Q, stream=stream)
                        e1.record()
                    torch.cuda.synchronize()
                    ms = [e0.elapsed_time(e1) for e0, e1 in evs]
                    launches_total += 110 * kernels_per_call(sg.select_config(Q, Q, Q, qc, qa, qb)[0])
                    # a band of rows against a float64 product on the device (relative to max(|ref|, rms(ref)))
                    a2 = xa.view(Q, Q) if qa == 0 else xa.view(Q, Q).T
                    b2 = xb.view(Q, Q) if qb == 0 else xb.view(Q, Q).T
                    c2 = xc.view(Q, Q) if qc == 0 else xc.view(Q, Q).T
                    ref = a2[:128].double() @ b2.double()
                    err = ((c2[:128].double() - ref).abs() / torch.maximum(ref.abs(), ref.pow(2).mean().sqrt())).max().item()
                    avg = fl / (statistics.mean(ms) * 1e-3) / 1e12
                    rows_l["".join("rc"[x] for x in (qa, qb, qc))] = {
                        "tflops_avg": avg, "tflops_median_time": fl / (statistics.median(ms) * 1e-3) / 1e12,
                        "tflops_min_time": fl / (min(ms) * 1e-3) / 1e12,
                        "pct_of_fp32_peak": 100.0 * avg / peak_nominal, "max_rel_err_vs_f64_128_rows": err}
                    worst = avg if worst is None else min(worst, avg)
        all_layouts = {"shape": "4096x4096x4096", "layouts_abc": rows_l, "min_tflops_avg": worst,
                       "min_pct_of_fp32_peak": 100.0 * worst / peak_nominal,
                       "tolerance_rel_err": 1e-5 * math.sqrt(Q),
                       "note": "b200_sgemm per layout (A,B,C), A,B~U[-1,1) generated on the device, 10 warm-ups + 100 "
                               "launches timed one by one with CUDA events; informational, not part of value"}
        del xa, xb, xc

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": G, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if G > 1 else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "desc": w["desc"], "M": M, "N": N, "K": K,
                       "layout_abc": "".join("rc"[x] for x in (la, lb, lc)),
                       "sharding": f"N-column blocks of C over {G} rank(s), {Nl} columns each",
                       "kernel": params.__dict__, "variant": variant,
                       "l2": "operands + result (%.0f MB per rank) exceed the 126 MB L2; no explicit flush"
                             % (4.0 * (M * K + K * Nl + M * Nl) / 1e6)},
            "tflops_avg": flops_total / (avg_ms * 1e-3) / 1e12, "tflops_min_time": flops_total / (min_ms * 1e-3) / 1e12,
            # (on some hosts about one launch per second, of any kernel, takes 2 to 3 ms longer: max shows it)
            "launch_ms": {"min": min_ms, "median": median_ms, "avg": avg_ms, "max": max_ms},
            "identity_bit_exact": check, "allgather_ms": allgather_ms,
            "roofline": roofline, "cpu_baseline": cpu_info, "clocks": clocks, "e2e": e2e,
            "tf32x3": tf32x3, "fused_gather": fused, "all_layouts": all_layouts,
            "single_gpu_same_workload_tflops": single_gpu["tflops"] if single_gpu else None,
            "single_gpu_same_workload_ms": single_gpu["ms_per_step"] if single_gpu else None,
            "speedup_vs_single_gpu": value / single_gpu["tflops"] if single_gpu else None,
            "gpu_launches": args.steps * launches_per_step}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="")
    ap.add_argument("--no-layouts", action="store_true", help="skip the all-layouts table of the 1-GPU run")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    w = parse_workload(args.workload, args.gpus)
    if args.impl == "reference":
        reference_arm(args, w)
    else:
        if args.warmup < 3:
            args.warmup = 3
        ours(args, w)


if __name__ == "__main__":
    main()
