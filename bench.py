#!/usr/bin/env python
"""Benchmark of the LUT-GEMM hot path (forward + both gradient-table gathers).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--bits 8] [--size 4096]

One "step" is one forward plus one backward (gW then gA) LUT-GEMM over a batch of synthetic codes:
M = K = N = --size (default 4096) at --bits (default 8), tables built like the benchmark's synthetic
multiplier (max(0, x*y + e), window-difference gradients, wire format uint16 / int16 x16).
Work unit: one LUT-MAC = one (m,k,n) gather-and-accumulate; a step is 3*M*K*N of them.
With N > 1 ranks (torchrun) every rank runs its own M-shard of the same size (weak scaling over the
batch dimension) and the weight gradient is summed across ranks with one NCCL all-reduce per step.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "appmult-aware-retraining_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
LSU_LOOKUPS_PER_CLK_PER_SM = 32


# ------------------------------------------------------------------------------------------------
# synthetic tables / inputs (definition shared with the tests through the benchmark's own formulae)
# ------------------------------------------------------------------------------------------------
def synthetic_wire_tables(bits: int, seed: int = 0):
    """L[x][y] = max(0, x*y + e), e ~ U{-2^(b-1)..2^(b-1)}; gradients = clipped window difference with
    half window 2^b/16; returned in the wire format (uint16, int16 = round(16*g)) as dense arrays."""
    q = 1 << bits
    h = max(1, q // 16)
    rng = np.random.default_rng(seed)
    e = rng.integers(-(q // 2), q // 2 + 1, size=(q, q))
    x = np.arange(q)
    L = np.maximum(0, x[:, None] * x[None, :] + e).astype(np.int64)
    hi, lo = np.minimum(x + h, q - 1), np.maximum(x - h, 0)
    ga = (L[hi, :] - L[lo, :]) / (hi - lo)[:, None]
    gb = (L[:, hi] - L[:, lo]) / (hi - lo)[None, :]
    return L, np.round(ga * 16).astype(np.int64), np.round(gb * 16).astype(np.int64)


def pack_wire(dense, bits, dtype):
    q = 1 << bits
    row, col = q + 1, q + 2
    pad = {4: 718, 6: 830, 7: 638, 8: 0}[bits]
    flat = np.zeros(row * col + pad, dtype)
    flat[: row * col].reshape(row, col)[:q, :q] = dense
    return flat


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=self.out, stderr=subprocess.DEVNULL)
        except (OSError, FileNotFoundError):
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, smmax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1])); smmax.append(float(parts[2]))
                except ValueError:
                    continue
                for nm, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smmax)), "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "sm_max_mhz": 1965.0}, "fallback"


# ------------------------------------------------------------------------------------------------
# reference arm / cpu baseline: the oracle port on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_port_rate(bits, K, N, lf, la, lw, w, target_seconds=12.0, rows_cap=4096, seed=0):
    """G LUT-MAC/s of the C/OpenMP oracle port for forward + backward on a bounded row sample of the
    same problem (same K, N and weight codes; `rows` activation rows)."""
    from oracle import OracleC
    oc = OracleC()
    # all the host threads this process may use: launchers such as torchrun export OMP_NUM_THREADS=1
    try:
        oc.set_num_threads(len(os.sched_getaffinity(0)))
    except AttributeError:
        oc.set_num_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(seed)
    q = 1 << bits

    def run(rows):
        a = rng.integers(0, q, (rows, K)).astype(np.uint8)
        gc = rng.standard_normal((rows, N)).astype(np.float32)
        t0 = time.perf_counter()
        oc.forward(a, w, lf, bits)
        oc.backward(gc, a, w, la, lw, bits)
        return time.perf_counter() - t0

    probe_rows = 16
    t_probe = run(probe_rows)
    rows = int(min(rows_cap, max(probe_rows, probe_rows * target_seconds / max(t_probe, 1e-6))))
    t = run(rows)
    return 3.0 * rows * K * N / t / 1e9, oc.num_threads(), rows, t


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    bits, S = args.bits, args.size
    L, qa, qb = synthetic_wire_tables(bits, 0)
    lf, la, lw = pack_wire(L, bits, np.uint16), pack_wire(qa, bits, np.int16), pack_wire(qb, bits, np.int16)
    rng = np.random.default_rng(1)
    w = rng.integers(0, 1 << bits, (S, S)).astype(np.uint8)
    per_step_seconds = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    rates, rows, cores, tsum = [], 0, 1, 0.0
    for i in range(args.warmup + args.steps):
        r, cores, rows, t = cpu_port_rate(bits, S, S, lf, la, lw, w, target_seconds=per_step_seconds, rows_cap=S, seed=i)
        if i >= args.warmup:
            rates.append(r); tsum += t
    value = float(np.mean(rates))
    line = {
        "impl": "reference", "metric": "lut_gemm_fwd_bwd_throughput", "value": value, "unit": "G LUT-MAC/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * tsum / max(1, args.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16 table -> u32 / f32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"lutgemm fwd+bwd {bits}-bit M=K=N={S}", "bits": bits, "M": S, "K": S, "N": S},
        "cpu_baseline": {"value": value, "unit": "G LUT-MAC/s", "cores": cores, "kind": "port",
                         "sample": f"{rows} of {S} activation rows per step, full K and N, fwd+bwd (C/OpenMP port of "
                                   "the reference gather semantics; the reference has no CPU implementation)"},
        "e2e": {"value": value, "unit": "G LUT-MAC/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# checker legs of our arm: sampled parity gate against the C oracle, the reference's CUDA kernels beside ours
# ------------------------------------------------------------------------------------------------
def parity_gate(bits, s, lf, la, lw, nsample=16):
    """Compares sampled rows and columns of one step's three results with the C oracle: forward bit-exact,
    gradients within 1e-5 of the sum of the absolute terms of each element.  Returns a dict for the JSON line;
    raises on a mismatch (nothing is timed on wrong results)."""
    from oracle import OracleC
    oc = OracleC()
    try:
        oc.set_num_threads(len(os.sched_getaffinity(0)))
    except AttributeError:
        oc.set_num_threads(os.cpu_count() or 1)
    a, w, gc = s["a"].cpu().numpy(), s["w"].cpu().numpy(), s["gc"].cpu().numpy()
    c, ga, gw = s["c"].cpu().numpy(), s["ga"].cpu().numpy(), s["gw"].cpu().numpy()
    lf_n, la_n, lw_n = lf.cpu().numpy(), la.cpu().numpy(), lw.cpu().numpy()
    M, K = a.shape
    N = w.shape[1]
    pick = lambda n: np.unique(np.linspace(0, n - 1, min(nsample, n)).astype(np.int64))
    ms, ks, ns = pick(M), pick(K), pick(N)
    checked = 0

    def close(got, ref, refabs, what):
        nonlocal checked
        bad = np.abs(got - ref) > 1e-5 * refabs + 1e-30
        if bad.any() or not np.isfinite(got).all():
            raise SystemExit(f"parity gate failed: {what}: {int(bad.sum())} of {bad.size} sampled entries off")
        checked += got.size

    # forward: sampled rows and sampled columns, bit-exact
    for got, ref, what in ((c[ms], oc.forward(a[ms], w, lf_n, bits), "forward rows"),
                           (c[:, ns], oc.forward(a, w[:, ns], lf_n, bits), "forward columns")):
        if not np.array_equal(got, ref):
            raise SystemExit(f"parity gate failed: {what} differ from the oracle")
        checked += got.size
    # grad_a rows (their sum over n is complete for a row subset)
    r_ga, _, r_gaa, _ = oc.backward_f64(gc[ms], a[ms], w, la_n, lw_n, bits)
    close(ga[ms], r_ga, r_gaa, "grad_a rows")
    # a k subset gives grad_a columns and grad_w rows, both complete sums
    r_ga, r_gw, r_gaa, r_gwa = oc.backward_f64(gc, a[:, ks], w[ks], la_n, lw_n, bits)
    close(ga[:, ks], r_ga, r_gaa, "grad_a columns")
    close(gw[ks], r_gw, r_gwa, "grad_w rows")
    # an n subset gives grad_w columns
    _, r_gw, _, r_gwa = oc.backward_f64(gc[:, ns], a, w[:, ns], la_n, lw_n, bits)
    close(gw[:, ns], r_gw, r_gwa, "grad_w columns")
    return {"status": "ok", "entries_checked": int(checked),
            "what": f"{len(ms)} rows and {len(ns)} columns of c (bit-exact), {len(ms)} rows / {len(ks)} columns of grad_a, "
                    f"{len(ks)} rows / {len(ns)} columns of grad_w (1e-5 of the sum of absolute terms) against the C oracle"}


def reference_cuda_leg(bits, s, lf, la, lw, reps=2):
    """The reference's own CUDA kernels (built unmodified for sm_100a into oracle/_ref by
    oracle/build_reference_ext.py) timed on the same inputs in this process, and their results compared with
    ours.  Checker leg: returns a dict for the JSON line, or why it is unavailable."""
    import glob
    import importlib.util
    import torch
    hits = glob.glob(os.path.join(ROOT, "oracle", "_ref", f"approx_ops_ref{bits}*.so"))
    if not hits:
        return {"unavailable": f"oracle/_ref/approx_ops_ref{bits} is not built (the reference fixes the bit-width at "
                               "compile time; modules exist for 7 and 8 bits where a reference checkout was at hand)"}
    try:
        spec = importlib.util.spec_from_file_location(f"approx_ops_ref{bits}", hits[0])
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
    except Exception as e:  # e.g. built against another PyTorch
        return {"unavailable": f"could not load {os.path.basename(hits[0])}: {e}"}
    a, w, gc = s["a"], s["w"], s["gc"]
    c = torch.zeros_like(s["c"])
    ga, gw = torch.zeros_like(s["ga"]), torch.zeros_like(s["gw"])
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    ref.approx_gemm_forward(a, w, c, lf)  # warm-up
    ref.approx_gemm_backward(gc, a, w, ga, gw, la, lw)
    torch.cuda.synchronize()
    fwd_ms = bwd_ms = 0.0
    for _ in range(reps):
        ev[0].record()
        ref.approx_gemm_forward(a, w, c, lf)
        ev[1].record()
        ref.approx_gemm_backward(gc, a, w, ga, gw, la, lw)
        ev[2].record()
        torch.cuda.synchronize()
        fwd_ms += ev[0].elapsed_time(ev[1]) / reps
        bwd_ms += ev[1].elapsed_time(ev[2]) / reps
    M, K = a.shape
    N = w.shape[1]
    out = {"kind": "the reference's unmodified kernels compiled for sm_100a (legacy default stream, texture gathers at 8 bits)",
           "forward_ms": fwd_ms, "backward_ms": bwd_ms, "ms_per_step": fwd_ms + bwd_ms,
           "value": 3.0 * M * K * N / ((fwd_ms + bwd_ms) * 1e-3) / 1e9, "unit": "G LUT-MAC/s", "reps": reps}
    # at 8 bits the reference adds LUT[0][0] per padded k when K is not a multiple of 8; otherwise results agree
    if bits < 8 or K % 8 == 0:
        out["forward_equal_to_ours"] = bool(torch.equal(c.view(torch.int32), s["c"].view(torch.int32)))
        for name, r, o in (("grad_a", ga, s["ga"]), ("grad_w", gw, s["gw"])):
            out[f"{name}_max_rel_diff_to_ours"] = float((r - o).abs().max() / r.abs().max().clamp_min(1e-30))
    return out


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import approx_ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device for --impl ours (there is no CPU fallback)")
    lib = approx_ops.library()
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)

    bits, S = args.bits, args.size
    K = N = S
    # weak scaling (default): every rank its own S rows; --shard-m: the S rows of one problem cut across the ranks
    M = (S + world - 1) // world if args.shard_m else S
    L, qa, qb = synthetic_wire_tables(bits, 0)
    lf = torch.from_numpy(pack_wire(L, bits, np.uint16)).to(dev)
    la = torch.from_numpy(pack_wire(qa, bits, np.int16)).to(dev)
    lw = torch.from_numpy(pack_wire(qb, bits, np.int16)).to(dev)

    # Two rotating input/output sets: a step touches ~3x the L2 capacity, and consecutive steps use
    # different buffers, so no operand of a step is L2-resident from the step before.
    nsets = 2
    g = torch.Generator(device="cpu").manual_seed(1000 + rank)
    w_host = torch.from_numpy(np.random.default_rng(1).integers(0, 1 << bits, (K, N)).astype(np.uint8))
    sets = []
    for s in range(nsets):
        a_h = torch.randint(0, 1 << bits, (M, K), generator=g, dtype=torch.uint8).pin_memory()
        gc_h = torch.randn(M, N, generator=g).pin_memory()
        sets.append({
            "a_h": a_h, "gc_h": gc_h, "w_h": w_host.clone().pin_memory(),
            "a": a_h.to(dev), "w": w_host.to(dev), "gc": gc_h.to(dev),
            "c": torch.empty(M, N, dtype=torch.uint32, device=dev),
            "ga": torch.empty(M, K, dtype=torch.float32, device=dev),
            "gw": torch.empty(K, N, dtype=torch.float32, device=dev),
        })
    scratch_bytes = lib.lutgemm_backward_scratch_bytes(bits, M, K, N)
    scratch = torch.empty(max(1, scratch_bytes), dtype=torch.uint8, device=dev)
    fwd_ws_bytes = lib.lutgemm_forward_scratch_bytes(bits, M, K, N)  # transposed activation codes
    fwd_ws = torch.empty(max(1, fwd_ws_bytes), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)

    def fwd(s):
        rc = lib.lutgemm_forward_ws(s["a"].data_ptr(), s["w"].data_ptr(), s["c"].data_ptr(), lf.data_ptr(), bits, M, K, N,
                                    fwd_ws.data_ptr() if fwd_ws_bytes else None, fwd_ws_bytes, stream.cuda_stream)
        assert rc == 0, lib.lutgemm_status_string(rc)

    def bwd_gw(s):
        # the forward pass of the same step left the transposed activation codes in its workspace
        rc = lib.lutgemm_backward_ws(s["gc"].data_ptr(), s["a"].data_ptr(), s["w"].data_ptr(), None, s["gw"].data_ptr(),
                                     None, lw.data_ptr(), bits, M, K, N, fwd_ws.data_ptr() if fwd_ws_bytes else None,
                                     scratch.data_ptr(), scratch_bytes, stream.cuda_stream)
        assert rc == 0, lib.lutgemm_status_string(rc)

    def bwd_ga(s):
        rc = lib.lutgemm_backward(s["gc"].data_ptr(), s["a"].data_ptr(), s["w"].data_ptr(), s["ga"].data_ptr(), None,
                                  la.data_ptr(), None, bits, M, K, N, scratch.data_ptr(), scratch_bytes, stream.cuda_stream)
        assert rc == 0, lib.lutgemm_status_string(rc)

    def step(i, evs=None, exchange=True):
        s = sets[i % nsets]
        if evs: evs[0].record()
        fwd(s)
        if evs: evs[1].record()
        bwd_gw(s)
        if evs: evs[2].record()
        work = dist.all_reduce(s["gw"], async_op=True) if world > 1 and exchange else None  # overlaps the grad_a kernel
        bwd_ga(s)
        if work is not None:
            work.wait()
        if evs: evs[3].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # parity gate before anything is timed: one step's results, sampled, against the C oracle (rank 0)
    # (this one step skips the grad_w all-reduce on every rank: the oracle knows this rank's shard only)
    gate = None
    step(0, exchange=False)
    torch.cuda.synchronize()
    if rank == 0 and not args.no_parity_gate:
        gate = parity_gate(bits, sets[0], lf, la, lw)
    for i in range(args.warmup):
        step(i)
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches_before = lib.lutgemm_kernel_launches()
    t_begin.record()
    for i in range(args.steps):
        step(i, evs[i])
    t_end.record()
    launches = lib.lutgemm_kernel_launches() - launches_before  # counted by the library, not estimated
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_begin.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    k_ms = np.array([[e[j].elapsed_time(e[j + 1]) for j in range(3)] for e in evs])  # fwd, gw(+allreduce), ga
    kern_ms = k_ms.mean(axis=0)

    # ---- end-to-end through the reference-facing ops with host buffers --------------------------
    # Every step copies its inputs from pinned host memory and its three results back, all inside the timed
    # region.  The copies run on two side streams (one per PCIe direction) and are double-buffered against
    # the kernels, as a training loop would overlap its data movement: step i+1's inputs arrive and step
    # i-1's results leave while step i computes.
    e2e_steps = max(2, min(args.steps, 6))
    out_h = {k: torch.empty(sets[0][k].shape, dtype=sets[0][k].dtype).pin_memory() for k in ("c", "ga", "gw")}
    in_d = [{k: torch.empty_like(sets[0][k]) for k in ("a", "w", "gc")} for _ in range(2)]
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]     # inputs of the slot have arrived
    ev_done = [torch.cuda.Event() for _ in range(2)]   # kernels of the slot have finished
    ev_out = [torch.cuda.Event() for _ in range(2)]    # results of the slot have left

    def issue_inputs(i):
        slot, src = i % 2, sets[i % nsets]
        s_in.wait_event(ev_done[slot])  # the kernels that read this slot two steps ago are done
        with torch.cuda.stream(s_in):
            for k in ("a", "w", "gc"):
                in_d[slot][k].copy_(src[k + "_h"], non_blocking=True)
            ev_in[slot].record(s_in)

    def e2e_run(nsteps):
        s_in.wait_stream(main)  # nothing of this run starts before the start event
        s_out.wait_stream(main)
        issue_inputs(0)
        for i in range(nsteps):
            slot, s = i % 2, sets[i % nsets]
            if i + 1 < nsteps:
                issue_inputs(i + 1)
            main.wait_event(ev_in[slot])
            main.wait_event(ev_out[slot])  # the results written two steps ago have left the output buffers
            approx_ops.approx_gemm_forward(in_d[slot]["a"], in_d[slot]["w"], s["c"], lf)
            approx_ops.approx_gemm_backward(in_d[slot]["gc"], in_d[slot]["a"], in_d[slot]["w"], s["ga"], s["gw"], la, lw)
            if world > 1:
                dist.all_reduce(s["gw"])
            ev_done[slot].record(main)
            s_out.wait_event(ev_done[slot])
            with torch.cuda.stream(s_out):
                for k in ("c", "ga", "gw"):
                    out_h[k].copy_(s[k], non_blocking=True)
                ev_out[slot].record(s_out)
        main.wait_stream(s_out)

    assert nsets == 2, "the output buffers are reused with the same period as the input slots"
    e2e_run(2)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    h2d = M * K + K * N + 4 * M * N
    d2h = 4 * M * N + 4 * M * K + 4 * K * N

    if rank != 0:
        return None

    macs_step = 3.0 * M * K * N
    value = world * macs_step * args.steps / (total_ms * 1e-3) / 1e9
    e2e_value = world * macs_step * e2e_steps / (e2e_ms * 1e-3) / 1e9

    peaks, peaks_kind = measured_peaks()
    props = torch.cuda.get_device_properties(dev)
    sms = props.multi_processor_count
    clk_max = float(peaks.get("sm_max_mhz") or (clocks or {}).get("sm_max_mhz") or 1965.0)
    clk_seen = (clocks or {}).get("sm_mhz") or clk_max
    peak_lookups = sms * clk_max * 1e6 * LSU_LOOKUPS_PER_CLK_PER_SM
    names = ["forward", "grad_w", "grad_a"]
    dom = int(np.argmax(kern_ms))
    dom_rate = M * K * N / (kern_ms[dom] * 1e-3)
    alg_bytes = [M * K + K * N + 4 * M * N, 4 * M * N + M * K + K * N + 4 * K * N, 4 * M * N + M * K + K * N + 4 * M * K]
    traffic, traffic_source = ncu_dram_traffic(names[dom], (bits, S, M))
    roofline = {
        "bound": "smem_lsu", "kernel": names[dom], "achieved": dom_rate / 1e9, "peak": peak_lookups / 1e9,
        "unit": "G lookups/s", "frac": dom_rate / peak_lookups,
        "peak_def": f"{sms} SMs x {clk_max:.0f} MHz ({peaks_kind} sm_max_mhz) x {LSU_LOOKUPS_PER_CLK_PER_SM} lookups/clk/SM",
        "frac_at_observed_clock": dom_rate / (sms * clk_seen * 1e6 * LSU_LOOKUPS_PER_CLK_PER_SM),
        "step_frac": (macs_step * args.steps / (total_ms * 1e-3)) / peak_lookups,
        "per_kernel_ms": {n: float(t) for n, t in zip(names, kern_ms)},
        "hbm": {"achieved_gbs": alg_bytes[dom] / (kern_ms[dom] * 1e-3) / 1e9, "peak_gbs": peaks["hbm_gbs"],
                "frac": alg_bytes[dom] / (kern_ms[dom] * 1e-3) / 1e9 / peaks["hbm_gbs"], "of": peaks_kind},
        # dram__bytes_read.sum + dram__bytes_write.sum per launch of that kernel: a property of the kernel and the
        # problem size, read from the committed summary of a separate ncu capture (a profiler cannot run inside a
        # timed run); null for configurations that were not captured
        "traffic": traffic, "traffic_source": traffic_source,
        "algorithmic_bytes": alg_bytes[dom],
    }
    ref_cuda = None
    if world == 1 and not args.no_reference_cuda:
        ref_cuda = reference_cuda_leg(bits, sets[0], lf, la, lw)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        lf_n, la_n, lw_n = lf.cpu().numpy(), la.cpu().numpy(), lw.cpu().numpy()
        rate, cores, rows, secs = cpu_port_rate(bits, K, N, lf_n, la_n, lw_n, w_host.numpy(), target_seconds=12.0, rows_cap=M)
        cpu = {"value": rate, "unit": "G LUT-MAC/s", "cores": cores, "kind": "port",
               "sample": f"{rows} of {M} activation rows, full K and N, fwd+bwd, {secs:.1f} s (C/OpenMP port of the "
                         "reference gather semantics; the reference has no CPU implementation)"}

    line = {
        "metric": "lut_gemm_fwd_bwd_throughput", "value": value, "unit": "G LUT-MAC/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if args.shard_m else "weak", "vs_baseline": None,
        "dtype": "u16 table -> u32 (fwd) / f32 (bwd) accumulate",
        "data": "synthetic",
        "config": {"workload": (f"lutgemm fwd+bwd {bits}-bit M=K=N={S}, M sharded over {world} GPUs" if args.shard_m
                                else f"lutgemm fwd+bwd {bits}-bit M=K=N={S} per GPU"), "bits": bits, "M_per_gpu": M, "K": K,
                   "N": N, "parallelism": f"dp{world} (M sharded, NCCL all-reduce of grad_w)" if world > 1 else "single GPU",
                   "l2": f"{nsets} rotating input/output sets; a step touches {(h2d + d2h) / 2**20:.0f} MiB > L2"},
        "roofline": roofline, "cpu_baseline": cpu, "parity_gate": gate, "reference_cuda": ref_cuda,
        "e2e": {"value": e2e_value, "unit": "G LUT-MAC/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "copies": "inside the timed region, double-buffered on two side streams against the kernels"},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    return line


# ------------------------------------------------------------------------------------------------
# ResNet-18 (CIFAR shape) data-parallel training step
# ------------------------------------------------------------------------------------------------
def run_model(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    import approx_ops
    import self_ops
    from lutgemm_models import MODELS, lut_macs_per_image
    from lutgemm_train import build, train_step

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device for --impl ours (there is no CPU fallback)")
    lib = approx_ops.library()
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    bits, batch = args.bits, args.batch
    L, qa, qb = synthetic_wire_tables(bits, 0)
    self_ops.set_lookup_tables(dev, L, qa, qb, bits)
    ctor, image_shape, classes = MODELS[args.workload]
    macs_img = lut_macs_per_image(ctor(classes).to(dev), image_shape)
    model, opt = build(dev, bits, conv_impl=args.conv_impl, use_ste=args.ste, model_name=args.workload)
    from lutgemm_dp import OverlappedGradReducer
    reducer = OverlappedGradReducer(model.parameters())
    g = torch.Generator().manual_seed(100 + rank)
    nsets = 4
    imgs_h = [torch.randn(batch, *image_shape, generator=g).pin_memory() for _ in range(nsets)]
    lbls_h = [torch.randint(0, classes, (batch,), generator=g).pin_memory() for _ in range(nsets)]
    imgs_d = [t.to(dev) for t in imgs_h]
    lbls_d = [t.to(dev) for t in lbls_h]

    def step(x, y):
        return train_step(model, opt, reducer, x, y)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(imgs_d[i % nsets], lbls_d[i % nsets])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches_before = lib.lutgemm_kernel_launches()
    e0.record()
    for i in range(args.steps):
        step(imgs_d[i % nsets], lbls_d[i % nsets])
    e1.record()
    launches = lib.lutgemm_kernel_launches() - launches_before
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = e0.elapsed_time(e1)
    # end to end: images and labels from pinned host memory, loss read back, every step
    e2e_steps = max(1, min(args.steps, 5))
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for i in range(e2e_steps):
        loss = step(imgs_h[i % nsets].to(dev, non_blocking=True), lbls_h[i % nsets].to(dev, non_blocking=True))
        loss_value = float(loss.item())
    e3.record()
    barrier()
    e2e_ms = e2.elapsed_time(e3)
    if world > 1:
        t = torch.tensor([total_ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = float(t[0]), float(t[1])
    err = approx_ops.device_error()
    reducer.close()
    if rank != 0:
        return None
    peaks, peaks_kind = measured_peaks()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    clk_max = float(peaks.get("sm_max_mhz") or 1965.0)
    peak_lookups = sms * clk_max * 1e6 * LSU_LOOKUPS_PER_CLK_PER_SM
    value = world * batch * args.steps / (total_ms * 1e-3)
    macs_step = 3.0 * macs_img * batch
    line = {
        "metric": f"appmult_{args.workload}_train_throughput", "value": value, "unit": "img/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u16 table -> u32 (fwd) / f32 (bwd) accumulate, f32 elsewhere",
        "data": "synthetic",
        "config": {"workload": f"{WORKLOAD_NAMES[args.workload]} AppMult training step, {bits}-bit, batch {batch}/GPU, SGD",
                   "bits": bits, "batch_per_gpu": batch, "conv_impl": args.conv_impl, "ste_backward": bool(args.ste),
                   "lut_macs_per_step_per_gpu": macs_step,
                   "parallelism": (f"dp{world} (batch sharded, bucketed NCCL all-reduce of gradients launched from hooks during backward)"
                                   if world > 1 else "single GPU"),
                   "l2": f"{nsets} rotating batches; activations of a step exceed L2"},
        "roofline": {"bound": "smem_lsu", "kernel": "whole step (LUT kernels + fp32 glue)",
                     "achieved": macs_step * args.steps / (total_ms * 1e-3) / 1e9, "peak": peak_lookups / 1e9,
                     "unit": "G lookups/s", "frac": macs_step * args.steps / (total_ms * 1e-3) / peak_lookups,
                     "peak_def": f"{sms} SMs x {clk_max:.0f} MHz ({peaks_kind} sm_max_mhz) x 32 lookups/clk/SM", "traffic": None},
        "cpu_baseline": None,
        "e2e": {"value": world * batch * e2e_steps / (e2e_ms * 1e-3), "unit": "img/s",
                "h2d_bytes_per_step": batch * (int(np.prod(image_shape)) * 4 + 8), "d2h_bytes_per_step": 4, "steps": e2e_steps,
                "ms_per_step": e2e_ms / e2e_steps, "last_loss": loss_value},
        "gpu_launches": int(launches), "clocks": clocks, "device_error": err,
    }
    return line


# ------------------------------------------------------------------------------------------------
# per-layer timing of the ResNet-18 (CIFAR shape) convolutions through the convolution entry points
# ------------------------------------------------------------------------------------------------
# name, Cin, H = W, Cout, kernel, stride, pad, occurrences in the network
RESNET18_LAYERS = [("stem", 3, 32, 64, 3, 1, 1, 1), ("s1", 64, 32, 64, 3, 1, 1, 4), ("s2a", 64, 32, 128, 3, 2, 1, 1),
                   ("s2", 128, 16, 128, 3, 1, 1, 3), ("s2sc", 64, 32, 128, 1, 2, 0, 1), ("s3a", 128, 16, 256, 3, 2, 1, 1),
                   ("s3", 256, 8, 256, 3, 1, 1, 3), ("s3sc", 128, 16, 256, 1, 2, 0, 1), ("s4a", 256, 8, 512, 3, 2, 1, 1),
                   ("s4", 512, 4, 512, 3, 1, 1, 3), ("s4sc", 256, 8, 512, 1, 2, 0, 1)]


def run_layers(args, local_rank):
    """--workload resnet18_layers: every distinct convolution of the network on its own - forward, grad_w and
    grad_x in ms (CUDA events) and as a fraction of the look-up roofline, plus per-step totals weighted by how
    often the layer occurs.  Each call is timed alone, so grad_w includes the code transposition that a
    training step shares with the forward pass.  The slab kernels' times do not depend on the codes, the broadcast
    kernels' bank conflicts do: --codes clustered draws them as a trained layer has them."""
    import torch

    import approx_ops
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    bits, B = args.bits, args.batch
    L, qa, qb = synthetic_wire_tables(bits, 0)
    lf = torch.from_numpy(pack_wire(L, bits, np.uint16)).to(dev)
    la = torch.from_numpy(pack_wire(qa, bits, np.int16)).to(dev)
    lw = torch.from_numpy(pack_wire(qb, bits, np.int16)).to(dev)
    peaks, peaks_kind = measured_peaks()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    roof = sms * float(peaks.get("sm_max_mhz") or 1965.0) * 1e6 * LSU_LOOKUPS_PER_CLK_PER_SM

    def timeit(fn, reps=3):
        fn(); fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    rows, tot = [], [0.0, 0.0, 0.0]
    for name, cin, hw, cout, k, st, p, cnt in RESNET18_LAYERS:
        if args.codes == "clustered":
            # codes as a trained layer has them: weights normal around the zero point, activations after a ReLU
            q = 1 << bits
            w = torch.randn(cin * k * k, cout, device=dev)
            wm = (torch.round(w / (w.abs().max() / (q / 2 - 1))) + q / 2).clamp(0, q - 1).to(torch.uint8)
            xa = torch.relu(torch.randn(B, cin, hw, hw, device=dev))
            x = torch.round(xa / (xa.max() / (q - 1))).clamp(0, q - 1).to(torch.uint8)
        else:
            x = torch.randint(0, 1 << bits, (B, cin, hw, hw), dtype=torch.uint8, device=dev)
            wm = torch.randint(0, 1 << bits, (cin * k * k, cout), dtype=torch.uint8, device=dev)
        ho = (hw + 2 * p - k) // st + 1
        M, K = B * ho * ho, cin * k * k
        y = torch.empty(M, cout, dtype=torch.uint32, device=dev)
        gy = torch.randn(M, cout, device=dev)
        gx, gw = torch.empty(B, cin, hw, hw, device=dev), torch.empty(K, cout, device=dev)
        tf = timeit(lambda: approx_ops.approx_conv2d_forward(x, wm, y, lf, k, k, st, p, 1))
        tw = timeit(lambda: approx_ops.approx_conv2d_backward(gy, x, wm, None, gw, la, lw, k, k, st, p, 1))
        tx = timeit(lambda: approx_ops.approx_conv2d_backward(gy, x, wm, gx, None, la, lw, k, k, st, p, 1)) if name != "stem" else 0.0
        look = float(M) * K * cout
        frac = lambda t: look / (t * 1e-3) / roof if t > 0 else None
        rows.append({"layer": name, "M": M, "K": K, "N": cout, "count": cnt, "forward_ms": tf, "forward_frac": frac(tf),
                     "grad_w_ms": tw, "grad_w_frac": frac(tw), "grad_x_ms": tx, "grad_x_frac": frac(tx)})
        for i, t in enumerate((tf, tw, tx)):
            tot[i] += t * cnt
    return {"metric": "appmult_resnet18_layer_times", "unit": "ms", "bits": bits, "batch": B, "codes": args.codes, "layers": rows,
            "per_step_ms": {"forward": tot[0], "grad_w": tot[1], "grad_x": tot[2], "sum": sum(tot)},
            "roofline_peak": roof / 1e9, "roofline_unit": "G lookups/s", "peak_of": peaks_kind}


# DRAM traffic of the three main kernels: read at run time from the committed summary of the ncu capture of this
# workload (a profiler cannot run inside a timed run, so the figure is a property of the kernel at that size)
NCU_TRAFFIC_PROFILE = {"config": (8, 4096, 4096), "file": os.path.join("profiles", "slab_kernels_b8_4096.md")}


def ncu_dram_traffic(kernel, config):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of `kernel` ("forward" | "grad_w" | "grad_a") from the
    metric table of the committed ncu summary, or (None, None) for a workload that was not captured."""
    if config != NCU_TRAFFIC_PROFILE["config"]:
        return None, None
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), NCU_TRAFFIC_PROFILE["file"])
    try:
        rows = [[c.strip() for c in line.strip().strip("|").split("|")] for line in open(path) if line.startswith("|")]
        header = next(r for r in rows if r and r[0] == "metric")
        col = next(i for i, c in enumerate(header) if f"({kernel})" in c)
        scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
        total = 0.0
        for name in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
            r = next(r for r in rows if r[0] == name)
            total += float(r[col].replace(",", "")) * scale[r[1]]
        return total, f"ncu --set full capture of one launch of this kernel at this size ({NCU_TRAFFIC_PROFILE['file']})"
    except (OSError, StopIteration, ValueError, KeyError, IndexError):
        return None, None


WORKLOAD_NAMES = {"resnet18": "ResNet-18 CIFAR-shape", "resnet50": "ResNet-50 ImageNet-shape", "vit_s": "ViT-S/16"}
# per-workload defaults of the benchmark configurations: (bits, per-GPU batch)
WORKLOAD_DEFAULTS = {"resnet18": (7, 256), "resnet50": (8, 128), "vit_s": (7, 64), "resnet18_layers": (7, 256)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--bits", type=int, default=8, choices=[4, 6, 7, 8])
    ap.add_argument("--size", type=int, default=4096)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", choices=["lutgemm", "resnet18", "resnet50", "vit_s", "resnet18_layers"], default="lutgemm")
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch of the model workloads")
    ap.add_argument("--conv-impl", choices=["layer", "fused", "unfold"], default="layer")
    ap.add_argument("--shard-m", action="store_true",
                    help="lutgemm workload: cut the M rows of ONE size^3 problem across the ranks (strong scaling)")
    ap.add_argument("--ste", action="store_true", help="model workloads: straight-through backward instead of the gradient tables")
    ap.add_argument("--codes", choices=["uniform", "clustered"], default="uniform",
                    help="resnet18_layers: uniform random codes, or codes distributed like a trained layer's")
    ap.add_argument("--no-parity-gate", action="store_true", help="lutgemm workload: skip the sampled oracle comparison")
    ap.add_argument("--no-reference-cuda", action="store_true",
                    help="lutgemm workload: do not time the reference's own CUDA kernels beside ours")
    ap.add_argument("--no-model", action="store_true",
                    help="lutgemm workload: do not append the ResNet-18 training-step measurement")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    import torch
    import torch.distributed as dist
    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    if args.workload != "lutgemm":
        if "--bits" not in sys.argv:
            args.bits = WORKLOAD_DEFAULTS[args.workload][0]
        if args.batch is None:
            args.batch = WORKLOAD_DEFAULTS[args.workload][1]
        if args.workload == "resnet18_layers":
            line = run_layers(args, local_rank) if rank == 0 else None
        else:
            line = run_model(args, rank, world, local_rank)
    else:
        line = run_ours(args, rank, world, local_rank)
        if not args.no_model and not args.shard_m:
            # the second half of the metric on the same GPUs in the same run: the ResNet-18 (CIFAR shape) AppMult
            # training step of benchmark configuration 1 - 7-bit, batch 256 per GPU, SGD
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            margs = argparse.Namespace(**vars(args))
            margs.workload, margs.bits, margs.batch = "resnet18", WORKLOAD_DEFAULTS["resnet18"][0], WORKLOAD_DEFAULTS["resnet18"][1]
            margs.steps, margs.warmup = max(5, min(args.steps, 20)), 3
            mline = run_model(margs, rank, world, local_rank)
            if line is not None:
                line["resnet18"] = {k: mline[k] for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                                                          "scaling", "config", "roofline", "e2e", "gpu_launches", "clocks")}
    if line is not None:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
