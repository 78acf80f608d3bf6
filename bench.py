#!/usr/bin/env python
"""Benchmark of the KV-cache hot path: streaming decode at 101.6k positions, 16 attention layers, 8 query tokens per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step: for each of the 16 layers, append the step's K / V rows (quantize into the q8_0 ring, spill rows
that left the window into the 5/6-bit tier) and run decode attention of 8 query tokens over the whole context; then 1..8 of
the positions are committed. N > 1 (torchrun): every rank streams its own sequence (independent sequence slots, no
collective). Prints one JSON line (rank 0).

Side modes (not the headline): --split-ctx L (config 2b: one sequence of L positions split by position over the ranks, NCCL
combine), --config 3 (32 sequences dealt to the ranks, whole-job tokens/s), --config 4 (snapshot / restore of 100,000 positions,
GB/s).

--impl reference times the CPU restatement of the reference's kernels (the parity oracle) on the host cores: the reference
engine has no CPU implementation of this path, and its CUDA kernels need its whole model runtime.
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

# Standard output carries the JSON line and nothing else: libraries that write to file descriptor 1 from native code (NCCL prints its
# version banner there) are sent to standard error for the whole run, the line goes to the saved descriptor.
_STDOUT_FD = None


def claim_stdout():
    global _STDOUT_FD
    if _STDOUT_FD is None:
        sys.stdout.flush()
        _STDOUT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(text):
    os.write(1 if _STDOUT_FD is None else _STDOUT_FD, (text + "\n").encode())
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

LAYERS, CTX0, T_STEP, WIN = 16, 101600, 8, 2048
SPEC = "K*=5r,V*=6"
NH, NKV, HD = 24, 4, 256
# dram__bytes_read.sum + dram__bytes_write.sum of one attention launch at this workload's shapes, from an ncu capture of the
# one-layer case of this benchmark (a launch of the 16-layer run processes the same one layer); NCU_TRAFFIC_FROM says which
NCU_TRAFFIC_BYTES = 164.2e6
NCU_TRAFFIC_FROM = "ncu capture of `bench.py --layers 1 --steps 2 --warmup 3 --no-cpu`, kernel attn_tc_kernel<5, 6> (since compiled as the one-job instance attn_tc_kernel<5, 6, false>, same code), one launch"
WORKLOAD = "config2: 16 attention layers, 101,600 positions, preset F layout K5r/V6 + q8_0 window 2048, 8 queries/step, streaming append+spill+attend"
REPEATS = 5  # the timed K-step loop is run this many times; the line's value is the median run


def algorithmic_bytes(n, T, kbits=5, vbits=6, win=WIN):
    """bytes one layer's decode attention must move at context n + T: every visible row's values + scales once (q8_0 rows
    from the window start on), Q in, O out; partials are not counted"""
    L = n + T
    B = 640
    ws = max(0, (L + B - 1) // B - 1 - (win + B - 1) // B) * B
    low = NKV * ((32 * kbits + 16) + (32 * vbits + 16))
    q8 = NKV * 2 * 272
    return ws * low + (L - ws) * q8 + T * NH * HD * 2 + T * NH * HD * 4


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the warm-up and timed steps run"""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                c = [x.strip() for x in line.split(",")]
                if len(c) < 9:
                    continue
                try:
                    sm.append(float(c[1])); mx.append(float(c[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        return out


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def run_reference(args):
    """The CPU arm: the oracle's append + attention, all host threads, rank 0 only. A step is the workload's step: 16 layer passes
    (append + attend of T rows at the same context). The 16 passes run on ONE layer's cache, which every pass streams from DRAM
    again (158 MB, far beyond the CPU's caches), so a step costs what 16 distinct layers cost while the set-up quantizes one."""
    rank, _, _ = dist_env()
    if rank != 0:
        return
    import numpy as np
    import kv_oracle as ko
    import kvdata
    cores = os.cpu_count() or 1
    L = CTX0
    orc = ko.Cache(1, L + 64 * T_STEP + 64, SPEC, WIN)
    for a in range(0, L, 8192):
        K, V = kvdata.kv_rows(2, 0, a, min(8192, L - a))
        orc.append(0, a, K, V)
    n = L
    rng = np.random.default_rng(2)
    times = []
    total = args.warmup + args.steps
    for s in range(total):
        T = ko.att_cap_T(n, T_STEP)
        K, V = kvdata.kv_rows(3, 0, n, T)
        Q = kvdata.q_rows(3, 0, n, T)
        t0 = time.perf_counter()
        for _ in range(LAYERS):
            orc.append(0, n, K, V)
            orc.attend(0, n, Q, threads=cores)
        dt = time.perf_counter() - t0
        if s >= args.warmup:
            times.append(dt)
        n += int(rng.integers(1, T + 1))
    ms_step = 1e3 * sum(times) / len(times)
    us = 1e3 * ms_step / LAYERS
    sample = "%d steps of %d layer passes (append + attend, T=%d, n~%d) by the CPU restatement of the reference's kernels" % (
        len(times), LAYERS, T_STEP, CTX0)
    line = {"impl": "reference", "metric": "decode_attn_us_per_layer", "value": us, "unit": "us/layer", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 operands / f32 accumulate over u8 packed 5/6/8-bit rows", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers": LAYERS, "context": CTX0, "queries": T_STEP, "kv_spec": SPEC, "kv_win": WIN,
                       "mode": "eager dual-write (the reference's own)", "sequences": 1, "parallelism": "host threads over (kv head, chunk) items",
                       "l2": "one layer's cache (158 MB) streamed from DRAM by each of the step's 16 layer passes"},
            "cpu_baseline": {"value": us, "unit": "us/layer", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": us, "unit": "us/layer", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gb_per_s": algorithmic_bytes(CTX0, T_STEP) / us / 1e3}
    emit(json.dumps(line))


def cpu_baseline_sample(seconds=12.0):
    """bounded CPU sample for the cpu_baseline object of our own line"""
    import numpy as np
    import kv_oracle as ko
    import kvdata
    cores = os.cpu_count() or 1
    L = CTX0
    orc = ko.Cache(1, L + 64, SPEC, WIN)
    for a in range(0, L, 8192):
        K, V = kvdata.kv_rows(2, 0, a, min(8192, L - a))
        orc.append(0, a, K, V)
    Q = kvdata.q_rows(3, 0, L - T_STEP, T_STEP)
    orc.attend(0, L - T_STEP, Q, threads=cores)
    times = []
    t_end = time.perf_counter() + seconds
    while time.perf_counter() < t_end or len(times) < 3:
        K, V = kvdata.kv_rows(3, 0, L - T_STEP, T_STEP)
        t0 = time.perf_counter()
        orc.append(0, L - T_STEP, K, V)
        orc.attend(0, L - T_STEP, Q, threads=cores)
        times.append(time.perf_counter() - t0)
    us = 1e6 * sum(times) / len(times)
    return {"value": us, "unit": "us/layer", "cores": cores, "kind": "port",
            "sample": "%d layer-steps of append + attend (T=8, context 101,600) by the CPU restatement of the reference's kernels" % len(times)}


def hbm_peak():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback"


def setup_dist():
    import torch
    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return rank, local_rank, world, dist


def measure_split(args, ctx0, steps, warmup, dist, rank, local_rank, world):
    """Config 2b: ONE sequence of ctx0 positions split by position over the ranks; every step each rank appends the rows it owns and
    attends over its own positions for all layers (one library call), the (max, sum, un-normalised output) partials are all-gathered
    over NCCL once per step and merged on every rank by one launch. Returns the line's extra figures (rank 0) or None."""
    import numpy as np
    import torch
    mk = importlib.import_module("qwen38-megakernel_b200")
    layers = args.layers
    total_steps = warmup + steps + 4
    cap = ctx0 + total_steps * T_STEP + 64
    stream = torch.cuda.current_stream()
    seq = mk.parallel.SplitSequence(mk.Engine, layers, cap, SPEC, WIN, rank, world, dist=dist, spill=not args.eager, stream=stream)
    g = torch.Generator(device="cuda")
    g.manual_seed(100 + rank)
    lo, hi = seq.lo, min(seq.hi, ctx0)
    for l in range(layers):  # every rank fills the positions it owns (timing run: the rows need not match across ranks)
        for a in range(lo, hi, 16384):
            m = min(16384, hi - a)
            K = (torch.randn((m, NKV, HD), generator=g, device="cuda") * 1.3).half()
            V = (torch.randn((m, NKV, HD), generator=g, device="cuda") * 1.3).half()
            seq.eng.append(l, a, K, V)
    g.manual_seed(5)  # the step's rows and queries are replicated: same seed on every rank
    Kd = (torch.randn((layers, T_STEP, NKV, HD), generator=g, device="cuda") * 1.3).half()
    Vd = (torch.randn((layers, T_STEP, NKV, HD), generator=g, device="cuda") * 1.3).half()
    Qd = torch.randn((layers, T_STEP, NH, HD), generator=g, device="cuda").half()
    Od = torch.empty((layers, T_STEP, NH, HD), dtype=torch.float32, device="cuda")
    rng = np.random.default_rng(2)
    state = {"n": ctx0}

    def one_step():
        n = state["n"]
        T = mk.cap_T(n, T_STEP)
        seq.step(n, Kd[:, :T], Vd[:, :T], Qd[:, :T], Od[:, :T])
        state["n"] = n + min(T, int(rng.integers(1, T_STEP + 1)))

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        one_step()
    barrier()
    l0 = seq.eng.launches()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        one_step()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = seq.eng.launches() - l0
    check = float(Od.abs().max())
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    seq.close()
    if rank != 0:
        return None
    peak, _ = hbm_peak()
    us_layer = 1e3 * ms / (layers * steps)
    nbytes = algorithmic_bytes(ctx0, T_STEP)
    return {"us_per_layer": us_layer, "ms_per_step": ms / steps, "context": ctx0, "layers": layers, "steps": steps, "n_gpus": world,
            "hbm_gbs_whole_job": nbytes / (us_layer * 1e-6) / 1e9, "frac_of_measured_peak_per_gpu": nbytes / (us_layer * 1e-6) / 1e9 / peak / world,
            "combine_bytes_per_rank_step": layers * 4 * 48 * 258 * 4, "collectives_per_step": 1 if world > 1 else 0,
            "gpu_launches": int(launches), "output_absmax": check}


def run_split(args):
    """--split-ctx L: config 2b alone, as its own JSON line"""
    rank, local_rank, world, dist = setup_dist()
    importlib.import_module("qwen38-megakernel_b200").load_library()
    sampler = ClockSampler(local_rank)
    sampler.start()
    r = measure_split(args, args.split_ctx, args.steps, args.warmup, dist, rank, local_rank, world)
    clocks = sampler.stop()
    if rank == 0:
        line = {"metric": "decode_attn_us_per_layer", "value": r["us_per_layer"], "unit": "us/layer", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16 operands / f32 accumulate over u8 packed 5/6/8-bit rows", "data": "synthetic",
                "config": {"workload": "config2b: one sequence of %d positions split by position over %d GPUs, %d layers, 8 queries/step, "
                                       "one NCCL all-gather of the (max, sum, output) partials of all layers per step + one merge launch"
                                       % (args.split_ctx, world, args.layers),
                           "layers": args.layers, "context": args.split_ctx, "kv_spec": SPEC, "kv_win": WIN},
                "clocks": clocks}
        line.update({k: v for k, v in r.items() if k not in ("us_per_layer", "ms_per_step")})
        emit(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def measure_config3(args, steps, warmup, dist, rank, local_rank, world):
    """Config 3: 32 independent sequences of log-uniform length [2,000, 100,000], 1..8 tokens each per step, dealt to the GPUs
    longest-first by KV bytes (no collective). A step is one batched launch sequence per layer over the rank's sequences; the figure
    is the whole job's tokens per second."""
    import numpy as np
    import torch
    mk = importlib.import_module("qwen38-megakernel_b200")
    layers, NS = args.layers, 32
    rng = np.random.default_rng(3)
    lens = np.exp(rng.uniform(np.log(2000), np.log(100000), size=NS)).astype(np.int64)
    Ts = rng.integers(1, T_STEP + 1, size=NS)
    mine = mk.parallel.lpt_partition([int(x) for x in lens], world)[rank]
    mine.sort(key=lambda i: -int(lens[i]))  # longest first: their CTAs (one per chunk, 4 x 20 per sequence) start first
    total_steps = warmup + steps + 2
    cap = int(max(lens[i] for i in mine)) + total_steps * T_STEP + 64
    stream = torch.cuda.current_stream()
    eng = mk.Engine(layers, 64, SPEC, WIN, spill=not args.eager, stream=stream)
    eng.slots_open(len(mine), cap)
    eng.reserve_batch(len(mine))
    g = torch.Generator(device="cuda")
    g.manual_seed(300 + rank)
    for si, i in enumerate(mine):
        for l in range(layers):
            for a in range(0, int(lens[i]), 16384):
                m = min(16384, int(lens[i]) - a)
                K = (torch.randn((m, NKV, HD), generator=g, device="cuda") * 1.3).half()
                V = (torch.randn((m, NKV, HD), generator=g, device="cuda") * 1.3).half()
                eng.append(l, a, K, V, seq=si)
    n = [int(lens[i]) for i in mine]
    T = [int(Ts[i]) for i in mine]
    sumT = sum(T)
    K = (torch.randn((layers, sumT, NKV, HD), generator=g, device="cuda") * 1.3).half()
    V = (torch.randn((layers, sumT, NKV, HD), generator=g, device="cuda") * 1.3).half()
    Q = torch.randn((layers, sumT, NH, HD), generator=g, device="cuda").half()
    O = torch.empty((layers, sumT, NH, HD), dtype=torch.float32, device="cuda")
    seqs = list(range(len(mine)))
    state = {"n": n}

    def one_step():
        nn = state["n"]
        Tc = [mk.cap_T(a, t) for a, t in zip(nn, T)]
        for l in range(layers):
            eng.step_batch(seqs, l, nn, Tc, K[l], V[l], Q[l], O[l])
        state["n"] = [a + t for a, t in zip(nn, Tc)]
        return sum(Tc)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        one_step()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    toks = 0
    for _ in range(steps):
        toks += one_step()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    tot = torch.tensor([ms, float(toks)], device="cuda", dtype=torch.float64)
    if dist is not None:
        mx = tot.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm_ = tot.clone(); dist.all_reduce(sm_, op=dist.ReduceOp.SUM)
        ms, toks = float(mx[0]), float(sm_[1])
    eng.close()
    if rank != 0:
        return None
    return {"tokens_per_s": toks / (ms * 1e-3), "ms_per_step": ms / steps, "steps": steps, "n_gpus": world, "layers": layers,
            "positions_total": int(lens.sum()), "tokens_per_step": int(Ts.sum())}


def run_config3(args):
    rank, local_rank, world, dist = setup_dist()
    importlib.import_module("qwen38-megakernel_b200").load_library()
    sampler = ClockSampler(local_rank)
    sampler.start()
    r = measure_config3(args, args.steps, args.warmup, dist, rank, local_rank, world)
    clocks = sampler.stop()
    if rank == 0:
        emit(json.dumps({"metric": "aggregate_decode_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                          "dtype": "f16 operands / f32 accumulate over u8 packed 5/6/8-bit rows", "data": "synthetic",
                          "config": {"workload": "config3: 32 sequences, lengths log-uniform [2,000, 100,000], 1..8 tokens each per step, %d attention "
                                                 "layers (attention + KV append only), dealt to the GPUs longest-first by KV bytes" % args.layers,
                                     "kv_spec": SPEC, "kv_win": WIN, "positions_total": r["positions_total"], "tokens_per_step": r["tokens_per_step"]},
                          "clocks": clocks}))
    if dist is not None:
        dist.destroy_process_group()


def measure_config4(args, runs):
    """Config 4: 100,000 positions x 16 layers parked in pinned host memory, the first 11,700 restored, 2,000 rows appended,
    8 tokens decoded. The figure is the restore rate (GB/s of KV rows brought back, host -> device)."""
    import torch
    mk = importlib.import_module("qwen38-megakernel_b200")
    layers, L, P, A = args.layers, 100000, 11700, 2000
    eng = mk.Engine(layers, L + 64, SPEC, WIN, spill=not args.eager)
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    for l in range(layers):
        for a in range(0, L, 20000):
            K = (torch.randn((20000, NKV, HD), generator=g, device="cuda") * 1.3).half()
            V = (torch.randn((20000, NKV, HD), generator=g, device="cuda") * 1.3).half()
            eng.append(l, a, K, V)
    eng.commit(L)
    eng.store_budget(4 << 30)
    eng.store_reserve(eng.park_need())  # the pinned chunks exist before the timed park
    eng.sync()
    t0 = time.perf_counter()
    pid = eng.park()
    eng.sync()
    t_park = time.perf_counter() - t0
    nbytes = eng.park_bytes(pid)
    row_bytes = layers * NKV * ((32 * 5 + 16) + (32 * 6 + 16))
    rates = []
    for _ in range(runs):
        eng.reset()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.restore_prefix(pid, P, wait=True)
        eng.sync()
        rates.append(P * row_bytes / (time.perf_counter() - t0) / 1e9)
    Kn = (torch.randn((A, NKV, HD), generator=g, device="cuda") * 1.3).half()
    Q = torch.randn((T_STEP, NH, HD), generator=g, device="cuda").half()
    O = torch.empty((T_STEP, NH, HD), dtype=torch.float32, device="cuda")
    t0 = time.perf_counter()
    for l in range(layers):
        eng.append(l, P, Kn, Kn)
    n = P + A - T_STEP
    eng.commit(n)
    for l in range(layers):
        eng.attend(l, n, Q, O)
    eng.sync()
    t_tail = time.perf_counter() - t0
    eng.close()
    return {"restore_gb_per_s": max(rates), "restore_gb_per_s_runs": rates, "park_gb_per_s": nbytes / t_park / 1e9, "parked_gb": nbytes / 1e9,
            "restored_mb": P * row_bytes / 1e6, "reappend_plus_decode_ms": 1e3 * t_tail, "layers": layers,
            "bound": "host link (PCIe, pinned memory)"}


def run_config4(args):
    import torch
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    torch.cuda.set_device(local_rank)
    importlib.import_module("qwen38-megakernel_b200").load_library()
    r = measure_config4(args, max(args.steps, 1) if args.steps < 16 else 5)
    emit(json.dumps({"metric": "kv_restore_gb_per_s", "value": r["restore_gb_per_s"], "unit": "GB/s", "n_gpus": 1, "higher_is_better": True, "vs_baseline": None,
                      "data": "synthetic", "dtype": "u8 packed rows",
                      "config": {"workload": "config4: park 100,000 positions x %d layers (%0.2f GB with the rings), restore positions [0, 11,700) "
                                             "(%0.1f MB of rows), append 2,000 rows, decode 8 tokens" % (r["layers"], r["parked_gb"], r["restored_mb"]),
                                 "kv_spec": SPEC, "kv_win": WIN},
                      "park_gb_per_s": r["park_gb_per_s"], "restore_gb_per_s_runs": r["restore_gb_per_s_runs"],
                      "reappend_plus_decode_ms": r["reappend_plus_decode_ms"], "bound": r["bound"]}))


def reference_kernel_us():
    """The reference's own decode-attention kernel (attn_core_w48m<8>, cut from its source into oracle/_ref by oracle/build_ref.py)
    timed on this GPU at the headline shape: K5r / V6 + window 2048, 101,600 positions, 8 queries, its own 82 x 512 launch, random
    cache bytes as its own harness uses. None when the witness library was not built (no reference tree at build time)."""
    import ctypes as C
    so = os.path.join(ROOT, "oracle", "_ref", "libref_attn_witness.so")
    if not os.path.exists(so):
        return None
    try:
        L = C.CDLL(so)
        L.ref_attn_time.argtypes = [C.c_int] * 7 + [C.c_void_p]
        us = C.c_float(0)
        if L.ref_attn_time(5, 6, 1, WIN, CTX0, T_STEP, 20, C.byref(us)) != 0:
            return None
        return float(us.value)
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--ctx", type=int, default=CTX0)
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--eager", action="store_true", help="dual-write every row at append instead of spilling on eviction")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample, the reference kernel's timing and the side modes")
    ap.add_argument("--split-ctx", type=int, default=0, help="config 2b alone: one sequence of this many positions split over the GPUs")
    ap.add_argument("--config", type=int, default=2, help="2 (default): the headline decode workload; 3: 32 sequences dealt to the GPUs; 4: snapshot / restore")
    args = ap.parse_args()
    claim_stdout()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else max(args.warmup, 1)
    if args.impl == "reference":
        return run_reference(args)
    if args.split_ctx > 0:
        return run_split(args)
    if args.config == 3:
        return run_config3(args)
    if args.config == 4:
        return run_config4(args)

    import numpy as np
    import torch
    rank, local_rank, world, dist = setup_dist()
    mk = importlib.import_module("qwen38-megakernel_b200")
    mk.load_library()  # no fallback: fails here when the CUDA library is missing
    layers, ctx0 = args.layers, args.ctx
    total_steps = args.warmup + (REPEATS + 1) * args.steps + 24
    cap = ctx0 + total_steps * T_STEP + 64
    stream = torch.cuda.current_stream()
    eng = mk.Engine(layers, cap, SPEC, WIN, spill=not args.eager, stream=stream)

    # synthetic cache: N(0,1) x per-channel scale U(0.5, 2), 1 % of channels x 20, seeded per rank and layer
    g = torch.Generator(device="cuda")
    def chscale(layer, side):
        g.manual_seed(1000 * (rank + 1) + 2 * layer + side)
        ch = torch.rand((NKV, HD), generator=g, device="cuda") * 1.5 + 0.5
        out = torch.rand((NKV, HD), generator=g, device="cuda") < 0.01
        return torch.where(out, ch * 20.0, ch)
    scales = [[chscale(l, s) for s in range(2)] for l in range(layers)]
    def rows(layer, n):
        K = (torch.randn((n, NKV, HD), generator=g, device="cuda") * scales[layer][0]).half()
        V = (torch.randn((n, NKV, HD), generator=g, device="cuda") * scales[layer][1]).half()
        return K, V
    g.manual_seed(7 + rank)
    for l in range(layers):
        for a in range(0, ctx0, 16384):
            K, V = rows(l, min(16384, ctx0 - a))
            eng.append(l, a, K, V)
    eng.commit(ctx0)
    eng.sync()

    # per-step inputs, device resident (value) and pinned host (e2e)
    rng = np.random.default_rng(2)
    accepted = rng.integers(1, T_STEP + 1, size=total_steps)
    Kl = [None] * layers; Vl = [None] * layers
    for l in range(layers):
        Kl[l], Vl[l] = rows(l, T_STEP)
    Kd = torch.stack(Kl); Vd = torch.stack(Vl)  # [layers][T][4][256]
    Qd = torch.randn((layers, T_STEP, NH, HD), generator=g, device="cuda").half()
    Od = torch.empty((layers, T_STEP, NH, HD), dtype=torch.float32, device="cuda")
    Kh = Kd.cpu().pin_memory(); Vh = Vd.cpu().pin_memory(); Qh = Qd.cpu().pin_memory()
    Oh = torch.empty((layers, T_STEP, NH, HD), dtype=torch.float32).pin_memory()
    Ks = torch.empty_like(Kd); Vs = torch.empty_like(Vd); Qs = torch.empty_like(Qd)

    state = {"n": ctx0, "i": 0, "bytes": 0}

    def advance(n, T):
        state["bytes"] += layers * algorithmic_bytes(n, T)
        state["n"] = n + min(T, int(accepted[state["i"]]))
        state["i"] += 1
        eng.commit(state["n"])

    def one_step(host=False):
        """one decode step: every layer appends T rows and attends (one library call for the whole step)"""
        n = state["n"]
        T = mk.cap_T(n, T_STEP)
        if host:  # end to end: this step's rows come from pinned host memory, the result goes back (one copy per tensor: cutting the
            # step into blocks of layers whose copies overlap the other blocks' attention measured slower, 114.6 against 109.8 us per
            # layer: a small copy and a cross-stream event cost about 10 us each)
            Ks.copy_(Kh, non_blocking=True); Vs.copy_(Vh, non_blocking=True); Qs.copy_(Qh, non_blocking=True)
            eng.step_layers(n, Ks[:, :T], Vs[:, :T], Qs[:, :T], Od[:, :T])
            Oh.copy_(Od, non_blocking=True)
            stream.synchronize()  # the caller reads the step's result
        else:
            eng.step_layers(n, Kd[:, :T], Vd[:, :T], Qd[:, :T], Od[:, :T])
        advance(n, T)


    def timed_attends(pairs):
        """a step whose attention launches (one per layer, back to back, nothing between them) sit inside one event pair; about 2 ms
        of device time (a spin, no memory traffic) is queued first so that the host is ahead of the device and the pair times device
        work only"""
        n = state["n"]
        T = mk.cap_T(n, T_STEP)
        for l in range(layers):
            eng.append_raw(l, n, T, Kd[l], Vd[l])
        torch.cuda._sleep(4_000_000)  # about 2 ms of device time without memory traffic: the launches below queue up behind it
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for l in range(layers):
            eng.attend(l, n, Qd[l, :T], Od[l, :T])
        e1.record(stream)
        pairs.append((e0, e1))
        advance(n, T)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_steps(host):
        """EXACTLY args.steps steps between a barrier + synchronize on both sides, on the device's clock; max over the ranks"""
        barrier()
        state["bytes"] = 0
        l0 = eng.launches()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            one_step(host)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, eng.launches() - l0, state["bytes"]

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        one_step()
    # --- device-resident timing: REPEATS runs of the K-step loop; the line reports the median run ---
    runs = [timed_steps(False) for _ in range(REPEATS)]
    order = sorted(range(REPEATS), key=lambda i: runs[i][0])
    ms, launches, step_bytes = runs[order[REPEATS // 2]]
    # --- the attention launch alone (dominant kernel + its merge), event pair per launch, same stream ---
    pairs = []
    state["bytes"] = 0
    for _ in range(min(args.steps, 8)):
        timed_attends(pairs)
    torch.cuda.synchronize()
    att_ms = [a.elapsed_time(b) for a, b in pairs]  # (each pair: one launch per layer)
    att_bytes = state["bytes"] / (len(pairs) * layers)
    att_us = 1e3 * sum(att_ms) / (len(att_ms) * layers)
    # --- end to end: host buffers in, host result out, every step ---
    one_step(host=True)
    ms_e2e, _, _ = timed_steps(True)
    clocks = sampler.stop()
    eng.sync()
    if dist is not None:
        t = torch.tensor([att_us], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        att_us = float(t.item())
    eng.close()
    torch.cuda.empty_cache()

    line = None
    if rank == 0:
        peak, peak_src = hbm_peak()
        us_layer = 1e3 * ms / (layers * args.steps)  # per GPU: every rank streams its own sequence, the slowest rank's time
        # the attention launch's duration: the event pair around a step's launches / layers, or, when smaller, the timed steps' time per
        # layer (a step is those launches plus one append launch, so its time per layer bounds the launch from above)
        att_from = "event pair around a step's %d attention launches" % layers
        if us_layer < att_us:
            att_us, att_from = us_layer, "timed steps (time per layer: the attention launch plus 1/%d of the step's append launch)" % layers
        achieved = att_bytes / att_us / 1e3  # GB/s
        full = layers == LAYERS and ctx0 == CTX0
        line = {
            "metric": "decode_attn_us_per_layer", "value": us_layer, "unit": "us/layer", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 operands / f32 accumulate over u8 packed 5/6/8-bit rows", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers": layers, "context": ctx0, "queries": T_STEP, "kv_spec": SPEC, "kv_win": WIN,
                       "mode": "eager dual-write" if args.eager else "spill on eviction (fp16 shadow)", "sequences": world,
                       "parallelism": "independent sequence per GPU, no collective",
                       "l2": "inputs larger than L2: %.0f MB per layer, %.2f GB per step" % (att_bytes / 1e6, att_bytes * layers / 1e9)},
            "value_is": "per-GPU us per layer-step (max over ranks): every GPU streams its own sequence, so the figure stays flat as N grows",
            "aggregate_us_per_layer": us_layer / world,
            "repeats": {"n": REPEATS, "us_per_layer_min": 1e3 * runs[order[0]][0] / (layers * args.steps), "us_per_layer_median": us_layer,
                        "us_per_layer_max": 1e3 * runs[order[-1]][0] / (layers * args.steps)},
            "hbm_gbs_step": step_bytes / (ms * 1e-3) / 1e9 * world,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES if full else None, "traffic_from": NCU_TRAFFIC_FROM if full else None,
                         "kernel": "attn_tc_kernel<5, 6, false> (the one-job instance; merge in its tail)", "us_per_launch": att_us, "us_per_launch_from": att_from, "bytes_per_launch": att_bytes, "peak_source": peak_src},
            "e2e": {"value": 1e3 * ms_e2e / (layers * args.steps), "unit": "us/layer",
                    "h2d_bytes_per_step": int(layers * (2 * T_STEP * NKV * HD * 2 + T_STEP * NH * HD * 2)),
                    "d2h_bytes_per_step": int(layers * T_STEP * NH * HD * 4)},
            "gpu_launches": int(launches), "clocks": clocks,
        }
    # --- figures of the other configurations, measured in the same run (bounded; a failure leaves the headline line intact) ---
    side = {}
    if not args.no_cpu and layers == LAYERS and ctx0 == CTX0:
        if world > 1:
            try:
                r = measure_split(args, 262144, steps=min(args.steps, 16), warmup=3, dist=dist, rank=rank, local_rank=local_rank, world=world)
                if rank == 0:
                    side["split_262144_us_per_layer"] = r["us_per_layer"]
                    side["split_262144"] = r
            except Exception as e:  # noqa: BLE001
                side["split_262144_error"] = str(e)[:300]
        else:
            try:
                r = measure_config3(args, steps=5, warmup=3, dist=None, rank=0, local_rank=local_rank, world=1)
                side["config3_tokens_per_s"] = r["tokens_per_s"]
                side["config3"] = r
            except Exception as e:  # noqa: BLE001
                side["config3_error"] = str(e)[:300]
            try:
                r = measure_config4(args, runs=3)
                side["config4_restore_gb_s"] = r["restore_gb_per_s"]
                side["config4"] = r
            except Exception as e:  # noqa: BLE001
                side["config4_error"] = str(e)[:300]
            ref_us = reference_kernel_us()
            if ref_us is not None:
                side["reference_kernel_us_per_layer"] = ref_us
                side["reference_kernel"] = "the reference's attn_core_w48m<8> (82 x 512 cooperative launch) at K5r/V6 + window 2048, 101,600 positions, 8 queries, same GPU, same run"
            line["cpu_baseline"] = cpu_baseline_sample()
    if rank == 0:
        line.update(side)
        emit(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
