"""Benchmark of the paged KV-cache decode path (append + paged GQA decode, every layer, per decode step).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): Qwen2.5-3B attention shape (16 query heads, 2 KV heads, head_dim 128, bf16 KV, 36 layers),
batch 32, context lengths uniform in [512, 4096], 16-token blocks in a 16384-block pool per layer with seeded
random block tables; Q/K/V activations N(0,1).  One "step" = one decode step: for each of the 36 layers the
fused RoPE + KV append of 32 new tokens followed by paged GQA decode attention; contexts grow by one token
per step.  Metric: decode tokens per second (batch / step time), with the KV-read bandwidth it implies.

With N > 1 (one process per GPU under torch.distributed.run) every rank runs its own batch of 32 sequences
over its own pool (sequences shard across GPUs, no data-path collective): weak scaling, value = all ranks'
tokens over the slowest rank's time.

`--impl reference` times the CPU restatement of the reference's path (oracle/, OpenMP over all host cores)
on a bounded sample of the same workload.
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

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from kriya_rt_b200 import workloads as W  # noqa: E402

METRIC = "paged_gqa_decode_tokens_per_s"
UNIT = "tokens/s"
SHAPE = W.QWEN25_3B
BATCH = 32
NUM_BLOCKS = 16384
CTX_LO, CTX_HI = 512, 4096
TIMED_DEVICE_S = 0.5   # device time the repeated timed region must add up to
MAX_REPEATS = 200
WORKLOAD = ("qwen2.5-3b attention decode: Hq16 Hkv2 D128 bf16, 36 layers, batch 32/GPU, ctx U[512,4096], "
            "16-token blocks, 16384-block pool/layer, append+attention per layer per step")


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []  # (arrival time, text)
        self.thread = None
        self.t0 = self.t1 = None

    def mark_start(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "10"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        # nvidia-smi is started before the warm-up (it takes tens of ms to print its first line); only the samples that
        # arrived inside the timed region count.  A region too short to hold one falls back to every sample of the run.
        inside = [ln for (t, ln) in self.lines if self.t0 is not None and self.t1 is not None and self.t0 <= t <= self.t1]
        window = "timed region"
        if not inside:
            inside, window = [ln for (_, ln) in self.lines], "warm-up + timed region"
        sm, mx, reasons = [], None, set()
        for ln in inside:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "window": window}


def contexts_for_rank(rank: int) -> np.ndarray:
    """Every rank serves a batch with the same context lengths (weak scaling: per-GPU work is fixed); block tables and
    tensor values differ per rank."""
    return W.config2_contexts(seed_tables=2002, batch=BATCH, lo=CTX_LO, hi=CTX_HI)


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle port on a bounded sample
# ---------------------------------------------------------------------------------------------------


def cpu_sample(layers_in_sample: int, repeats: int, seed: int = 1002):
    """Times `layers_in_sample` layers of one decode step (append + whole-row decode per layer) on the host
    cores with the C oracle.  Returns (seconds per sample, cores, description)."""
    from oracle import c_oracle as O

    ctx = contexts_for_rank(0)
    batch = W.make_decode_batch(SHAPE, ctx, NUM_BLOCKS, seed=2002)
    rng = np.random.default_rng(seed)
    Hq, Hkv, D = SHAPE.num_q_heads, SHAPE.num_kv_heads, SHAPE.head_dim
    # only the blocks the tables name need real data; the pool is allocated once and shared by the layers
    ck = np.zeros((NUM_BLOCKS, 16, Hkv, D), np.uint16)
    cv = np.zeros((NUM_BLOCKS, 16, Hkv, D), np.uint16)
    used = batch.page_indices
    ck[used] = W.normal16(rng, (used.size, 16, Hkv, D), W.BF16)
    cv[used] = W.normal16(rng, (used.size, 16, Hkv, D), W.BF16)
    q = W.normal16(rng, (BATCH, Hq, D), W.BF16)
    k = W.normal16(rng, (BATCH, Hkv, D), W.BF16)
    v = W.normal16(rng, (BATCH, Hkv, D), W.BF16)
    rp = O.RopeParams(Hq, Hkv, D, D, 16, 0, 1e-6, SHAPE.rope_theta, 8192, 1, 0, 0)
    gp = O.GqaParams(Hq, Hkv, D, 16, 16, 1, float(np.float32(1.0) / np.sqrt(np.float32(D))), 0.0)
    table = O.rope_table(8192, D, SHAPE.rope_theta)
    # all the host cores this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for its workers)
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    O.set_num_threads(max(1, avail))
    cores = O.num_threads()

    def one_sample():
        for _ in range(layers_in_sample):
            qq = q.copy()
            O.rope_kv_append(qq, k, v, ck, cv, batch.page_indptr, batch.page_indices, batch.last_page_len,
                             batch.positions, rp, W.BF16, table=table)
            O.decode(qq, ck, cv, batch.page_indptr, batch.page_indices, batch.last_page_len, gp, W.BF16)

    one_sample()  # warm caches / OpenMP pool
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        one_sample()
        times.append(time.perf_counter() - t0)
    desc = (f"{layers_in_sample} of {SHAPE.num_layers} layers of one decode step (batch {BATCH}, "
            f"{batch.attended_tokens} attended tokens/layer), scaled by {SHAPE.num_layers}/{layers_in_sample}")
    return float(np.median(times)), cores, desc


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # size the sample from one layer so that warmup + steps stay within a few minutes
    t1, cores, _ = cpu_sample(1, 1)
    budget_s = 150.0
    per_step_budget = budget_s / max(args.steps + args.warmup, 1)
    layers = int(max(1, min(SHAPE.num_layers, per_step_budget / max(t1, 1e-6))))
    from oracle import c_oracle as O  # noqa: F401

    times = []
    for i in range(args.warmup + args.steps):
        t, cores, desc = cpu_sample(layers, 1, seed=1002 + i)
        if i >= args.warmup:
            times.append(t)
    step_s = float(np.mean(times)) * SHAPE.num_layers / layers
    value = BATCH / step_s
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference path (the reference is Rust + Metal "
                   "and cannot run here); rank 0 host cores only"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------


def run_gpu_arm(args):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from kriya_rt_b200.executor import CudaExecutor
    from kriya_rt_b200.kv import PagedKvCacheManager

    L, Hq, Hkv, D = SHAPE.num_layers, SHAPE.num_q_heads, SHAPE.num_kv_heads, SHAPE.head_dim
    K, Wu = args.steps, args.warmup
    ex = CudaExecutor(num_layers=L, num_kv_blocks=NUM_BLOCKS, block_size_tokens=16, num_q_heads=Hq, num_kv_heads=Hkv,
                      head_dim=D, dtype=W.BF16, device=local_rank, rope_theta=SHAPE.rope_theta, rope_max_seq_len=8192,
                      max_batch_rows=64, max_page_indices=NUM_BLOCKS, max_tiles=4096, max_query_tokens=64)
    stream = torch.cuda.ExternalStream(ex.stream_ptr, device=torch.device("cuda", local_rank))

    # KV pool: N(0,1) in every block of every layer (bf16), generated on the device
    gen = torch.Generator(device="cuda").manual_seed(1002 + rank)
    for layer in range(L):
        kview, vview = ex.layer_cache_views(layer)
        for view in (kview, vview):
            flat = view.view(-1)
            chunk = 1 << 25
            for s in range(0, flat.numel(), chunk):
                n = min(chunk, flat.numel() - s)
                flat[s:s + n] = torch.randn(n, device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16)
    # activations for all layers, resident in HBM (one buffer set reused every step)
    q = torch.randn(L, BATCH, Hq, D, device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16)
    k = torch.randn(L, BATCH, Hkv, D, device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16)
    v = torch.randn(L, BATCH, Hkv, D, device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16)
    out = torch.zeros_like(q)
    torch.cuda.synchronize()

    ctx0 = contexts_for_rank(rank)
    rp = ex.rope_params()
    gp = ex.gqa_params()

    # Bookkeeping runs in the compiled manager exactly as a scheduler would drive it: one append_token_slot
    # per sequence, then build_schedule_plan, every step.
    def fresh_manager():
        mgr = PagedKvCacheManager(NUM_BLOCKS, 0, 16)
        rng = np.random.default_rng(2002 + 17 * rank)
        # a seeded shuffle of the free list: allocate every block once in random order and free in that order
        order = rng.permutation(NUM_BLOCKS)
        ids = [mgr.gpu_allocator.allocate_block() for _ in range(NUM_BLOCKS)]
        for b in order:
            mgr.gpu_allocator.free_block(int(ids[b]))
        for i, c in enumerate(ctx0):
            mgr.allocate_sequence(i, (np.arange(int(c), dtype=np.uint32) + np.uint32(100000 * (i + 1))))
        return mgr

    seq_ids = list(range(BATCH))

    def step_plan(mgr, t):
        mgr.append_token_slots(seq_ids)  # one append_token_slot per sequence, in the scheduler's order
        plan = mgr.build_schedule_plan(seq_ids, 8)
        positions = (ctx0 + t).astype(np.uint32)
        return plan, positions

    def barrier():
        if dist is not None:
            dist.barrier()

    host_times = {}

    def device_pass(mode, steps, warm):
        """`warm` untimed and exactly `steps` timed decode steps from a fresh sequence state, bracketed by a barrier and
        a device synchronisation on both sides; returns (device ms of the timed steps, launches in them)."""
        ex.set_fused_append(mode)
        mgr = fresh_manager()
        for t in range(warm):
            plan, pos = step_plan(mgr, t)
            ex.upload_schedule_plan(plan, pos)
            ex.decode_step(q, k, v, out, BATCH, rp, gp)
        ex.sync()
        barrier()
        torch.cuda.synchronize()
        launches0 = ex.launch_count
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        host_issue = 0.0
        for t in range(warm, warm + steps):
            plan, pos = step_plan(mgr, t)
            ex.upload_schedule_plan(plan, pos)
            h1 = time.perf_counter()
            ex.decode_step(q, k, v, out, BATCH, rp, gp)
            host_issue += time.perf_counter() - h1
        ev1.record(stream)
        ex.sync()
        torch.cuda.synchronize()
        barrier()
        host_times["issue_ms_per_step"] = host_issue / steps * 1e3  # the host's time to issue the step's 36 launches
        # the host's own work for a step (bookkeeping, plan, upload call) with the GPU idle: inside the loop above the upload
        # also waits for the plan buffer of two steps ago, i.e. for the GPU, which the host runs ahead of
        host_plan = 0.0
        for t in range(warm + steps, warm + steps + 8):
            h0 = time.perf_counter()
            plan, pos = step_plan(mgr, t)
            ex.upload_schedule_plan(plan, pos)
            host_plan += time.perf_counter() - h0
            ex.sync()
        host_times["plan_ms_per_step"] = host_plan / 8 * 1e3
        return ev0.elapsed_time(ev1), ex.launch_count - launches0

    # ---- leg 1: device-resident throughput (`value`) -------------------------------------------------
    # The region of exactly --steps steps is repeated (every repeat from the same sequence state, so the work does not
    # drift) until at least TIMED_DEVICE_S of device time has been measured; the median repeat is the figure.
    attended = [int((ctx0 + t + 1).sum()) for t in range(Wu, Wu + K)]
    ex.timing_enable(False)
    sampler = ClockSampler(local_rank)
    sampler.start()
    device_pass(1, min(K, 3), Wu)  # module load, first-launch set-up, clocks up
    sampler.mark_start()
    repeats_ms, gpu_launches = [], 0
    while not repeats_ms or (sum(repeats_ms) < args.min_device_s * 1e3 and len(repeats_ms) < MAX_REPEATS):
        ms, n_launch = device_pass(1, K, Wu)
        if dist is not None:  # every rank must agree on the repeat count: the slowest rank's time decides
            t_rep = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t_rep, op=dist.ReduceOp.MAX)
            ms = float(t_rep[0])
        repeats_ms.append(ms)
        gpu_launches = n_launch
    sampler.mark_end()
    clocks = sampler.stop()
    elapsed_ms = float(np.median(repeats_ms))

    # ---- leg 1b: the same steps under three more launch disciplines (one repeat each), for the per-launch figures -----
    #   serialised: a layer's launch may be set up early but touches nothing before the previous layer has completed;
    #   dependent : a layer's activations wait for the previous layer (as in a model), its cached K/V streams at once;
    #   bracketed : every launch between two CUDA events (which costs idle time around each launch).
    host_step = dict(host_times)  # of the last repeat of the device-resident leg
    serial_ms, n_serial = device_pass(3, K, Wu)
    dep_ms, n_dep = device_pass(5, K, Wu)
    ex.set_fused_append(1)
    mgr_b = fresh_manager()
    for t in range(Wu):
        step_plan(mgr_b, t)
    ex.timing_enable(True)
    for t in range(Wu, Wu + K):
        plan, pos = step_plan(mgr_b, t)
        ex.upload_schedule_plan(plan, pos)
        ex.decode_step(q, k, v, out, BATCH, rp, gp)
    ex.sync()
    n_dec, ms_dec = ex.timing_read(0)
    ex.timing_enable(False)

    # ---- leg 2: end to end through host buffers ---------------------------------------------------------
    qh = torch.empty(L, BATCH, Hq, D, dtype=torch.int16).pin_memory()
    kh = torch.empty(L, BATCH, Hkv, D, dtype=torch.int16).pin_memory()
    vh = torch.empty(L, BATCH, Hkv, D, dtype=torch.int16).pin_memory()
    oh = torch.empty(L, BATCH, Hq, D, dtype=torch.int16).pin_memory()
    qh.copy_(q.cpu()); kh.copy_(k.cpu()); vh.copy_(v.cpu())
    plan_bytes = 0
    e2e_repeats = []
    while not e2e_repeats or (sum(e2e_repeats) < args.min_device_s and len(e2e_repeats) < MAX_REPEATS):
        mgr2 = fresh_manager()
        for t in range(Wu):
            plan, pos = step_plan(mgr2, t)
            ex.upload_schedule_plan(plan, pos)
            ex.decode_step_host(qh, kh, vh, oh, BATCH, rp, gp)
        barrier()
        # Every timed step copies its inputs from pinned host memory, runs the 36 layers, copies the result back and waits
        # for it.  The host's work for the NEXT step (block allocation, plan build, plan upload) runs between the begin and
        # the end of the current step, i.e. while the GPU is busy; the upload queues behind the step on the same stream.
        t0 = time.perf_counter()
        plan, pos = step_plan(mgr2, Wu)
        ex.upload_schedule_plan(plan, pos)
        for t in range(Wu, Wu + K):
            plan_bytes = 4 * (plan.page_indptr.size + plan.page_indices.size + plan.last_page_len.size + pos.size) + \
                16 * plan.cta_work_tiles.shape[0]
            ex.decode_step_host_begin(qh, kh, vh, oh, BATCH, rp, gp)
            if t + 1 < Wu + K:
                plan, pos = step_plan(mgr2, t + 1)
                ex.upload_schedule_plan(plan, pos)
            ex.decode_step_host_end()  # the step's result is in host memory
        dt = time.perf_counter() - t0
        if dist is not None:
            t_rep = torch.tensor([dt], device="cuda", dtype=torch.float64)
            dist.all_reduce(t_rep, op=dist.ReduceOp.MAX)
            dt = float(t_rep[0])
        e2e_repeats.append(dt)
        barrier()
    e2e_ms = float(np.median(e2e_repeats)) * 1e3

    # max over ranks (the repeats were reduced as they were taken)
    ms_per_step = elapsed_ms / K
    value = world * BATCH / (ms_per_step * 1e-3)
    e2e_value = world * BATCH / (e2e_ms / K * 1e-3)

    # roofline of the dominant kernel (paged decode): algorithmic bytes per launch / mean launch time
    kv_bytes_launch = float(np.mean(attended)) * SHAPE.kv_bytes_per_token  # K and V, each element once
    qo_bytes = 2 * BATCH * Hq * D * 2
    table_bytes = 4 * float(np.mean([(c + 15) // 16 for c in attended])) + 4 * (2 * BATCH + 1)
    alg_bytes = kv_bytes_launch + qo_bytes + table_bytes
    peaks, peak_kind = measured_peaks()
    peak = peaks["hbm_gbs"]

    def gbs(us):
        return alg_bytes / (us * 1e-6) / 1e9

    dec_us = ms_dec / max(n_dec, 1) * 1e3
    instream_us = elapsed_ms * 1e3 / max(gpu_launches, 1)
    serial_us = serial_ms * 1e3 / max(n_serial, 1)
    dep_us = dep_ms * 1e3 / max(n_dep, 1)
    achieved = gbs(instream_us)
    traffic = None
    tfile = ROOT / "profiles" / "decode_traffic.json"
    if tfile.exists():
        try:
            traffic = json.loads(tfile.read_text()).get("dram_bytes_per_attended_token", None)
            traffic = traffic * float(np.mean(attended)) if traffic else None
        except Exception:
            traffic = None

    ex.close()
    del q, k, v, out
    torch.cuda.empty_cache()
    config5 = None if args.no_config5 else run_config5(args, rank, local_rank, world, dist, peak)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wu,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "inputs larger than L2: each step streams %.2f GB of KV" %
                       (kv_bytes_launch * L / 1e9), "plan": "rebuilt on the host every step by the C++ manager and uploaded inside the timed region",
                       "host_ms_per_step": host_step, "kv_read_gbs_whole_step": kv_bytes_launch * L / (ms_per_step * 1e-3) / 1e9,
                       "kernels_per_layer": gpu_launches / K / L,
                       "timed_region": {"repeats": len(repeats_ms), "steps_per_repeat": K, "device_s_total": sum(repeats_ms) / 1e3,
                                        "ms_per_step_median": ms_per_step, "ms_per_step_min": min(repeats_ms) / K,
                                        "ms_per_step_max": max(repeats_ms) / K,
                                        "ms_per_step_x_sm_mhz": (ms_per_step * clocks["sm_mhz"]) if clocks.get("sm_mhz") else None,
                                        "how": "exactly --steps steps per repeat between barrier + synchronize, every repeat from the same "
                                               "sequence state; value is the median repeat (max over ranks per repeat)"},
                       "e2e_repeats": len(e2e_repeats)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic,
                         "launch_us_in_stream": instream_us,
                         "launch_us_dependent": dep_us, "achieved_dependent": gbs(dep_us), "frac_dependent": gbs(dep_us) / peak,
                         "launch_us_serial": serial_us, "achieved_serial": gbs(serial_us), "frac_serial": gbs(serial_us) / peak,
                         "launch_us_isolated": dec_us, "achieved_isolated": gbs(dec_us) if n_dec else None,
                         "frac_isolated": (gbs(dec_us) / peak) if n_dec else None,
                         "how": "achieved = algorithmic bytes per launch / (device time of the timed region / launches in it), CUDA events on "
                                "the launching stream.  in_stream: the 36 launches of a step have independent inputs and may overlap (programmatic "
                                "dependent launch; such launches take the plan's work list with at least 14 tiles per CTA, so about two "
                                "launches are in flight; the other legs take the list of a single launch, at least 8 tiles); dependent: every layer's queries and new K/V wait for the previous "
                                "layer's launch, only its cached K/V streams early; serial: nothing of a launch but its set-up precedes the "
                                "previous launch's completion; isolated: every launch between two events of its own (includes the idle time "
                                "the events cost)",
                         "kernel": "decode_tcp_kernel (fused RoPE + append + paged GQA decode, whole pages per copy)",
                         "algorithmic_bytes_per_launch": alg_bytes, "peak_source": peak_kind,
                         "frac_of_nominal_8000": achieved / 8000.0},
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": int(plan_bytes + qh.numel() * 2 + kh.numel() * 2 + vh.numel() * 2),
                    "d2h_bytes_per_step": int(oh.numel() * 2 + 4)},
            "gpu_launches": int(gpu_launches),
            "clocks": clocks,
            "config5": config5,
        }
        if world > 1 and config5 and "one_sequence_131072" in config5:  # the KV-axis split through the product entry point
            one = config5["one_sequence_131072"]
            line["kvsplit"] = {"max_abs_err": one.get("max_abs_err"), "us_per_layer": one.get("us_per_layer"),
                               "entry_point": "kriya_cuda_kvsplit_decode", "check": one.get("check")}
        if world == 1 and not args.no_cpu_baseline:
            t1, cores, _ = cpu_sample(1, 1)
            layers = int(max(1, min(L, 15.0 / max(t1, 1e-6))))
            ts, cores, desc = cpu_sample(layers, 1)
            line["cpu_baseline"] = {"value": BATCH / (ts * L / layers), "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": desc}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_config5(args, rank, local_rank, world, dist, peak):
    """BASELINE config 5 on the GPUs of this run, one layer resident (36 layers of it are 193 GB):
    (a) 256 sequences of U[8192,32768] tokens dealt longest-first over the ranks (strong scaling: the total is fixed),
        one fused append + decode launch per rank and layer;
    (b) one 131072-token sequence: on one GPU as a whole; on N > 1 GPUs split along the KV axis, every rank holding its
        block range, partial-state decode + exchange over NVLink + merge through kriya_cuda_kvsplit_decode.  Before it is
        timed, a small split case is compared with the CPU oracle on rank 0 (max_abs_err)."""
    import torch

    from kriya_rt_b200 import sharding
    from kriya_rt_b200.executor import CudaExecutor

    dev = torch.device("cuda", local_rank)
    gen = torch.Generator(device="cuda").manual_seed(7 + rank)
    reps = 10

    def fill_all(ex):
        for view in ex.layer_cache_views(0):
            flat = view.view(-1)
            chunk = 1 << 26
            for s in range(0, flat.numel(), chunk):
                n = min(chunk, flat.numel() - s)
                flat[s:s + n] = torch.randn(n, device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16)

    def rnd(*shape):
        return torch.randn(*shape, device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16)

    def reduce_max_sum(us, nbytes):
        t = torch.tensor([us, float(nbytes)], device="cuda", dtype=torch.float64)
        if dist is None:
            return float(t[0]), float(t[1])
        tmax, tsum = t.clone(), t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        return float(tmax[0]), float(tsum[1])

    res = {}
    # ---- (a) sequences partitioned over the ranks -------------------------------------------------------------
    lengths = np.random.default_rng(2005).integers(8192, 32768 + 1, size=256)
    mine = sharding.assign_sequences(lengths, world)[rank]
    ctx = lengths[mine]
    nblocks = int(((ctx + 16) // 16).sum()) + 16
    batch = W.make_decode_batch(SHAPE, ctx, nblocks, seed=2005 + rank)
    ex = CudaExecutor(num_layers=1, num_kv_blocks=nblocks, block_size_tokens=16, num_q_heads=16, num_kv_heads=2, head_dim=128,
                      device=local_rank, rope_theta=SHAPE.rope_theta, rope_max_seq_len=32768 + 64, max_batch_rows=256,
                      max_page_indices=nblocks, max_tiles=65536)
    fill_all(ex)  # the whole pool holds N(0,1) data
    n = len(mine)
    q, k, v = rnd(n, 16, 128), rnd(n, 2, 128), rnd(n, 2, 128)
    out = torch.zeros_like(q)
    torch.cuda.synchronize()
    ex.upload_schedule_plan(batch, batch.positions)
    rp, gp = ex.rope_params(), ex.gqa_params()
    stream = torch.cuda.ExternalStream(ex.stream_ptr, device=dev)
    for _ in range(3):
        ex.append_decode(0, q, k, v, out, rp, gp)
    ex.sync()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        ex.append_decode(0, q, k, v, out, rp, gp)
    e1.record(stream)
    ex.sync()
    torch.cuda.synchronize()
    us, total_bytes = reduce_max_sum(e0.elapsed_time(e1) / reps * 1e3, batch.kv_bytes_per_layer)
    res["sequences_partitioned"] = {
        "sequences": 256, "ctx": "U[8192,32768]", "assignment": "longest first", "us_per_layer": us, "kv_bytes_all_gpus": total_bytes,
        "kv_gbs_aggregate": total_bytes / (us * 1e-6) / 1e9, "kv_gbs_per_gpu": total_bytes / world / (us * 1e-6) / 1e9,
        "frac_of_hbm_peak_per_gpu": total_bytes / world / (us * 1e-6) / 1e9 / peak,
        "tokens_per_s_36_layers": 256 / (us * 36e-6), "launches_timed": reps, "pool": "whole pool filled with N(0,1)"}
    ex.close()
    del q, k, v, out
    torch.cuda.empty_cache()

    # ---- (b) one 131072-token sequence ------------------------------------------------------------------------
    def kvsplit_case(tokens, check):
        nb = (tokens + 15) // 16
        b, e = sharding.kv_axis_ranges([nb], world)[rank]
        b0, e0_ = int(b[0]), int(e[0])
        n_local = e0_ - b0
        exs = CudaExecutor(num_layers=1, num_kv_blocks=max(n_local, 1), block_size_tokens=16, num_q_heads=16, num_kv_heads=2,
                           head_dim=128, device=local_rank, max_page_indices=nb, rope_max_seq_len=4096)
        local_ids = np.random.default_rng(90 + rank).permutation(max(n_local, 1))[:n_local]
        if check:
            rng = np.random.default_rng(81)  # the same stream on every rank: the whole K/V exists on the host only
            kk = W.normal16(rng, (nb, 16, 2, 128), W.BF16)
            vv = W.normal16(rng, (nb, 16, 2, 128), W.BF16)
            q16 = W.normal16(rng, (1, 16, 128), W.BF16)
            kview, vview = exs.layer_cache_views(0)
            ids = torch.from_numpy(local_ids.astype(np.int64)).cuda()
            kview[ids] = torch.from_numpy(kk[b0:e0_].view(np.int16)).cuda()
            vview[ids] = torch.from_numpy(vv[b0:e0_].view(np.int16)).cuda()
            qd = torch.from_numpy(q16.view(np.int16)).cuda()
        else:
            fill_all(exs)
            qd = rnd(1, 16, 128)
        table = sharding.local_block_table(np.zeros(nb), b0, e0_, local_ids)
        outd = torch.zeros_like(qd)
        torch.cuda.synchronize()
        exs.plan_upload([0, nb], table, [tokens - (nb - 1) * 16], None, [tokens - 1])
        exs.plan_set_ranges(b, e)
        gps = exs.gqa_params()
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, exs.comm_export(1))
            exs.comm_init(rank, handles)
            call = lambda: exs.kvsplit_decode(0, qd, outd, gps)  # noqa: E731
        else:
            call = lambda: exs.paged_gqa_decode(0, qd, outd, gps)  # noqa: E731
        if check:
            call()
            exs.sync()
            err = None
            if rank == 0:
                from oracle import c_oracle as O

                p = O.GqaParams(16, 2, 128, 16, 16, 1, float(np.float32(1.0) / np.sqrt(np.float32(128))), 0.0)
                _, ref = O.decode(q16, kk, vv, [0, nb], np.arange(nb), [tokens - (nb - 1) * 16], p, W.BF16)
                err = float(np.abs(W.from_storage(outd.cpu().numpy().view(np.uint16), W.BF16) - ref).max())
            if dist is not None:
                dist.barrier()
            exs.close()
            return err
        st = torch.cuda.ExternalStream(exs.stream_ptr, device=dev)
        for _ in range(5):
            call()
        exs.sync()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_calls = 50
        a0.record(st)
        for _ in range(n_calls):
            call()
        a1.record(st)
        exs.sync()
        torch.cuda.synchronize()
        us_l, _ = reduce_max_sum(a0.elapsed_time(a1) / n_calls * 1e3, 0)
        exs.close()
        return us_l

    err = kvsplit_case(16384 + 5, True)
    us_split = kvsplit_case(131072, False)
    res["one_sequence_131072"] = {
        "n_gpus": world, "us_per_layer": us_split,
        "how": ("whole sequence on one GPU, one decode launch per layer" if world == 1 else
                "KV axis split over the ranks: partial-state decode + one exchange kernel (peer stores into every rank's buffer "
                "over NVLink, bounded wait, merge) per layer through kriya_cuda_kvsplit_decode; no collective library"),
        "kv_bytes_per_gpu": 131072 * 1024 // world, "max_abs_err": err,
        "check": "16389-token sequence split the same way, against the CPU oracle on rank 0 (bar 1e-2 for bf16)"}
    return res


def run_kernel_case(args):
    """A small single-kernel case for profiling under ncu: a few launches of one kernel, nothing else.
    decode : Qwen2.5-3B shape, one layer, batch 32, contexts U[2048,8192] (about 170 MB of KV, larger than L2)
    decode_fused: the benchmark's own layer (contexts U[512,4096], about 80 MB) through the fused append + decode launch
    prefill: Qwen2.5-1.5B shape, one 2048-token prompt, last 512-token chunk (prefix 1536)
    append : Qwen2.5-3B shape, 32 tokens;  copy: 64 pairs x 36 layers"""
    import torch

    from kriya_rt_b200.executor import CudaExecutor

    case, reps = args.kernel_case, args.steps
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(7)

    def fill(ex, layers):
        for layer in range(layers):
            for view in ex.layer_cache_views(layer):
                view.view(-1).copy_(torch.randn(view.numel(), device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16))

    def rnd(*shape):
        return torch.randn(*shape, device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16)

    if case in ("decode", "append", "decode_fused"):
        sh = SHAPE
        lo, hi = (CTX_LO, CTX_HI) if case == "decode_fused" else (2048, 8192)
        ctx = W.config2_contexts(seed_tables=2002, batch=BATCH, lo=lo, hi=hi)
        batch = W.make_decode_batch(sh, ctx, NUM_BLOCKS, seed=2002)
        ex = CudaExecutor(num_layers=1, num_kv_blocks=NUM_BLOCKS, block_size_tokens=16, num_q_heads=16, num_kv_heads=2,
                          head_dim=128, rope_theta=sh.rope_theta, rope_max_seq_len=16384, max_page_indices=NUM_BLOCKS)
        fill(ex, 1)
        q, k, v = rnd(BATCH, 16, 128), rnd(BATCH, 2, 128), rnd(BATCH, 2, 128)
        out = torch.zeros_like(q)
        torch.cuda.synchronize()
        ex.upload_schedule_plan(batch, batch.positions)
        rp, gp = ex.rope_params(), ex.gqa_params()
        def one():
            if case == "append":
                ex.rope_kv_append(0, q, k, v, BATCH, rp)
            elif case == "decode_fused":
                ex.append_decode(0, q, k, v, out, rp, gp)
            else:
                ex.paged_gqa_decode(0, q, out, gp)

        for _ in range(2):  # untimed: module load and first-launch set-up
            one()
        ex.timing_enable(True)
        for _ in range(reps):
            one()
        n, ms = ex.timing_read(1 if case == "append" else 0)
        kv_bytes = batch.kv_bytes_per_layer
        print(json.dumps({"case": case, "launches": n, "us_per_launch": ms / max(n, 1) * 1e3,
                          "kv_bytes_per_launch": kv_bytes, "attended_tokens": batch.attended_tokens,
                          "kv_gbs": kv_bytes / (ms / max(n, 1) * 1e-3) / 1e9 if case != "append" and n else None}))
        ex.close()
    elif case == "decode_ctx":
        # batch 32, every context the same length (--case-ctx), 8 layers with pools of their own (every layer cold), the
        # fused append + decode step in the stream; the three dependency modes of the step beside one another
        sh, layers, ctxlen = SHAPE, 8, args.case_ctx
        nblk = BATCH * ((ctxlen + 15) // 16) + 64
        batch = W.make_decode_batch(sh, np.full(BATCH, ctxlen - 1), nblk, seed=2003)
        ex = CudaExecutor(num_layers=layers, num_kv_blocks=nblk, block_size_tokens=16, num_q_heads=16, num_kv_heads=2,
                          head_dim=128, rope_theta=sh.rope_theta, rope_max_seq_len=max(8192, ctxlen + 64), max_page_indices=nblk,
                          max_batch_rows=BATCH)
        fill(ex, layers)
        q, k, v = rnd(layers, BATCH, 16, 128), rnd(layers, BATCH, 2, 128), rnd(layers, BATCH, 2, 128)
        out = torch.zeros_like(q)
        torch.cuda.synchronize()
        ex.upload_schedule_plan(batch, batch.positions)
        rp, gp = ex.rope_params(), ex.gqa_params()
        stream = torch.cuda.ExternalStream(ex.stream_ptr)
        kv_bytes = batch.kv_bytes_per_layer
        peak = float(measured_peaks()[0]["hbm_gbs"])
        res = {"case": case, "ctx": ctxlen, "batch": BATCH, "layers": layers, "kv_bytes_per_launch": kv_bytes, "peak_gbs": peak}
        for name, mode in (("in_stream", 1), ("dependent", 5), ("serial", 3), ("plain", 7)):
            ex.set_fused_append(mode)
            for _ in range(3):
                ex.decode_step(q, k, v, out, BATCH, rp, gp)
            ex.sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                ex.decode_step(q, k, v, out, BATCH, rp, gp)
            e1.record(stream)
            ex.sync()
            us = e0.elapsed_time(e1) / (reps * layers) * 1e3
            res[name] = {"us_per_launch": us, "kv_gbs": kv_bytes / (us * 1e-6) / 1e9, "frac_of_peak": kv_bytes / (us * 1e-6) / 1e9 / peak}
        print(json.dumps(res))
        ex.close()
    elif case == "decode_q4":
        # the same rows over a Q4KvGroup32 cache (CUDA-core decode kernel): GB/s on the STORED bytes, 20 per 32 values
        from kriya_rt_b200.executor import KV_Q4_GROUP32
        sh, ctxlen = SHAPE, args.case_ctx
        nblk = BATCH * ((ctxlen + 15) // 16) + 64
        batch = W.make_decode_batch(sh, np.full(BATCH, ctxlen - 1), nblk, seed=2004)
        res = {"case": case, "ctx": ctxlen, "batch": BATCH}
        for name, fmt in (("q4", KV_Q4_GROUP32), ("bf16_same_kernel", 0)):
            ex = CudaExecutor(num_layers=1, num_kv_blocks=nblk, block_size_tokens=16, num_q_heads=16, num_kv_heads=2, head_dim=128,
                              rope_theta=sh.rope_theta, max_page_indices=nblk, max_batch_rows=BATCH, kv_format=fmt)
            ex.set_decode_path(1)
            for view in ex.layer_cache_views(0):
                if fmt:  # valid groups: any codes, scale 2^-6 (f16 0x2400), min -0.1 (f16 0xAE66)
                    grp = torch.randint(-32768, 32767, (view.numel() // 10, 10), device="cuda", dtype=torch.int16)
                    grp[:, 8] = 0x2400
                    grp[:, 9] = -0x519A
                    view.view(-1).copy_(grp.view(-1))
                else:
                    view.view(-1).copy_(torch.randn(view.numel(), device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16))
            q = rnd(BATCH, 16, 128)
            out = torch.zeros_like(q)
            torch.cuda.synchronize()
            ex.upload_schedule_plan(batch, batch.positions)
            gp = ex.gqa_params()
            for _ in range(2):
                ex.paged_gqa_decode(0, q, out, gp)
            ex.timing_enable(True)
            for _ in range(reps):
                ex.paged_gqa_decode(0, q, out, gp)
            n, ms = ex.timing_read(0)
            stored = batch.attended_tokens * 2 * 2 * (128 // 32 * 20 if fmt else 128 * 2)
            res[name] = {"us_per_launch": ms / max(n, 1) * 1e3, "stored_kv_bytes": stored,
                         "stored_gbs": stored / (ms / max(n, 1) * 1e-3) / 1e9, "finite": bool(torch.isfinite(out.view(torch.bfloat16).float()).all())}
            ex.close()
        print(json.dumps(res))
    elif case == "kvsplit":
        # one 131072-token sequence (Qwen2.5-3B shape) cut along the KV axis over WORLD_SIZE GPUs: per layer, the
        # partial-state decode over this rank's block range, one all-gather of (m, l, o), the merge
        import torch.distributed as dist

        from kriya_rt_b200 import sharding

        rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        tokens, nb = 131072, 8192
        b, e = sharding.kv_axis_ranges([nb], world)[rank]
        n_local = int(e[0] - b[0])
        ex = CudaExecutor(num_layers=1, num_kv_blocks=n_local, block_size_tokens=16, num_q_heads=16, num_kv_heads=2,
                          head_dim=128, device=torch.cuda.current_device(), max_page_indices=nb)
        fill(ex, 1)
        table = sharding.local_block_table(np.zeros(nb), int(b[0]), int(e[0]), np.random.default_rng(rank).permutation(n_local))
        ex.plan_upload([0, nb], table, [16], None, [tokens - 1])
        q = rnd(1, 16, 128)
        out = torch.zeros_like(q)
        gp = ex.gqa_params()
        rows = 16
        local = torch.empty(rows * 130, device="cuda")
        stream = torch.cuda.ExternalStream(ex.stream_ptr)
        torch.cuda.synchronize()

        ex.plan_set_ranges(b, e)  # once per plan; every layer re-uses the split
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, ex.comm_export(1))
            ex.comm_init(rank, handles)

        def one(gather=True):
            if world > 1 and gather:
                ex.kvsplit_decode(0, q, out, gp)  # partial decode + exchange over NVLink + merge, all behind the C ABI
            else:
                ex.paged_gqa_decode_partial(0, q, None, None, local[:rows], local[rows:2 * rows], local[2 * rows:], gp)
                ex.merge_packed_states(local, 1, rows, out)

        res = {}
        for name, gather in (("with_gather", True), ("local_only", False)):
            for _ in range(3):
                one(gather)
            ex.sync()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                one(gather)
            e1.record(stream)
            ex.sync()
            torch.cuda.synchronize()
            dt = torch.tensor([e0.elapsed_time(e1) / reps * 1e3], device="cuda", dtype=torch.float64)
            if world > 1:
                dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            res[name] = float(dt[0])
        if rank == 0:
            print(json.dumps({"case": case, "n_gpus": world, "tokens": tokens, "us_per_layer": res["with_gather"],
                              "us_per_layer_without_gather": res["local_only"],
                              "kv_bytes_per_gpu": n_local * 16 * 1024,
                              "note": "CUDA events on the executor's stream, max over ranks; the exchange is one kernel per rank and layer (peer stores over NVLink, bounded wait, merge)"}))
        ex.close()
        if world > 1:
            dist.destroy_process_group()
    elif case == "decode_long":
        # long-context sharded decode: 256 sequences, contexts U[8192,32768], Qwen2.5-3B shape, ONE layer resident
        # (36 layers of this workload are 193 GB); with WORLD_SIZE > 1 the sequences are dealt to ranks longest-first
        import torch.distributed as dist

        from kriya_rt_b200 import sharding

        rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        lengths = np.random.default_rng(2005).integers(8192, 32768 + 1, size=args.case_long_seqs)
        mine = sharding.assign_sequences(lengths, world)[rank]
        ctx = lengths[mine]
        nblocks = int(((ctx + 16) // 16).sum()) + 16
        batch = W.make_decode_batch(SHAPE, ctx, nblocks, seed=2005 + rank)
        ex = CudaExecutor(num_layers=1, num_kv_blocks=nblocks, block_size_tokens=16, num_q_heads=16, num_kv_heads=2,
                          head_dim=128, device=torch.cuda.current_device(), rope_theta=SHAPE.rope_theta, rope_max_seq_len=32768 + 64,
                          max_batch_rows=256, max_page_indices=nblocks, max_tiles=65536)
        for view in ex.layer_cache_views(0):  # the whole pool holds N(0,1) data
            flat = view.view(-1)
            for s0 in range(0, flat.numel(), 1 << 26):
                nfill = min(1 << 26, flat.numel() - s0)
                flat[s0:s0 + nfill] = torch.randn(nfill, device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16)
        n = len(mine)
        q, k, v = rnd(n, 16, 128), rnd(n, 2, 128), rnd(n, 2, 128)
        out = torch.zeros_like(q)
        torch.cuda.synchronize()
        ex.upload_schedule_plan(batch, batch.positions)
        rp, gp = ex.rope_params(), ex.gqa_params()
        stream = torch.cuda.ExternalStream(ex.stream_ptr)
        for _ in range(3):
            ex.append_decode(0, q, k, v, out, rp, gp)
        ex.sync()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            ex.append_decode(0, q, k, v, out, rp, gp)
        e1.record(stream)
        ex.sync()
        t = torch.tensor([e0.elapsed_time(e1) / reps * 1e3, float(batch.kv_bytes_per_layer)], device="cuda", dtype=torch.float64)
        if world > 1:
            tmax = t.clone(); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            tsum = t.clone(); dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
            us, total_bytes = float(tmax[0]), float(tsum[1])
        else:
            us, total_bytes = float(t[0]), float(t[1])
        if rank == 0:
            print(json.dumps({"case": case, "n_gpus": world, "sequences": 256, "us_per_layer": us,
                              "kv_bytes_all_gpus": total_bytes, "kv_gbs_aggregate": total_bytes / (us * 1e-6) / 1e9,
                              "kv_gbs_per_gpu": total_bytes / world / (us * 1e-6) / 1e9,
                              "tokens_per_s_one_layer": 256 / (us * 1e-6), "tokens_per_s_36_layers": 256 / (us * 36e-6)}))
        ex.close()
        if world > 1:
            dist.destroy_process_group()
    elif case == "prefill_batch":
        # Qwen2.5-1.5B shape, --case-seqs (default eight) 2048-token prompts, the four 512-token chunks of every prompt, one launch per chunk index
        sh = W.QWEN25_1P5B
        n_seq, total, chunk = args.case_seqs, 2048, 512
        nb = n_seq * total // 16
        ex = CudaExecutor(num_layers=1, num_kv_blocks=nb, block_size_tokens=16, num_q_heads=12, num_kv_heads=2,
                          head_dim=128, rope_theta=sh.rope_theta, max_query_tokens=n_seq * chunk)
        fill(ex, 1)
        perm = np.random.default_rng(3).permutation(nb).astype(np.int32)
        per = total // 16
        ex.plan_upload(np.arange(n_seq + 1) * per, perm, [16] * n_seq)
        q = rnd(n_seq * chunk, 12, 128)
        kin, vin = rnd(n_seq * chunk, 2, 128), rnd(n_seq * chunk, 2, 128)
        out = torch.zeros_like(q)
        torch.cuda.synchronize()
        gp = ex.gqa_params(max_query_tokens=chunk)
        rp = ex.rope_params()
        stream = torch.cuda.ExternalStream(ex.stream_ptr)
        starts = np.arange(n_seq) * chunk

        def all_chunks(with_append):
            for prefix in range(0, total, chunk):
                if with_append:  # each chunk writes its RoPE'd K/V into the 16-token blocks, then attends
                    ex.rope_kv_append_chunk_batch(0, q, kin, vin, starts, [prefix] * n_seq, [chunk] * n_seq, rp)
                if with_append != 2:
                    ex.paged_gqa_prefill_batch(0, q, out, starts, [prefix] * n_seq, [chunk] * n_seq, gp)

        res = {}
        for name, with_append in (("append_and_attention", True), ("attention_only", False), ("append_only", 2)):
            all_chunks(with_append)
            ex.sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                all_chunks(with_append)
            e1.record(stream)
            ex.sync()
            res[name] = e0.elapsed_time(e1) / reps * 1e3
        us = res["append_and_attention"]
        flop = n_seq * 4 * 12 * 128 * (total * (total + 1) // 2)
        print(json.dumps({"case": case, "launches_per_pass": 2 * (total // chunk), "us_per_pass": us, "flop_per_pass": flop,
                          "tflops": flop / (us * 1e-6) / 1e12, "us_per_pass_attention_only": res["attention_only"],
                          "tflops_attention_only": flop / (res["attention_only"] * 1e-6) / 1e12,
                          "prompt_tokens_per_s_per_layer": n_seq * total / (us * 1e-6),
                          "us_per_pass_append_only": res["append_only"],
                          # the append reads q, k, v rows and writes q back and K/V into their blocks: 2 * (Hq + 2 Hkv) * D * 2 B per token
                          "append_gbs": n_seq * total * 2 * (12 + 4) * 128 * 2 / (res["append_only"] * 1e-6) / 1e9,
                          "append_frac_of_hbm_peak": n_seq * total * 2 * (12 + 4) * 128 * 2 / (res["append_only"] * 1e-6) / 1e9 / float(measured_peaks()[0]["hbm_gbs"]),
                          "note": "every chunk: one append launch (RoPE + K/V into the paged cache, all prompts) + one attention launch"}))
        ex.close()
    elif case == "prefill":
        sh = W.QWEN25_1P5B
        total, chunk = 2048, 512
        nb = 256
        ex = CudaExecutor(num_layers=1, num_kv_blocks=nb, block_size_tokens=16, num_q_heads=12, num_kv_heads=2,
                          head_dim=128, rope_theta=sh.rope_theta)
        fill(ex, 1)
        perm = np.random.default_rng(3).permutation(nb)[: total // 16].astype(np.int32)
        ex.plan_upload([0, perm.size], perm, [16])
        q = rnd(chunk, 12, 128)
        out = torch.zeros_like(q)
        torch.cuda.synchronize()
        gp = ex.gqa_params(max_query_tokens=chunk)
        stream = torch.cuda.ExternalStream(ex.stream_ptr)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ex.paged_gqa_prefill(0, q, out, total - chunk, chunk, gp)
        ex.sync()
        e0.record(stream)
        for _ in range(reps):
            ex.paged_gqa_prefill(0, q, out, total - chunk, chunk, gp)
        e1.record(stream)
        ex.sync()
        us = e0.elapsed_time(e1) / reps * 1e3
        flop = 4 * 12 * 128 * sum(total - chunk + i + 1 for i in range(chunk))
        print(json.dumps({"case": case, "launches": reps, "us_per_launch": us, "flop_per_launch": flop,
                          "tflops": flop / (us * 1e-6) / 1e12}))
        ex.close()
    elif case == "tree_verify":
        # Qwen2.5-3B shape: a draft tree of 11 nodes (root + 10) verified over a cached prefix of 4096 tokens, one layer
        n, prefix, nb = 11, 4096, 512
        ex = CudaExecutor(num_layers=1, num_kv_blocks=nb, block_size_tokens=16, num_q_heads=16, num_kv_heads=2, head_dim=128,
                          rope_theta=1e6, max_batch_rows=32)
        fill(ex, 1)
        blocks = prefix // 16
        table = np.random.default_rng(5).permutation(nb)[:blocks].astype(np.int32)
        ex.plan_upload(np.arange(n + 1) * blocks, np.tile(table, n), [16] * n, seq_positions=np.full(n, prefix, np.uint32))
        tq, tk, tv = rnd(n, 16, 128), rnd(n, 2, 128), rnd(n, 2, 128)
        out = torch.zeros_like(tq)
        mask = np.tril(np.ones((n, n), np.uint8))
        tp = ex.tree_verify_params(n, prefix)
        rp = ex.rope_params()
        torch.cuda.synchronize()
        stream = torch.cuda.ExternalStream(ex.stream_ptr)

        def one():
            ex.rope_inplace(tq, tk, n, rp)
            ex.tree_verify(0, tq, tk, tv, mask, out, tp)

        one(); one()
        ex.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            one()
        e1.record(stream)
        ex.sync()
        us = e0.elapsed_time(e1) / reps * 1e3
        kv_bytes = prefix * 2 * 2 * 128 * 2
        print(json.dumps({"case": case, "nodes": n, "prefix_tokens": prefix, "launches_per_call": 3, "us_per_layer": us,
                          "prefix_kv_bytes": kv_bytes, "kv_gbs_read_once": kv_bytes / (us * 1e-6) / 1e9,
                          "note": "rope_inplace + prefix decode of 11 rows over the same blocks + draft-tree kernel; the 4 MB prefix stays in L2"}))
        ex.close()
    elif case == "copy":
        layers, nb = 36, 2048
        ex = CudaExecutor(num_layers=layers, num_kv_blocks=nb, block_size_tokens=16, num_q_heads=16, num_kv_heads=2, head_dim=128)
        pairs = np.stack([np.arange(64, dtype=np.uint32), np.arange(1000, 1064, dtype=np.uint32)], 1)
        stream = torch.cuda.ExternalStream(ex.stream_ptr)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ex.kv_block_copy(pairs)
        ex.sync()
        e0.record(stream)
        for _ in range(reps):
            ex.kv_block_copy(pairs)
        e1.record(stream)
        ex.sync()
        us = e0.elapsed_time(e1) / reps * 1e3
        nbytes = 2 * 64 * layers * 2 * 8192
        print(json.dumps({"case": case, "launches": reps, "us_per_launch": us, "bytes_moved": nbytes,
                          "gbs": nbytes / (us * 1e-6) / 1e9}))
        ex.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--min-device-s", type=float, default=TIMED_DEVICE_S,
                    help="the timed region is repeated until it adds up to this much device time (0: once; for runs under a profiler)")
    ap.add_argument("--no-config5", action="store_true", help="skip the config 5 object (it fills the whole pool)")
    ap.add_argument("--case-long-seqs", type=int, default=256, help="sequences in the decode_long kernel case")
    ap.add_argument("--case-seqs", type=int, default=8, help="prompts in the prefill_batch kernel case")
    ap.add_argument("--case-ctx", type=int, default=4096, help="context length of every row in the decode_ctx / decode_q4 kernel cases")
    ap.add_argument("--kernel-case", default=None, choices=["decode", "decode_fused", "decode_ctx", "decode_q4", "decode_long", "prefill", "prefill_batch", "append", "copy", "kvsplit", "tree_verify"],
                    help="run a few launches of one kernel on a small case (for ncu), --steps = launches")
    args = ap.parse_args()
    if args.kernel_case:
        run_kernel_case(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
