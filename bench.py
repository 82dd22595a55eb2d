#!/usr/bin/env python3
"""Benchmark of the logits sampling path: sampled rows/s at vocab 151 936.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the sampler over one batch of synthetic rows (the "throughput"
workload: 4096 float32 rows x 151 936 columns per GPU, temperature 0.6, top-k 20,
top-p 0.95, repeat penalty 1.1 over a 1024-id history).  Rows are independent, so with
N GPUs every rank samples its own 4096 rows and there is no collective in the data path
(weak scaling); `value` is the rows all ranks sampled divided by the slowest rank's time.

Prints ONE JSON line on rank 0.  `value` is timed with the batch resident in HBM;
`e2e` is the same metric through the host-buffer C-ABI call (pinned host inputs, copies
inside the timed region) with the bare link rate beside it; `e2e_device_resident` is a step
of the batched decode loop (logits already on the device, one parameter record per row up,
one token per row back); `roofline` relates the streaming kernel to measured HBM bandwidth;
`cpu_baseline` is the CPU port of the reference sampler timed on this host.

Under torchrun (N > 1) the same line also carries `strong` -- the one 4096-row batch split
4096/N rows per GPU -- and `vocab_sharded` -- 1024 rows x 262 144 columns split by columns over
the N GPUs, local shortlist, one NCCL all-gather, merge -- each timed like the headline.

`--impl reference` times that CPU port alone, with every host thread, on the same
workload and step size, and prints the same kind of line.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "sampled rows/s at vocab 151936"
UNIT = "rows/s"
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0

WORKLOAD_NOTES = {
    "single_row": "temp 0.6 top_k 20 top_p 0.95 repeat_penalty 1.1, seeded N(0,3^2) logits with 16 boosted ids",
    "throughput": "temp 0.6 top_k 20 top_p 0.95 repeat_penalty 1.1, seeded N(0,3^2) logits with 16 boosted ids per row",
    "mixed_batch": "per-row temp U[0.2,1.5] top_k {40,1,20,50,200} top_p U[0.8,1] repeat_penalty U[1,1.3], "
                   "seeded N(0,3^2) logits with Zipf(1.1) spikes",
    "full_vocab_nucleus": "temp 1.0 top_k = vocabulary top_p 0.9 no penalty, seeded N(0,2^2) logits rounded to bf16",
}



def dram_traffic_ratio(kernel):
    """DRAM bytes a launch of `kernel` moves per algorithmic byte, from the recorded ncu capture
    of that kernel (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the
    captured launch).  Traffic grows with the rows processed, so a full launch is this ratio
    times its algorithmic bytes.  None when no capture of the kernel is on record."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            rec = json.load(f)[kernel]
        return (rec["dram_read_bytes"] + rec["dram_write_bytes"]) / rec["algorithmic_bytes"]
    except Exception:
        return None


def workload_string(name, w):
    """The one description of a workload both arms print."""
    return "%s: %d rows x %d %s columns per GPU, history %d ids, %s" % (
        name, w.rows, w.vocab, "bf16" if w.logits.dtype == torch.bfloat16 else "f32",
        0 if w.history is None else w.history.shape[1], WORKLOAD_NOTES.get(name, ""))


def load_oracle():
    """The CPU port of the reference sampler (oracle/): used here only as the timed CPU
    baseline and as the checker of a few rows, never on the measured GPU path."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib

    oracle_lib.lib()
    return oracle_lib


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed
    regions run (read-only queries)."""

    REASONS = {
        0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
        0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index):
        super().__init__(daemon=True)
        self.samples = []
        self.windows = []
        self.stop_flag = False
        self.ok = False
        self.max_mhz = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(0.001)

    def window(self, t0, t1):
        self.windows.append((t0, t1))

    def summary(self):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "note": "NVML unavailable"}
        inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in self.windows)]
        if not inside:  # a region shorter than one sampling period: take the nearest samples
            inside = self.samples[-3:]
        mask = 0
        for s in inside:
            mask |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if mask & bit]
        return {
            "sm_mhz": statistics.median([s[1] for s in inside]) if inside else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": reasons,
            "samples": len(inside),
        }


def dist_setup(gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


def max_over_ranks(x, world, device):
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(fn, steps, world, device, clocks=None):
    """Times exactly `steps` calls of fn with CUDA events on the launching stream, between
    a barrier + synchronize on both sides; returns the slowest rank's milliseconds per step."""
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    barrier(world)
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize(device)
    t1 = time.perf_counter()
    barrier(world)
    if clocks is not None:
        clocks.window(t0, t1)
    return max_over_ranks(start.elapsed_time(end) / steps, world, device)


def cpu_baseline(O, w, seconds=3.0):
    """Times the CPU port of the reference sampler with every host thread (one sampler state
    per row, rows handed out dynamically) on a bounded sample: whole passes over the
    workload's first rows, repeated until `seconds` of wall time have gone by."""
    if w.logits.dtype == torch.bfloat16:  # the CPU port takes bfloat16 rows as uint16 bit patterns
        logits = w.logits.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    else:
        logits = w.logits.cpu().numpy()
    hist = None if w.history is None else w.history.cpu().numpy()
    n = min(w.rows, 4096)
    first = O.sample_rows(logits[:n].copy(), w.params[:n], history=None if hist is None else hist[:n])  # warm-up
    passes, spent, used = 0, 0.0, int(first["threads"])
    while spent < seconds and passes < 200:
        work = logits[:n].copy()  # the penalty patches the rows in place: a fresh copy per pass
        t = time.perf_counter()
        out = O.sample_rows(work, w.params[:n], history=None if hist is None else hist[:n])
        spent += time.perf_counter() - t
        used = int(out["threads"])
        passes += 1
    return {
        "value": n * passes / spent, "unit": UNIT, "cores": used, "kind": "port",
        "sample": "%d passes over %d rows of the same workload, %.2f s of wall time on %d threads"
                  % (passes, n, spent, used),
    }, first["next"], n


def run_reference(args):
    """The reference arm: the CPU port of internal/logits/sampler.go on the host cores."""
    world, rank, _ = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), 0
    if rank != 0:
        return
    from mantle_b200 import workloads

    O = load_oracle()
    cores = O.lib().mantle_oracle_max_threads()
    w = workloads.make(args.workload, rows=args.rows, device="cpu")
    logits = w.logits.numpy()
    hist = None if w.history is None else w.history.numpy()
    n = w.rows  # a step is the whole batch, as on the GPU arm
    times = []
    used = cores
    for i in range(args.warmup + args.steps):
        work = logits[:n].copy()
        t = time.perf_counter()
        out = O.sample_rows(work, w.params[:n], history=None if hist is None else hist[:n])
        dt = time.perf_counter() - t
        used = int(out["threads"])
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = n / (ms / 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_string(args.workload, w), "rows_per_gpu": n, "vocab": w.vocab},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": used, "kind": "port",
                         "sample": "%d rows per step, %d steps" % (n, args.steps)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "C port of the reference's Go sampler (no Go toolchain on this image), all host threads",
    }
    print(json.dumps(line), flush=True)


def time_link(host_tensor, dev_tensor, world, device, copies=3):
    """GB/s of a bare pinned host-to-device cudaMemcpyAsync of the e2e leg's logits on this
    rank's stream (what the link and the host side deliver with nothing else in the way):
    (this rank, the slowest rank)."""
    def copy():
        dev_tensor.copy_(host_tensor, non_blocking=True)

    copy()
    torch.cuda.synchronize(device)
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    barrier(world)
    start.record()
    for _ in range(copies):
        copy()
    end.record()
    torch.cuda.synchronize(device)
    ms = start.elapsed_time(end) / copies
    nbytes = host_tensor.numel() * host_tensor.element_size()
    mine = nbytes / (ms / 1e3) / 1e9
    slowest = nbytes / (max_over_ranks(ms, world, device) / 1e3) / 1e9
    return mine, slowest


def device_resident_leg(sampler, w, tokens, steps, world, device, clocks):
    """A step of the batched decode loop through MantleBatchSampler: the logits are where the LM
    head left them, on the device; per step one parameter record per row goes up (it carries the
    row's uniform draw) and one token and one flag per row come back.  Histories live on the
    device and grow by a token per step."""
    H = 0 if w.history is None else w.history.shape[1]
    bs = sampler.BatchSampler(w.rows, w.vocab, 2 * max(H, int(w.params["repeat_last_n"].max()), 32), (), device=device)
    hist = None if w.history is None else w.history.cpu().numpy()
    for r in range(w.rows):
        p = w.params[r]
        cfg = sampler.SamplerConfig(temperature=0.0 if p["greedy"] else float(p["temperature"]), top_k=int(p["top_k"]),
                                    top_p=float(p["top_p"]), min_p=float(p["min_p"]),
                                    repeat_penalty=float(p["repeat_penalty"]), repeat_last_n=int(p["repeat_last_n"]))
        bs.set_row(r, cfg, () if hist is None else hist[r])
    uniforms = np.ascontiguousarray(w.params["uniform"], dtype=np.float64)
    stream = torch.cuda.current_stream(device)

    def step():
        bs.step_async(w.logits, uniforms)
        stream.synchronize()  # the caller reads the tokens after every step

    step()
    first, _, status = bs.results()
    # same logits, histories, parameters and uniforms as the headline launch: same tokens
    assert np.array_equal(first, tokens) and status == 0, "the batched decode step disagrees with mantleCudaSampleRows"
    for _ in range(2):
        step()
    n = max(3, min(steps, 10))
    ms = time_steps(step, n, world, device, clocks)
    bs.close()
    return {
        "value": w.rows * world / (ms / 1e3), "unit": UNIT, "ms_per_step": ms, "steps": n,
        "h2d_bytes_per_step": int(w.rows * 40), "d2h_bytes_per_step": int(w.rows * 8 + 4),
        "api": "mantleBatchSamplerStep: device logits, parameter records up, tokens and flags down",
    }


def strong_leg(sampler, w, p_dev, ms_full, steps, world, device):
    """The stated sweep of the throughput configuration: ONE batch of `w.rows` rows split
    rows / N per GPU (each rank times its share), against this run's own full-batch time."""
    n = w.rows // world
    plan = sampler.BatchPlan(w.logits[:n], p_dev[: n * 40], w.max_top_k,
                             history=None if w.history is None else w.history[:n], want_counts=False)
    for _ in range(3):
        plan.launch()
    ms = time_steps(plan.launch, steps, world, device)
    return {
        "rows_total": n * world, "rows_per_gpu": n, "ms_per_step": ms, "value": n * world / (ms / 1e3), "unit": UNIT,
        "ctas_per_row": plan.splits, "efficiency_vs_n1": (ms_full / world) / ms,
        "note": "efficiency = (this run's time for the whole batch on one GPU / N) / time for rows/N per GPU; "
                "the share of a GPU (%.0f MB) %s" % (n * w.bytes_per_row / 1e6,
                                                      "exceeds the L2" if n * w.bytes_per_row > 2 * 126e6 else "is L2-sized"),
    }


def time_events(fn, steps, device):
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize(device)
    return start.elapsed_time(end) / steps


def vocab_sharded_leg(args, world, rank, device, with_parts=True):
    """The vocabulary-sharded configuration: 1024 rows x 262 144 columns split evenly over the
    ranks; a step is mantleCudaSampleVocabSharded -- local shortlist kernel, ncclAllGather of the
    packed shortlists, merge kernel -- queued by one C call per rank."""
    import ctypes as C

    import torch.distributed as dist

    from mantle_b200 import nccl, sampler, sharded, workloads

    rows = 1024
    V = workloads.SPECS["vocab_sharded"]["vocab"]
    off, width = sharded.vocab_shard(V, world, rank)
    # every rank generates its own columns on the device from a seed of its own; history and
    # parameters come from one seed and are identical everywhere
    w = workloads.make("vocab_sharded", rows=rows, device=device, vocab=width, seed=workloads.BASE_SEED + 4000 + rank)
    ref = workloads.make("vocab_sharded", rows=rows, device="cpu", vocab=64, seed=workloads.BASE_SEED + 4000)
    hist = torch.randint(0, V, (rows, 512), generator=torch.Generator().manual_seed(7), dtype=torch.int32).to(device)
    p_dev = sampler.params_to_device(ref.params, device)
    comm = nccl.communicator_from_torch()
    plan = sharded.NcclVocabShardedPlan(comm, w.logits, p_dev, w.max_top_k, V, history=hist)
    for _ in range(max(args.warmup, 3)):
        plan.step()
    ms = time_steps(plan.step, args.steps, world, device)
    out = {
        "rows": rows, "vocab_total": V, "columns_per_gpu": width, "ms_per_step": ms, "value": rows / (ms / 1e3),
        "unit": UNIT, "scaling": "strong", "api": "mantleCudaSampleVocabSharded (one C call per rank and step)",
        "scan_gbs_per_gpu": None,
    }
    if with_parts:
        # the three pieces on their own, each in a loop of its own (so their sum need not be the step)
        lib, stream = plan.lib, C.c_void_p(torch.cuda.current_stream().cuda_stream)
        p = lambda t: C.c_void_p(t.data_ptr())
        scan = lambda: lib.mantleCudaSampleLocalTopK(C.byref(plan.local), plan.offset, V, p(plan.val), p(plan.idx),
                                                      p(plan.cnt), plan.k, stream)
        gather = lambda: dist.all_gather_into_tensor(plan.gathered, plan.block)
        merge = lambda: lib.mantleCudaSampleMergePacked(C.byref(plan.merge), world, p(plan.gathered), plan.k, stream)
        parts = {}
        for name, fn in (("scan_us", scan), ("allgather_us", gather), ("merge_us", merge)):
            for _ in range(3):
                fn()
            barrier(world)
            parts[name] = 1e3 * max_over_ranks(time_events(fn, args.steps, device), world, device)
        out.update(parts)
        out["scan_gbs_per_gpu"] = rows * (width * 4 + 4 * 512) / (parts["scan_us"] / 1e6) / 1e9
    # parity, outside the timed regions: the first 64 rows against the oracle on the whole row
    n_chk = 64
    shards = [torch.empty((n_chk, width), dtype=torch.float32, device=device) for _ in range(world)]
    dist.all_gather(shards, w.logits[:n_chk].contiguous())
    got = plan.out.next[:n_chk].cpu().numpy()
    if rank == 0:
        O = load_oracle()
        full = torch.cat(shards, dim=1).cpu().numpy()
        want = O.sample_rows(full, ref.params[:n_chk], history=hist[:n_chk].cpu().numpy())["next"]
        assert np.array_equal(got, want), "vocabulary-sharded tokens differ from the CPU port on the whole row"
        out["parity_rows_checked"] = n_chk
    torch.cuda.synchronize(device)
    barrier(world)
    comm.close()
    return out


def run_ours(args):
    from mantle_b200 import native, sampler, workloads

    native.load()  # raises if the CUDA library is missing: there is no other path
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the sampler has no CPU path")
    world, rank, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)

    if args.workload == "vocab_sharded":
        return run_vocab_sharded(args, world, rank, device)
    w = workloads.make(args.workload, rows=args.rows, device=device, seed=workloads.BASE_SEED + 3000 + rank)
    if args.top_k > 0:  # a side measurement of another shortlist length: the device arm only
        w.params["top_k"] = args.top_k
        w.max_top_k = min(args.top_k, w.vocab)
        args.no_e2e = args.no_cpu = True
    p_dev = sampler.params_to_device(w.params, device)
    post = bool(args.logit_scale or args.logit_softcap)
    if post:  # a side measurement of the fused head post-processing: the device arm only
        args.no_e2e = args.no_cpu = True
    plan = sampler.BatchPlan(w.logits, p_dev, w.max_top_k, history=w.history, want_counts=False, splits=args.splits,
                             logit_scale=args.logit_scale, logit_softcap=args.logit_softcap)
    step = plan.launch

    clocks = ClockSampler(local)
    clocks.start()

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize(device)
    ms = time_steps(step, args.steps, world, device, clocks)
    tokens = plan.out.next.cpu().numpy().copy()
    status = int(plan.out.status.item())

    # ---- end to end: pinned host buffers through the host-buffer C-ABI call -------------------
    e2e = None
    resident = None
    if not args.no_e2e:
        host_logits = torch.empty(w.logits.shape, dtype=w.logits.dtype, pin_memory=True)
        host_logits.copy_(w.logits)
        host_hist = None
        if w.history is not None:
            host_hist = torch.empty(w.history.shape, dtype=torch.int32, pin_memory=True)
            host_hist.copy_(w.history)
        hplan = sampler.HostBatchPlan(host_logits, w.params, w.max_top_k, history=host_hist, device=device,
                                      splits=args.splits)

        def e2e_step():
            hplan.launch()
            torch.cuda.current_stream().synchronize()  # the caller reads the tokens after every step

        for _ in range(3):
            e2e_step()
        e2e_steps = max(3, min(args.steps, 10))
        e2e_ms = time_steps(e2e_step, e2e_steps, world, device, clocks)
        assert np.array_equal(hplan.out.next.numpy(), tokens), "host-buffer path disagrees with the device path"
        h2d_bytes, d2h_bytes = int(hplan.h2d_bytes), int(hplan.d2h_bytes)
        del hplan
        # what the link alone delivers for the same bytes, right beside the number it explains
        scratch = torch.empty_like(w.logits)
        link_mine, link_slowest = time_link(host_logits, scratch, world, device)
        del scratch
        h2d = host_logits.numel() * host_logits.element_size()
        e2e = {
            "value": w.rows * world / (e2e_ms / 1e3), "unit": UNIT, "ms_per_step": e2e_ms, "steps": e2e_steps,
            "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
            "link_gbs": link_mine, "link_gbs_slowest_rank": link_slowest,
            "frac_of_link": (h2d / (e2e_ms / 1e3) / 1e9) / link_slowest,
            "api": "mantleCudaSampleRowsHost: pinned host logits, histories and parameters in, tokens out",
        }
        del host_logits
    if not args.no_e2e and w.max_top_k <= native.MAX_TOP_K:
        resident = device_resident_leg(sampler, w, tokens, args.steps, world, device, clocks)

    clocks.stop_flag = True
    clocks.join(timeout=2)

    # ---- the two multi-GPU configurations that are not the headline ---------------------------------
    strong = sharded_rec = None
    if world > 1 and args.workload == "throughput" and not post:
        strong = strong_leg(sampler, w, p_dev, ms, args.steps, world, device)
        sharded_rec = vocab_sharded_leg(args, world, rank, device)

    # ---- CPU baseline and a parity spot check (rank 0, one GPU only) --------------------------------
    cpu = None
    parity_rows = 0
    if rank == 0 and world == 1 and not args.no_cpu:
        O = load_oracle()
        cpu, cpu_tokens, n = cpu_baseline(O, w)
        assert np.array_equal(cpu_tokens, tokens[:n]), "GPU tokens differ from the CPU port on the sampled rows"
        parity_rows = n

    if rank == 0:
        peak, peak_kind = measured_peak()
        rows_total = w.rows * world
        kernel_bytes = w.rows * w.bytes_per_row  # one launch, one GPU
        achieved = kernel_bytes / (ms / 1e3) / 1e9
        kernel = plan.kernel_name
        ratio = dram_traffic_ratio(kernel) if args.workload == "throughput" and not post and not args.top_k else None
        line = {
            "metric": METRIC, "value": rows_total / (ms / 1e3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": workload_string(args.workload, w),
                "rows_per_gpu": w.rows, "vocab": w.vocab, "parallelism": "rows sharded over %d GPU(s), no collective" % world,
                "l2": ("inputs (%.2f GB per GPU) exceed the 126 MB L2, no flush needed" % (kernel_bytes / 1e9))
                      if kernel_bytes > 2 * 126e6 else
                      ("inputs (%.1f MB) fit the 126 MB L2 and are not flushed: an L2-resident timing" % (kernel_bytes / 1e6)),
                "ctas_per_row": plan.splits,
                **({"logit_scale": args.logit_scale, "logit_softcap": args.logit_softcap} if post else {}),
                **({"top_k_override": args.top_k} if args.top_k > 0 else {}),
            },
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None if ratio is None else ratio * kernel_bytes,
                "traffic_source": None if ratio is None else "ncu capture of a smaller launch, scaled by rows",
                "peak_kind": "of %s" % peak_kind, "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                "kernel": kernel, "algorithmic_bytes_per_launch": kernel_bytes,
                "bytes_per_row": w.bytes_per_row,
            },
            "cpu_baseline": cpu,
            "e2e": e2e,
            "e2e_device_resident": resident,
            "gpu_launches": args.steps * plan.kernels_per_launch,
            "clocks": clocks.summary(),
            "status_word": status,
            "parity_rows_checked": parity_rows,
        }
        if strong is not None:
            line["strong"] = strong
            line["vocab_sharded"] = sharded_rec
            line["vocab_sharded_parity_rows"] = sharded_rec.get("parity_rows_checked", 0)
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def run_vocab_sharded(args, world, rank, device):
    """`--workload vocab_sharded`: the vocabulary-sharded configuration as a line of its own."""
    import torch.distributed as dist

    if world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    rec = vocab_sharded_leg(args, world, rank, device)
    if rank == 0:
        peak, peak_kind = measured_peak()
        line = {
            "metric": METRIC.replace("151936", "262144 (vocabulary-sharded)"), "value": rec["value"], "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "vocab_sharded: %d rows x 262144 f32 columns over %d GPU(s) (%d columns each), "
                                   "top_k 50 top_p 0.95 temp 0.7 repeat_penalty 1.15, history 512 ids; local top-k, "
                                   "one NCCL all-gather of the packed shortlists, merge"
                                   % (rec["rows"], world, rec["columns_per_gpu"]),
                       "l2": "per-GPU inputs of %.0f MB; L2-resident below 126 MB"
                             % (rec["rows"] * (rec["columns_per_gpu"] * 4 + 2048) / 1e6)},
            "roofline": {"bound": "hbm", "achieved": rec.get("scan_gbs_per_gpu"), "peak": peak, "unit": "GB/s",
                         "frac": None if not rec.get("scan_gbs_per_gpu") else rec["scan_gbs_per_gpu"] / peak,
                         "traffic": None, "peak_kind": "of %s" % peak_kind,
                         "note": "the local shortlist kernel alone; the step is latency-bound: two launches and one collective"},
            "vocab_sharded": rec,
            "gpu_launches": args.steps * 2,
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="throughput")
    ap.add_argument("--rows", type=int, default=4096, help="rows per GPU")
    ap.add_argument("--splits", type=int, default=0, help="CTAs per row (0: library's choice)")
    ap.add_argument("--logit-scale", type=float, default=0.0, help="fuse the model head's multiplier (side measurement)")
    ap.add_argument("--logit-softcap", type=float, default=0.0, help="fuse the model head's soft cap (side measurement)")
    ap.add_argument("--top-k", type=int, default=0, help="override every row's top_k (side measurement)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
