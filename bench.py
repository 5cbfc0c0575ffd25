#!/usr/bin/env python
"""Benchmark of the decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one decode-attention call over the whole batch.  The headline workload is the
GQA bf16 variable-length batch (256 sequences per GPU, 32/8 heads, dim 128, lengths uniform in
[512, 4096]); with N GPUs the global batch is 256*N sequences cut into per-rank groups (no
collective on the data path; weak scaling).  `value` is KV-cache GB/s = algorithmic KV bytes of
all ranks / (max-over-ranks device time per step), inputs resident in HBM.  `e2e` is the same
metric through the host-buffer C-ABI call (pinned host tensors; H2D of q, k, v, cu_seq_k and D2H of
o inside the timed region).  `--impl reference` times the reference project's own CPU attention
(oracle/_ref, compiled from its tester.h) on a bounded sample of the same workload.
Prints ONE JSON line on stdout.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from decoding_attention_b200 import sharded, synth  # noqa: E402

METRIC = "decode_attention_kv_read_bandwidth"
UNIT = "GB/s"
SEQS_PER_GPU = 256
L2_BYTES = 126 * 1024 * 1024


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ["clocks.sm", "clocks.max.sm", "power.draw", "clocks_event_reasons.hw_slowdown",
              "clocks_event_reasons.hw_thermal_slowdown", "clocks_event_reasons.sw_thermal_slowdown",
              "clocks_event_reasons.sw_power_cap"]

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + ",".join(self.FIELDS),
                 "--format=csv,noheader,nounits", "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) != len(self.FIELDS):
                continue
            try:
                sm.append(float(f[0]))
                smax.append(float(f[1]))
                power.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(self.FIELDS[3:], f[3:]):
                if val.lower().startswith("active"):
                    reasons.add(name.split(".")[-1])
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------

def make_call(cabi, w, q, k, v, cu, o, **kw):
    args = cabi.make_args(q, k, v, o, cu, max(w.max_seq_k, 1), w.dim_v, is_alibi=w.is_alibi,
                          stream=torch.cuda.current_stream().cuda_stream, **kw)
    return args


def time_resident(cabi, args, steps, warmup, barrier, flush=None):
    """K back-to-back steps between two events (after W warm-ups), exactly as a caller would issue them;
    then, outside the timed region, the same K steps again with the profiling hook, which brackets the
    main (key-streaming) kernel of every call with its own events.  (The hook's event records sit between
    the kernels of a call and keep them from overlapping, so it must not run inside the timed region.)
    Returns (seconds per step, seconds per main-kernel launch, launches in the timed region)."""
    for _ in range(warmup):
        cabi.decode_fwd(args)
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    l0 = cabi.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        cabi.decode_fwd(args)
    t1.record()
    torch.cuda.synchronize()
    barrier()
    launches = cabi.launch_count() - l0
    total = t0.elapsed_time(t1) * 1e-3

    # (20 calls are enough for the mean; a long second pass only pushes the GPU into its power cap)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(min(steps, 20))]
    for a, b in ev:  # create the underlying events
        a.record()
        b.record()
    torch.cuda.synchronize()
    for a, b in ev:
        cabi.set_profile_events(a, b)
        cabi.decode_fwd(args)
    cabi.set_profile_events(None, None)
    torch.cuda.synchronize()
    kern = statistics.mean(a.elapsed_time(b) for a, b in ev) * 1e-3
    return total / steps, kern, launches


def time_flushed(cabi, args, iters, flush_buf, spread=None, clean_buf=None):
    """Per-call events with an L2 flush between calls (for working sets that fit in L2): 256 MB are rewritten,
    which leaves L2 full of the flush's dirty lines, so that the timed call's first 126 MB of reads also pay
    for their write-back (measured: +4 us on a 134 MB call).  With `clean_buf` a second 256 MB buffer is then
    read, which evicts the dirty lines: the call starts on a cold L2 that owes DRAM nothing.
    Returns the median; `spread`, if given, receives the 10th and 90th percentiles (seconds)."""
    times = []
    for i in range(iters + 3):
        flush_buf.add_(1)
        if clean_buf is not None:
            clean_buf.sum()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        cabi.decode_fwd(args)
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(a.elapsed_time(b) * 1e-3)
    times.sort()
    if spread is not None:
        spread[:] = [times[len(times) // 10], times[(len(times) * 9) // 10]]
    return statistics.median(times)


def time_e2e(cabi, w, host, steps, warmup, barrier):
    q, k, v, cu, o = host
    args = cabi.make_args(q, k, v, o, cu, max(w.max_seq_k, 1), w.dim_v, is_alibi=w.is_alibi, packed=True,
                          stream=torch.cuda.current_stream().cuda_stream)
    for _ in range(warmup):
        cabi.decode_fwd_host(args)
    torch.cuda.synchronize()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        cabi.decode_fwd_host(args)
    t1.record()
    torch.cuda.synchronize()
    barrier()
    h2d = sum(t.numel() * t.element_size() for t in (q, k, v, cu) if t is not None)
    d2h = o.numel() * o.element_size()
    return t0.elapsed_time(t1) * 1e-3 / steps, h2d, d2h


def cpu_reference_sample(w, budget_s, threads):
    """The reference's CPU attention (oracle/_ref) on the first sequences of the workload, one Tester
    instance per sequence (its harness needs equal lengths inside a batch), spread over `threads`
    host threads.  Falls back to the oracle restatement when oracle/_ref is not built."""
    from oracle import attn_oracle
    kind = "reference" if attn_oracle.ref_available() else "port"

    def run_seq(b):
        q, k, v, cu = w.make("cpu", seqs=[b])
        t = time.perf_counter()
        if kind == "reference":
            attn_oracle.ref_attn_cpu(q, k, v, w.seq_lens[b], dim_v=w.dim_v, is_alibi=w.is_alibi, threads=1)
        else:
            attn_oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v, is_alibi=w.is_alibi, threads=1)
        return time.perf_counter() - t

    t_one = run_seq(0)
    per_key = t_one / max(w.seq_lens[0], 1)
    n, keys = 0, 0
    while n < w.batch and (keys * per_key / threads < budget_s or n < threads):
        keys += w.seq_lens[n]
        n += 1
    seqs = list(range(n))
    data = [w.make("cpu", seqs=[b]) for b in seqs]  # generation is not part of the timed region

    def run_prepared(i):
        q, k, v, cu = data[i]
        if kind == "reference":
            attn_oracle.ref_attn_cpu(q, k, v, w.seq_lens[i], dim_v=w.dim_v, is_alibi=w.is_alibi, threads=1)
        else:
            attn_oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v, is_alibi=w.is_alibi, threads=1)

    def timed():
        t = time.perf_counter()
        with ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(run_prepared, range(n)))
        return time.perf_counter() - t

    kv = w.kv_bytes(seq_lens=[w.seq_lens[b] for b in seqs])
    return kind, n, kv, timed


def parity_vs_oracle(w, o, seqs):
    """Max |out - oracle| over the sequences `seqs` of workload `w` (oracle inputs regenerated on the CPU from the
    same seed; `o` holds one output row per entry of `seqs`, in that order).  Checker only: runs after the timed
    regions."""
    from oracle import attn_oracle
    worst, bad = 0.0, 0
    for i, b in enumerate(seqs):
        q, k, v, cu = w.make("cpu", seqs=[b])
        expect = attn_oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v, is_alibi=w.is_alibi).float()
        err = (o[i:i + 1].float().cpu() - expect).abs()
        worst = max(worst, err.max().item())
        bad += int((err > 2e-3 + 1e-2 * expect.abs()).sum().item())
    return worst, bad


def run_ours(opt):
    from decoding_attention_b200 import cabi
    cabi.lib()  # fail loudly if the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if opt.gpus != world:
        log(f"note: --gpus {opt.gpus} but WORLD_SIZE {world}; using WORLD_SIZE")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        # NCCL prints its version banner on stdout when NCCL_DEBUG is set; stdout carries the JSON line only.
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def sum_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t.item()

    hbm_peak, peak_kind = load_peaks()
    w = synth.config_gqa_varlen(batch=opt.seqs * world)
    mine = sharded.partition_batch(w.seq_lens, world)[rank]
    my_lens = [w.seq_lens[b] for b in mine]
    q, k, v, cu = w.make(dev, seqs=mine)
    o = torch.empty(len(mine), w.head_q, w.dim_v, dtype=w.dtype, device=dev)
    local = synth.Workload(w.name, w.dtype, w.head_q, w.head_k, w.dim, w.dim_v, my_lens, dist=w.dist, scale=w.scale)
    args = make_call(cabi, local, q, k, v, cu, o)
    my_bytes = local.kv_bytes()
    total_bytes = sum_over_ranks(my_bytes)

    sampler = ClockSampler(local_rank)
    sampler.start()
    sec, kern_sec, launches = time_resident(cabi, args, opt.steps, opt.warmup, barrier)
    clocks = sampler.stop()
    sec_max = max_over_ranks(sec)
    status = cabi.device_status()
    assert status == cabi.DA_OK, "a kernel reported a timed-out wait"

    # spread: further blocks of K steps each (same protocol), so that one block's dip can be told from noise
    block_ms = [sec_max * 1e3]
    for _ in range(4):
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(opt.steps):
            cabi.decode_fwd(args)
        t1.record()
        torch.cuda.synchronize()
        block_ms.append(max_over_ranks(t0.elapsed_time(t1) / opt.steps))
    block_ms_sorted = sorted(block_ms)
    # sustained: at least a second of back-to-back calls, clocks sampled meanwhile (the power cap shows here)
    n_sus = max(opt.steps, int(1.0 / max(sec, 1e-6)))
    sus_sampler = ClockSampler(local_rank)
    sus_sampler.start()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(n_sus):
        cabi.decode_fwd(args)
    t1.record()
    torch.cuda.synchronize()
    sus_clocks = sus_sampler.stop()
    sus_sec = max_over_ranks(t0.elapsed_time(t1) * 1e-3 / n_sus)

    # parity of this rank's results against the CPU oracle (a bounded subset when several ranks share the host)
    torch.cuda.synchronize()
    n_check = len(mine) if world == 1 else min(len(mine), 32)
    worst, bad = parity_vs_oracle(w, o[:n_check], mine[:n_check])
    worst, bad = max_over_ranks(worst), sum_over_ranks(bad)

    # end to end through the host-buffer entry point
    e2e_steps = max(1, min(opt.steps, 10))
    if opt.no_e2e:
        e2e_sec, h2d, d2h, e2e_ok = float("nan"), 0, 0, False
    else:
        host = [t.cpu().pin_memory() if t is not None else None for t in (q, k, v, cu)]
        host.append(torch.empty_like(o, device="cpu").pin_memory())
        e2e_sec, h2d, d2h = time_e2e(cabi, local, host, e2e_steps, min(opt.warmup, 3), barrier)
        e2e_sec = max_over_ranks(e2e_sec)
        e2e_ok = torch.equal(host[4].to(dev), o)

    out = {
        "metric": METRIC, "value": round(total_bytes / sec_max / 1e9, 2), "unit": UNIT, "n_gpus": world,
        "steps": opt.steps, "warmup": opt.warmup, "ms_per_step": round(sec_max * 1e3, 4),
        "us_per_call": round(sec_max * 1e6, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 in/out, fp32 accumulate", "data": "synthetic (seeded, decoding_attention_b200.synth)",
        "config": {"workload": "GQA decode bf16, batch-sharded: %d sequences per GPU, head_q 32, head_k 8, "
                               "dim 128, seq_k ~ U[512,4096], N(0,1)*0.5, ALiBi off (BASELINE config 2)" % opt.seqs,
                   "sequences": w.batch, "total_keys": w.total_k, "kv_bytes": int(total_bytes),
                   "l2": "inputs (%.2f GB per GPU) larger than the 126 MB L2" % (my_bytes / 1e9),
                   "num_splits": cabi.num_splits(args)},
        "clocks": clocks,
        "blocks": {"n": len(block_ms), "steps_each": opt.steps, "median_ms": round(statistics.median(block_ms), 4),
                   "min_ms": round(block_ms_sorted[0], 4), "max_ms": round(block_ms_sorted[-1], 4),
                   "note": "the first block is the one `value` reports"},
        "sustained": {"steps": n_sus, "ms_per_step": round(sus_sec * 1e3, 4),
                      "value": round(total_bytes / sus_sec / 1e9, 2), "unit": UNIT, "clocks": sus_clocks,
                      "ms_x_sm_ghz": round(sus_sec * 1e3 * (sus_clocks.get("sm_mhz") or 0) / 1e3, 4)},
        "parity": {"max_abs_err_vs_oracle": worst, "elements_outside_tolerance": int(bad),
                   "tolerance": "2e-3 + 1e-2 |oracle|", "sequences_checked_per_rank": n_check,
                   "oracle": "CPU restatement of the reference's attn_cpu, same seeded inputs"},
        "e2e": {"value": round(total_bytes / e2e_sec / 1e9, 3), "unit": UNIT, "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_sec * 1e3, 3), "steps": e2e_steps,
                "matches_resident_result": bool(e2e_ok),
                "call": "da_decode_fwd_host (pinned host q, k, v, cu_seq_k -> device, kernels, o -> host)"},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": round(my_bytes / kern_sec / 1e9, 2), "peak": hbm_peak,
                     "unit": "GB/s", "frac": round(my_bytes / kern_sec / 1e9 / hbm_peak, 4), "of": peak_kind,
                     "frac_of_nominal_8000": round(my_bytes / kern_sec / 1e9 / 8000.0, 4),
                     "kernel": "da_split_kernel (GQA, dim 128, 4 heads per CTA)",
                     "kernel_us": round(kern_sec * 1e6, 2), "algorithmic_bytes": int(my_bytes),
                     "traffic": opt.traffic},
    }

    if rank == 0 and world == 1 and not opt.no_cpu:
        threads = os.cpu_count() or 1
        kind, n, kv, timed = cpu_reference_sample(w, 12.0, threads)
        t = timed()
        out["cpu_baseline"] = {"value": round(kv / t / 1e9, 4), "unit": UNIT, "cores": threads, "kind": kind,
                               "seconds": round(t, 2),
                               "sample": f"first {n} of {w.batch} sequences ({kv / 1e6:.0f} MB of KV), one "
                                         f"single-threaded attn_cpu per sequence over {threads} host threads"}
    if not opt.no_extra:
        try:
            out["other_configs"] = other_configs(cabi, dev, world, rank, barrier, max_over_ranks, hbm_peak)
        except Exception as e:  # the headline line must survive a failure in the extras
            out["other_configs"] = {"error": repr(e)}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(out), flush=True)


def other_configs(cabi, dev, world, rank, barrier, max_over_ranks, hbm_peak):
    """The remaining BASELINE configurations: 1-GPU numbers (rank 0 of a 1-GPU run) and the key-range
    sharded long sequence at every N."""
    res = {}
    flush = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=dev)
    clean = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=dev)

    def one(name, w, flushed):
        q, k, v, cu = w.make(dev)
        o = torch.empty(w.batch, w.head_q, w.dim_v, dtype=w.dtype, device=dev)
        args = make_call(cabi, w, q, k, v, cu, o)
        for _ in range(3):
            cabi.decode_fwd(args)
        torch.cuda.synchronize()
        spread = []
        sec_dirty = None
        if flushed:
            sec = time_flushed(cabi, args, 50, flush, spread, clean)
            sec_dirty = time_flushed(cabi, args, 50, flush)
        else:
            sec, _, _ = time_resident(cabi, args, 20, 3, lambda: None)
        res[name] = {"us_per_call": round(sec * 1e6, 2), "kv_GBps": round(w.kv_bytes() / sec / 1e9, 1),
                     "frac_of_hbm_peak": round(w.kv_bytes() / sec / 1e9 / hbm_peak, 4),
                     "ref_tflops": round(w.ref_flops() / sec / 1e12, 3), "num_splits": cabi.num_splits(args),
                     "timing": "median of 50 calls; between calls 256 MB are written and a second 256 MB read "
                               "(cold L2 without the flush's dirty lines)" if flushed else
                               "20 back-to-back calls, inputs larger than L2"}
        if spread:
            res[name]["us_p10_p90"] = [round(x * 1e6, 2) for x in spread]
        if sec_dirty is not None:  # the write-only flush: the call also pays for the write-back of the flush's lines
            res[name]["us_per_call_after_write_only_flush"] = round(sec_dirty * 1e6, 2)
        del q, k, v, o

    def paged(name, w, page):
        """The same workload read through a block table over a shuffled pool of `page`-key pages
        (device-side scatter of the packed cache; the call is what is timed)."""
        q, k, v, cu = w.make(dev)
        blocks = [(n + page - 1) // page for n in w.seq_lens]
        n_pages = sum(blocks)
        order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1234)).to(torch.int32)
        table = torch.zeros(w.batch, max(blocks), dtype=torch.int32)
        rows = torch.empty(w.total_k, dtype=torch.int64)  # pool row of every packed row
        nxt = 0
        for b, n in enumerate(w.seq_lens):
            pages = order[nxt:nxt + blocks[b]]
            nxt += blocks[b]
            table[b, :blocks[b]] = pages
            j = torch.arange(n)
            rows[w.cu[b]:w.cu[b] + n] = pages[j // page].to(torch.int64) * page + j % page
        rows = rows.to(dev)
        k_pool = torch.zeros(n_pages * page, w.head_k, w.dim, dtype=w.dtype, device=dev)
        k_pool[rows] = k
        v_pool = None
        if v is not None:
            v_pool = torch.zeros(n_pages * page, w.head_k, w.dim_v, dtype=w.dtype, device=dev)
            v_pool[rows] = v
        del k, v, rows
        o = torch.empty(w.batch, w.head_q, w.dim_v, dtype=w.dtype, device=dev)
        args = cabi.make_args(q, k_pool, v_pool, o, cu, w.max_seq_k, w.dim_v, is_alibi=w.is_alibi,
                              stream=torch.cuda.current_stream().cuda_stream, block_table=table.to(dev), page_size=page)
        sec, _, _ = time_resident(cabi, args, 20, 3, lambda: None)
        res[name] = {"us_per_call": round(sec * 1e6, 2), "kv_GBps": round(w.kv_bytes() / sec / 1e9, 1),
                     "frac_of_hbm_peak": round(w.kv_bytes() / sec / 1e9 / hbm_peak, 4), "page_size": page,
                     "num_splits": cabi.num_splits(args), "timing": "20 back-to-back calls, inputs larger than L2"}

    if world == 1:
        paged("gqa_bf16_b256_varlen_paged64", synth.config_gqa_varlen(), 64)
        paged("gqa_bf16_b256_varlen_paged16", synth.config_gqa_varlen(), 16)
        paged("mla_bf16_b128_sk4096_paged64", synth.config_mla(batch=128), 64)
        paged("mla_bf16_b128_sk4096_paged16", synth.config_mla(batch=128), 16)
        one("mha_fp16_b4_sk1024", synth.config_mha_small(), True)
        one("mqa_alibi_fp16_b128_sk2048", synth.config_mqa_alibi(), True)
        for b in (1, 8, 32, 128):
            one(f"mla_bf16_b{b}_sk4096", synth.config_mla(batch=b), b <= 8)
        # the same latent cache with 16 query heads: one GPU's share of the 128 heads under 8-way tensor parallelism
        one("mla_bf16_h16_b128_sk4096", synth.Workload("mla_h16", torch.bfloat16, 16, 1, 576, 512, [4096] * 128,
                                                       dist="normal", scale=0.3, mla=True), False)

    # BASELINE config 2 as stated: 256 sequences IN TOTAL, cut into per-rank groups (strong scaling; the headline
    # keeps 256 per GPU).  No collective on the data path; time = max over ranks.
    w2 = synth.config_gqa_varlen()
    mine2 = sharded.partition_batch(w2.seq_lens, world)[rank]
    q, k, v, cu = w2.make(dev, seqs=mine2)
    o2 = torch.empty(len(mine2), w2.head_q, w2.dim_v, dtype=w2.dtype, device=dev)
    local2 = synth.Workload(w2.name, w2.dtype, w2.head_q, w2.head_k, w2.dim, w2.dim_v, [w2.seq_lens[b] for b in mine2],
                            dist=w2.dist, scale=w2.scale)
    a2 = make_call(cabi, local2, q, k, v, cu, o2)
    sec2, _, _ = time_resident(cabi, a2, 20, 3, barrier, flush if world >= 4 else None)
    sec2 = max_over_ranks(sec2)
    torch.cuda.synchronize()
    n_chk = min(len(mine2), 16)
    worst2, bad2 = parity_vs_oracle(w2, o2[:n_chk], mine2[:n_chk])
    res["gqa_bf16_b256_total_batch_sharded"] = {
        "n_gpus": world, "sequences_per_rank": len(mine2), "us_per_call": round(sec2 * 1e6, 2),
        "kv_GBps": round(w2.kv_bytes() / sec2 / 1e9, 1),
        "frac_of_hbm_peak_per_gpu": round(w2.kv_bytes() / world / sec2 / 1e9 / hbm_peak, 4), "scaling": "strong",
        "timing": "20 back-to-back calls, max over ranks",
        "parity": {"max_abs_err_vs_oracle": max_over_ranks(worst2), "elements_outside_tolerance": int(bad2),
                   "sequences_checked_per_rank": n_chk}}
    del q, k, v, o2

    # key-range sharded long sequence (strong scaling: 131072 keys in total at every N)
    w = synth.config_long_mha()
    lo, hi = sharded.key_range(w.seq_lens[0], rank, world)
    q, k, v, cu = w.make(dev, key_range=(lo, hi))
    fused = os.environ.get("DA_SHARD_EXCHANGE", "fused") != "nccl"
    dec = sharded.KeyRangeShardedDecoder(1, w.head_q, w.dim_v, w.dtype, dev, fused=fused)
    off = torch.tensor([lo], dtype=torch.int32, device=dev)
    tot = torch.tensor([w.seq_lens[0]], dtype=torch.int32, device=dev)
    for _ in range(5):
        dec.step(q, k, v, cu, hi - lo, kv_pos_offset=off, kv_total_len=tot)
    torch.cuda.synchronize()
    barrier()
    steps = 50
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        dec.step(q, k, v, cu, hi - lo, kv_pos_offset=off, kv_total_len=tot)
    t1.record()
    torch.cuda.synchronize()
    barrier()
    sec = max_over_ranks(t0.elapsed_time(t1) * 1e-3 / steps)

    # Where a step's time goes, measured apart from the timed region above: the local call alone (attention kernel
    # + split merge into the record), then the exchange + merge alone on records that are already there.
    def timed(fn, n=30):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e-3 / n

    local_sec = timed(lambda: dec.local_partial(q, k, v, cu, hi - lo, False, off, tot))
    if fused:
        xchg_sec = timed(dec.exchange_merge)
    else:
        xchg_sec = timed(lambda: (dec.exchange(), dec.merge()))
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
    for a, b in ev:
        a.record()
        b.record()
    torch.cuda.synchronize()
    for a, b in ev:
        cabi.set_profile_events(a, b)
        dec.local_partial(q, k, v, cu, hi - lo, False, off, tot)
    cabi.set_profile_events(None, None)
    torch.cuda.synchronize()
    kern_sec = statistics.mean(a.elapsed_time(b) for a, b in ev) * 1e-3
    local_all = [max_over_ranks(local_sec), -max_over_ranks(-local_sec)]

    # parity: every rank's merged result against the oracle on the UNSHARDED sequence, and rank-to-rank equality
    dec.step(q, k, v, cu, hi - lo, kv_pos_offset=off, kv_total_len=tot)
    torch.cuda.synchronize()
    worst5, bad5 = parity_vs_oracle(w, dec.out, [0]) if rank == 0 else (0.0, 0)
    same = True
    if world > 1:
        import torch.distributed as dist
        ref = dec.out.clone()
        dist.broadcast(ref, src=0)
        same = bool(torch.equal(ref, dec.out))
        flag = torch.tensor([1.0 if same else 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        same = bool(flag.item() > 0.5)
        worst5 = max_over_ranks(worst5)
    res["mha_bf16_b1_sk131072_key_range_sharded"] = {
        "n_gpus": world, "us_per_call": round(sec * 1e6, 2), "kv_GBps": round(w.kv_bytes() / sec / 1e9, 1),
        "frac_of_hbm_peak_per_gpu": round(w.kv_bytes() / world / sec / 1e9 / hbm_peak, 4), "scaling": "strong",
        "breakdown_us": {"attention_kernel": round(kern_sec * 1e6, 2),
                         "local_call_slowest_rank": round(local_all[0] * 1e6, 2),
                         "local_call_fastest_rank": round(local_all[1] * 1e6, 2),
                         "exchange_and_merge_alone": round(max_over_ranks(xchg_sec) * 1e6, 2),
                         "hbm_time_of_the_shard": round(w.kv_bytes() / world / hbm_peak / 1e3, 2),
                         "note": "each leg timed alone over 30 back-to-back calls; in a step they overlap through "
                                 "programmatic dependent launches"},
        "parity": {"max_abs_err_vs_oracle": worst5, "elements_outside_tolerance": int(bad5),
                   "ranks_bit_equal": same, "oracle": "attn_cpu on the unsharded 131072-key sequence"},
        "steps": ("local partial (o fp32, lse) -> one kernel: peer stores of the %d-byte record + flags, bounded wait, "
                  "LSE merge" if fused else
                  "local partial (o fp32, lse) -> NCCL all-gather of %d-byte records -> on-device LSE merge") % (
            dec.rec.numel() * 4)}
    return res


# ------------------------------------------------------------------------------------------------
# reference arm
# ------------------------------------------------------------------------------------------------

def run_reference(opt):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    w = synth.config_gqa_varlen(batch=opt.seqs * world)
    budget = max(0.5, min(4.0, 150.0 / (opt.steps + opt.warmup)))
    kind, n, kv, timed = cpu_reference_sample(w, budget, threads)
    for _ in range(opt.warmup):
        timed()
    t = time.perf_counter()
    for _ in range(opt.steps):
        timed()
    sec = (time.perf_counter() - t) / opt.steps
    val = round(kv / sec / 1e9, 4)
    sample = (f"first {n} of {w.batch} sequences ({kv / 1e6:.0f} MB of KV) per step, one single-threaded attn_cpu "
              f"(the reference's csrc/common/tester.h:133-259, compiled unmodified) per sequence over {threads} "
              "host threads")
    out = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": world, "steps": opt.steps,
           "warmup": opt.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16 in/out, fp32 accumulate", "data": "synthetic (seeded)",
           "config": {"workload": "GQA decode bf16, batch-sharded: 256 sequences per GPU, head_q 32, head_k 8, "
                                  "dim 128, seq_k ~ U[512,4096], N(0,1)*0.5, ALiBi off (BASELINE config 2)",
                      "sequences": w.batch, "total_keys": w.total_k},
           "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
           "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out), flush=True)


def run_profile_config(opt):
    """A few calls of one configuration, nothing else: the command line that ncu captures wrap."""
    from decoding_attention_b200 import cabi
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    make = synth.CONFIGS[opt.profile_config]
    if opt.profile_batch is None:
        w = make()
    elif opt.profile_config == "long_mha":
        w = make(seq_k=opt.profile_batch)
    elif opt.profile_config == "mha_small":
        w = make()
    else:
        w = make(batch=opt.profile_batch)
    q, k, v, cu = w.make(dev)
    o = torch.empty(w.batch, w.head_q, w.dim_v, dtype=w.dtype, device=dev)
    args = make_call(cabi, w, q, k, v, cu, o)
    sec, kern, launches = time_resident(cabi, args, opt.steps, opt.warmup, lambda: None)
    print(json.dumps({"config": w.name, "kv_bytes": w.kv_bytes(), "us_per_call": round(sec * 1e6, 2),
                      "main_kernel_us": round(kern * 1e6, 2), "kv_GBps": round(w.kv_bytes() / sec / 1e9, 1),
                      "num_splits": cabi.num_splits(args), "launches": int(launches)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqs", type=int, default=SEQS_PER_GPU,
                    help="sequences per GPU (256 = the benchmark workload; smaller values are for profiler captures)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the other BASELINE configurations")
    ap.add_argument("--profile-config", default=None, choices=sorted(synth.CONFIGS),
                    help="run only this BASELINE configuration for --steps calls on one GPU (for ncu captures)")
    ap.add_argument("--profile-batch", type=int, default=None, help="batch (or seq_k for long_mha) of that run")
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch of the dominant kernel from an ncu capture")
    opt = ap.parse_args()
    opt.warmup = max(opt.warmup, 3)
    if opt.traffic is None and opt.seqs == SEQS_PER_GPU:
        # DRAM bytes of one da_split_kernel launch, from an ncu capture of the 32-sequence case (291.27 MB read
        # for 290.94 MB of KV: x 1.0011, which grows with the keys read) plus the 2.1 MB of output rows the
        # unsplit full launch writes (the small case runs split and also writes partials, which this launch does not).
        opt.traffic = 2.4313e9
    if opt.profile_config:
        run_profile_config(opt)
    elif opt.impl == "reference":
        run_reference(opt)
    else:
        run_ours(opt)


if __name__ == "__main__":
    main()
