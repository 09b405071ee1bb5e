"""Decode-throughput benchmark of the B200 token loop (and of the CPU oracle beside it).

Workload ("c2"): Qwen3-0.6B architecture, bf16, random-init weights N(0, 0.02) from seed 0,
batch 64, prompt lengths uniform in [512, 2048] from seed 2 with token ids uniform over the
vocabulary, every 4 requests sharing a 256-token prefix, paged KV cache with page size 16, greedy
decode.  A "step" is one decode step of the whole batch: every per-token quantity derived on the
device, 28 layers, lm_head, argmax, token write-back.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  `value` is decode tokens/s with the steps enqueued back to back (device
time, CUDA events); `e2e` is the same loop driven the way a scheduler drives it — per step the
host arrays go through the C ABI from host memory, the step's metadata is copied host-to-device
from pinned memory and the sampled tokens are copied device-to-host and waited for.  With
--gpus N > 1 (launched under torchrun) every rank runs an independent replica of the workload
(the 0.6B model does not shard); the job's time is the max over ranks.

The K timed steps are repeated from the same state (re-warmed each time) until at least a second
has been timed, and the median repeat is reported, so that the clock samples taken beside it mean
something.  After the headline the same ranks run workload "c4" (Llama-3-8B, tensor parallel over
all N ranks, the fused all-reduce kernels on the data path) and attach it as the `tp` key: that is
the part of the path that shards, and the replicas of the headline cannot show it.

Other workloads (not the headline metric): --context N gives every prompt N tokens (the
"batch 64 / 2048-token context" point); --workload c3 is the prefill-heavy mixed case (8 prompts
of 4096 tokens prefilled in chunks, alternating with sampled decode steps of 56 running requests:
prefill tokens/s, decode ms/step, fraction of the tensor-pipe rate); --workload c4 is Llama-3-8B under tensor parallelism and
--workload c5 Qwen3-30B-A3B under expert parallelism + attention TP over the N ranks (strong
scaling, weights drawn on the device); --eager / --profile-region / --profile-prefill shape a run
for a profiler's launch list.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode tokens/s at bs=64 (Qwen3-0.6B, ctx 512-2048 + generated, page 16)"
PAGE_SIZE = 16
BATCH = 64
PROMPT_LO, PROMPT_HI = 512, 2048
SHARED_PREFIX = 256
MAX_EXTEND_TOKENS = 8192


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def dram_traffic_ratio(kernel: str):
    """DRAM bytes per algorithmic byte of a kernel, from the table of ncu captures kept in
    profiles/dram_traffic_ratios.md (None when the kernel has no row)."""
    p = ROOT / "profiles" / "dram_traffic_ratios.md"
    if not p.exists():
        return None
    for line in p.read_text().splitlines():
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) >= 4 and cells[0] == kernel:
            try:
                return float(cells[3])
            except ValueError:
                return None
    return None


def workload_config(world: int, context: int = 0):
    """The `config` object of the JSON line: the same for this arm and for --impl reference."""
    return {"workload": "c2: Qwen3-0.6B decode, batch 64, prompts %s seed 2, 256-token shared prefix per 4 "
                        "requests, page size 16, greedy" % ("of %d tokens" % context if context else "U[512,2048]"),
            "l2": "inputs larger than L2: every step streams about 10 GB of K/V and 1.19 GB of weights",
            "parallelism": "replicas" if world > 1 else "single GPU"}


def make_prompts(vocab: int, fixed_len: int = 0):
    """Seed 2: lengths uniform in [512, 2048] (or all ``fixed_len``), ids uniform over the
    vocabulary, groups of 4 requests share their first 256 ids."""
    rng = np.random.default_rng(2)
    lens = rng.integers(PROMPT_LO, PROMPT_HI + 1, size=BATCH)
    if fixed_len:
        lens[:] = fixed_len
    prompts = []
    for b in range(BATCH):
        if b % 4 == 0:
            shared = rng.integers(0, vocab, size=SHARED_PREFIX)
        body = rng.integers(0, vocab, size=int(lens[b]) - SHARED_PREFIX)
        prompts.append(np.concatenate([shared, body]).astype(np.int32))
    return prompts


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        rows = [l.strip().split(", ") for l in Path(self.tmp.name).read_text().splitlines() if l.strip()]
        os.unlink(self.tmp.name)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.strip().lower() == "active":
                    reasons.add(name)
        # The clock under load is what matters: take the median of the upper half of the samples.
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def algorithmic_bytes(cfg, ctx_lens):
    """HBM bytes one decode step must move: every layer weight and the lm_head once, K and V of
    every cached token once, the new token's K/V written, the logits written."""
    d, L = cfg.head_dim, cfg.num_layers
    per_layer = ((cfg.num_qo_heads + 2 * cfg.num_kv_heads) * d * cfg.hidden_size
                 + cfg.hidden_size * cfg.num_qo_heads * d + 3 * cfg.intermediate_size * cfg.hidden_size)
    weights = 2 * (L * per_layer + cfg.vocab_size * cfg.hidden_size)
    kv_tok = 2 * cfg.num_kv_heads * d * L * 2
    kv = int(sum(ctx_lens)) * kv_tok
    out = len(ctx_lens) * (kv_tok + cfg.vocab_size * 2)
    return weights + kv + out, kv // L


def run_gpu(args):
    import __graft_entry__ as entry
    from oracle import token_loop_oracle as O

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    pkg = entry.load_package()
    pkg.load_library()
    from sglang_cpp_b200.engine import Engine, EngineConfig
    from sglang_cpp_b200.host_batch import HostBatcher

    if args.eager:
        os.environ["B200_PDL"] = "0"  # read by the engine at creation
    cfg = O.qwen3_0_6b()
    K, W = args.steps, args.warmup
    total_new = 2 * (K + W) + 24
    prompts = make_prompts(cfg.vocab_size, args.context)
    max_len = max(len(p) for p in prompts) + total_new + 1
    num_pages = sum(math.ceil((len(p) + total_new + 1) / PAGE_SIZE) for p in prompts) + 8
    engine = Engine(cfg, EngineConfig(PAGE_SIZE, num_pages, BATCH, max_len, MAX_EXTEND_TOKENS))
    engine.load_weights(O.init_weights(cfg, seed=0, std=0.02))
    hb = HostBatcher(engine, num_pages, PAGE_SIZE, BATCH)

    # ---- prefill through the engine, in scheduler-sized batches; prefixes are cached as they finish
    reqs, batch, tokens = [], [], 0
    profiled = [False]
    t_prefill0 = time.perf_counter()
    prefill_tokens = 0

    def flush():
        nonlocal batch, tokens, prefill_tokens
        if batch:
            if args.profile_prefill and prefill_tokens > 0 and not profiled[0]:
                # the second prefill batch (the first pays one-time set-up) inside the profiler region
                profiled[0] = True
                torch.cuda.profiler.start()
                hb.prefill(batch).synchronize()
                torch.cuda.profiler.stop()
            else:
                hb.prefill(batch).synchronize()
            prefill_tokens += tokens
            for r in batch:
                hb.cache_prefix(r)
            batch, tokens = [], 0

    for p in prompts:
        probe = len(p)
        if tokens + probe > MAX_EXTEND_TOKENS:
            flush()
        r = hb.add_request(p, total_new)
        reqs.append(r)
        batch.append(r)
        tokens += r.extend_len()
    flush()
    prefill_s = time.perf_counter() - t_prefill0
    if not args.eager:
        engine.capture_graphs([BATCH])
    state0 = [(r.cached_len, r.device_len) for r in reqs]

    def reset():
        for r, (c, dl) in zip(reqs, state0):
            r.cached_len, r.device_len = c, dl

    def barrier():
        engine.synchronize()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.ExternalStream(pkg.load_library().b200_engine_stream(engine._h))
    sampler = ClockSampler(local_rank)

    # ---- phase A: device-timed, steps enqueued back to back ----
    # The K steps are repeated from the same state until at least a second has been timed; every
    # repeat is re-warmed with W steps and bracketed by barrier + synchronize on both sides.
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dev_ms_all, ctx_a, launches_per_step = [], None, 0
    while True:
        reset()
        for _ in range(W):
            hb.decode(reqs)
        barrier()
        ctx_a = [r.device_len for r in reqs]
        if args.profile_region and not dev_ms_all:
            torch.cuda.profiler.start()
        ev0.record(stream)
        for _ in range(K):
            hb.decode(reqs)
        ev1.record(stream)
        barrier()
        if args.profile_region and not dev_ms_all:
            torch.cuda.profiler.stop()
        ms = ev0.elapsed_time(ev1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)   # the job's time is the slowest rank's
            ms = float(t[0])
        dev_ms_all.append(ms)
        _, _, launches_per_step = engine.read_profile()
        if sum(dev_ms_all) >= args.min_timed_ms or len(dev_ms_all) >= 64 or args.profile_region:
            break
    dev_ms = statistics.median(dev_ms_all)

    # ---- phase B: end to end, the host waits for every step's tokens ----
    # Driven the way the scheduler's decode loop drives the engine: per step the host arrays cross
    # the C ABI, the metadata goes host-to-device from pinned memory, the tokens, finish flags and
    # status words land in the engine's pinned result ring and the host waits on that step's event
    # after it has launched the step behind it.
    # (DecodeSession keeps the per-step host bookkeeping in vector form.)
    from sglang_cpp_b200.host_batch import DecodeSession
    e2e_ms_all, step_ms = [], []
    while True:
        reset()
        for _ in range(W):
            hb.decode(reqs).synchronize()
        barrier()
        session = DecodeSession(hb, reqs, ring=True)
        t0 = time.perf_counter()
        pending = None
        for _ in range(K):
            ts = time.perf_counter()
            # the order of the reference's default decode loop (Scheduler::step_overlap,
            # src/scheduler/scheduler.cc:636-675): launch the next forward, then process the previous
            # step's output (its event only; tokens and finish flags are in pinned memory)
            ticket = session.step()
            if pending is not None:
                toks, finished = session.wait(pending)
                _ = int(toks[0]) + int(finished[0])
            pending = ticket
            step_ms.append((time.perf_counter() - ts) * 1e3)
        toks, finished = session.wait(pending)   # the last step's output, still inside the timed region
        _ = int(toks[0]) + int(finished[0])
        barrier()
        ms = (time.perf_counter() - t0) * 1e3
        session.sync_back()
        if dist is not None:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        e2e_ms_all.append(ms)
        if sum(e2e_ms_all) >= args.min_timed_ms or len(e2e_ms_all) >= 64:
            break
    e2e_ms = statistics.median(e2e_ms_all)
    clocks = sampler.stop()

    # ---- phase C: attention launches timed one by one (eager steps, event pair per launch) ----
    reset()
    for _ in range(W + K // 2):
        hb.decode(reqs)
    engine.set_profiling(True)
    hb.decode(reqs).synchronize()  # warm the eager path
    attn_ms, attn_n, ctx_c = 0.0, 0, []
    for _ in range(8):
        ctx_c.append(sum(r.device_len for r in reqs))
        hb.decode(reqs).synchronize()
        ms, n, _k = engine.read_profile()
        attn_ms += ms
        attn_n += n
    engine.set_profiling(False)

    peak, peak_kind = measured_peaks()
    mean_ctx = [c + (K - 1) / 2 for c in ctx_a]  # context grows by one per step
    step_bytes, _ = algorithmic_bytes(cfg, mean_ctx)
    kv_layer_bytes = statistics.mean(ctx_c) * 2 * cfg.num_kv_heads * cfg.head_dim * 2
    attn_launch_ms = attn_ms / max(attn_n, 1)
    attn_gbs = kv_layer_bytes / (attn_launch_ms * 1e-3) / 1e9 if attn_launch_ms > 0 else 0.0
    value = world * BATCH * K / (dev_ms * 1e-3)
    e2e_value = world * BATCH * K / (e2e_ms * 1e-3)
    ratio = dram_traffic_ratio("attention_decode_kernel")
    line = {
        "metric": METRIC,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world, args.context),
        "workload_stats": {"mean_context": round(statistics.mean(mean_ctx), 1),
                           "kv_gb_per_step": round(sum(mean_ctx) * 114688 / 1e9, 2),
                           "prefix_cache_hit_tokens": hb.prefix_hits,
                           "timed_repeats": len(dev_ms_all), "timed_ms_total": round(sum(dev_ms_all), 1),
                           "repeat_ms_min_max": [round(min(dev_ms_all), 3), round(max(dev_ms_all), 3)]},
        "p50_tpot_ms": round(statistics.median(step_ms), 4),
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": (4 * BATCH + 1) * 4, "d2h_bytes_per_step": BATCH * 5 + 16,
                "ms_per_step": round(e2e_ms / K, 4), "timed_repeats": len(e2e_ms_all)},
        "gpu_launches": int(launches_per_step) * K,
        "roofline": {"bound": "hbm", "kernel": "attention_decode_kernel",
                     "achieved": round(attn_gbs, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(attn_gbs / peak, 4), "peak_kind": peak_kind + " (copy bandwidth)",
                     # DRAM bytes per launch: the ratio of DRAM traffic to algorithmic bytes that ncu measured
                     # for this kernel on a smaller case (traffic grows with the sum of contexts), from
                     # profiles/dram_traffic_ratios.md, applied to this launch's algorithmic bytes
                     "traffic": int(kv_layer_bytes * ratio) if ratio else None,
                     "traffic_source": "profiles/dram_traffic_ratios.md (ncu capture of a smaller case, scaled by bytes of K/V)",
                     "launch_ms": round(attn_launch_ms, 5),
                     "algorithmic_bytes_per_launch": int(kv_layer_bytes), "launches_timed": attn_n},
        "step_roofline": {"algorithmic_bytes_per_step": int(step_bytes),
                          "achieved_gbs": round(step_bytes / (dev_ms / K * 1e-3) / 1e9, 1),
                          "frac_of_measured_hbm": round(step_bytes / (dev_ms / K * 1e-3) / 1e9 / peak, 4),
                          "frac_of_nominal_8tbs": round(step_bytes / (dev_ms / K * 1e-3) / 1e9 / 8000.0, 4)},
        "prefill": {"tokens": prefill_tokens, "seconds": round(prefill_s, 3),
                    "tokens_per_s": round(prefill_tokens / prefill_s, 1)},
        "clocks": clocks,
    }
    engine.close()
    del engine, hb, reqs
    torch.cuda.empty_cache()
    if not args.no_tp_record and not args.context and not args.profile_region and not args.eager:
        # the part of the path that shards: Llama-3-8B, tensor parallel over the same ranks
        try:
            line["tp"] = run_gpu_tp(args, dist_ready=dist is not None, as_record=True)
        except Exception as e:   # the headline stands on its own
            line["tp"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(seconds_budget=12.0)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------- mixed workload
def run_gpu_c3(args):
    """Workload "c3": Qwen3-0.6B, 8 new prompts of 4096 tokens prefilled in chunks while 56 requests
    at contexts U[128, 8192] (seed 3) keep decoding, everything sampled (temperature 0.7, top-k 50,
    top-p 0.9, one fixed seed per request).  A batch is prefill or decode, never both
    (src/scheduler/scheduler.cc:366-388), so a step here is one prefill batch of 8192 tokens (four
    prompts advancing by one 2048-token chunk: the second chunk attends to the first through the
    page table) followed by one decode step of the 56 running requests.  After four steps the eight
    prompts are complete and are wound back to position 0 (they keep their pages), so every timed
    step does the same amount of work.  Prefill and decode are timed separately with CUDA events on
    the engine's stream; prefill FLOPs (every linear layer, causal attention) are set against the
    sustained bf16 rate of a large cuBLAS GEMM on this pool."""
    import __graft_entry__ as entry
    from oracle import token_loop_oracle as O

    torch.cuda.set_device(0)
    pkg = entry.load_package()
    pkg.load_library()
    from sglang_cpp_b200.engine import Engine, EngineConfig
    from sglang_cpp_b200.host_batch import HostBatcher

    cfg = O.qwen3_0_6b()
    K, W = args.steps, max(args.warmup, 4)
    n_new, new_len, n_run, chunk, per_step = 8, 4096, 56, args.chunk_tokens, 4
    chunks_per_prompt = -(-new_len // chunk)
    cycle = (n_new // per_step) * chunks_per_prompt
    rng = np.random.default_rng(3)
    ctx = rng.integers(128, 8192 + 1, size=n_run)
    total_new = 64 * (K + W) + 64    # every repeat of the timed region continues decoding
    run_prompts = [rng.integers(0, cfg.vocab_size, size=int(n)).astype(np.int32) for n in ctx]
    new_prompts = [rng.integers(0, cfg.vocab_size, size=new_len).astype(np.int32) for _ in range(n_new)]
    max_len = 8192 + total_new + 2
    num_pages = (sum(math.ceil((len(p) + total_new + 1) / PAGE_SIZE) for p in run_prompts)
                 + n_new * math.ceil((new_len + 2) / PAGE_SIZE) + 8)
    engine = Engine(cfg, EngineConfig(PAGE_SIZE, num_pages, n_run + n_new, max_len, MAX_EXTEND_TOKENS))
    engine.load_weights(O.init_weights(cfg, seed=0, std=0.02))
    hb = HostBatcher(engine, num_pages, PAGE_SIZE, n_run + n_new, enable_prefix_cache=False)

    def sampling(reqs):
        return dict(temperatures=[0.7] * len(reqs), top_k=[50] * len(reqs), top_p=[0.9] * len(reqs),
                    seeds=[1000 + r.table_idx for r in reqs])

    # the 56 running requests reach their contexts by ordinary prefill batches
    running, batch, tokens = [], [], 0
    for p in run_prompts:
        if tokens + len(p) > MAX_EXTEND_TOKENS and batch:
            hb.prefill(batch, None, sampling(batch)).synchronize()
            batch, tokens = [], 0
        r = hb.add_request(p, total_new)
        running.append(r)
        batch.append(r)
        tokens += len(p)
    if batch:
        hb.prefill(batch, None, sampling(batch)).synchronize()
    fresh = [hb.add_request(p, 1) for p in new_prompts]
    engine.capture_graphs([64])

    stream = torch.cuda.ExternalStream(pkg.load_library().b200_engine_stream(engine._h))
    state = {"i": 0, "prefill_wall_ms": 0.0, "launches": [0, 0]}

    def one_step(ev=None, wait=False):
        """Prefill chunk + decode step; `ev` = three events recorded before, between and after."""
        i = state["i"] % cycle
        state["i"] += 1
        group = fresh[(i // chunks_per_prompt) * per_step:(i // chunks_per_prompt + 1) * per_step]
        if i % chunks_per_prompt == 0:
            for r in group:                      # wound back: the pages stay
                r.cached_len, r.device_len, r.is_chunked_prefill = 0, len(r.input_ids), False
        if ev:
            ev[0].record(stream)
        t0 = time.perf_counter()
        out = hb.prefill(group, chunk, sampling(group))
        if wait:
            out.synchronize()
            _ = out.next_tokens_cpu[0].item()
            state["prefill_wall_ms"] += (time.perf_counter() - t0) * 1e3
            state["launches"][0] = engine.read_profile()[2]
        if ev:
            ev[1].record(stream)
        out = hb.decode(running, sampling=sampling(running))
        if wait:
            out.synchronize()
            _ = out.next_tokens_cpu[0].item()
            state["launches"][1] = engine.read_profile()[2]
        if ev:
            ev[2].record(stream)

    def sync():
        engine.synchronize()
        torch.cuda.synchronize()

    sampler = ClockSampler(0)
    sampler.start()
    pre_ms, dec_ms, tot_ms, ctx_sum = [], [], [], []
    while True:
        state["i"] = 0
        for _ in range(W):
            one_step()
        sync()
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record(stream)
        for k in range(K):
            ctx_sum.append(sum(r.device_len for r in running))
            one_step(evs[k])
        last.record(stream)
        sync()
        pre_ms += [e[0].elapsed_time(e[1]) for e in evs]
        dec_ms += [e[1].elapsed_time(e[2]) for e in evs]
        tot_ms.append(first.elapsed_time(last))
        if sum(tot_ms) >= args.min_timed_ms or len(tot_ms) >= 16:
            break
    # end to end: the host waits for every batch's tokens
    e2e_ms, e2e_prefill_ms = [], []
    while True:
        state["i"] = 0
        for _ in range(W):
            one_step(wait=True)
        sync()
        state["prefill_wall_ms"] = 0.0
        t0 = time.perf_counter()
        for _ in range(K):
            one_step(wait=True)
        sync()
        e2e_ms.append((time.perf_counter() - t0) * 1e3)
        e2e_prefill_ms.append(state["prefill_wall_ms"])
        if sum(e2e_ms) >= args.min_timed_ms or len(e2e_ms) >= 16:
            break
    clocks = sampler.stop()

    d, L, Hq, Hkv = cfg.head_dim, cfg.num_layers, cfg.num_qo_heads, cfg.num_kv_heads
    per_layer = (Hq + 2 * Hkv) * d * cfg.hidden_size + cfg.hidden_size * Hq * d + 3 * cfg.intermediate_size * cfg.hidden_size
    step_tokens = per_step * chunk
    linear_flops = 2.0 * per_layer * L * step_tokens
    # causal attention of a chunk at positions [c, c + n): each query meets c + (its offset + 1) keys
    attn_flops = 0.0
    for j in range(chunks_per_prompt):
        c, n = j * chunk, min(chunk, new_len - j * chunk)
        attn_flops += 4.0 * Hq * d * (n * c + n * (n + 1) / 2) * L * per_step
    attn_flops /= chunks_per_prompt                              # mean over the steps of a cycle
    pre = statistics.median(pre_ms)
    dec = statistics.median(dec_ms)
    tflops = (linear_flops + attn_flops) / (pre * 1e-3) / 1e12
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    tensor_peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    hbm_peak, peak_kind = measured_peaks()
    kv_tok = 2 * Hkv * d * L * 2
    dec_bytes = 2 * (L * per_layer + cfg.vocab_size * cfg.hidden_size) + statistics.mean(ctx_sum) * kv_tok \
        + n_run * (kv_tok + cfg.vocab_size * 2)
    total = statistics.median(tot_ms)
    line = {
        "metric": "prefill tokens/s and sampled-decode ms/step, interleaved (Qwen3-0.6B, 8 x 4096 new + 56 running)",
        "value": round(step_tokens / (pre * 1e-3), 1), "unit": "prefill tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(total / K, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "c3: Qwen3-0.6B, 8 new prompts of 4096 tokens prefilled in %d-token chunks (4 prompts = %d tokens per "
                               "batch) alternating with decode steps of 56 requests at contexts U[128,8192] seed 3, page size 16, "
                               "temperature 0.7 / top-k 50 / top-p 0.9 with a fixed seed per request" % (chunk, step_tokens),
                   "l2": "inputs larger than L2: a decode step streams about %.0f GB of K/V" % (statistics.mean(ctx_sum) * kv_tok / 1e9),
                   "parallelism": "single GPU"},
        "prefill": {"ms_per_batch": round(pre, 4), "tokens_per_batch": step_tokens,
                    "tokens_per_s": round(step_tokens / (pre * 1e-3), 1), "tflops": round(tflops, 1),
                    "linear_share_of_flops": round(linear_flops / (linear_flops + attn_flops), 3)},
        "decode": {"ms_per_step": round(dec, 4), "requests": n_run, "mean_context": round(statistics.mean(ctx_sum) / n_run, 1),
                   "tokens_per_s": round(n_run / (dec * 1e-3), 1), "replayed_graph": "64-row sampled graph (8 dummy rows)",
                   "achieved_gbs": round(dec_bytes / (dec * 1e-3) / 1e9, 1),
                   "frac_of_measured_hbm": round(dec_bytes / (dec * 1e-3) / 1e9 / hbm_peak, 4)},
        # the same loop with the host waiting for every batch's tokens; the prefill share by wall clock
        "e2e": {"value": round(step_tokens * K / (statistics.median(e2e_prefill_ms) * 1e-3), 1), "unit": "prefill tokens/s",
                "ms_per_step": round(statistics.median(e2e_ms) / K, 4),
                "decode_ms_per_step": round((statistics.median(e2e_ms) - statistics.median(e2e_prefill_ms)) / K, 4),
                "h2d_bytes_per_step": (4 * per_step + 1) * 4 + 16 * per_step + (4 * 64 + 1) * 4 + 16 * 64,
                "d2h_bytes_per_step": (per_step + n_run) * 4},
        "gpu_launches": int(sum(state["launches"])) * K,
        "roofline": {"bound": "tensor", "kernel": "prefill batch (tile GEMMs + prefill attention)", "achieved": round(tflops, 1),
                     "peak": tensor_peak, "unit": "TFLOP/s", "frac": round(tflops / tensor_peak, 4),
                     "peak_kind": "measured (sustained cuBLAS bf16)" if peaks else "fallback", "traffic": None},
        "timed_repeats": len(tot_ms),
        "clocks": clocks,
    }
    engine.close()
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------- TP workload
def run_gpu_tp(args, dist_ready=False, as_record=False):
    """Workload "c4": Llama-3-8B architecture, bf16, random-init weights drawn on the device,
    tensor parallel over all ranks (heads and MLP columns split, the post-projection all-reduce
    fused with add + norm over NVLink peer memory), batch 128, prompts of 1024 uniform-random
    tokens, greedy decode, page size 16.  Strong scaling: the same job on N GPUs."""
    import __graft_entry__ as entry
    from oracle import token_loop_oracle as O
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1 and not dist_ready:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pkg = entry.load_package()
    pkg.load_library()
    from sglang_cpp_b200.engine import Engine, EngineConfig
    from sglang_cpp_b200.host_batch import HostBatcher

    moe = args.workload == "c5" and not as_record
    cfg = O.qwen3_30b_a3b() if moe else O.llama3_8b()
    B, PROMPT = (256, 512) if moe else (128, 1024)
    K, W = args.steps, args.warmup
    total_new = (K + W) + 24
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg.vocab_size, size=PROMPT).astype(np.int32) for _ in range(B)]
    num_pages = B * math.ceil((PROMPT + total_new + 1) / PAGE_SIZE) + 8
    # MoE under more than one GPU: whole experts per rank (expert parallelism), attention heads split,
    # a KV head replicated where there are more ranks than KV heads
    engine = Engine(cfg, EngineConfig(PAGE_SIZE, num_pages, B, PROMPT + total_new + 1, MAX_EXTEND_TOKENS, rank, world,
                                      expert_parallel=moe and world > 1))
    engine.fill_random(seed=0)
    in_switch = False
    if world > 1:
        engine.connect_tp()
        lib = pkg.load_library()
        in_switch = bool(lib.b200_comm_uses_multicast(ctypes.c_void_p(lib.b200_engine_comm(engine._h))))
    data_path = ("allreduce kernels of csrc/allreduce.cu, sums formed inside the NVLink switch (multimem.ld_reduce / "
                 "multimem.st on a symmetric-memory multicast address); NCCL only for the rendezvous" if in_switch else
                 "allreduce kernels of csrc/allreduce.cu over CUDA-IPC peer memory; NCCL only for the rendezvous")
    hb = HostBatcher(engine, num_pages, PAGE_SIZE, B, enable_prefix_cache=False)
    reqs, batch = [], []
    t0 = time.perf_counter()
    for p in prompts:
        r = hb.add_request(p, total_new)
        reqs.append(r)
        batch.append(r)
        if len(batch) * PROMPT >= MAX_EXTEND_TOKENS:
            hb.prefill(batch).synchronize()
            batch = []
    if batch:
        hb.prefill(batch).synchronize()
    prefill_s = time.perf_counter() - t0
    engine.capture_graphs([B])
    stream = torch.cuda.ExternalStream(pkg.load_library().b200_engine_stream(engine._h))

    def barrier():
        engine.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        hb.decode(reqs)
    barrier()
    ctx0 = reqs[0].device_len
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    toks = None
    for _ in range(K):
        toks = hb.decode(reqs)
    ev1.record(stream)
    barrier()
    clocks = sampler.stop()
    dev_ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([dev_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms = float(t[0])
        # lock-step check: every rank sampled the same tokens
        mine = toks.next_tokens_cpu.clone().cuda()
        ref = mine.clone()
        dist.broadcast(ref, 0)
        same = torch.tensor([int(torch.equal(mine, ref))], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        lockstep = bool(same.item())
    else:
        lockstep = True
    # per-kernel timing of attention and all-reduce launches: eager steps, one event pair per launch
    engine.set_profiling(True)
    hb.decode(reqs).synchronize()
    attn_ms = ar_ms = 0.0
    attn_n = ar_n = 0
    for _ in range(4):
        hb.decode(reqs).synchronize()
        ms, n, _k = engine.read_profile()
        attn_ms, attn_n = attn_ms + ms, attn_n + n
        if world > 1:
            ms, n = engine.read_profile_allreduce()
            ar_ms, ar_n = ar_ms + ms, ar_n + n
    engine.set_profiling(False)
    peak, peak_kind = measured_peaks()
    d, L = cfg.head_dim, cfg.num_layers
    attn_w = (cfg.num_qo_heads + 2 * cfg.num_kv_heads) * d * cfg.hidden_size + cfg.hidden_size * cfg.num_qo_heads * d
    if moe:   # every expert is hit at batch 256 with top-8 routing: all expert weights are read each step
        mlp_w = cfg.num_experts * 3 * cfg.moe_intermediate_size * cfg.hidden_size + cfg.num_experts * cfg.hidden_size
    else:
        mlp_w = 3 * cfg.intermediate_size * cfg.hidden_size
    per_layer = attn_w + mlp_w
    mean_ctx = ctx0 + (K - 1) / 2
    kv_tok = 2 * cfg.num_kv_heads * d * L * 2
    kv_share = max(world, 1) if cfg.num_kv_heads >= world else cfg.num_kv_heads   # replicated KV heads do not shrink
    # per GPU: sharded layers and KV, replicated lm_head
    bytes_gpu = 2 * L * per_layer / world + 2 * cfg.vocab_size * cfg.hidden_size + B * mean_ctx * kv_tok / kv_share
    line = {
        "metric": ("decode tokens/s at bs=256 (Qwen3-30B-A3B, EP + attention TP over all GPUs)" if moe else
                   "decode tokens/s at bs=128 (Llama-3-8B, TP over all GPUs)"),
        "value": round(B * K / (dev_ms * 1e-3), 1),
        "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": ("c5: Qwen3-30B-A3B decode, batch 256, prompts of 512 random tokens, page size 16, greedy"
                                if moe else
                         "c4: Llama-3-8B decode, batch 128, prompts of 1024 random tokens, page size 16, greedy"),
                   "parallelism": (f"ep{world}+tp{world}" if moe else f"tp{world}"), "mean_context": mean_ctx,
                   "ranks_in_lockstep": lockstep, "data_path": data_path if world > 1 else "single GPU"},
        "step_roofline": {"algorithmic_bytes_per_step_per_gpu": int(bytes_gpu),
                          "frac_of_measured_hbm": round(bytes_gpu / (dev_ms / K * 1e-3) / 1e9 / peak, 4)},
        "prefill": {"tokens": B * PROMPT, "seconds": round(prefill_s, 3)},
        "kernels": {"attention_us_per_launch": round(attn_ms * 1e3 / max(attn_n, 1), 2),
                    "allreduce_us_per_launch": round(ar_ms * 1e3 / max(ar_n, 1), 2) if ar_n else None,
                    "allreduce_launches_per_step": ar_n // 4},
        "clocks": clocks,
    }
    engine.close()
    if as_record:
        # attached to the headline line: the sharded path on the same ranks.  Speed-up over one GPU is
        # this `ms_per_step` against the `tp.ms_per_step` of the N = 1 run of the same command.
        return {"workload": line["config"]["workload"], "parallelism": line["config"]["parallelism"],
                "scaling": "strong", "steps": K, "warmup": W, "ms_per_step": line["ms_per_step"],
                "tokens_per_s": line["value"], "ranks_in_lockstep": lockstep,
                "frac_of_measured_hbm_per_gpu": line["step_roofline"]["frac_of_measured_hbm"],
                "attention_us_per_launch": line["kernels"]["attention_us_per_launch"],
                "allreduce_us_per_launch": line["kernels"]["allreduce_us_per_launch"],
                "allreduce_launches_per_step": line["kernels"]["allreduce_launches_per_step"],
                "data_path": data_path}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------- CPU side
def cpu_decode_sample(steps: int, warmup: int, seconds_budget: float = 0.0, num_reqs: int = BATCH):
    """Times the CPU oracle (a port: the reference has no CPU forward) on decode steps of the
    workload's batch: `num_reqs` requests (all 64 unless host memory is short) at their real context
    lengths.  The K/V contents are whatever the allocation holds (the cost does not depend on the
    values) and are kept in bf16, as the GPU pool keeps them."""
    from oracle import token_loop_oracle as O

    cfg = O.qwen3_0_6b()
    torch.set_num_threads(os.cpu_count() or 1)
    prompts = make_prompts(cfg.vocab_size)[:num_reqs]
    lens = np.array([len(p) for p in prompts], dtype=np.int32)
    n_slots = int(lens.sum()) + (steps + warmup + 1) * num_reqs
    kv_bytes = 2 * cfg.num_layers * n_slots * cfg.num_kv_heads * cfg.head_dim * 2
    try:
        import psutil
        if kv_bytes + (8 << 30) > psutil.virtual_memory().available and num_reqs > 8:
            return cpu_decode_sample(steps, warmup, seconds_budget, max(8, num_reqs // 2))
    except ImportError:
        pass
    w = O.init_weights(cfg, seed=0, std=0.02)
    model = O.OracleModel(cfg, w, O.store_bf16)
    shape = (cfg.num_layers, n_slots, cfg.num_kv_heads, cfg.head_dim)
    kv = O.KVState(torch.zeros(shape, dtype=torch.bfloat16), torch.zeros(shape, dtype=torch.bfloat16))
    cols = int(lens.max()) + steps + warmup + 2
    pt = np.zeros((num_reqs, cols), dtype=np.int32)
    cur = 0
    for b in range(num_reqs):
        n = int(lens[b]) + steps + warmup + 1
        pt[b, :n] = np.arange(cur, cur + n)
        cur += n
    tok = np.array([int(p[-1]) for p in prompts], dtype=np.int32)
    times = []
    for s in range(warmup + steps):
        pos = lens + s
        batch = O.StepBatch(tok, pos.astype(np.int32), pt[np.arange(num_reqs), pos].copy(),
                            np.arange(num_reqs, dtype=np.int32), (pos + 1).astype(np.int32),
                            np.arange(num_reqs + 1, dtype=np.int32), False)
        t0 = time.perf_counter()
        logits = model.forward(batch, kv, pt)
        tok = logits.argmax(-1).numpy().astype(np.int32)
        if s >= warmup:
            times.append(time.perf_counter() - t0)
            if seconds_budget and len(times) >= 2 and sum(times) >= seconds_budget:
                break   # the sample is bounded by time: at most `steps` steps, about `seconds_budget` seconds
    return times, torch.get_num_threads(), num_reqs


def cpu_baseline(seconds_budget: float):
    times, cores, n = cpu_decode_sample(steps=16, warmup=1, seconds_budget=seconds_budget)
    per_step = statistics.mean(times)
    return {"value": round(n / per_step, 2), "unit": "tokens/s", "cores": cores,
            "kind": "port",
            "sample": f"CPU oracle (torch fp32 restatement; the reference has no CPU forward), decode steps of "
                      f"{n} of the 64 requests at their real contexts, {len(times)} steps after 1 warm-up, "
                      f"{per_step * 1e3:.0f} ms per step"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 32))   # one step of the whole batch takes a second or two on the host cores
    warmup = max(1, min(args.warmup, 8))
    times, cores, n = cpu_decode_sample(steps, warmup)
    total = sum(times)
    value = n * len(times) / total
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(times), "warmup": warmup,
        "ms_per_step": round(total / len(times) * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": round(value, 2), "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"CPU oracle, each step = one decode step of {n} of the 64 requests at their real "
                                   f"contexts (K/V contents arbitrary); the reference's own dense forward is CUDA-only, "
                                   f"so this is a port"},
        "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--chunk-tokens", type=int, default=2048, help="c3: tokens a prompt advances per prefill batch")
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5"],
                    help="c2 (default, the headline metric): Qwen3-0.6B decode, replicas when N > 1; "
                         "c3: Qwen3-0.6B chunked prefill alternating with sampled decode, one GPU; "
                         "c4: Llama-3-8B decode, tensor parallel over the N ranks; "
                         "c5: Qwen3-30B-A3B decode, experts and attention heads split over the N ranks")
    ap.add_argument("--context", type=int, default=0,
                    help="c2 only: give every prompt this length instead of U[512,2048]")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp-record", action="store_true",
                    help="c2 only: do not run the tensor-parallel workload after the headline")
    ap.add_argument("--min-timed-ms", type=float, default=1000.0,
                    help="repeat the K timed steps until this much time has been timed; the median repeat is reported")
    ap.add_argument("--profile-prefill", action="store_true",
                    help="c2 only: bracket the second prefill batch with cudaProfilerStart/Stop")
    ap.add_argument("--eager", action="store_true",
                    help="c2 only: plain launches, no graph replay and no programmatic dependent launches "
                         "(the form a profiler can list kernel by kernel); not a bench value")
    ap.add_argument("--profile-region", action="store_true",
                    help="bracket the device-timed steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "b200":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("c4", "c5"):
        run_gpu_tp(args)
    elif args.workload == "c3":
        if args.gpus != 1:
            raise SystemExit("workload c3 runs on one GPU")
        run_gpu_c3(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
