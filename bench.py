#!/usr/bin/env python
"""Benchmark of the ragged speculative verify step on B200.

    python bench.py --gpus 1 --steps 20 --warmup 5                 # our CUDA path, 27B-class single-stream verify
    python bench.py --impl reference --steps 2 --warmup 1          # the CPU restatement timed on the host cores
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W                     # N sequence-sharded replicas, no collective

A step is one verify pass over one packed batch: pack the trees, 64-layer forward, argmax, greedy tree acceptance,
KV compaction and DeltaNet commit.  Rank 0 prints ONE JSON line.

  value      packed rows verified per second over all GPUs, inputs resident in HBM (descriptors staged once, the timed
             region is K graph replays bracketed by CUDA events on the launching stream; max over ranks)
  e2e        the same through the host-buffer entry point ling_b200_verify_step (descriptor H2D copy, graph replay,
             result D2H copy inside the timed region)
  roofline   the weight GEMM (gemm_fp8_tcgen05_kernel): algorithmic bytes = FP8 codes + fp32 block scales of every
             matrix one step streams, divided by the device time of the step's 257 GEMM launches in the step's order and
             with the step's launch attributes (dependent launch), nothing else between them, measured with two CUDA
             events on the launching stream around five passes (average launch duration = that time / 257), against the
             measured HBM copy bandwidth; per_launch_events = the same launches in one eager replay with an event pair
             around EACH launch (every launch then carries its own ramp-up and an event gap: a lower bound)
             roofline.frac (0.87) is the GEMM chain's share of the copy bandwidth, NOT the step's: the step's own figure is
             hbm_fraction_weights_plus_kv = (weight bytes + KV bytes) / step time / measured copy bandwidth (0.54), the
             north star's fraction, printed beside it
  cpu_baseline the scalar C++ restatement of the same step (oracle/, test infrastructure) timed on this box's host
             cores on a bounded sample (one DeltaNet layer, one attention layer, a slice of the LM head), scaled by the
             layer counts; a reported baseline, not a target

Other workloads (one JSON line each, same keys): --workload ragged4 (4 sequences, 74 rows), churn64 (64 sequences sharded over
the ranks, ~10 % completions and admissions per step through the page pool), served64 (the same 64-sequence load produced by
the scheduler loop: ling-engine_b200/ling_serve_headless), mixed (a 4096-row prefill chunk through the NVFP4 prefill path -- DeltaNet mixers and feed-forward blocks --
beside an 8-sequence verify step; roofline against the NVFP4 tensor rate measured in the same run), toy.  --micro gemm |
nvfp4 | nvfp4-swiglu | gdn-chunk | gdn-layer times one kernel (gdn-layer: one DeltaNet layer's prefill mixer) alone on resident operands (the small cases the profiler captures;
gdn-chunk takes its row count from --shape's first number).

Inputs are synthetic (seeded): they stand in for the reference's private replay workload, whose shapes they take.
Weights are 26.4 GB, far larger than the 126 MB L2, so consecutive steps cannot hit in L2 (no flush between steps).
"""
import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

METRIC = "verify_step_tokens_per_s"
UNIT = "tokens/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def chain_plus_branch(chain_rows, branch_rows):
    parent = [-1] + list(range(chain_rows - 1))
    for b in range(branch_rows):
        parent.append(0 if b == 0 else chain_rows + b - 1)
    return parent


def workload(name, rank, vocab):
    """The sequences of one step (per GPU).  Token ids uniform over the vocabulary; accepted lengths imposed so that the
    compaction and the commit do representative work (6 drafts + the anchor, the reference's ~6.7 tokens per step)."""
    rng = np.random.default_rng(1000 + rank)
    if name == "single":      # single-stream 27B-class verify: context 8192, 16-token chain + 8-node lookup branch
        specs = [(8192, chain_plus_branch(16, 8), 15)]
    elif name == "ragged4":   # 4 sequences sharing one weight read: trees of 24, 17, 9 and 24 nodes = 74 rows
        specs = [(2048, chain_plus_branch(16, 8), 15), (9216, chain_plus_branch(12, 5), 11), (31000, chain_plus_branch(9, 0), 8),
                 (60000, chain_plus_branch(16, 8), 15)]
    elif name == "churn64":   # 64 sequences of a continuous-batching server, sharded by sequence over the GPUs: contexts
        # lognormal (median 6k, at most 128k), trees of 1-32 nodes (a chain plus a lookup branch off the anchor)
        world = max(1, int(os.environ.get("WORLD_SIZE", 1)))
        all_rng = np.random.default_rng(64)
        ctxs = np.clip(all_rng.lognormal(np.log(6000.0), 1.0, 64), 256, 131072 - 64).astype(int)
        sizes = all_rng.integers(1, 33, 64)
        specs = []
        # whole sequences, the estimated step time (rows, KV positions, sequences) balanced over the GPUs
        for i in shard_sequences([int(c) for c in ctxs], world, rows=[int(n) for n in sizes])[rank]:
            n = int(sizes[i])
            chain_rows = max(1, (2 * n + 2) // 3)
            specs.append((int(ctxs[i]), chain_plus_branch(chain_rows, n - chain_rows), chain_rows - 1))
    elif name == "mixed":     # the decode half of the mixed pass: 8 sequences with 24-node trees, contexts uniform in 1k-32k
        specs = [(int(c), chain_plus_branch(16, 8), 15) for c in rng.integers(1024, 32769, 8)]
    elif name == "toy":
        specs = [(c, chain_plus_branch(16, 4), 15) for c in (3, 37, 512, 1029)]
    else:
        raise SystemExit("unknown workload " + name)
    seqs = []
    for s, (ctx, parent, chain) in enumerate(specs):
        n = len(parent)
        tokens = rng.integers(0, vocab, n).astype(np.int32)
        accept = int(rng.integers(1, chain + 2)) if name in ("ragged4", "churn64") else min(7, chain + 1)
        force = rng.integers(0, vocab, n).astype(np.int32)
        for r in range(accept - 1):
            force[r] = tokens[r + 1]
        force[accept - 1] = (int(tokens[accept]) + 1) % vocab if accept < n else 0
        seqs.append({"slot": s, "pos": ctx, "tokens": tokens, "parent": np.array(parent, np.int32), "chain": chain,
                     "force": force, "accept": accept})
    return seqs


class PagePool:
    """The KV page pool (ling_b200_kvpool_*, the reference's KvPool) with one caller-owned page table per session slot."""

    def __init__(self, lbm, pages, page_tokens, slots, cap):
        import ctypes as C
        self.C, self.L, self.cap = C, lbm.lib(), cap
        self.h = C.c_void_p(self.L.ling_b200_kvpool_create(pages, page_tokens))
        self.tab = [(C.c_int * cap)() for _ in range(slots)]
        self.len = [C.c_int(0) for _ in range(slots)]

    def ensure(self, slot, upto):
        """Maps positions [0, upto); returns the table, or None when the pool cannot cover it (nothing changes then)."""
        nc = self.C.c_int(0)
        if self.L.ling_b200_kvpool_ensure(self.h, self.tab[slot], self.C.byref(self.len[slot]), self.cap, 0, upto, None, 0,
                                          self.C.byref(nc)) != 1:
            return None
        return np.array(self.tab[slot][:self.len[slot].value], np.int32)

    def drop(self, slot):
        pages = set(p for p in self.tab[slot][:self.len[slot].value] if p)
        self.L.ling_b200_kvpool_truncate(self.h, self.tab[slot], self.len[slot].value, 0)
        self.len[slot].value = 0
        return pages

    def retire(self):
        self.L.ling_b200_kvpool_retire(self.h)


def churn_step(ctx, pool, seqs, rng, max_context):
    """Completions and admissions between two steps: ~10 % of the sequences finish, their pages go back to the pool (deferred
    retire), and the same session slots are admitted again with a new context length on whatever pages the pool hands out.
    The admitted sequence's KV is what the reused pages hold (valid FP8 codes): the prefill that would write it is not part
    of this path.  Returns (admitted, pages reused)."""
    k = max(1, len(seqs) // 10)
    done = [int(i) for i in rng.choice(len(seqs), k, replace=False)]
    freed = set()
    for i in done:
        freed |= pool.drop(seqs[i]["slot"])
    pool.retire()
    reused = 0
    for i in done:
        q = seqs[i]
        pos = int(np.clip(rng.lognormal(np.log(6000.0), 1.0), 256, max_context - 64))
        table = pool.ensure(q["slot"], pos + 64)
        while table is None:   # the pool cannot take this context: admit a shorter one
            pos //= 2
            table = pool.ensure(q["slot"], pos + 64)
        q["pos"] = pos
        reused += len(freed & set(int(p) for p in table))
        ctx.kv_table_set(q["slot"], np.arange(len(table), dtype=np.int32), table)
    return len(done), reused


class ClockSampler:
    """nvidia-smi sampled during the timed region (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = self.proc.communicate()[0]
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not f[1].isdigit():
                continue
            sm.append(int(f[1])), mx.append(int(f[2]))
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v == "Active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


class Dist:
    """torch.distributed only as plumbing: a barrier and a max / sum over ranks.  NCCL on GPUs; `backend="gloo"` is the
    CPU stand-in the multi-rank tests use.  Not used at one GPU: the replicas exchange no data."""

    def __init__(self, world, local_rank, backend="nccl"):
        self.world, self.backend = world, backend
        if world > 1:
            import torch
            import torch.distributed as dist
            if backend == "nccl":
                torch.cuda.set_device(local_rank)
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group(backend)
            self.torch, self.dist = torch, dist
            self.device = "cuda" if backend == "nccl" else "cpu"

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
            if self.backend == "nccl":
                self.torch.cuda.synchronize()

    def _reduce(self, x, op):
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=op)
        return float(t.item())

    def max(self, x):
        return self._reduce(x, self.dist.ReduceOp.MAX if self.world > 1 else None)

    def sum(self, x):
        return self._reduce(x, self.dist.ReduceOp.SUM if self.world > 1 else None)

    def select(self, rank, x):
        """Rank `rank`'s value of x on every rank (a sum in which the others contribute zero)."""
        if self.world == 1:
            return x
        me = self.dist.get_rank()
        return self._reduce(x if me == rank else 0.0, self.dist.ReduceOp.SUM)

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def model_for(lbm, name, layers):
    if name == "toy":
        return lbm.toy_config()
    return lbm.config_27b(layers)


def algorithmic_bytes(cfg, seqs, weight_bytes):
    """Weight bytes one step streams (FP8 codes + fp32 scale per 1x128 + BF16 extras) plus the FP8 KV of the context
    (codes + one fp32 scale per position and head), and the DeltaNet state traffic reported beside it."""
    n_attn = len(cfg.attn_layers())
    n_gdn = cfg.layers - n_attn
    kv_per_token = n_attn * 2 * cfg.kv_heads * (cfg.head_dim + 4)
    kv = sum(q["pos"] for q in seqs) * kv_per_token
    state = n_gdn * cfg.lin_v_heads * cfg.lin_k_dim * cfg.lin_v_dim * 4
    return {"weights": weight_bytes, "kv": kv, "state_verify_read": state * len(seqs), "state_commit_rw": 2 * state * len(seqs)}


class CpuSample:
    """The oracle on a bounded sample of the same step (one DeltaNet layer, one attention layer, a slice of the LM head),
    scaled to the whole model by the layer counts and the vocabulary."""

    def __init__(self, lbm, cfg, seqs, threads):
        from oracle import lo as lom
        self.lom, self.lbm, self.cfg, self.threads = lom, lbm, cfg, threads
        lom.lo().lo_set_threads(threads)
        self.attn, self.gdn = cfg.attn_layers(), cfg.gdn_layers()
        self.layers = self.gdn[:1] + self.attn[:1]
        self.head_rows = min(cfg.vocab, 8192)
        max_ctx = max(q["pos"] for q in seqs) + 64
        pages = sum((q["pos"] + 32 + 15) // 16 for q in seqs) + 1
        opt = lbm.Options(len(seqs), max_ctx, 16, pages, len(seqs), sum(len(q["tokens"]) for q in seqs), 0, 0, 0, 0, 0)
        self.m = lom.Model(cfg, opt, lbm)
        self.m.synth_weights_layers(0, self.layers, self.head_rows)
        page = 1
        self.seqs = []
        for q in seqs:
            n = (q["pos"] + 32 + 15) // 16
            self.m.kv_table_set(q["slot"], np.arange(n, dtype=np.int32), np.arange(page, page + n, dtype=np.int32))
            page += n
            if q["pos"] > 0:
                self.m.synth_kv(q["slot"], q["pos"], 0)
            self.m.synth_state(q["slot"], 0)
            self.seqs.append(dict(q, tokens=q["tokens"] % self.head_rows, force=None))
        self.rows = sum(len(q["tokens"]) for q in seqs)

    def time_once(self):
        """Returns (tokens/s of the whole step as estimated, estimated seconds per step, measured seconds)."""
        times = {}
        for name, ls, hr in (("gdn", self.gdn[:1], 0), ("attn", self.attn[:1], 0), ("head", [], self.head_rows)):
            t0 = time.perf_counter()
            self.m.verify_step_sample(self.seqs, ls if ls else [-1], hr, make_steps=self.lbm.make_steps)
            times[name] = time.perf_counter() - t0
        est = (len(self.gdn) * times["gdn"] + len(self.attn) * times["attn"] +
               times["head"] * (self.cfg.vocab / self.head_rows))
        return self.rows / est, est, sum(times.values())

    def describe(self, measured):
        return ("oracle step on layers %s + %d of %d LM-head rows, %d rows; scaled by %d DeltaNet + %d attention layers and the "
                "vocabulary (%.1f s wall on %d threads measured per pass)" % (self.layers, self.head_rows, self.cfg.vocab, self.rows,
                                                                              len(self.gdn), len(self.attn), measured, self.threads))

    def close(self):
        self.m.close()
        self.lom.lo().lo_set_threads(1)


def cpu_sample(lbm, cfg, seqs, threads):
    c = CpuSample(lbm, cfg, seqs, threads)
    runs = [c.time_once() for _ in range(3)]  # three passes over the sample: ~20-30 core-seconds of CPU work in all
    v, est, measured = sorted(runs, key=lambda r: r[1])[1]
    desc = c.describe(measured) + "; median of 3 passes"
    c.close()
    return v, est, desc


def run_reference(args, rank, world):
    """The reference has no CPU (and no sm_100a) implementation of the forward pass; its stand-in is the scalar C++
    restatement under oracle/ (kind "port"), timed on all host cores.  Every step is the same bounded sample."""
    if rank != 0:
        return
    lbm = importlib.import_module("ling-engine_b200")
    cfg = model_for(lbm, args.workload, args.layers)
    seqs = workload(args.workload, 0, cfg.vocab)
    threads = max(1, min(os.cpu_count() or 1, 64))
    c = CpuSample(lbm, cfg, seqs, threads)
    for _ in range(min(args.warmup, 1)):
        c.time_once()
    vals = [c.time_once() for _ in range(max(1, min(args.steps, 5)))]
    v = statistics.median(x[0] for x in vals)
    est = statistics.median(x[1] for x in vals)
    sample = c.describe(statistics.median(x[2] for x in vals))
    c.close()
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": est * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": args.workload, "model": "27B-class hybrid, %d layers" % cfg.layers if args.workload != "toy" else "toy",
                       "rows": c.rows, "parallelism": "host threads", "timed_steps": len(vals)},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def setup_context(lbm, cfg, seqs, args, rank, local_rank, churn, chunk_rows=0):
    """A context sized for `seqs` with synthetic weights, page tables from the page pool, synthetic KV and DeltaNet state.
    chunk_rows > 0: one more session (slot len(seqs)) with pages for a prefill chunk of that many positions."""
    rows = sum(len(q["tokens"]) for q in seqs)
    page_tokens = 16
    pages = sum((q["pos"] + 64 + page_tokens - 1) // page_tokens for q in seqs) + 1
    max_context = 131072 if churn else -(-(max(q["pos"] for q in seqs) + 64) // page_tokens) * page_tokens
    if churn:
        pages = int(pages * 1.25)   # room for admissions that are longer than the completions they replace
    n_sessions, max_seqs, max_rows = len(seqs), len(seqs), max(rows, 32)
    if chunk_rows:
        pages += chunk_rows // page_tokens + 1
        n_sessions, max_context = n_sessions + 1, max(max_context, chunk_rows + 64)
    ctx = lbm.Context(cfg, sessions=n_sessions, max_context=max_context, page_tokens=page_tokens,
                      pool_pages=pages, max_seqs=max_seqs, max_rows=max_rows, gemm_impl=args.gemm_impl, use_graph=1,
                      device=local_rank, debug_rows=0, pdl=args.pdl, chain=args.chain, gating_stream=args.gating_stream, fuse_swiglu=args.fuse_swiglu)
    ctx.synth_weights(0)
    pool = PagePool(lbm, pages, page_tokens, n_sessions, max_context // page_tokens)  # ids 1 .. pages - 1 (page 0 is reserved)
    if chunk_rows:
        table = pool.ensure(len(seqs), chunk_rows)
        ctx.kv_table_set(len(seqs), np.arange(len(table), dtype=np.int32), table)
    for q in seqs:
        table = pool.ensure(q["slot"], q["pos"] + 64)
        ctx.kv_table_set(q["slot"], np.arange(len(table), dtype=np.int32), table)
        ctx.synth_kv(q["slot"], q["pos"], rank)
        ctx.synth_state(q["slot"], rank)
    return ctx, pool, max_context


def device_timed_steps(ctx, dist, seqs, flags, steps, warmup):
    """Descriptors staged once, `warmup` untimed graph replays, then `steps` replays between two CUDA events on the
    context's stream, bracketed by a barrier + synchronize on both sides.  Returns this rank's milliseconds."""
    ctx.stage(seqs, flags)
    for _ in range(warmup):
        ctx.launch()
    res = ctx.fetch()
    assert all(r.status == 0 and r.n_path == q["accept"] for r, q in zip(res, seqs)), "acceptance differs from the imposed paths"
    dist.barrier()
    ctx.sync()
    ctx.timer_begin()
    for _ in range(steps):
        ctx.launch()
    ms = ctx.timer_end()
    ctx.sync()
    dist.barrier()
    return ms


def churn64_sharded(lbm, dist, args, rank, local_rank, world):
    """The 64-sequence batch (contexts lognormal up to 128k, trees of 1-32 rows) sharded by sequence over the ranks (whole
    sequences, estimated step time balanced: shard_sequences), timed on the device: total work fixed, so strong scaling.  Each
    rank reads the full weights for its share of the rows; no data-path collective."""
    cfg = model_for(lbm, "churn64", args.layers)
    seqs = workload("churn64", rank, cfg.vocab)
    ctx, _, _ = setup_context(lbm, cfg, seqs, args, rank, local_rank, True)
    steps = max(3, min(args.steps, 10))
    ms = device_timed_steps(ctx, dist, seqs, lbm.STEP_COMMIT, steps, 3) / steps
    fam, _ = ctx.profile_step()
    ctx.fetch()
    ctx.close()
    rows, kv_pos, accept = sum(len(q["tokens"]) for q in seqs), sum(q["pos"] for q in seqs), sum(q["accept"] for q in seqs)
    worst = dist.max(ms)
    per_rank = [dist.select(r, v) for r in range(world) for v in (rows, kv_pos, ms)]
    return {"sequences": 64, "scaling": "strong", "sharding": "whole sequences, estimated step time balanced (rows, KV positions, sequences; costliest first onto the lightest GPU)",
            "steps": steps, "ms_per_step": worst, "tokens_per_s": dist.sum(rows) / (worst * 1e-3),
            "accepted_tokens_per_s": dist.sum(accept) / (worst * 1e-3),
            "per_rank": [{"rows": int(per_rank[3 * r]), "kv_positions": int(per_rank[3 * r + 1]), "ms_per_step": per_rank[3 * r + 2]}
                         for r in range(world)],
            "rank0_family_ms": {"weight_gemms": fam[0], "attention": fam[1], "deltanet": fam[2], "norm_quant_elementwise": fam[3],
                                "head_argmax": fam[4], "pack_accept_compact_commit": fam[5]}}


def run_ours(args, rank, local_rank, world):
    lbm = importlib.import_module("ling-engine_b200")
    lbm.lib()
    if lbm.lib().ling_b200_device_count() < 1:
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path")
    dist = Dist(world, local_rank)
    cfg = model_for(lbm, args.workload, args.layers)
    seqs = workload(args.workload, rank, cfg.vocab)
    rows = sum(len(q["tokens"]) for q in seqs)
    churn = args.workload == "churn64"
    ctx, pool, max_context = setup_context(lbm, cfg, seqs, args, rank, local_rank, churn)
    flags = lbm.STEP_COMMIT
    clocks = ClockSampler(local_rank)

    # ---- device-timed: descriptors staged once, K graph replays
    clocks.start()
    ms = device_timed_steps(ctx, dist, seqs, flags, args.steps, args.warmup if args.quick else max(args.warmup, 3))
    ms = dist.max(ms)
    launches = ctx.launch_count()

    if args.quick:
        clk = clocks.stop()
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": dist.sum(rows) / (ms / args.steps * 1e-3), "unit": UNIT,
                              "ms_per_step": ms / args.steps, "launches_per_step": launches, "quick": True, "clocks": clk}), flush=True)
        ctx.close()
        dist.close()
        return

    # ---- end to end: host buffers in, host buffers out, every step
    for _ in range(2):
        ctx.verify_step(seqs, flags)
    dist.barrier()
    churn_rng, admitted, reused = np.random.default_rng(7 + rank), 0, 0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        if churn:   # ~10 % of the sequences complete and as many are admitted on the pages they gave back
            a, r = churn_step(ctx, pool, seqs, churn_rng, max_context)
            admitted, reused = admitted + a, reused + r
        ctx.verify_step(seqs, flags)
    e2e_s = dist.max(time.perf_counter() - t0)
    clk = clocks.stop()
    dist.barrier()

    # ---- the GEMM's own time: one eager replay with CUDA events around every launch
    ctx.stage(seqs, flags)
    fam, _ = ctx.profile_step()
    ctx.fetch()
    ctx.stage(seqs, flags)
    chain_ms = ctx.gemm_chain_ms(5)   # the same 257 launches back to back, nothing between them
    peak, peak_kind = measured_peaks()
    wbytes = ctx.weight_bytes()
    alg = algorithmic_bytes(cfg, seqs, wbytes)
    n_gemm = 4 * cfg.layers + 1
    gemm_ms = fam[0] + fam[4]  # weight GEMMs + the head GEMM with its fused argmax, an event pair around each launch
    per_launch = wbytes / (gemm_ms * 1e-3) / 1e9 if gemm_ms > 0 else 0.0
    achieved = wbytes / (chain_ms * 1e-3) / 1e9 if chain_ms > 0 else 0.0
    step_ms = ms / args.steps
    total_rows = dist.sum(rows)
    total_accept = dist.sum(sum(q["accept"] for q in seqs))
    churn_line = None
    if args.workload == "single" and args.layers == 64 and not args.no_churn64:
        # beside the headline: the 64-sequence batch sharded by sequence over the same GPUs (the contexts are closed one after
        # the other: two sets of weights are never resident together)
        ctx.close()
        ctx = None
        churn_line = churn64_sharded(lbm, dist, args, rank, local_rank, world)
    if rank == 0:
        cpu_v, cpu_est, cpu_desc = (None, None, "skipped (--no-cpu-baseline)")
        cores = max(1, min(os.cpu_count() or 1, 64))
        if churn:
            cpu_desc = "skipped: 64 sequences of up to 128k context do not fit a bounded CPU sample"
        elif not args.no_cpu_baseline and world == 1:
            cpu_v, cpu_est, cpu_desc = cpu_sample(lbm, cfg, seqs, cores)
        line = {
            "metric": METRIC, "value": total_rows / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": args.workload, "model": "27B-class hybrid, %d layers" % cfg.layers if args.workload != "toy" else "toy",
                       "rows_per_gpu": rows, "sequences_per_gpu": len(seqs), "contexts": [q["pos"] for q in seqs],
                       "parallelism": "replicas, sequences sharded over %d GPU(s), no collective" % world,
                       "l2": "inputs larger than L2 (weights %.1f GB per step), no flush" % (wbytes / 1e9),
                       "churn": ({"admitted_per_step": admitted / args.steps, "pages_reused_per_step": reused / args.steps}
                                 if churn else None),
                       "pdl": args.pdl, "chain": args.chain, "gemm_impl": "tcgen05" if args.gemm_impl == 0 else "cuda-core cross-check"},
            "accepted_tokens_per_s": total_accept / (step_ms * 1e-3),
            "hbm_fraction_weights_plus_kv": (alg["weights"] + alg["kv"]) / (step_ms * 1e-3) / 1e9 / peak,
            "algorithmic_bytes": alg,
            "family_ms": {"weight_gemms": fam[0], "attention": fam[1], "deltanet": fam[2], "norm_quant_elementwise": fam[3],
                          "head_argmax": fam[4], "pack_accept_compact_commit": fam[5]},
            "e2e": {"value": total_rows * args.steps / e2e_s, "unit": UNIT, "ms_per_step": e2e_s / args.steps * 1e3,
                    "h2d_bytes_per_step": int(ctx_stage_bytes(lbm, len(seqs))), "d2h_bytes_per_step": int(len(seqs) * __import__("ctypes").sizeof(lbm.SeqResult) + 4)},
            "gpu_launches": launches * args.steps,
            "launches_per_step": launches,
            "roofline": {"bound": "hbm", "kernel": "gemm_fp8_tcgen05_kernel (%d launches per step)" % n_gemm,
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                         # DRAM read + write bytes per launch: 1.021 x the algorithmic bytes, the ratio ncu measured on the
                         # gate|up launch (24 x 34816 x 5120), scaled to the average launch
                         "traffic": 1.021 * wbytes / n_gemm, "traffic_source": "ncu dram__bytes ratio 1.021 of one gate|up launch, scaled by bytes",
                         "bytes_per_launch_avg": wbytes / n_gemm, "ms_per_launch_avg": chain_ms / n_gemm,
                         "ms_per_step": chain_ms,
                         # the same launches with an event pair around each one (eager replay): a lower bound
                         "per_launch_events": {"ms_per_step": gemm_ms, "achieved": per_launch, "frac": per_launch / peak}},
            "cpu_baseline": {"value": cpu_v, "unit": UNIT, "cores": cores, "kind": "port", "sample": cpu_desc,
                             "est_ms_per_step": None if cpu_est is None else cpu_est * 1e3},
            "churn64": churn_line,
            "clocks": clk,
        }
        print(json.dumps(line), flush=True)
    if ctx is not None:
        ctx.close()
    dist.close()


def run_mixed(args, rank, local_rank, world):
    """The mixed ragged pass: one 4096-token prefill chunk through the NVFP4 prefill path -- in the 48 DeltaNet layers the mixer
    (norm, in projections, conv, gating, chunked delta rule, gated norm, out projection), in all 64 layers the feed-forward
    block (norm + quantize, gate|up with fused SwiGLU, down into the residual) -- beside 8 decoding sequences' verify step
    (24-node trees, contexts uniform in 1k-32k) on every GPU.  The 16 full-attention layers' mixer on the prefill path
    (attention over the chunk's 4096 query rows) is not part of this build: said in `config`.  --chunk-scope ffn leaves the
    DeltaNet mixers out too (the feed-forward blocks alone).
      value     rows per second with both halves launched together on their own streams (device events per half; the
                step's time is the longer of the two totals, max over ranks)
      e2e       the same through the host-buffer calls: the chunk's residual copied in and out (pinned staging) and the
                verify step's descriptors in / results out, inside the timed region
      roofline  the NVFP4 GEMMs (gemm_nvfp4_tcgen05_kernel) timed alone at the chunk's two shapes against the NVFP4 tensor
                rate measured on this GPU in the same run (bound: tensor)."""
    import threading
    lbm = importlib.import_module("ling-engine_b200")
    lbm.lib()
    if lbm.lib().ling_b200_device_count() < 1:
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path")
    dist = Dist(world, local_rank)
    cfg = model_for(lbm, "mixed", args.layers)
    seqs = workload("mixed", rank, cfg.vocab)
    rows = sum(len(q["tokens"]) for q in seqs)
    chunk = 4096
    whole = args.chunk_scope == "all"
    ctx, _, _ = setup_context(lbm, cfg, seqs, args, rank, local_rank, False, chunk if whole else 0)
    ffn = lbm.Nvfp4Ffn(cfg.layers, cfg.hidden, cfg.intermediate, chunk, seed=rank, device=local_rank)
    with_mixers = args.chunk_scope != "ffn"
    n_mix = sum(1 for l in range(cfg.layers) if l % 4 != 3) if with_mixers else 0
    if with_mixers:
        ffn.add_mixers(cfg.lin_k_heads, cfg.lin_v_heads, 4, seed=rank)
    if whole:
        return run_mixed_whole(args, lbm, dist, cfg, ctx, ffn, seqs, rows, chunk, n_mix, rank, local_rank, world)
    h0 = np.random.default_rng(50 + rank).standard_normal((chunk, cfg.hidden)).astype(np.float32)
    ffn.set_residual(h0)
    flags, K, W = lbm.STEP_COMMIT, args.steps, max(args.warmup, 3)
    clocks = ClockSampler(local_rank)
    ctx.stage(seqs, flags)
    for _ in range(W):
        ctx.launch()
    ffn.launch(chunk, W)
    ffn.wait()
    res = ctx.fetch()
    assert all(r.status == 0 and r.n_path == q["accept"] for r, q in zip(res, seqs)), "acceptance differs from the imposed paths"
    # ---- each half alone
    ffn.launch(chunk, K)
    ffn_alone = ffn.wait() / K
    ctx.timer_begin()
    for _ in range(K):
        ctx.launch()
    verify_alone = ctx.timer_end() / K
    # ---- both together: the chunk's stack is enqueued on its stream, the verify graphs on theirs
    clocks.start()
    dist.barrier()
    ctx.sync()
    ffn.launch(chunk, K)
    ctx.timer_begin()
    for _ in range(K):
        ctx.launch()
    verify_ms = ctx.timer_end()
    ffn_ms = ffn.wait()
    ctx.sync()
    dist.barrier()
    step_ms = dist.max(max(verify_ms, ffn_ms)) / K
    launches = ctx.launch_count() + 3 * cfg.layers + 10 * n_mix
    # ---- end to end: host buffers in and out of both halves every step (two host threads, one per half)
    out = [None]
    def chunk_thread():
        for _ in range(K):
            out[0] = ffn.forward(h0)
    ctx.verify_step(seqs, flags)
    ffn.forward(h0)
    dist.barrier()
    t0 = time.perf_counter()
    th = threading.Thread(target=chunk_thread)
    th.start()
    for _ in range(K):
        ctx.verify_step(seqs, flags)
    th.join()
    e2e_s = dist.max(time.perf_counter() - t0)
    clk = clocks.stop()
    assert np.isfinite(out[0]).all()
    # ---- the NVFP4 GEMMs alone, and the tensor pipe's measured rate
    gu_ms = lbm.nvfp4_gemm_bench(chunk, cfg.intermediate, cfg.hidden, fused=True, iters=10, device=local_rank)
    dn_ms = lbm.nvfp4_gemm_bench(chunk, cfg.hidden, cfg.intermediate, fused=False, iters=10, device=local_rank)
    peak_burst, _ = lbm.fp4_tensor_peak(20000, device=local_rank)
    peak_sustained, _ = lbm.fp4_tensor_peak(400000, device=local_rank)
    flops = 2.0 * chunk * cfg.intermediate * cfg.hidden
    achieved = 3 * flops / ((gu_ms + dn_ms) * 1e-3) / 1e12
    total_rows = dist.sum(rows + chunk)
    if rank == 0:
        line = {
            "metric": METRIC, "value": total_rows / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4 (e2m1 x ue4m3 per 16, fp32 accumulate) chunk + fp8_e4m3 verify", "data": "synthetic",
            "config": {"workload": "mixed", "model": "27B-class hybrid, %d layers" % cfg.layers, "chunk_rows": chunk,
                       "chunk_scope": ("the %d DeltaNet layers' mixers (norm, NVFP4 in projections, conv, gating, chunked delta rule, gated "
                                       "norm, NVFP4 out projection) and every layer's feed-forward block; the %d full-attention layers' "
                                       "mixer on the prefill path is not built" % (n_mix, cfg.layers - n_mix)) if with_mixers else
                                      "feed-forward blocks only (norm+quantize, gate|up+SwiGLU, down)",
                       "decode_sequences": len(seqs), "decode_rows": rows, "contexts": [q["pos"] for q in seqs],
                       "parallelism": "replicas, one chunk and one decode batch per GPU, no collective",
                       "l2": "inputs larger than L2 (FP8 weights %.1f GB + NVFP4 chunk weights %.1f GB per step), no flush"
                             % (ctx.weight_bytes() / 1e9, (3 * cfg.layers * cfg.intermediate + n_mix * (4 * cfg.lin_v_heads + 2 * cfg.lin_k_heads) * 128)
                                * cfg.hidden * 0.5625 / 1e9)},
            "halves_ms": {"chunk_alone": ffn_alone, "verify_alone": verify_alone, "serial": ffn_alone + verify_alone,
                          "chunk_together": ffn_ms / K, "verify_together": verify_ms / K},
            "e2e": {"value": total_rows * K / e2e_s, "unit": UNIT, "ms_per_step": e2e_s / K * 1e3,
                    "h2d_bytes_per_step": int(h0.nbytes + ctx_stage_bytes(lbm, len(seqs))),
                    "d2h_bytes_per_step": int(h0.nbytes + len(seqs) * __import__("ctypes").sizeof(lbm.SeqResult) + 4)},
            "gpu_launches": launches * K, "launches_per_step": launches,
            "roofline": {"bound": "tensor", "kernel": "gemm_nvfp4_tcgen05_kernel (gate|up fused %d x %d x %d, down %d x %d x %d)"
                         % (chunk, 2 * cfg.intermediate, cfg.hidden, chunk, cfg.hidden, cfg.intermediate),
                         "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s", "frac": achieved / peak_burst,
                         "peak_kind": "measured in this run: tcgen05.mma kind::mxf4nvf4.block_scale on resident operands, 6 ms burst",
                         "peak_sustained": peak_sustained, "traffic": None,
                         "ms_per_launch": {"gate_up_swiglu": gu_ms, "down": dn_ms}},
            "cpu_baseline": {"value": None, "unit": UNIT, "cores": 0, "kind": "port",
                             "sample": "not timed for this workload (the single-stream line carries the CPU baseline)"},
            "clocks": clk,
        }
        print(json.dumps(line), flush=True)
    ffn.close()
    ctx.close()
    dist.close()


def run_mixed_whole(args, lbm, dist, cfg, ctx, ffn, seqs, rows, chunk, n_mix, rank, local_rank, world):
    """--chunk-scope all: the prefill chunk through EVERY layer -- the DeltaNet layers' NVFP4 mixers, the full-attention layers'
    mixers (the verify model's own FP8 q|k|v and o projections, the step's prepare / attention / combine kernels over the chunk's
    rows as 32-row chains of the chunk's session, 64 chains a launch) and all NVFP4 feed-forward blocks -- beside the 8 decoding
    sequences' verify step.  The chunk's attention layers run on a sibling context (its own step buffers on the verify
    context's weights, pages and sessions), so the two halves run together as in the default scope: the chunk's stack from a
    second host thread (its attention layers wait for the device between launches of chains), the verify graphs from the main
    one; a step's time is the longer of the two halves' device times (max over ranks)."""
    import threading
    n_attn = cfg.layers - n_mix
    sib = ctx.sibling(64, 2048)
    ffn.attach_context(sib, len(seqs), 0, 4)
    h0 = np.random.default_rng(50 + rank).standard_normal((chunk, cfg.hidden)).astype(np.float32)
    ffn.set_residual(h0)
    flags, K, W = lbm.STEP_COMMIT, args.steps, max(args.warmup, 3)
    clocks = ClockSampler(local_rank)
    ctx.stage(seqs, flags)
    for _ in range(W):
        ctx.launch()
    ffn.launch(chunk, W)
    ffn.wait()
    res = ctx.fetch()
    assert all(r.status == 0 and r.n_path == q["accept"] for r, q in zip(res, seqs)), "acceptance differs from the imposed paths"
    # each half alone
    ffn.launch(chunk, K)
    f_alone = ffn.wait() / K
    ctx.timer_begin()
    for _ in range(K):
        ctx.launch()
    v_alone = ctx.timer_end() / K
    # both together
    clocks.start()
    dist.barrier()
    ctx.sync()
    box = [0.0]

    def chunk_half():
        ffn.launch(chunk, K)
        box[0] = ffn.wait()
    th = threading.Thread(target=chunk_half)
    th.start()
    ctx.timer_begin()
    for _ in range(K):
        ctx.launch()
    v_tot = ctx.timer_end()
    th.join()
    f_tot = box[0]
    ctx.sync()
    dist.barrier()
    step_ms = dist.max(max(f_tot, v_tot)) / K
    passes = -(-chunk // 2048)
    launches = ctx.launch_count() + 3 * cfg.layers + 10 * n_mix + 8 * passes * n_attn
    # end to end: the chunk's residual in and out of host memory (second thread), the verify step's descriptors in and results out
    outs = [None]

    def chunk_thread():
        for _ in range(K):
            outs[0] = ffn.forward(h0)
    ffn.forward(h0), ctx.verify_step(seqs, flags)
    dist.barrier()
    t0 = time.perf_counter()
    th = threading.Thread(target=chunk_thread)
    th.start()
    for _ in range(K):
        ctx.verify_step(seqs, flags)
    th.join()
    e2e_s = dist.max(time.perf_counter() - t0)
    out = outs[0]
    clk = clocks.stop()
    assert np.isfinite(out).all()
    gu_ms = lbm.nvfp4_gemm_bench(chunk, cfg.intermediate, cfg.hidden, fused=True, iters=10, device=local_rank)
    dn_ms = lbm.nvfp4_gemm_bench(chunk, cfg.hidden, cfg.intermediate, fused=False, iters=10, device=local_rank)
    peak_burst, _ = lbm.fp4_tensor_peak(20000, device=local_rank)
    flops = 2.0 * chunk * cfg.intermediate * cfg.hidden
    achieved = 3 * flops / ((gu_ms + dn_ms) * 1e-3) / 1e12
    total_rows = dist.sum(rows + chunk)
    if rank == 0:
        line = {
            "metric": METRIC, "value": total_rows / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4 (e2m1 x ue4m3 per 16, fp32 accumulate) chunk, fp8_e4m3 attention projections and KV + fp8_e4m3 verify",
            "data": "synthetic",
            "config": {"workload": "mixed", "model": "27B-class hybrid, %d layers" % cfg.layers, "chunk_rows": chunk,
                       "chunk_scope": "every layer: %d DeltaNet mixers (NVFP4), %d full-attention mixers (FP8 projections, attention over the "
                                      "chunk's rows as 32-row chains through the step's kernels, %d launches of up to 64 chains a layer) and "
                                      "%d NVFP4 feed-forward blocks; beside the verify step (the attention layers on a sibling context)"
                                      % (n_mix, n_attn, passes, cfg.layers),
                       "decode_sequences": len(seqs), "decode_rows": rows, "contexts": [q["pos"] for q in seqs],
                       "parallelism": "replicas, one chunk and one decode batch per GPU, no collective",
                       "l2": "inputs larger than L2 (FP8 weights %.1f GB + NVFP4 chunk weights per step), no flush" % (ctx.weight_bytes() / 1e9)},
            "halves_ms": {"chunk_alone": f_alone, "verify_alone": v_alone, "serial": f_alone + v_alone, "chunk_together": f_tot / K,
                          "verify_together": v_tot / K},
            "e2e": {"value": total_rows * K / e2e_s, "unit": UNIT, "ms_per_step": e2e_s / K * 1e3,
                    "h2d_bytes_per_step": int(h0.nbytes + ctx_stage_bytes(lbm, len(seqs))),
                    "d2h_bytes_per_step": int(h0.nbytes + len(seqs) * __import__("ctypes").sizeof(lbm.SeqResult) + 4)},
            "gpu_launches": launches * K, "launches_per_step": launches,
            "roofline": {"bound": "tensor", "kernel": "gemm_nvfp4_tcgen05_kernel (gate|up fused %d x %d x %d, down %d x %d x %d)"
                         % (chunk, 2 * cfg.intermediate, cfg.hidden, chunk, cfg.hidden, cfg.intermediate),
                         "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s", "frac": achieved / peak_burst,
                         "peak_kind": "measured in this run: tcgen05.mma kind::mxf4nvf4.block_scale on resident operands, 6 ms burst",
                         "traffic": None, "ms_per_launch": {"gate_up_swiglu": gu_ms, "down": dn_ms}},
            "cpu_baseline": {"value": None, "unit": UNIT, "cores": 0, "kind": "port",
                             "sample": "not timed for this workload (the single-stream line carries the CPU baseline)"},
            "clocks": clk,
        }
        print(json.dumps(line), flush=True)
    ffn.close()
    sib.close()
    ctx.close()
    dist.close()


def run_served(args, rank, local_rank, world):
    """The 64-sequence continuous-batching workload produced by the scheduler loop itself (the headless serving driver,
    ling-engine_b200/ling_serve_headless: requests queue up, are admitted into session slots and the KV page pool, share
    verify passes, finish and hand their pages on) instead of a scripted batch.  Sessions and requests are sharded over the
    ranks (whole requests, no collective).  value = tree rows verified per second of pass time, summed over ranks with the
    slowest rank's pass time; the driver's own counters ride along."""
    exe = os.path.join(ROOT, "ling-engine_b200", "ling_serve_headless")
    if not os.path.exists(exe):
        importlib.import_module("ling-engine_b200.build").build()
    dist = Dist(world, local_rank)
    sessions, requests = max(1, 64 // world), max(1, 96 // world)
    cmd = [exe, "--layers", str(args.layers), "--sessions", str(sessions), "--batch", str(sessions), "--requests", str(requests),
           "--seed", str(1 + rank), "--device", str(local_rank), "--max-tokens", "128"]
    if args.systems > 0:  # prompts begin with one of a few shared system messages; the prefix KV store keeps each once
        cmd += ["--systems", str(args.systems), "--prefix-kv-mb", str(args.prefix_kv_mb)]
    if args.pool_pages > 0:
        cmd += ["--pool-pages", str(args.pool_pages)]
    clocks = ClockSampler(local_rank)
    clocks.start()
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=3000)
    clk = clocks.stop()
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    if out.returncode != 0 or not lines:
        raise SystemExit("ling_serve_headless failed (%d): %s" % (out.returncode, out.stderr[-2000:]))
    d = json.loads(lines[-1])
    rows = d["rows_per_pass"] * d["decode_passes"]
    pass_s = dist.max(d["pass_seconds"])
    total_rows, total_tokens, passes = dist.sum(rows), dist.sum(d["produced_tokens"]), dist.sum(d["decode_passes"])
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": total_rows / pass_s, "unit": UNIT, "n_gpus": world, "steps": int(passes), "warmup": 0,
            "ms_per_step": pass_s / max(1.0, passes / world) * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "served64: 96 queued requests through 64 session slots under the scheduler loop", "model":
                       "27B-class hybrid, %d layers" % args.layers, "parallelism": "requests and sessions sharded over %d GPU(s), no collective" % world,
                       "l2": "inputs larger than L2 (weights 26.4 GB per pass), no flush"},
            "accepted_tokens_per_s": total_tokens / pass_s, "rank0_driver": d,
            "gpu_launches": int(d["launches_last_pass"] * passes), "clocks": clk}), flush=True)
    dist.close()


def run_micro_gemm(args):
    """One weight GEMM alone (synthetic FP8 weights and activations resident in HBM), `iters` launches back to back after
    three warm-up launches; the small case the profiler captures.  A matrix smaller than L2 is served from L2 here."""
    lbm = importlib.import_module("ling-engine_b200")
    M, N, K = (int(x) for x in args.shape.split(","))
    if args.micro == "gdn-chunk":
        # the prefill path's chunked delta rule alone: M rows of one sequence, the 27B model's 16 key / 48 value heads of 128
        ms = lbm.gdn_chunk_bench(16, 48, M, iters=args.iters)
        print(json.dumps({"micro": "gdn_chunk_prepare_kernel + gdn_chunk_apply_kernel", "rows": M, "heads": [16, 48], "iters": args.iters, "us_per_launch": ms * 1e3,
                          "us_per_32_token_chunk": ms * 1e3 / ((M + 31) // 32), "rows_per_s": M / (ms * 1e-3)}), flush=True)
        return
    if args.micro == "sparse-head":
        # the drafter's sparse head: the selection of the rows a draft step scores (M step rows against the 248,320 x 256 BF16 factor)
        V, dyn, cap = 248320, 16384, 32768
        sc_ms, all_ms = lbm.sparse_select_bench(V, M, dyn, cap, iters=args.iters)
        peak = measured_peaks()[0]
        gbs = V * 512 / (sc_ms * 1e-3) / 1e9
        print(json.dumps({"micro": "sparse_scores_kernel (+ sparse_level x 3, count, scan, scatter)", "vocab": V, "step_rows": M, "dynamic": dyn, "cap": cap,
                          "iters": args.iters, "us_scores": sc_ms * 1e3, "us_selection": all_ms * 1e3,
                          "roofline": {"bound": "hbm", "achieved": gbs, "unit": "GB/s", "peak": peak, "frac": gbs / peak if peak else None,
                                       "bytes": "vocab x 512 (the factor, read once)"}}), flush=True)
        return
    if args.micro == "gdn-layer":
        # one DeltaNet layer's whole mixer on the prefill path (eight launches), M rows, the 27B model's widths
        layer = lbm.PrefillGdnLayer(5120, 16, 48, M, seed=1)
        ms = layer.bench(M, args.iters)
        layer.close()
        print(json.dumps({"micro": "prefill DeltaNet mixer (rmsnorm_quant, 2 NVFP4 GEMMs, ab_gating, conv_rows, gdn_chunk, gated_norm_quant, NVFP4 GEMM)",
                          "rows": M, "iters": args.iters, "ms_per_layer": ms, "rows_per_s": M / (ms * 1e-3)}), flush=True)
        return
    if args.micro in ("nvfp4", "nvfp4-swiglu"):
        # one NVFP4 GEMM alone: N weight rows (N features from 2 N rows in the fused gate|up form), operands resident
        fused = args.micro == "nvfp4-swiglu"
        ms = lbm.nvfp4_gemm_bench(M, N, K, fused=fused, iters=args.iters)
        flops = 2.0 * M * N * K * (2 if fused else 1)
        print(json.dumps({"micro": "gemm_nvfp4_tcgen05_kernel", "fused_swiglu": fused, "shape": [M, N, K], "iters": args.iters,
                          "us_per_launch": ms * 1e3, "TFLOP_per_s": flops / (ms * 1e-3) / 1e12,
                          "operand_bytes": int((M + N * (2 if fused else 1)) * K * 0.5625)}), flush=True)
        return
    lbm.lib().ling_b200_set_pdl(args.pdl)
    ms = lbm.gemm_fp8_bench(M, N, K, impl=args.gemm_impl, splits=0, iters=args.iters)
    lbm.lib().ling_b200_set_pdl(0)
    peak, kind = measured_peaks()
    nbytes = N * K + (K // 128) * N * 4
    print(json.dumps({"micro": "gemm_fp8_tcgen05_kernel", "shape": [M, N, K], "iters": args.iters, "us_per_launch": ms * 1e3,
                      "weight_bytes": nbytes, "GB_per_s": nbytes / (ms * 1e-3) / 1e9, "frac_of_%s_hbm" % kind: nbytes / (ms * 1e-3) / 1e9 / peak,
                      "larger_than_l2": nbytes > 126e6, "pdl": args.pdl}), flush=True)


def ctx_stage_bytes(lbm, n_seqs):
    # the host-written descriptor block: count, per-sequence records, parent / token / forced-argmax rows
    return 16 + ((n_seqs * 24 + 15) // 16) * 16 + 3 * n_seqs * 32 * 4


# What a GPU's share of a many-sequence step costs, in milliseconds: per 32 tree rows (the step runs in capacity classes of 32
# rows and the GEMMs pick the token tile with the least padding, so their time follows the padded rows: 63 ms for 1152),
# per tree row (norms, the DeltaNet paths), per KV position (attention) and per sequence; the last three fitted to the
# per-rank step times of the 64-sequence batch on four GPUs.  Only the ratios matter.
COST_PER_32_ROWS, COST_PER_ROW, COST_PER_KV, COST_PER_SEQ = 63.0 / 36, 0.03, 5.0e-5, 0.3


def shard_cost(contexts, rows, members):
    """Estimated step time of the GPU that gets the sequences `members`."""
    r = sum(rows[i] for i in members)
    return (COST_PER_32_ROWS * -(-r // 32) + COST_PER_ROW * r + COST_PER_KV * sum(contexts[i] for i in members)
            + COST_PER_SEQ * len(members))


def shard_sequences(contexts, world, rows=None):
    """Sequence sharding for a many-sequence batch: sequences are independent (own KV pages, own state slot, own tree), so
    each goes whole to one GPU (the weights are replicated).  Without `rows`: longest context first onto the GPU with the
    fewest KV positions so far.  With the sequences' tree rows the estimated step time (shard_cost) is balanced instead:
    costliest sequence first onto the GPU whose estimate grows least, then single moves and swaps between the slowest GPU
    and the others while they lower the slowest estimate.  Returns, per rank, the indices of its sequences."""
    n = len(contexts)
    shards = [[] for _ in range(world)]
    if rows is None:
        load = [0] * world
        for i in sorted(range(n), key=lambda i: (-contexts[i], i)):
            r = min(range(world), key=lambda k: (load[k], k))
            shards[r].append(i)
            load[r] += contexts[i]
        return [sorted(s) for s in shards]
    cost = lambda m: shard_cost(contexts, rows, m)
    for i in sorted(range(n), key=lambda i: (-cost([i]), i)):
        r = min(range(world), key=lambda k: (cost(shards[k] + [i]), k))
        shards[r].append(i)
    for _ in range(200):   # local search on the slowest GPU
        costs = [cost(m) for m in shards]
        worst = max(range(world), key=lambda k: (costs[k], -k))
        best = None
        for k in range(world):
            if k == worst:
                continue
            for i in shards[worst]:
                moved = max(cost([x for x in shards[worst] if x != i]), cost(shards[k] + [i]))
                cand = [(moved, i, None)]
                for j in shards[k]:
                    cand.append((max(cost([x for x in shards[worst] if x != i] + [j]), cost([x for x in shards[k] if x != j] + [i])), i, j))
                for c, a, b_ in cand:
                    others = max([costs[q] for q in range(world) if q not in (worst, k)] or [0.0])
                    if max(c, others) < costs[worst] - 1e-9 and (best is None or max(c, others) < best[0]):
                        best = (max(c, others), k, a, b_)
        if best is None:
            break
        _, k, a, b_ = best
        shards[worst].remove(a)
        shards[k].append(a)
        if b_ is not None:
            shards[k].remove(b_)
            shards[worst].append(b_)
    return [sorted(s) for s in shards]


def aggregate(dist, rows, accepted, ms_total, steps):
    """The whole-job figures from per-rank ones: units summed over ranks, time the maximum over ranks."""
    ms = dist.max(ms_total)
    return {"rows_per_s": dist.sum(rows) * steps / (ms * 1e-3), "accepted_per_s": dist.sum(accepted) * steps / (ms * 1e-3),
            "ms_per_step": ms / steps}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="single", choices=["single", "ragged4", "churn64", "served64", "mixed", "toy"])
    ap.add_argument("--layers", type=int, default=64, help="layers of the 27B-class stack (64 = the named configuration)")
    ap.add_argument("--gemm-impl", type=int, default=0)
    ap.add_argument("--pdl", type=int, default=1, help="programmatic dependent launch (bit-identical results; on by default)")
    ap.add_argument("--chain", type=int, default=0, help="layer segments of steps of at most 32 rows as persistent kernels with counter "
                    "dependencies (bit-identical results; measured slower than the separate launches, so off by default)")
    ap.add_argument("--gating-stream", type=int, default=0, help="0/1: the DeltaNet gating projections on a second stream beside the in "
                    "projection (default); -1: in the step's one stream")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-churn64", action="store_true", help="leave out the 64-sequence sharded batch reported beside the headline")
    ap.add_argument("--quick", action="store_true", help="device-timed steps only (no end-to-end, per-family or CPU legs): "
                    "the short run the profiler's launch list is taken from")
    ap.add_argument("--fuse-swiglu", type=int, default=0, help="1: silu(gate)*up and its FP8 copy written by the gate|up GEMM itself (measured slower; default 0: a kernel of its own)")
    ap.add_argument("--chunk-scope", default="ffn+gdn", choices=["ffn+gdn", "ffn", "all"], help="mixed: what the prefill chunk runs through")
    ap.add_argument("--systems", type=int, default=0, help="served64: prompts begin with one of this many shared system messages")
    ap.add_argument("--prefix-kv-mb", type=int, default=0, help="served64 with --systems: the prefix KV store's budget for saved states (0: store off)")
    ap.add_argument("--pool-pages", type=int, default=0, help="served64: KV page pool size (0: sized for the resident sessions)")
    ap.add_argument("--micro", default="", choices=["", "gemm", "nvfp4", "nvfp4-swiglu", "gdn-chunk", "gdn-layer", "sparse-head"], help="time one kernel alone on resident operands")
    ap.add_argument("--shape", default="24,34816,5120", help="--micro gemm: rows,N,K (default: the gate|up projection)")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    rank, local_rank, world = dist_env()
    if args.micro:
        return run_micro_gemm(args)
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus and world > 1:
        raise SystemExit("bench.py: --gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    if args.workload == "mixed":
        return run_mixed(args, rank, local_rank, world)
    if args.workload == "served64":
        return run_served(args, rank, local_rank, world)
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
