#!/usr/bin/env python
"""Benchmark of the encode-and-scan hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--vectors N_VECTORS] [--batch NQ]

Workload (N = 1): 10,000,000 x 1536 fp32 rows (anisotropic Gaussian, L2-normalised; synthetic stand-in for the
OpenAI-1536 embeddings the reference measures on), 4-bit codes, k = 10, an id-mapped index whose ids are a seeded
permutation of [1e9, 1e9 + n).  One step = one search batch of 1,024 queries.  `value` is queries/s with queries
and results resident in HBM; `e2e` is the same through the host API (pinned host queries in, host results out,
copies inside the timed region).  Extra keys on the same line: batch-1 latency, ingest rate, recall@10, filtered
searches, online mutation, a `parity` block (the device's codes, scales and scores re-derived by the CPU oracle on
the index the numbers were measured on) and `configs`: short legs on the other shapes of the baseline.
With N > 1 (torchrun, one rank per GPU) the same 10 M vectors are slot-sharded over the ranks
(turbovec_b200.sharded.ShardedIdMapIndex: round-robin chunks of 32 Ki slots) and every search ends in one NCCL
all-gather of result keys and one merge kernel (strong scaling).

`--impl reference` times the CPU restatement of the reference's algorithm (the reference is a Rust crate and
cannot be built without a Rust toolchain) on all host threads, on the same index size and batch.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DIM, BITS, K = 1536, 4, 10
METRIC = "search_qps_k10_10Mx1536_4bit_batch1024"
UNIT = "queries/s"
CHUNK = 1 << 18           # rows generated and ingested at a time (1.6 GB of fp32 at d1536)
ID_BASE = 10**9


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tensor_tflops": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tensor_tflops": 1400.0, "source": "fallback"}


def workload_config(n, dim, bits, nq):
    """The same text in both arms."""
    return {"workload": f"{n} x {dim} {bits}-bit, k={K}, batch {nq}",
            "l2": "inputs larger than L2: each step streams the whole code array"}


def ngroups(dim, bits):
    return dim // (4 if bits == 2 else 2)        # 3-bit codes sit in 4-bit fields


def fnv1a64(data: bytes) -> str:
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return f"{h:016x}"


# ------------------------------------------------------------------------------------------ data
def dim_scale(seed: int, dim: int):
    return np.exp(0.5 * np.random.default_rng(seed).standard_normal(dim)).astype(np.float32)


def gen_rows_torch(torch, device, scale_t, seed: int, chunk_id: int, rows: int):
    """Rows of global chunk `chunk_id`: identical for any GPU count."""
    g = torch.Generator(device=device)
    g.manual_seed(seed * 1_000_003 + chunk_id)
    x = torch.randn((rows, scale_t.numel()), generator=g, device=device, dtype=torch.float32) * scale_t
    x /= x.norm(dim=1, keepdim=True)
    return x.contiguous()


def gen_clustered_torch(torch, device, centres, seed: int, chunk_id: int, rows: int, sigma: float = 0.3):
    """Mixture of Gaussian clusters (centres N(0,1), within-cluster sigma, uniform weights), L2-normalised."""
    g = torch.Generator(device=device)
    g.manual_seed(seed * 1_000_003 + chunk_id)
    pick = torch.randint(0, centres.shape[0], (rows,), generator=g, device=device)
    x = centres[pick] + sigma * torch.randn((rows, centres.shape[1]), generator=g, device=device, dtype=torch.float32)
    x /= x.norm(dim=1, keepdim=True)
    return x.contiguous()


def gen_rows_numpy(seed: int, n: int, offset: int, dim: int = None):
    dim = dim or DIM
    s = dim_scale(seed, dim)
    x = np.random.default_rng(seed * 7919 + 13 + offset).standard_normal((n, dim)).astype(np.float32) * s
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    return np.ascontiguousarray(x, dtype=np.float32)


def seeded_ids(n: int):
    return (np.random.default_rng(5).permutation(n) + ID_BASE).astype(np.uint64)


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for j, n in enumerate(names) if any(len(r) > 2 + j and r[2 + j].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------ CPU arm
class CpuArm:
    """The reference's CPU algorithm on all host threads, on an index of the benchmark's full size: a 200,000-row
    sample is encoded by the oracle and its blocks are repeated (with slightly different per-copy scales, so that
    the copies do not tie) until the index holds `n_full` vectors, so that every step streams the full code array
    from DRAM.  With AVX-512 VNNI the restatement of the reference's fastest x86 kernel (permute-dot on the
    vector-major layout, search.rs:1392-1543) runs; otherwise the scalar oracle."""

    def __init__(self, n_full: int, nq: int):
        from oracle import oracle as O
        self.O, self.nq, self.cores = O, nq, os.cpu_count() or 1
        n_sample = 200_000
        simd = O.simd_available() and BITS == 4
        # without AVX-512 VNNI only the scalar oracle exists: it scans the sample alone and the rate is scaled
        reps = max(1, -(-n_full // n_sample)) if simd else 1
        self.n_full = n_full
        self.n = min(n_full, reps * n_sample) // 32 * 32 if n_full >= 32 else n_full
        x = gen_rows_numpy(1, n_sample, 0)
        enc = O.encode(x, BITS)
        blocked = O.packed_to_blocked(enc["packed"], BITS, DIM)
        self.simd = simd
        codes = O.to_vector_major(blocked, n_sample, DIM) if self.simd else blocked
        block_bytes = ngroups(DIM, BITS) * 32
        self.codes = np.tile(codes, reps)[: (self.n // 32) * block_bytes] if reps > 1 else codes[: (self.n // 32) * block_bytes]
        self.scales = np.concatenate([enc["scales"] * np.float32(1.0 - 1e-4 * r) for r in range(reps)])[: self.n].astype(np.float32)
        self.q = gen_rows_numpy(1, nq, 10_000_000)
        self.kernel = "avx512-vnni permute-dot restatement" if self.simd else "scalar restatement"
        self.reps = reps

    def step(self, nq=None):
        q = self.q if nq is None else self.q[:nq]
        t0 = time.perf_counter()
        if self.simd:
            self.O.search_simd(q, self.codes, self.scales, self.n, DIM, K, threads=self.cores)
        else:
            self.O.search(q, self.codes, self.scales, self.n, DIM, BITS, K)
        return time.perf_counter() - t0

    def run(self, steps: int, warmup: int, budget_s: float):
        """Times `steps` steps after `warmup`.  When a whole step would not fit `budget_s` in total, every step
        scans the full index with fewer queries (the rate per query does not depend on the batch beyond the
        kernel's own batch width of 8)."""
        self.step(8)                                             # first touch of the arrays
        probe_q = min(self.nq, 64)
        per_query = self.step(probe_q) / probe_q
        nq_step = self.nq
        if per_query * self.nq * (steps + warmup) > budget_s:
            nq_step = int(max(8, min(self.nq, budget_s / (per_query * (steps + warmup)))) // 8 * 8)
        for _ in range(warmup):
            self.step(nq_step)
        times = [self.step(nq_step) for _ in range(steps)]
        sec = float(np.mean(times))
        if self.n < self.n_full:
            scale = self.n / self.n_full
            return nq_step / sec * scale, sec * 1e3 / scale, (f"{nq_step} queries x {self.n} vectors per step, {steps} steps, {self.kernel}; "
                                                               f"rate scaled linearly to {self.n_full} vectors")
        sample = (f"{nq_step} of {self.nq} queries per step against all {self.n} vectors ({self.reps} copies of a 200,000-row encoded "
                  f"sample, {self.codes.nbytes / 1e9:.2f} GB of codes streamed per step), {steps} steps, {self.kernel}")
        return nq_step / sec, sec * 1e3, sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    arm = CpuArm(args.n, args.batch)
    qps, ms, sample = arm.run(args.steps, args.warmup, budget_s=200.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": qps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": workload_config(args.n, DIM, BITS, args.batch),
        "cpu_baseline": {"value": qps, "unit": UNIT, "cores": arm.cores, "kind": "port", "sample": sample},
        "e2e": {"value": qps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference is a Rust crate; no Rust toolchain on this box, so the C++ restatement of its algorithm is timed",
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------ parity
def parity_block(O, torch, local_idx, dim, bits, q_host, scores, local_slots, slice_rows_host, slice_slot0=0):
    """Re-derives on the CPU what the device holds and returned, on the measured index:
      codes / scales: the rows `slice_rows_host` (the fp32 inputs of local slots slice_slot0 ..) encoded by the oracle
        against the stored byte-groups and scales of those slots;
      scores: for every query the rows of its returned slots are fetched from the device and scored by the oracle's
        search; the scores must be bit-equal and the order the same."""
    ng = ngroups(dim, bits)
    out = {}
    enc = O.encode(slice_rows_host, bits)
    blocked = O.packed_to_blocked(enc["packed"], bits, dim).reshape(-1, ng, 32)
    bad_codes = bad_scales = 0
    for j in range(slice_rows_host.shape[0]):
        groups, scale = local_idx.get_row(slice_slot0 + j)
        bad_codes += int(np.count_nonzero(groups != blocked[j // 32, :, j % 32]))
        bad_scales += int(np.float32(scale).view(np.uint32) != enc["scales"][j].view(np.uint32))
    out["rows_compared"] = int(slice_rows_host.shape[0])
    out["codes_mismatch"] = bad_codes
    out["scales_mismatch"] = bad_scales
    equal, checked = True, 0
    for j in range(q_host.shape[0]):
        kk = local_slots.shape[1]
        mini = np.zeros(((kk + 31) // 32, ng, 32), np.uint8)      # the returned rows as a small blocked array, in rank order
        sc = np.zeros(kk, np.float32)
        for r in range(kk):
            groups, scale = local_idx.get_row(int(local_slots[j, r]))
            mini[r // 32, :, r % 32] = groups
            sc[r] = scale
        ref_s, ref_i = O.search(q_host[j:j + 1], mini.reshape(-1), sc, kk, dim, bits, kk)
        equal &= bool(np.array_equal(ref_i[0], np.arange(kk)) and np.array_equal(ref_s[0].view(np.uint32), scores[j].view(np.uint32)))
        checked += kk
    out["scores_checked"] = checked
    out["scores_bit_equal"] = bool(equal)
    return out


# ------------------------------------------------------------------------------------------ GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    import turbovec_b200 as T
    from oracle import oracle as O          # the checker of the parity block, outside every timed region

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: turbovec_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    pk = peaks()
    int8_peak = T.measure_int8_peak(local_rank) / 1e12           # TOP/s of this library's MMA form on this device: a burst
    int8_peak_sustained = T.measure_int8_peak(local_rank, 1.5) / 1e12   # and what it sustains at the power limit
    n_total, nq = args.n, args.batch
    ng = ngroups(DIM, BITS)

    # ---- build the index: every rank generates the same global chunks and keeps the rows of its slots ----
    scale_t = torch.from_numpy(dim_scale(1, DIM)).to(device)
    ids_all = seeded_ids(n_total)
    if world == 1:
        idx = T.IdMapIndex(DIM, BITS, device=local_rank)
        local = idx
    else:
        from turbovec_b200.sharded import ShardedIdMapIndex
        idx = ShardedIdMapIndex(DIM, BITS, device=device)
        local = idx.local
    for opt, val in ((T.OPT_MMA_MIN_BATCH, args.tc_min_batch), (T.OPT_INGEST_PIPELINE, args.ingest_pipeline),
                     (T.OPT_SMALL_SCAN, args.small_scan), (T.OPT_TC_WIDE, args.tc_wide),
                     (T.OPT_TC_EXPANDED, args.tc_expanded), (T.OPT_DENSE_PAIR, args.dense_pair)):
        if val is not None:
            local.set_option(opt, val)
    n_recall_q = 64
    q_all = torch.from_numpy(gen_rows_numpy(1, max(nq, n_recall_q), 10_000_000)).to(device)
    truth_s = torch.full((n_recall_q, K), -float("inf"), device=device)
    truth_i = torch.zeros((n_recall_q, K), dtype=torch.int64, device=device)
    ingest_ms, ingest_rows, ingest_launches = 0.0, 0, 0
    first_rows_host = None
    n_chunks = (n_total + CHUNK - 1) // CHUNK
    for c in range(n_chunks):
        c_lo, c_hi = c * CHUNK, min(n_total, (c + 1) * CHUNK)
        x = gen_rows_torch(torch, device, scale_t, 1, c, c_hi - c_lo)
        if c == 0:
            first_rows_host = x[:4096].cpu().numpy()             # global slots 0..4095 = rank 0's local slots 0..4095
        if c % world == rank:                                     # exact fp32 ground truth, one rank per chunk
            s, i = torch.topk(q_all[:n_recall_q] @ x.T, K, dim=1)
            truth_s, sel = torch.topk(torch.cat([truth_s, s], 1), K, dim=1)
            truth_i = torch.gather(torch.cat([truth_i, i + c_lo], 1), 1, sel)
        torch.cuda.synchronize()
        before = len(local)
        if world == 1:
            idx.add_with_ids_device(x.data_ptr(), c_hi - c_lo, DIM, ids_all[c_lo:c_hi])
            ms, nl = idx.last_main_kernel()
        else:
            ms, nl = idx.add_with_ids_device(x, ids_all[c_lo:c_hi]), 0
        rows = len(local) - before
        if c > 0 and c_hi - c_lo == CHUNK:            # the first chunk pays table set-up and allocation
            ingest_ms += ms
            ingest_rows += rows
            ingest_launches += nl
        del x
    n_local = len(local)

    d_scores = torch.empty((max(nq, n_recall_q), K), dtype=torch.float32, device=device)
    d_slots = torch.empty((max(nq, n_recall_q), K), dtype=torch.int64, device=device)
    q_dev = q_all[:nq].contiguous()
    q_host = q_dev.cpu().pin_memory()

    def step_device(qd, nqq):
        if world == 1:
            ke = idx.search_device(qd.data_ptr(), nqq, K, d_scores.data_ptr(), d_slots.data_ptr())
            return d_scores.view(-1)[: nqq * ke].view(nqq, ke), d_slots.view(-1)[: nqq * ke].view(nqq, ke)
        return idx.search_device(qd, K)              # local scan -> all-gather of keys -> merge kernel, all on the device

    def step_host(qh, nqq):
        """qh: pinned host tensor.  Host buffers in, host results out."""
        if world == 1:
            return idx.search(qh.numpy(), K)
        qd = qh.to(device, non_blocking=True)
        s, i = idx.search_device(qd, K)
        return s.cpu().numpy(), i.cpu().numpy()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, warmup, handle=None):
        handle = handle or local
        for _ in range(warmup):
            fn()
        barrier()
        scan_ms, scan_launches = 0.0, 0
        l0 = handle.launch_count
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
            ms, nl = handle.last_main_kernel()
            scan_ms += ms
            scan_launches += nl
        barrier()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        return dt, scan_ms, scan_launches, handle.launch_count - l0

    # The code array of one shard (>= 0.9 GB) is far larger than L2 (126 MB), so every step streams it from HBM.
    sampler = ClockSampler(local_rank)
    sampler.start()
    dt, scan_ms, scan_launches, launches = timed(lambda: step_device(q_dev, nq), args.steps, args.warmup)
    clocks = sampler.stop()
    dt_e2e, _, _, _ = timed(lambda: step_host(q_host, nq), args.steps, max(1, args.warmup // 2))
    q1_dev = q_dev[:1].contiguous()
    b1_steps = max(args.steps, 20)
    dt1, scan1_ms, scan1_launches, _ = timed(lambda: step_device(q1_dev, 1), b1_steps, args.warmup)
    q1_host = q_host[:1].contiguous().pin_memory()
    dt1_e2e, _, _, _ = timed(lambda: step_host(q1_host, 1), b1_steps, 2)

    # ---- recall@10 and the parity block, on the index just measured ----
    rs, ri = step_device(q_all[:n_recall_q].contiguous(), n_recall_q)
    rs, ri = rs.clone(), ri.clone()
    if world > 1:
        gs = [torch.empty_like(truth_s) for _ in range(world)]
        gi = [torch.empty_like(truth_i) for _ in range(world)]
        dist.all_gather(gs, truth_s)
        dist.all_gather(gi, truth_i)
        truth_s, sel = torch.topk(torch.cat(gs, 1), K, dim=1)
        truth_i = torch.gather(torch.cat(gi, 1), 1, sel)
    got, want = ri.cpu().numpy(), truth_i.cpu().numpy()
    recall = float(np.mean([len(set(got[j]) & set(want[j])) / K for j in range(n_recall_q)]))
    parity = None
    if not args.no_parity:
        # this rank's own top-k of the 64 queries (local slots), re-scored by the oracle from the stored rows
        ke = local.search_device(q_all[:n_recall_q].contiguous().data_ptr(), n_recall_q, K, d_scores.data_ptr(), d_slots.data_ptr())
        loc_s = d_scores.view(-1)[: n_recall_q * ke].view(n_recall_q, ke).cpu().numpy()
        loc_i = d_slots.view(-1)[: n_recall_q * ke].view(n_recall_q, ke).cpu().numpy()
        slice_rows = first_rows_host[: min(4096, n_local)] if rank == 0 else first_rows_host[:0]
        parity = parity_block(O, torch, local, DIM, BITS, q_all[:n_recall_q].cpu().numpy(), loc_s, loc_i, slice_rows)
        if world > 1:
            t = torch.tensor([parity["codes_mismatch"], parity["scales_mismatch"], 0 if parity["scores_bit_equal"] else 1,
                              parity["scores_checked"]], device=device, dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            parity.update(codes_mismatch=int(t[0]), scales_mismatch=int(t[1]), scores_bit_equal=bool(int(t[2]) == 0),
                          scores_checked=int(t[3]))
        # the merged result of the 64 queries: global slots and score bits, identical for every number of GPUs
        parity["ids_checksum"] = fnv1a64(np.ascontiguousarray(got, np.int64).tobytes())
        parity["scores_checksum"] = fnv1a64(np.ascontiguousarray(rs.cpu().numpy(), np.float32).tobytes())
        parity["checked_against"] = "oracle/tv_oracle.c (scalar restatement of the reference's encode and search)"

    # ---- filtered search (slot bitmask resident on the device): selectivity x layout of the allowed slots ----
    filtered = []
    if world == 1 and not args.no_filtered:
        rng = np.random.default_rng(7)
        nb_total = (n_local + 31) // 32
        for sel, kind in [(0.001, "random"), (0.01, "random"), (0.1, "random"), (0.5, "random"), (0.01, "range"), (0.1, "range")]:
            allowed = np.zeros(((n_local + 63) // 64) * 64, dtype=bool)
            if kind == "random":
                allowed[:n_local] = rng.random(n_local) < sel
            else:
                lo = int(rng.integers(0, max(1, n_local - int(sel * n_local))))
                allowed[lo: lo + int(sel * n_local)] = True
            live_blocks = int(allowed[: nb_total * 32].reshape(-1, 32).any(axis=1).sum())
            words = torch.from_numpy(np.packbits(allowed, bitorder="little").view(np.uint64).copy().view(np.int64)).to(device)
            f_steps = max(2, args.steps // 3)

            def step_f(qd, nqq):
                return idx.search_device(qd.data_ptr(), nqq, K, d_scores.data_ptr(), d_slots.data_ptr(), words.data_ptr())

            def step_p(qd, nqq):
                return idx.search_device_prepared(qd.data_ptr(), nqq, K, d_scores.data_ptr(), d_slots.data_ptr())
            dtf, _, _, _ = timed(lambda: step_f(q_dev, nq), f_steps, 1)
            dtf1, scanf1_ms, _, _ = timed(lambda: step_f(q1_dev, 1), 10, 2)
            idx.prepare_mask_device(words.data_ptr())            # the filter is analysed once, then reused per query
            dtp1, scanp1_ms, _, _ = timed(lambda: step_p(q1_dev, 1), 10, 2)
            live_bytes = live_blocks * 32 * (ng + 4)
            filtered.append({"selectivity": sel, "layout": kind, "n_allowed": int(allowed.sum()),
                             "live_block_fraction": live_blocks / nb_total,
                             "batch": {"size": nq, "value": nq * f_steps / dtf, "unit": UNIT},
                             "batch1": {"value": 10 / dtf1, "unit": UNIT, "ms_per_query": dtf1 / 10 * 1e3,
                                        "scan_gbs_over_live_blocks": live_bytes / (scanf1_ms / 10 / 1e3) / 1e9 if scanf1_ms > 0 else None},
                             "batch1_prepared_mask": {"value": 10 / dtp1, "unit": UNIT, "ms_per_query": dtp1 / 10 * 1e3,
                                                      "scan_gbs_over_live_blocks": live_bytes / (scanp1_ms / 10 / 1e3) / 1e9 if scanp1_ms > 0 else None,
                                                      "frac_of_hbm": live_bytes / (scanp1_ms / 10 / 1e3) / 1e9 / pk["hbm_gbs"] if scanp1_ms > 0 else None}})
            del words

    # ---- allocation-free entry point (one GPU): batch 1 and batch 8 ----
    noalloc = None
    if world == 1 and not args.no_filtered and DIM <= 4096:
        noalloc = {}
        for b in (1, 8):
            qb = q_dev[:b].contiguous()
            dtn, scann_ms, _, _ = timed(lambda: idx.search_device_noalloc(qb.data_ptr(), b, K, d_scores.data_ptr(), d_slots.data_ptr()), 10, 3)
            noalloc[f"batch{b}"] = {"ms_per_call": dtn / 10 * 1e3, "scan_ms_per_call": scann_ms / 10}

    # ---- online mutation: adds of 10,000 rows, searches of 1,024 queries and removal of 1 % of the ids, interleaved ----
    mutation = None
    if not args.no_mutation:
        rows_m, rounds = 10_000, 10
        next_id = ID_BASE * 50
        rng_m = np.random.default_rng(11)
        x_m = gen_rows_torch(torch, device, scale_t, 3, 0, rows_m)

        def add_batch():
            nonlocal next_id
            new_ids = (np.arange(rows_m) + next_id).astype(np.uint64)
            next_id += rows_m
            if world == 1:
                idx.add_with_ids_device(x_m.data_ptr(), rows_m, DIM, new_ids)
            else:
                idx.add_with_ids_device(x_m, new_ids)
            return new_ids
        added = [add_batch()]                                     # warm-up (may grow the arrays)
        barrier()
        t_add = t_search = t_remove = 0.0
        n_removed = 0
        for _ in range(rounds):
            t0 = time.perf_counter()
            added.append(add_batch())
            barrier()
            t_add += time.perf_counter() - t0
            t0 = time.perf_counter()
            step_device(q_dev, nq)
            barrier()
            t_search += time.perf_counter() - t0
            victims = rng_m.choice(added[-1], rows_m // 100, replace=False)       # 1 % of the ids just added
            t0 = time.perf_counter()
            for v in victims:
                idx.remove(int(v))
            barrier()
            t_remove += time.perf_counter() - t0
            n_removed += victims.size
        mutation = {"add_batch_rows": rows_m, "rounds": rounds, "add_vectors_per_s": rows_m * rounds / t_add,
                    "add_ms_per_batch": t_add / rounds * 1e3, "search_qps_interleaved": nq * rounds / t_search,
                    "remove_us_per_id": t_remove / max(1, n_removed) * 1e6, "removed": int(n_removed),
                    "note": "wall clock over all ranks; rows and queries resident on the device"}

    ingest_rate = ingest_rows / (ingest_ms / 1e3) if ingest_ms > 0 else None     # this rank's GPU
    ingest_job = ingest_rate                                                      # all ranks ingest their shards at once
    if world > 1:
        t = torch.tensor([float(ingest_rows), ingest_ms], device=device, dtype=torch.float64)
        rows_all, ms_all = t[:1].clone(), t[1:].clone()
        dist.all_reduce(rows_all, op=dist.ReduceOp.SUM)
        dist.all_reduce(ms_all, op=dist.ReduceOp.MAX)
        ingest_job = float(rows_all.item()) / (float(ms_all.item()) / 1e3) if float(ms_all.item()) > 0 else None

    configs = None
    if world == 1 and not args.no_configs and (DIM, BITS) == (1536, 4):
        configs = other_configs(torch, T, O, device, local_rank, idx, ids_all, q_all, pk, int8_peak, args)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    qps = nq * args.steps / dt
    # dominant kernel of the headline step: the permute-dot scan, an exact int8 contraction
    ops_per_step = 2.0 * nq * n_local * DIM
    scan_s = scan_ms / 1e3 / args.steps
    achieved_tops = ops_per_step / scan_s / 1e12 if scan_s > 0 else None
    bytes_b1 = n_local * (ng + 4)
    scan1_s = scan1_ms / 1e3 / b1_steps
    achieved_gbs = bytes_b1 / scan1_s / 1e9 if scan1_s > 0 else None
    ingest_bytes = 4 * DIM + ng + 4

    tc_min = local.get_option(T.OPT_MMA_MIN_BATCH)
    permute_dot = BITS == 4 and ng % 4 == 0
    tc_min = ((17 if local.get_option(T.OPT_EXPANDED_BYTES) > 0 else 33) if permute_dot else 8) if tc_min < 0 else tc_min       # library defaults
    small_kernel = ("scan_small_kernel (mma.sync, vectors on M)" if local.get_option(T.OPT_SMALL_SCAN) >= 0 else "scan_pd_kernel (mma.sync)") \
        if permute_dot else "scan_lut_kernel (CUDA cores)"
    expanded_bytes = local.get_option(T.OPT_EXPANDED_BYTES)
    if not permute_dot:
        tc_kernel = "scan_tc_wide_kernel (tcgen05, one-hot u8 LUT)" if nq > 256 else "scan_tc_kernel (tcgen05, one-hot u8 LUT)"
    elif expanded_bytes > 0:
        tc_kernel = ("scan_tc_dense_pair_kernel (tcgen05 cta_group::2; int8 copy of the index and query weights by TMA)"
                     if local.get_option(T.OPT_DENSE_PAIR) else "scan_tc_dense_kernel (tcgen05; int8 copy of the index and query weights by TMA)")
    else:
        tc_kernel = ("scan_tc_wide_kernel" if nq > 256 and local.get_option(T.OPT_TC_WIDE) else "scan_tc_kernel") + " (tcgen05, codes expanded in the kernel)"
    main_uses_tc = tc_min > 0 and nq >= tc_min and ng % 4 == 0
    main_kernel = tc_kernel if main_uses_tc else small_kernel
    cpu = None
    if world == 1 and not args.no_cpu:
        arm = CpuArm(n_total, nq)
        cpu_qps, cpu_ms, sample = arm.run(1, 0, budget_s=25.0)
        cpu = {"value": cpu_qps, "unit": UNIT, "cores": arm.cores, "kind": "port", "sample": sample}

    line = {
        "metric": METRIC, "value": qps, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": workload_config(n_total, DIM, BITS, nq),
        "details": {"index": "IdMapIndex" if world == 1 else f"ShardedIdMapIndex over {world} GPUs (round-robin chunks of 32768 slots)",
                    "score_mode": "permute-dot int8 (what an AVX-512-VNNI host runs)" if permute_dot else "u8 LUT (the reference's 2/3-bit and odd-geometry family)",
                    "vectors_per_gpu": n_local},
        "e2e": {"value": nq * args.steps / dt_e2e, "unit": UNIT, "h2d_bytes_per_step": int(nq * DIM * 4),
                "d2h_bytes_per_step": int(nq * K * 12)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved_tops, "peak": int8_peak, "unit": "TOP/s",
                     "frac": achieved_tops / int8_peak if achieved_tops and int8_peak else None,
                     "int8_peak_measured": int8_peak,
                     "peak_source": "tv_measure_int8_peak: back-to-back tcgen05 kind::i8 MMAs (M128 N256 K32) on shared-memory operands, "
                                    "one CTA per SM, best of three 2 ms launches on this device in this run (a burst: the clocks have "
                                    "not yet met the power limit)",
                     "int8_peak_sustained": int8_peak_sustained,
                     "frac_of_sustained_int8_peak": achieved_tops / int8_peak_sustained if achieved_tops and int8_peak_sustained else None,
                     "sustained_peak_source": "the same kernel launched back to back for 1.5 s, rate over the last 0.75 s (power-limited clocks)",
                     "bf16_peak": pk["tensor_tflops"], "frac_of_bf16_peak": achieved_tops / pk["tensor_tflops"] if achieved_tops else None,
                     "bf16_peak_source": f"{pk['source']} sustained cuBLAS bf16 (MEASURED_PEAKS.json); an int8 kernel may exceed it",
                     # DRAM bytes per step: the int8 copy (or the codes) and the scales, read once; the query groups of a
                     # vector tile share them through L2.  ncu on 421,888 vectors of a 524,288-vector index: 1.003x these
                     # bytes for the scan over the int8 copy (1.02x for the scans over the codes); scaled by vectors
                     "traffic": (1.003 * ((DIM + 127) // 128 * 128 + 4) if expanded_bytes and permute_dot and main_uses_tc else 1.02 * (ng + 4)) * n_local,
                     "expanded_copy_bytes": int(expanded_bytes),
                     "kernel": main_kernel, "launches_per_step": scan_launches / args.steps,
                     "note": "int8 multiply-adds counted as 2 ops"},
        "batch1": {"value": b1_steps / dt1, "unit": UNIT, "ms_per_query": dt1 / b1_steps * 1e3,
                   "e2e": {"value": b1_steps / dt1_e2e, "unit": UNIT, "h2d_bytes_per_step": DIM * 4, "d2h_bytes_per_step": K * 12},
                   "roofline": {"bound": "hbm", "achieved": achieved_gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                                "frac": achieved_gbs / pk["hbm_gbs"] if achieved_gbs else None,
                                "traffic": 1.004 * bytes_b1,   # ncu: DRAM bytes read = 1.004x the algorithmic bytes, scaled
                                "kernel": small_kernel, "launches_per_step": scan1_launches / b1_steps}},
        "ingest": {"value": ingest_job, "unit": "vectors/s", "per_gpu": ingest_rate, "rows": ingest_rows,
                   "roofline": {"bound": "hbm", "achieved": ingest_rate * ingest_bytes / 1e9 if ingest_rate else None,
                                "peak": pk["hbm_gbs"], "unit": "GB/s",
                                "frac": ingest_rate * ingest_bytes / 1e9 / pk["hbm_gbs"] if ingest_rate else None,
                                "traffic": None, "launches": ingest_launches,
                                "kernel": "ingest_fast_kernel (pipelined; whole 32-slot blocks)"
                                if DIM in (128, 256, 384, 512, 768, 1024, 1536, 2048, 3072) and args.ingest_pipeline != 0
                                else "ingest_kernel (block at a time)"}},
        "recall_at_10": recall,
    }
    if parity:
        line["parity"] = parity
    if filtered:
        line["filtered"] = filtered
    if noalloc:
        line["noalloc"] = noalloc
    if mutation:
        line["mutation"] = mutation
    if configs:
        line["configs"] = configs
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------ other baseline shapes
def other_configs(torch, T, O, device, dev_index, main_idx, ids_all, q_all, pk, int8_peak, args):
    """Short legs (one GPU) on the other configurations of the baseline, each with its own roofline and parity block:
    2-bit d3072 at batches 1 / 32 / 256 / 1,024; clustered d200 at 4 and 2 bits, k = 10 and 100; filtered search by
    uint64 allowlists through IdMapIndex.search on the 10 M index, k = 10 and 100, including n_allowed < k."""
    out = {}

    def timed_search(idx, qd, nqq, k, steps, warmup=2):
        s_out = torch.empty((nqq, k), dtype=torch.float32, device=device)
        i_out = torch.empty((nqq, k), dtype=torch.int64, device=device)
        for _ in range(warmup):
            idx.search_device(qd.data_ptr(), nqq, k, s_out.data_ptr(), i_out.data_ptr())
        torch.cuda.synchronize()
        t0, scan = time.perf_counter(), 0.0
        for _ in range(steps):
            idx.search_device(qd.data_ptr(), nqq, k, s_out.data_ptr(), i_out.data_ptr())
            scan += idx.last_main_kernel()[0]
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps, scan / steps / 1e3, s_out, i_out

    def leg(name, dim, bits, n, gen, batches, ks):
        idx = T.TurboQuantIndex(dim, bits, device=dev_index)
        first = None
        rows_per = max(32, (1 << 29) // (dim * 4) // 32 * 32)    # 512 MB of fp32 per generated chunk
        for c, lo in enumerate(range(0, n, rows_per)):
            x = gen(c, min(rows_per, n - lo))
            if c == 0:
                first = x[:1024].cpu().numpy()
            torch.cuda.synchronize()
            idx.add_device(x.data_ptr(), x.shape[0], dim)
            del x
        q = gen(10_000, 1024)
        ngl = ngroups(dim, bits)
        res = {"n": n, "dim": dim, "bits": bits, "score_mode": int(idx.get_option(T.OPT_SCORE_MODE)), "searches": []}
        for k in ks:
            for b in batches:
                sec, scan_s, s_out, i_out = timed_search(idx, q[:b].contiguous(), b, k, steps=5 if b >= 256 else 10)
                entry = {"batch": b, "k": k, "value": b / sec, "unit": UNIT, "ms_per_step": sec * 1e3, "scan_ms": scan_s * 1e3}
                if scan_s > 0:
                    gbs = n * (ngl + 4) / scan_s / 1e9
                    tops = 2.0 * b * n * dim / scan_s / 1e12
                    entry["roofline"] = {"hbm_gbs": gbs, "frac_of_hbm": gbs / pk["hbm_gbs"], "tensor_tops": tops,
                                         "frac_of_int8_peak": tops / int8_peak if int8_peak else None}
                res["searches"].append(entry)
        # parity on this index: 1,024 encoded rows and the results of 16 queries at the largest k
        kk = max(ks)
        sec, _, s_out, i_out = timed_search(idx, q[:16].contiguous(), 16, kk, steps=1, warmup=0)
        res["parity"] = parity_block(O, torch, idx, dim, bits, q[:16].cpu().numpy(), s_out.cpu().numpy(), i_out.cpu().numpy(), first)
        out[name] = res
        del idx
        torch.cuda.empty_cache()

    if not args.no_config2:
        s3072 = torch.from_numpy(dim_scale(1, 3072)).to(device)
        leg("config2_d3072_2bit_1M", 3072, 2, 1_000_000, lambda c, rows: gen_rows_torch(torch, device, s3072, 21, c, rows), (1, 32, 256, 1024), (10,))
    g = torch.Generator(device=device)
    g.manual_seed(4)
    centres = torch.randn((1000, 200), generator=g, device=device)
    for bits in (4, 2):
        leg(f"config4_d200_{bits}bit_1.2M_clustered", 200, bits, 1_200_000,
            lambda c, rows: gen_clustered_torch(torch, device, centres, 22, c, rows), (1, 1024), (10, 100))

    # config 3: uint64 allowlists through the reference-facing call, host buffers in and out
    n = len(main_idx)
    ids_now = main_idx.ids()
    rng = np.random.default_rng(17)
    nq = 1024
    qh = q_all[:nq].cpu().numpy()
    legs = []
    cases = [(sel, kind) for sel in (0.001, 0.01, 0.1, 0.5) for kind in ("random", "id-range")]
    for sel, kind in cases:
        m = max(1, int(sel * n))
        if kind == "random":
            allow = np.ascontiguousarray(rng.choice(ids_now, m, replace=False))
        else:
            lo = int(rng.integers(ID_BASE, ID_BASE + max(1, ids_all.size - m)))
            allow = np.ascontiguousarray(ids_now[(ids_now >= lo) & (ids_now < lo + m)])   # a contiguous range of ids
        for k in (10, 100):
            main_idx.search(qh[:8], k, allowlist=allow)
            t0 = time.perf_counter()
            s, got = main_idx.search(qh, k, allowlist=allow)
            sec = time.perf_counter() - t0
            ok = bool(s.shape == (nq, min(k, allow.size)) and np.isin(got[:32], allow).all() and np.all(s[:, :-1] >= s[:, 1:]))
            legs.append({"selectivity": sel, "layout": kind, "k": k, "n_allowed": int(allow.size), "value": nq / sec, "unit": UNIT,
                         "ms_per_step": sec * 1e3, "rows_ok": ok})
    few = np.ascontiguousarray(rng.choice(ids_now, 7, replace=False))            # n_allowed < k
    s, got = main_idx.search(qh[:64], 100, allowlist=few)
    out["config3_allowlists_10M"] = {"through": "IdMapIndex.search(queries, k, allowlist=ids), host arrays in and out", "searches": legs,
                                     "n_allowed_below_k": {"n_allowed": 7, "k": 100, "row_width": int(s.shape[1]),
                                                           "only_allowed_ids": bool(np.isin(got, few).all() and s.shape == (64, 7))}}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--vectors", dest="n", type=int, default=10_000_000)
    ap.add_argument("--batch", type=int, default=1024)
    ap.add_argument("--dim", type=int, default=1536, help="other shapes of the baseline (3072, 200, ...); the headline is 1536")
    ap.add_argument("--bits", type=int, default=4, choices=[2, 3, 4])
    ap.add_argument("--ingest-pipeline", type=int, default=None, choices=[0, 1, 2],
                    help="TV_OPT_INGEST_PIPELINE: 0 = block-at-a-time ingest kernel only (default: library default, 1)")
    ap.add_argument("--small-scan", type=int, default=None, help="TV_OPT_SMALL_SCAN variant (-1 = scan_pd_kernel)")
    ap.add_argument("--tc-wide", type=int, default=None, choices=[0, 1], help="TV_OPT_TC_WIDE: two query groups per expanded code slab")
    ap.add_argument("--tc-expanded", type=int, default=None, choices=[0, 1, 2],
                    help="TV_OPT_TC_EXPANDED: large permute-dot batches scan an int8 copy of the index (0 never, 1 if it fits, 2 always)")
    ap.add_argument("--dense-pair", type=int, default=None, choices=[0, 1], help="TV_OPT_DENSE_PAIR: that scan on CTA pairs")
    ap.add_argument("--skip-cpu", dest="no_cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--skip-filtered", dest="no_filtered", action="store_true", help="skip the filtered-search and allocation-free legs")
    ap.add_argument("--skip-mutation", dest="no_mutation", action="store_true", help="skip the online-mutation leg")
    ap.add_argument("--skip-configs", dest="no_configs", action="store_true", help="skip the legs on the other baseline shapes")
    ap.add_argument("--skip-config2", dest="no_config2", action="store_true", help="skip the 1 M x 3072 2-bit leg")
    ap.add_argument("--skip-parity", dest="no_parity", action="store_true", help="skip the oracle re-derivation of codes, scales and scores")
    ap.add_argument("--tc-min-batch", type=int, default=None,
                    help="query batches of at least this size use the tcgen05 scan (library default if omitted; 0 = never)")
    args = ap.parse_args()
    global DIM, BITS, METRIC
    DIM, BITS = args.dim, args.bits
    if (DIM, BITS) != (1536, 4) or args.n != 10_000_000 or args.batch != 1024:
        METRIC = f"search_qps_k10_{args.n}x{DIM}_{BITS}bit_batch{args.batch}"
        if (DIM, BITS) != (1536, 4):
            args.no_cpu = True          # the restated CPU kernel covers the 4-bit permute-dot family only
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
