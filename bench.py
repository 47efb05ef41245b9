#!/usr/bin/env python
"""bench.py — the decode-attention benchmark of the B200 attention silicon family.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
           bench.py --gpus N --steps K --warmup W

Headline (one JSON line on rank 0): `decode attn KV GB/s` on configuration 3 of the path's five — batched paged decode of 32
sequences with lengths uniform in [1,024, 100,000], 16 query heads on 2 kv heads, head_dim 256, bf16, 256-position
pages in a randomly permuted pool, int32 page table.  A step is one pass of the fused paged-decode kernel over the
whole batch.  Each GPU holds its own batch (sequences are independent: no collective on the data path), so N GPUs
process N batches: weak scaling.

  value        all ranks' KV bytes per step / the slowest rank's device time per step (CUDA events), inputs resident
  e2e          the same metric with, inside every timed step, the host-side plan, the upload of the step's inputs
               (queries and each sequence's newest K/V row, from pinned host memory through the family's memory_write
               door) and the read-back of the outputs (memory_read door)
  roofline     algorithmic KV bytes per launch / mean launch duration, against the measured HBM copy bandwidth
  cpu_baseline the reference's own CPU family (compiled unmodified by the checker's build recipe) on this host's cores, over the same batch
  others       the remaining configurations (1, 2, 4, 5), each with its own roofline fraction, single GPU

The KV pool of a step is 3.3 GB, far larger than the 126 MB L2, so no L2 flush is needed between iterations.
Synthetic data (there is no dataset for this path): numpy PCG64, fixed seeds a configuration; the headline's pools are
made on the host and uploaded before any timing, so the reference arm (`--impl reference`, which times the reference's
CPU family on the host's cores) reads the very same values.  `--only long_context` runs configuration 4 alone at any N.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC, UNIT = "decode attn KV GB/s", "GB/s"
WORKLOAD = "config3: batched paged decode, 32 seqs U[1024,100000], 16q/2kv heads, head_dim 256, bf16, 256-pos pages"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs."""
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
               0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.stop_flag, self.max_mhz = [], set(), threading.Event(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self.stop_flag.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(self.nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.05)

    def __enter__(self):
        if self.nv:
            self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop_flag.set()
        if self.nv:
            self.thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def device_index() -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ---------------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------------

def time_loop(torch, fn, steps, warmup):
    """Mean milliseconds per call of fn over `steps` calls after `warmup`, CUDA events on the current (default) stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def paged_inputs(rank=0):
    """Configuration 3's layout (seed 1003) and, for `rank`, its queries and the two pools as numpy bit arrays — PCG64,
    seed 1004 + 1000 * rank.  Both arms of the benchmark read these same arrays: this arm as bf16, the reference arm as
    the fp16 values that are the same real numbers."""
    from silvann_b200 import workloads
    L = workloads.config3_layout()
    q, k_pool, v_pool = workloads.config3_fill(L, seed=1003 + 1000 * rank)
    return L, q, k_pool, v_pool


def config_of(L):
    """The `config` object of the JSON line: what the workload is, identical for both arms."""
    return {"workload": WORKLOAD, "seqs": int(len(L.seq_lens)), "positions": int(L.positions), "kv_bytes_per_step": int(L.kv_bytes),
            "page_positions": 256, "pool_pages": int(L.pool_pages), "data": "numpy PCG64: layout seed 1003, values seed 1004 (+1000 a rank), fp16-exact bf16 N(0,1)"}


def reference_planes(L, q, k_pool, v_pool, which=None):
    """Every sequence (or those in `which`) gathered from the pools to the contiguous [len][kv_heads][head_dim] planes the
    reference's doors take, as fp16 bits of the same real numbers (the reference has neither paging nor bf16).  Outside any
    timed region."""
    from silvann_b200 import workloads
    to16 = lambda b: (b.astype(np.uint32) << 16).view(np.float32).astype(np.float16).view(np.uint16)
    from concurrent.futures import ThreadPoolExecutor

    def one(s):
        return (to16(q[s]), to16(workloads.gather_sequence(L, k_pool, s)), to16(workloads.gather_sequence(L, v_pool, s)), int(L.seq_lens[s]))
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        return list(pool.map(one, range(len(L.seq_lens)) if which is None else which))


class PagedWorkload:
    """Configuration 3 resident on the current device."""

    def __init__(self, torch, rank=0):
        from silvann_b200 import ext, workloads
        self.torch, self.ext = torch, ext
        L, q, k_pool, v_pool = paged_inputs(rank)
        self.layout, self.host = L, (q, k_pool, v_pool)
        self.seqs = len(L.seq_lens)
        up = lambda a: torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
        self.k_pool, self.v_pool, self.q = up(k_pool), up(v_pool), up(q)
        self.table = torch.from_numpy(L.page_table).cuda()
        self.out = torch.zeros((self.seqs, L.q_heads, L.head_dim), device="cuda", dtype=torch.bfloat16)
        self.plan = ext.Plan()
        self.plan.plan(L.seq_lens, L.q_heads, L.kv_heads, L.head_dim)
        self.page_positions = workloads.PAGE_POSITIONS
        self.kv_bytes = L.kv_bytes

    def step(self):
        L = self.layout
        self.plan.decode(self.out, None, self.q, self.k_pool, self.v_pool, L.pool_pages, self.page_positions, self.table,
                         L.page_table.shape[1], self.ext.BF16)


class EndToEnd:
    """A decoding step as a caller with host buffers sees it: plan, upload this step's inputs, decode, read back."""

    def __init__(self, torch, wl: PagedWorkload, fam):
        import ctypes as C
        self.C, self.wl, self.fam, self.torch = C, wl, fam, torch
        L = wl.layout
        row = L.kv_heads * L.head_dim
        self.q_bytes = wl.seqs * L.q_heads * L.head_dim * 2
        self.row_bytes = row * 2
        self.o_bytes = self.q_bytes
        n = self.q_bytes + 2 * wl.seqs * self.row_bytes + self.o_bytes
        host, card = C.c_void_p(), C.c_void_p()
        assert fam.sys.memory_allocate_host_ram_mapped(C.byref(host), C.byref(card), n), "pinned host buffer"
        self.host = host
        buf = np.ctypeslib.as_array(C.cast(host, C.POINTER(C.c_uint16)), shape=(n // 2,))
        rng = np.random.default_rng(3)
        buf[:] = (rng.standard_normal(n // 2).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        self.h_q = host.value
        self.h_rows = host.value + self.q_bytes
        self.h_out = self.h_rows + 2 * wl.seqs * self.row_bytes
        # the step's inputs land in ONE device buffer, as they lie in the host buffer: queries, then the newest K rows, then the V rows
        # — one upload a step instead of two (a synchronous copy costs about 12 us before its first byte moves)
        q_elems = self.q_bytes // 2
        self.in_dev = torch.zeros((q_elems + 2 * wl.seqs * row,), device="cuda", dtype=torch.bfloat16)
        self.in_dev[:q_elems].copy_(wl.q.reshape(-1))
        wl.q = self.in_dev[:q_elems].view(wl.q.shape)
        self.rows_dev = self.in_dev[q_elems:].view(2, wl.seqs, row)
        self.k_rows, self.v_rows = self.rows_dev[0], self.rows_dev[1]
        self.h2d = self.q_bytes + 2 * wl.seqs * self.row_bytes
        self.d2h = self.o_bytes

    def step(self):
        wl, sysd, L = self.wl, self.fam.sys, self.wl.layout
        wl.plan.plan(L.seq_lens, L.q_heads, L.kv_heads, L.head_dim)
        sysd.memory_write(self.in_dev.data_ptr(), self.h_q, self.h2d)
        wl.plan.append(wl.k_pool, wl.v_pool, self.k_rows, self.v_rows, L.pool_pages, wl.page_positions, wl.table, L.page_table.shape[1])
        wl.step()
        sysd.memory_read(self.h_out, wl.out.data_ptr(), self.o_bytes)

    def close(self):
        self.fam.sys.memory_free_host_ram(self.host)


def cpu_cores(R):
    """(threads the reference family used, its own report): its pool beside the caller, plus the caller, who works too."""
    threads, line = R.pool()
    return (threads + 1 if threads is not None else (os.cpu_count() or 1)), line


def cpu_baseline_paged(wl: PagedWorkload, budget_s=25.0):
    """The reference's CPU family over configuration 3 — every sequence of the same batch, gathered to the contiguous fp16
    planes its doors take, attention_scores + attention_mix each — or, where only the restatement is at hand, one short
    sequence through it."""
    import oracle
    R = oracle.reference()
    L = wl.layout
    q, k_pool, v_pool = wl.host
    if R is None:
        P = oracle.port()
        s = int(np.argmin(L.seq_lens))
        qs, ks, vs, n = reference_planes(L, q, k_pool, v_pool, [s])[0]
        t0 = time.perf_counter(); P.decode(qs, ks, vs, L.q_heads, L.kv_heads, L.head_dim, n, 0); dt = time.perf_counter() - t0
        nbytes = n * 2 * L.kv_heads * L.head_dim * 2
        return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": 1, "kind": "port", "sample": f"the shortest sequence of the batch ({n} positions), the C restatement, one pass"}
    planes = reference_planes(L, q, k_pool, v_pool)
    pbuf = np.empty(L.q_heads * int(L.seq_lens.max()), np.float32)
    best, t_all, passes = None, time.time(), 0
    while passes < 3 and (passes == 0 or time.time() - t_all < budget_s):
        t0 = time.perf_counter()
        for qs, ks, vs, n in planes:
            R.decode(qs, ks, vs, L.q_heads, L.kv_heads, L.head_dim, n, pbuf[:L.q_heads * n].reshape(L.q_heads, n))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        passes += 1
    cores, line = cpu_cores(R)
    return {"value": L.kv_bytes / best / 1e9, "unit": UNIT, "cores": cores, "kind": "reference", "ms_per_step": best * 1e3, "pool_report": line,
            "sample": f"the whole batch: {len(planes)} sequences, {L.positions} positions, {L.kv_bytes / 1e6:.0f} MB of KV, as fp16 copies of the same values; best of {passes} pass(es); SILVANN_CPU_AVX512=0"}


def cpu_baselines_others():
    """The reference's CPU family timed beside configurations 1, 2, 4 and 5 on this host's cores — the same seeded inputs
    the parity tests use (numpy PCG64 seeds 1001, 1002, 1004, 1005), one warm-up pass and the best of a few timed ones each
    and, on drawn values, beside the other entries door for door (under a minute in all).  Reported baselines, not targets."""
    import ctypes as C
    import oracle
    from silvann_b200 import workloads
    R = oracle.reference()
    if R is None:
        return {}
    cores, line = cpu_cores(R)
    to16 = lambda b: (b.astype(np.uint32) << 16).view(np.float32).astype(np.float16).view(np.uint16)
    out = {}

    def best_of(fn, passes):
        fn()
        best = None
        for _ in range(passes):
            t0 = time.perf_counter(); fn(); dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        return best

    def entry(value, unit, secs, sample):
        return {"value": value, "unit": unit, "cores": cores, "kind": "reference", "ms": secs * 1e3, "pool_report": line, "sample": sample}

    w = workloads.config1()
    p = np.empty((16, 8192), np.float32)
    t = best_of(lambda: R.decode(w.q, w.k, w.v, 16, 4, 128, 8192, p), 20)
    out["config1"] = entry(w.kv_bytes / t / 1e9, UNIT, t, "configuration 1 whole: attention_scores + attention_mix, fp16, 8,192 positions; best of 20")
    w = workloads.config2()
    q2, k2, v2 = to16(w.q), to16(w.k), to16(w.v)
    t = best_of(lambda: R.prefill(q2, k2, v2, 16, 2, 256, 4096), 1)
    out["config2"] = entry(w.flops / t / 1e12, "TFLOP/s", t, "configuration 2 whole: the three causal doors in 256-row chunks as the reference's runtime drives them, 4,096 rows; one timed pass")
    w = workloads.config4()
    q4, k4, v4 = to16(w.q), to16(w.k), to16(w.v)
    p4 = np.empty((32, 262144), np.float32)
    t = best_of(lambda: R.residual(q4, k4, v4, 32, 4, 128, 262144, p4), 3)
    out["config4"] = entry(w.kv_bytes / t / 1e9, UNIT, t, "configuration 4 whole, every position in host RAM: attention_weights + attention_residual_mix, 262,144 positions; best of 3")
    w = workloads.config5()
    c5, z5, b5, g5, w5 = (to16(x) for x in (w.conved, w.z, w.beta, w.g, w.w))
    T = 8192

    def prompt():
        S = np.zeros((32, 128, 128), np.float32)
        R.deltanet(S, c5[:T], z5[:T], b5[:T], g5[:T], w5, 32, 32, 128, T)
    t = best_of(prompt, 1)
    out["config5_prefill"] = entry(T / t, "positions/s", t, "configuration 5's prompt: deltanet_steps_gate over 8,192 positions (the reference has no chunked form); one timed pass")
    S = np.zeros((32, 128, 128), np.float32)

    def steps():
        for i in range(T, T + 512):
            R.deltanet(S, c5[i:i + 1], z5[i:i + 1], b5[i:i + 1], g5[i:i + 1], w5, 32, 32, 128, 1)
    t = best_of(steps, 1)
    nbytes = 512 * (2 * 32 * 128 * 128 * 4 + 3 * 32 * 128 * 2 + 2 * 32 * 128 * 2 + 2 * 32 * 2 + 128 * 2)
    out["config5_decode"] = entry(nbytes / t / 1e9, UNIT, t, "configuration 5's 512 decode steps: deltanet_step a position, one sequence; one timed pass")

    # the other entries of `others`, door for door on the same family (values drawn here: these are timings, the parity tests hold the checks)
    P_, rng = oracle._p, np.random.default_rng(7)
    f16 = lambda a: np.ascontiguousarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)
    S64 = (rng.standard_normal((64, 32, 128, 128)) * 0.05).astype(np.float32)

    def steps64():
        for b in range(64):
            R.deltanet(S64[b], c5[b:b + 1], z5[b:b + 1], b5[b:b + 1], g5[b:b + 1], w5, 32, 32, 128, 1)
    t = best_of(steps64, 2)
    out["config5_decode_64seq"] = entry(64 * (2 * 32 * 128 * 128 * 4 + 3 * 32 * 128 * 2 + 2 * 32 * 128 * 2 + 2 * 32 * 2 + 128 * 2) / t / 1e9, UNIT, t,
                                        "one decode step of 64 sequences: deltanet_step a sequence (the door takes one); best of 2")
    qh_, kvh_, dh_, Lt = 32, 4, 128, 262144
    for width in (8, 4):
        rb = dh_ * width // 8
        kc, vc = (rng.integers(0, 256, (Lt * kvh_, rb), dtype=np.uint8) for _ in range(2))
        ks, vs = (f16(rng.random(Lt * kvh_) * 0.5 + 0.75) for _ in range(2))
        tq_q = f16(rng.standard_normal((qh_, dh_)) * 0.25)
        tp, tres = np.zeros((qh_, Lt), np.float32), np.zeros((qh_, dh_ + 2), np.float32)

        def tier():
            R.nn.attention_weights_tq(P_(tp), P_(tres), P_(tq_q), P_(kc), P_(ks), qh_, kvh_, dh_, Lt, width)
            R.nn.attention_residual_mix_tq(P_(tres), P_(tp), P_(vc), P_(vs), qh_, kvh_, dh_, Lt, width)
            R.wait()
        t = best_of(tier, 2)
        out[f"tq{width}_tier_d128"] = entry(2 * Lt * kvh_ * (rb + 2) / t / 1e9, UNIT, t, f"attention_weights_tq + attention_residual_mix_tq over 262,144 coded positions at {width} bits; best of 2")
    for width in (4, 8):
        rows_, cols_ = 16384, 4096
        codes = rng.integers(0, 256, (rows_, cols_ * width // 8), dtype=np.uint8)
        scales = f16((rng.random(rows_) * 0.5 + 0.75) * (3.0 / cols_ ** 0.5))
        xv, ov = f16(rng.standard_normal(cols_)), np.zeros(rows_, np.uint16)

        def gemv():
            R.nn.turboquant_gemv(P_(ov), P_(codes), codes.nbytes, P_(scales), scales.nbytes, P_(xv), width, rows_, cols_, P_(R.over))
            R.wait()
        t = best_of(gemv, 5)
        out[f"tq{width}_gemv_16384x4096"] = entry((codes.nbytes + scales.nbytes) / t / 1e9, UNIT, t, f"turboquant_gemv, 16,384 x 4,096 at {width} bits; best of 5")
    for Lm in (2048, 65536):
        lat, qm = f16(rng.standard_normal((Lm, 512))), f16(rng.standard_normal((64, 512)) * 2.0)
        pm, om = np.zeros((64, Lm), np.float32), np.zeros((64, 512), np.uint16)

        def latent():
            R.nn.attention_scores_grouped(P_(pm), P_(qm), P_(lat), 64, 1, 512, Lm)
            R.nn.attention_softmax_rows(P_(pm), 64, Lm)
            R.nn.attention_mix(P_(om), P_(pm), P_(lat), 64, 1, 512, Lm, P_(R.over))
            R.wait()
        t = best_of(latent, 3)
        out[f"mla_decode_64heads_{Lm}"] = entry((Lm * 512 * 2 + 2 * 64 * 512 * 2) / t / 1e9, UNIT, t, f"scores_grouped + softmax_rows + mix, 64 heads over {Lm} latents of 512; best of 3")
    T_, er, ec = 256, 8192, 5120
    ecodes = rng.integers(0, 256, (er, ec // 2), dtype=np.uint8)
    escales = f16((rng.random(er) * 0.5 + 0.75) * (3.0 / ec ** 0.5))
    ex, eout = f16(rng.standard_normal((T_, ec))), np.zeros((T_, er), np.uint16)
    epairs = np.repeat(np.arange(T_, dtype=np.uint32), 2).copy()

    def project():
        R.nn.expert_rows(P_(eout), P_(ecodes), ecodes.nbytes, P_(escales), escales.nbytes, P_(ex), P_(epairs), T_, 4, er, ec, P_(R.over))
        R.wait()
    t = best_of(project, 2)
    out["prompt_projection_256rows_q4"] = entry(2.0 * T_ * er * ec / t / 1e12, "TFLOP/s", t, "expert_rows, 256 rows x 5,120 through 8,192 coded rows at 4 bits; best of 2")
    er, ec = 5120, 4096
    ecodes = rng.integers(0, 256, (er, ec), dtype=np.uint8)
    escales = f16((rng.random(er) * 0.5 + 0.75) * (3.0 / ec ** 0.5))
    ex, eout = f16(rng.standard_normal((T_, ec))), np.zeros((T_, er), np.uint16)
    t = best_of(lambda: (R.nn.expert_rows(P_(eout), P_(ecodes), ecodes.nbytes, P_(escales), escales.nbytes, P_(ex), P_(epairs), T_, 8, er, ec, P_(R.over)), R.wait()), 2)
    out["prompt_projection_256rows_o8"] = entry(2.0 * T_ * er * ec / t / 1e12, "TFLOP/s", t, "expert_rows, 256 rows x 4,096 through 5,120 coded rows at 8 bits; best of 2")

    # the coded tiers at head_dim 256, and 16 rows of a prompt chunk over the 8-bit tier at 128 (a bounded sample: 65,536 positions)
    qh_, kvh_, dh_ = 16, 2, 256
    for width in (8, 4):
        rb = dh_ * width // 8
        kc, vc = (rng.integers(0, 256, (Lt * kvh_, rb), dtype=np.uint8) for _ in range(2))
        ks, vs = (f16(rng.random(Lt * kvh_) * 0.5 + 0.75) for _ in range(2))
        tq_q = f16(rng.standard_normal((qh_, dh_)) * 0.25)
        tp, tres = np.zeros((qh_, Lt), np.float32), np.zeros((qh_, dh_ + 2), np.float32)

        def tier256():
            R.nn.attention_weights_tq(P_(tp), P_(tres), P_(tq_q), P_(kc), P_(ks), qh_, kvh_, dh_, Lt, width)
            R.nn.attention_residual_mix_tq(P_(tres), P_(tp), P_(vc), P_(vs), qh_, kvh_, dh_, Lt, width)
            R.wait()
        t = best_of(tier256, 2)
        out[f"tq{width}_tier_d256"] = entry(2 * Lt * kvh_ * (rb + 2) / t / 1e9, UNIT, t, f"attention_weights_tq + attention_residual_mix_tq over 262,144 coded positions at {width} bits, head_dim 256; best of 2")
    qh_, kvh_, dh_, Ls, rows16 = 32, 4, 128, 65536, 16
    kc, vc = (rng.integers(0, 256, (Ls * kvh_, dh_), dtype=np.uint8) for _ in range(2))
    ks, vs = (f16(rng.random(Ls * kvh_) * 0.5 + 0.75) for _ in range(2))
    q16 = f16(rng.standard_normal((rows16, qh_, dh_)) * 0.25)
    tp16, res16 = np.zeros((rows16, qh_, Ls), np.float32), np.zeros((rows16, qh_, dh_ + 2), np.float32)

    def rows_tier():
        R.nn.attention_weights_tq_rows(P_(tp16), P_(res16), P_(q16), P_(kc), P_(ks), qh_, kvh_, dh_, Ls, 8, rows16)
        R.nn.attention_residual_mix_tq_rows(P_(res16), P_(tp16), P_(vc), P_(vs), qh_, kvh_, dh_, Ls, 8, rows16)
        R.wait()
    t = best_of(rows_tier, 2)
    out["tq8_tier_d128_rows16"] = entry(rows16 * Ls / t, "row-positions/s", t, "the _rows door pair, 16 rows over 65,536 of the 262,144 coded positions at 8 bits; best of 2")

    # Kimi Delta Attention's decode step, the latent projections and the indexer, door for door
    heads, d = 64, 128
    W_ = heads * d
    Sk = (rng.standard_normal((heads, d, d)) * 0.05).astype(np.float32)
    kc3, kf, kg = f16(rng.standard_normal((3, 1, W_))), f16(rng.standard_normal((1, W_))), f16(rng.standard_normal((1, W_)))
    kb, kdt, kal = f16(rng.standard_normal((1, heads))), f16(rng.standard_normal(W_)), f16(rng.standard_normal(heads) * 0.3)
    kw, ko = f16(np.ones(d)), np.zeros((1, W_), np.uint16)
    t = best_of(lambda: (R.nn.kda_step(P_(Sk), P_(kc3), P_(kf), P_(kb), P_(kdt), P_(kal), P_(kg), P_(kw), P_(ko), heads, d, C.c_float(-5.0), C.c_float(1e-5), P_(R.over)), R.wait()), 20)
    out["kda_decode_64heads"] = entry((2 * heads * d * d * 4 + 6 * heads * d * 2) / t / 1e9, UNIT, t, "kda_step, 64 heads of 128; best of 20")
    mh, nope, vd, lat_ = 64, 192, 256, 512
    Wl = f16(rng.standard_normal((mh * (nope + vd), lat_)) * 0.05)
    qa, oa = f16(rng.standard_normal(mh * nope)), f16(rng.standard_normal(mh * lat_))
    absorbed, expanded = np.zeros(mh * lat_, np.uint16), np.zeros(mh * vd, np.uint16)
    t = best_of(lambda: (R.nn.attention_absorb(P_(absorbed), P_(qa), P_(Wl), mh, nope, lat_, nope + vd, C.c_float(0.0722), P_(R.over)), R.wait()), 10)
    out["mla_absorb_64heads"] = entry((mh * nope * lat_ * 2 + mh * nope * 2 + mh * lat_ * 2) / t / 1e9, UNIT, t, "attention_absorb, 64 heads; best of 10")
    t = best_of(lambda: (R.nn.attention_expand(P_(expanded), P_(oa), P_(Wl), mh, vd, lat_, nope + vd, nope, P_(R.over)), R.wait()), 10)
    out["mla_expand_64heads"] = entry((mh * vd * lat_ * 2 + mh * lat_ * 2 + mh * vd * 2) / t / 1e9, UNIT, t, "attention_expand, 64 heads; best of 10")
    ih, idim, pools, topk, kpool = 32, 128, 8192, 512, 4
    iq, iw, pooled = f16(rng.standard_normal(ih * idim)), f16(rng.standard_normal(ih)), f16(rng.standard_normal((pools, idim)))
    iscores, iindex, icount = np.zeros(pools, np.float32), np.zeros(topk * kpool + kpool, np.int32), np.zeros(1, np.int32)

    def indexer():
        R.nn.index_scores(P_(iscores), P_(iq), P_(iw), P_(pooled), ih, idim, pools, C.c_float(0.088))
        R.nn.index_select(P_(iindex), P_(icount), P_(iscores), pools, topk, kpool, pools * kpool, 3)
        R.wait()
    t = best_of(indexer, 10)
    out["glm_indexer_8192pools"] = entry(pools / t, "pools/s", t, "index_scores + index_select, 32 heads of 128 over 8,192 pooled keys; best of 10")
    return out


def roofline(bound, work, ms, pk, kernel, traffic=None, how=None):
    """The roofline object of one kernel: algorithmic bytes (bound "hbm") or flops ("tensor") a launch over the measured time,
    against the measured peak; `traffic` = DRAM bytes a launch from the kernel's profiler capture (scaled where `how` says)."""
    if bound == "hbm":
        achieved, peak, unit, key = work / ms / 1e6, pk["hbm_gbs"], "GB/s", "algorithmic_bytes_per_launch"
    else:
        achieved, peak, unit, key = work / ms / 1e9, pk["bf16_tflops"], "TFLOP/s", "algorithmic_flops_per_launch"
    if traffic is not None and traffic < 100.0:            # a ratio of DRAM bytes to algorithmic bytes, from a capture of a smaller case
        traffic = traffic * work if bound == "hbm" else None
    r = {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, "traffic": None if traffic is None else int(traffic),
         "kernel": kernel, key: int(work), "peak_source": pk["source"]}
    if bound == "hbm":
        r["peak_note"] = "the measured peak is a copy (read + write); a read-only stream can exceed it slightly"
    if how:
        r["traffic_from"] = how
    return r


def gpu_baseline(torch, wl: PagedWorkload, pk, steps):
    """The reference's own CUDA family (nvidia_cuda12, built unmodified for sm_100 by the checker's build recipe) on the same card, door
    for door: a reported baseline beside the CPU one.  Configuration 3 has no paged form there, so — as for the CPU
    baseline — whole sequences are gathered to the contiguous planes its doors take (outside the timed region) and each is
    attended with attention_scores + attention_mix; configurations 1, 2 and 5 are the door sequences the reference's
    runtime issues.  fp16 throughout: the reference has no bf16 door, and the inputs are fp16-exact."""
    import oracle
    R = oracle.reference_cuda()
    if R is None:
        return {"unavailable": "the reference's nvidia_cuda12 family was not built here, or it counts no card"}
    out = {"kind": "reference nvidia_cuda12 family (sm_100 build), same card, CUDA events"}
    L = wl.layout
    order = np.argsort(L.seq_lens)[::-1][:8]
    planes, positions = [], 0
    for s in order:
        n = int(L.seq_lens[s]); positions += n
        pages = torch.from_numpy(L.page_table[s, :(n + wl.page_positions - 1) // wl.page_positions].astype(np.int64)).cuda()
        ks = wl.k_pool[pages].reshape(-1, L.kv_heads, L.head_dim)[:n].to(torch.float16).contiguous()
        vs = wl.v_pool[pages].reshape(-1, L.kv_heads, L.head_dim)[:n].to(torch.float16).contiguous()
        planes.append((wl.q[s].to(torch.float16).contiguous(), ks, vs, n))
    p = torch.zeros(L.q_heads * int(L.seq_lens.max()), device="cuda", dtype=torch.float32)
    o = torch.zeros((L.q_heads, L.head_dim), device="cuda", dtype=torch.float16)
    over = torch.zeros(4, device="cuda", dtype=torch.int32)          # the fault word every door that rounds is handed

    def sample():
        for qs, ks, vs, n in planes:
            R.nn.attention_scores(p.data_ptr(), qs.data_ptr(), ks.data_ptr(), L.q_heads, L.kv_heads, L.head_dim, n)
            R.nn.attention_mix(o.data_ptr(), p.data_ptr(), vs.data_ptr(), L.q_heads, L.kv_heads, L.head_dim, n, over.data_ptr())
    ms = time_loop(torch, sample, max(2, min(steps, 5)), 1)
    nbytes = positions * 2 * L.kv_heads * L.head_dim * 2
    out["value"], out["unit"] = nbytes / ms / 1e6, UNIT
    out["sample"] = f"the 8 longest sequences of the batch ({positions} positions, {nbytes / 1e6:.0f} MB of KV), gathered to contiguous fp16 planes outside the timed region"
    del planes
    gen = torch.Generator(device="cuda"); gen.manual_seed(78)

    # configuration 1: the door pair, 64 caches cycled
    qh, kvh, d, n, copies = 16, 4, 128, 8192, 64
    k = torch.randn((copies, n, kvh, d), generator=gen, device="cuda", dtype=torch.float16)
    v = torch.randn((copies, n, kvh, d), generator=gen, device="cuda", dtype=torch.float16)
    q = torch.randn((qh, d), generator=gen, device="cuda", dtype=torch.float16)
    o1 = torch.zeros((qh, d), device="cuda", dtype=torch.float16)
    state = {"i": 0}

    def pair():
        i = state["i"] = (state["i"] + 1) % copies
        R.nn.attention_scores(p.data_ptr(), q.data_ptr(), k[i].data_ptr(), qh, kvh, d, n)
        R.nn.attention_mix(o1.data_ptr(), p.data_ptr(), v[i].data_ptr(), qh, kvh, d, n, over.data_ptr())
    ms = time_loop(torch, pair, 100, 10)
    out["config1_decode_doors"] = {"value": 2 * n * kvh * d * 2 / ms / 1e6, "unit": UNIT, "ms_per_call": ms}
    del k, v

    # configuration 2: the three causal doors, 256 rows a call as the reference's runtime drives them
    qh, kvh, d, T, chunk = 16, 2, 256, 4096, 256
    q = (torch.randn((T, qh, d), generator=gen, device="cuda", dtype=torch.float16) * 0.5)
    k = (torch.randn((T, kvh, d), generator=gen, device="cuda", dtype=torch.float16) * 0.5)
    v = (torch.randn((T, kvh, d), generator=gen, device="cuda", dtype=torch.float16) * 0.5)
    o2 = torch.zeros((T, qh, d), device="cuda", dtype=torch.float16)
    pc = torch.zeros(chunk * qh * T, device="cuda", dtype=torch.float32)

    def prefill():
        for first in range(0, T, chunk):
            R.nn.attention_causal_scores_grouped(pc.data_ptr(), q[first].data_ptr(), k.data_ptr(), qh, kvh, d, first, chunk)
            R.nn.attention_causal_softmax(pc.data_ptr(), qh, first, chunk)
            R.nn.attention_causal_mix(o2[first].data_ptr(), pc.data_ptr(), v.data_ptr(), qh, kvh, d, first, chunk, over.data_ptr())
    ms = time_loop(torch, prefill, 3, 1)
    out["config2_causal_prefill"] = {"value": 4.0 * qh * d * T * (T + 1) / 2 / ms / 1e9, "unit": "TFLOP/s", "ms_per_call": ms}
    del q, k, v, o2, pc

    # configuration 5: one recurrent step (one sequence), and the 8,192-position prompt through deltanet_steps_gate
    heads, d, T = 32, 128, 8192
    S = torch.zeros((heads, d, d), device="cuda", dtype=torch.float32)
    conved = torch.randn((T, 3 * heads * d), generator=gen, device="cuda", dtype=torch.float16) * 0.1
    z = torch.randn((T, heads * d), generator=gen, device="cuda", dtype=torch.float16)
    beta = torch.rand((T, heads), generator=gen, device="cuda", dtype=torch.float32).to(torch.float16)
    g = (-torch.rand((T, heads), generator=gen, device="cuda", dtype=torch.float32)).to(torch.float16)
    w = torch.ones(d, device="cuda", dtype=torch.float16)
    o5 = torch.zeros((T, heads * d), device="cuda", dtype=torch.float16)
    ms = time_loop(torch, lambda: R.nn.deltanet_step(S.data_ptr(), conved.data_ptr(), z.data_ptr(), beta.data_ptr(), g.data_ptr(), w.data_ptr(),
                                                     o5.data_ptr(), heads, heads, d, over.data_ptr()), 100, 10)
    out["config5_deltanet_decode_1seq"] = {"ms_per_step": ms}
    S.zero_()
    ms = time_loop(torch, lambda: R.nn.deltanet_steps_gate(S.data_ptr(), conved.data_ptr(), z.data_ptr(), beta.data_ptr(), g.data_ptr(), w.data_ptr(),
                                                           o5.data_ptr(), heads, heads, d, T, 0, over.data_ptr()), 2, 1)
    out["config5_deltanet_prefill_8192"] = {"value": T / ms * 1e3, "unit": "positions/s", "ms": ms}
    del S, conved, z, beta, g, o5
    torch.cuda.empty_cache()

    # the coded matrix-vector door on the same matrices as `others` times it on (the reference's CUDA family has a kernel of its
    # own for widths 4 and 8: silicon_families/nvidia_cuda12/overrides/turboquant.cuh)
    for width, copies in ((4, 8), (8, 4)):
        rows, cols = 16384, 4096
        codes, scales, xv, ov, rb = coded_weights(torch, gen, copies, rows, cols, width)
        gstate = {"i": 0}

        def gemv():
            i = gstate["i"] = (gstate["i"] + 1) % copies
            R.nn.turboquant_gemv(ov.data_ptr(), codes[i].data_ptr(), rows * rb, scales[i].data_ptr(), rows * 2, xv.data_ptr(), width, rows, cols, over.data_ptr())
        ms = time_loop(torch, gemv, 50, 5)
        nbytes = rows * (rb + 2) + cols * 2 + rows * 2
        out[f"tq{width}_gemv_16384x4096"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_call": ms}
        del codes, scales
    torch.cuda.empty_cache()

    # a coded tier of 262,144 positions (32q/4kv heads of 128) through the reference's own weights_tq + residual_mix_tq kernels
    dh, tqh, tkvh, Lt = 128, 32, 4, 262144
    for width in (8, 4):
        rb = dh * width // 8
        kc = torch.randint(0, 256, (Lt * tkvh, rb), generator=gen, device="cuda", dtype=torch.uint8)
        vc = torch.randint(0, 256, (Lt * tkvh, rb), generator=gen, device="cuda", dtype=torch.uint8)
        ks = (torch.rand((Lt * tkvh,), generator=gen, device="cuda") * 0.5 + 0.75).to(torch.float16)
        vs = (torch.rand((Lt * tkvh,), generator=gen, device="cuda") * 0.5 + 0.75).to(torch.float16)
        tq_q = torch.randn((tqh, dh), generator=gen, device="cuda", dtype=torch.float16) * 0.25
        tp = torch.zeros((tqh, Lt), device="cuda", dtype=torch.float32)
        tres = torch.zeros((tqh, dh + 2), device="cuda", dtype=torch.float32)

        def tq_pair():
            R.nn.attention_weights_tq(tp.data_ptr(), tres.data_ptr(), tq_q.data_ptr(), kc.data_ptr(), ks.data_ptr(), tqh, tkvh, dh, Lt, width)
            R.nn.attention_residual_mix_tq(tres.data_ptr(), tp.data_ptr(), vc.data_ptr(), vs.data_ptr(), tqh, tkvh, dh, Lt, width)
        ms = time_loop(torch, tq_pair, 5, 2)
        nbytes = 2 * Lt * tkvh * (rb + 2)
        out[f"tq{width}_tier_d128"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_call": ms}
        del kc, vc, ks, vs, tp
    # latent attention at decode through the reference's own kernels for the three doors (its shared-memory tiled scores kernel)
    for Lm, copies in ((2048, 16), (65536, 4)):
        lat = torch.randn((copies, Lm, 512), generator=gen, device="cuda", dtype=torch.float16)
        qm = torch.randn((64, 512), generator=gen, device="cuda", dtype=torch.float16) * 2.0
        pm = torch.zeros((64, Lm), device="cuda", dtype=torch.float32)
        om = torch.zeros((64, 512), device="cuda", dtype=torch.float16)
        lstate = {"i": 0}

        def latent():
            i = lstate["i"] = (lstate["i"] + 1) % copies
            R.nn.attention_scores_grouped(pm.data_ptr(), qm.data_ptr(), lat[i].data_ptr(), 64, 1, 512, Lm)
            R.nn.attention_softmax_rows(pm.data_ptr(), 64, Lm)
            R.nn.attention_mix(om.data_ptr(), pm.data_ptr(), lat[i].data_ptr(), 64, 1, 512, Lm, over.data_ptr())
        ms = time_loop(torch, latent, 30, 5)
        nbytes = Lm * 512 * 2 + 2 * 64 * 512 * 2
        out[f"mla_decode_64heads_{Lm}"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_call": ms}
        del lat, pm
    # a prompt chunk's projection through the reference's expert_rows (its own tiled kernel): 256 rows through 8,192 x 5,120 at 4 bits
    T, er, ec = 256, 8192, 5120
    ecodes = torch.randint(0, 256, (er, ec // 2), generator=gen, device="cuda", dtype=torch.uint8)
    escales = ((torch.rand((er,), generator=gen, device="cuda") * 0.5 + 0.75) * (3.0 / ec ** 0.5)).to(torch.float16)
    ex = torch.randn((T, ec), generator=gen, device="cuda", dtype=torch.float16)
    epairs = torch.arange(T, device="cuda", dtype=torch.int32).repeat_interleave(2).contiguous()
    eout = torch.zeros((T, er), device="cuda", dtype=torch.float16)
    ms = time_loop(torch, lambda: R.nn.expert_rows(eout.data_ptr(), ecodes.data_ptr(), ecodes.numel(), escales.data_ptr(), escales.numel() * 2, ex.data_ptr(),
                                                   epairs.data_ptr(), T, 4, er, ec, over.data_ptr()), 5, 2)
    out["prompt_projection_256rows_q4"] = {"value": 2.0 * T * er * ec / ms / 1e9, "unit": "TFLOP/s", "ms_per_call": ms}
    del ecodes, ex, eout
    torch.cuda.empty_cache()
    # Kimi Delta Attention, one decode step of 64 heads of 128, through the reference's kda_step
    import ctypes as C
    S, conved, f, b, dt, a_log, gate, w, o = kda_workload(torch, gen, 64, 128, 1)
    ms = time_loop(torch, lambda: R.nn.kda_step(S.data_ptr(), conved.data_ptr(), f.data_ptr(), b.data_ptr(), dt.data_ptr(), a_log.data_ptr(), gate.data_ptr(),
                                                w.data_ptr(), o.data_ptr(), 64, 128, C.c_float(-5.0), C.c_float(1e-5), over.data_ptr()), 50, 5)
    out["kda_decode_64heads"] = {"ms_per_step": ms}
    R.sys.compute_completed()
    return out


def config1_graph(torch, ext, gen, copies=64):
    """Configuration 1 without the host in the loop: `copies` decode launches (the extension call the door pair fuses into),
    one per distinct cache, captured once into a CUDA graph on a side stream.  Answers (replay, bytes a launch, unit)."""
    qh, kvh, d, n = 16, 4, 128, 8192
    k = torch.randn((copies, n, kvh, d), generator=gen, device="cuda", dtype=torch.float16)
    v = torch.randn((copies, n, kvh, d), generator=gen, device="cuda", dtype=torch.float16)
    q = torch.randn((qh, d), generator=gen, device="cuda", dtype=torch.float16)
    o = torch.zeros((copies, qh, d), device="cuda", dtype=torch.float16)
    side = torch.cuda.Stream()
    ext.decode(o[0], None, q, k[0], v[0], qh, kvh, d, n, ext.FP16)          # scratch is allocated outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(copies):
            ext.decode(o[i], None, q, k[i], v[i], qh, kvh, d, n, ext.FP16, stream=side.cuda_stream)
    keep = (k, v, q, o, side)

    def replay(_keep=keep):
        graph.replay()
    return replay, 2 * n * kvh * d * 2, "bytes"


def mla_graph(torch, ext, lat, qm, om, Lm):
    """One CUDA graph of a latent-attention call a latent of `lat`, captured on a side stream.  Answers the replay."""
    side = torch.cuda.Stream()
    ext.mla_decode(om, None, qm, lat[0], 64, Lm, ext.FP16)                  # scratch is allocated outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(lat.shape[0]):
            ext.mla_decode(om, None, qm, lat[i], 64, Lm, ext.FP16, stream=side.cuda_stream)
    keep = (lat, qm, om, side)

    def replay(_keep=keep):
        graph.replay()
    return replay


def coded_weights(torch, gen, copies, rows, cols, width):
    """`copies` distinct coded matrices (random codes, scales near 1/sqrt(cols)) and one input vector, on the card."""
    rb = cols * width // 8
    codes = torch.randint(0, 256, (copies, rows, rb), generator=gen, device="cuda", dtype=torch.uint8)
    scales = ((torch.rand((copies, rows), generator=gen, device="cuda") * 0.5 + 0.75) * (3.0 / cols ** 0.5)).to(torch.float16)
    x = torch.randn((cols,), generator=gen, device="cuda", dtype=torch.float16)
    out = torch.zeros((rows,), device="cuda", dtype=torch.float16)
    return codes, scales, x, out, rb


def kda_workload(torch, gen, heads, d, rows):
    W = heads * d
    S = torch.randn((heads, d, d), generator=gen, device="cuda", dtype=torch.float32) * 0.05
    conved = torch.randn((3, rows, W), generator=gen, device="cuda", dtype=torch.float16)
    f = torch.randn((rows, W), generator=gen, device="cuda", dtype=torch.float16)
    b = torch.randn((rows, heads), generator=gen, device="cuda", dtype=torch.float16)
    dt = torch.randn((W,), generator=gen, device="cuda", dtype=torch.float16)
    a_log = torch.randn((heads,), generator=gen, device="cuda", dtype=torch.float16) * 0.3
    gate = torch.randn((rows, W), generator=gen, device="cuda", dtype=torch.float16)
    w = torch.ones((d,), device="cuda", dtype=torch.float16)
    out = torch.zeros((rows, W), device="cuda", dtype=torch.float16)
    return S, conved, f, b, dt, a_log, gate, w, out


def other_workloads(torch, fam, pk, steps, warmup):
    """Configurations 1, 4 and 5 (and 2 when the prefill kernel fits), each timed alone on one GPU."""
    from silvann_b200 import ext, workloads
    out = {}
    hbm = pk["hbm_gbs"]
    gen = torch.Generator(device="cuda"); gen.manual_seed(77)

    # configuration 1 through the two doors, cycling 64 distinct caches (1.07 GB) so that nothing stays in L2
    qh, kvh, d, L = 16, 4, 128, 8192
    copies = 64
    k = torch.randn((copies, L, kvh, d), generator=gen, device="cuda", dtype=torch.float16)
    v = torch.randn((copies, L, kvh, d), generator=gen, device="cuda", dtype=torch.float16)
    q = torch.randn((qh, d), generator=gen, device="cuda", dtype=torch.float16)
    p = torch.zeros((qh, L), device="cuda", dtype=torch.float32)
    o = torch.zeros((qh, d), device="cuda", dtype=torch.float16)
    state = {"i": 0}

    def door_pair():
        i = state["i"] = (state["i"] + 1) % copies
        fam.nn.attention_scores(p.data_ptr(), q.data_ptr(), k[i].data_ptr(), qh, kvh, d, L)
        fam.nn.attention_mix(o.data_ptr(), p.data_ptr(), v[i].data_ptr(), qh, kvh, d, L, None)
    ms = time_loop(torch, door_pair, max(steps * 20, 200), max(warmup * 5, 20))
    nbytes = 2 * L * kvh * d * 2
    out["config1_decode_doors"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_call": ms, "frac_hbm": nbytes / ms / 1e6 / hbm,
                                   "note": "attention_scores+attention_mix door pair, fp16, 16.8 MB of KV a call, 64 caches cycled"}
    del k, v
    replay, nb1, _ = config1_graph(torch, ext, gen)
    ms = time_loop(torch, replay, 20, 3) / 64
    out["config1_decode_kernel"] = {"value": nb1 / ms / 1e6, "unit": UNIT, "ms_per_call": ms, "frac_hbm": nb1 / ms / 1e6 / hbm,
                                    "note": "the same fused launch without the host in the loop: a CUDA graph of 64 launches, a distinct cache each"}
    del replay
    torch.cuda.empty_cache()

    # configuration 4 on one GPU, everything in HBM (537 MB a pass)
    qh, kvh, d, L = 32, 4, 128, 262144
    k = torch.randn((L, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16)
    v = torch.randn((L, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16)
    q = torch.randn((qh, d), generator=gen, device="cuda", dtype=torch.bfloat16)
    o = torch.zeros((qh, d), device="cuda", dtype=torch.bfloat16)
    ms = time_loop(torch, lambda: ext.decode(o, None, q, k, v, qh, kvh, d, L, ext.BF16), max(steps, 20), max(warmup, 3))
    nbytes = 2 * L * kvh * d * 2
    out["config4_long_context_1gpu_resident"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_call": ms, "frac_hbm": nbytes / ms / 1e6 / hbm,
                                                 "note": "262,144 positions, 32q/4kv, d128, bf16, all KV in HBM"}
    del k, v

    # a TurboQuant-coded tier (the reference's default cache for Qwen): one query over 262,144 coded positions through the
    # attention_weights_tq + attention_residual_mix_tq door pair (one fused launch), two distinct tiers alternated
    for dh, tqh, tkvh in ((128, 32, 4), (256, 16, 2)):
        for width in (8, 4):
            Lt = 262144
            rb = dh * width // 8
            kc = torch.randint(0, 256, (2, Lt * tkvh, rb), generator=gen, device="cuda", dtype=torch.uint8)
            vc = torch.randint(0, 256, (2, Lt * tkvh, rb), generator=gen, device="cuda", dtype=torch.uint8)
            ks = (torch.rand((2, Lt * tkvh), generator=gen, device="cuda") * 0.5 + 0.75).to(torch.float16)
            vs = (torch.rand((2, Lt * tkvh), generator=gen, device="cuda") * 0.5 + 0.75).to(torch.float16)
            tq_q = torch.randn((tqh, dh), generator=gen, device="cuda", dtype=torch.float16) * 0.25
            tp = torch.zeros((tqh, 8), device="cuda", dtype=torch.float32)        # never written by the fused pair
            tres = torch.zeros((tqh, dh + 2), device="cuda", dtype=torch.float32)
            tstate = {"i": 0}

            def tq_pair():
                i = tstate["i"] = 1 - tstate["i"]
                fam.nn.attention_weights_tq(tp.data_ptr(), tres.data_ptr(), tq_q.data_ptr(), kc[i].data_ptr(), ks[i].data_ptr(), tqh, tkvh, dh, Lt, width)
                fam.nn.attention_residual_mix_tq(tres.data_ptr(), tp.data_ptr(), vc[i].data_ptr(), vs[i].data_ptr(), tqh, tkvh, dh, Lt, width)
            before = ext.counters()["fused_residual"]
            ms = time_loop(torch, tq_pair, max(steps, 20), max(warmup, 3))
            assert ext.counters()["fused_residual"] > before, "the coded pair did not take the fused kernel"
            nbytes = 2 * Lt * tkvh * (rb + 2)
            out[f"tq{width}_tier_d{dh}"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_call": ms, "frac_hbm": nbytes / ms / 1e6 / hbm,
                                            "positions_per_s": Lt / ms * 1e3,
                                            "note": f"262,144 positions coded at {width} bits, {tqh}q/{tkvh}kv heads of {dh}: {nbytes / 1e6:.0f} MB of codes and scales a call"}
            if dh == 128 and width == 8:
                # a prompt chunk's 16 rows over the same tier through the _rows door pair (one fused launch): the rows are more
                # query heads of the same kv heads; the codes are read once a block of 16 of them
                rows16 = 16
                q16 = torch.randn((rows16, tqh, dh), generator=gen, device="cuda", dtype=torch.float16) * 0.25
                res16 = torch.zeros((rows16, tqh, dh + 2), device="cuda", dtype=torch.float32)

                def tq_rows():
                    i = tstate["i"] = 1 - tstate["i"]
                    fam.nn.attention_weights_tq_rows(tp.data_ptr(), res16.data_ptr(), q16.data_ptr(), kc[i].data_ptr(), ks[i].data_ptr(), tqh, tkvh, dh, Lt, width, rows16)
                    fam.nn.attention_residual_mix_tq_rows(res16.data_ptr(), tp.data_ptr(), vc[i].data_ptr(), vs[i].data_ptr(), tqh, tkvh, dh, Lt, width, rows16)
                before = ext.counters()["fused_residual"]
                ms = time_loop(torch, tq_rows, max(steps // 2, 10), 3)
                assert ext.counters()["fused_residual"] > before, "the coded rows pair did not take the fused kernel"
                flops = 4.0 * rows16 * tqh * dh * Lt
                out["tq8_tier_d128_rows16"] = {"value": rows16 * Lt / ms * 1e3, "unit": "row-positions/s", "ms_per_call": ms, "tflops": flops / ms / 1e9, "algorithmic_bytes": nbytes,
                                               "note": "16 rows of a prompt chunk x 32q/4kv heads of 128 over 262,144 positions coded at 8 bits, one launch"}
            del kc, vc, ks, vs
    torch.cuda.empty_cache()

    # the weight path of a decode step: a coded matrix times one vector through the turboquant_gemv door, distinct matrices
    # cycled so that every call reads its codes from HBM (8 x 33.5 MB at 4 bits, 4 x 67 MB at 8)
    import ctypes as C
    for width, copies in ((4, 8), (8, 4)):
        rows, cols = 16384, 4096
        codes, scales, xv, ov, rb = coded_weights(torch, gen, copies, rows, cols, width)
        gstate = {"i": 0}

        def gemv():
            i = gstate["i"] = (gstate["i"] + 1) % copies
            fam.nn.turboquant_gemv(ov.data_ptr(), codes[i].data_ptr(), rows * rb, scales[i].data_ptr(), rows * 2, xv.data_ptr(), width, rows, cols, None)
        before = ext.counters()["gemv_fast"]
        ms = time_loop(torch, gemv, max(steps * 5, 50), max(warmup, 5))
        assert ext.counters()["gemv_fast"] > before, "the coded matrix did not take the tensor-core kernel"
        nbytes = rows * (rb + 2) + cols * 2 + rows * 2
        out[f"tq{width}_gemv_16384x4096"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_call": ms, "frac_hbm": nbytes / ms / 1e6 / hbm,
                                             "note": f"turboquant_gemv door, 16,384 rows of 4,096 codes at {width} bits: {nbytes / 1e6:.1f} MB a call, {copies} matrices cycled"}
        del codes, scales
    torch.cuda.empty_cache()

    # Kimi Delta Attention, one decode step of 64 heads of 128 (GLM's shape): the state read and written once, 8.4 MB
    heads, d = 64, 128
    S, conved, f, b, dt, a_log, gate, w, o = kda_workload(torch, gen, heads, d, 1)
    ms = time_loop(torch, lambda: fam.nn.kda_step(S.data_ptr(), conved.data_ptr(), f.data_ptr(), b.data_ptr(), dt.data_ptr(), a_log.data_ptr(), gate.data_ptr(),
                                                  w.data_ptr(), o.data_ptr(), heads, d, C.c_float(-5.0), C.c_float(1e-5), None), max(steps * 10, 100), 10)
    nbytes = 2 * heads * d * d * 4 + 6 * heads * d * 2
    out["kda_decode_64heads"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_step": ms, "frac_hbm": nbytes / ms / 1e6 / hbm,
                                 "note": "kda_step door, 64 heads x 128x128 fp32 state (8.4 MB: stays in L2 between steps), one block a head"}

    # the latent attention's two projections at decode (GLM's shape: 64 heads, 192 + 256 rows of a 512-wide latent a head):
    # a head's key rows fold its query into the latent (absorb), its value rows unfold the answer (expand); 8 distinct W cycled
    mh, nope, vd, lat, copies = 64, 192, 256, 512, 8
    Wl = (torch.randn((copies, mh * (nope + vd), lat), generator=gen, device="cuda", dtype=torch.float16) * 0.05)
    qa = torch.randn((mh * nope,), generator=gen, device="cuda", dtype=torch.float16)
    oa = torch.randn((mh * lat,), generator=gen, device="cuda", dtype=torch.float16)
    absorbed = torch.zeros((mh * lat,), device="cuda", dtype=torch.float16)
    expanded = torch.zeros((mh * vd,), device="cuda", dtype=torch.float16)
    mstate = {"i": 0}

    def absorb():
        i = mstate["i"] = (mstate["i"] + 1) % copies
        fam.nn.attention_absorb(absorbed.data_ptr(), qa.data_ptr(), Wl[i].data_ptr(), mh, nope, lat, nope + vd, C.c_float(0.0722), None)

    def expand():
        i = mstate["i"] = (mstate["i"] + 1) % copies
        fam.nn.attention_expand(expanded.data_ptr(), oa.data_ptr(), Wl[i].data_ptr(), mh, vd, lat, nope + vd, nope, None)
    for tag, fn, nbytes in (("mla_absorb_64heads", absorb, mh * nope * lat * 2 + mh * nope * 2 + mh * lat * 2),
                            ("mla_expand_64heads", expand, mh * vd * lat * 2 + mh * lat * 2 + mh * vd * 2)):
        ms = time_loop(torch, fn, max(steps * 5, 50), 5)
        out[tag] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_call": ms, "frac_hbm": nbytes / ms / 1e6 / hbm,
                    "note": f"{tag.split('_')[1]} door, 64 heads: {nbytes / 1e6:.1f} MB of the latent's expansion a call, 8 matrices cycled"}
    del Wl
    torch.cuda.empty_cache()

    # latent attention at decode (GLM's shape: 64 heads over one 512-wide latent that is key and value) through the three doors
    # scores_grouped + softmax_rows + mix — one fused launch (two when the positions are cut over blocks): 2,048 positions (what
    # the sparse attention gathers) with 16 latents cycled, and 65,536 (dense) with 4
    for Lm, copies in ((2048, 16), (65536, 4)):
        lat = torch.randn((copies, Lm, 512), generator=gen, device="cuda", dtype=torch.float16)
        qm = torch.randn((64, 512), generator=gen, device="cuda", dtype=torch.float16) * 2.0
        pm = torch.zeros((64, 8), device="cuda", dtype=torch.float32)          # never written by the fused triple
        om = torch.zeros((64, 512), device="cuda", dtype=torch.float16)
        lstate = {"i": 0}

        def latent():
            i = lstate["i"] = (lstate["i"] + 1) % copies
            fam.nn.attention_scores_grouped(pm.data_ptr(), qm.data_ptr(), lat[i].data_ptr(), 64, 1, 512, Lm)
            fam.nn.attention_softmax_rows(pm.data_ptr(), 64, Lm)
            fam.nn.attention_mix(om.data_ptr(), pm.data_ptr(), lat[i].data_ptr(), 64, 1, 512, Lm, None)
        before = ext.counters()["fused_latent"]
        ms = time_loop(torch, latent, max(steps * 5, 100), 10)
        assert ext.counters()["fused_latent"] > before, "the latent triple did not take the fused kernel"
        nbytes = Lm * 512 * 2 + 2 * 64 * 512 * 2
        out[f"mla_decode_64heads_{Lm}"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_call": ms, "frac_hbm": nbytes / ms / 1e6 / hbm, "tflops": 4.0 * 64 * 512 * Lm / ms / 1e9,
                                            "note": f"scores_grouped + softmax_rows + mix doors, 64 heads over {Lm} latents of 512: {nbytes / 1e6:.1f} MB a call, {copies} latents cycled"}
        try:
            # the same calls as the card sees them: one CUDA graph of `copies` launches (the three doors from Python cost the host
            # about as much as a short call costs the card)
            replay = mla_graph(torch, ext, lat, qm, om, Lm)
            out[f"mla_decode_64heads_{Lm}"]["ms_per_call_in_a_graph"] = time_loop(torch, replay, 20, 3) / copies
        except Exception as exc:                       # noqa: BLE001 - a capture the driver refuses is reported, not fatal
            out[f"mla_decode_64heads_{Lm}"]["ms_per_call_in_a_graph"] = None
            out[f"mla_decode_64heads_{Lm}"]["graph_note"] = str(exc)[:200]
        del lat
    torch.cuda.empty_cache()

    # a prompt chunk's projections through the expert-major GEMM door: 256 rows of 5,120 through a q projection of 8,192 rows at 4 bits,
    # and 256 rows of 4,096 through an o projection of 5,120 rows at 8 bits (4 coded matrices cycled: the weights come from HBM)
    for tag, er, ec, width in (("prompt_projection_256rows_q4", 8192, 5120, 4), ("prompt_projection_256rows_o8", 5120, 4096, 8)):
        T, copies = 256, 4
        ecodes = torch.randint(0, 256, (copies, er, ec * width // 8), generator=gen, device="cuda", dtype=torch.uint8)
        escales = ((torch.rand((er,), generator=gen, device="cuda") * 0.5 + 0.75) * (3.0 / ec ** 0.5)).to(torch.float16)
        ex = torch.randn((T, ec), generator=gen, device="cuda", dtype=torch.float16)
        epairs = torch.arange(T, device="cuda", dtype=torch.int32).repeat_interleave(2).contiguous()
        eout = torch.zeros((T, er), device="cuda", dtype=torch.float16)
        estate = {"i": 0}

        def project():
            i = estate["i"] = (estate["i"] + 1) % copies
            fam.nn.expert_rows(eout.data_ptr(), ecodes[i].data_ptr(), ecodes[i].numel(), escales.data_ptr(), escales.numel() * 2, ex.data_ptr(), epairs.data_ptr(),
                               T, width, er, ec, None)
        before = ext.counters()["expert_fast"]
        ms = time_loop(torch, project, max(steps * 3, 40), 5)
        assert ext.counters()["expert_fast"] > before, "the projection did not take the tcgen05 kernel"
        flops = 2.0 * T * er * ec
        out[tag] = {"value": flops / ms / 1e9, "unit": "TFLOP/s", "ms_per_call": ms, "frac_bf16_burst": flops / ms / 1e9 / pk["bf16_tflops"], "algorithmic_flops": flops,
                    "weights_gbs": er * ec * width / 8 / ms / 1e6,
                    "note": f"expert_rows door: {T} rows x {ec} through {er} coded rows at {width} bits ({er * ec * width / 8 / 1e6:.1f} MB of codes a call), one tcgen05 launch"}
        del ecodes, ex, eout
    torch.cuda.empty_cache()

    # the sparse attention's indexer at decode: 32 index heads of 128 score 8,192 pooled keys, the top 512 pools chosen
    ih, idim, pools, topk, kpool = 32, 128, 8192, 512, 4
    iq = torch.randn((ih * idim,), generator=gen, device="cuda", dtype=torch.float16)
    iw = torch.randn((ih,), generator=gen, device="cuda", dtype=torch.float16)
    pooled = torch.randn((pools, idim), generator=gen, device="cuda", dtype=torch.float16)
    iscores = torch.zeros((pools,), device="cuda", dtype=torch.float32)
    iindex = torch.zeros((topk * kpool + kpool,), device="cuda", dtype=torch.int32)
    icount = torch.zeros((1,), device="cuda", dtype=torch.int32)

    def indexer():
        fam.nn.index_scores(iscores.data_ptr(), iq.data_ptr(), iw.data_ptr(), pooled.data_ptr(), ih, idim, pools, C.c_float(0.088))
        fam.nn.index_select(iindex.data_ptr(), icount.data_ptr(), iscores.data_ptr(), pools, topk, kpool, pools * kpool, 3)
    ms = time_loop(torch, indexer, max(steps * 5, 50), 5)
    out["glm_indexer_8192pools"] = {"value": pools / ms * 1e3, "unit": "pools/s", "ms_per_call": ms, "algorithmic_bytes": pools * idim * 2 + ih * idim * 2 + pools * 4 * 2 + topk * kpool * 4,
                                    "note": "index_scores + index_select: 32 heads of 128 over 8,192 pooled keys, the top 512 pools as positions (two launches)"}

    # configuration 5: recurrent decode steps (batched so that state traffic is real) and the prompt
    heads, d = 32, 128
    for seqs, tag in ((1, "config5_deltanet_decode_1seq"), (64, "config5_deltanet_decode_64seq")):
        S = torch.zeros((seqs, heads, d, d), device="cuda", dtype=torch.float32)
        conved = torch.randn((seqs, 1, 3 * heads * d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.1
        z = torch.randn((seqs, 1, heads * d), generator=gen, device="cuda", dtype=torch.bfloat16)
        beta = torch.rand((seqs, 1, heads), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        g = (-torch.rand((seqs, 1, heads), generator=gen, device="cuda", dtype=torch.float32)).to(torch.bfloat16)
        w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
        o = torch.zeros((seqs, 1, heads * d), device="cuda", dtype=torch.bfloat16)
        ms = time_loop(torch, lambda: ext.deltanet(S, conved, z, beta, g, w, o, heads, heads, d, 1, seqs, 0, ext.BF16), max(steps * 10, 100), 10)
        nbytes = seqs * (2 * heads * d * d * 4 + 3 * heads * d * 2 + 2 * heads * d * 2 + 2 * heads * 2 + d * 2)
        out[tag] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_step": ms, "frac_hbm": nbytes / ms / 1e6 / hbm,
                    "note": f"{seqs} sequence(s) x 32 heads x 128x128 fp32 state, read and written once a step"
                            + (" (2 MiB of state: stays in L2 between steps)" if seqs == 1 else "")}
    # the one-sequence step without the host in the loop: 64 steps captured once in a CUDA graph
    S = torch.zeros((1, heads, d, d), device="cuda", dtype=torch.float32)
    conved = torch.randn((64, 3 * heads * d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.1
    z = torch.randn((64, heads * d), generator=gen, device="cuda", dtype=torch.bfloat16)
    beta = torch.rand((64, heads), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    g = (-torch.rand((64, heads), generator=gen, device="cuda", dtype=torch.float32)).to(torch.bfloat16)
    o = torch.zeros((64, heads * d), device="cuda", dtype=torch.bfloat16)
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(64):
            ext.deltanet(S, conved[i], z[i], beta[i], g[i], w, o[i], heads, heads, d, 1, 1, 0, ext.BF16, stream=side.cuda_stream)
    ms = time_loop(torch, graph.replay, 20, 3) / 64
    nbytes = 2 * heads * d * d * 4 + 3 * heads * d * 2 + 2 * heads * d * 2 + 2 * heads * 2 + d * 2
    out["config5_deltanet_decode_1seq_graph"] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_step": ms, "frac_hbm": nbytes / ms / 1e6 / hbm,
                                                 "note": "the same step, 64 consecutive positions of one sequence captured in a CUDA graph (no host between launches)"}
    del graph
    T = 8192
    S = torch.zeros((1, heads, d, d), device="cuda", dtype=torch.float32)
    conved = torch.randn((T, 3 * heads * d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.1
    z = torch.randn((T, heads * d), generator=gen, device="cuda", dtype=torch.bfloat16)
    beta = torch.rand((T, heads), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    g = (-torch.rand((T, heads), generator=gen, device="cuda", dtype=torch.float32)).to(torch.bfloat16)
    o = torch.zeros((T, heads * d), device="cuda", dtype=torch.bfloat16)
    ms = time_loop(torch, lambda: ext.deltanet(S, conved, z, beta, g, w, o, heads, heads, d, T, 1, 0, ext.BF16), 3, 1)
    nbytes = T * (3 * heads * d * 2 + 2 * heads * d * 2 + 4 * heads) + 2 * heads * d * d * 4
    out["config5_deltanet_prefill_8192"] = {"value": T / ms * 1e3, "unit": "positions/s", "ms": ms, "frac_hbm": nbytes / ms / 1e6 / hbm, "algorithmic_bytes": nbytes,
                                            "tflops": 7.0 * d * d * heads * T / ms / 1e9,
                                            "note": "one sequence, 8,192 positions, 64 at a time (chunked form), fp32 FMA"}

    # configuration 2: causal prefill
    qh, kvh, d, T = 16, 2, 256, 4096
    q = torch.randn((T, qh, d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.5
    k = torch.randn((T, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.5
    v = torch.randn((T, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.5
    o = torch.zeros((T, qh, d), device="cuda", dtype=torch.bfloat16)
    try:
        ms = time_loop(torch, lambda: ext.prefill(o, q, k, v, qh, kvh, d, 0, T, ext.BF16), max(steps, 20), max(warmup, 3))
        flops = 4.0 * qh * d * T * (T + 1) / 2
        out["config2_causal_prefill"] = {"value": flops / ms / 1e9, "unit": "TFLOP/s", "ms_per_call": ms, "frac_bf16_burst": flops / ms / 1e9 / pk["bf16_tflops"],
                                         "note": "4,096 rows, 16q/2kv, d256, bf16, one fused kernel"}
    except ext.B200Error as e:
        out["config2_causal_prefill"] = {"value": None, "unit": "TFLOP/s", "note": f"fused prefill not available: {e}"}
    return out


# DRAM bytes a launch (dram__bytes_read.sum + dram__bytes_write.sum) over algorithmic bytes, from each kernel's profiler
# capture on a small case of the same kernel (one summary a kernel and workload is kept with the sources).  A
# ratio is scaled to the full launch by the launch's algorithmic bytes — each of these kernels passes over its input once,
# so traffic grows in proportion — and an absolute figure is a capture of the very workload timed here.
ROOFLINES = {
    # entry: (bound, kernel, traffic ratio or absolute bytes or None, where the traffic figure comes from)
    "config1_decode_doors": ("hbm", "sv::decode_kernel<128, fp16, 1>", 1.016, "ratio of the capture of this kernel on a 65,536-position cache, scaled by bytes"),
    "config1_decode_kernel": ("hbm", "sv::decode_kernel<128, fp16, 1>", 1.016, "ratio of the capture of this kernel on a 65,536-position cache, scaled by bytes"),
    "config4_long_context_1gpu_resident": ("hbm", "sv::decode_kernel<128, bf16, 1>", 1.016, "ratio of the capture of this kernel on a 65,536-position cache, scaled by bytes"),
    "tq8_tier_d128": ("hbm", "sv::tq_attend_kernel<128, 8, 1>", 276.6e6, "capture of this workload"),
    "tq4_tier_d128": ("hbm", "sv::tq_attend_kernel<128, 4, 1>", 142.0e6, "capture of this workload"),
    "tq8_tier_d128_rows16": ("hbm", "sv::tq_attend_kernel<128, 8, 2> (16 rows a launch: latency- and issue-bound, far from either roof)", None, None),
    "glm_indexer_8192pools": ("hbm", "sv::index_scores_kernel + sv::index_select_kernel (two launches, 2 MB: launch-bound)", None, None),
    "tq8_tier_d256": ("hbm", "sv::tq_attend_kernel<256, 8, 1>", 1.015, "ratio of the head_dim-128 capture, scaled by bytes"),
    "tq4_tier_d256": ("hbm", "sv::tq_attend_kernel<256, 4, 1>", 1.026, "ratio of the head_dim-128 capture, scaled by bytes"),
    "tq4_gemv_16384x4096": ("hbm", "sv::tq_gemv_fast_kernel<1, 4>", 33.69e6, "capture of this workload"),
    "tq8_gemv_16384x4096": ("hbm", "sv::tq_gemv_fast_kernel<1, 8>", 67.43e6, "capture of this workload"),
    "kda_decode_64heads": ("hbm", "sv::kda_steps_kernel<128, false>", 4.31e6, "capture of this workload (the 8.4 MB state stays in L2 between steps)"),
    "mla_absorb_64heads": ("hbm", "sv::absorb_kernel", None, None),
    "mla_expand_64heads": ("hbm", "sv::expand_kernel", None, None),
    "mla_decode_64heads_2048": ("hbm", "sv::mla_decode_kernel<64, fp16> + sv::mla_fold_kernel (2 MB: latency-bound)", 0.95, "ratio of the capture of this workload (2.23 MB for 2.36 MB)"),
    "mla_decode_64heads_65536": ("hbm", "sv::mla_decode_kernel<64, fp16> + sv::mla_fold_kernel", 0.96, "ratio of the capture of this workload (72.3 MB for 75.5 MB: a tail of the latent is still in L2)"),
    "prompt_projection_256rows_q4": ("tensor", "sv::expert_fast_kernel", None, None),
    "prompt_projection_256rows_o8": ("tensor", "sv::expert_fast_kernel", None, None),
    "config5_deltanet_decode_1seq": ("hbm", "sv::deltanet_steps_kernel<128, bf16, false, true> (one cluster a head)", None, None),
    "config5_deltanet_decode_1seq_graph": ("hbm", "sv::deltanet_steps_kernel<128, bf16, false, true> (one cluster a head)", None, None),
    "config5_deltanet_decode_64seq": ("hbm", "sv::deltanet_step_head_kernel<128, bf16> (one launch a step of the batch)", 215.8e6, "capture of this workload (part of the written state is still in L2 when the kernel ends)"),
    "config5_deltanet_prefill_8192": ("hbm", "sv::deltanet_prep_kernel + deltanet_chunk_kernel + deltanet_norm_kernel", 1.921, "ratio of the capture of the three kernels on 2,048 positions (163.3 MB for 85.0 MB), scaled by bytes"),
    "config2_causal_prefill": ("tensor", "sv::prefill_kernel<256, bf16>", 41.9e6 * 1.001, "the capture on 2,048 rows read its inputs once (21.02 MB for 21.0 MB); scaled by input bytes"),
}


def attach_rooflines(others, pk, cpu):
    """Gives every entry of `others` its roofline object and, for configurations 1, 2, 4 and 5, the reference CPU family's
    figure on the same configuration."""
    beside = {"config1_decode_doors": "config1", "config1_decode_kernel": "config1", "config2_causal_prefill": "config2",
              "config4_long_context_1gpu_resident": "config4", "config5_deltanet_decode_1seq": "config5_decode",
              "config5_deltanet_decode_1seq_graph": "config5_decode", "config5_deltanet_prefill_8192": "config5_prefill",
              "config5_deltanet_decode_64seq": "config5_decode_64seq", "tq8_tier_d128": "tq8_tier_d128", "tq4_tier_d128": "tq4_tier_d128",
              "tq4_gemv_16384x4096": "tq4_gemv_16384x4096", "tq8_gemv_16384x4096": "tq8_gemv_16384x4096", "mla_decode_64heads_2048": "mla_decode_64heads_2048",
              "mla_decode_64heads_65536": "mla_decode_64heads_65536", "prompt_projection_256rows_q4": "prompt_projection_256rows_q4",
              **{n: n for n in ("prompt_projection_256rows_o8", "tq8_tier_d256", "tq4_tier_d256", "tq8_tier_d128_rows16", "kda_decode_64heads",
                                "mla_absorb_64heads", "mla_expand_64heads", "glm_indexer_8192pools")}}
    for name, e in others.items():
        ms = e.get("ms_per_call", e.get("ms_per_step", e.get("ms")))
        spec = ROOFLINES.get(name)
        if spec and ms and e.get("value") is not None:
            bound, kernel, traffic, how = spec
            work = e.get("algorithmic_bytes") if bound == "hbm" else e.get("algorithmic_flops")
            if work is None:
                work = e["value"] * ms * (1e6 if e.get("unit") == UNIT else 1e9)
            e["roofline"] = roofline(bound, work, ms, pk, kernel, traffic, how)
        if name in beside and beside[name] in cpu:
            e["cpu_baseline"] = cpu[beside[name]]


def pinned_h2d_peak(torch):
    """This box's pinned host-to-device copy rate: one 1 GiB cudaMemcpyAsync from pinned memory, best of 3, CUDA events."""
    n = 1 << 30
    host = torch.empty(n, dtype=torch.uint8).pin_memory()
    card = torch.empty(n, dtype=torch.uint8, device="cuda")
    best = None
    for _ in range(4):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); card.copy_(host, non_blocking=True); b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        best = ms if best is None else min(best, ms)
    del host, card
    return n / best / 1e6


def long_context(torch, dist, rank, world, steps, pk):
    """Configuration 4 on `world` GPUs: one sequence of 262,144 positions, 32 q heads on 4 kv heads, head_dim 128, bf16;
    kv heads sharded over the ranks (and the range halved among the two ranks of a kv head at 8), the first 65,536
    positions in pinned host RAM and streamed on a side stream.  Timed twice: as specified, and with every position
    already on the card.  Strong scaling: the whole job's bytes over the slowest rank's device time, with rank 0's own
    one-GPU time of the whole problem measured in the same run beside it."""
    from silvann_b200 import ext, sharded, workloads
    qh, kvh, d, L, HOST = 32, 4, 128, 262144, 65536
    if world not in (1, 2, 4, 8):
        return {"note": f"not run at {world} GPUs"}
    nbytes = 2 * L * kvh * d * 2
    shard = sharded.shard_plan(qh, kvh, L, world)[rank]
    w = workloads.config4()                                   # numpy PCG64 seed 1004: the same sequence on every rank, each keeps its share
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()
    out = {}

    def timed(fn, n):
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / n], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # the whole problem on rank 0 alone, every position on the card: the t_1 of this run's strong-scaling figure
    t1 = torch.zeros(1, device="cuda", dtype=torch.float64)
    if rank == 0:
        k1, v1, q1 = up(w.k), up(w.v), up(w.q)
        o1 = torch.zeros((qh, d), dtype=torch.int16, device="cuda")
        for _ in range(3):
            ext.decode(o1, None, q1, k1, v1, qh, kvh, d, L, ext.BF16)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            ext.decode(o1, None, q1, k1, v1, qh, kvh, d, L, ext.BF16)
        b.record()
        torch.cuda.synchronize()
        t1[0] = a.elapsed_time(b) / steps
        del k1, v1, q1
    if world > 1:
        dist.broadcast(t1, 0)
    t1 = float(t1.item())

    n, heads = shard.positions, shard.kv_heads
    k = up(w.k[shard.pos_lo:shard.pos_hi, shard.kv_head_lo:shard.kv_head_hi])
    v = up(w.v[shard.pos_lo:shard.pos_hi, shard.kv_head_lo:shard.kv_head_hi])
    q = up(w.q[shard.q_head_lo:shard.q_head_hi])
    del w
    h_len = max(0, min(HOST, shard.pos_hi) - shard.pos_lo)
    k_host = k[:h_len].cpu().pin_memory() if h_len else None
    v_host = v[:h_len].cpu().pin_memory() if h_len else None
    # the box's pinned host-to-device rate: rank 0 alone, and then every rank that holds a share of the host tier at once (the
    # ranks' copies may share host links and memory channels: what a GPU can get while its neighbours stream too is the bound of
    # the tiered step at N > 1)
    h2d_alone = torch.zeros(1, device="cuda", dtype=torch.float64)
    if rank == 0:
        h2d_alone[0] = pinned_h2d_peak(torch)
    if world > 1:
        dist.broadcast(h2d_alone, 0)
        dist.barrier()
    h2d_alone = float(h2d_alone.item())
    h2d_peak = h2d_alone
    if world > 1:
        # (only the ranks that hold a share of the host tier copy in the tiered step: only they copy here)
        together = torch.tensor([pinned_h2d_peak(torch) if h_len else float("inf")], device="cuda", dtype=torch.float64)
        dist.all_reduce(together, op=dist.ReduceOp.MIN)
        h2d_peak = float(together.item())
        dist.barrier()
    # the ranks that split a kv head's range exchange residuals through the library's own kernel over peer memory; the
    # buffers' handles travel once, here
    exchange = sharded.connect_exchange(torch, ext, dist, shard.group, rank, shard.q_heads * (d + 2) * 4) if world > 1 else None
    if len(shard.group) == 1:
        exchange = None
    for tag, (kh, vh, hl, kd, vd, dl) in {"tiered": (k_host, v_host, h_len, k[h_len:] if n > h_len else None, v[h_len:] if n > h_len else None, n - h_len),
                                           "resident": (None, None, 0, k, v, n)}.items():
        runner = sharded.LongContextRank(torch, ext, shard, d, ext.BF16, kh, vh, hl, kd, vd, dl, dist, None, chunk_positions=0, stages=3, exchange=exchange)
        ms = timed(lambda: runner.step(q), steps)
        out[tag] = {"value": nbytes / ms / 1e6, "unit": UNIT, "ms_per_step": ms, "frac_hbm_of_n_gpus": nbytes / ms / 1e6 / (pk["hbm_gbs"] * world)}
        runner.close()
    out["resident"]["one_gpu_ms_same_run"] = t1
    out["resident"]["strong_scaling_efficiency"] = t1 / (world * out["resident"]["ms_per_step"])
    out["resident"]["roofline"] = roofline("hbm", nbytes / world, out["resident"]["ms_per_step"], pk, "sv::decode_kernel<128, bf16, 1>" + (" + sv::exchange_merge_kernel" if exchange else ""),
                                           1.016, "ratio of the capture of this kernel on a 65,536-position cache, scaled by bytes; per GPU")
    host_bytes = 2 * HOST * kvh * d * 2
    gbs = host_bytes / out["tiered"]["ms_per_step"] / 1e6
    holders = min(world, kvh)                                 # ranks that hold a share of the host tier (the first range half of every kv head)
    out["tiered"].update({"host_tier_bytes": host_bytes, "host_tier_gbs": gbs, "host_tier_gbs_per_holding_gpu": gbs / holders,
                          "pinned_h2d_peak_gbs_measured": h2d_alone, "pinned_h2d_peak_gbs_holding_ranks_at_once": h2d_peak,
                          "host_tier_frac_of_h2d_peak": gbs / holders / h2d_peak, "host_tier_frac_of_h2d_peak_one_gpu_alone": gbs / holders / h2d_alone,
                          "lower_bound_ms": max(host_bytes / holders / h2d_peak / 1e6, (nbytes - host_bytes) / world / pk["hbm_gbs"] / 1e6)})
    if exchange is not None:
        # the exchange alone: a residual each, pushed, waited for and folded — the merge latency of the range split
        res = torch.zeros((shard.q_heads, d + 2), dtype=torch.float32, device="cuda"); res[:, 1] = 1.0
        o = torch.zeros((shard.q_heads, d), dtype=torch.int16, device="cuda")
        out["merge_latency_us"] = timed(lambda: exchange.merge_finish(o, None, res, shard.q_heads, d, ext.BF16), 200) * 1e3
        exchange.close()
    if world > 1:
        # the tensor-parallel sum that follows head-sharded attention, HIDDEN = 5,120 halves: one launch a rank over peer memory,
        # and the all-gather + vector_sum form beside it
        hidden = 5120
        part = torch.from_numpy(np.random.default_rng(50 + rank).standard_normal(hidden).astype(np.float16).view(np.int16)).cuda()
        peer = sharded.PeerSum(torch, ext, dist, hidden, ext.FP16)
        total = torch.empty_like(part)
        out["tp_sum_us"] = timed(lambda: peer.sum(part, total), 200) * 1e3
        import silvann_b200
        vsum = sharded.family_vector_sum(torch, silvann_b200.family())
        out["tp_sum_allgather_us"] = timed(lambda: sharded.sum_over_ranks(part, dist, vsum), 50) * 1e3
        # the same sum with its producer: each rank's share (4,096 / N columns) of a 4-bit coded 5,120-row output projection, the partials
        # exchanged and added in the kernel's epilogue — against the door followed by the sum above
        cols = 4096 // world
        gen = torch.Generator(device="cuda"); gen.manual_seed(90 + rank)
        codes = torch.randint(0, 256, (hidden, cols // 2), generator=gen, device="cuda", dtype=torch.uint8)
        scales = ((torch.rand((hidden,), generator=gen, device="cuda") * 0.5 + 0.75) * (3.0 / 4096 ** 0.5)).to(torch.float16)
        vec = torch.randn((cols,), generator=gen, device="cuda", dtype=torch.float16)
        fused = torch.empty_like(part)
        out["o_projection_and_tp_sum_fused_us"] = timed(lambda: peer.exchange.gemv_sum(fused, codes, scales, vec, 4, hidden, cols), 200) * 1e3
        fam = silvann_b200.family()

        def unfused():
            fam.nn.turboquant_gemv(part.data_ptr(), codes.data_ptr(), codes.numel(), scales.data_ptr(), scales.numel() * 2, vec.data_ptr(), 4, hidden, cols, None)
            peer.sum(part, total)
        out["o_projection_then_tp_sum_us"] = timed(unfused, 200) * 1e3
        peer.close()
    out["note"] = ("kv heads sharded over ranks" + (", each kv head's range halved over two ranks, residuals pushed into the partner's memory and folded by one kernel a rank (no NCCL on the data path)" if world > kvh else ", no exchange")
                   + "; tiered: first 65,536 positions streamed from pinned host RAM each step (PCIe-bound); resident: all positions in HBM; strong scaling: whole-job bytes over the slowest rank's time")
    assert ext.device_status() == 0, "a bounded device-side wait ran out during the long-context runs"
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import silvann_b200
    from silvann_b200 import ext
    fam = silvann_b200.family()
    assert fam.sys.bind_device(local) == 1, "the family does not take this device (needs sm_100)"
    pk = peaks()
    steps, warmup = args.steps, max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.only == "long_context":
        lc = long_context(torch, dist, rank, world, max(steps, 10), pk)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        if rank == 0:
            print(json.dumps({"only": "long_context_config4", "n_gpus": world, "long_context_config4": lc}))
        return

    wl = PagedWorkload(torch, rank)

    # ---- value: K steps, inputs resident ----
    for _ in range(warmup):
        wl.step()
    barrier()
    c0 = ext.counters()["launches"]
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    with ClockSampler(device_index()) as clocks:
        barrier()
        ev[0].record()
        for i in range(steps):
            wl.step()
            ev[i + 1].record()
        barrier()
    launches = ext.counters()["launches"] - c0
    total_ms = ev[0].elapsed_time(ev[steps])
    per_launch_ms = float(np.mean([ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]))
    t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / steps
    status = ext.device_status()

    # ---- e2e: host buffers, copies inside the timed region ----
    e2e = EndToEnd(torch, wl, fam)
    for _ in range(2):
        e2e.step()
    barrier()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    e_steps = max(3, min(steps, 20))
    t0.record()
    for _ in range(e_steps):
        e2e.step()
    t1.record()
    barrier()
    te = torch.tensor([t0.elapsed_time(t1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item()) / e_steps

    kv_all = wl.kv_bytes * world
    line = {
        "metric": METRIC, "value": kv_all / ms_step / 1e6, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_of(wl.layout),
        "sharding": "one independent batch per GPU (sequences are independent: no collective); the sharded path with an exchange is configuration 4, under long_context_config4",
        "l2": "inputs (3.3 GB a step) larger than L2; no flush needed",
        "e2e": {"value": kv_all / e2e_ms / 1e6, "unit": UNIT, "h2d_bytes_per_step": e2e.h2d, "d2h_bytes_per_step": e2e.d2h, "ms_per_step": e2e_ms,
                "note": "plan + upload of queries and each sequence's newest K/V row (pinned host memory, memory_write door) + row append into the pool + decode + memory_read of outputs; the KV pool is the path's resident state"},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "device_status": status,
    }
    if rank == 0:
        line["roofline"] = roofline("hbm", wl.kv_bytes, per_launch_ms, pk, "sv::decode_kernel<256, bf16, 1>", 1.016,
                                    "ratio of the capture of this kernel on a batch of 180,181 positions (374.9 MB for 369.0 MB), scaled by positions")
        if world == 1:
            line["cpu_baseline"] = cpu_baseline_paged(wl)
            if not args.no_others:
                line["gpu_baseline"] = gpu_baseline(torch, wl, pk, steps)
                others = other_workloads(torch, fam, pk, steps, warmup)
                attach_rooflines(others, pk, cpu_baselines_others())
                line["others"] = others
    e2e.close()
    if not args.no_others:
        del wl, e2e
        torch.cuda.empty_cache()
        try:
            lc = long_context(torch, dist, rank, world, max(steps, 10), pk)
        except Exception as e:                                   # the headline line is still printed; the failure is said in it
            lc = {"error": f"{type(e).__name__}: {e}"}
        if rank == 0:
            line["long_context_config4"] = lc
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU implementation of the path on this host's cores
# ---------------------------------------------------------------------------------------------------------------------

def run_reference(args):
    """The reference's CPU family (compiled unmodified by the checker's build recipe; the C restatement where that is absent) on rank 0's batch of configuration 3:
    the same layout and the same values this arm reads (numpy PCG64), every sequence gathered to the contiguous fp16 planes
    the reference's doors take — it has neither paging nor bf16 — outside the timed region.  A step attends the whole batch,
    attention_scores + attention_mix a sequence, with every host thread the family's pool takes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    R = oracle.reference()
    L, q, k_pool, v_pool = paged_inputs(0)
    steps, warmup = args.steps, max(args.warmup, 3)
    if R is not None:
        planes = reference_planes(L, q, k_pool, v_pool)
        del k_pool, v_pool
        pbuf = np.empty(L.q_heads * int(L.seq_lens.max()), np.float32)
        nbytes, kind = L.kv_bytes, "reference"
        cores, pool_line = cpu_cores(R)
        sample = f"the whole batch every step: {len(planes)} sequences, {L.positions} positions, {nbytes / 1e6:.0f} MB of KV, fp16 copies of the same values, attention_scores + attention_mix a sequence"

        def step():
            for qs, ks, vs, n in planes:
                R.decode(qs, ks, vs, L.q_heads, L.kv_heads, L.head_dim, n, pbuf[:L.q_heads * n].reshape(L.q_heads, n))
    else:
        P = oracle.port()
        s = int(np.argmin(L.seq_lens))
        planes = reference_planes(L, q, k_pool, v_pool, [s])
        nbytes, kind, cores, pool_line = planes[0][3] * 2 * L.kv_heads * L.head_dim * 2, "port", 1, None
        sample = f"the shortest sequence of the batch ({planes[0][3]} positions) through the scalar C restatement every step"

        def step():
            qs, ks, vs, n = planes[0]
            P.decode(qs, ks, vs, L.q_heads, L.kv_heads, L.head_dim, n, 0)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    value = nbytes / ms / 1e6
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over fp16", "data": "synthetic",
        "config": config_of(L),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample, "pool_report": pool_line},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ---------------------------------------------------------------------------------------------------------------------
# small single-kernel cases, sized for a profiler capture (a few hundred MB on the device, a handful of launches)
# ---------------------------------------------------------------------------------------------------------------------

def run_case(args):
    import torch
    import silvann_b200
    from silvann_b200 import ext, workloads
    torch.cuda.set_device(0)
    fam = silvann_b200.family()
    assert fam.sys.bind_device(0) == 1
    gen = torch.Generator(device="cuda"); gen.manual_seed(5)
    name, steps = args.case, args.steps
    if name == "paged_small":
        # configuration 3's shape with 8 sequences of up to 40,000 positions: ~0.3 GB of KV a launch, larger than L2
        L = workloads.config3_layout(seqs=8, lo=8000, hi=40000)
        shape = (L.pool_pages, workloads.PAGE_POSITIONS, L.kv_heads, L.head_dim)
        kp = torch.randn(shape, generator=gen, device="cuda", dtype=torch.bfloat16)
        vp = torch.randn(shape, generator=gen, device="cuda", dtype=torch.bfloat16)
        q = torch.randn((8, L.q_heads, L.head_dim), generator=gen, device="cuda", dtype=torch.bfloat16)
        o = torch.zeros_like(q)
        table = torch.from_numpy(L.page_table).cuda()
        plan = ext.Plan(); plan.plan(L.seq_lens, L.q_heads, L.kv_heads, L.head_dim)
        fn = lambda: plan.decode(o, None, q, kp, vp, L.pool_pages, workloads.PAGE_POSITIONS, table, L.page_table.shape[1], ext.BF16)
        work, unit = L.kv_bytes, "bytes"
    elif name == "long_small":
        # configuration 4's shape (32q/4kv, d128, bf16), 131,072 positions: 268 MB of KV a launch
        qh, kvh, d, n = 32, 4, 128, 131072
        k = torch.randn((n, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16)
        v = torch.randn((n, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16)
        q = torch.randn((qh, d), generator=gen, device="cuda", dtype=torch.bfloat16)
        o = torch.zeros_like(q)
        fn = lambda: ext.decode(o, None, q, k, v, qh, kvh, d, n, ext.BF16)
        work, unit = 2 * n * kvh * d * 2, "bytes"
    elif name == "decode_cfg1":
        # configuration 1 through the two doors (one fused launch a pair), 16 distinct caches cycled: 268 MB in all
        qh, kvh, d, n, copies = 16, 4, 128, 8192, 16
        k = torch.randn((copies, n, kvh, d), generator=gen, device="cuda", dtype=torch.float16)
        v = torch.randn((copies, n, kvh, d), generator=gen, device="cuda", dtype=torch.float16)
        q = torch.randn((qh, d), generator=gen, device="cuda", dtype=torch.float16)
        p = torch.zeros((qh, n), device="cuda", dtype=torch.float32)
        o = torch.zeros((qh, d), device="cuda", dtype=torch.float16)
        state = {"i": 0}

        def fn():
            i = state["i"] = (state["i"] + 1) % copies
            fam.nn.attention_scores(p.data_ptr(), q.data_ptr(), k[i].data_ptr(), qh, kvh, d, n)
            fam.nn.attention_mix(o.data_ptr(), p.data_ptr(), v[i].data_ptr(), qh, kvh, d, n, None)
        work, unit = 2 * n * kvh * d * 2, "bytes"
    elif name == "decode_cfg1_graph":
        # configuration 1 as the card sees it: one CUDA graph of 64 decode launches, a distinct cache each (1.07 GB)
        fn, work, unit = config1_graph(torch, ext, gen)
        work *= 64
    elif name in ("tq8_small", "tq4_small"):
        # a coded tier of 262,144 positions, 32q/4kv heads of 128, through the door pair (one fused launch): 273 / 138 MB
        width, dh, tqh, tkvh, Lt = (8 if name == "tq8_small" else 4), 128, 32, 4, 262144
        rb = dh * width // 8
        kc = torch.randint(0, 256, (2, Lt * tkvh, rb), generator=gen, device="cuda", dtype=torch.uint8)
        vc = torch.randint(0, 256, (2, Lt * tkvh, rb), generator=gen, device="cuda", dtype=torch.uint8)
        ks = (torch.rand((2, Lt * tkvh), generator=gen, device="cuda") * 0.5 + 0.75).to(torch.float16)
        vs = (torch.rand((2, Lt * tkvh), generator=gen, device="cuda") * 0.5 + 0.75).to(torch.float16)
        tq_q = torch.randn((tqh, dh), generator=gen, device="cuda", dtype=torch.float16) * 0.25
        tp = torch.zeros((tqh, 8), device="cuda", dtype=torch.float32)
        tres = torch.zeros((tqh, dh + 2), device="cuda", dtype=torch.float32)
        tstate = {"i": 0}

        def fn():
            i = tstate["i"] = 1 - tstate["i"]
            fam.nn.attention_weights_tq(tp.data_ptr(), tres.data_ptr(), tq_q.data_ptr(), kc[i].data_ptr(), ks[i].data_ptr(), tqh, tkvh, dh, Lt, width)
            fam.nn.attention_residual_mix_tq(tres.data_ptr(), tp.data_ptr(), vc[i].data_ptr(), vs[i].data_ptr(), tqh, tkvh, dh, Lt, width)
        work, unit = 2 * Lt * tkvh * (rb + 2), "bytes"
    elif name in ("gemv4_small", "gemv8_small"):
        # a coded matrix of 16,384 x 4,096 through the turboquant_gemv door, 8 / 4 distinct matrices cycled (268 MB)
        width = 4 if name == "gemv4_small" else 8
        rows, cols, copies = 16384, 4096, (8 if width == 4 else 4)
        codes, scales, xv, ov, rb = coded_weights(torch, gen, copies, rows, cols, width)
        gstate = {"i": 0}

        def fn():
            i = gstate["i"] = (gstate["i"] + 1) % copies
            fam.nn.turboquant_gemv(ov.data_ptr(), codes[i].data_ptr(), rows * rb, scales[i].data_ptr(), rows * 2, xv.data_ptr(), width, rows, cols, None)
        work, unit = rows * (rb + 2) + cols * 2 + rows * 2, "bytes"
    elif name in ("mla_absorb", "mla_expand"):
        import ctypes as C
        mh, nope, vd, lat, copies = 64, 192, 256, 512, 8
        Wl = (torch.randn((copies, mh * (nope + vd), lat), generator=gen, device="cuda", dtype=torch.float16) * 0.05)
        qa = torch.randn((mh * nope,), generator=gen, device="cuda", dtype=torch.float16)
        oa = torch.randn((mh * lat,), generator=gen, device="cuda", dtype=torch.float16)
        absorbed = torch.zeros((mh * lat,), device="cuda", dtype=torch.float16)
        expanded = torch.zeros((mh * vd,), device="cuda", dtype=torch.float16)
        mstate = {"i": 0}
        if name == "mla_absorb":
            def fn():
                i = mstate["i"] = (mstate["i"] + 1) % copies
                fam.nn.attention_absorb(absorbed.data_ptr(), qa.data_ptr(), Wl[i].data_ptr(), mh, nope, lat, nope + vd, C.c_float(0.0722), None)
            work = mh * nope * lat * 2 + mh * nope * 2 + mh * lat * 2
        else:
            def fn():
                i = mstate["i"] = (mstate["i"] + 1) % copies
                fam.nn.attention_expand(expanded.data_ptr(), oa.data_ptr(), Wl[i].data_ptr(), mh, vd, lat, nope + vd, nope, None)
            work = mh * vd * lat * 2 + mh * lat * 2 + mh * vd * 2
        unit = "bytes"
    elif name == "kda_decode":
        import ctypes as C
        heads, d = 64, 128
        S, conved, f, b, dt, a_log, gate, w, o = kda_workload(torch, gen, heads, d, 1)
        fn = lambda: fam.nn.kda_step(S.data_ptr(), conved.data_ptr(), f.data_ptr(), b.data_ptr(), dt.data_ptr(), a_log.data_ptr(), gate.data_ptr(),
                                     w.data_ptr(), o.data_ptr(), heads, d, C.c_float(-5.0), C.c_float(1e-5), None)
        work, unit = 2 * heads * d * d * 4 + 6 * heads * d * 2, "bytes"
    elif name == "deltanet_64":
        heads, d, seqs = 32, 128, 64
        S = torch.zeros((seqs, heads, d, d), device="cuda", dtype=torch.float32)
        conved = torch.randn((seqs, 1, 3 * heads * d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.1
        z = torch.randn((seqs, 1, heads * d), generator=gen, device="cuda", dtype=torch.bfloat16)
        beta = torch.rand((seqs, 1, heads), generator=gen, device="cuda").to(torch.bfloat16)
        g = (-torch.rand((seqs, 1, heads), generator=gen, device="cuda")).to(torch.bfloat16)
        w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
        o = torch.zeros((seqs, 1, heads * d), device="cuda", dtype=torch.bfloat16)
        fn = lambda: ext.deltanet(S, conved, z, beta, g, w, o, heads, heads, d, 1, seqs, 0, ext.BF16)
        work, unit = seqs * (2 * heads * d * d * 4 + 3 * heads * d * 2 + 2 * heads * d * 2 + 2 * heads * 2 + d * 2), "bytes"
    elif name == "deltanet_prefill":
        heads, d, T = 32, 128, 2048
        S = torch.zeros((1, heads, d, d), device="cuda", dtype=torch.float32)
        conved = torch.randn((T, 3 * heads * d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.1
        z = torch.randn((T, heads * d), generator=gen, device="cuda", dtype=torch.bfloat16)
        beta = torch.rand((T, heads), generator=gen, device="cuda").to(torch.bfloat16)
        g = (-torch.rand((T, heads), generator=gen, device="cuda")).to(torch.bfloat16)
        w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
        o = torch.zeros((T, heads * d), device="cuda", dtype=torch.bfloat16)
        fn = lambda: ext.deltanet(S, conved, z, beta, g, w, o, heads, heads, d, T, 1, 0, ext.BF16)
        work, unit = 7.0 * d * d * heads * T, "flop"
    elif name in ("mla_2048", "mla_65536"):
        # latent attention at decode through the extension entry: 64 heads over 2,048 / 65,536 latents of 512, 8 / 4 latents cycled
        Lm, copies = (2048, 8) if name == "mla_2048" else (65536, 4)
        lat = torch.randn((copies, Lm, 512), generator=gen, device="cuda", dtype=torch.float16)
        qm = torch.randn((64, 512), generator=gen, device="cuda", dtype=torch.float16) * 2.0
        om = torch.zeros((64, 512), device="cuda", dtype=torch.float16)
        lstate = {"i": 0}

        def fn():
            i = lstate["i"] = (lstate["i"] + 1) % copies
            ext.mla_decode(om, None, qm, lat[i], 64, Lm, ext.FP16, int(os.environ.get("MLA_BLOCKS", "0")))
        work, unit = Lm * 512 * 2 + 2 * 64 * 512 * 2, "bytes"
        if os.environ.get("MLA_GRAPH"):
            fn = mla_graph(torch, ext, lat, qm, om, Lm)
            work *= copies
    elif name == "exchange_small":
        # the exchange's fold alone on one card: 8 heads of 128 (configuration 4's share at 8 GPUs), the partner's push deposited
        x = ext.Exchange(2, 0, 8 * 130 * 4)
        x.connect_alone()
        mine = torch.randn((8, 130), generator=gen, device="cuda", dtype=torch.float32).abs() + 0.5
        theirs = torch.randn((8, 130), generator=gen, device="cuda", dtype=torch.float32).abs() + 0.5
        om = torch.zeros((8, 128), device="cuda", dtype=torch.bfloat16)

        def fn():
            x.deposit(1, theirs, 8 * 130 * 4)
            x.merge_finish(om, None, mine, 8, 128, ext.BF16, wait_ms=200)
        work, unit = 2 * 8 * 130 * 4, "bytes"
    elif name in ("expert_q4", "expert_o8", "expert_q4_64rows"):
        # a prompt chunk's projection through the expert_rows door: 256 (or 64) rows through 8,192 x 5,120 at 4 bits / 5,120 x 4,096 at 8
        er, ec, width = (5120, 4096, 8) if name == "expert_o8" else (8192, 5120, 4)
        ec = int(os.environ.get("EXPERT_COLS", ec))
        T, copies = (64 if name.endswith("64rows") else 256), 4
        ecodes = torch.randint(0, 256, (copies, er, ec * width // 8), generator=gen, device="cuda", dtype=torch.uint8)
        escales = ((torch.rand((er,), generator=gen, device="cuda") * 0.5 + 0.75) * (3.0 / ec ** 0.5)).to(torch.float16)
        ex = torch.randn((T, ec), generator=gen, device="cuda", dtype=torch.float16)
        epairs = torch.arange(T, device="cuda", dtype=torch.int32).repeat_interleave(2).contiguous()
        eout = torch.zeros((T, er), device="cuda", dtype=torch.float16)
        estate = {"i": 0}

        def fn():
            i = estate["i"] = (estate["i"] + 1) % copies
            fam.nn.expert_rows(eout.data_ptr(), ecodes[i].data_ptr(), ecodes[i].numel(), escales.data_ptr(), escales.numel() * 2, ex.data_ptr(), epairs.data_ptr(),
                               T, width, er, ec, None)
        work, unit = 2.0 * T * er * ec, "flop"
    elif name in ("range_share_fused", "range_share_apart"):
        # a rank's share of configuration 4 at 8 GPUs (131,072 positions of one kv head, 8 query heads) with its exchange step, the
        # partner's push deposited: the exchange in the decode kernel's last block, or as a launch of its own after the decode
        qh, kvh, d, Ls = 8, 1, 128, 131072
        k = torch.randn((Ls, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.5
        v = torch.randn((Ls, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.5
        q = torch.randn((qh, d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.5
        theirs = torch.randn((qh, d + 2), generator=gen, device="cuda", dtype=torch.float32).abs() + 0.5
        x = ext.Exchange(2, 0, qh * (d + 2) * 4)
        x.connect_alone()
        tier = ext.Tier(qh, kvh, d, ext.BF16)
        om = torch.zeros((qh, d), device="cuda", dtype=torch.bfloat16)
        mine = torch.zeros((qh, d + 2), device="cuda", dtype=torch.float32)

        def fn():
            x.deposit(1, theirs, qh * (d + 2) * 4)
            if name == "range_share_fused":
                tier.decode_exchange(x, om, None, q, None, None, 0, k, v, Ls, wait_ms=200)
            else:
                tier.decode(None, mine, q, None, None, 0, k, v, Ls)
                x.merge_finish(om, None, mine, qh, d, ext.BF16, wait_ms=200)
        work, unit = 2 * Ls * kvh * d * 2, "bytes"
    elif name == "prefill_small":
        qh, kvh, d, T = 16, 2, 256, 2048
        q = torch.randn((T, qh, d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.5
        k = torch.randn((T, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.5
        v = torch.randn((T, kvh, d), generator=gen, device="cuda", dtype=torch.bfloat16) * 0.5
        o = torch.zeros_like(q)
        fn = lambda: ext.prefill(o, q, k, v, qh, kvh, d, 0, T, ext.BF16)
        work, unit = 4.0 * qh * d * T * (T + 1) / 2, "flop"
    else:
        raise SystemExit(f"unknown case {name}")
    ms = time_loop(torch, fn, steps, 1)
    print(json.dumps({"case": name, "steps": steps, "ms_per_launch": ms, "work_per_launch": work, "work_unit": unit,
                      "rate": work / ms / 1e6, "rate_unit": "GB/s" if unit == "bytes" else "GFLOP/s", "device_status": ext.device_status()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-others", action="store_true", help="skip the secondary configurations (faster; used under profilers)")
    ap.add_argument("--only", default=None, choices=["long_context"], help="run configuration 4 alone (any N) and print its object")
    ap.add_argument("--case", default=None, help="run one small single-kernel case instead (paged_small, long_small, decode_cfg1, decode_cfg1_graph, tq8_small, tq4_small, deltanet_64, deltanet_prefill, prefill_small, mla_2048, mla_65536, exchange_small, expert_q4, expert_o8, expert_q4_64rows, range_share_fused, range_share_apart)")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
