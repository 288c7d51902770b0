#!/usr/bin/env python
"""Decode-step benchmark of the sparse entmax path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one pass of the hot path over one batch of seeded synthetic input:
append the new token, select pages (top-k or Gaussian-aware), paged entmax decode.
Prints ONE JSON line (rank 0).  ``value`` is the device-timed step latency with all
inputs resident in HBM; ``e2e`` is the same step through the public Python API with
q / k_new / v_new coming from pinned host memory and the output read back (the step
replayed as a captured graph); ``e2e_eager`` is the same through the two drop-in
functions called directly.

Headline (every N): one replica of the workload per GPU - the path partitions by batch
row and KV head, there is no data-path collective - i.e. weak scaling.  Beside it, in
``other_workloads``: the other single-GPU configurations (N = 1), the million-token
request (unsharded at N = 1, sequence-sharded over the N GPUs otherwise, with its
speed-up over one GPU measured in the same run) and, for N > 1, the 128k batch split by
batch row over the N GPUs (strong scaling, B = 32 in total).

``--impl reference`` times the reference's CPU path on the host cores: its own CPU code
(cache object, key-range page scores, top-k, Gaussian statistics, tau solver, tau
clamp; imported from ``baseline/_ref``) plus a CPU restatement (``oracle/``) of the two
pieces it only has as Triton kernels (threshold select + pack, paged decode).
"""

from __future__ import annotations

import argparse
import ctypes
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode_step_latency"
UNIT = "us"
HBM_NOMINAL_GBS = 8000.0
L2_NOTE = "flushed between timed steps (512 MiB write + 512 MiB read)"
DTYPE_NAME = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}


# --------------------------------------------------------------------------- helpers

def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons (query mode only) while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "samples": len(sm),
                "reasons": sorted(reasons)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


class Ranks:
    """The process group as the benchmark uses it: a barrier and a maximum / sum over ranks."""

    def __init__(self):
        self.rank, self.local_rank, self.world = dist_env()
        torch.cuda.set_device(self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max(self, x: float) -> float:
        if self.world == 1:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum(self, x: float) -> float:
        if self.world == 1:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        self.dist.all_reduce(t)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def static_config(w, parallelism: str, batch_per_gpu=None) -> dict:
    """The part of ``config`` that depends on the workload only (both arms print the same)."""
    return {"workload": w.name, "mode": w.mode, "batch_per_gpu": w.batch if batch_per_gpu is None else batch_per_gpu,
            "q_heads": w.q_heads, "kv_heads": w.kv_heads, "head_dim": w.head_dim, "context": w.context,
            "page_size": w.page_size, "token_budget": w.token_budget if w.mode == "topk" else None,
            "alpha": w.alpha, "seed": w.seed, "needle_fraction": w.needle_fraction, "l2": L2_NOTE,
            "parallelism": parallelism, "launch": "whole step replayed as one CUDA graph"}


class L2Flush:
    """Write 512 MiB, then read another 512 MiB: the read pushes the written (dirty) lines out to
    HBM, so the timed step starts with a cold L2 and no write-back in flight."""

    def __init__(self):
        self.w = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
        self.r = torch.zeros(512 << 18, dtype=torch.int32, device="cuda")

    def __call__(self):
        self.w.fill_(1)
        self.r.max()


# --------------------------------------------------------------------------- GPU arm: one cache, steps on it

class StepRunner:
    """Owns one cache (a whole workload, or rows [rows.start, rows.stop) of it) on the current
    device and runs decode steps on it."""

    def __init__(self, w, headroom: int, seed_shift: int = 0, rows=None, sigma_mean=None):
        import entmaxkv_b200 as E
        from entmaxkv_b200 import workloads
        self.E = E
        if seed_shift:
            w = dataclasses.replace(w, seed=w.seed + seed_shift)
        self.w = w
        inp = workloads.make_inputs(w, device="cuda", batch_slice=rows)
        self.rows = rows
        self.cache = E.PagedKVCache(page_size=w.page_size)
        self.cache.initialize(inp["k"], inp["v"], seq_lens=inp["seq_lens"], capacity=w.context + headroom)
        del inp["k"], inp["v"]          # K/V now live in the cache; drop the staging copies
        torch.cuda.empty_cache()
        self.q, self.k_new, self.v_new = inp["q"], inp["k_new"], inp["v_new"]
        # a decode loop appends a different token every step: a pool of seeded tokens, iid normal like the
        # rest of the cache, taken in turn (the same key appended a hundred times piles identical
        # scores onto every head and distorts the supports after ~75 steps)
        self.k_pool, self.v_pool = workloads.token_pool(w, 16, "cuda", batch_slice=rows)
        self.k_pool[0].copy_(self.k_new)
        self.v_pool[0].copy_(self.v_new)
        self.steps_done = 0
        self.out = torch.zeros_like(self.q)
        self.flush_l2 = L2Flush()
        self.sigma_mean = sigma_mean
        self.graph = None
        self.switch_workload(w)

    def switch_workload(self, w2):
        """(Re-)use the resident cache and inputs for a selection mode of the same shapes."""
        from entmaxkv_b200.graph import DecodeStepGraph
        self.w = w2
        if w2.mode == "topk":
            self.graph = DecodeStepGraph(self.cache, w2.q_heads, "topk", token_budget=w2.token_budget,
                                         alpha=w2.alpha, niter=2)
        else:
            extra = {} if self.sigma_mean is None else {"sigma_mean": self.sigma_mean}
            self.graph = DecodeStepGraph(self.cache, w2.q_heads, "gaussian", alpha=w2.alpha,
                                         tau_mode=w2.tau_mode, **extra)

    def next_token(self):
        """K/V rows of the token the next step appends (device tensors from the pool, in turn)."""
        i = self.steps_done % self.k_pool.shape[0]
        self.steps_done += 1
        return self.k_pool[i], self.v_pool[i]

    def step(self, q=None, k_new=None, v_new=None):
        """One decode step replayed as a CUDA graph (inputs are copied into its buffers)."""
        if k_new is None or v_new is None:
            k_new, v_new = self.next_token()
        return self.graph.step(self.q if q is None else q, k_new, v_new)

    def eager_step(self, q=None, k_new=None, v_new=None, out=None):
        """The same step through the drop-in functions, launched kernel by kernel."""
        w, E = self.w, self.E
        q = self.q if q is None else q
        if k_new is None or v_new is None:
            k_new, v_new = self.next_token()
        out = self.out if out is None else out
        if w.mode == "topk":
            E.sparse_attention_decode_paged(q, self.cache, k_new, v_new, out, w.token_budget,
                                            alpha=w.alpha, niter=2, append_cache=True)
        else:
            extra = {} if self.sigma_mean is None else {"sigma_mean": self.sigma_mean}
            E.sparse_attention_decode_gaussian_aware_entmax(q, self.cache, k_new, v_new, out, alpha=w.alpha,
                                                            append_cache=True, tau_mode=w.tau_mode, **extra)
        return out

    def timed_steps(self, K, W, ranks=None):
        """W warm-up + K timed graph replays with a cold L2; returns (ms per step: sum over this rank's
        steps / K, maximum over ranks; this rank's per-step statistics)."""
        for _ in range(W):
            self.flush_l2()
            self.step()
        if ranks is not None:
            ranks.barrier()
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
        for i in range(K):
            self.flush_l2()
            starts[i].record()
            self.step()
            stops[i].record()
        if ranks is not None:
            ranks.barrier()
        torch.cuda.synchronize()
        times = [a.elapsed_time(b) for a, b in zip(starts, stops)]
        ordered = sorted(times)
        stats = {"min": ordered[0] * 1e3, "median": ordered[len(ordered) // 2] * 1e3, "max": ordered[-1] * 1e3,
                 "first": times[0] * 1e3, "last": times[-1] * 1e3}
        ms = sum(times) / K
        return (ms if ranks is None else ranks.max(ms)), stats

    def timed_e2e(self, K, ranks=None, eager=False):
        """The step with q / k_new / v_new coming from pinned host memory and the output copied back,
        wall clock including the synchronisation; microseconds per step (maximum over ranks)."""
        hq = self.q.cpu().pin_memory()
        hk_pool, hv_pool = self.k_pool.cpu().pin_memory(), self.v_pool.cpu().pin_memory()
        hout = torch.empty_like(hq).pin_memory()
        dq, dk, dv = torch.empty_like(self.q), torch.empty_like(self.k_new), torch.empty_like(self.v_new)
        counter = [0]

        io = None if eager else self.graph.pinned_io()

        def prepare():
            """Untimed: this step's inputs are put where a caller would have them - in page-locked host memory."""
            i = counter[0] % hk_pool.shape[0]
            counter[0] += 1
            if io is not None:      # the captured step reads its own pinned staging buffers
                io["q"].copy_(hq)
                io["k_new"].copy_(hk_pool[i])
                io["v_new"].copy_(hv_pool[i])
            return i

        def one(i):
            if eager:
                dq.copy_(hq, non_blocking=True)              # H2D copies of the three inputs
                dk.copy_(hk_pool[i], non_blocking=True)
                dv.copy_(hv_pool[i], non_blocking=True)
                dout = self.eager_step(dq, dk, dv)
                hout.copy_(dout, non_blocking=True)          # D2H of the result
            else:
                self.graph.step_pinned()     # one launch: one H2D copy node (q | k_new | v_new), the step; its last kernel stores the result rows to host memory
            torch.cuda.current_stream().synchronize()

        for _ in range(3):
            one(prepare())
        if ranks is not None:
            ranks.barrier()
        tt = 0.0
        for _ in range(K):
            i = prepare()
            self.flush_l2()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            one(i)
            tt += time.perf_counter() - t0
        if ranks is not None:
            ranks.barrier()
        us = tt / K * 1e6
        us = us if ranks is None else ranks.max(us)
        esz = self.q.element_size()
        return {"value": us, "unit": UNIT,
                "h2d_bytes_per_step": (hq.numel() + hk_pool[0].numel() + hv_pool[0].numel()) * esz,
                "d2h_bytes_per_step": hout.numel() * esz}

    # ---- what the last step selected / moved

    def _sel(self):
        return self.cache.last_topk_selection if self.w.mode == "topk" else self.cache.last_gaussian_selection

    def selected_tokens(self) -> int:
        return int(self._sel()["tok_counts"].sum().item())

    def union_tokens(self) -> int:
        """Tokens selected by at least one query head of each GQA group, summed over (batch row, KV
        head): the K/V rows a step has to fetch when heads of a group share what they both picked."""
        sel = self._sel()
        pages, counts = sel["page_indices"], sel["num_selected"]
        B, Hq, width = pages.shape
        G = self.w.q_heads // self.w.kv_heads
        P = self.w.page_size
        big = torch.iinfo(torch.int32).max
        total = 0
        lens = torch.tensor(self.cache.host_seq_lens, device=pages.device)
        last_tokens = lens - (torch.div(lens + P - 1, P, rounding_mode="floor") - 1) * P
        for b in range(B):       # row by row bounds the sort's scratch
            valid = torch.arange(width, device=pages.device)[None, :] < counts[b][:, None]
            ids = torch.where(valid, pages[b], torch.full_like(pages[b], big)).reshape(Hq // G, G * width)
            ids = ids.sort(dim=-1).values
            new = torch.ones_like(ids, dtype=torch.bool)
            new[..., 1:] = ids[..., 1:] != ids[..., :-1]
            n_pages = (new & (ids != big)).sum(dim=-1)          # [H_kv] distinct pages incl. the last one
            total += int(((n_pages - 1).clamp(min=0) * P + last_tokens[b]).sum().item())
        return total

    def support_tokens(self):
        """Tokens whose weight was non-zero in the last step (the value rows it really needed), or None."""
        from entmaxkv_b200 import _lib
        c = self.cache
        sel = self._sel()
        if self.w.mode == "topk" and sel.get("support") is not None:      # the many-head kernel counts them itself
            return int(sel["support"].sum().item())
        ws = next((v for k, v in c._scratch.items() if k[0] == "decode_ws"), None)
        if ws is None:
            return None
        B, Hq, _, D = self.q.shape
        max_tokens = c.capacity if self.w.mode != "topk" else \
            (min(self.w.token_budget // c.page_size, max(c.page_capacity - 1, 0)) + 1) * c.page_size
        counts = torch.empty(B * Hq, dtype=torch.int32, device="cuda")
        rc = _lib.load().ekv_decode_support_counts(ws.data_ptr(), ws.numel(), B, Hq, D, max_tokens,
                                                   counts.data_ptr(), _lib.stream_ptr())
        if rc != 0 or bool((counts < 0).any()):
            return None
        return int(counts.sum().item())

    # ---- stage-by-stage timing (same launches as step(), one event pair per stage)
    def staged_step(self, ev):
        from entmaxkv_b200 import _lib, attention_topk as AT, attention_gaussian as AG
        C = ctypes
        w, c, q = self.w, self.cache, self.q
        lib = _lib.load()
        B, Hq, _, D = q.shape
        P = c.page_size
        stream = torch.cuda.current_stream()
        marks = []

        def mark(name):
            e = ev()
            e.record(stream)
            marks.append((name, e))

        mark("start")
        c.append(*self.next_token())
        mark("append")
        desc = C.byref(c.desc())
        st = _lib.stream_ptr()
        if w.mode == "topk" and AT._fused_small_step(q, c, self.out, w.token_budget, w.alpha, 2, None):
            mark("fused_topk_small_kernel")      # a small problem: the rest of the step is this one launch
            return marks
        if w.mode == "topk" and AT._stream_step(q, c, self.out, w.token_budget, w.alpha, 2, None, on_launch=mark):
            mark("topk_decode_stream_kernel")    # many heads: selection, K pass, tau, values and output in one launch
            return marks
        if w.mode == "topk":
            S = c.capacity
            k_max = min(w.token_budget // P, max(c.page_capacity - 1, 0))
            stride = max(c.page_capacity, 1)     # same shape as attention_topk._score_and_select: same buffer
            scores = c.scratch("topk_scores", (B, Hq, stride), q.dtype)
            pages = c.scratch("topk_pages", (B, Hq, k_max + 1), torch.int32)
            nsel = c.scratch("topk_counts", (B, Hq), torch.int32)
            ntok = c.scratch("topk_tokens", (B, Hq), torch.int32)
            n_items = B * Hq * lib.ekv_work_items_per_head((k_max + 1) * P)
            items = c.scratch("topk_work", (n_items,), torch.int64)
            _lib.check(lib.ekv_page_scores(desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, S,
                                           scores.data_ptr(), stride, st), "ekv_page_scores")
            mark("page_score_kernel")
            _lib.check(lib.ekv_topk_pack(desc, Hq, w.token_budget, S, scores.data_ptr(), stride,
                                         pages.data_ptr(), k_max + 1, nsel.data_ptr(), ntok.data_ptr(),
                                         None, 0, 0, items.data_ptr(), st), "ekv_topk_pack")
            mark("topk_select_kernel")
            tau = c.scratch("tau", (B, Hq), torch.float32)
            max_tokens, mode, iters = (k_max + 1) * P, _lib.TAU_EXACT, 2
            wl_tensor, wt_tensor = items, None
        else:
            S, pcap = c.capacity, c.page_capacity
            mu = c.scratch("g_mu", (B, Hq, pcap), torch.float32)
            sigma = c.scratch("g_sigma", (B, Hq, pcap), torch.float32)
            hsum = c.scratch("g_head_sums", (B, Hq, 4), torch.float32)
            hstat = c.scratch("g_head_stats", (B, Hq, 4), torch.float32)
            wsb = lib.ekv_gaussian_workspace_bytes(B, Hq, pcap)
            gws = c.scratch("g_ws", (wsb,), torch.uint8, zero=True)
            _lib.check(lib.ekv_gaussian_moments(desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, S, 1,
                                                float(w.alpha), 1, mu.data_ptr(), sigma.data_ptr(), pcap,
                                                hsum.data_ptr(), hstat.data_ptr(), gws.data_ptr(), wsb, st),
                       "ekv_gaussian_moments")
            mark("gaussian_moments_kernel")
            pages = c.scratch("g_pages", (B, Hq, pcap), torch.int32)
            nsel = c.scratch("g_counts", (B, Hq), torch.int32)
            ntok = c.scratch("g_tokens", (B, Hq), torch.int32)
            tfl = c.scratch("g_tau_floor", (B, Hq), torch.float32)
            cap = c.scratch("g_cap", (B, Hq), torch.float32)
            tau = c.scratch("g_tau", (B, Hq), torch.float32)
            nch = (c.capacity + 255) // 256
            wl_tensor = c.scratch("g_work", (B * Hq * nch,), torch.int64)
            wt_tensor = c.scratch("g_work_total", (2 + (B * Hq + 1023) // 1024,), torch.int32, zero=True)
            grouped = AG.grouped_enabled(q, c)     # the wrapper then builds no per-head work list
            _lib.check(lib.ekv_gaussian_select(
                desc, Hq, S, 1, 1, float(w.alpha), 0.2, AG._z_of_quantile(0.99, P), AG._z_of_quantile(0.995, P),
                AG._z_of_quantile(0.5, P), 1, None, mu.data_ptr(), sigma.data_ptr(), pcap, hstat.data_ptr(),
                pages.data_ptr(), pcap, nsel.data_ptr(), ntok.data_ptr(), tfl.data_ptr(), cap.data_ptr(),
                tau.data_ptr(), None if grouped else wl_tensor.data_ptr(),
                None if grouped else wt_tensor.data_ptr(), st), "ekv_gaussian_select")
            mark("gaussian_select_kernel")
            max_tokens, mode = c.capacity, _lib.TAU_CORRECTED
            iters = {"fixed": 0, "corrected": 1}.get(w.tau_mode, 1)
        evs = [ev() for _ in range(3)]
        if w.mode != "topk" and AG.grouped_enabled(q, c):
            AG.grouped_decode(q, c, self.out, dict(page_indices=pages, num_selected=nsel, tau=tau), w.alpha,
                              mode, iters, stage_events=evs, on_launch=mark)
            marks.append(("decode_scores_group_kernel", evs[0]))
        else:
            AT._paged_decode(q, c, self.out, pages, ntok, max_tokens, w.alpha, mode, iters, tau, wl_tensor,
                             work_total=wt_tensor, stage_events=evs)
            marks.append(("decode_scores_kernel", evs[0]))
        marks.append(("tau_solve_kernel", evs[1]))
        marks.append(("decode_values_kernel", evs[2]))
        mark("out_reduce_kernel")
        return marks

    def stage_times_ms(self, reps):
        acc = {}
        for _ in range(reps):
            self.flush_l2()
            marks = self.staged_step(lambda: torch.cuda.Event(enable_timing=True))
            torch.cuda.synchronize()
            for (_, e0), (name, e1) in zip(marks[:-1], marks[1:]):
                acc.setdefault(name, []).append(e0.elapsed_time(e1))
        # median over the repetitions: one pass that happens to (re)allocate a scratch buffer inside a
        # stage must not colour the per-kernel figure
        return {k: statistics.median(v) for k, v in acc.items()}


def byte_counts(runner, ms_per_step, peak):
    """Algorithmic and actually-moved bytes of the runner's last step, with the step-level rates."""
    from entmaxkv_b200 import workloads
    w = runner.w
    lens = [n - 1 for n in runner.cache.host_seq_lens]
    sel = runner.selected_tokens()
    uni = runner.union_tokens()
    sup = runner.support_tokens()
    by = workloads.algorithmic_bytes(w, lens, sel)
    bu = workloads.algorithmic_bytes(w, lens, uni)
    e = torch.empty((), dtype=w.dtype).element_size()
    sec = ms_per_step * 1e-3
    out = {"selected_tokens_per_step": sel, "union_tokens_per_step": uni, "support_tokens_per_step": sup,
           "algorithmic_bytes_per_step": by["total"], "metadata_bytes": by["metadata"], "kv_bytes": by["kv"],
           "union_bytes_per_step": bu["total"],
           "step_achieved_gbs": by["total"] / sec / 1e9,
           "step_frac_of_measured": by["total"] / sec / 1e9 / peak,
           "step_frac_of_8tbs": by["total"] / sec / 1e9 / HBM_NOMINAL_GBS,
           "union_step_achieved_gbs": bu["total"] / sec / 1e9,
           "union_step_frac_of_8tbs": bu["total"] / sec / 1e9 / HBM_NOMINAL_GBS}
    if sup is not None:
        # bytes the step has to move however it is organised: the statistics sweep, the K rows of every
        # page some head of the group selected (once per group), and the value rows with non-zero weight
        moved = by["metadata"] + bu["kv"] // 2 + sup * w.head_dim * e
        out.update({"moved_bytes_per_step": moved, "moved_achieved_gbs": moved / sec / 1e9,
                    "moved_frac_of_measured": moved / sec / 1e9 / peak,
                    "moved_frac_of_8tbs": moved / sec / 1e9 / HBM_NOMINAL_GBS})
    return out, by, bu


def load_traffic():
    """DRAM traffic per algorithmic byte of the streaming kernels, from the ncu captures summarised
    under profiles/ (captured on a batch slice; traffic grows in proportion to the pages / rows a
    launch processes), stamped with the commit the capture was taken at."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            return json.load(f)
    except Exception:
        return {}


# --------------------------------------------------------------------------- GPU arm: the sharded request

def run_million(ranks: Ranks, K: int, W: int, collective: str = "peer", stages: bool = True):
    """The million-token request on the N GPUs of the process group: unsharded on one GPU when N = 1,
    otherwise pages split contiguously over the ranks (strong scaling) with the four reductions of a
    step fused into their consumer kernels over NVLink peer memory (``collective='nccl'``: NCCL
    all-reduces instead).  For N > 1 rank 0 also times the unsharded step, so the record carries the
    speed-up over one GPU measured in the same run.  Returns the record (rank 0) or None."""
    from entmaxkv_b200 import sharded, workloads
    w = workloads.CONFIGS["million_gaussian"]
    rank, world = ranks.rank, ranks.world
    peak, _ = measured_peak_gbs()
    one_gpu = None
    if rank == 0:
        r1 = StepRunner(w, 4 * 4 * (K + W) + 1024)
        ms, stats = r1.timed_steps(K, W)
        e2e = r1.timed_e2e(min(K, 50))
        e2e_eager = r1.timed_e2e(min(K, 50), eager=True)
        bc, _, _ = byte_counts(r1, ms, peak)
        stage = r1.stage_times_ms(5)
        one_gpu = {"value": ms * 1e3, "step_us": stats, "e2e": e2e, "e2e_eager": e2e_eager,
                   "kernels_us": {k: v * 1e3 for k, v in stage.items()}, **bc}
        r1.graph = None
        del r1
        torch.cuda.empty_cache()
    if world == 1:
        return {"workload": w.name, "n_gpus": 1, "scaling": "strong", "value": one_gpu["value"], "unit": UNIT,
                "e2e": one_gpu["e2e"], "e2e_eager": one_gpu["e2e_eager"], "speedup_vs_1gpu": 1.0,
                "config": static_config(w, "unsharded"), "stage_us": one_gpu["kernels_us"],
                "selected_tokens": one_gpu["selected_tokens_per_step"], "step_us": one_gpu["step_us"],
                "achieved_gbs": one_gpu["step_achieved_gbs"], "frac_of_measured": one_gpu["step_frac_of_measured"],
                "frac_of_8tbs": one_gpu["step_frac_of_8tbs"], "union_frac_of_8tbs": one_gpu["union_step_frac_of_8tbs"],
                "moved_frac_of_measured": one_gpu.get("moved_frac_of_measured"),
                "moved_bytes_per_step": one_gpu.get("moved_bytes_per_step"),
                "algorithmic_bytes_per_step": one_gpu["algorithmic_bytes_per_step"]}
    ranks.barrier()
    dist = ranks.dist
    P, S = w.page_size, w.context
    lo, hi = sharded.split_pages(S, P, world)[rank]
    inp = workloads.make_inputs(w, device="cuda", token_slice=slice(lo, hi))   # this rank's pages only
    shard = sharded.GpuSequenceShard(P, rank, world)
    shard.initialize(inp["k"], inp["v"], capacity=(hi - lo) + 4 * 4 * (K + W) + 1024)
    del inp["k"], inp["v"]
    torch.cuda.empty_cache()
    q, kn, vn = inp["q"], inp["k_new"], inp["v_new"]
    shard.set_global_lengths([S] * w.batch)
    reduce = sharded.dist_reduce()
    exchange = None
    if collective == "peer":
        from entmaxkv_b200.exchange import PeerExchange
        exchange = PeerExchange(rank, world, max_floats=max(1 << 14, w.batch * w.q_heads * w.head_dim))
    graph = sharded.ShardedStepGraph(shard, reduce, w.q_heads, alpha=w.alpha, tau_mode=w.tau_mode, exchange=exchange)
    flush = L2Flush()
    for _ in range(W):
        flush()
        graph.step(q, kn, vn)
    ranks.barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    align = torch.zeros(4, dtype=torch.float32, device="cuda")
    for i in range(K):
        flush()
        dist.barrier()
        if exchange is not None:
            # device-side barrier queued in front of the start event: the hosts leave dist.barrier()
            # tens of microseconds apart, and without it the first exchange of the step would count
            # that launch skew as step time
            exchange.all_reduce(align, "sum", slot=1)
        starts[i].record()
        graph.step(q, kn, vn)
        stops[i].record()
    ranks.barrier()
    if exchange is not None:
        exchange.check()         # a timed-out wait would make the numbers meaningless: fail loudly
    ms = ranks.max(sum(a.elapsed_time(b) for a, b in zip(starts, stops)) / K)
    # end to end: inputs from pinned host memory every step, the result read back to the host
    hq, hk, hv = q.cpu().pin_memory(), kn.cpu().pin_memory(), vn.cpu().pin_memory()
    hout = torch.empty((w.batch, w.q_heads, 1, w.head_dim), dtype=torch.float32).pin_memory()

    io = graph.pinned_io()                      # the inputs sit in page-locked host memory before a step is timed
    io["q"].copy_(hq)
    io["k_new"].copy_(hk)
    io["v_new"].copy_(hv)

    def e2e_step():
        graph.step_pinned()     # one launch: one H2D copy node (q | k_new | v_new), the step, the D2H copy node of the result
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    tt, K2 = 0.0, min(K, 50)
    for _ in range(K2):
        flush()
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e2e_step()
        tt += time.perf_counter() - t0
    e2e = {"value": ranks.max(tt / K2 * 1e6), "unit": UNIT,
           "h2d_bytes_per_step": (hq.numel() + hk.numel() + hv.numel()) * hq.element_size(),
           "d2h_bytes_per_step": hout.numel() * 4}
    if exchange is not None:
        exchange.check()
    stage_us = None
    if exchange is not None and stages:
        # the same launches issued eagerly with an event after each stage; maximum over ranks per stage
        names = ["append", "moments_x", "select_x", "decode_x"]
        calls = [lambda: shard.append(kn, vn), lambda: shard.moments_x(q, w.alpha, exchange),
                 lambda: shard.select_x(exchange), lambda: shard.decode_x(exchange, 1)]
        reps, acc = 10, [0.0] * len(names)
        for _ in range(reps):
            flush()
            dist.barrier()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
            ev[0].record()
            for i, fn in enumerate(calls):
                fn()
                ev[i + 1].record()
            torch.cuda.synchronize()
            for i in range(len(names)):
                acc[i] += ev[i].elapsed_time(ev[i + 1]) * 1e3 / reps
        mine = torch.tensor(acc, device="cuda", dtype=torch.float64)
        dist.all_reduce(mine, op=dist.ReduceOp.MAX)
        stage_us = {n: round(float(v), 1) for n, v in zip(names, mine.tolist())}
        exchange.check()
    sel = ranks.sum(float(shard.tokens.sum().item()))
    from entmaxkv_b200.attention_gaussian import grouped_enabled
    grouped = grouped_enabled(q, shard.cache)
    # a CUDA graph that holds captured collectives must be gone before the communicator is torn down
    graph.release()
    del graph
    torch.cuda.synchronize()
    dist.barrier()
    if exchange is not None:
        exchange.close()
        dist.barrier()
    del shard
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    by = workloads.algorithmic_bytes(w, [S], int(sel))
    gbs = by["total"] / (ms * 1e-3) / 1e9
    # fused exchange: input staging, append, moments, select, (group union,) K pass, tau, V pass, output fold
    n_launch = (8 + int(grouped)) if exchange is not None else 12
    return {"workload": w.name, "n_gpus": world, "scaling": "strong", "value": ms * 1e3, "unit": UNIT, "e2e": e2e,
            "speedup_vs_1gpu": one_gpu["value"] / (ms * 1e3), "one_gpu_value": one_gpu["value"],
            "one_gpu_e2e": one_gpu["e2e"]["value"], "one_gpu_stage_us": one_gpu["kernels_us"],
            "config": static_config(w, f"sequence pages x{world}, " +
                                    ("4 reductions fused into their consumer kernels over NVLink peer memory"
                                     if exchange is not None else "4 NCCL all-reduces per step")),
            "start_alignment": "device-side peer barrier before each start event" if exchange is not None else "host barrier",
            "stage_us": stage_us, "selected_tokens": int(sel), "gpu_launches_per_step": n_launch,
            "achieved_gbs": gbs, "frac_of_measured_xN": gbs / (peak * world),
            "algorithmic_bytes_per_step": by["total"], "status_checked": True}


# --------------------------------------------------------------------------- GPU arm: B = 32 in total over N GPUs

def run_strong_batch(ranks: Ranks, base_w, K: int, W: int, one_gpu_us=None, collective: str = "peer"):
    """The 128k GQA batch as the configuration states it - B = 32 IN TOTAL, split by batch row over
    the N GPUs (32/N rows each; each GPU holds its rows' cache and statistics) - for top-k and for
    Gaussian-aware selection.  The top-k step needs no exchange; the Gaussian-aware step needs the
    batch-wide mean of sigma_global: one scalar all-reduce per step, captured in the step's graph - through
    NVLink peer memory (``ekv_exchange_allreduce``: every rank stores its float into the others' inboxes and
    sums what it finds in its own) or, with ``collective='nccl'``, one NCCL all-reduce.
    Step time = maximum over ranks.  Returns records (rank 0) or []."""
    from entmaxkv_b200 import workloads
    rank, world = ranks.rank, ranks.world
    if base_w.batch % world:
        return []
    per = base_w.batch // world
    rows = slice(rank * per, (rank + 1) * per)
    total_heads = base_w.batch * base_w.q_heads
    dist = ranks.dist

    exchange = None
    if collective == "peer" and world > 1:
        from entmaxkv_b200.exchange import PeerExchange
        try:
            exchange = PeerExchange(rank, world, max_floats=1 << 10)
            ok = 1.0
        except Exception:       # no peer access between these devices: every rank falls back to NCCL together
            exchange, ok = None, 0.0
        if -ranks.max(-ok) < 1.0:
            if exchange is not None:
                exchange.close()
            exchange = None

    def sigma_mean(local_sum, _local_heads):
        if exchange is not None:
            return exchange.all_reduce(local_sum) / total_heads
        dist.all_reduce(local_sum)
        return local_sum / total_heads

    runner = StepRunner(base_w, 4 * 4 * (K + W) + 1024, rows=rows, sigma_mean=sigma_mean)
    out = []
    peak, _ = measured_peak_gbs()
    for w2 in (base_w, dataclasses.replace(workloads.CONFIGS["gqa_128k_gaussian"], seed=base_w.seed)):
        runner.switch_workload(w2)
        ms, stats = runner.timed_steps(K, W, ranks)
        e2e = runner.timed_e2e(min(K, 20), ranks)
        sel = ranks.sum(float(runner.selected_tokens()))
        if rank == 0:
            by = workloads.algorithmic_bytes(dataclasses.replace(w2, batch=base_w.batch),
                                             [base_w.context] * base_w.batch, int(sel))
            gbs = by["total"] / (ms * 1e-3) / 1e9
            rec = {"workload": w2.name + "_strong", "n_gpus": world, "scaling": "strong", "value": ms * 1e3,
                   "unit": UNIT, "e2e": e2e, "step_us_rank0": stats,
                   "config": static_config(w2, f"batch rows x{world} (B = {base_w.batch} in total, {per} rows per GPU)" +
                                           (("; one scalar all-reduce per step (mean of sigma_global) through " +
                                             ("NVLink peer memory" if exchange is not None else "NCCL"))
                                            if w2.mode == "gaussian" else "; no exchange"), batch_per_gpu=per),
                   "selected_tokens": int(sel), "algorithmic_bytes_per_step": by["total"],
                   "achieved_gbs": gbs, "frac_of_measured_xN": gbs / (peak * world)}
            if one_gpu_us and w2.name in one_gpu_us:
                rec["one_gpu_value"] = one_gpu_us[w2.name]
                rec["speedup_vs_1gpu"] = one_gpu_us[w2.name] / (ms * 1e3)
            out.append(rec)
    runner.graph = None
    del runner
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    ranks.barrier()
    if exchange is not None:
        exchange.check()
        exchange.close()
    return out


# --------------------------------------------------------------------------- GPU arm: the line

def run_gpu(args):
    from entmaxkv_b200 import workloads
    ranks = Ranks()
    rank, world = ranks.rank, ranks.world
    w = workloads.CONFIGS[args.workload]
    if args.batch:
        w = dataclasses.replace(w, batch=args.batch)   # a slice of the workload (profiling captures)
    if args.alpha:
        w = dataclasses.replace(w, alpha=args.alpha, name=f"{w.name}_alpha{args.alpha:g}")
    if args.token_budget and w.mode == "topk":
        # a budget of at least the context selects every page: dense entmax attention through the same kernels
        w = dataclasses.replace(w, token_budget=args.token_budget,
                                name=w.name + ("_dense" if args.token_budget >= w.context else f"_budget{args.token_budget}"))
    K, W = args.steps, max(args.warmup, 3)
    headroom = 4 * 4 * (K + W) + 1024
    runner = StepRunner(w, headroom, seed_shift=1000 * rank)

    # ---- headline: W warm-up steps, then EXACTLY K timed steps between barriers, maximum over ranks
    for _ in range(W):
        runner.flush_l2()
        runner.step()
    ranks.barrier()
    sampler = ClockSampler(ranks.local_rank)
    if rank == 0:
        sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    wall0 = time.perf_counter()
    for i in range(K):
        runner.flush_l2()
        starts[i].record()
        runner.step()
        stops[i].record()
    ranks.barrier()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop() if rank == 0 else None
    step_times = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    ordered = sorted(step_times)
    step_us = {"min": ordered[0] * 1e3, "median": ordered[K // 2] * 1e3, "max": ordered[-1] * 1e3,
               "first": step_times[0] * 1e3, "last": step_times[-1] * 1e3}      # this rank's steps
    ms_per_step = ranks.max(sum(step_times) / K)

    peak, peak_src = measured_peak_gbs()
    bc, by, by_union = (None, None, None)
    stage_ms, launches = {}, 0
    if rank == 0:
        bc, by, by_union = byte_counts(runner, ms_per_step, peak)
        stage_ms = runner.stage_times_ms(max(3, min(K, 20)))     # per-kernel breakdown, same launches
        launches = len(stage_ms) + 1        # + the launch that stages q / k_new / v_new into the captured step's buffers

    e2e = e2e_eager = None
    if not args.no_e2e:
        e2e = runner.timed_e2e(K, ranks)
        e2e_eager = runner.timed_e2e(min(K, 50), ranks, eager=True)

    roofline = None
    if rank == 0 and stage_ms:
        kernel_bytes = {
            "page_score_kernel": by["metadata"], "gaussian_moments_kernel": by["metadata"],
            "decode_scores_kernel": by["kv"] / 2, "decode_values_kernel": by["kv"] / 2,
            # the group-shared K pass fetches every row once per GQA group: its bytes are the union's
            "decode_scores_group_kernel": by_union["kv"] / 2,
            "fused_topk_small_kernel": by["metadata"] + by["kv"],       # the whole step after the append
            # what the kernel fetches: the K rows of the selected tokens and the value rows of the supports (by the
            # benchmark's definition, which counts the value rows of every selected token, it would be by["kv"])
            "topk_decode_stream_kernel": by["kv"] / 2 + (bc.get("support_tokens_per_step") or 0) * w.head_dim
                                         * runner.q.element_size(),
        }
        dom = max((k for k in stage_ms if k in kernel_bytes), key=lambda k: stage_ms[k])
        ach = kernel_bytes[dom] / (stage_ms[dom] * 1e-3) / 1e9
        tr = load_traffic()
        per_byte = tr.get("dram_bytes_per_algorithmic_byte", {}).get(dom)
        traffic = int(per_byte * kernel_bytes[dom]) if per_byte else None
        roofline = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peak, "unit": "GB/s",
                    "frac": ach / peak, "peak_source": peak_src, "traffic": traffic,
                    "traffic_source": tr.get("source"), "traffic_taken_at_commit": tr.get("taken_at_commit"),
                    "algorithmic_bytes_per_launch": kernel_bytes[dom], "launch_us": stage_ms[dom] * 1e3,
                    "kernels_us": {k: v * 1e3 for k, v in stage_ms.items()},
                    "kernels_frac_of_measured": {k: kernel_bytes[k] / (stage_ms[k] * 1e-3) / 1e9 / peak
                                                 for k in stage_ms if k in kernel_bytes and k != "decode_values_kernel"},
                    **{k: v for k, v in bc.items() if k != "selected_tokens_per_step"}}

    # ---- the other configurations, for the record (not the headline)
    others = []
    headline_default = (not args.no_extra and not args.batch and not args.token_budget and not args.alpha
                        and w.name == "gqa_128k_topk")
    one_gpu_us = {}
    if headline_default:
        def summarize(r, wl, with_e2e=False):
            ms, stats = r.timed_steps(min(K, 20), 3)
            b2, _, _ = byte_counts(r, ms, peak)
            rec = {"workload": wl.name, "n_gpus": 1, "value": ms * 1e3, "unit": UNIT, "step_us": stats,
                   "achieved_gbs": b2["step_achieved_gbs"], "frac_of_measured": b2["step_frac_of_measured"],
                   "frac_of_8tbs": b2["step_frac_of_8tbs"], "union_frac_of_8tbs": b2["union_step_frac_of_8tbs"],
                   "moved_frac_of_measured": b2.get("moved_frac_of_measured"),
                   "moved_bytes_per_step": b2.get("moved_bytes_per_step"),
                   "algorithmic_bytes_per_step": b2["algorithmic_bytes_per_step"],
                   "selected_tokens_per_step": b2["selected_tokens_per_step"],
                   "one_launch_step": bool(wl.mode == "topk" and r._sel().get("fused", False))}
            if with_e2e:
                rec["e2e"] = r.timed_e2e(min(K, 20))
                rec["e2e_eager"] = r.timed_e2e(min(K, 20), eager=True)
            return rec
        try:
            if rank == 0:
                one_gpu_us[w.name] = ms_per_step * 1e3
                if world == 1:
                    w_a2 = dataclasses.replace(w, alpha=2.0, name=w.name + "_alpha2")
                    runner.switch_workload(w_a2)
                    others.append(summarize(runner, w_a2))
                for a2 in ((1.5, 2.0) if world == 1 else (1.5,)):
                    wg = dataclasses.replace(workloads.CONFIGS["gqa_128k_gaussian"], alpha=a2,
                                             name="gqa_128k_gaussian" + ("" if a2 == 1.5 else "_alpha2"))
                    runner.switch_workload(wg)     # same seed, shapes and cache
                    rec = summarize(runner, wg)
                    others.append(rec)
                    one_gpu_us[wg.name] = rec["value"]
            runner.graph = None
            del runner
            torch.cuda.empty_cache()
            ranks.barrier()
            if rank == 0 and world == 1:
                for name in ("topk_32k", "gaussian_ragged"):
                    w2 = workloads.CONFIGS[name]
                    r2 = StepRunner(w2, 1024)
                    others.append(summarize(r2, w2, with_e2e=True))
                    r2.graph = None
                    del r2
                    torch.cuda.empty_cache()
                # dense entmax attention (every page selected) through the same kernels: the "Entmax dense" bar
                # of the reference's figure, at 32k MHA and on four rows of the 128k GQA batch
                for base, nb in ((workloads.CONFIGS["topk_32k"], 1), (w, 4)):
                    wd = dataclasses.replace(base, batch=nb, token_budget=base.context + 4096,
                                             name=f"{base.name}_dense_b{nb}")
                    r2 = StepRunner(wd, 1024)
                    others.append(summarize(r2, wd))
                    r2.graph = None
                    del r2
                    torch.cuda.empty_cache()
            rec = run_million(ranks, min(K, 50), 5)
            if rec:
                others.append(rec)
            if world > 1:
                others.extend(run_strong_batch(ranks, w, min(K, 20), 3, one_gpu_us, collective=args.collective))
        except Exception as exc:      # the headline line must not be lost to a side measurement
            import traceback
            others.append({"error": repr(exc), "where": traceback.format_exc()[-1500:]})

    if rank != 0:
        ranks.close()
        return

    cpu_baseline = None
    if not args.no_cpu_baseline:
        try:
            cpu_baseline = run_cpu_reference(w, steps=args.cpu_steps, warmup=1)["cpu_baseline"]
        except Exception as exc:
            cpu_baseline = {"error": repr(exc)}

    config = static_config(w, f"replica x{world}")
    config.update({"selected_tokens_per_step": bc["selected_tokens_per_step"],
                   "algorithmic_bytes_per_step": bc["algorithmic_bytes_per_step"]})
    line = {
        "metric": METRIC, "value": ms_per_step * 1e3, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "step_us": step_us, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE_NAME[w.dtype], "data": "synthetic", "config": config,
        "tokens_per_s": w.batch * world / (ms_per_step * 1e-3),
        "achieved_tbs": bc["step_achieved_gbs"] / 1e3,
        "clocks": clocks, "e2e": e2e, "e2e_eager": e2e_eager,
        "gpu_launches": launches * K, "gpu_launches_per_step": launches,
        "roofline": roofline, "cpu_baseline": cpu_baseline, "wall_s_timed_region": wall,
        "other_workloads": others,
    }
    print(json.dumps(line))
    ranks.close()


def run_gpu_sequence_sharded(args):
    """``--workload million_gaussian``: the sharded request alone, as its own line."""
    ranks = Ranks()
    sampler = ClockSampler(ranks.local_rank)
    if ranks.rank == 0:
        sampler.start()
    rec = run_million(ranks, args.steps, max(args.warmup, 3), collective=args.collective)
    clocks = sampler.stop() if ranks.rank == 0 else None
    if ranks.rank == 0:
        peak, peak_src = measured_peak_gbs()
        line = {"metric": METRIC, "value": rec["value"], "unit": UNIT, "n_gpus": ranks.world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": rec["value"] / 1e3, "higher_is_better": False,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": rec["config"], "clocks": clocks, "e2e": rec["e2e"],
                "gpu_launches": rec.get("gpu_launches_per_step", 9) * args.steps,
                "roofline": {"bound": "hbm", "kernel": "whole step (all ranks)", "achieved": rec["achieved_gbs"],
                             "peak": peak * ranks.world, "unit": "GB/s",
                             "frac": rec["achieved_gbs"] / (peak * ranks.world), "peak_source": peak_src,
                             "traffic": None},
                "cpu_baseline": None, "record": rec}
        print(json.dumps(line))
    ranks.close()


# --------------------------------------------------------------------------- CPU arm

def _reference_modules():
    """The unmodified reference's CPU-capable modules from baseline/_ref, or None."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "entmaxkv")):
        return None
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    try:
        from entmaxkv.kv_cache import PagedKVCache as RefCache
        from entmaxkv import gaussian_utils as ref_gu
        return RefCache, ref_gu
    except Exception:
        return None


def run_cpu_reference(w, steps: int, warmup: int, rows: int = 0):
    """Time the reference's CPU path for one decode step of ``w`` on this host's cores.

    What a step is (the reference's own step, attention_topk.py:39-100 / attention_gaussian.py:58-142,
    with the new token already in the cache as in its benchmark script, tests/run_benchmarks.py:56-105):
      top-k:    key-range page scores -> torch.topk -> paged entmax decode over the selected pages;
      Gaussian: page statistics + tau_hat -> threshold selection -> tau clamp -> corrected decode.
    The reference's own CPU code runs where it has any (cache object, ``estimate_page_criticality(
    use_triton=False)``, ``compute_gaussian_aware_statistics`` torch fallback with its CPU tau solver, the
    CPU branch of the tau clamp); threshold select + pack and the two paged decodes exist only as Triton
    kernels there and are the restatements in ``oracle/``.  fp32 on the CPU (the reference's CPU case),
    K/V repeated per query head as the reference needs for GQA.  The sample is bounded: ``rows`` batch
    rows (default: 2, or the batch if smaller) at full context, scaled to the batch.
    Dense entmax attention over the whole cache (the reference tests' yardstick) is timed once beside it.
    """
    from entmaxkv_b200 import workloads
    from oracle import cache as ocache, decode as od, dense as odense, gaussian as og, topk as otopk

    try:      # launchers such as torchrun pin OMP_NUM_THREADS to 1; the baseline gets every core it may use
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except Exception:
        pass
    threads = torch.get_num_threads()
    rows = min(w.batch, rows or 2)
    G = w.q_heads // w.kv_heads
    P = w.page_size
    _, lens_all = workloads.workload_lengths(w)
    mods = _reference_modules()
    per_row = []          # (cache object, q, S) per sampled row
    for b in range(rows):
        inp = workloads.make_inputs(w, device="cpu", batch_slice=slice(b, b + 1))
        n0 = lens_all[b]
        k = torch.cat([inp["k"][:, :, :n0], inp["k_new"]], dim=2).float()
        v = torch.cat([inp["v"][:, :, :n0], inp["v_new"]], dim=2).float()
        if G > 1:
            k, v = k.repeat_interleave(G, dim=1), v.repeat_interleave(G, dim=1)
        q = inp["q"].float()
        c = mods[0](page_size=P) if mods is not None else ocache.OracleCache(P)
        # the statistics are prefill-time state, not part of the step; the reference builds them with a
        # Python loop over pages, the vectorised restatement gives the same tensors in seconds
        c.k_cache, c.v_cache = k, v
        c.k_min, c.k_max, c.k_mean, c.k_std = ocache.page_stats(k, P)
        per_row.append((c, q, n0 + 1))

    def step():
        outs = []
        for c, q, S in per_row:
            Hq = q.shape[1]
            n_pages = (S + P - 1) // P
            if w.mode == "topk":
                if mods is not None:
                    sc = c.estimate_page_criticality(q, use_triton=False, exclude_last_page=True)
                else:
                    sc = otopk.criticality_scores(q, c.k_min, c.k_max)
                k_sel = min(w.token_budget // P, n_pages - 1)
                idx = torch.topk(sc, k_sel, dim=-1).indices.sort(dim=-1).values
                tables = [[idx[0, h].tolist() + [n_pages - 1] for h in range(Hq)]]
                T = k_sel * P + (S - (n_pages - 1) * P)
                outs.append(od.decode(q, c.k_cache, c.v_cache, tables, [[T] * Hq], P, w.alpha, mode="exact", niter=2)[0])
            else:
                if mods is not None:
                    st = mods[1].compute_gaussian_aware_statistics(q, c.k_mean, c.k_std, S, P, alpha=w.alpha,
                                                                   use_triton_stats=False)
                    mu, sg = st["mu_scores_per_page"], st["sigma_scores_per_page"]
                    th, sig_g = st["tau_hat"], st["sigma_global"].squeeze(-1)
                    margin_z, max_q = st["safety_margin_z"], st["max_quantile"]
                else:
                    n_stats = n_pages - 1
                    mu, var, sg = og.page_moments(q, c.k_mean, c.k_std, n_stats)
                    mean, mv, vm = og.head_moments(mu, var)
                    sig_g = og.global_sigma(mv, vm)
                    th = og.tau_hat(mean, sig_g, n_stats * P, w.alpha)
                    margin_z, max_q = og.auto_margin(sig_g)
                pages, tau_floor, _ = og.select_threshold_pack(
                    mu, sg, th, sig_g, page_size=P, alpha=w.alpha, safety_margin_z=margin_z, max_quantile=max_q,
                    threshold_excess_margin_fraction=0.2, num_pages=n_pages)
                if mods is not None:
                    width = max(len(p) for p in pages[0])
                    pi = torch.zeros(1, Hq, width, dtype=torch.int32)
                    for h in range(Hq):
                        pi[0, h, :len(pages[0][h])] = pages[0][h]
                    cnt = torch.tensor([[len(p) for p in pages[0]]], dtype=torch.int32)
                    st["tau_floor"] = tau_floor
                    tau0 = mods[1].clamp_tau_to_selected_page_statistics(th, st, pi, cnt, P, w.alpha)
                else:
                    tau0 = og.clamp_tau(th, mu, sg, pages, tau_floor, page_size=P, alpha=w.alpha)
                last = og.last_page_size(S, P)
                tables = [[p.tolist() for p in pages[0]]]
                ntok = [[max(len(t) - 1, 0) * P + last for t in tables[0]]]
                outs.append(od.decode(q, c.k_cache, c.v_cache, tables, ntok, P, w.alpha, mode="corrected",
                                      tau0=tau0.numpy(), iters=1)[0])
        return outs

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    # the dense yardstick, once, on one row
    c0, q0, _ = per_row[0]
    t1 = time.perf_counter()
    odense.dense_entmax_decode(q0, c0.k_cache, c0.v_cache, w.alpha)
    dense_s = time.perf_counter() - t1
    scale = w.batch / rows
    what = ("key-range scores + top-k + paged decode" if w.mode == "topk"
            else "page statistics + tau_hat + threshold selection + clamp + corrected decode")
    cb = {"value": dt * scale * 1e6, "unit": UNIT, "cores": threads, "host_cpus": os.cpu_count(),
          "kind": "reference" if mods is not None else "port",
          "parts": ({"cache object, page scores, top-k, Gaussian statistics, tau solver, tau clamp":
                     "reference (baseline/_ref, its CPU code paths)",
                     "threshold select + pack, paged entmax decode": "port (oracle/): Triton-only in the reference"}
                    if mods is not None else {"all": "port (oracle/): baseline/_ref not importable"}),
          "sample": f"{steps} steps of {rows}/{w.batch} batch rows at full context ({what}; new token already "
                    f"appended, fp32, K/V repeated per query head), scaled x{scale:g}",
          "dense_entmax_us": dense_s * w.batch * 1e6,
          "dense_entmax_note": f"dense entmax decode attention over the whole cache (port), 1 row x{w.batch}"}
    return {"cpu_baseline": cb, "sampled_rows": rows, "scaled_by": scale}


def run_reference_arm(args):
    from entmaxkv_b200 import workloads
    rank, _, world = dist_env()
    if rank != 0:
        return
    w = workloads.CONFIGS[args.workload]
    K, W = args.steps, args.warmup
    res = run_cpu_reference(w, steps=K, warmup=W)
    cb = res["cpu_baseline"]
    config = static_config(w, f"replica x{world}")
    config.update({"sampled_rows": res["sampled_rows"], "scaled_by": res["scaled_by"],
                   "reference_arm": "host cores; value = time of the sampled rows x scaled_by"})
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": cb["value"] / 1e3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_reference_triton(args):
    """Side measurement, not part of the contract lines: the UNMODIFIED reference's Triton step
    (installed under baseline/_ref) on this GPU, same shapes and timing rules as the default arm.

    The reference wrappers cannot express GQA (their page tables are per query head while the
    kernels want them per KV head), and its cache appends by concatenation, so the workload is run
    the way the reference's own benchmark script runs it (tests/run_benchmarks.py:56-105): K/V
    repeated to one KV head per query head, the new token appended before timing and
    ``append_cache=False`` in the timed call.  ``--batch`` bounds memory (the repeat makes the
    cache G times larger and initialize() clones it); the time is scaled to the full batch.
    """
    from entmaxkv_b200 import workloads
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "entmaxkv")):
        print(json.dumps({"impl": "reference_triton", "unavailable": "baseline/_ref holds no install of the reference"}))
        return
    sys.path.insert(0, ref_root)
    from entmaxkv.kv_cache import PagedKVCache
    from entmaxkv.attention_topk import sparse_attention_decode_paged
    from entmaxkv.attention_gaussian import sparse_attention_decode_gaussian_aware_entmax

    w = workloads.CONFIGS[args.workload]
    full_batch = w.batch
    if args.batch:
        w = dataclasses.replace(w, batch=args.batch)
    # The reference forms cache addresses as int32 (program id x batch stride in elements,
    # kernels/adadecode_paged.py:110): a cache of 2^31 elements or more wraps the offset and the
    # kernel reads out of range.  Such a size is never launched here.
    cache_elems = w.batch * w.q_heads * (w.context + 1) * w.head_dim
    if cache_elems >= 2 ** 31:
        print(json.dumps({"impl": "reference_triton", "unavailable":
                          f"reference kernels index the cache with int32 offsets; batch {w.batch} x heads {w.q_heads} "
                          f"x tokens {w.context + 1} x dim {w.head_dim} = {cache_elems} elements >= 2^31 "
                          "(use --batch to pick an addressable slice)"}))
        return
    torch.cuda.set_device(0)
    inp = workloads.make_inputs(w, device="cuda")
    G = w.q_heads // w.kv_heads
    S1, P = w.context + 1, w.page_size
    cache = PagedKVCache(page_size=P)
    k = inp.pop("k").repeat_interleave(G, dim=1) if G > 1 else inp.pop("k")
    v = inp.pop("v").repeat_interleave(G, dim=1) if G > 1 else inp.pop("v")
    cache.initialize(k, v)
    del k, v
    torch.cuda.empty_cache()
    k_new = inp["k_new"].repeat_interleave(G, dim=1)
    v_new = inp["v_new"].repeat_interleave(G, dim=1)
    cache.append(k_new, v_new)
    torch.cuda.empty_cache()
    q = inp["q"]
    out = torch.zeros_like(q)
    q_seqlens = torch.full((w.batch,), S1, device="cuda", dtype=torch.int32)
    if w.mode == "topk":
        pages = (S1 + P - 1) // P
        n_sel = min(w.token_budget // P, pages - 1)
        eff = n_sel * P + (S1 - (pages - 1) * P)
        cache_seqlens = torch.full((w.batch,), eff, device="cuda", dtype=torch.int32)

        def step():
            sparse_attention_decode_paged(q=q, kv_cache=cache, k_new=k_new, v_new=v_new, out=out,
                                          token_budget=w.token_budget, cache_seqlens=cache_seqlens,
                                          q_seqlens=q_seqlens, alpha=w.alpha, niter=2, append_cache=False)
    else:
        def step():
            sparse_attention_decode_gaussian_aware_entmax(q=q, kv_cache=cache, k_new=k_new, v_new=v_new, out=out,
                                                          alpha=w.alpha, append_cache=False, tau_mode=w.tau_mode,
                                                          q_seqlens=q_seqlens)
    flush = L2Flush()
    K, W = args.steps, max(args.warmup, 3)
    for _ in range(W):
        step()
    torch.cuda.synchronize()
    times = []
    for _ in range(K):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    scale = full_batch / w.batch
    med = statistics.median(times)
    print(json.dumps({
        "impl": "reference_triton", "metric": METRIC, "unit": UNIT, "value": med * 1e3 * scale,
        "ms_per_step": med * scale, "measured_ms": med, "min_ms": min(times), "scaled_by": scale,
        "steps": K, "warmup": W, "higher_is_better": False, "dtype": str(w.dtype).replace("torch.", ""),
        "config": {"workload": w.name, "mode": w.mode, "batch_measured": w.batch, "batch_full": full_batch,
                   "context": w.context, "kv_heads_as_run": w.q_heads,
                   "note": "append excluded (done before timing), K/V repeated per query head, L2 flushed"},
        "gpu": torch.cuda.get_device_name(0)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_triton"])
    ap.add_argument("--workload", default="gqa_128k_topk")
    ap.add_argument("--cpu-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch size (small profiling cases)")
    ap.add_argument("--token-budget", type=int, default=0,
                    help="override the top-k token budget (>= context: every page, i.e. dense entmax attention)")
    ap.add_argument("--alpha", type=float, default=0.0, help="override the workload's entmax alpha (side measurements)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="sequence-sharded mode: reductions fused over peer memory (default) or NCCL all-reduces")
    ap.add_argument("--no-extra", action="store_true", help="skip the side measurements of the other workloads")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.impl == "reference_triton":
        run_reference_triton(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU fallback")
        if args.workload == "million_gaussian":
            run_gpu_sequence_sharded(args)
        else:
            run_gpu(args)


if __name__ == "__main__":
    main()
