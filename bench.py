#!/usr/bin/env python
"""Decode-step benchmark of the sparse entmax path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one pass of the hot path over one batch of seeded synthetic input:
append the new token, select pages (top-k or Gaussian-aware), paged entmax decode.
Prints ONE JSON line (rank 0).  ``value`` is the device-timed step latency with all
inputs resident in HBM; ``e2e`` is the same step through the public Python API with
q / k_new / v_new coming from pinned host memory and the output read back.

With N > 1 every rank runs its own replica of the workload on its own GPU (the path
partitions by batch row and KV head, there is no data-path collective): weak scaling.
``--impl reference`` times the reference's CPU path (dense entmax decode attention +
tau solver + page selection) restated in ``oracle/`` on the host cores.
"""

from __future__ import annotations

import argparse
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


# --------------------------------------------------------------------------- helpers

def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

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


# --------------------------------------------------------------------------- GPU arm

class StepRunner:
    """Owns one workload replica on the current device and runs decode steps on it."""

    def __init__(self, w, rank: int, headroom: int):
        import entmaxkv_b200 as E
        from entmaxkv_b200 import workloads
        self.E, self.w = E, w
        if rank:
            w = type(w)(**{**w.__dict__, "seed": w.seed + 1000 * rank})
        inp = workloads.make_inputs(w, device="cuda")
        self.inp = inp
        self.cache = E.PagedKVCache(page_size=w.page_size)
        self.cache.initialize(inp["k"], inp["v"], seq_lens=inp["seq_lens"],
                              capacity=w.context + headroom)
        self.seq_lens0 = list(inp["seq_lens"])
        # K/V now live in the cache; drop the staging copies
        del inp["k"], inp["v"]
        torch.cuda.empty_cache()
        self.q, self.k_new, self.v_new = inp["q"], inp["k_new"], inp["v_new"]
        # a decode loop appends a different token every step: a pool of seeded tokens, iid normal like the
        # rest of the cache, taken in turn (the same key appended a hundred times piles identical
        # scores onto every head and distorts the supports after ~75 steps)
        self.k_pool, self.v_pool = workloads.token_pool(w, 16, "cuda")
        self.k_pool[0].copy_(self.k_new)
        self.v_pool[0].copy_(self.v_new)
        self.steps_done = 0
        self.out = torch.zeros_like(self.q)
        self.flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
        self.flush_src = torch.zeros(512 << 18, dtype=torch.int32, device="cuda")
        from entmaxkv_b200.graph import DecodeStepGraph
        if w.mode == "topk":
            self.graph = DecodeStepGraph(self.cache, w.q_heads, "topk", token_budget=w.token_budget,
                                         alpha=w.alpha, niter=2)
        else:
            self.graph = DecodeStepGraph(self.cache, w.q_heads, "gaussian", alpha=w.alpha,
                                         tau_mode=w.tau_mode)

    def switch_workload(self, w2):
        """Re-use the resident cache and inputs for another selection mode of the same shapes."""
        from entmaxkv_b200.graph import DecodeStepGraph
        self.w = w2
        if w2.mode == "topk":
            self.graph = DecodeStepGraph(self.cache, w2.q_heads, "topk", token_budget=w2.token_budget,
                                         alpha=w2.alpha, niter=2)
        else:
            self.graph = DecodeStepGraph(self.cache, w2.q_heads, "gaussian", alpha=w2.alpha,
                                         tau_mode=w2.tau_mode)

    def timed_steps(self, K, W):
        """W warm-up + K timed graph replays with a cold L2; returns ms per step."""
        for _ in range(W):
            self.flush_l2()
            self.step()
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
        for i in range(K):
            self.flush_l2()
            starts[i].record()
            self.step()
            stops[i].record()
        torch.cuda.synchronize()
        times = [a.elapsed_time(b) for a, b in zip(starts, stops)]
        ordered = sorted(times)
        self.last_step_us = {"min": ordered[0] * 1e3, "median": ordered[len(ordered) // 2] * 1e3,
                             "max": ordered[-1] * 1e3, "first": times[0] * 1e3, "last": times[-1] * 1e3}
        return sum(times) / K

    def flush_l2(self):
        """Write 512 MiB, then read another 512 MiB: the read pushes the written (dirty)
        lines out to HBM, so the timed step starts with a cold L2 and no write-back in flight."""
        self.flush_buf.fill_(1)
        self.flush_src.max()

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
        w, E = self.w, self.E
        q = self.q if q is None else q
        if k_new is None or v_new is None:
            k_new, v_new = self.next_token()
        out = self.out if out is None else out
        if w.mode == "topk":
            E.sparse_attention_decode_paged(q, self.cache, k_new, v_new, out, w.token_budget,
                                            alpha=w.alpha, niter=2, append_cache=True)
        else:
            E.sparse_attention_decode_gaussian_aware_entmax(q, self.cache, k_new, v_new, out, alpha=w.alpha,
                                                            append_cache=True, tau_mode=w.tau_mode)
        return out

    def selected_tokens(self) -> int:
        sel = (self.cache.last_topk_selection if self.w.mode == "topk"
               else self.cache.last_gaussian_selection)
        return int(sel["tok_counts"].sum().item())

    def union_tokens(self) -> int:
        """Tokens selected by at least one query head of each GQA group, summed over (batch row, KV
        head): the K/V rows a step has to fetch when heads of a group share what they both picked."""
        sel = (self.cache.last_topk_selection if self.w.mode == "topk"
               else self.cache.last_gaussian_selection)
        pages, counts = sel["page_indices"], sel["num_selected"]
        B, Hq, width = pages.shape
        G = self.w.q_heads // self.w.kv_heads
        P = self.w.page_size
        valid = torch.arange(width, device=pages.device)[None, None, :] < counts[:, :, None]
        big = torch.iinfo(torch.int32).max
        ids = torch.where(valid, pages, torch.full_like(pages, big)).reshape(B, Hq // G, G * width)
        ids = ids.sort(dim=-1).values
        new = torch.ones_like(ids, dtype=torch.bool)
        new[..., 1:] = ids[..., 1:] != ids[..., :-1]
        n_pages = (new & (ids != big)).sum(dim=-1)                      # [B, H_kv] distinct pages incl. the last one
        lens = torch.tensor(self.cache.host_seq_lens, device=pages.device)
        last_tokens = lens - (torch.div(lens + P - 1, P, rounding_mode="floor") - 1) * P
        return int(((n_pages - 1).clamp(min=0) * P + last_tokens[:, None]).sum().item())

    # -- stage-by-stage timing (same launches as step(), one event pair per stage)
    def staged_step(self, ev):
        import ctypes as C
        from entmaxkv_b200 import _lib, attention_topk as AT, attention_gaussian as AG
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
            max_tokens, mode, iters, wl, wt = (k_max + 1) * P, _lib.TAU_EXACT, 2, items.data_ptr(), None
        else:
            import entmaxkv_b200.attention_gaussian as G
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
            wl_t = c.scratch("g_work", (B * Hq * nch,), torch.int64)
            n_items = wl_t.numel()
            wt_t = c.scratch("g_work_total", (1 + (B * Hq + 1023) // 1024,), torch.int32, zero=True)
            grouped = AG.grouped_enabled(q, c)     # the wrapper then builds no per-head work list
            _lib.check(lib.ekv_gaussian_select(
                desc, Hq, S, 1, 1, float(w.alpha), 0.2, G._z_of_quantile(0.99, P), G._z_of_quantile(0.995, P),
                G._z_of_quantile(0.5, P), 1, None, mu.data_ptr(), sigma.data_ptr(), pcap, hstat.data_ptr(),
                pages.data_ptr(), pcap, nsel.data_ptr(), ntok.data_ptr(), tfl.data_ptr(), cap.data_ptr(),
                tau.data_ptr(), None if grouped else wl_t.data_ptr(), None if grouped else wt_t.data_ptr(), st),
                "ekv_gaussian_select")
            mark("gaussian_select_kernel")
            max_tokens, mode = c.capacity, _lib.TAU_CORRECTED
            iters = {"fixed": 0, "corrected": 1}.get(w.tau_mode, 1)
            wl, wt = wl_t.data_ptr(), wt_t.data_ptr()
        evs = [ev() for _ in range(3)]
        if wt is None:
            wl_tensor, wt_tensor = items, None
        else:
            wl_tensor, wt_tensor = wl_t, wt_t
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
        del AG
        return marks


def run_gpu(args):
    import torch.distributed as dist
    from entmaxkv_b200 import workloads

    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    w = workloads.CONFIGS[args.workload]
    if args.batch:
        import dataclasses
        w = dataclasses.replace(w, batch=args.batch)   # a slice of the workload (profiling captures)
    if args.alpha:
        import dataclasses
        w = dataclasses.replace(w, alpha=args.alpha, name=f"{w.name}_alpha{args.alpha:g}")
    if args.token_budget and w.mode == "topk":
        import dataclasses
        # a budget of at least the context selects every page: dense entmax attention through the same kernels
        w = dataclasses.replace(w, token_budget=args.token_budget,
                                name=w.name + ("_dense" if args.token_budget >= w.context else f"_budget{args.token_budget}"))
    headroom = 4 * (args.steps + args.warmup) + 1024
    runner = StepRunner(w, rank, headroom)
    K, W = args.steps, max(args.warmup, 3)

    for _ in range(W):
        runner.flush_l2()
        runner.step()
    barrier()
    sampler = ClockSampler(local_rank)
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
    barrier()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop() if rank == 0 else None
    step_times = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    total_ms = sum(step_times)
    ordered = sorted(step_times)
    step_us = {"min": ordered[0] * 1e3, "median": ordered[K // 2] * 1e3, "max": ordered[-1] * 1e3,
               "first": step_times[0] * 1e3, "last": step_times[-1] * 1e3}      # this rank's steps
    if os.environ.get("EKV_BENCH_STEP_TIMES"):
        print("step_us", [round(x * 1e3, 1) for x in step_times], file=sys.stderr)
    if world > 1:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / K
    sel_tokens = runner.selected_tokens()
    lens_now = runner.cache.host_seq_lens

    # ---- per-kernel breakdown (rank 0), same launches with an event after each
    stage_ms, launches = {}, 0
    if rank == 0:
        n_b = max(3, min(K, 20))
        acc = {}
        for _ in range(n_b):
            runner.flush_l2()
            marks = runner.staged_step(lambda: torch.cuda.Event(enable_timing=True))
            torch.cuda.synchronize()
            for (_, e0), (name, e1) in zip(marks[:-1], marks[1:]):
                acc.setdefault(name, []).append(e0.elapsed_time(e1))
        # median over the repetitions: one pass that happens to (re)allocate a scratch buffer inside a
        # stage must not colour the per-kernel figure
        stage_ms = {k: statistics.median(v) for k, v in acc.items()}
        launches = len(stage_ms)

    # ---- end to end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        hq = runner.q.cpu().pin_memory()
        hk_pool = runner.k_pool.cpu().pin_memory()   # the host's copies of the tokens to append, taken in turn
        hv_pool = runner.v_pool.cpu().pin_memory()
        hk, hv = hk_pool[0], hv_pool[0]
        hout = torch.empty_like(hq).pin_memory()
        e2e_no = [0]

        def e2e_step():
            i = e2e_no[0] % hk_pool.shape[0]
            e2e_no[0] += 1
            dout = runner.step(hq, hk_pool[i], hv_pool[i])   # H2D copies of the three inputs + graph replay
            hout.copy_(dout, non_blocking=True)     # D2H of the result
            torch.cuda.current_stream().synchronize()

        for _ in range(3):
            e2e_step()
        barrier()
        tt = 0.0
        for _ in range(K):
            runner.flush_l2()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            e2e_step()
            tt += time.perf_counter() - t0
        barrier()
        e2e_us = tt / K * 1e6
        if world > 1:
            t = torch.tensor([e2e_us], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_us = float(t.item())
        esz = runner.q.element_size()
        e2e = {"value": e2e_us, "unit": UNIT,
               "h2d_bytes_per_step": (hq.numel() + hk.numel() + hv.numel()) * esz,
               "d2h_bytes_per_step": hout.numel() * esz}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak_gbs()
    by = workloads.algorithmic_bytes(w, [n - 1 for n in lens_now], sel_tokens)
    by_union = workloads.algorithmic_bytes(w, [n - 1 for n in lens_now], runner.union_tokens())
    step_gbs = by["total"] / (ms_per_step * 1e-3) / 1e9
    kernel_bytes = {
        "page_score_kernel": by["metadata"], "gaussian_moments_kernel": by["metadata"],
        "decode_scores_kernel": by["kv"] / 2, "decode_values_kernel": by["kv"] / 2,
        # the group-shared K pass fetches every row once per GQA group: its bytes are the union's
        "decode_scores_group_kernel": by_union["kv"] / 2,
    }
    roofline = None
    if stage_ms:
        dom = max((k for k in stage_ms if k in kernel_bytes), key=lambda k: stage_ms[k])
        ach = kernel_bytes[dom] / (stage_ms[dom] * 1e-3) / 1e9
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
                traffic = json.load(f).get(f"{dom}:{w.name}")
        except Exception:
            pass
        roofline = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peak, "unit": "GB/s",
                    "frac": ach / peak, "peak_source": peak_src, "traffic": traffic,
                    "algorithmic_bytes_per_launch": kernel_bytes[dom],
                    "launch_us": stage_ms[dom] * 1e3,
                    "step_achieved_gbs": step_gbs, "step_frac_of_measured": step_gbs / peak,
                    "step_frac_of_8tbs": step_gbs / HBM_NOMINAL_GBS,
                    # the same with K/V rows counted once per GQA group (union over its query heads)
                    "union_bytes_per_step": by_union["total"],
                    "union_step_achieved_gbs": by_union["total"] / (ms_per_step * 1e-3) / 1e9,
                    "union_step_frac_of_8tbs": by_union["total"] / (ms_per_step * 1e-3) / 1e9 / HBM_NOMINAL_GBS,
                    "kernels_us": {k: v * 1e3 for k, v in stage_ms.items()}}

    # ---- the other single-GPU configurations, for the record (not the headline)
    others = []
    if world == 1 and not args.no_extra and not args.batch and not args.token_budget and w.name == "gqa_128k_topk":
        def summarize(r, wl):
            ms = r.timed_steps(min(K, 20), 3)
            b2 = workloads.algorithmic_bytes(wl, [n - 1 for n in r.cache.host_seq_lens], r.selected_tokens())
            gbs = b2["total"] / (ms * 1e-3) / 1e9
            bu = workloads.algorithmic_bytes(wl, [n - 1 for n in r.cache.host_seq_lens], r.union_tokens())
            return {"workload": wl.name, "value": ms * 1e3, "unit": UNIT, "achieved_gbs": gbs,
                    "frac_of_measured": gbs / peak, "frac_of_8tbs": gbs / HBM_NOMINAL_GBS,
                    "union_frac_of_8tbs": bu["total"] / (ms * 1e-3) / 1e9 / HBM_NOMINAL_GBS,
                    "algorithmic_bytes_per_step": b2["total"], "selected_tokens_per_step": r.selected_tokens()}
        try:
            import dataclasses
            for a2 in (2.0,):
                w_a2 = dataclasses.replace(w, alpha=a2, name=w.name + "_alpha2")
                runner.switch_workload(w_a2)
                others.append(summarize(runner, w_a2))
            for a2 in (1.5, 2.0):
                wg = dataclasses.replace(workloads.CONFIGS["gqa_128k_gaussian"], alpha=a2,
                                         name="gqa_128k_gaussian" + ("" if a2 == 1.5 else "_alpha2"))
                runner.switch_workload(wg)     # same seed, shapes and cache
                others.append(summarize(runner, wg))
            del runner
            torch.cuda.empty_cache()
            for name in ("topk_32k", "gaussian_ragged"):
                w2 = workloads.CONFIGS[name]
                r2 = StepRunner(w2, 0, 1024)
                others.append(summarize(r2, w2))
                del r2
                torch.cuda.empty_cache()
        except Exception as exc:      # the headline line must not be lost to a side measurement
            others.append({"error": repr(exc)})

    cpu_baseline = None
    if not args.no_cpu_baseline and world >= 1:
        cpu_baseline = run_cpu_reference(w, steps=args.cpu_steps, warmup=1, quiet=True)

    line = {
        "metric": METRIC, "value": ms_per_step * 1e3, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "step_us": step_us, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None,
        "dtype": {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}[w.dtype],
        "data": "synthetic",
        "config": {"workload": w.name, "mode": w.mode, "batch_per_gpu": w.batch, "q_heads": w.q_heads,
                   "kv_heads": w.kv_heads, "head_dim": w.head_dim, "context": w.context,
                   "page_size": w.page_size, "token_budget": w.token_budget if w.mode == "topk" else None,
                   "alpha": w.alpha, "seed": w.seed, "needle_fraction": w.needle_fraction,
                   "l2": "flushed between timed steps (512 MiB write + 512 MiB read)", "parallelism": f"replica x{world}",
                   "launch": "whole step replayed as one CUDA graph",
                   "selected_tokens_per_step": sel_tokens, "algorithmic_bytes_per_step": by["total"]},
        "tokens_per_s": w.batch * world / (ms_per_step * 1e-3),
        "achieved_tbs": step_gbs / 1e3,
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches * K, "gpu_launches_per_step": launches,
        "roofline": roofline, "cpu_baseline": cpu_baseline, "wall_s_timed_region": wall,
        "other_workloads": others,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_gpu_sequence_sharded(args):
    """One long request, pages split contiguously across the ranks (strong scaling): local
    moments / selection / K pass / V pass per rank, four small NCCL all-reduces per step."""
    import torch.distributed as dist
    from entmaxkv_b200 import sharded, workloads

    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    if world == 1:
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    w = workloads.CONFIGS[args.workload]
    P = w.page_size
    inp = workloads.make_inputs(w, device="cuda")      # same seed on every rank -> same tensors
    S = w.context
    # --emulate-world N (single process): hold the last rank's 1/N shard alone, with a one-rank
    # exchange - the per-rank kernel cost of an N-GPU run without its peers (profiling aid)
    split_world = args.emulate_world if (world == 1 and args.emulate_world) else world
    split_rank = split_world - 1 if split_world != world else rank
    lo, hi = sharded.split_pages(S, P, split_world)[split_rank]
    shard = sharded.GpuSequenceShard(P, split_rank, split_world)
    K, W = args.steps, max(args.warmup, 3)
    shard.initialize(inp["k"][:, :, lo:hi].contiguous(), inp["v"][:, :, lo:hi].contiguous(),
                     capacity=(hi - lo) + 4 * (K + W) + 1024)
    del inp["k"], inp["v"]
    torch.cuda.empty_cache()
    q, kn, vn = inp["q"], inp["k_new"], inp["v_new"]
    reduce = sharded.dist_reduce()
    # emulation: the shard is a complete (shorter) request of its own, so its statistics are consistent
    shard.set_global_lengths([(hi - lo) if split_world != world else S] * w.batch)
    exchange = None
    if args.collective == "peer":
        from entmaxkv_b200.exchange import PeerExchange
        exchange = PeerExchange(rank, world, max_floats=max(1 << 14, w.batch * w.q_heads * w.head_dim))
    graph = sharded.ShardedStepGraph(shard, reduce, w.q_heads, alpha=w.alpha, tau_mode=w.tau_mode,
                                     exchange=exchange)
    flush_w = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    flush_r = torch.zeros(512 << 18, dtype=torch.int32, device="cuda")
    total = [S]

    def step():
        if args.no_graph:
            out = sharded.sharded_gaussian_decode_step([shard], reduce, [q], [kn], [vn], alpha=w.alpha,
                                                       tau_mode=w.tau_mode, exchange=exchange)[0]
        else:
            out = graph.step(q, kn, vn)      # kernels and the four all-reduces replayed as one CUDA graph
        total[0] += 1
        return out

    def flush():
        flush_w.fill_(1)
        flush_r.max()

    for _ in range(W):
        flush()
        step()
    dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
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
        step()
        stops[i].record()
    dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if exchange is not None:
        exchange.check()         # a timed-out wait would make the numbers meaningless: fail loudly
    # ---- end to end: inputs from pinned host memory every step, the result read back to the host
    e2e = None
    if not args.no_e2e and not args.no_graph:
        hq, hk, hv = q.cpu().pin_memory(), kn.cpu().pin_memory(), vn.cpu().pin_memory()
        hout = torch.empty((w.batch, w.q_heads, 1, w.head_dim), dtype=torch.float32).pin_memory()

        def e2e_step():
            dout = graph.step(hq, hk, hv)           # H2D copies of the three inputs + graph replay
            hout.copy_(dout, non_blocking=True)     # D2H of the result (rank 0's copy is the user's)
            torch.cuda.current_stream().synchronize()
            total[0] += 1

        for _ in range(3):
            e2e_step()
        tt = 0.0
        K2 = min(K, 50)
        for _ in range(K2):
            flush()
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            e2e_step()
            tt += time.perf_counter() - t0
        t = torch.tensor([tt / K2 * 1e6], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {"value": float(t.item()), "unit": UNIT,
               "h2d_bytes_per_step": (hq.numel() + hk.numel() + hv.numel()) * hq.element_size(),
               "d2h_bytes_per_step": hout.numel() * 4}
        if exchange is not None:
            exchange.check()
    stage_us = None
    if exchange is not None and not args.no_stages:
        # the same launches issued eagerly with an event after each stage, per rank
        names = ["append", "moments", "x_finalize", "select", "x_clamp", "decode_x"]
        calls = [lambda: shard.append(kn, vn), lambda: shard.moments(q, w.alpha), lambda: shard.finalize_x(exchange),
                 lambda: shard.select(), lambda: shard.clamp_x(exchange), lambda: shard.decode_x(exchange, 1)]
        reps = 10
        acc = [0.0] * len(names)
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
            total[0] += 1
        mine = torch.tensor(acc, device="cuda", dtype=torch.float64)
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        stage_us = {f"rank{r}": {n: round(float(v), 1) for n, v in zip(names, t.tolist())}
                    for r, t in enumerate(everyone)}
        toks = [torch.empty_like(shard.tokens) for _ in range(world)]
        dist.all_gather(toks, shard.tokens)
        stage_us["selected_tokens_per_rank"] = [int(t.sum().item()) for t in toks]
        exchange.check()
    t = torch.tensor([sum(a.elapsed_time(b) for a, b in zip(starts, stops))], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / K
    sel = shard.tokens.sum().to(torch.float64)
    dist.all_reduce(sel)
    # this library's kernels per step: append, moments, finalize, select, clamp, K pass, tau, V pass, fold
    # (peer) / + three small kernels and the chunk reduce, minus the fused ones (NCCL path)
    n_launch = 9 if exchange is not None else 11
    if rank == 0:
        peak, peak_src = measured_peak_gbs()
        by = workloads.algorithmic_bytes(w, [S], int(sel.item()))
        gbs = by["total"] / (ms_per_step * 1e-3) / 1e9
        print(json.dumps({
            "metric": METRIC, "value": ms_per_step * 1e3, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16" if w.dtype == torch.bfloat16 else "f16", "data": "synthetic",
            "config": {"workload": w.name, "mode": w.mode, "batch": w.batch, "q_heads": w.q_heads,
                       "kv_heads": w.kv_heads, "head_dim": w.head_dim, "context": w.context,
                       "page_size": P, "alpha": w.alpha, "seed": w.seed,
                       "emulated_shard_of": split_world if split_world != world else None,
                       "parallelism": f"sequence pages x{world}, " +
                                      ("4 reductions fused into their consumer kernels over NVLink peer memory"
                                       if exchange is not None else "4 NCCL all-reduces per step") +
                                      ("" if args.no_graph else ", step replayed as one CUDA graph"),
                       "l2": "flushed between timed steps (512 MiB write + 512 MiB read)",
                       "start_alignment": "device-side peer barrier before each start event" if exchange is not None else "host barrier",
                       "selected_tokens_per_step": int(sel.item()), "algorithmic_bytes_per_step": by["total"]},
            "achieved_tbs": gbs / 1e3, "clocks": clocks, "e2e": e2e, "gpu_launches": n_launch * K,
            "gpu_launches_per_step": n_launch, "status_checked": True,
            "roofline": {"bound": "hbm", "kernel": "whole step (all ranks)", "achieved": gbs, "peak": peak * world,
                         "unit": "GB/s", "frac": gbs / (peak * world), "peak_source": peak_src, "traffic": None},
            "stage_us_eager": stage_us, "cpu_baseline": None}))
    # a CUDA graph that holds captured collectives must be gone before the communicator is
    # torn down, or the teardown waits for it forever
    graph.graph = None
    del graph
    torch.cuda.synchronize()
    dist.barrier()
    if exchange is not None:
        exchange.close()
        dist.barrier()
    dist.destroy_process_group()


# --------------------------------------------------------------------------- CPU arm

def run_cpu_reference(w, steps: int, warmup: int, quiet: bool = False):
    """Time the reference's CPU path on this host: dense entmax decode attention over the
    whole cache, Gaussian statistics + scalar tau solver, and key-range top-k selection.

    The sample is bounded: at most 4 batch rows of the workload at its real context
    length (the per-row cost is independent of the batch size), scaled to the full batch.
    """
    from entmaxkv_b200 import workloads
    from oracle import cache as ocache, dense as odense, gaussian as og, topk as otopk

    try:      # launchers such as torchrun pin OMP_NUM_THREADS to 1; the baseline gets every core it may use
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except Exception:
        pass
    rows = min(w.batch, 4)
    ws = type(w)(**{**w.__dict__, "batch": rows})
    inp = workloads.make_inputs(ws, device="cpu")
    S = max(inp["seq_lens"])
    P = w.page_size
    k = torch.cat([inp["k"][:, :, :S], inp["k_new"]], dim=2)
    v = torch.cat([inp["v"][:, :, :S], inp["v_new"]], dim=2)
    q = inp["q"]
    n_pages = (S + 1 + P - 1) // P
    # page statistics are prefill-time state, not part of the step
    kmin, kmax, kmean, kstd = ocache.page_stats(k, P)
    threads = torch.get_num_threads()

    def step():
        out = odense.dense_entmax_decode(q, k, v, w.alpha)
        sel = None
        if w.mode == "gaussian":
            mu, var, sigma = og.page_moments(q, kmean, kstd, n_pages - 1)
            mean, mv, vm = og.head_moments(mu, var)
            sg = og.global_sigma(mv, vm)
            sel = og.tau_hat(mean, sg, (n_pages - 1) * P, w.alpha)
        else:
            sc = otopk.criticality_scores(q, kmin, kmax)
            sel = otopk.topk_page_sets(sc, min(w.token_budget // P, n_pages - 1))
        return out, sel

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    scale = w.batch / rows
    return {"value": dt * scale * 1e6, "unit": UNIT, "cores": threads, "kind": "port",
            "host_cpus": os.cpu_count(),
            "sample": f"{steps} steps of {rows}/{w.batch} batch rows at full context {S + 1} "
                      f"(dense entmax decode + {'tau_hat' if w.mode == 'gaussian' else 'top-k selection'}), "
                      f"scaled x{scale:g}"}


def run_reference_arm(args):
    from entmaxkv_b200 import workloads
    rank, _, world = dist_env()
    if rank != 0:
        return
    w = workloads.CONFIGS[args.workload]
    K, W = args.steps, max(args.warmup, 1)
    K = min(K, 20)
    cb = run_cpu_reference(w, steps=K, warmup=min(W, 3))
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": world,
        "steps": K, "warmup": min(W, 3), "ms_per_step": cb["value"] / 1e3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "mode": w.mode, "batch_per_gpu": w.batch, "context": w.context},
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
        w = type(w)(**{**w.__dict__, "batch": args.batch})
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
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    flush_src = torch.zeros(512 << 18, dtype=torch.int32, device="cuda")
    K, W = args.steps, max(args.warmup, 3)
    for _ in range(W):
        step()
    torch.cuda.synchronize()
    times = []
    for _ in range(K):
        flush_buf.fill_(1)
        flush_src.max()
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
    ap.add_argument("--cpu-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch size (small profiling cases)")
    ap.add_argument("--token-budget", type=int, default=0,
                    help="override the top-k token budget (>= context: every page, i.e. dense entmax attention)")
    ap.add_argument("--alpha", type=float, default=0.0, help="override the workload's entmax alpha (side measurements)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="sequence-sharded mode: launch the step eagerly")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="sequence-sharded mode: reductions fused over peer memory (default) or NCCL all-reduces")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="single process: time one rank's 1/N shard of the sequence-sharded step alone")
    ap.add_argument("--no-stages", action="store_true", help="sequence-sharded mode: skip the per-stage timing")
    ap.add_argument("--no-extra", action="store_true", help="skip the side measurements of the other workloads")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.impl == "reference_triton":
        run_reference_triton(args)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU fallback")
        if args.workload == "million_gaussian" and (dist_env()[2] > 1 or args.emulate_world):
            run_gpu_sequence_sharded(args)
        else:
            run_gpu(args)


if __name__ == "__main__":
    main()
