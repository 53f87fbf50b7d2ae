#!/usr/bin/env python3
"""Benchmark of the decode-time top-k sparse-attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2|cfg2_shared|cfg0|cfg1|cfg3|cfg4]

One step = one decode step of the fused path (scan K, exact top-k, softmax over the kept keys,
mix V) on synthetic inputs of the headline configuration: batch 4, 32 heads, head_dim 128,
context 131072, top-k 2048, fp16, one cache per batch row with 2 % planted keys.  Prints one JSON
line.  `value` is tokens scanned per second with the caches resident in HBM; `e2e` is the same
quantity through the public operator with the step's query coming from pinned host memory and
its output read back to the host inside the timed region (the KV cache is decode state that
lives in HBM across steps, like weights, so it is not re-uploaded per step).

With --gpus N > 1 (launched under torchrun, one rank per GPU) the context is sharded by tokens:
every rank holds a 131072-token shard of every sequence (weak scaling), proposes its local
top-k, candidates are merged over NCCL and partial outputs are combined through their
log-sum-exp.  `--impl reference` times the CPU oracle (the reference's torch path) on the host
cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


class nvtx_range:
    """NVTX range around one phase of the harness, the way the reference's profiling scripts mark
    theirs (torch_topk_nvtx.py:102-123, baseline_1.py:32-41,133-143)."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self):
        self._halt.set()
        self.join(timeout=1.0)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


def make_workload(name: str, device):
    from topk_attn_b200 import workloads as W
    if name == "cfg2":
        return W.fused_topk_128k(device=device)
    if name == "cfg2_n32k":      # the headline geometry at a quarter of the context (profiling)
        return W.fused_topk_128k(device=device, n=32768)
    if name == "cfg2_shared":
        return W.fused_topk_128k(device=device, shared_cache=True)
    if name == "cfg2_shared_n32k":   # the shared-cache geometry at a quarter of the context (profiling)
        return W.fused_topk_128k(device=device, shared_cache=True, n=32768)
    if name == "cfg0":
        return W.reference_cpu_case(device=device)
    if name == "cfg1":
        w = W.dense_flash_decoding(device=device)
        w.sm_scale = 1.0
        return w
    if name == "cfg1_shared":
        return W.dense_flash_decoding(device=device, shared_cache=True)
    if name == "cfg3":
        w = W.centroid_retrieval(device=device)
        w.sm_scale = 1.0
        return w
    if name == "cfg4":
        return W.sharded_long_context_shard(0, 1, device=device)
    if name == "legacy":         # the reference extension's own test shape: 4 chunks of 2048, top-128 each
        w = W.legacy_test_case(device=device)
        w.topk, w.num_segments = 128, 4
        return w
    raise SystemExit(f"workload {name} is not available in this bench")


def cpu_sample(workload: str):
    """A bounded sample of the workload for the CPU oracle: one batch row."""
    from topk_attn_b200 import workloads as W
    if workload in ("cfg2", "cfg2_shared", "cfg2_n32k", "cfg2_shared_n32k"):
        return W.fused_topk_128k(device="cpu", batch=1), "one batch row of cfg2 (N=131072, 32 heads, k=2048)"
    if workload == "cfg0":
        return W.reference_cpu_case(), "cfg0 in full"
    if workload == "cfg4":
        return (W.sharded_long_context_shard(0, 8, device="cpu"),
                "one eighth of cfg4 (131072 tokens, 32 q / 8 kv heads, k=4096)")
    if workload in ("cfg1", "cfg1_shared"):
        return W.dense_flash_decoding(device="cpu", batch=1), "one batch row of cfg1 (N=32768, 32 q / 8 kv heads)"
    if workload == "cfg3":
        return W.centroid_retrieval(device="cpu"), "cfg3 in full"
    if workload == "legacy":
        w = W.legacy_test_case()
        w.topk, w.num_segments = 128, 4
        return w, "the extension's test shape in full (B=4, N=8192, 4 chunks, top-128)"
    raise SystemExit(f"no CPU sample for {workload}")


def time_cpu_oracle(w, repeats: int):
    from oracle import topk_attn_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        if w.num_splits:
            O.split_kv_attention(w.q, w.k, w.v, w.sm_scale, w.num_splits)
        elif w.centers is not None:
            O.center_only_attention(w.q, w.centers, w.k, w.v, w.topc, w.clen, w.sm_scale)
        else:
            O.topk_sparse_attention(w.q, w.k, w.v, w.topk, w.sm_scale, w.num_segments)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w, what = cpu_sample(args.workload)
    for _ in range(min(args.warmup, 1)):
        time_cpu_oracle(w, 1)
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    times = [time_cpu_oracle(w, 1) for _ in range(steps)]
    total = time.perf_counter() - t0
    per = sum(times) / len(times)
    tokens = w.batch * w.n_tokens
    val = tokens / per
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "tokens_scanned_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "sample": what},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": what},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "wall_s": total,
    }
    print(json.dumps(line))


def run_center_published(args):
    """The one workload the reference publishes numbers for (a source comment,
    center_only_topk/gemv_topk.cu:2-7): centroid-only selection, H=32, D=128, 1024 centroids per head,
    keep the top 64, expand to 64 x 128 = 8192 token ids per head; average latency of back-to-back
    launches after warm-ups, inputs left warm in L2 exactly as the reference's timing loop leaves
    them (:546-575).  Published: 16.401 us (sm_90, 5-CTA cluster) ... 24.594 us (sm_90, one CTA)."""
    from topk_attn_b200 import ops, workloads as W
    dev = torch.device("cuda", 0)
    w = W.centroid_retrieval(device=dev, csz=1024, clen=128, topc=64)
    q, centers = w.q, w.centers
    for _ in range(max(args.warmup, 10)):
        ops.center_only_topk(q, centers, 64, 128)
    ops.check_status(dev)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    # one graph holds `inner` back-to-back steps: replaying a one-launch graph from Python takes
    # longer than the launch itself, and the reference's loop is back-to-back launches from C++
    inner = 50
    replays = max(1, args.steps // inner)
    from topk_attn_b200 import capi
    c0 = capi.lib().ra_launch_count()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(inner):
                ops.center_only_topk(q, centers, 64, 128)
    launches_per_step = (capi.lib().ra_launch_count() - c0) // inner
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    steps = replays * inner
    us = e0.elapsed_time(e1) * 1e3 / steps
    published = 16.401
    print(json.dumps({
        "metric": "centroid_only_selection_latency", "value": us, "unit": "us", "n_gpus": 1,
        "steps": steps, "warmup": max(args.warmup, 10), "ms_per_step": us * 1e-3,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": us / published,
        "dtype": "f16 inputs, f32 accumulate", "data": "synthetic",
        "config": {"workload": "center_pub", "heads": 32, "head_dim": 128, "centroids": 1024,
                   "top_clusters": 64, "cluster_len": 128, "l2": "warm, as in the reference's loop",
                   "published_us": {"sm_90 cluster": 16.401, "sm_120a cluster": 18.446,
                                    "sm_120a single CTA": 20.561, "sm_90 single CTA": 24.594}},
        "gpu_launches": steps * launches_per_step}))


def phase_breakdown(step, steps):
    """Where the time of the fused kernel goes, in the manner of the reference's split profile
    (gemv_profile_split.cu: GEMV alone, then with the selection): the same launch repeated with
    parts of the kernel switched off through the library's RA_DEBUG_FLAGS tuning aid (1 = no
    scoring, 4 = no list appends, 8 = no list cuts, 16 = return before select + softmax.V).  The
    outputs of those launches are meaningless; only their durations are used.  The switches exist
    only in the tuning build of the library, which these launches go through."""
    from topk_attn_b200 import capi

    def timed(flags):
        if flags:
            os.environ["RA_DEBUG_FLAGS"] = str(flags)
        else:
            os.environ.pop("RA_DEBUG_FLAGS", None)
        with capi.tuning_library(), nvtx_range(f"phase flags={flags}"):
            for _ in range(3):
                step()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(steps):
                step()
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / steps
    try:
        stream = timed(1 | 4 | 8 | 16)
        score = timed(4 | 8 | 16)
        select = timed(16)
    finally:
        os.environ.pop("RA_DEBUG_FLAGS", None)
    full = timed(0)
    return {"stream_only_us": stream, "stream_score_us": score, "stream_score_select_us": select,
            "full_step_us": full, "attend_us": full - select,
            "note": "each figure is a whole launch with the later parts switched off"}


def run_ours(args):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    if args.workload == "center_pub":
        return run_center_published(args)
    from topk_attn_b200 import ops
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    if world > 1:
        from topk_attn_b200 import sharded
        return sharded.bench(args, rank, local, world, ClockSampler, measured_peak_gbs)

    w = make_workload(args.workload, dev)
    q, k, v = w.q, w.k, w.v
    out = torch.empty_like(q)
    kind = "dense" if w.num_splits else ("centroid" if w.centers is not None else "topk")
    kernel_name = {"dense": "flash_decode_kernel", "centroid": "center_attend_kernel",
                   "topk": "scan_select_kernel"}[kind]
    if args.workload == "legacy":
        kernel_name = "dense_select_kernel + gather_flash_kernel"
    if args.workload in ("cfg2_shared", "cfg2_shared_n32k", "cfg4"):
        kernel_name = "scan_store_kernel + select_stored_kernel"

    def op(q_in):
        if kind == "dense":
            ops.flash_decoding(q_in, k, v, w.sm_scale, w.num_splits, out=out)
        elif kind == "centroid":
            ops.center_only_topk(q_in, w.centers, w.topc, w.clen, k, v, w.sm_scale, out=out)
        else:
            ops.topk_attention(q_in, k, v, w.topk, w.sm_scale, w.num_segments, out=out)

    def step():
        op(q)

    from topk_attn_b200 import capi
    count = capi.lib().ra_launch_count                # kernels launched by the library so far
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    with nvtx_range("warmup"):
        # the asked-for warm-up steps, then more until the GPU has been busy for 0.3 s, so that the
        # clock sampler sees the clocks under load even when the timed region is short
        t_w = time.perf_counter()
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        while time.perf_counter() - t_w < 0.3:
            for _ in range(10):
                step()
            torch.cuda.synchronize()
    ops.check_status(dev)
    torch.cuda.synchronize()
    small = w.algorithmic_bytes() <= (256 << 20)     # would sit in the 126 MB L2
    if not small:
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        torch.cuda.synchronize()
        c0 = count()
        with nvtx_range("timed steps"):
            evs[0].record()
            for i in range(args.steps):
                step()
                evs[i + 1].record()
            torch.cuda.synchronize()
        gpu_launches = count() - c0
        clocks = sampler.stop()
        total_ms = evs[0].elapsed_time(evs[-1])
        per_ms = total_ms / args.steps
        launch_ms = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps))
        l2_note = "inputs_exceed_l2"
    else:
        # Inputs fit in L2: every step is replayed from a CUDA graph (one step is a few tens of
        # microseconds, less than the host needs to issue it) and L2 is flushed by overwriting a
        # 512 MB buffer between steps; only the step itself sits between the two events.
        flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            if args.consecutive:
                # consecutive decode steps of one sequence: the cache is asked to persist in L2
                ops.l2_persist(w.centers if kind == "centroid" else k)
            step()
            c0 = count()
            with torch.cuda.graph(graph, stream=side):
                step()
            gpu_launches = (count() - c0) * args.steps   # every replay runs the captured launches
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                 for _ in range(args.steps)]
        with nvtx_range("timed steps"):
            for a, bq in pairs:
                if not args.consecutive:
                    flush.fill_(1)
                a.record()
                graph.replay()
                bq.record()
            torch.cuda.synchronize()
        clocks = sampler.stop()
        launch_ms = sorted(a.elapsed_time(bq) for a, bq in pairs)
        per_ms = sum(launch_ms) / len(launch_ms)
        l2_note = ("consecutive steps, no flush, cache persisting in L2 (ra_l2_persist), "
                   "step replayed from a CUDA graph") if args.consecutive else \
            "l2_flushed_between_steps (512 MB overwrite), step replayed from a CUDA graph"
        if args.consecutive:
            with torch.cuda.stream(side):
                ops.l2_persist(None)
    ops.check_status(dev)

    # what this GPU delivers to a kernel that only reads (the copy figure of the roofline reads and
    # writes): one read-only stream over the key cache, when it is much larger than L2
    read_gbs = None
    if not small:
        for _ in range(2):
            ops.stream_read_probe(k)
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(5):
            ops.stream_read_probe(k)
        r1.record()
        torch.cuda.synchronize()
        read_gbs = 5 * k.numel() * 2 / (r0.elapsed_time(r1) * 1e-3) / 1e9

    # end to end: query from pinned host memory, output read back, every step
    q_host = q.cpu().pin_memory()
    out_host = torch.empty_like(q_host).pin_memory()
    q_dev = torch.empty_like(q)
    e2e_steps = args.steps

    def e2e_step():
        q_dev.copy_(q_host, non_blocking=True)
        op(q_dev)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    with nvtx_range("end-to-end steps"):
        for _ in range(3):
            e2e_step()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_s = (time.perf_counter() - t0) / e2e_steps

    tokens = w.batch * w.n_tokens
    alg_bytes = w.algorithmic_bytes()
    peak, peak_kind = measured_peak_gbs()
    achieved = alg_bytes / (per_ms * 1e-3) / 1e9

    if args.no_cpu:
        cw, what, cpu_t = None, "skipped (--no-cpu)", None
    else:
        cw, what = cpu_sample(args.workload)
        with nvtx_range("cpu baseline"):
            cpu_t = time_cpu_oracle(cw, 2)
    line = {
        "metric": "tokens_scanned_per_s", "value": tokens / (per_ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": per_ms, "us_per_step": per_ms * 1e3,
        "us_per_step_median": launch_ms[len(launch_ms) // 2] * 1e3,
        "us_per_step_min": launch_ms[0] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 inputs, f32 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "batch": w.batch, "heads_q": q.size(1),
                   "heads_kv": k.size(-2), "head_dim": 128, "context": w.n_tokens,
                   "topk": w.topk, "caches": w.bkv, "l2": l2_note},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": peak_kind + " (burst copy)",
                     "algorithmic_bytes": alg_bytes, "traffic": None,
                     "kernel": kernel_name,
                     "read_only_stream_gbs": read_gbs,
                     "frac_of_read_only_stream": (achieved / read_gbs) if read_gbs else None,
                     "ms_x_sm_mhz": per_ms * clocks["sm_mhz"] if clocks.get("sm_mhz") else None},
        "cpu_baseline": {"value": (cw.batch * cw.n_tokens / cpu_t) if cw is not None else None,
                         "unit": "tokens/s",
                         "cores": torch.get_num_threads(), "kind": "port", "sample": what},
        "e2e": {"value": tokens / e2e_s, "unit": "tokens/s", "us_per_step": e2e_s * 1e6,
                "h2d_bytes_per_step": q_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2},
        "gpu_launches": gpu_launches,
        "clocks": clocks,
    }
    if args.phases:
        if kind != "topk" or small or gpu_launches != args.steps:
            line["phases"] = "only for a step that is one launch of the fused kernel"
        else:
            line["phases"] = phase_breakdown(step, min(args.steps, 50))
            ops.check_status(dev)
    traffic_file = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(traffic_file):
        try:
            t = json.load(open(traffic_file)).get(args.workload)
            if isinstance(t, dict):
                line["roofline"]["traffic"] = t.get("bytes")
                line["roofline"]["traffic_source"] = t.get("source")
            else:
                line["roofline"]["traffic"] = t
        except Exception:
            pass
    if args.workload == "cfg2" and not args.no_cfg4:
        # configuration 4 on this one GPU: the base of the strong-scaling series that
        # `--gpus 2|4|8` continues; same record, same on-device check of the result
        from topk_attn_b200 import sharded
        del w, q, k, v, out, q_dev
        torch.cuda.empty_cache()
        with nvtx_range("cfg4 on one GPU"):
            line["cfg4_strong"] = sharded.bench_long_context(0, 1, dev, min(args.steps, 100),
                                                             args.warmup, peak)
        if not line["cfg4_strong"]["parity"]["ok"]:
            print(json.dumps(line))
            raise SystemExit("parity check of configuration 4 failed: " +
                             json.dumps(line["cfg4_strong"]["parity"]))
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling)")
    ap.add_argument("--consecutive", action="store_true",
                    help="small workloads: time consecutive decode steps of one sequence (no L2 flush, "
                         "the cache marked persisting in L2) instead of cold steps")
    ap.add_argument("--collectives", action="store_true",
                    help="multi-GPU: exchange through NCCL all-gathers instead of peer stores")
    ap.add_argument("--candidates", action="store_true",
                    help="multi-GPU, configuration 4: exchange candidate lists instead of histograms")
    ap.add_argument("--no-cfg4", action="store_true",
                    help="skip the configuration-4 strong-scaling record that follows the headline run")
    ap.add_argument("--phases", action="store_true",
                    help="also time the fused kernel with selection / attention switched off; on several "
                         "GPUs: per-rank phase times of the histogram route's selection kernel (tuning build)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
