#!/usr/bin/env python
"""Benchmark of the attention KV-cache path: decode attention tokens/s and KV-read GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (the one the headline metric is quoted on): GLM-4-9B-shaped batched decode, a 40-layer
attention stack, 32 q heads / 2 kv heads, head_dim 128, f16 caches of max_length 8192, 64 independent
sequences per GPU with n_past drawn uniformly from [1024, 8191] by a seed.  A step is one decode step of all
sequences through all 40 layers: 40 calls of cglm_attn_forward (fused RoPE + f16 append + attention).
Sequences are independent, so N GPUs hold 64 sequences each and exchange nothing (weak scaling).

Prints ONE JSON line (rank 0).  `value` is whole-job tokens/s with inputs resident in HBM; `e2e` is the
same metric through cglm_attn_forward_host with pinned host activations (H2D and D2H inside the timed
region); `roofline` is the decode kernel's KV bytes per launch over its measured duration against the
measured HBM copy bandwidth; `cpu_baseline` is the CPU restatement of the reference path timed on this
box's host cores on a bounded sample.  --impl reference times only that CPU path.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: H, G, D, max_length, layers, seqs per GPU, n_past range, rope, theta, interleaved, mask
    "glm4_9b_batched_decode": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=64, n_past=(1024, 8191), rope=8,
                                   theta=10000.0, interleaved=False, mask=0, seed=1003),
    # 1/20 of the default workload (2 layers, 1 GiB of caches): small enough for an ncu --set full capture
    "glm4_9b_batched_decode_small": dict(H=32, G=2, D=128, M=8192, layers=2, seqs=64, n_past=(1024, 8191), rope=8,
                                         theta=10000.0, interleaved=False, mask=0, seed=1003),
    # the default workload's layer call at other batch sizes: separates fixed per-launch cost from streaming rate
    "glm4_9b_batched_decode_b32": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=32, n_past=(1024, 8191), rope=8,
                                       theta=10000.0, interleaved=False, mask=0, seed=1003),
    "glm4_9b_batched_decode_b128": dict(H=32, G=2, D=128, M=8192, layers=20, seqs=128, n_past=(1024, 8191), rope=8,
                                        theta=10000.0, interleaved=False, mask=0, seed=1003),
    "glm3_6b_decode_512": dict(H=32, G=2, D=128, M=2048, layers=1, seqs=1, n_past=(512, 512), rope=8, theta=10000.0,
                               interleaved=False, mask=0, seed=1001),
    # BASELINE config 4: one sequence, KV length split over the GPUs, log-sum-exp combine after an all-gather
    "glm4_9b_long_131072": dict(H=32, G=2, D=128, M=131072 + 64, layers=1, seqs=1, n_past=(131072, 131072), rope=8,
                                theta=5.0e6, interleaved=False, mask=0, seed=1004, split_kv=True),
    # BASELINE config 2: one 1024-token prompt into an empty cache, causal; the tcgen05 path
    "glm3_6b_prefill_1024": dict(H=32, G=2, D=128, M=2048, layers=1, seqs=1, n_past=(0, 0), rope=8, theta=10000.0,
                                 interleaved=False, mask=0, seed=1002, prefill=1024),
    "glm1_6b_mha_decode": dict(H=32, G=32, D=128, M=4096, layers=28, seqs=4, n_past=(2048, 2048), rope=4,
                               theta=10000.0, interleaved=True, mask=1, seed=1005),
}
HBM_FALLBACK_GBS = 6650.0   # B200 copy bandwidth from an earlier measurement, used only without MEASURED_PEAKS.json
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic KV bytes of one decode launch, from the ncu capture of
# the _small workload, whose launches are identical to the default workload's (see profiles/): 316.5 MB / 303.5 MB.
NCU_TRAFFIC_PER_KV_BYTE = 1.043


def kv_bytes(w, n_past):
    """Algorithmic bytes of one layer call: K and V^T of every attended token, f16 (4*G*D*(n_past+1))."""
    return int(sum(4 * w["G"] * w["D"] * (p + 1) for p in n_past))


def draw_n_past(w, rank):
    rng = np.random.default_rng(w["seed"] + 7919 * rank)
    lo, hi = w["n_past"]
    return rng.integers(lo, hi + 1, w["seqs"]).astype(np.int32)


def qkv_row(w):
    return 3 * w["H"] * w["D"] if w["interleaved"] else (w["H"] + 2 * w["G"]) * w["D"]


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU during the timed region (read-only NVML queries)."""

    def __init__(self, index):
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
        names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                 nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.05)

    def finish(self):
        self._halt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def host_threads():
    return os.cpu_count() or 1


def cpu_leg(w, n_past, host_caches, steps, warmup):
    """Times the CPU oracle on one layer of the workload.  Returns (tokens/s scaled to all layers, seconds/layer)."""
    from oracle import attn_oracle as O
    cfg = O.make_cfg(w["H"], w["G"], w["D"], w["M"], 0, w["rope"], w["theta"], w["mask"], "ggml")
    rng = np.random.default_rng(w["seed"])
    n, H, G, D = len(n_past), w["H"], w["G"], w["D"]
    qkv = rng.standard_normal((n, qkv_row(w))).astype(np.float32)
    if w["interleaved"]:
        q = [qkv[i] for i in range(n)]; k = [qkv[i][D:] for i in range(n)]; v = [qkv[i][2 * D:] for i in range(n)]
        hs = 3 * D
    else:
        q = [qkv[i] for i in range(n)]; k = [qkv[i][H * D:] for i in range(n)]; v = [qkv[i][(H + G) * D:] for i in range(n)]
        hs = D
    kc = [c[0] for c in host_caches]
    vc = [c[1] for c in host_caches]
    n_ctx = np.maximum(n_past // 2, 2).astype(np.int32)
    thr = host_threads()
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        O.attn_decode_batch(cfg, q, k, v, hs, hs, kc, vc, n_past, n_ctx, n_threads=thr)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    per_layer = float(np.mean(times))
    return n / (per_layer * w["layers"]), per_layer, thr


def synth_host_caches(w, n_past, seed):
    """Host caches for the reference arm: N(0,1) f16 tiled from a 4M-value pool (fast to make, same distribution)."""
    rng = np.random.default_rng(seed)
    pool = rng.standard_normal(1 << 22).astype(np.float16).view(np.uint16)
    G, M, D = w["G"], w["M"], w["D"]
    out = []
    for i, p in enumerate(n_past):
        n = G * M * D
        off = (i * 104729) % (pool.size // 2)
        k = np.resize(pool[off:], n).reshape(G, M, D).copy()
        v = np.resize(pool[off + 17:], n).reshape(G, D, M).copy()
        out.append((k, v))
    return out


def run_reference(args, w):
    """--impl reference: the reference's CPU path (our CPU restatement of it: the reference's own arithmetic lives
    in the ggml submodule, which is absent and unpinned, so it cannot be compiled here)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_past = draw_n_past(w, 0)
    caches = synth_host_caches(w, n_past, w["seed"])
    # each step: one of the workload's layers over all sequences
    tps, per_layer, thr = cpu_leg(w, n_past, caches, args.steps, max(1, min(args.warmup, 3)))
    sample = f"1 of {w['layers']} layers x {w['seqs']} sequences per step, scaled to {w['layers']} layers"
    line = {
        "impl": "reference", "metric": "decode_attention_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_layer * w["layers"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(args, w, n_past),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": thr, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, w, n_past):
    return {"workload": args.workload, "n_head": w["H"], "n_kv_head": w["G"], "head_dim": w["D"],
            "max_length": w["M"], "layers": w["layers"], "seqs_per_gpu": w["seqs"],
            "global_batch": w["seqs"] * args.gpus, "n_past_range": list(w["n_past"]),
            "n_past_mean": float(np.mean(n_past)), "parallelism": f"sequence-sharded x{args.gpus}, no collective",
            "l2_policy": "inputs larger than L2 (each launch streams its own cache slabs; a step touches every layer's)"}


def run_split_kv(args, w):
    """Config 4: strong scaling of ONE long sequence.  Rank r holds a contiguous slice of the KV length in its own
    arena, runs the fused decode over it into an (acc, m, l) partial, the partials are all-gathered (NCCL) into
    every rank's memory and merged by the log-sum-exp combine kernel.  Each step rotates through enough copies of
    the slice that the working set is at least four times the L2."""
    import torch
    import torch.distributed as dist

    from chatglm_cpp_b200 import _lib, sharding
    from chatglm_cpp_b200 import attention as A

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = _lib.lib()
    H, G, D = w["H"], w["G"], w["D"]
    P = w["n_past"][0]
    sl = sharding.split_kv(P, 0, world, rank)
    cap = sharding.slice_capacity(P, 0, world) + 64
    desc = _lib.AttnDesc(H, G, D, cap, 0, w["rope"], w["theta"], w["mask"])
    local_bytes = 4 * G * D * (sl.n_local + (1 if sl.owns_new else 0))
    n_rot = max(2, int(np.ceil(4 * 126e6 / max(local_bytes, 1))))
    arena = A.KVArena(desc, n_rot)
    g = torch.Generator(device="cuda"); g.manual_seed(w["seed"] + rank)
    arena.k_all().view(-1).copy_(torch.randn(arena.k_all().numel(), device="cuda", generator=g).half())
    arena.v_all().view(-1).copy_(torch.randn(arena.v_all().numel(), device="cuda", generator=g).half())
    ws = A.Workspace(desc, 1, 1)
    g0 = torch.Generator(device="cuda"); g0.manual_seed(w["seed"])           # q is replicated on every rank
    qkv = torch.randn(1, qkv_row(w), device="cuda", generator=g0)
    partial = torch.zeros(H, D + 2, device="cuda")
    gathered = torch.zeros(world, H, D + 2, device="cuda")
    # Exchange of the partials: "p2p" = every rank stores its partial into every peer's exchange buffer over NVLink
    # (buffers mapped with CUDA IPC) and the combine waits for the arrival words; "nccl" = all-gather + combine.
    xchg = None
    if world > 1 and args.exchange == "p2p":
        # every kernel of the step runs once locally before the ranks meet (module loading happens here, not inside
        # the first bounded wait)
        solo = A.SplitKVExchange([A.SplitKVExchange.new_buffer(1, H, D)], 0, H, D)
        warm = (_lib.AttnSeq * 1)()
        A.fill_seq(warm[0], desc, A.SeqCall(qkv=qkv, slot=0, n_past=P, kv_local=sl.n_local,
                                            flags=_lib.SEQ_USE_KV_LOCAL | _lib.SEQ_NO_APPEND), False)
        solo.step(arena, ws, warm, torch.zeros(H * D, device="cuda"))
        torch.cuda.synchronize()
        mine, handle = A.SplitKVExchange.alloc_exported(world, H, D)
        handles = [None] * world
        dist.all_gather_object(handles, (local, handle))
        # imported with this rank's device current (the mapping must belong to the context whose kernels use it)
        peers = [mine if r == rank else A.SplitKVExchange.import_handle(handles[r][1], handles[r][0]) for r in range(world)]
        xchg = A.SplitKVExchange(peers, rank, H, D)
        dist.barrier()
    out = torch.zeros(1, H * D, device="cuda")
    settled = 0 if args.no_settled else _lib.SEQ_CACHE_SETTLED     # no step writes rows below n_past of any slot
    flags = settled | ((_lib.SEQ_USE_KV_LOCAL | (0 if sl.owns_new else _lib.SEQ_NO_APPEND)) if world > 1 else 0)
    if world > 1 and xchg is None:
        flags |= _lib.SEQ_PARTIAL
    arrs = []
    for s in range(n_rot):
        arr = (_lib.AttnSeq * 1)()
        A.fill_seq(arr[0], desc, A.SeqCall(qkv=qkv, slot=s, n_past=P, out=out if world == 1 else None,
                                           partial=partial if flags & _lib.SEQ_PARTIAL else None,
                                           kv_local=sl.n_local if world > 1 else 0, flags=flags), False)
        arrs.append(arr)
    it = [0]
    timeout_us = 50000   # a rank that is more than 50 ms behind is treated as gone

    def step():
        """One decode step of the long sequence.  1 GPU: one fused decode launch.  N GPUs, peer stores: one fused launch
        per rank (attention over the slice + exchange + combine).  N GPUs, NCCL: decode, all-gather, combine kernel."""
        stream = torch.cuda.current_stream().cuda_stream
        arr = arrs[it[0] % n_rot]
        it[0] += 1
        if xchg is not None:
            xchg.step(arena, ws, arr, out, combine=True, timeout_us=timeout_us)
            return
        rc = L.cglm_attn_forward(arena._h, arr, 1, ws.ptr, ws.bytes, stream)
        if rc != 0:
            raise _lib.CglmError(rc, "cglm_attn_forward")
        if world > 1:
            dist.all_gather_into_tensor(gathered, partial)
            A.splitkv_combine(gathered, out.view(-1))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    st = ws.status()
    if st != 0:   # e.g. a peer's partial never arrived: every further step would run into the same bounded wait
        raise SystemExit(f"[rank {rank}] device-side status {st} after the warm-up steps")
    # A step is three launches (decode over the slice, all-gather, combine) of 20-50 us in total: issued one by one
    # from Python the host is the bottleneck, so one pass over the rotating slices is captured in a CUDA graph and
    # the timed region replays it.  --no-graph times the eager loop instead.
    graph = None
    steps = args.steps
    launches_per_step = 1 if (xchg is not None or world == 1) else 2   # this library's kernels: decode (+ combine)
    if not args.no_graph:
        it[0] = 0
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                step()
        torch.cuda.current_stream().wait_stream(side)
        barrier()
        it[0] = 0
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(n_rot):
                step()
        replays = max(1, (args.steps + n_rot - 1) // n_rot)
        steps = replays * n_rot
        for _ in range(2):
            graph.replay()
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local); sampler.start()
    e0.record()
    if graph is not None:
        for _ in range(replays):
            graph.replay()
    else:
        for _ in range(steps):
            step()
    e1.record()
    barrier()
    clocks = sampler.finish()
    launches = steps * launches_per_step
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if ws.status() != 0:
        raise SystemExit("device-side status is not clean after the timed region")
    peak, peak_src = HBM_FALLBACK_GBS, "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, peak_src = float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        pass
    if rank == 0:
        step_ms = ms / steps
        achieved = local_bytes / (step_ms * 1e-3) / 1e9
        line = {
            "metric": "decode_attention_tokens_per_s", "value": steps / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "n_head": H, "n_kv_head": G, "head_dim": D, "n_past": P,
                       "kv_bytes_total": 4 * G * D * (P + 1), "kv_bytes_this_rank": local_bytes,
                       "parallelism": ("one GPU, one fused decode launch per step" if world == 1 else
                                       f"KV length split x{world}, " +
                                       ("one fused launch per rank: attention + peer stores of the partial rows + LSE combine"
                                        if xchg is not None else "decode + NCCL all-gather + combine kernel") +
                                       f", {H * (D + 2) * 4} B per rank"),
                       "l2_policy": f"rotates through {n_rot} copies of the slice (working set >= 4 x L2)",
                       "issue": "eager" if graph is None else f"CUDA graph of {n_rot} steps, replayed"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "kernel": "decode_kernel (the step time includes the exchange and the combine)",
                         "algorithmic_bytes_per_launch": local_bytes, "launch_us": step_ms * 1e3, "traffic": None},
            "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches) * world, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # a captured graph holds the communicator's resources: release it before the group goes away, and do not let
        # a slow teardown outlive the measurement
        graph = None
        torch.cuda.synchronize()
        killer = threading.Timer(30.0, lambda: os._exit(0))
        killer.daemon = True
        killer.start()
        dist.barrier()
        dist.destroy_process_group()
        killer.cancel()


def run_prefill(args, w):
    """Config 2: a step is one prefill call (RoPE + f16 cache write + causal attention over the prompt).  Slots
    rotate so that consecutive steps do not reuse a warm cache slab; q/k/v activations (f32) and the output are
    re-read / re-written every step by construction."""
    import torch

    from chatglm_cpp_b200 import _lib
    from chatglm_cpp_b200 import attention as A

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    L = _lib.lib()
    H, G, D, S = w["H"], w["G"], w["D"], w["prefill"]
    desc = _lib.AttnDesc(H, G, D, w["M"], 0, w["rope"], w["theta"], w["mask"])
    n_rot = 16
    arena = A.KVArena(desc, n_rot)
    ws = A.Workspace(desc, 1, S)
    g = torch.Generator(device="cuda"); g.manual_seed(w["seed"])
    qkv = [torch.randn(S, qkv_row(w), device="cuda", generator=g) for _ in range(n_rot)]
    out = [torch.empty(S, H * D, device="cuda") for _ in range(n_rot)]
    arrs = []
    for s in range(n_rot):
        arr = (_lib.AttnSeq * 1)()
        A.fill_seq(arr[0], desc, A.SeqCall(qkv=qkv[s], slot=s, n_past=0, out=out[s]), False)
        arrs.append(arr)
    stream = torch.cuda.current_stream().cuda_stream
    it = [0]

    def step():
        rc = L.cglm_attn_forward(arena._h, arrs[it[0] % n_rot], 1, ws.ptr, ws.bytes, stream)
        if rc != 0:
            raise _lib.CglmError(rc, "cglm_attn_forward")
        it[0] += 1

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0); sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = L.cglm_launch_count()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.finish()
    ms = e0.elapsed_time(e1) / args.steps
    if ws.status() != 0:
        raise SystemExit("device-side status is not clean after the timed region")
    flops = 4.0 * H * D * S * (S + 1) / 2          # useful (causal) FLOPs of QK^T and PV
    peak, peak_src = 1590.0, "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, peak_src = float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        pass
    achieved = flops / (ms * 1e-3) / 1e12
    line = {"metric": "prefill_attention_tokens_per_s", "value": S / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "n_head": H, "n_kv_head": G, "head_dim": D, "prompt_tokens": S,
                       "l2_policy": f"rotates through {n_rot} slots and activation buffers (560 MB)"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": peak_src, "kernel": "prefill_prepare_kernel + prefill_attn_kernel (whole call)",
                         "useful_flops_per_call": flops, "traffic": None},
            "cpu_baseline": None, "e2e": None, "gpu_launches": int(L.cglm_launch_count() - launches0), "clocks": clocks}
    print(json.dumps(line), flush=True)


def run_ours(args, w):
    if w.get("split_kv"):
        return run_split_kv(args, w)
    if w.get("prefill"):
        return run_prefill(args, w)
    import torch
    import torch.distributed as dist

    from chatglm_cpp_b200 import _lib
    from chatglm_cpp_b200 import attention as A

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = _lib.lib()
    H, G, D, M, layers, n = w["H"], w["G"], w["D"], w["M"], w["layers"], w["seqs"]
    desc = _lib.AttnDesc(H, G, D, M, 0, w["rope"], w["theta"], w["mask"])
    n_past = draw_n_past(w, rank)
    n_ctx = np.maximum(n_past // 2, 2).astype(np.int32)

    # ---- state: caches for every (layer, sequence), filled with N(0,1) f16 on the device ------------------
    arena = A.KVArena(desc, layers * n)
    g = torch.Generator(device="cuda")
    g.manual_seed(w["seed"] + rank)
    for view in (arena.k_all(), arena.v_all()):
        flat = view.view(-1)
        step = 1 << 28
        for o in range(0, flat.numel(), step):
            seg = flat[o:o + step]
            seg.copy_(torch.randn(seg.numel(), device="cuda", generator=g, dtype=torch.float32).half())
    ws = A.Workspace(desc, n, 1)
    row, orow = qkv_row(w), H * D
    qkv_dev = torch.randn(layers, n, row, device="cuda", generator=g)
    out_dev = torch.empty(layers, n, orow, device="cuda")
    qkv_host = qkv_dev.cpu().pin_memory()
    out_host = torch.empty(layers, n, orow).pin_memory()
    n_stage = 3   # staging pairs rotated over the layers so that a layer's copies overlap its neighbours' kernels
    stage_qkv = [torch.empty(n, row, device="cuda") for _ in range(n_stage)]
    stage_out = [torch.empty(n, orow, device="cuda") for _ in range(n_stage)]

    # one descriptor array per layer, built once: slot of (layer l, sequence i) is l*n + i.  Every layer call reads
    # cache rows that no kernel of the step writes (a call appends at n_past of its own layer's slots only), which is
    # what CGLM_SEQ_CACHE_SETTLED promises: a launch may stream cache tiles while the previous layer's launch drains.
    seq_flags = 0 if args.no_settled else _lib.SEQ_CACHE_SETTLED
    seq_arrays = []
    for l in range(layers):
        arr = (_lib.AttnSeq * n)()
        for i in range(n):
            call = A.SeqCall(qkv=qkv_dev[l, i:i + 1], slot=l * n + i, n_past=int(n_past[i]), n_ctx=int(n_ctx[i]),
                             out=out_dev[l, i:i + 1], flags=seq_flags)
            A.fill_seq(arr[i], desc, call, w["interleaved"])
        seq_arrays.append(arr)
    stream = torch.cuda.current_stream().cuda_stream

    def step_device():
        for l in range(layers):
            rc = L.cglm_attn_forward(arena._h, seq_arrays[l], n, ws.ptr, ws.bytes, stream)
            if rc != 0:
                raise _lib.CglmError(rc, "cglm_attn_forward")

    def step_host():
        for l in range(layers):
            rc = L.cglm_attn_forward_host(arena._h, seq_arrays[l], n, int(w["interleaved"]), qkv_host[l].data_ptr(),
                                          out_host[l].data_ptr(), stage_qkv[l % n_stage].data_ptr(),
                                          stage_out[l % n_stage].data_ptr(), ws.ptr, ws.bytes, stream)
            if rc != 0:
                raise _lib.CglmError(rc, "cglm_attn_forward_host")
        rc = L.cglm_attn_host_drain(arena._h, stream)   # the step's results are read back here
        if rc != 0:
            raise _lib.CglmError(rc, "cglm_attn_host_drain")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = L.cglm_launch_count()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, L.cglm_launch_count() - launches0

    sampler = ClockSampler(local)
    sampler.start()
    ms, launches = timed(step_device, args.steps, args.warmup)
    clocks = sampler.finish()
    if ws.status() != 0:
        raise SystemExit("device-side status is not clean after the timed region")
    ms_e2e, _ = timed(step_host, max(3, args.steps // 2), max(3, args.warmup))
    e2e_steps = max(3, args.steps // 2)

    # Optional: the same step issued as ONE CUDA graph whose layer calls read n_past from device words
    # (CGLM_SEQ_N_PAST_DEVICE), the form a caller uses to replay a decode step for every new token without rebuilding
    # anything.  The words are advanced by 0 here so that every replay is the step the other figures measure.
    step_graph = None
    if args.step_graph:
        n_past_dev = torch.tensor([int(p) for p in n_past], dtype=torch.int32, device="cuda")
        dyn_arrays = []
        for l in range(layers):
            arr = (_lib.AttnSeq * n)()
            for i in range(n):
                call = A.SeqCall(qkv=qkv_dev[l, i:i + 1], slot=l * n + i, n_past=int(n_past[i]), n_ctx=int(n_ctx[i]),
                                 out=out_dev[l, i:i + 1], flags=_lib.SEQ_N_PAST_DEVICE, n_past_dev=n_past_dev[i:i + 1])
                A.fill_seq(arr[i], desc, call, w["interleaved"])
            dyn_arrays.append(arr)

        def step_dyn():
            st = torch.cuda.current_stream().cuda_stream
            for l in range(layers):
                rc = L.cglm_attn_forward(arena._h, dyn_arrays[l], n, ws.ptr, ws.bytes, st)
                if rc != 0:
                    raise _lib.CglmError(rc, "cglm_attn_forward")
            rc = L.cglm_seq_advance(n_past_dev.data_ptr(), n, 0, st)
            if rc != 0:
                raise _lib.CglmError(rc, "cglm_seq_advance")

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step_dyn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step_dyn()
        ms_graph, _ = timed(graph.replay, args.steps, args.warmup)
        if ws.status() != 0:
            raise SystemExit("device-side status is not clean after the step-graph region")
        step_graph = {"value": n * world * args.steps / (ms_graph * 1e-3), "unit": "tokens/s",
                      "ms_per_step": ms_graph / args.steps, "launches_per_step": layers + 1,
                      "note": "one CUDA graph per decode step, n_past read from device words, replayed"}
        graph = None

    tokens_per_step = n * world
    value = tokens_per_step * args.steps / (ms * 1e-3)
    e2e_value = tokens_per_step * e2e_steps / (ms_e2e * 1e-3)
    bytes_per_launch = kv_bytes(w, n_past)
    launch_ms = ms / (args.steps * layers)
    achieved = bytes_per_launch / (launch_ms * 1e-3) / 1e9
    peak, peak_src = HBM_FALLBACK_GBS, "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, peak_src = float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        pass

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        # bounded sample: layer 0 of the same workload, with the device's cache contents
        torch.cuda.synchronize()
        host_caches = [(arena.k_cache(i).cpu().numpy().view(np.uint16), arena.v_cache(i).cpu().numpy().view(np.uint16))
                       for i in range(n)]
        tps, per_layer, thr = cpu_leg(w, n_past, host_caches, 3, 1)
        cpu = {"value": tps, "unit": "tokens/s", "cores": thr, "kind": "port",
               "sample": f"layer 0 of {layers} x {n} sequences (same cache bits), 3 repetitions, scaled to {layers} layers"}

    if rank == 0:
        line = {
            "metric": "decode_attention_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args, w, n_past),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "kernel": "decode_kernel",
                         "algorithmic_bytes_per_launch": bytes_per_launch, "launch_us": launch_ms * 1e3,
                         "traffic": (NCU_TRAFFIC_PER_KV_BYTE * bytes_per_launch
                                     if NCU_TRAFFIC_PER_KV_BYTE is not None else None),
                         "frac_of_nominal_8000": achieved / 8000.0},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / e2e_steps,
                    "h2d_bytes_per_step": layers * n * row * 4, "d2h_bytes_per_step": layers * n * orow * 4},
            "gpu_launches": int(launches) * world,
            "clocks": clocks,
        }
        if step_graph is not None:
            line["step_graph"] = step_graph
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="glm4_9b_batched_decode")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-settled", action="store_true",
                    help="decode workloads: do not pass CGLM_SEQ_CACHE_SETTLED (every launch waits for the previous one to drain)")
    ap.add_argument("--no-graph", action="store_true", help="split-KV workload: issue every step eagerly")
    ap.add_argument("--exchange", choices=["p2p", "nccl"], default="p2p", help="split-KV workload: how partials travel")
    ap.add_argument("--step-graph", action="store_true",
                    help="batched decode workloads: also time the step as one replayed CUDA graph (device-side n_past)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
