#!/usr/bin/env python
"""Benchmark of the attention KV-cache path: decode attention tokens/s and KV-read GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline workload (the one the metric is quoted on): GLM-4-9B-shaped batched decode, a 40-layer attention stack,
32 q heads / 2 kv heads, head_dim 128, f16 caches of max_length 8192, 64 independent sequences per GPU with n_past
drawn uniformly from [1024, 8191] by a seed.  A step is one decode step of all sequences through all 40 layers:
40 calls of cglm_attn_forward (fused RoPE + f16 append + attention).

Prints ONE JSON line (rank 0).  `value` is whole-job tokens/s with inputs resident in HBM; `e2e` is the same metric
through cglm_attn_forward_host with pinned host activations (H2D and D2H inside the timed region); `roofline` is the
decode kernel's KV bytes per launch over its measured duration against the measured HBM copy bandwidth;
`cpu_baseline` is the CPU restatement of the reference path timed on this box's host cores on a bounded sample, and
`parity` compares that sample's outputs and cache rows with what the timed GPU launches produced.  With the default
workload the line also carries `configs` (the other benchmark configurations, short runs), `step_graph`, and under
N > 1 GPUs `strong` (the 64 sequences sharded over the GPUs) and `split_kv` (one 131072-token sequence cut along its
KV length, fused exchange).  --impl reference times only the CPU path.

All inputs are synthetic: counter-based N(0,1) values (cglm_synth_fill_* on the device, oracle_synth_fill_* on the
host: the same bits), shaped after the model configurations named in the workloads.
"""
from __future__ import annotations

import argparse
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
    "glm4_9b_batched_decode_b16": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=16, n_past=(1024, 8191), rope=8,
                                       theta=10000.0, interleaved=False, mask=0, seed=1003),
    "glm4_9b_batched_decode_b8": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=8, n_past=(1024, 8191), rope=8,
                                      theta=10000.0, interleaved=False, mask=0, seed=1003),
    "glm4_9b_batched_decode_b128": dict(H=32, G=2, D=128, M=8192, layers=20, seqs=128, n_past=(1024, 8191), rope=8,
                                        theta=10000.0, interleaved=False, mask=0, seed=1003),
    # every sequence at the end of its cache: the condition the 70 %-of-HBM target is quoted on (n_past >= 8k)
    "glm4_9b_batched_decode_8k": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=64, n_past=(8191, 8191), rope=8,
                                      theta=10000.0, interleaved=False, mask=0, seed=1003),
    # benchmark configuration 1: one sequence at n_past 512; 64 "layers" so that consecutive launches stream different slabs
    "glm3_6b_decode_512": dict(H=32, G=2, D=128, M=2048, layers=64, seqs=1, n_past=(512, 512), rope=8, theta=10000.0,
                               interleaved=False, mask=0, seed=1001),
    # benchmark configuration 4: one sequence; with N GPUs the KV length is split and the partials are exchanged over NVLink
    "glm4_9b_long_131072": dict(H=32, G=2, D=128, M=131072 + 64, layers=1, seqs=1, n_past=(131072, 131072), rope=8,
                                theta=5.0e6, interleaved=False, mask=0, seed=1004, split_kv=True),
    # benchmark configuration 2: one 1024-token prompt into an empty cache, causal; the tcgen05 path
    "glm3_6b_prefill_1024": dict(H=32, G=2, D=128, M=2048, layers=1, seqs=1, n_past=(0, 0), rope=8, theta=10000.0,
                                 interleaved=False, mask=0, seed=1002, prefill=1024),
    # the query_key_value Linear in front of the path, fused with RoPE and the K/V append (decode-sized batch; a step is the
    # 40 layers' Linears, every layer its own 37.7 MB f16 weight, so the weights stream from HBM)
    "glm4_9b_qkv_linear_b64": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=64, n_past=(1024, 8191), rope=8, theta=5.0e6,
                                   interleaved=False, mask=0, seed=1003, qkv_linear=4096),
    # BasicAttention::forward as the reference calls it, per layer: fused query_key_value GEMM, decode kernel, dense GEMM
    "glm4_9b_attention_block_b64": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=64, n_past=(1024, 8191), rope=8, theta=5.0e6,
                                        mask=0, interleaved=False, seed=20240603, attention_block=4096),
    # the reference's own decode loop: one sequence, ChatGLM3-6B shape (benchmark configuration 1 with its two Linears)
    "glm3_6b_attention_block_b1": dict(H=32, G=2, D=128, M=2048, layers=28, seqs=1, n_past=(512, 512), rope=8, theta=10000.0,
                                       mask=0, interleaved=False, seed=20240604, attention_block=4096),
    "glm4_9b_attention_block_b8": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=8, n_past=(1024, 8191), rope=8, theta=5.0e6,
                                       mask=0, interleaved=False, seed=20240603, attention_block=4096),
    "glm4_9b_qkv_linear_b8": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=8, n_past=(1024, 8191), rope=8, theta=5.0e6,
                                  interleaved=False, mask=0, seed=1003, qkv_linear=4096),
    "glm4_9b_qkv_linear_b128": dict(H=32, G=2, D=128, M=8192, layers=40, seqs=128, n_past=(1024, 8191), rope=8, theta=5.0e6,
                                    interleaved=False, mask=0, seed=1003, qkv_linear=4096),
    "glm3_6b_prefill_8192": dict(H=32, G=2, D=128, M=8192, layers=1, seqs=1, n_past=(0, 0), rope=8, theta=10000.0,
                                 interleaved=False, mask=0, seed=1002, prefill=8192),
    # benchmark configuration 5: ChatGLM-6B v1, MHA, interleaved qkv, 2-D rope
    "glm1_6b_mha_decode": dict(H=32, G=32, D=128, M=4096, layers=28, seqs=4, n_past=(2048, 2048), rope=4,
                               theta=10000.0, interleaved=True, mask=1, seed=1005),
}
HEADLINE = "glm4_9b_batched_decode"
HBM_FALLBACK_GBS = 6650.0   # B200 copy bandwidth from an earlier measurement, used only without MEASURED_PEAKS.json
TENSOR_FALLBACK_TFLOPS = 1590.0
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic KV bytes of one decode launch, from the ncu capture of
# the _small workload, whose launches are identical to the default workload's (see profiles/).
NCU_TRAFFIC_PER_KV_BYTE = 1.050
TID_K, TID_V, TID_QKV = 1, 2, 3   # tensor ids of the synthetic generator


def kv_bytes(w, n_past):
    """Algorithmic bytes of one layer call: K and V^T of every attended token, f16 (4*G*D*(n_past+1))."""
    return int(sum(4 * w["G"] * w["D"] * (int(p) + 1) for p in n_past))


def draw_n_past(w, rank, n=None):
    """The workload's sequence lengths.  Every rank gets the SAME lengths in its own order (weak scaling means the same
    work per GPU: lengths drawn per rank differed by up to 8 % in total bytes, and the step time, a maximum over ranks,
    followed the heaviest rank)."""
    lo, hi = w["n_past"]
    lengths = np.random.default_rng(w["seed"]).integers(lo, hi + 1, n or w["seqs"]).astype(np.int32)
    return lengths if rank == 0 else np.random.default_rng(w["seed"] + 7919 * rank).permutation(lengths)


def qkv_row(w):
    return 3 * w["H"] * w["D"] if w["interleaved"] else (w["H"] + 2 * w["G"]) * w["D"]


def peak(key, fallback):
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)[key]), "measured"
    except Exception:
        return fallback, "fallback"


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
            self._halt.wait(0.02)

    def finish(self):
        self._halt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def host_threads():
    return os.cpu_count() or 1


# ---- synthetic data: the same bits on the host and on the device -------------------------------------------------
class Synth:
    def __init__(self, device=True):
        from oracle import attn_oracle as O
        self.O = O
        self.t32, self.t16 = O.synth_table()
        if device:
            import torch
            from chatglm_cpp_b200 import _lib
            self.L = _lib.lib()
            self.d32 = torch.from_numpy(self.t32).cuda()
            self.d16 = torch.from_numpy(self.t16.view(np.int16)).cuda()

    def fill(self, tensor, seed, tid, first=0):
        import torch
        assert tensor.is_cuda and tensor.is_contiguous()
        stream = torch.cuda.current_stream().cuda_stream
        if tensor.dtype == torch.float16:
            rc = self.L.cglm_synth_fill_f16(tensor.data_ptr(), tensor.numel(), seed, tid, first, self.d16.data_ptr(), stream)
        else:
            rc = self.L.cglm_synth_fill_f32(tensor.data_ptr(), tensor.numel(), seed, tid, first, self.d32.data_ptr(), stream)
        assert rc == 0

    def host_f16(self, n, seed, tid, first):
        return self.O.synth_fill(n, seed, tid, first, self.t16)

    def host_f32(self, n, seed, tid, first):
        return self.O.synth_fill(n, seed, tid, first, self.t32)

    def host_caches(self, w, seed, slots):
        """(k, v) uint16 arrays of the given arena slots, as the device fill wrote them."""
        G, M, D = w["G"], w["M"], w["D"]
        per = G * M * D
        return [(self.host_f16(per, seed, TID_K, s * per).reshape(G, M, D), self.host_f16(per, seed, TID_V, s * per).reshape(G, D, M))
                for s in slots]


# ---- the CPU path (our restatement of the reference's) --------------------------------------------------------------
def cpu_decode_layer(w, n_past, n_ctx, qkv, caches, reps, warmup, calls=1):
    """`calls` layer calls of the workload on the host cores per repetition (all over the given layer's caches, which are
    far larger than the CPU's own caches).  Returns (seconds per repetition, outputs [n][H*D], threads)."""
    from oracle import attn_oracle as O
    cfg = O.make_cfg(w["H"], w["G"], w["D"], w["M"], 0, w["rope"], w["theta"], w["mask"], "ggml")
    n, H, G, D = len(n_past), w["H"], w["G"], w["D"]
    if w["interleaved"]:
        q = [qkv[i] for i in range(n)]; k = [qkv[i][D:] for i in range(n)]; v = [qkv[i][2 * D:] for i in range(n)]
        hs = 3 * D
    else:
        q = [qkv[i] for i in range(n)]; k = [qkv[i][H * D:] for i in range(n)]; v = [qkv[i][(H + G) * D:] for i in range(n)]
        hs = D
    kc = [c[0] for c in caches]
    vc = [c[1] for c in caches]
    thr = host_threads()
    times, out = [], None
    for it in range(warmup + reps):
        t0 = time.perf_counter()
        for _ in range(calls):
            out = O.attn_decode_batch(cfg, q, k, v, hs, hs, kc, vc, n_past, n_ctx, n_threads=thr)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    return float(np.mean(times)), np.asarray(out), thr


def run_reference(args, name, w):
    """--impl reference: the reference's CPU path (our CPU restatement of it: the reference's own arithmetic lives in
    the ggml submodule, which is absent and unpinned, so it cannot be compiled here).  Same synthetic bits as the GPU arm."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if w.get("prefill") or w.get("split_kv"):
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm times the batched decode workloads only"}), flush=True)
        return
    syn = Synth(device=False)
    n_past = draw_n_past(w, 0)
    n = len(n_past)
    n_ctx = np.maximum(n_past // 2, 2).astype(np.int32)
    caches = syn.host_caches(w, w["seed"], range(n))      # layer 0: slots [0, n)
    qkv = syn.host_f32(n * qkv_row(w), w["seed"], TID_QKV, 0).reshape(n, qkv_row(w))
    # each step: all of the workload's layer calls, really executed (over layer 0's caches: 0.6 GB, beyond the CPU's
    # caches, so repeating it costs what a new layer would), unless that would take more than about four minutes
    calls = w["layers"]
    probe, _, thr = cpu_decode_layer(w, n_past, n_ctx, qkv, caches, 1, 0)
    total = probe * calls * (args.steps + max(1, min(args.warmup, 3)))
    if total > 240.0:
        calls = max(1, int(calls * 240.0 / total))
    per_step, _, thr = cpu_decode_layer(w, n_past, n_ctx, qkv, caches, args.steps, max(1, min(args.warmup, 3)), calls=calls)
    per_layer = per_step / calls
    tps = n / (per_layer * w["layers"])
    sample = (f"every step executes {calls} of the {w['layers']} layer calls x {w['seqs']} sequences on the host cores"
              + ("" if calls == w["layers"] else f", time scaled to {w['layers']} layers"))
    line = {
        "impl": "reference", "metric": "decode_attention_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_layer * w["layers"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(name, w, n_past, args.gpus),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": thr, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(name, w, n_past, gpus):
    return {"workload": name, "n_head": w["H"], "n_kv_head": w["G"], "head_dim": w["D"],
            "max_length": w["M"], "layers": w["layers"], "seqs_per_gpu": len(n_past),
            "global_batch": len(n_past) * gpus, "n_past_range": list(w["n_past"]),
            "n_past_mean": float(np.mean(n_past)), "parallelism": f"sequence-sharded x{gpus}, no collective",
            "l2_policy": "inputs larger than L2 (each launch streams its own cache slabs; a step touches every layer's)"}


# ---- distributed plumbing -----------------------------------------------------------------------------------------
class Dist:
    def __init__(self):
        import torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU path")
        torch.cuda.set_device(self.local)
        self.cores = None
        if self.world > 1 and hasattr(os, "sched_setaffinity") and not os.environ.get("CGLM_BENCH_NO_PIN"):
            # every rank on its own share of the cores this job may use: the ranks' host threads (launches, the copies of the
            # host-buffer path) otherwise migrate over the same cores
            avail = sorted(os.sched_getaffinity(0))
            share = len(avail) // self.world
            if share >= 2:
                self.cores = avail[self.local * share:(self.local + 1) * share]
                os.sched_setaffinity(0, self.cores)
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist

    def barrier(self):
        import torch
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_ms(self, ms):
        import torch
        if self.world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def close(self):
        if self.world > 1:
            import torch
            torch.cuda.synchronize()
            killer = threading.Timer(30.0, lambda: os._exit(0))   # a slow teardown must not outlive the measurement
            killer.daemon = True
            killer.start()
            self.dist.barrier()
            self.dist.destroy_process_group()
            killer.cancel()


def timed(dd, fn, steps, warmup):
    """W untimed calls, then K timed calls between CUDA events on the launching stream, barrier + device synchronise on
    both sides, max over ranks.  Returns (milliseconds for the K calls, this library's launches on this rank)."""
    import torch
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    for _ in range(warmup):
        fn()
    dd.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = L.cglm_launch_count()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    dd.barrier()
    return dd.max_ms(e0.elapsed_time(e1)), L.cglm_launch_count() - launches0


# ---- batched decode (configs 1, 3, 5 and the batch-size / length variants) ----------------------------------------------
class DecodeState:
    """Caches of (layers x sequences) in one arena, activations per layer, all filled by the counter-based generator."""

    def __init__(self, w, rank, syn, layers=None, seqs=None):
        import torch
        from chatglm_cpp_b200 import _lib
        from chatglm_cpp_b200 import attention as A
        self.w, self.syn, self.A, self._lib = w, syn, A, _lib
        self.layers, self.n = layers or w["layers"], seqs or w["seqs"]
        self.seed = w["seed"] + 7919 * rank
        self.desc = _lib.AttnDesc(w["H"], w["G"], w["D"], w["M"], 0, w["rope"], w["theta"], w["mask"])
        self.arena = A.KVArena(self.desc, self.layers * self.n)
        syn.fill(self.arena.k_all(), self.seed, TID_K)
        syn.fill(self.arena.v_all(), self.seed, TID_V)
        self.ws = A.Workspace(self.desc, max(self.n, 128), 1)
        self.row, self.orow = qkv_row(w), w["H"] * w["D"]
        self.qkv = torch.empty(self.layers, self.n, self.row, device="cuda")
        syn.fill(self.qkv, self.seed, TID_QKV)
        self.out = torch.empty(self.layers, self.n, self.orow, device="cuda")
        torch.cuda.synchronize()

    def seq_arrays(self, n_past, n_ctx, seq_ids=None, layers=None, flags=0, n_past_dev=None):
        """One descriptor array per layer: slot of (layer l, sequence i) is l * n + i."""
        A, _lib = self.A, self._lib
        seq_ids = list(range(len(n_past))) if seq_ids is None else seq_ids
        arrays = []
        for l in range(layers or self.layers):
            arr = (_lib.AttnSeq * len(seq_ids))()
            for j, i in enumerate(seq_ids):
                call = A.SeqCall(qkv=self.qkv[l, i:i + 1], slot=l * self.n + i, n_past=int(n_past[j]), n_ctx=int(n_ctx[j]),
                                 out=self.out[l, i:i + 1], flags=flags,
                                 n_past_dev=None if n_past_dev is None else n_past_dev[j:j + 1])
                A.fill_seq(arr[j], self.desc, call, self.w["interleaved"])
            arrays.append(arr)
        return arrays

    def close(self):
        self.arena.close()


def decode_measure(dd, st, name, n_past, args, seq_ids=None, layers=None, device=True, e2e=True, step_graph=False, steps=None):
    """Times one decode workload on the state's arena.  Returns a dict of results (launch counts are this rank's; times
    are the max over ranks)."""
    import torch
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    w = st.w
    layers = layers or st.layers
    steps = steps or args.steps
    n = len(n_past)
    n_ctx = np.maximum(np.asarray(n_past) // 2, 2).astype(np.int32)
    # Every layer call reads cache rows that no kernel still running can write (a call appends at n_past of its own
    # layer's slots only), which is what CGLM_SEQ_CACHE_SETTLED promises.  Measured per step, with the flag against
    # without: 64 sequences resident 2.39-2.41 against 2.42-2.44 ms but through host buffers 2.50-2.52 against 2.48-2.50,
    # 32 sequences 1.62 against 1.58, 8 sequences 1.45 against 1.29: it pays only for long launches on resident inputs,
    # so it is off unless asked for (--settled).
    flags = _lib.SEQ_CACHE_SETTLED if args.settled else 0
    arrays = st.seq_arrays(n_past, n_ctx, seq_ids, layers, flags)
    stream = torch.cuda.current_stream().cuda_stream
    res = {"workload": name, "n_seq": n, "layers": layers, "kv_bytes_per_launch": kv_bytes(w, n_past)}

    def step_device():
        for l in range(layers):
            rc = L.cglm_attn_forward(st.arena._h, arrays[l], n, st.ws.ptr, st.ws.bytes, stream)
            if rc != 0:
                raise _lib.CglmError(rc, "cglm_attn_forward")

    if device:
        ms, launches = timed(dd, step_device, steps, args.warmup)
        if st.ws.status() != 0:
            raise SystemExit(f"{name}: device-side status is not clean after the timed region")
        res.update(ms_per_step=ms / steps, launches=int(launches), steps=steps)

    if e2e:
        # the same step through host buffers: the activations (f16: the hand-off the library offers to f16 Linears;
        # f32 with --e2e-f32) cross the bus in both directions inside the timed region
        host_dt = torch.float32 if args.e2e_f32 else torch.float16
        ids = list(range(n)) if seq_ids is None else seq_ids
        qkv_host = st.qkv[:layers][:, ids].to(host_dt).cpu().pin_memory()
        out_host = torch.empty(layers, n, st.orow, dtype=host_dt).pin_memory()
        n_stage = 3
        stage_qkv = [torch.empty(n, st.row, device="cuda", dtype=host_dt) for _ in range(n_stage)]
        stage_out = [torch.empty(n, st.orow, device="cuda", dtype=host_dt) for _ in range(n_stage)]
        layout = (_lib.HOST_INTERLEAVED_QKV if w["interleaved"] else 0) | (0 if args.e2e_f32 else _lib.HOST_F16)

        host_s = [0.0]
        # plain integers for the call: indexing a tensor and asking for its pointer costs microseconds per call in Python,
        # which a compiled host would not pay
        p_in = [qkv_host[l].data_ptr() for l in range(layers)]
        p_out = [out_host[l].data_ptr() for l in range(layers)]
        p_sq = [t.data_ptr() for t in stage_qkv]
        p_so = [t.data_ptr() for t in stage_out]
        arena_h, ws_ptr, ws_bytes = st.arena._h, st.ws.ptr, st.ws.bytes

        def step_host():
            t_host = time.perf_counter()
            for l in range(layers):
                rc = L.cglm_attn_forward_host(arena_h, arrays[l], n, layout, p_in[l], p_out[l], p_sq[l % n_stage], p_so[l % n_stage],
                                              ws_ptr, ws_bytes, stream)
                if rc != 0:
                    raise _lib.CglmError(rc, "cglm_attn_forward_host")
            rc = L.cglm_attn_host_drain(st.arena._h, stream)   # the step's results are read back here
            if rc != 0:
                raise _lib.CglmError(rc, "cglm_attn_host_drain")
            host_s[0] += time.perf_counter() - t_host

        e2e_steps = max(3, steps // 2)
        n_warm = max(3, args.warmup)
        ms_e2e, _ = timed(dd, step_host, e2e_steps, n_warm)
        if st.ws.status() != 0:
            raise SystemExit(f"{name}: device-side status is not clean after the host-buffer region")
        esz = 4 if args.e2e_f32 else 2
        # host_issue_ms_per_step: what the host needs to enqueue a step (all calls, warm-up included in the average); when it
        # is close to ms_per_step the host, not the GPU or the bus, sets the end-to-end rate
        res["e2e"] = {"ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps, "activation_dtype": "f32" if args.e2e_f32 else "f16",
                      "host_issue_ms_per_step": host_s[0] * 1e3 / (e2e_steps + n_warm),
                      "h2d_bytes_per_step": layers * n * st.row * esz, "d2h_bytes_per_step": layers * n * st.orow * esz}
        res["_out_host"] = out_host

    if step_graph:
        # The step issued as ONE CUDA graph whose layer calls read n_past from device words (CGLM_SEQ_N_PAST_DEVICE): the
        # form a caller replays for every new token without rebuilding anything.  The words are advanced by 0 here so
        # that every replay is the step the other figures measure.
        n_past_dev = torch.tensor([int(p) for p in n_past], dtype=torch.int32, device="cuda")
        dyn = st.seq_arrays(n_past, n_ctx, seq_ids, layers, _lib.SEQ_N_PAST_DEVICE, n_past_dev)

        def step_dyn():
            s2 = torch.cuda.current_stream().cuda_stream
            for l in range(layers):
                rc = L.cglm_attn_forward(st.arena._h, dyn[l], n, st.ws.ptr, st.ws.bytes, s2)
                if rc != 0:
                    raise _lib.CglmError(rc, "cglm_attn_forward")
            rc = L.cglm_seq_advance(n_past_dev.data_ptr(), n, 0, s2)
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
        ms_graph, _ = timed(dd, graph.replay, steps, args.warmup)
        ms_dyn, _ = timed(dd, step_dyn, steps, args.warmup)   # the same launches issued eagerly: what the graph itself costs or saves
        if st.ws.status() != 0:
            raise SystemExit(f"{name}: device-side status is not clean after the step-graph region")
        res["step_graph"] = {"ms_per_step": ms_graph / steps, "launches_per_step": layers + 1,
                             "same_launches_eager_ms_per_step": ms_dyn / steps,
                             "note": "one CUDA graph per decode step, n_past read from device words, replayed"}
        graph = None
    return res


def decode_summary(res, world, hbm_peak):
    """The short per-config entry of the JSON line."""
    launch_ms = res["ms_per_step"] / res["layers"]
    achieved = res["kv_bytes_per_launch"] / (launch_ms * 1e-3) / 1e9
    out = {"value": res["n_seq"] * world / (res["ms_per_step"] * 1e-3), "unit": "tokens/s", "ms_per_step": res["ms_per_step"],
           "steps": res["steps"], "launch_us": launch_ms * 1e3,
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                        "algorithmic_bytes_per_launch": res["kv_bytes_per_launch"]}}
    if "e2e" in res:
        e = res["e2e"]
        out["e2e"] = {"value": res["n_seq"] * world / (e["ms_per_step"] * 1e-3), "unit": "tokens/s", "ms_per_step": e["ms_per_step"],
                      "h2d_bytes_per_step": e["h2d_bytes_per_step"], "d2h_bytes_per_step": e["d2h_bytes_per_step"],
                      "activation_dtype": e["activation_dtype"], "host_issue_ms_per_step": e["host_issue_ms_per_step"]}
    if "step_graph" in res:
        g = res["step_graph"]
        out["step_graph"] = dict(g, value=res["n_seq"] * world / (g["ms_per_step"] * 1e-3), unit="tokens/s")
    return out


def parity_check(st, n_past, out_host_l0, reps=3):
    """Layer 0 of the workload on the host cores (same bits: the host twin of the generator rebuilds the caches and the
    activations) against what the timed GPU launches left behind: outputs of layer 0 and the appended cache rows.
    Also the cpu_baseline timing.  Returns (cpu_baseline dict, parity dict)."""
    import torch
    w, syn, n = st.w, st.syn, len(n_past)
    n_ctx = np.maximum(np.asarray(n_past) // 2, 2).astype(np.int32)
    caches = syn.host_caches(w, st.seed, range(n))
    qkv = syn.host_f32(n * st.row, st.seed, TID_QKV, 0).reshape(n, st.row)
    # a bounded sample: `reps` whole steps (every layer call executed, over layer 0's caches), a few seconds of CPU work
    per_step, want, thr = cpu_decode_layer(w, n_past, n_ctx, qkv, caches, reps, 0, calls=w["layers"])
    per_layer = per_step / w["layers"]
    got = st.out[0, :n].cpu().numpy()
    err = float(np.abs(got - want).max())
    bit_exact = True
    for i, p in enumerate(n_past):
        gk = st.arena.k_cache(i)[:, int(p)].cpu().numpy().view(np.uint16)
        gv = st.arena.v_cache(i)[:, :, int(p)].cpu().numpy().view(np.uint16)
        bit_exact = bit_exact and np.array_equal(gk, caches[i][0][:, int(p)]) and np.array_equal(gv, caches[i][1][:, :, int(p)])
    parity = {"max_abs": err, "tolerance": 2e-3, "cache_bit_exact": bool(bit_exact),
              "checked": f"layer 0, {n} sequences: outputs of the device-resident run and the appended cache rows against the CPU restatement"}
    if out_host_l0 is not None:   # the host-buffer run's layer 0 (f16 in, f16 out unless --e2e-f32)
        parity["e2e_max_abs"] = float(np.abs(out_host_l0.float().numpy() - want).max())
        # f16 hand-off: inputs rounded to f16 (2^-11 relative each) and the output rounded once more
        parity["e2e_tolerance"] = 2e-3 if out_host_l0.dtype == torch.float32 else 6e-3
    tps = n / (per_layer * w["layers"])
    cpu = {"value": tps, "unit": "tokens/s", "cores": thr, "kind": "port",
           "sample": f"{reps} whole steps: {w['layers']} layer calls x {n} sequences each, executed over layer 0's caches (same bits as the GPU arm)"}
    return cpu, parity


# ---- prefill (config 2) -------------------------------------------------------------------------------------------------
def prefill_measure(dd, name, w, args, syn, steps=None):
    """A step is one prefill call (RoPE + f16 cache write + causal attention over the prompt).  Slots rotate so that
    consecutive steps do not reuse a warm cache slab; q/k/v activations and the output are re-read / re-written."""
    import torch
    from chatglm_cpp_b200 import _lib
    from chatglm_cpp_b200 import attention as A
    L = _lib.lib()
    H, G, D, S = w["H"], w["G"], w["D"], w["prefill"]
    steps = steps or args.steps
    desc = _lib.AttnDesc(H, G, D, w["M"], 0, w["rope"], w["theta"], w["mask"])
    n_rot = 16 if S <= 2048 else 4
    arena = A.KVArena(desc, n_rot)
    ws = A.Workspace(desc, 1, S)
    qkv = torch.empty(n_rot, S, qkv_row(w), device="cuda")
    syn.fill(qkv, w["seed"], TID_QKV)
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

    ms, launches = timed(dd, step, steps, max(args.warmup, 3))
    if ws.status() != 0:
        raise SystemExit(f"{name}: device-side status is not clean after the timed region")
    ms /= steps
    flops = 4.0 * H * D * S * (S + 1) / 2          # useful (causal) FLOPs of QK^T and PV
    pk, src = peak("bf16_tflops", TENSOR_FALLBACK_TFLOPS)
    achieved = flops / (ms * 1e-3) / 1e12
    arena.close()
    return {"metric": "prefill_attention_tokens_per_s", "value": S / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "steps": steps, "launches": int(launches), "prompt_tokens": S,
            "l2_policy": f"rotates through {n_rot} slots and activation buffers",
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk, "unit": "TFLOP/s", "frac": achieved / pk,
                         "peak_source": src, "kernel": "prefill kernels (whole call)", "useful_flops_per_call": flops}}


# ---- the Linear in front of the path ------------------------------------------------------------------------------------
def qkv_linear_measure(dd, name, w, args, syn, steps=None):
    """A step is the fused query_key_value Linear (bias, RoPE, K/V append in the epilogue) of every layer for a batch of
    one-token sequences: `layers` launches, each streaming its own f16 weight.  Bound: the weight bytes over HBM."""
    import torch
    from chatglm_cpp_b200 import _lib
    from chatglm_cpp_b200 import attention as A
    L = _lib.lib()
    H, G, D, hidden, layers, n = w["H"], w["G"], w["D"], w["qkv_linear"], w["layers"], w["seqs"]
    steps = steps or args.steps
    n_feat = (H + 2 * G) * D
    desc = _lib.AttnDesc(H, G, D, w["M"], 0, w["rope"], w["theta"], w["mask"])
    arena = A.KVArena(desc, n)            # the layers append into the same slots: irrelevant for the timing
    ws = A.Workspace(desc, n, 1)
    weight = torch.empty(layers, n_feat, hidden, device="cuda", dtype=torch.float16)
    syn.fill(weight, w["seed"], 11)
    weight.mul_(1.0 / np.sqrt(hidden))
    x = torch.empty(n, hidden, device="cuda", dtype=torch.float16)
    syn.fill(x, w["seed"], 12)
    bias = torch.zeros(n_feat, device="cuda")
    q_roped = torch.empty(n, H * D, device="cuda")
    n_past = draw_n_past(w, dd.rank)
    arr = (_lib.AttnSeq * n)()
    for i in range(n):
        arr[i].slot, arr[i].qlen, arr[i].n_past = i, 1, int(n_past[i])

    def step():
        stream = torch.cuda.current_stream().cuda_stream
        for l in range(layers):
            rc = L.cglm_qkv_linear_forward(arena._h, arr, n, x.data_ptr(), hidden, weight[l].data_ptr(), bias.data_ptr(),
                                           q_roped.data_ptr(), ws.ptr, ws.bytes, stream)
            if rc != 0:
                raise _lib.CglmError(rc, "cglm_qkv_linear_forward")

    # the step as a replayed CUDA graph: an eager call (two tensor maps encoded on the host per call, through ctypes) takes
    # about as long to issue as the kernel runs
    ms_eager, launches = timed(dd, step, steps, max(args.warmup, 3))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    ms, _ = timed(dd, graph.replay, steps, max(args.warmup, 3))
    graph = None
    if ws.status() != 0:
        raise SystemExit(f"{name}: device-side status is not clean after the timed region")
    ms /= steps
    pk, src = peak("hbm_gbs", HBM_FALLBACK_GBS)
    w_bytes = n_feat * hidden * 2
    achieved = w_bytes * layers / (ms * 1e-3) / 1e9
    arena.close()
    return {"metric": "qkv_linear_tokens_per_s", "value": n * dd.world / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "steps": steps, "launches": int(launches), "tokens": n,
            "l2_policy": f"every layer call streams its own {w_bytes / 1e6:.1f} MB weight ({layers} layers > L2)",
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk, "unit": "GB/s", "frac": achieved / pk,
                         "peak_source": src, "kernel": "qkv_linear_kernel", "algorithmic_bytes_per_launch": w_bytes,
                         "launch_us": ms * 1e3 / layers, "issue": "CUDA graph of the step, replayed",
                         "eager_launch_us": ms_eager / steps * 1e3 / layers}}


def attention_block_measure(dd, name, w, args, syn, steps=None):
    """A step is BasicAttention::forward (chatglm.cpp:625-722) of every layer for a batch of one-token sequences:
    hidden_states f16 -> query_key_value GEMM -> decode kernel over the cache (context out in f16) -> dense GEMM ->
    attn_output f32.  Three launches per layer, each layer with its own weights and caches.  Bound: KV bytes plus both
    weights over HBM."""
    import torch
    from chatglm_cpp_b200 import _lib
    from chatglm_cpp_b200 import attention as A
    L = _lib.lib()
    H, G, D, hidden, layers, n = w["H"], w["G"], w["D"], w["attention_block"], w["layers"], w["seqs"]
    steps = steps or args.steps
    n_feat = (H + 2 * G) * D
    seed = w["seed"] + 7919 * dd.rank
    desc = _lib.AttnDesc(H, G, D, w["M"], 0, w["rope"], w["theta"], w["mask"])
    arena = A.KVArena(desc, layers * n)
    syn.fill(arena.k_all(), seed, TID_K)
    syn.fill(arena.v_all(), seed, TID_V)
    ws = A.Workspace(desc, max(n, 128), 1)
    w_qkv = torch.empty(layers, n_feat, hidden, device="cuda", dtype=torch.float16)
    w_dense = torch.empty(layers, hidden, H * D, device="cuda", dtype=torch.float16)
    syn.fill(w_qkv, seed, 11)
    syn.fill(w_dense, seed, 13)
    w_qkv.mul_(1.0 / np.sqrt(hidden))
    w_dense.mul_(1.0 / np.sqrt(H * D))
    x = torch.empty(n, hidden, device="cuda", dtype=torch.float16)
    syn.fill(x, seed, 12)
    bias = torch.zeros(n_feat, device="cuda")
    # Up to 32 sequences the query_key_value GEMM carries bias, RoPE and the cache append in its epilogue and hands roped
    # q (f32) to the decode kernel; beyond, the plain GEMM with an f16 qkv row and the decode kernel's own RoPE + append are
    # faster (the fused epilogue's V^T scatter falls on two thread blocks; measured at 64 sequences).
    fused = n <= 32
    q_roped = torch.empty(2, n, H * D if fused else n_feat, device="cuda", dtype=torch.float32 if fused else torch.float16)
    context = torch.empty(2, n, H * D, device="cuda", dtype=torch.float16)
    out = torch.empty(layers, n, hidden, device="cuda")
    n_past = draw_n_past(w, dd.rank)
    lin_arr, att_arr = [], []
    for l in range(layers):
        a1, a2 = (_lib.AttnSeq * n)(), (_lib.AttnSeq * n)()
        for i in range(n):
            P = int(n_past[i])
            a1[i].slot, a1[i].qlen, a1[i].n_past = l * n + i, 1, P
            q = q_roped[l % 2, i].data_ptr()
            a2[i].q_head_stride = a2[i].kv_head_stride = D
            a2[i].slot, a2[i].qlen, a2[i].n_past = l * n + i, 1, P
            if fused:
                a2[i].q = a2[i].k = a2[i].v = q                              # k and v are not read
                a2[i].q_tok_stride = a2[i].kv_tok_stride = H * D
                a2[i].kv_local = P + 1
                a2[i].flags = _lib.SEQ_Q_ROPED | _lib.SEQ_NO_APPEND | _lib.SEQ_USE_KV_LOCAL | _lib.SEQ_OUT_F16
            else:                                                            # blocked f16 qkv row (chatglm.cpp:646-652)
                a2[i].q, a2[i].k, a2[i].v = q, q + 2 * H * D, q + 2 * (H + G) * D
                a2[i].q_tok_stride = a2[i].kv_tok_stride = n_feat
                a2[i].flags = _lib.SEQ_QKV_F16 | _lib.SEQ_OUT_F16
            a2[i].out = context[l % 2, i].data_ptr()
        lin_arr.append(a1)
        att_arr.append(a2)

    def step():
        stream = torch.cuda.current_stream().cuda_stream
        for l in range(layers):
            if fused:
                rc = L.cglm_qkv_linear_forward(arena._h, lin_arr[l], n, x.data_ptr(), hidden, w_qkv[l].data_ptr(), bias.data_ptr(),
                                               q_roped[l % 2].data_ptr(), ws.ptr, ws.bytes, stream)
            else:
                rc = L.cglm_linear_forward(x.data_ptr(), n, hidden, w_qkv[l].data_ptr(), n_feat, bias.data_ptr(),
                                           q_roped[l % 2].data_ptr(), 1, ws.ptr, ws.bytes, stream)
            if rc == 0:
                rc = L.cglm_attn_forward(arena._h, att_arr[l], n, ws.ptr, ws.bytes, stream)
            if rc == 0:
                rc = L.cglm_linear_forward(context[l % 2].data_ptr(), n, H * D, w_dense[l].data_ptr(), hidden, None,
                                           out[l].data_ptr(), 0, ws.ptr, ws.bytes, stream)
            if rc != 0:
                raise _lib.CglmError(rc, "attention block")

    # issued as a replayed CUDA graph (an eager GEMM call encodes two tensor maps on the host, through ctypes, and takes
    # about as long to issue as the kernel runs); the eager figure is reported beside it
    ms_eager, launches = timed(dd, step, max(3, steps // 4), max(args.warmup, 3))
    ms_eager /= max(3, steps // 4)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    ms, _ = timed(dd, graph.replay, steps, max(args.warmup, 3))
    graph = None
    if ws.status() != 0:
        raise SystemExit(f"{name}: device-side status is not clean after the timed region")
    if not bool(torch.isfinite(out).all()):
        raise SystemExit(f"{name}: non-finite attn_output")
    ms /= steps
    pk, src = peak("hbm_gbs", HBM_FALLBACK_GBS)
    w_bytes = (n_feat * hidden + hidden * H * D) * 2
    kv = kv_bytes(w, n_past)
    achieved = (w_bytes + kv) * layers / (ms * 1e-3) / 1e9
    arena.close()
    return {"metric": "attention_block_tokens_per_s", "value": n * dd.world / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "steps": steps, "launches": int(launches) // max(3, steps // 4) * steps, "tokens": n,
            "l2_policy": f"every layer streams its own caches ({kv / 1e6:.0f} MB) and weights ({w_bytes / 1e6:.1f} MB): {layers} layers > L2",
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk, "unit": "GB/s", "frac": achieved / pk,
                         "peak_source": src, "kernel": ("linear_fm_kernel<false>" if fused else "linear_fm_kernel<true>") + " + decode_kernel + linear_fm_kernel<true>",
                         "qkv_route": "fused epilogue (RoPE + append in the GEMM)" if fused else "plain GEMM, f16 qkv row, RoPE + append in the decode kernel",
                         "algorithmic_bytes_per_layer": w_bytes + kv, "layer_us": ms * 1e3 / layers,
                         "issue": "CUDA graph of the step, replayed", "eager_layer_us": ms_eager * 1e3 / layers}}


# ---- one long sequence (config 4) ----------------------------------------------------------------------------------------
def split_kv_rotation(n_past, world, n_kv_head, head_dim):
    """Copies of a rank's KV slice the split-KV workload rotates through, so that the working set is at least four times
    the L2.  The same on every rank: it is taken from the slice CAPACITY (the ranks' slices differ by a few tokens; a
    count taken from the local slice came out 15 on three ranks and 16 on the fourth, and the ranks then captured graphs
    of different lengths and ran different numbers of steps)."""
    from chatglm_cpp_b200 import sharding
    cap = sharding.slice_capacity(n_past, 0, world)
    return max(2, int(np.ceil(4 * 126e6 / (4 * n_kv_head * head_dim * cap))))


def split_kv_measure(dd, name, w, args, syn, steps=None):
    """Strong scaling of ONE long sequence.  1 GPU: one fused decode launch per step.  N GPUs: rank r holds a contiguous
    slice of the KV length in its own arena; `p2p`: one fused launch per rank and step (attention over the slice, peer
    stores of the partial rows into every rank's exchange buffer, bounded wait, log-sum-exp combine); `nccl`: decode,
    all-gather, combine kernel.  Each step rotates through enough copies of the slice that the working set is at
    least four times the L2.  The steps of one rotation are captured in a CUDA graph and the timed region replays it."""
    import torch
    from chatglm_cpp_b200 import _lib, sharding
    from chatglm_cpp_b200 import attention as A
    L = _lib.lib()
    rank, world = dd.rank, dd.world
    H, G, D = w["H"], w["G"], w["D"]
    P = w["n_past"][0]
    steps = steps or args.steps
    sl = sharding.split_kv(P, 0, world, rank)
    cap = sharding.slice_capacity(P, 0, world) + 64
    desc = _lib.AttnDesc(H, G, D, cap, 0, w["rope"], w["theta"], w["mask"])
    local_bytes = 4 * G * D * (sl.n_local + (1 if sl.owns_new else 0))
    n_rot = split_kv_rotation(P, world, G, D)
    arena = A.KVArena(desc, n_rot)
    syn.fill(arena.k_all(), w["seed"] + rank, TID_K)
    syn.fill(arena.v_all(), w["seed"] + rank, TID_V)
    ws = A.Workspace(desc, 1, 1)
    qkv = torch.empty(1, qkv_row(w), device="cuda")
    syn.fill(qkv, w["seed"], TID_QKV)                       # q is replicated on every rank
    partial = torch.zeros(H, D + 2, device="cuda")
    gathered = torch.zeros(world, H, D + 2, device="cuda")
    out = torch.zeros(1, H * D, device="cuda")
    xchg = None
    if world > 1 and args.exchange == "p2p":
        # every kernel of the step runs once locally before the ranks meet (module loading happens here, not inside the
        # first bounded wait)
        solo = A.SplitKVExchange([A.SplitKVExchange.new_buffer(1, H, D)], 0, H, D)
        warm = (_lib.AttnSeq * 1)()
        A.fill_seq(warm[0], desc, A.SeqCall(qkv=qkv, slot=0, n_past=P, kv_local=max(sl.n_local, 1),
                                            flags=_lib.SEQ_USE_KV_LOCAL | _lib.SEQ_NO_APPEND), False)
        solo.step(arena, ws, warm, torch.zeros(H * D, device="cuda"))
        torch.cuda.synchronize()
        mine, handle = A.SplitKVExchange.alloc_exported(world, H, D)
        handles = [None] * world
        dd.dist.all_gather_object(handles, (dd.local, handle))
        # imported with this rank's device current (the mapping must belong to the context whose kernels use it)
        peers = [mine if r == rank else A.SplitKVExchange.import_handle(handles[r][1], handles[r][0]) for r in range(world)]
        xchg = A.SplitKVExchange(peers, rank, H, D)
        dd.barrier()
    settled = _lib.SEQ_CACHE_SETTLED if args.settled else 0     # no step writes rows below n_past of any slot
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
    timeout_us = 200000   # a rank that is more than 200 ms behind is treated as gone
    # NCCL's collectives inside a replayed graph did not complete at 4 ranks here (no output for 300 s); that exchange is the
    # comparison path, so beyond 2 ranks it is issued eagerly
    use_graph = args.issue == "graph" and not (world > 2 and xchg is None)

    def step():
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
            dd.dist.all_gather_into_tensor(gathered, partial)
            A.splitkv_combine(gathered, out.view(-1))

    def check_status(where):
        # a peer's rows never arrived: every further step would run into the same bounded wait, so stop here
        st = torch.tensor([ws.status()], device="cuda", dtype=torch.int32)
        if world > 1:
            dd.dist.all_reduce(st, op=dd.dist.ReduceOp.MIN)
        if int(st.item()) != 0:
            detail = ""
            if xchg is not None:   # which arrival words are missing: [set][rank][kv head], and this rank's step counter
                words = xchg.read_words(32 + 2 * 16 * 32)
                flags = [[[int(words[32 + (s_ * 16 + r_) * 32 + g_]) for g_ in range(G)] for r_ in range(world)] for s_ in range(2)]
                detail = f"; step counter {int(words[0])}, arrival words {flags}"
            raise SystemExit(f"[rank {rank}] device-side status {int(st.item())} {where}{detail}")

    for _ in range(max(args.warmup, 3)):
        step()
    dd.barrier()
    check_status("after the warm-up steps")
    launches_per_step = 1 if (xchg is not None or world == 1) else 2   # this library's kernels: decode (+ combine)
    it[0] = 0
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    dd.barrier()
    it[0] = 0
    graph = None
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(n_rot):
                step()

    def rotation():
        if graph is not None:
            graph.replay()
        else:
            for _ in range(n_rot):
                step()

    replays = max(1, (steps + n_rot - 1) // n_rot)
    steps = replays * n_rot
    # instantiating a graph takes a different time on every rank: the ranks meet again before the first replay, whose
    # bounded waits would otherwise count the slowest rank's instantiation
    dd.barrier()
    for _ in range(2):
        rotation()
    dd.barrier()
    check_status("after the first graph replays")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        rotation()
    e1.record()
    dd.barrier()
    ms = dd.max_ms(e0.elapsed_time(e1))
    check_status("after the timed region")
    step_ms = ms / steps
    pk, src = peak("hbm_gbs", HBM_FALLBACK_GBS)
    achieved = local_bytes / (step_ms * 1e-3) / 1e9
    res = {"metric": "decode_attention_tokens_per_s", "value": steps / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": step_ms,
           "steps": steps, "launches": steps * launches_per_step, "n_past": P, "kv_bytes_total": 4 * G * D * (P + 1),
           "kv_bytes_this_rank": local_bytes,
           "parallelism": ("one GPU, one fused decode launch per step" if world == 1 else
                           f"KV length split x{world}, " +
                           ("one fused launch per rank: attention + peer stores of the partial rows + LSE combine"
                            if xchg is not None else "decode + NCCL all-gather + combine kernel") +
                           f", {H * (D + 2) * 4} B per rank"),
           "l2_policy": f"rotates through {n_rot} copies of the slice (working set >= 4 x L2)",
           "issue": f"CUDA graph of {n_rot} steps, replayed" if use_graph else "eager launches",
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk, "unit": "GB/s", "frac": achieved / pk, "peak_source": src,
                        "kernel": "decode_kernel (the step time includes the exchange and the combine)",
                        "algorithmic_bytes_per_launch": local_bytes, "launch_us": step_ms * 1e3}}
    graph = None
    torch.cuda.synchronize()
    arena.close()
    return res


# ---- drivers ------------------------------------------------------------------------------------------------------------
def base_line(args, dd, metric="decode_attention_tokens_per_s", scaling="weak"):
    return {"metric": metric, "unit": "tokens/s", "n_gpus": dd.world, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f16", "data": "synthetic"}


def decode_line(args, dd, name, w, n_past, r, s, src, cpu, parity, clocks):
    line = dict(base_line(args, dd), value=s["value"], ms_per_step=s["ms_per_step"],
                config=workload_config(name, w, n_past, dd.world),
                roofline=dict(s["roofline"], peak_source=src, kernel="decode_kernel", launch_us=s["launch_us"],
                              traffic=NCU_TRAFFIC_PER_KV_BYTE * r["kv_bytes_per_launch"],
                              frac_of_nominal_8000=s["roofline"]["achieved"] / 8000.0),
                cpu_baseline=cpu, e2e=s.get("e2e"), gpu_launches=r["launches"] * dd.world, clocks=clocks)
    if parity is not None:
        line["parity"] = parity
    if "step_graph" in s:
        line["step_graph"] = s["step_graph"]
    return line


def run_single(args, dd, name, w):
    """--workload NAME: that workload alone as the line (used for profiling and for the tables in the documents)."""
    syn = Synth()
    pk, src = peak("hbm_gbs", HBM_FALLBACK_GBS)
    sampler = ClockSampler(dd.local)
    sampler.start()
    if w.get("prefill"):
        r = prefill_measure(dd, name, w, args, syn)
        line = dict(base_line(args, dd, r["metric"]), value=r["value"], ms_per_step=r["ms_per_step"],
                    config={"workload": name, "n_head": w["H"], "n_kv_head": w["G"], "head_dim": w["D"],
                            "prompt_tokens": w["prefill"], "l2_policy": r["l2_policy"]},
                    roofline=dict(r["roofline"], traffic=None), cpu_baseline=None, e2e=None, gpu_launches=r["launches"],
                    clocks=sampler.finish())
    elif w.get("qkv_linear"):
        r = qkv_linear_measure(dd, name, w, args, syn)
        line = dict(base_line(args, dd, r["metric"]), value=r["value"], ms_per_step=r["ms_per_step"],
                    config={"workload": name, "n_head": w["H"], "n_kv_head": w["G"], "head_dim": w["D"], "hidden": w["qkv_linear"],
                            "layers": w["layers"], "tokens": r["tokens"], "l2_policy": r["l2_policy"]},
                    roofline=dict(r["roofline"], traffic=None), cpu_baseline=None, e2e=None, gpu_launches=r["launches"] * dd.world,
                    clocks=sampler.finish())
    elif w.get("attention_block"):
        r = attention_block_measure(dd, name, w, args, syn)
        line = dict(base_line(args, dd, r["metric"]), value=r["value"], ms_per_step=r["ms_per_step"],
                    config={"workload": name, "n_head": w["H"], "n_kv_head": w["G"], "head_dim": w["D"], "hidden": w["attention_block"],
                            "layers": w["layers"], "tokens": r["tokens"], "l2_policy": r["l2_policy"]},
                    roofline=dict(r["roofline"], traffic=None), cpu_baseline=None, e2e=None, gpu_launches=r["launches"] * dd.world,
                    clocks=sampler.finish())
    elif w.get("split_kv"):
        r = split_kv_measure(dd, name, w, args, syn)
        line = dict(base_line(args, dd, scaling="strong"), value=r["value"], ms_per_step=r["ms_per_step"], steps=r["steps"],
                    config={"workload": name, "n_head": w["H"], "n_kv_head": w["G"], "head_dim": w["D"], "n_past": r["n_past"],
                            "kv_bytes_total": r["kv_bytes_total"], "kv_bytes_this_rank": r["kv_bytes_this_rank"],
                            "parallelism": r["parallelism"], "l2_policy": r["l2_policy"], "issue": r["issue"]},
                    roofline=dict(r["roofline"], traffic=None), cpu_baseline=None, e2e=None,
                    gpu_launches=r["launches"] * dd.world, clocks=sampler.finish())
    else:
        st = DecodeState(w, dd.rank, syn)
        n_past = draw_n_past(w, dd.rank)
        r = decode_measure(dd, st, name, n_past, args, e2e=True, step_graph=args.step_graph)
        clocks = sampler.finish()
        s = decode_summary(r, dd.world, pk)
        cpu = parity = None
        if dd.rank == 0 and dd.world == 1 and not args.no_cpu_baseline:
            cpu, parity = parity_check(st, n_past, r["_out_host"][0])
        line = decode_line(args, dd, name, w, n_past, r, s, src, cpu, parity, clocks)
        st.close()
    return line


def run_default(args, dd):
    """The headline workload plus, in the same line, the other benchmark configurations and the multi-GPU partitions."""
    import torch
    name, w = HEADLINE, WORKLOADS[HEADLINE]
    syn = Synth()
    pk, src = peak("hbm_gbs", HBM_FALLBACK_GBS)
    st = DecodeState(w, dd.rank, syn)
    n_past = draw_n_past(w, dd.rank)
    sampler = ClockSampler(dd.local)
    sampler.start()
    r = decode_measure(dd, st, name, n_past, args, e2e=False)
    clocks = sampler.finish()
    cpu = parity = None
    check = dd.rank == 0 and dd.world == 1 and not args.no_cpu_baseline
    if check:
        # st.out holds what the last timed step wrote; the CPU leg recomputes layer 0 from the same bits
        got_dev = st.out[0].clone()
    r.update(decode_measure(dd, st, name, n_past, args, device=False, e2e=True, step_graph=True))
    if check:
        st.out[0].copy_(got_dev)
        cpu, parity = parity_check(st, n_past, r["_out_host"][0])
    s = decode_summary(r, dd.world, pk)
    line = decode_line(args, dd, name, w, n_past, r, s, src, cpu, parity, clocks)
    short = max(5, min(args.steps, 10))
    configs = {}
    if not args.headline_only:
        # same arena, other batch sizes and lengths (slots are addressed as layer * 64 + sequence)
        for nm, ids, npast in (
            ("glm4_9b_batched_decode_8k", list(range(64)), np.full(64, 8191, np.int32)),
            ("glm4_9b_batched_decode_b32", list(range(32)), n_past[:32]),
        ):
            rr = decode_measure(dd, st, nm, npast, args, seq_ids=ids, e2e=False, steps=short)
            configs[nm] = decode_summary(rr, dd.world, pk)
        if dd.world > 1:
            # strong scaling of benchmark configuration 3: the SAME 64 sequences (lengths of rank 0's draw) sharded over the GPUs
            from chatglm_cpp_b200 import sharding
            glob = draw_n_past(w, 0)
            mine = sharding.shard_sequences(len(glob), dd.world, dd.rank)
            rr = decode_measure(dd, st, name + "_strong", glob[mine], args, seq_ids=list(range(len(mine))), e2e=True, step_graph=True,
                                steps=args.steps)
            ss = decode_summary(rr, 1, pk)
            total = len(glob)
            line["strong"] = {"global_batch": total, "seqs_per_gpu": len(mine), "value": total / (rr["ms_per_step"] * 1e-3),
                              "unit": "tokens/s", "ms_per_step": rr["ms_per_step"], "launch_us": ss["launch_us"],
                              "roofline_frac_rank0": ss["roofline"]["frac"],
                              "e2e": {"value": total / (rr["e2e"]["ms_per_step"] * 1e-3), "unit": "tokens/s",
                                      "ms_per_step": rr["e2e"]["ms_per_step"]},
                              # few sequences per GPU make a launch shorter than an eager call through Python takes to issue:
                              # the replayed step graph is the same work without the host in the loop
                              "step_graph": {"ms_per_step": rr["step_graph"]["ms_per_step"], "unit": "tokens/s",
                                             "value": total / (rr["step_graph"]["ms_per_step"] * 1e-3)},
                              "note": "the 64 sequences of the 1-GPU workload, sequence i on GPU i mod N, no collective"}
    st.close()
    del st
    torch.cuda.empty_cache()
    if not args.headline_only:
        for nm in ("glm3_6b_decode_512", "glm1_6b_mha_decode"):
            ww = WORKLOADS[nm]
            s2 = DecodeState(ww, dd.rank, syn)
            rr = decode_measure(dd, s2, nm, draw_n_past(ww, dd.rank), args, e2e=True, step_graph=(nm == "glm3_6b_decode_512"), steps=short)
            configs[nm] = decode_summary(rr, dd.world, pk)
            s2.close()
        for nm in ("glm3_6b_prefill_1024", "glm3_6b_prefill_8192"):
            rr = prefill_measure(dd, nm, WORKLOADS[nm], args, syn, steps=short)
            configs[nm] = {k: rr[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "prompt_tokens", "roofline")}
        nm = "glm4_9b_qkv_linear_b64"
        rr = qkv_linear_measure(dd, nm, WORKLOADS[nm], args, syn, steps=short)
        configs[nm] = {k: rr[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "tokens", "roofline")}
        nm = "glm4_9b_attention_block_b64"
        rr = attention_block_measure(dd, nm, WORKLOADS[nm], args, syn, steps=short)
        configs[nm] = {k: rr[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "tokens", "roofline")}
        torch.cuda.empty_cache()
        nm = "glm4_9b_long_131072"
        rr = split_kv_measure(dd, nm, WORKLOADS[nm], args, syn, steps=short)
        entry = {k: rr[k] for k in ("value", "unit", "ms_per_step", "steps", "parallelism", "kv_bytes_this_rank", "roofline", "issue")}
        if dd.world > 1:
            line["split_kv"] = entry
        else:
            configs[nm] = entry
    line["configs"] = configs
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                    help="run this workload alone (default: the headline workload plus the other configurations)")
    ap.add_argument("--headline-only", action="store_true", help="default run without the other configurations")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--settled", action="store_true",
                    help="decode workloads: pass CGLM_SEQ_CACHE_SETTLED (a launch may stream cache tiles while the previous one drains)")
    ap.add_argument("--e2e-f32", action="store_true", help="host-buffer runs with f32 activations instead of the f16 hand-off")
    ap.add_argument("--exchange", choices=["p2p", "nccl"], default="p2p", help="split-KV workload: how partials travel")
    ap.add_argument("--issue", choices=["graph", "eager"], default="graph", help="split-KV workload: replayed CUDA graph or eager launches")
    ap.add_argument("--step-graph", action="store_true",
                    help="with --workload: also time the step as one replayed CUDA graph (device-side n_past)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        name = args.workload or HEADLINE
        run_reference(args, name, WORKLOADS[name])
        return
    dd = Dist()
    if args.workload:
        line = run_single(args, dd, args.workload, WORKLOADS[args.workload])
    else:
        line = run_default(args, dd)
    if dd.rank == 0:
        par = line.get("parity")
        print(json.dumps(line), flush=True)
        if par is not None and (par["max_abs"] > par["tolerance"] or not par["cache_bit_exact"] or
                                par.get("e2e_max_abs", 0.0) > par.get("e2e_tolerance", 1.0)):
            dd.close()
            raise SystemExit(f"parity check failed: {par}")
    dd.close()


if __name__ == "__main__":
    main()
