#!/usr/bin/env python
"""Decode throughput of the quantized Llama-style hot path on B200, next to the CPU restatement.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): random-init 8B-shape decoder in Q4_K_M (Q6_K for output and attn_v), 32 layers,
d_model 4096, 32 query / 8 KV heads of 128, FFN 14336, vocab 128256; one sequence with a 4096-token
context of uniformly random token ids (prefilled through the same library), then greedy decode at
batch 1.  A step is one decode step (one new token per sequence).  N > 1 runs the same model
tensor-parallel over N GPUs of one node (one process per GPU, NCCL all-reduce after the attention-output
and FFN-down products), so the total work is fixed: strong scaling.

One JSON line on stdout (rank 0):
  value      tokens/s over the K timed steps with the loop resident on the device (ob_decode_loop),
             device time from CUDA events, max over ranks
  e2e        the same metric through ob_decode_greedy, one host round trip per token: the token id and
             position go up from pinned host memory and the sampled id comes back, inside the timed region
  roofline   the dominant kernel (Q4_K single-token GEMV) run alone over every layer's Q4_K matrices,
             timed with CUDA events on its launching stream, against the measured HBM copy bandwidth
  cpu_baseline  the CPU restatement of the reference's path (oracle/) timed on this host's cores

--impl reference times that CPU path as the whole job.  The reference engine is Rust and there is no Rust
toolchain on these machines, so the arm runs oracle/, its line-by-line C++ restatement.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))  # tests/oracle.py: the ctypes binding of the CPU oracle

# torch.distributed.run exports OMP_NUM_THREADS=1; the synthetic-weight generator and the CPU oracle are OpenMP code and
# would take minutes on one thread.  Give every rank its share of the host cores (before any OpenMP runtime starts).
if int(os.environ.get("WORLD_SIZE", "1")) > 1 and os.environ.get("OMP_NUM_THREADS", "1") == "1":
    # the reference arm works on rank 0 alone (the other ranks return at once): it gets all the cores
    _ranks_at_work = 1 if "reference" in sys.argv else int(os.environ.get("LOCAL_WORLD_SIZE", os.environ["WORLD_SIZE"]))
    os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 1) // _ranks_at_work))

import numpy as np  # noqa: E402

METRIC = "decode tok/s (8B-shape Q4_K_M, bs1 & bs64); quantized GEMV HBM GB/s vs peak"
UNIT = "tok/s"
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="8b", help="shape from orangu_b200.synth.CONFIGS")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only; invalidates the number)")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--batch64-steps", type=int, default=16, help="steps of the 64-sequence decode measured as an extra (0 = skip)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi clock / throttle-reason samples every 200 ms while a timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.path = tempfile.mktemp(prefix="ob_clocks_", suffix=".csv")
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------- weights
def model_config(args):
    from orangu_b200 import synth

    cfg = dict(synth.CONFIGS[args.model])
    if args.layers:
        cfg["n_layer"] = args.layers
    return cfg


def build_tensors(cfg, rank: int, world: int, barrier):
    """Seeded synthetic tensors.  The generator is counter-based, so with several ranks every rank makes only its own
    tensor-parallel shards (the same bytes the whole tensors hold there) and hands them over as they are (tp_presliced)."""
    from orangu_b200 import synth

    return synth.model_tensors(cfg, seed=20240, tp=(rank, world) if world > 1 else None)


def algorithmic_bytes_per_token(cfg, context: int) -> int:
    """Quantized weight bytes every layer and the output projection read for one token, the f32 norm vectors,
    and the fp16 K/V of the attended window.  The embedding row and activations are not counted."""
    from orangu_b200.backend import tensor_byte_size

    e, hd = cfg["n_embd"], cfg["head_dim"]
    qd, kvd, ff, V = cfg["n_head"] * hd, cfg["n_head_kv"] * hd, cfg["n_ff"], cfg["n_vocab"]
    q4 = lambda o, i: o * tensor_byte_size(12, i)  # noqa: E731
    q6 = lambda o, i: o * tensor_byte_size(14, i)  # noqa: E731
    layer = q4(qd, e) + q4(kvd, e) + q6(kvd, e) + q4(e, qd) + 2 * q4(ff, e) + q4(e, ff) + 2 * e * 4
    return cfg["n_layer"] * layer + q6(V, e) + e * 4 + 2 * kvd * 2 * cfg["n_layer"] * context



# ---------------------------------------------------------------------------------------- single products (configs 1 and 2)
def operator_gemv_rooflines(be, peak):
    """The Backend::matmul operator at one token on device-resident buffers: BASELINE.json's single Q8_0 GEMV (4096 x 4096) and
    the Q4_K / Q6_K sweep shapes.  A single product moves 10-50 MB -- a few microseconds -- so it is timed inside a CUDA graph
    of `reps` back-to-back launches; the launches rotate over enough copies of the matrix to exceed the 126 MB L2, so every
    launch reads its weights from HBM.  Algorithmic bytes = GGUF bytes of the matrix + the fp32 input and output vectors."""
    import torch

    from orangu_b200 import QuantMatrix, capi, synth
    from orangu_b200.backend import tensor_byte_size

    L = capi.load()
    out = {}
    cases = [("config 1: Q8_0 4096x4096", 8, 4096, 4096)] + [
        (f"config 2: {'Q4_K' if t == 12 else 'Q6_K'} {o}x{i}", t, o, i) for t in (12, 14) for (o, i) in ((4096, 4096), (14336, 4096), (4096, 14336))]
    stream = torch.cuda.Stream()
    for name, t, out_dim, in_dim in cases:
        wbytes = out_dim * tensor_byte_size(t, in_dim)
        copies = max(2, -(-160_000_000 // wbytes))
        mats = [synth.matrix(t, out_dim, in_dim, 900 + c) for c in range(copies)]
        handles = [be._weight(QuantMatrix(m["data"], t, in_dim, out_dim)) for m in mats]
        x = torch.randn(in_dim, device="cuda", dtype=torch.float32)
        y = torch.empty(out_dim, device="cuda", dtype=torch.float32)
        reps = 4 * copies
        with torch.cuda.stream(stream):
            for h in handles:  # warm-up outside capture: scratch allocation, one-time kernel attributes
                capi.check(be._h, L.ob_matmul_device(be._h, x.data_ptr(), 1, h, y.data_ptr(), 0, stream.cuda_stream))
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for r in range(reps):
                    capi.check(be._h, L.ob_matmul_device(be._h, x.data_ptr(), 1, handles[r % copies], y.data_ptr(), 0, stream.cuda_stream))
            g.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(5):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (5 * reps)
        nbytes = wbytes + 4 * (in_dim + out_dim)
        out[name] = {"avg_launch_us": us, "algorithmic_bytes": nbytes, "GB/s": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak,
                     "timed": f"CUDA graph of {reps} products rotating over {copies} copies of the matrix ({copies * wbytes / 1e6:.0f} MB > L2), 5 replays",
                     "kernels_per_product": 1}
        for h in handles:
            L.ob_weight_release(be._h, h)
            be._weights.remove(h)
    return out


# ---------------------------------------------------------------------------------------- 70B shape under tensor parallel
def run_70b(be, rank, world, uid, barrier, max_over_ranks, peak):
    """BASELINE.json's last configuration: 70B-shape Q4_K_M decoder (80 layers, d_model 8192, 64 query / 8 KV heads, FFN 28672),
    tensor parallel over this run's GPUs, batch-1 and batch-32 greedy decode at an 8192-token context.  Every rank generates
    only its own shards.  Reports tokens/s (device time, max over ranks) and the per-GPU fraction of the HBM roofline."""
    import orangu_b200
    from orangu_b200 import synth

    cfg = dict(synth.CONFIGS["70b"])
    ctx_len, steps1, steps32, n_seq = 8192, 8, 4, 32
    t0 = time.time()
    tensors = synth.model_tensors(cfg, seed=20270, tp=(rank, world))
    t_gen = time.time() - t0
    per_seq = ctx_len + 64
    model = orangu_b200.LlamaModel(be, cfg, tensors, max_seq_len=per_seq, max_batch_tokens=512, kv_pool_tokens=n_seq * per_seq + 64,
                                   tp_rank=rank, tp_size=world, tp_unique_id=uid, tp_presliced=True)
    del tensors
    kv = model.new_kv_cache(per_seq)
    prompt = np.random.default_rng(13).integers(0, cfg["n_vocab"], ctx_len).astype(np.uint32)
    t0 = time.time()
    first = model.forward_maybe_sampling(kv, prompt, 0)
    t_prefill = time.time() - t0
    model.decode_loop([kv], [first], 3)
    barrier()
    model.decode_loop([kv], [int(first)], steps1)
    ms1 = max_over_ranks(be.last_device_ms()) / steps1
    kv.truncate(ctx_len)
    caches = [kv]
    for _ in range(n_seq - 1):
        c = model.new_kv_cache(per_seq)
        c.copy_prefix_from(kv, ctx_len)
        caches.append(c)
    firsts = [int(first)] * n_seq
    model.decode_loop(caches, firsts, 2)
    barrier()
    model.decode_loop(caches, firsts, steps32)
    ms32 = max_over_ranks(be.last_device_ms()) / steps32
    w_bytes = algorithmic_bytes_per_token(cfg, 0)
    kv_bytes = algorithmic_bytes_per_token(cfg, ctx_len) - w_bytes
    out = {"workload": "70B-shape Llama decoder, Q4_K_M (Q6_K output and attn_v), 80 layers, context 8192 prefilled through the library",
           "parallelism": f"tp{world}", "setup_s": {"synthetic_shards": round(t_gen, 1), "prefill_8192": round(t_prefill, 1)},
           "batch1": {"value": 1e3 / ms1, "unit": UNIT, "ms_per_step": ms1, "steps": steps1,
                      "hbm_frac_per_gpu": (w_bytes + kv_bytes) / world / (ms1 * 1e-3) / 1e9 / peak},
           "batch32": {"value": n_seq * 1e3 / ms32, "unit": UNIT, "ms_per_step": ms32, "steps": steps32, "sequences": n_seq,
                       "kv": "31 sequences share the first one's prefilled pages by device copy (KvCache::copy_prefix_from)",
                       "hbm_frac_per_gpu": (w_bytes + n_seq * kv_bytes) / world / (ms32 * 1e-3) / 1e9 / peak}}
    model.close()
    return out

# ---------------------------------------------------------------------------------------- CPU arm
def cpu_decode_tokens_per_s(cfg, tensors, budget_s: float, max_tokens: int):
    """Times greedy decode of the CPU oracle on all host cores.  Bounded: a short prompt (the CPU prefill of a
    4096-token context would take minutes), then as many single-token steps as fit the budget."""
    import oracle as O

    ref = O.Model(cfg, tensors)
    cores = O.hardware_threads()
    prompt = np.random.default_rng(7).integers(0, cfg["n_vocab"], 4).astype(np.uint32)
    kv = ref.new_kv(4 + max_tokens + 2, f16=True)
    tok = O.argmax(ref.forward(kv, prompt, 0))
    tok = O.argmax(ref.forward(kv, [tok], 4))  # one untimed step: page the weights in
    n, t0 = 0, time.perf_counter()
    while n < max_tokens:
        tok = O.argmax(ref.forward(kv, [tok], 5 + n))
        n += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return n / dt, cores, f"{n} greedy decode steps at batch 1 after a 4-token prompt (context {5}..{5 + n}), {dt:.1f} s, OpenMP over output rows"


def run_reference(args, rank: int, world: int):
    """The reference arm: the reference's CPU path (its C++ restatement under oracle/) as the whole job."""
    if rank != 0:
        return
    from orangu_b200 import synth  # noqa: F401  (the synthetic tensors are shared with our arm)

    cfg = model_config(args)
    tensors = build_tensors(cfg, 0, 1, lambda: None)
    import oracle as O

    ref = O.Model(cfg, tensors)
    cores = O.hardware_threads()
    prompt = np.random.default_rng(7).integers(0, cfg["n_vocab"], 4).astype(np.uint32)
    kv = ref.new_kv(8 + args.warmup + args.steps, f16=True)
    tok = O.argmax(ref.forward(kv, prompt, 0))
    pos = 4
    for _ in range(args.warmup):
        tok = O.argmax(ref.forward(kv, [tok], pos))
        pos += 1
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok = O.argmax(ref.forward(kv, [tok], pos))
        pos += 1
    dt = time.perf_counter() - t0
    value = args.steps / dt
    sample = (f"{args.steps} greedy decode steps at batch 1 after a 4-token prompt; the 4096-token context is not prefilled on the CPU "
              f"(its attention share at that length is under 10% of a step)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": f"{args.model}-shape Q4_K_M decode, batch 1, CPU path of the reference restated in C++ (oracle/); no Rust toolchain here",
                   "n_layer": cfg["n_layer"], "host_cores": cores, "context": f"{4 + args.warmup}..{4 + args.warmup + args.steps} positions (a 4-token prompt; the GPU arm decodes at {args.context})"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------- our arm
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    import orangu_b200
    from orangu_b200 import capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cfg = model_config(args)
    t_build = time.time()
    tensors = build_tensors(cfg, rank, world, barrier)
    t_build = time.time() - t_build

    be = orangu_b200.CudaBackend.init(local_rank)

    def make_uid():
        """A fresh communicator id from rank 0, the same 128 bytes on every rank."""
        if world == 1:
            return None
        buf = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            import ctypes as C

            cbuf = (C.c_uint8 * 128)()
            capi.check(None, capi.load().ob_tp_unique_id(cbuf))
            buf.copy_(torch.tensor(list(cbuf), dtype=torch.uint8))
        dist.broadcast(buf, 0)
        return bytes(buf.cpu().tolist())

    uid = make_uid()

    ctx_len, K, W = args.context, args.steps, args.warmup
    b64 = args.batch64_steps
    margin = 2 * (K + W) + 96
    per_seq = ctx_len + margin
    model = orangu_b200.LlamaModel(be, cfg, tensors, max_seq_len=per_seq, max_batch_tokens=512,
                                   kv_pool_tokens=per_seq + (63 * (ctx_len + b64 + 64 + 16) if b64 else 0) + 64,
                                   tp_rank=rank, tp_size=world, tp_unique_id=uid, tp_presliced=world > 1)
    kv = model.new_kv_cache(per_seq)
    prompt = np.random.default_rng(11).integers(0, cfg["n_vocab"], ctx_len).astype(np.uint32)
    t_prefill = time.time()
    first = model.forward_maybe_sampling(kv, prompt, 0)
    t_prefill = time.time() - t_prefill

    sampler = ClockSampler(local_rank)
    # ---- value: device-resident loop -------------------------------------------------------------
    model.decode_loop([kv], [first], max(W, 3))
    barrier()
    sampler.start()
    launches0 = be.launch_count()
    out = model.decode_loop([kv], [int(first)], K)
    dev_ms = be.last_device_ms()
    launches = be.launch_count() - launches0
    barrier()
    dev_ms = max_over_ranks(dev_ms)
    value = K / (dev_ms * 1e-3)

    # ---- e2e: one host round trip per token --------------------------------------------------------
    tok = int(out[-1, 0])
    for _ in range(max(W, 3)):
        tok = model.decode_greedy(kv, tok)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        tok = model.decode_greedy(kv, tok)
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    clocks = sampler.stop()
    T = model.max_batch_tokens
    h2d = ((T * 12 + 15) // 16) * 16 + T * 8  # the step's metadata block: token ids, positions, window lengths, page-table pointers
    e2e = {"value": K / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "ms_per_step": e2e_s / K * 1e3}

    # ---- roofline of the dominant kernel --------------------------------------------------------------
    peak, peak_kind = measured_peak_gbs()
    iters = 20
    step_bytes = algorithmic_bytes_per_token(cfg, len(kv)) // world
    # the fused decode kernels, each timed back to back over all layers (every launch streams its own layer's weights; on
    # several GPUs: this rank's slices); the gate/up kernel carries 43% of a token's bytes and is the one reported
    names = {1: "attn_q/k/v + RoPE + KV append", 2: "attn_output + residual", 3: "ffn_gate + ffn_up + SwiGLU + int8 output",
             4: "ffn_down + residual", 5: "output projection"}
    kernels = {}
    for v in (1, 2, 3, 4, 5):
        ms, nbytes, nl = model.profile_gemv(12, iters, v)
        us = max_over_ranks(ms * 1e3 / (iters * nl))
        kernels[names[v]] = {"avg_launch_us": us, "algorithmic_bytes_per_launch": nbytes // nl, "GB/s": nbytes / nl / us / 1e3,
                             "frac": nbytes / nl / us / 1e3 / peak, "launches_per_token": nl}
    dom = kernels[names[3]]
    kname = "stream_gemv_kernel<lanes per row pair 32, Q4_K> (" + names[3] + ")"
    per_launch_s, bytes_per_launch, timed = dom["avg_launch_us"] * 1e-6, dom["algorithmic_bytes_per_launch"], iters * cfg["n_layer"]
    achieved = bytes_per_launch / per_launch_s / 1e9
    # DRAM read + write bytes of one launch of the gate/up kernel of the 8B shape on one GPU, from the ncu capture of this kernel on
    # a two-layer model of the same shape (a capture cannot run inside a timed bench): dram__bytes_read.sum + dram__bytes_write.sum
    traffic = 66128896 + 896000 if world == 1 and (cfg["n_embd"], cfg["n_ff"]) == (4096, 14336) else None
    roofline = {"bound": "hbm", "kernel": kname, "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "traffic_source": "profiles/decode_step_kernels_8b_ncu_full.md" if traffic else None,
                "launches_timed": timed, "avg_launch_us": per_launch_s * 1e6, "algorithmic_bytes_per_launch": bytes_per_launch,
                "step": {"algorithmic_bytes_per_token_per_gpu": step_bytes, "achieved": step_bytes / (dev_ms * 1e-3 / K) / 1e9,
                         "frac": step_bytes / (dev_ms * 1e-3 / K) / 1e9 / peak},
                "kernels": kernels}
    if world == 1:
        roofline["operator_gemv"] = operator_gemv_rooflines(be, peak)

    # ---- batch 64 extra ---------------------------------------------------------------------------------
    batch64 = None
    if b64:
        caches = [kv]
        for _ in range(63):
            c = model.new_kv_cache(ctx_len + b64 + 64)
            c.copy_prefix_from(kv, ctx_len)
            caches.append(c)
        kv.truncate(ctx_len)
        firsts = [int(first)] * 64
        model.decode_loop(caches, firsts, 3)
        barrier()
        out64 = model.decode_loop(caches, firsts, b64)
        ms64 = max_over_ranks(be.last_device_ms())
        batch64 = {"value": 64 * b64 / (ms64 * 1e-3), "unit": UNIT, "steps": b64, "ms_per_step": ms64 / b64, "sequences": 64,
                   "context": ctx_len, "kv": "63 sequences share the first one's prefilled pages by device copy (KvCache::copy_prefix_from)",
                   "algorithmic_bytes_per_step": algorithmic_bytes_per_token(cfg, 0) + 64 * (algorithmic_bytes_per_token(cfg, ctx_len) - algorithmic_bytes_per_token(cfg, 0))}
        batch64["hbm_frac_per_gpu"] = batch64["algorithmic_bytes_per_step"] / world / (ms64 / b64 * 1e-3) / 1e9 / peak
        batch64["parallelism"] = f"tp{world}"

    # ---- serving extra: eight request threads through the slot pool and the decode window (one GPU) ------------------------
    serving = None
    if b64 and world == 1:
        import threading

        from orangu_b200 import SlotPool

        for c in caches[1:]:
            c.close()  # their pages go back to the pool the slots draw from
        n_req, n_prompt, n_new = 8, 256, 33
        pool = SlotPool(model, n_slots=n_req, slot_capacity_tokens=n_prompt + n_new + 16, batch_wait_ms=0, prefill_batch=512, batch_decode=True)
        prompts = [np.random.default_rng(100 + i).integers(0, cfg["n_vocab"], n_prompt).astype(np.uint32) for i in range(n_req)]
        done_tokens, failures = [0] * n_req, []

        def request(i):
            try:
                with pool.try_acquire() as slot:
                    tok = slot.prefill(prompts[i])
                    for _ in range(n_new - 1):
                        tok = slot.decode(tok)
                        done_tokens[i] += 1
            except Exception as e:  # noqa: BLE001
                failures.append(repr(e)[:200])

        threads = [threading.Thread(target=request, args=(i,)) for i in range(n_req)]
        t0 = time.perf_counter()
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        wall = time.perf_counter() - t0
        st = pool.stats()
        pool.close()
        serving = {"requests": n_req, "prompt_tokens": n_prompt, "new_tokens": n_new, "wall_s": wall,
                   "tok_s_generated": sum(done_tokens) / wall, "tok_s_prefill_and_decode": (n_req * n_prompt + sum(done_tokens)) / wall,
                   "decode_batches": st["batches"], "mean_decode_batch": st["batched_seqs"] / max(1, st["batches"]), "refused": st["refused"],
                   "failures": failures, "how": "one thread per request: ob_slot_acquire, ob_slot_prefill, ob_slot_decode per token through the default 4 ms "
                   "collection window, ob_slot_release; on-demand KV pages; host round trip per token"}

    # ---- CPU baseline (rank 0, single GPU runs only) --------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, cores, sample = cpu_decode_tokens_per_s(cfg, tensors, budget_s=15.0, max_tokens=400)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    # ---- 70B shape, tensor parallel (2, 4, 8 GPUs): batch 1 and batch 32 at context 8192 --------------------------------
    model70b = None
    if world > 1 and args.model == "8b" and not args.layers and os.environ.get("OB_BENCH_70B", "1") != "0":
        model.close()
        model = None
        try:
            model70b = run_70b(be, rank, world, make_uid(), barrier, max_over_ranks, peak)
        except Exception as e:  # the headline line must not depend on the extra
            model70b = {"error": f"{type(e).__name__}: {e}"[:300]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": max(W, 3), "ms_per_step": dev_ms / K,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": f"{args.model}-shape Llama decoder, Q4_K_M (Q6_K output and attn_v), {cfg['n_layer']} layers, greedy decode at batch 1, "
                                   f"context {ctx_len} prefilled through the library, fp16 KV in 16-token pages",
                       "parallelism": f"tp{world}", "context": ctx_len, "batch": 1,
                       "l2": "inputs larger than L2: every step streams the whole quantized model (4.4 GB) through a 126 MB L2",
                       "attention": "windows above 1024 positions use the flash-decode kernel (not bit-exact: at this shape and context the logits differ from the "
                                    "CPU oracle by 0.10 max-abs at 2 layers and 0.17 at 4, above the 2e-2 bar, with identical greedy top-1; "
                                    "tests/test_gpu_model.py measures it); shorter windows use the exact-order kernels and are bit-identical",
                       "setup_s": {"synthetic_weights": round(t_build, 1), "prefill": round(t_prefill, 1)},
                       "launches_before_timed_region": int(launches0)},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu,
        }
        if batch64:
            line["batch64"] = batch64
        if serving:
            line["serving"] = serving
        if model70b:
            line["model70b"] = model70b
        print(json.dumps(line), flush=True)
    if model is not None:
        model.close()
    be.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
