"""Small, self-contained runs of single kernels of the path, for timing them alone and for capturing them under a profiler
(few launches, a few hundred MB on the device, inputs larger than L2 where that matters).

    python -m orangu_b200.profile_kernels fused --model 8b --layers 4 --variant 3 --iters 2
        the fused single-token decode kernels of every layer back to back (ob_profile_gemv):
        1 norm + q/k/v + RoPE + KV append, 2 attention output + residual, 3 norm + gate/up + SwiGLU, 4 down + residual,
        5 norm + output projection
    python -m orangu_b200.profile_kernels matmul --type 12 --out-dim 14336 --in-dim 4096 --tokens 512 --order prefill --iters 3
        one many-token product on device-resident buffers (ob_matmul_device): the tcgen05 kernels at 16 tokens or more
    python -m orangu_b200.profile_kernels decode --model 8b --layers 2 --context 512 --steps 4
        a few whole decode steps of a short model (launch lists)

Prints microseconds per launch from CUDA events on the library's stream."""
from __future__ import annotations

import argparse
import ctypes as C
import time

import numpy as np


def _model(be, name, layers, vocab, **kw):
    from . import LlamaModel, synth

    cfg = dict(synth.CONFIGS[name])
    if layers:
        cfg["n_layer"] = layers
    if vocab:
        cfg["n_vocab"] = vocab
    return cfg, LlamaModel(be, cfg, synth.model_tensors(cfg, seed=1), **kw)


def fused(args):
    import orangu_b200

    be = orangu_b200.CudaBackend.init(0)
    cfg, m = _model(be, args.model, args.layers, args.vocab, max_seq_len=256, max_batch_tokens=16)
    kv = m.new_kv_cache(64)
    m.forward(kv, [1, 2, 3], 0)
    m.forward(kv, [4], 3)  # one decode step: the fused kernels read its position and page table
    for v in args.variant:
        ms, nbytes, nl = m.profile_gemv(12, args.iters, v)
        us = ms * 1e3 / args.iters / nl
        print(f"variant {v}: {us:8.2f} us per launch, {nbytes / nl / 1e6:7.2f} MB -> {nbytes / nl / us / 1e6:6.3f} TB/s ({nl} launches per pass)", flush=True)


def matmul(args):
    import torch

    import orangu_b200
    from orangu_b200 import QuantMatrix, capi, synth

    be = orangu_b200.CudaBackend.init(0)
    L = capi.load()
    w = synth.matrix(args.type, args.out_dim, args.in_dim, 42)
    h = be._weight(QuantMatrix(w["data"], args.type, args.in_dim, args.out_dim))
    x = torch.from_numpy(synth.normal(args.tokens * args.in_dim, 43)).cuda()
    y = torch.empty(args.tokens * args.out_dim, dtype=torch.float32, device="cuda")
    decode = 0 if args.order == "prefill" else 1
    for it in range(args.iters + 1):  # the first call is a warm-up
        if it == 1:
            be.synchronize()
            t0 = time.perf_counter()
        capi.check(be._h, L.ob_matmul_device(be._h, x.data_ptr(), args.tokens, h, y.data_ptr(), decode, None))
    be.synchronize()
    dt = (time.perf_counter() - t0) / args.iters
    print(f"type {args.type} [{args.out_dim} x {args.in_dim}] x {args.tokens} tokens, {args.order} order: {dt * 1e6:9.1f} us per call "
          f"(quantize + product), {2 * args.tokens * args.out_dim * args.in_dim / dt / 1e12:6.2f} Tops/s", flush=True)


def decode(args):
    import orangu_b200

    be = orangu_b200.CudaBackend.init(0)
    cfg, m = _model(be, args.model, args.layers, args.vocab, max_seq_len=args.context + 64, max_batch_tokens=512, kv_pool_tokens=args.context + 128)
    kv = m.new_kv_cache(args.context + 48)
    toks = np.random.default_rng(0).integers(0, cfg["n_vocab"], args.context).astype(np.uint32)
    first = m.forward_maybe_sampling(kv, toks, 0)
    m.decode_loop([kv], [first], 2)
    m.decode_loop([kv], [first], args.steps)
    print(f"{args.model} x {cfg['n_layer']} layers, context {len(kv)}: {be.last_device_ms() / args.steps * 1e3:8.1f} us per step", flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    f = sub.add_parser("fused")
    f.add_argument("--model", default="8b")
    f.add_argument("--layers", type=int, default=4)
    f.add_argument("--vocab", type=int, default=4096)
    f.add_argument("--variant", type=int, nargs="+", default=[1, 2, 3, 4])
    f.add_argument("--iters", type=int, default=2)
    g = sub.add_parser("matmul")
    g.add_argument("--type", type=int, default=12)
    g.add_argument("--out-dim", type=int, default=14336)
    g.add_argument("--in-dim", type=int, default=4096)
    g.add_argument("--tokens", type=int, default=512)
    g.add_argument("--order", choices=["prefill", "decode"], default="prefill")
    g.add_argument("--iters", type=int, default=3)
    d = sub.add_parser("decode")
    d.add_argument("--model", default="8b")
    d.add_argument("--layers", type=int, default=2)
    d.add_argument("--vocab", type=int, default=4096)
    d.add_argument("--context", type=int, default=512)
    d.add_argument("--steps", type=int, default=4)
    args = ap.parse_args()
    {"fused": fused, "matmul": matmul, "decode": decode}[args.cmd](args)


if __name__ == "__main__":
    main()
