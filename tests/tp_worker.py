"""One rank of a tensor-parallel run (started by test_gpu_tp.py through torch.distributed.run).

Every rank builds the same seeded synthetic model, registers its own slice of every matrix (rows of
Q/K/V/gate/up/output, block columns of Wo/down), prefills a prompt and decodes greedily.  Rank 0
compares logits and tokens with the CPU oracle's single-process run and prints one JSON line.

Across ranks only the fp32 order of the two per-layer sums changes, so this is a tolerance check, and
it is made on a shallow model: on random weights every further layer of int8 re-quantisation amplifies
a last-bit difference."""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    import torch
    import torch.distributed as dist

    import oracle as O
    import orangu_b200
    from orangu_b200 import capi, synth

    name, n_layer, n_prompt, n_decode = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    presliced = len(sys.argv) > 5 and sys.argv[5] == "presliced"  # every rank builds only its own shards
    absent = len(sys.argv) > 5 and sys.argv[5] == "absent"        # the last rank stays away from one step (made on the host, between steps)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    dist.init_process_group("gloo")
    torch.cuda.set_device(local)

    import ctypes as C
    box = [None]
    if rank == 0:
        buf = C.create_string_buffer(128)
        capi.check(None, capi.load().ob_tp_unique_id(buf))
        box[0] = buf.raw
    dist.broadcast_object_list(box, src=0)

    cfg = dict(synth.CONFIGS[name])
    cfg["n_layer"] = n_layer
    tensors = synth.model_tensors(cfg, seed=11, tp=(rank, world) if presliced else None)
    be = orangu_b200.CudaBackend.init(local)
    model = orangu_b200.LlamaModel(be, cfg, tensors, max_seq_len=n_prompt + n_decode + 16, max_batch_tokens=32,
                                   kv_pool_tokens=n_prompt + n_decode + 64, tp_rank=rank, tp_size=world, tp_unique_id=box[0], tp_presliced=presliced)
    toks = np.random.default_rng(5).integers(0, cfg["n_vocab"], n_prompt).astype(np.uint32)
    kv = model.new_kv_cache(n_prompt + n_decode + 8)
    logits = [model.forward(kv, toks, 0)]
    got = [int(np.argmax(logits[0]))]
    for i in range(n_decode):
        logits.append(model.forward(kv, [got[-1]], n_prompt + i))
        got.append(be.argmax(logits[-1]))

    if absent:
        # One more step, which the last rank does not take part in (as if it had refused the call on its own arguments, or
        # died between steps).  The others meet on the host first, find it missing after OB_TP_RENDEZVOUS_MS, and return
        # OB_ERR_COMM without having launched anything; afterwards the model refuses further steps.
        import time

        outcome = None
        if rank != world - 1:
            t0 = time.time()
            try:
                model.forward(kv, [got[-1]], n_prompt + n_decode)
                outcome = {"status": 0}
            except orangu_b200.OranguError as e:
                outcome = {"status": e.status, "message": e.message, "seconds": time.time() - t0, "kv_len": len(kv)}
            try:
                model.forward(kv, [got[-1]], n_prompt + n_decode)
                outcome["second"] = 0
            except orangu_b200.OranguError as e:
                outcome["second"] = e.status
        outcomes = [None] * world
        dist.all_gather_object(outcomes, outcome)
        if rank == 0:
            print(json.dumps({"world": world, "absent": outcomes}), flush=True)
        dist.barrier()
        model.close()
        dist.destroy_process_group()
        return

    # every rank must hold the same logits (the gather completed) -- compare a digest through the store
    digest = [float(np.sum(np.stack(logits).astype(np.float64)))]
    all_digests = [None] * world
    dist.all_gather_object(all_digests, digest)

    if rank == 0:
        ref = O.Model(cfg, synth.model_tensors(cfg, seed=11) if presliced else tensors)
        rkv = ref.new_kv(n_prompt + n_decode + 8, f16=True)
        want = [ref.forward(rkv, toks, 0)]
        want_tok = [O.argmax(want[0])]
        first_diverged = None
        for i in range(n_decode):
            # teacher-forced with the GPU's token so that one flipped argmax does not void the later comparisons
            want.append(ref.forward(rkv, [got[i]], n_prompt + i))
            want_tok.append(O.argmax(want[-1]))
            if first_diverged is None and want_tok[-1] != got[i + 1]:
                first_diverged = i + 1
        err = [float(np.abs(a - b).max()) for a, b in zip(logits, want)]
        scale = float(np.abs(np.stack(want)).max())
        digest_all = float(np.sum(np.stack(logits).astype(np.float64)))
        print(json.dumps({"world": world, "digest": digest_all, "max_abs_err": max(err), "prefill_err": err[0], "logit_scale": scale,
                          "tokens_equal": first_diverged is None and got[0] == want_tok[0], "first_diverged": first_diverged,
                          "ranks_agree": all(d == all_digests[0] for d in all_digests), "launches": be.launch_count()}), flush=True)
    dist.barrier()
    model.close() if hasattr(model, "close") else None
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
