"""Tensor-parallel sharding on the CPU: two gloo ranks, each holding its slice, reproduce the single-process oracle.

What crosses ranks is only what the device path sends through NCCL: row-split products are gathered (bit-exact), the
two contraction-split products are summed (integer partials exact, fp32 sum to rounding), logits are gathered and the
greedy token obeys the last-index tie rule."""
import os
import socket
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def rank_main(rank, world, port, results):
    import torch
    import torch.distributed as dist

    import oracle as O
    from orangu_b200 import synth
    import tp_shard

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = dict(synth.CONFIGS["small"])
        tensors = synth.model_tensors(cfg, seed=17, n_layer=1)
        plan = tp_shard.plan(cfg, world, rank)
        rng = np.random.default_rng(3)
        x = rng.standard_normal(cfg["n_embd"]).astype(np.float32)
        checks = {}

        def gather(local):
            parts = [torch.empty_like(torch.from_numpy(local)) for _ in range(world)]
            dist.all_gather(parts, torch.from_numpy(local))
            return np.concatenate([p.numpy() for p in parts], axis=-1)

        # rows: every output element is computed by one rank from the whole input -> identical bits
        for suffix in ("attn_q", "attn_v", "ffn_gate", "output"):
            name = "output.weight" if suffix == "output" else f"blk.0.{suffix}.weight"
            full, mine = tensors[name], tp_shard.slice_matrix(tensors[name], plan[suffix])
            want = O.matmul_decode(x, 1, full["data"], full["type"], full["in_dim"], full["out_dim"])
            got = gather(O.matmul_decode(x, 1, mine["data"], mine["type"], mine["in_dim"], mine["out_dim"]))
            checks[suffix] = bool((got.view(np.uint32) == want.view(np.uint32)).all())

        # block columns: integer partials are the full product's, only the fp32 sum over blocks crosses ranks
        for suffix, width in (("attn_output", cfg["n_head"] * cfg["head_dim"]), ("ffn_down", cfg["n_ff"])):
            full = tensors[f"blk.0.{suffix}.weight"]
            xin = rng.standard_normal(width).astype(np.float32)
            xin = np.ascontiguousarray(torch.from_numpy(xin).clone().numpy())
            t = torch.from_numpy(xin)
            dist.broadcast(t, 0)
            xin = t.numpy()
            _, first, count = plan[suffix]
            mine = tp_shard.slice_matrix(full, plan[suffix])
            part = torch.from_numpy(O.matmul_decode(xin[first:first + count], 1, mine["data"], mine["type"], mine["in_dim"], mine["out_dim"]))
            dist.all_reduce(part)
            want = O.matmul_decode(xin, 1, full["data"], full["type"], full["in_dim"], full["out_dim"])
            scale = np.abs(want).max()
            checks[suffix + "_sum"] = bool(np.abs(part.numpy() - want).max() <= 1e-5 * scale)
            # integer partials of row 0
            bb = tp_shard.BLOCK[full["type"]][0]
            rb_full, rb_mine = full["in_dim"] // 256 * bb, mine["in_dim"] // 256 * bb
            isum_f, imin_f = O.row_partials(full["type"], full["data"][:rb_full], xin)
            isum_m, imin_m = O.row_partials(mine["type"], mine["data"][:rb_mine], xin[first:first + count])
            b0, nb = first // 256, count // 256
            checks[suffix + "_int"] = bool((isum_m == isum_f[b0:b0 + nb]).all() and (imin_m == imin_f[b0:b0 + nb]).all())

        # greedy token over sharded logits: ties go to the last index, across shards too
        v_l = cfg["n_vocab"] // world
        logits = np.zeros(cfg["n_vocab"], np.float32)
        logits[[5, v_l - 1, v_l + 7, cfg["n_vocab"] - 3]] = 2.5  # equal maxima in both shards
        mine = logits[rank * v_l:(rank + 1) * v_l]
        local = (float(mine.max()), int(rank * v_l + (len(mine) - 1 - np.argmax(mine[::-1]))))
        pairs = [None] * world
        dist.all_gather_object(pairs, local)
        checks["argmax"] = tp_shard.merge_argmax(pairs) == O.argmax(logits) == cfg["n_vocab"] - 3
        results[rank] = checks
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_process_products():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        port = free_port()
        procs = [ctx.Process(target=rank_main, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        for r in range(2):
            assert all(results[r].values()), results[r]


def test_plan_rejects_shapes_that_do_not_split():
    from orangu_b200 import synth
    import tp_shard

    with pytest.raises(ValueError):
        tp_shard.plan(dict(synth.CONFIGS["tiny"]), 2, 0)  # 2 heads x 64 per rank is not a multiple of 256
    p = tp_shard.plan(dict(synth.CONFIGS["8b"]), 8, 3)
    assert p["attn_k"] == ("rows", 3 * 128, 128) and p["ffn_down"] == ("cols", 3 * 1792, 1792)


# ---------------------------------------------------------------- the ranks' host-side meeting point (no device, no NCCL)
def _rendezvous_rank(rank, world, ident, n_steps, timeout_ms, out):
    import ctypes as C

    from orangu_b200 import capi

    missing = C.c_int32(-1)
    rc = capi.load().ob_tp_rendezvous_selftest(ident, rank, world, n_steps, timeout_ms, C.byref(missing))
    out.put((rank, rc, missing.value))


def _run_ranks(steps_of_rank, timeout_ms):
    import multiprocessing as mp

    ctx = mp.get_context("spawn")
    ident = os.urandom(128)
    out = ctx.Queue()
    procs = [ctx.Process(target=_rendezvous_rank, args=(r, len(steps_of_rank), ident, n, timeout_ms, out)) for r, n in enumerate(steps_of_rank)]
    for p in procs:
        p.start()
    got = sorted(out.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(30)
    return got


def test_ranks_that_all_arrive_pass_every_step():
    assert _run_ranks([50, 50, 50], 5000) == [(0, 0, -1), (1, 0, -1), (2, 0, -1)]


def test_a_rank_that_stays_away_costs_a_time_limit_on_the_host_and_is_named():
    """Rank 1 leaves after two steps (between steps, nothing in flight); rank 0 finds out at its third arrival, on the host, after
    the limit, and learns which rank is missing: the status ob_forward returns as OB_ERR_COMM with nothing launched."""
    import time

    t0 = time.time()
    got = _run_ranks([3, 2], 300)
    assert got[1] == (1, 0, -1)
    assert got[0] == (0, -7, 1)
    assert time.time() - t0 < 30
