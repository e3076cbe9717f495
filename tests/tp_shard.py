"""Host-side tensor-parallel sharding plan: which rows or block columns of every matrix a rank keeps.

Mirrors what `ob_model_create(tp_rank, tp_size)` does on the device side (csrc/model.cu, slice_weight): Q/K/V, gate, up
and the output matrix are split by output rows (whole heads for Q/K/V), attn_output and ffn_down by the contraction
dimension in units of 256-element super-blocks, so that every integer partial sum of a product is computed by exactly
one rank and only the fp32 sums over blocks cross ranks (the reference only has a layer split: backend/multi.rs:16-35;
a row range of a matrix is its QuantMatrix::rows view, engine/loader.rs:627-646).
"""
from __future__ import annotations

import numpy as np

BLOCK = {8: (34, 32), 12: (144, 256), 14: (210, 256), 2: (18, 32), 6: (22, 32), 20: (18, 32)}  # ggml type -> (bytes, elements) per block


def check(cfg: dict, tp_size: int) -> None:
    hd = cfg["head_dim"]
    if cfg["n_head_kv"] % tp_size or cfg["n_head"] % tp_size:
        raise ValueError("heads must divide by tp_size")
    if (cfg["n_head"] // tp_size * hd) % 256 or cfg["n_ff"] % (tp_size * 256):
        raise ValueError("per-rank contraction widths must be multiples of 256")
    if cfg["n_vocab"] % tp_size:
        raise ValueError("vocabulary must divide by tp_size")


def plan(cfg: dict, tp_size: int, rank: int) -> dict:
    """suffix -> ("rows", first, count) | ("cols", first_element, count_elements) | ("all",)"""
    check(cfg, tp_size)
    hd = cfg["head_dim"]
    q_l, kv_l, ff_l, v_l = cfg["n_head"] // tp_size * hd, cfg["n_head_kv"] // tp_size * hd, cfg["n_ff"] // tp_size, cfg["n_vocab"] // tp_size
    return {
        "attn_q": ("rows", rank * q_l, q_l), "attn_k": ("rows", rank * kv_l, kv_l), "attn_v": ("rows", rank * kv_l, kv_l),
        "attn_output": ("cols", rank * q_l, q_l),
        "ffn_gate": ("rows", rank * ff_l, ff_l), "ffn_up": ("rows", rank * ff_l, ff_l), "ffn_down": ("cols", rank * ff_l, ff_l),
        "output": ("rows", rank * v_l, v_l), "token_embd": ("all",), "attn_norm": ("all",), "ffn_norm": ("all",), "output_norm": ("all",),
    }


def slice_matrix(mat: dict, how: tuple) -> dict:
    """A matrix dict {"data": uint8 rows, "type", "in_dim", "out_dim"} cut as the plan says (copies)."""
    if how[0] == "all":
        return mat
    bb, be = BLOCK[mat["type"]]
    row_bytes = mat["in_dim"] // be * bb
    raw = np.ascontiguousarray(mat["data"], np.uint8).reshape(mat["out_dim"], row_bytes)
    if how[0] == "rows":
        _, first, count = how
        return {"data": raw[first:first + count].copy().reshape(-1), "type": mat["type"], "in_dim": mat["in_dim"], "out_dim": count}
    _, first, count = how
    if first % be or count % be:
        raise ValueError("column ranges are whole blocks")
    b0, nb = first // be, count // be
    return {"data": raw[:, b0 * bb:(b0 + nb) * bb].copy().reshape(-1), "type": mat["type"], "in_dim": count, "out_dim": mat["out_dim"]}


def merge_argmax(local_best: list[tuple[float, int]]) -> int:
    """Greedy token from per-rank (best logit, global index) pairs with the reference's tie rule: the last index among
    equal maxima wins (engine/sampling.rs:336-343, max_by with total_cmp)."""
    best = local_best[0]
    for cand in local_best[1:]:
        if cand[0] > best[0] or (cand[0] == best[0] and cand[1] > best[1]):
            best = cand
    return best[1]
