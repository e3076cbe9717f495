"""Tensor parallel on 2 (and 4) GPUs of one node: one process per GPU, NCCL for the two sums per layer.

Skipped when the box has fewer GPUs than ranks.  The ranks are child processes started through
torch.distributed.run on 127.0.0.1; rank 0 reports the comparison with the CPU oracle."""
import json
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def gpu_count():
    import torch

    return torch.cuda.device_count()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(world, args, timeout=900, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="8", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(HERE, "tp_worker.py")] + [str(a) for a in args]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert lines, p.stdout[-2000:] + p.stderr[-2000:]
    return json.loads(lines[-1])


@pytest.mark.parametrize("world,name,n_layer", [(2, "small", 1), (2, "small", 3), (2, "1b", 2), (4, "1b", 2), (8, "8b", 2), (8, "8b", 1)])
def test_tensor_parallel_matches_the_oracle(world, name, n_layer):
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    r = run_ranks(world, [name, n_layer, 40, 12])
    assert r["ranks_agree"], r
    # Across ranks only the fp32 order of the two per-layer sums changes.  One layer: the bar itself, 2e-2.  Deeper: the next
    # int8 quantisation turns a few last-bit differences into one-code differences, so the bound scales with the logits.
    bound = 2e-2 if n_layer == 1 else 2e-2 * max(1.0, r["logit_scale"])
    assert r["max_abs_err"] < bound, r
    assert r["launches"] > 0


def test_peer_exchange_and_nccl_forms_agree():
    """The single-token step exchanges partials through peer memory (rank-ordered sums); OB_TP_PEER=0 keeps ncclAllReduce.
    Both have to stay within the same bound of the oracle, and of each other."""
    if gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    a = run_ranks(2, ["small", 1, 40, 12])
    b = run_ranks(2, ["small", 1, 40, 12], OB_TP_PEER="0")
    assert a["ranks_agree"] and b["ranks_agree"], (a, b)
    assert a["max_abs_err"] < 2e-2 and b["max_abs_err"] < 2e-2, (a, b)
    assert a["launches"] != b["launches"], "both runs took the same kernels: the switch did nothing"


def test_presliced_shards_give_the_same_model():
    """Every rank builds only its own shards (synth.model_tensors(tp=...), ob_model_desc.tp_presliced): the logits are the
    ones the whole tensors give, bit for bit (same digest), since the shards hold the same bytes."""
    if gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    whole = run_ranks(2, ["small", 2, 40, 6])
    shards = run_ranks(2, ["small", 2, 40, 6, "presliced"])
    assert shards["ranks_agree"], shards
    assert shards["digest"] == whole["digest"], (whole, shards)


def test_a_rank_that_stays_away_from_a_step_is_found_on_the_host_before_anything_is_launched():
    """Failure made on the host, between steps: the last of two ranks skips one step.  The other meets nobody at the host-side
    rendezvous, gives up after OB_TP_RENDEZVOUS_MS, reports OB_ERR_COMM naming the rank, leaves its KV cache where it was and
    refuses further steps -- no kernel or collective was enqueued, so no GPU waits for anybody."""
    if gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = run_ranks(2, ["small", 1, 20, 2, "absent"], OB_TP_RENDEZVOUS_MS="1500")
    present, away = r["absent"]
    assert away is None
    assert present["status"] == -7 and "rank 1 did not arrive" in present["message"] and "nothing was launched" in present["message"]
    assert 1.4 < present["seconds"] < 20 and present["kv_len"] == 22
    assert present["second"] == -7


def test_exchange_wait_runs_out_and_reports_instead_of_hanging():
    """One GPU, no fault, no hang: a two-rank exchange whose second rank's slot is local memory nobody writes in some rounds.
    The consumer kernel's wait ends after the limit (50 ms here), the round is reported as OB_ERR_COMM (-7), and the rounds
    after it -- delivered again -- give the right sums: the context stays usable."""
    import ctypes as C
    import time

    import numpy as np

    import orangu_b200
    from orangu_b200 import capi

    be = orangu_b200.CudaBackend.init(0)
    L = capi.load()
    try:
        delivers = np.array([1, 0, 1, 1, 0, 1], np.uint8)
        sums = np.zeros(len(delivers), np.float32)
        t0 = time.time()
        rc = L.ob_tp_exchange_selftest(be._h, 4096, 50, len(delivers), delivers.ctypes.data, sums.ctypes.data)
        dt = time.time() - t0
        assert rc == -7, rc
        assert b"did not deliver" in L.ob_last_error(be._h)
        assert sums.tolist() == [3.0, -1.0, 3.0, 3.0, -1.0, 3.0], sums
        assert 0.09 < dt < 5.0, dt  # two waits of 50 ms ran out, nothing spun on
        ok = np.ones(4, np.uint8)
        sums = np.zeros(4, np.float32)
        assert L.ob_tp_exchange_selftest(be._h, 2048, 50, 4, ok.ctypes.data, sums.ctypes.data) == 0
        assert sums.tolist() == [3.0] * 4
        # and ordinary work still runs on the context
        assert be.argmax(np.arange(100, dtype=np.float32)) == 99
    finally:
        be.close()


def test_few_rows_exchange_kernel_on_one_gpu():
    """The one-kernel all-reduce + residual add of decode batches, as rank 0 of 2 with the peer's chunks and arrival words
    written beforehand (delivered rounds) or missing (the bounded wait runs out and reports; nothing hangs).  Counts that end
    inside a chunk, several chunks, both parities."""
    import ctypes as C
    import time

    import numpy as np

    import orangu_b200
    from orangu_b200 import capi

    be = orangu_b200.CudaBackend.init(0)
    L = capi.load()
    try:
        for count in (2048, 4 * 4096, 64 * 4096, 3 * 4096 + 1028):
            delivers = np.array([1, 1, 0, 1, 1], np.uint8)
            out = np.zeros((len(delivers), count), np.float32)
            t0 = time.time()
            rc = L.ob_tp_bulk_selftest(be._h, count, 50, len(delivers), delivers.ctypes.data, out.ctypes.data)
            assert rc == 0, (count, L.ob_last_error(be._h))
            assert time.time() - t0 < 5.0
            i = (np.arange(count) % 1000).astype(np.float32)
            full, alone = np.float32(0.5) + (i + (2 * i + 1)), np.float32(0.5) + (i + np.float32(0.0))
            for k, d in enumerate(delivers):
                want = full if d else None
                if d:
                    assert (out[k] == want).all(), (count, k)
                else:  # the peer's landing area of this parity holds whatever an earlier round left: only this rank's part is certain
                    assert np.isfinite(out[k]).all() and (out[k] >= alone).all()
        assert be.argmax(np.arange(100, dtype=np.float32)) == 99
    finally:
        be.close()
