"""ob_attention_decode_static: the attention entry point that allocates nothing.

Some callers of this library cannot allocate device memory while they run: a slot's worker thread in the middle
of a request (cudaMalloc / cudaFree synchronise the whole device and would stall the other slots), or a server
whose KV pool has already taken the remaining memory.  For them the split flash-decode attention exists in a
form whose only scratch is a fixed array inside the library image.  This test calls it through the C ABI with
caller-owned device buffers and checks it, twice in a row (the array is shared between calls and keeps the previous
call's contents), against two things: the CPU oracle's attention over the same fp16-rounded K and V (the values), and
the allocating entry point, ob_attention_decode (the plumbing).

Collected last on purpose (file name), so a run that stops at the first failure has already run everything else.
It needs no state from the other tests and passes alone in a fresh process too.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 2e-5  # the tolerance test_gpu_glue.py holds the flash-decode kernel to


def pages_from_rows(x, n_head_kv, head_dim):
    """[n_pos, n_head_kv*head_dim] f32 -> fp16 pages [page][kv head][16][head_dim], identity page order."""
    n_pos = x.shape[0]
    n_pages = (n_pos + 15) // 16
    out = np.zeros((n_pages, n_head_kv, 16, head_dim), np.float16)
    x3 = x.reshape(n_pos, n_head_kv, head_dim).astype(np.float16)
    for p in range(n_pos):
        out[p // 16, :, p % 16, :] = x3[p]
    return out


@pytest.mark.parametrize("n_head,n_head_kv,head_dim,n_pos_pair", [(32, 8, 128, (700, 4133)), (8, 2, 64, (331, 40)), (8, 8, 128, (64, 65))])
def test_static_scratch_attention_matches_the_allocating_entry_point(n_head, n_head_kv, head_dim, n_pos_pair):
    import torch

    import oracle as O
    import orangu_b200
    from orangu_b200 import capi, synth

    be = orangu_b200.CudaBackend.init(0)
    L = capi.load()
    try:
        for call, n_pos in enumerate(n_pos_pair):  # two calls in a row on the same context: the scratch is reused
            kv_dim = n_head_kv * head_dim
            k = synth.normal(n_pos * kv_dim, 100 + call).reshape(n_pos, kv_dim)
            v = synth.normal(n_pos * kv_dim, 200 + call).reshape(n_pos, kv_dim)
            q = synth.normal(n_head * head_dim, 300 + call)
            scale = float(1.0 / np.sqrt(head_dim))
            want = be.attention_decode(q, k, v, n_head, n_head_kv, head_dim, scale, exact_order=False)
            f16 = lambda a: a.astype(np.float16).astype(np.float32)  # the cache holds f16 (engine/kv_cache.rs:26-32)
            cpu = O.attention(q, f16(k), f16(v), n_head, n_head_kv, head_dim, scale, 1, n_pos - 1)[0]

            q_d = torch.from_numpy(q).cuda()
            k_d = torch.from_numpy(pages_from_rows(k, n_head_kv, head_dim)).cuda()
            v_d = torch.from_numpy(pages_from_rows(v, n_head_kv, head_dim)).cuda()
            table_d = torch.arange(k_d.shape[0], dtype=torch.int32, device="cuda")
            out_d = torch.full((n_head * head_dim,), float("nan"), dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            rc = L.ob_attention_decode_static(be._h, q_d.data_ptr(), k_d.data_ptr(), v_d.data_ptr(), table_d.data_ptr(), n_pos, n_head,
                                              n_head_kv, head_dim, scale, out_d.data_ptr(), None)
            capi.check(be._h, rc)
            be.synchronize()
            got = out_d.cpu().numpy()
            assert np.isfinite(got).all()
            assert np.abs(got - cpu).max() < TOL, f"call {call}, {n_pos} positions: differs from the CPU oracle"
            assert np.abs(got - want).max() < TOL, f"call {call}, {n_pos} positions: differs from ob_attention_decode"
    finally:
        be.close()


def test_static_scratch_attention_refuses_what_does_not_fit():
    import torch

    import orangu_b200
    from orangu_b200 import capi

    be = orangu_b200.CudaBackend.init(0)
    L = capi.load()
    try:
        dummy = torch.zeros(16, device="cuda")
        args = (dummy.data_ptr(),) * 4
        # 256 heads x 16 splits x 130 floats x 4 B = 2.1 MB of partials: above the 1 MiB array
        assert L.ob_attention_decode_static(be._h, *args, 4096, 256, 32, 128, 0.1, dummy.data_ptr(), None) == -6
        assert b"1 MiB" in L.ob_last_error(be._h)
        assert L.ob_attention_decode_static(be._h, *args, 64, 8, 2, 96, 0.1, dummy.data_ptr(), None) == -2   # head_dim
        assert L.ob_attention_decode_static(be._h, *args, 64, 6, 2, 64, 0.1, dummy.data_ptr(), None) == -2   # group of 3
        assert L.ob_attention_decode_static(be._h, None, *args[1:], 64, 8, 2, 64, 0.1, dummy.data_ptr(), None) == -1
    finally:
        be.close()
