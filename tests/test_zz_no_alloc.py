"""ullm_decode_attention_static, the entry point for callers that cannot
allocate device memory (hosts with a fixed memory budget, allocator-free
sections of another framework, plug-in interfaces that forbid cudaMalloc).

The test calls it through its exported C symbol, straight from the shared
library, and checks its output against the regular entry point's (which gets
its scratch from the caller), on two calls in a row with different inputs: the
library-resident scratch keeps the first call's contents and the second call
must not be disturbed by them.  It also checks that a call whose partials
would not fit the fixed array is refused.  This file sorts last on purpose.
"""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.needs_cuda]


def _lib():
    from ullm_b200.csrc.build import build

    lib = ctypes.CDLL(build())
    P, I, F, LL = c_void_p, c_int, c_float, c_longlong
    lib.ullm_decode_attention.argtypes = [P, LL, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, I, LL, P, P]
    lib.ullm_decode_attention.restype = c_int
    lib.ullm_decode_attention_static.argtypes = [P, LL, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, LL, P, P]
    lib.ullm_decode_attention_static.restype = c_int
    lib.ullm_decode_attention_static_capacity.restype = c_longlong
    lib.ullm_decode_attention_scratch_floats.argtypes = [I, I, I, I]
    lib.ullm_decode_attention_scratch_floats.restype = c_longlong
    lib.ullm_decode_attention_cluster_merge.argtypes = [I]
    lib.ullm_decode_attention_cluster_merge.restype = None
    lib.ullm_decode_attention_last_used_cluster.restype = c_int
    return lib


def _case(seed, batch, Hq, Hkv, D, page, lens):
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // page) for n in lens]
    pages = sum(pages_per) + 2
    perm = torch.randperm(pages, generator=g)
    bt = torch.full((batch, max(pages_per) + 1), -1, dtype=torch.int32)
    used = 0
    for r, n in enumerate(pages_per):
        bt[r, :n] = perm[used:used + n].int()
        used += n
    mk = lambda *s: (torch.randn(*s, generator=g)).to(torch.bfloat16).cuda()
    return dict(qkv=mk(batch, (Hq + 2 * Hkv) * D), k=mk(pages, page, Hkv, D), v=mk(pages, page, Hkv, D), bt=bt.cuda(),
                slots=torch.arange(batch, dtype=torch.int32).cuda(), kv=torch.tensor(lens, dtype=torch.int32).cuda(),
                pages=pages)


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    """Three calls in a row on different inputs.  The kernel has two ways to merge a request's splits: inside a
    thread-block cluster (2 to 8 splits; no scratch at all) or through the scratch arrays and a merge kernel.
    Only the second reads the library's array, so it is forced: once by switching the cluster form off, once by
    more splits than a cluster takes; the third call takes the cluster form."""
    lib = _lib()
    Hq, Hkv, D, page = 16, 4, 128, 16
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    cases = ((1, 3, 7, [700, 33, 1500], 0), (2, 5, 12, [64, 1, 999, 130, 17], 1), (3, 2, 4, [300, 41], 1))
    try:
        for seed, batch, splits, lens, cluster in cases:
            lib.ullm_decode_attention_cluster_merge(cluster)
            c = _case(seed, batch, Hq, Hkv, D, page, lens)
            need = lib.ullm_decode_attention_scratch_floats(batch, Hq, D, splits)
            assert need <= lib.ullm_decode_attention_static_capacity()
            scratch = torch.empty(need, dtype=torch.float32, device="cuda")
            ref = torch.empty(batch, Hq * D, dtype=torch.bfloat16, device="cuda")
            got = torch.full_like(ref, 3.0)
            p = lambda t: c_void_p(t.data_ptr())
            common = (p(c["k"]), p(c["v"]), p(c["bt"]), c["bt"].shape[1], p(c["slots"]), p(c["kv"]))
            sizes = (batch, Hq, Hkv, D, page, 0, D ** -0.5, splits, c["pages"], p(status), stream)
            rc = lib.ullm_decode_attention(p(c["qkv"]), c["qkv"].stride(0), *common, p(ref), p(scratch), *sizes)
            assert rc == 0
            rc = lib.ullm_decode_attention_static(p(c["qkv"]), c["qkv"].stride(0), *common, p(got), *sizes)
            assert rc == 0
            through_scratch = cluster == 0 or splits > 8
            assert lib.ullm_decode_attention_last_used_cluster() == (0 if through_scratch else 1)
            torch.cuda.synchronize()
            assert status.tolist()[0] == 0
            assert torch.isfinite(got.float()).all()
            # same kernel, same split count: the two must agree to the tolerance of the kernel tests
            err = (got.float() - ref.float()).abs().max().item() / max(ref.float().abs().max().item(), 1e-6)
            assert err <= 2e-2, f"seed {seed}: max err {err:.3e} of scale"
    finally:
        lib.ullm_decode_attention_cluster_merge(1)  # the library's default


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    c = _case(3, 64, 32, 8, 128, 16, [100] * 64)
    out = torch.zeros(64, 32 * 128, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    p = lambda t: c_void_p(t.data_ptr())
    splits = 8  # 64 * 32 * 8 * 130 floats = 2.1 M > 1 M
    assert lib.ullm_decode_attention_scratch_floats(64, 32, 128, splits) > lib.ullm_decode_attention_static_capacity()
    rc = lib.ullm_decode_attention_static(p(c["qkv"]), c["qkv"].stride(0), p(c["k"]), p(c["v"]), p(c["bt"]),
                                          c["bt"].shape[1], p(c["slots"]), p(c["kv"]), p(out), 64, 32, 8, 128, 16, 0,
                                          128 ** -0.5, splits, c["pages"], p(status),
                                          c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 5, "ULLM_ERR_SCRATCH_TOO_LARGE"
    assert (out == 0).all(), "a refused call launches nothing"
    # one split has no partials and touches nothing of the array: a batch whose formula value is over the limit
    # is taken all the same
    big = 256
    c = _case(4, big, 32, 8, 128, 16, [20] * big)
    out = torch.zeros(big, 32 * 128, dtype=torch.bfloat16, device="cuda")
    assert lib.ullm_decode_attention_scratch_floats(big, 32, 128, 1) > lib.ullm_decode_attention_static_capacity()
    rc = lib.ullm_decode_attention_static(p(c["qkv"]), c["qkv"].stride(0), p(c["k"]), p(c["v"]), p(c["bt"]),
                                          c["bt"].shape[1], p(c["slots"]), p(c["kv"]), p(out), big, 32, 8, 128, 16, 0,
                                          128 ** -0.5, 1, c["pages"], p(status),
                                          c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 0 and status.tolist()[0] == 0 and torch.isfinite(out.float()).all() and (out != 0).any()
