"""Each CUDA kernel alone against a plain float32 torch reference of the same
operation, at sizes other than the engine's tiny models: row lengths and
vocabularies that are no power of two, head sizes in steps of 16, odd head
counts and groups, windows, ragged batches."""

import math

import pytest
import torch

import plain_model as pm

pytestmark = [pytest.mark.gpu, pytest.mark.needs_cuda]

DTYPES = [torch.float32, torch.bfloat16]
ATOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def K():
    from ullm_b200.csrc import kernels

    return kernels()


def close(got, ref, dtype, scale=None):
    got, ref = got.float().cpu(), ref.float().cpu()
    s = scale if scale is not None else max(ref.abs().max().item(), 1e-6)
    err = (got - ref).abs().max().item() / s
    assert err <= ATOL[dtype], f"max err {err:.3e} of scale (limit {ATOL[dtype]})"


def rnd(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [24, 100, 1000, 4096])
def test_embedding_and_gather(dtype, H):
    V, T = 777, 53
    table = rnd(V, H, seed=1, dtype=dtype)
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(2)).int().cuda()
    out = torch.empty(T, H, dtype=dtype, device="cuda")
    K().embedding(ids, table, out)
    assert torch.equal(out, table[ids.long()])
    rows = torch.tensor([5, 0, 52, 7], dtype=torch.int32, device="cuda")
    g = torch.empty(4, H, dtype=dtype, device="cuda")
    K().gather_rows(out, rows, g)
    assert torch.equal(g, out[rows.long()])


def test_embedding_refuses_bad_id():
    from ullm_b200.csrc.ops import KernelError

    table = rnd(10, 16)
    ids = torch.tensor([1, 10], dtype=torch.int32, device="cuda")
    out = torch.empty(2, 16, device="cuda")
    K().embedding(ids, table, out)
    with pytest.raises(KernelError, match="token id"):
        K().raise_on_status()
    K().raise_on_status()  # cleared


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [16, 100, 1000, 4096, 13000])
@pytest.mark.parametrize("with_res", [False, True])
def test_add_rmsnorm(dtype, H, with_res):
    T, eps = 37, 3e-6
    x = rnd(T, H, seed=3, dtype=dtype)
    res = rnd(T, H, seed=4, dtype=dtype) if with_res else None
    w = (1 + 0.3 * torch.randn(H, generator=torch.Generator().manual_seed(5))).cuda()
    s = x.float() + (res.float() if with_res else 0)
    ref = pm.rms_norm(s, w, eps)
    res_in = res.clone() if with_res else None
    out = torch.empty_like(x)
    K().add_rmsnorm(x, res_in, w, eps, out)
    close(out, ref, dtype)
    if with_res:
        assert torch.equal(res_in, s.to(dtype)), "the stored residual is the rounded 32-bit sum"
    # in place
    x2 = x.clone()
    K().add_rmsnorm(x2, res.clone() if with_res else None, w, eps, x2)
    assert torch.equal(x2, out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("I", [8, 100, 176, 3072])
def test_act_mul(dtype, I):
    T = 29
    gu = rnd(T, 2 * I, seed=6, dtype=dtype, scale=2.0)
    out = torch.empty(T, I, dtype=dtype, device="cuda")
    K().act_mul(gu, out, 0)
    close(out, pm.silu_mul(gu[:, :I].float(), gu[:, I:].float()), dtype)
    K().act_mul(gu, out, 1)
    g = gu[:, :I].float()
    close(out, torch.nn.functional.gelu(g, approximate="tanh") * gu[:, I:].float(), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,rot", [(4, 2, 16, 16), (6, 1, 48, 48), (5, 5, 80, 40), (8, 2, 128, 128), (3, 1, 256, 256), (2, 2, 96, 0)])
def test_qk_norm_rope_store(dtype, Hq, Hkv, D, rot):
    T, max_pos, page, pages, eps = 23, 300, 8, 7, 1e-5
    W = (Hq + 2 * Hkv) * D
    qkv = rnd(T, W, seed=7, dtype=dtype)
    qw = (1 + 0.2 * torch.randn(D, generator=torch.Generator().manual_seed(8))).cuda()
    kw = (1 + 0.2 * torch.randn(D, generator=torch.Generator().manual_seed(9))).cuda()
    pos = torch.randint(0, max_pos, (T,), generator=torch.Generator().manual_seed(10)).int().cuda()
    slots = torch.randperm(page * pages, generator=torch.Generator().manual_seed(11))[:T].int()
    slots[3] = -1
    slots = slots.cuda()
    cos = sin = None
    if rot:
        c, s = pm.rope_table(rot, 50000.0, max_pos)
        cos, sin = c.cuda(), s.cuda()
    kp = torch.full((pages, page, Hkv, D), 7.0, dtype=dtype, device="cuda")
    vp = torch.full((pages, page, Hkv, D), 7.0, dtype=dtype, device="cuda")
    x = qkv.float().view(T, Hq + 2 * Hkv, D)
    q = pm.rms_norm(x[:, :Hq], qw, eps)
    k = pm.rms_norm(x[:, Hq:Hq + Hkv], kw, eps)
    v = x[:, Hq + Hkv:]
    if rot:
        def rope(t):
            r = pm.apply_rope(t[..., :rot], cos[pos.long()], sin[pos.long()])
            return torch.cat((r, t[..., rot:]), -1)
        q, k = rope(q), rope(k)
    work = qkv.clone()
    K().qk_norm_rope_store(work, Hq, Hkv, D, qw, kw, eps, cos, sin, rot, pos, slots, kp, vp)
    close(work[:, : Hq * D].view(T, Hq, D), q, dtype)
    assert torch.equal(work[:, Hq * D:], qkv[:, Hq * D:]), "k and v columns of the projection stay as they were"
    kf, vf = kp.view(-1, Hkv, D), vp.view(-1, Hkv, D)
    keep = slots >= 0
    close(kf[slots[keep].long()], k[keep], dtype)
    assert torch.equal(vf[slots[keep].long()], v[keep].to(dtype))
    untouched = torch.ones(page * pages, dtype=torch.bool)
    untouched[slots[keep].long().cpu()] = False
    assert (kf[untouched.cuda()] == 7.0).all() and (vf[untouched.cuda()] == 7.0).all()


def attention_reference(q, kf, vf, block_table, req_slots, q_lens, kv_lens, Hq, Hkv, D, page, window, scale):
    T = q.shape[0]
    out = torch.zeros(T, Hq, D)
    t = 0
    for r, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        for j in range(ql):
            pos = kl - ql + j
            lo = max(0, pos - window + 1) if window else 0
            keys = torch.arange(lo, pos + 1)
            slots = block_table[req_slots[r]][keys // page] * page + keys % page
            for h in range(Hq):
                kh = h // (Hq // Hkv)
                s = (kf[slots, kh] @ q[t, h]) * scale
                out[t, h] = torch.softmax(s, 0) @ vf[slots, kh]
            t += 1
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,page,window", [
    (4, 2, 16, 4, 0), (9, 3, 32, 16, 0), (6, 1, 48, 16, 24), (5, 5, 80, 8, 0), (8, 2, 128, 16, 0),
    (8, 2, 128, 16, 33), (2, 1, 256, 32, 0), (3, 3, 64, 16, 7),
])
def test_paged_attention_ragged_batch(dtype, Hq, Hkv, D, page, window):
    q_lens = [1, 37, 1, 2, 64]
    kv_lens = [150, 37, 1, 100, 130]
    B, T = len(q_lens), sum(q_lens)
    max_pages = 16 if page >= 16 else 64
    pages = sum(-(-k // page) for k in kv_lens) + 3
    g = torch.Generator().manual_seed(12)
    perm = torch.randperm(pages, generator=g)
    slots_of_req = [4, 0, 6, 2, 1]
    bt = torch.full((8, max_pages), -1, dtype=torch.int32)
    used = 0
    for r, kl in enumerate(kv_lens):
        n = -(-kl // page)
        bt[slots_of_req[r], :n] = perm[used:used + n].int()
        used += n
    kp = rnd(pages, page, Hkv, D, seed=13, dtype=dtype)
    vp = rnd(pages, page, Hkv, D, seed=14, dtype=dtype)
    W = (Hq + 2 * Hkv) * D
    qkv = rnd(T, W, seed=15, dtype=dtype)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32).cuda()
    token_req = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(q_lens)]).cuda()
    out = torch.empty(T, Hq * D, dtype=dtype, device="cuda")
    scale = D ** -0.5
    K().paged_attention(qkv, out, kp, vp, bt.cuda(), torch.tensor(slots_of_req, dtype=torch.int32).cuda(), cu,
                        torch.tensor(kv_lens, dtype=torch.int32).cuda(), token_req, Hq, Hkv, D, page, window, scale)
    K().raise_on_status()
    ref = attention_reference(qkv[:, : Hq * D].float().cpu().view(T, Hq, D), kp.float().cpu().view(-1, Hkv, D),
                              vp.float().cpu().view(-1, Hkv, D), bt.long(), slots_of_req, q_lens, kv_lens, Hq, Hkv, D,
                              page, window, scale)
    close(out.view(T, Hq, D), ref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_finds_one_far_key(dtype):
    """One key among 700 matches the query (score far above the rest): the
    output must be that key's value, wherever it lies: first position, a
    page's last slot, a page's first slot, the newest position."""
    Hq, Hkv, D, page = 4, 2, 64, 16
    n = 700
    pages = -(-n // page)
    for hot in (0, 15, 16, 351, 687, 699):
        k = torch.randn(n, Hkv, D, generator=torch.Generator().manual_seed(16)) * 0.1
        v = torch.randn(n, Hkv, D, generator=torch.Generator().manual_seed(17))
        qv = torch.randn(Hq, D, generator=torch.Generator().manual_seed(18))
        qv = qv / qv.norm(dim=-1, keepdim=True) * 12.0
        for h in range(Hq):
            k[hot, h // 2] = 0
        k[hot, 0] = (qv[0] + qv[1]) / 2
        k[hot, 1] = (qv[2] + qv[3]) / 2
        perm = torch.randperm(pages, generator=torch.Generator().manual_seed(19))
        kp = torch.zeros(pages, page, Hkv, D)
        vp = torch.zeros(pages, page, Hkv, D)
        for p in range(n):
            kp[perm[p // page], p % page] = k[p]
            vp[perm[p // page], p % page] = v[p]
        qkv = torch.zeros(1, (Hq + 2 * Hkv) * D)
        qkv[0, : Hq * D] = qv.reshape(-1)
        out = torch.empty(1, Hq * D, dtype=dtype, device="cuda")
        bt = perm.int()[None].cuda()
        z = torch.zeros(1, dtype=torch.int32, device="cuda")
        K().paged_attention(qkv.to(dtype).cuda(), out, kp.to(dtype).cuda(), vp.to(dtype).cuda(), bt, z,
                            torch.tensor([0, 1], dtype=torch.int32).cuda(), torch.tensor([n], dtype=torch.int32).cuda(),
                            z, Hq, Hkv, D, page, 0, 1.0)
        ref = attention_reference(qkv[:, : Hq * D].to(dtype).float().view(1, Hq, D), kp.to(dtype).float().view(-1, Hkv, D),
                                  vp.to(dtype).float().view(-1, Hkv, D), perm[None], [0], [1], [n], Hq, Hkv, D, page, 0, 1.0)
        close(out.view(1, Hq, D), ref, dtype)
        got = out.float().cpu().view(Hq, D)
        for h in range(Hq):
            assert (got[h] - v[hot, h // 2]).abs().max() < 0.15, f"hot key at {hot} not found by head {h}"


@pytest.mark.parametrize("V", [17, 331, 1000, 151936])
def test_argmax_lowest_index_on_ties(V):
    R = 5
    lg = rnd(R, V, seed=20)
    lg[1, 3] = lg[1, V - 1] = 50.0
    lg[2, :] = 0.0
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    K().argmax(lg, out)
    ref = [int(torch.argmax(r)) for r in lg.cpu()]
    ref[1], ref[2] = 3, 0
    assert out.tolist() == ref


@pytest.mark.parametrize("V", [331, 5000, 151936])
def test_sampling_filters_and_draws(V):
    cases = [(0.7, 20, 0.95, 0.0), (1.0, -1, 0.5, 0.0), (1.3, 5, 1.0, 0.1), (0.5, -1, 1.0, 0.3), (1.0, -1, 1.0, 0.0),
             (0.0, -1, 1.0, 0.0), (2.0, 1, 1.0, 0.0), (0.9, 50, 0.3, 0.05)]
    R = len(cases)
    lg = rnd(R, V, seed=21, scale=2.5)
    us = [0.0, 0.13, 0.5, 0.77, 0.999999, 0.3, 0.6, 0.42]
    dev = lambda xs, dt: torch.tensor(xs, dtype=dt, device="cuda")
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    probs = torch.empty(R, V, device="cuda")
    K().sample(lg, dev([c[0] for c in cases], torch.float32), dev([c[1] for c in cases], torch.int32),
               dev([c[2] for c in cases], torch.float32), dev([c[3] for c in cases], torch.float32),
               dev(us, torch.float32), out, probs)
    for r, (t, k, p, mp) in enumerate(cases):
        row = lg[r].cpu()
        if t <= 0:
            assert int(out[r]) == pm.greedy(row)
            continue
        ref = pm.filtered_distribution(row, t, k, p, mp)
        got = probs[r].cpu()
        # the kept sets agree except for entries within rounding of a threshold
        differ = (got > 0) != (ref > 0)
        assert differ.sum().item() <= 2, f"case {r}: kept sets differ in {differ.sum().item()} entries"
        if differ.sum().item() == 0:
            assert (got - ref).abs().max().item() < 1e-5
        ref_draw = pm.inverse_cdf_draw(got, us[r])
        assert got[int(out[r])] > 0, "a filtered-out token was drawn"
        c = torch.cumsum(got.double(), 0)
        i = int(out[r])
        lo = float(c[i - 1]) if i > 0 else 0.0
        assert lo - 1e-5 <= us[r] * float(c[-1]) <= float(c[i]) + 1e-5, f"case {r}: drew {i}, inverse CDF gives {ref_draw}"


@pytest.mark.parametrize("V", [5, 331, 4099, 50257, 151936])
def test_sampling_over_a_cluster_gives_the_tokens_and_probabilities_of_the_one_block_kernel(V):
    """A row spread over a cluster of eight blocks (slices in shared memory, histograms and sums exchanged
    through distributed shared memory) against one block per row: all sums are integer sums, so tokens and
    probabilities agree bit for bit, for every filter combination, with rows that start on no 16-byte boundary."""
    cases = [(0.7, 20, 0.95, 0.0), (1.0, -1, 0.5, 0.0), (1.3, 5, 1.0, 0.1), (0.5, -1, 1.0, 0.3), (1.0, -1, 1.0, 0.0),
             (0.0, -1, 1.0, 0.0), (2.0, 1, 1.0, 0.0), (0.9, 50, 0.3, 0.05), (0.6, 20, 0.95, 0.0), (1.0, 3, 0.01, 0.0),
             (1.5, -1, 0.999, 0.0), (0.8, 100000, 0.9, 0.5)]
    R = len(cases)
    wide = rnd(R, V + 3, seed=23, scale=2.5)
    wide[2, 10 % V] = wide[2, 3 % V]  # equal values
    wide[4, :] = wide[4, 0]           # a flat row
    dev = lambda xs, dt: torch.tensor(xs, dtype=dt, device="cuda")
    args = (dev([c[0] for c in cases], torch.float32), dev([c[1] for c in cases], torch.int32),
            dev([c[2] for c in cases], torch.float32), dev([c[3] for c in cases], torch.float32))
    for shift in (0, 1):  # rows at 16-byte boundaries (if V allows) and off them
        lg = wide[:, shift:shift + V]
        for seed in range(3):
            us = dev([((r * 37 + seed * 101) % 1000) / 1000.0 for r in range(R)], torch.float32)
            got, ref = [], []
            for one_block, res in ((False, got), (True, ref)):
                out = torch.full((R,), -7, dtype=torch.int32, device="cuda")
                probs = torch.full((R, V), -1.0, device="cuda")
                slots = torch.arange(R, dtype=torch.int32, device="cuda")
                last = torch.full((R,), -9, dtype=torch.int32, device="cuda")
                K().sample_force_one_block(one_block)
                try:
                    K().sample(lg, *args, us, out, probs, row_slots=slots, last_tokens=last)
                    assert K().sample_used_cluster() == (not one_block)
                finally:
                    K().sample_force_one_block(False)
                res += [out.cpu(), probs.cpu(), last.cpu()]
            assert torch.equal(got[0], ref[0]), (got[0].tolist(), ref[0].tolist())
            assert torch.equal(got[1], ref[1])
            assert torch.equal(got[2], ref[2]) and torch.equal(got[2], got[0])


def test_sampling_is_independent_of_batch():
    V = 4099
    lg = rnd(6, V, seed=22, scale=2.0)
    f = lambda xs: torch.tensor(xs, dtype=torch.float32, device="cuda")
    t, p, mp, u = f([0.8] * 6), f([0.9] * 6), f([0.02] * 6), f([0.1, 0.3, 0.5, 0.7, 0.9, 0.2])
    k = torch.tensor([40] * 6, dtype=torch.int32, device="cuda")
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    K().sample(lg, t, k, p, mp, u, out)
    one = torch.empty(1, dtype=torch.int32, device="cuda")
    for r in range(6):
        K().sample(lg[r:r + 1], t[r:r + 1], k[r:r + 1], p[r:r + 1], mp[r:r + 1], u[r:r + 1], one)
        assert int(one) == int(out[r])


class _DecodeCtx:
    """What the attention dispatcher reads of a step's context."""

    def __init__(self, batch):
        from ullm_b200.engine.batch import Workspace

        self.decode_only = True
        self.num_requests = batch
        self.workspace = Workspace(torch.device("cuda"))
        self.max_q_len = 1


@pytest.mark.parametrize("Hq,Hkv,D,page,window", [
    (32, 8, 128, 16, 0), (8, 8, 128, 16, 0), (16, 1, 64, 16, 0), (12, 3, 64, 8, 0), (6, 2, 128, 32, 0),
    (32, 8, 128, 16, 100), (4, 2, 64, 4, 37), (9, 3, 128, 1, 0), (24, 2, 128, 8, 0), (16, 1, 128, 128, 300),
])
@pytest.mark.parametrize("batch", [1, 3, 24, 40])  # (24 requests x 8 kv heads: the pairs that run unsplit in one wave)
@pytest.mark.parametrize("mode", ["split", "split-merge-kernel", "balanced", "tcgen05"])
def test_decode_attention_bf16(Hq, Hkv, D, page, window, batch, mode):
    """The three tensor-core decode kernels (every request split alike; the whole batch's keys cut evenly over
    the warps; the same over the blocks with the products on tcgen05) against the plain reference: contexts of
    1 token, around page and tile edges, and long ones, ragged within a batch; padding rows (length 0) give
    zeros."""
    balanced = mode == "balanced"
    if mode == "tcgen05" and not K().lib.ullm_decode_attention_tcgen05_supported(D, Hq, Hkv, batch, page):
        pytest.skip("the tcgen05 decode kernel takes head size 128 and pages of 8 to 128 tokens")
    dtype = torch.bfloat16
    lens = [1, 15, 16, 17, 63, 64, 65, 300, 1000, 2049, 0, 33, 129, 511, 77, 5]
    kv_lens = [lens[(i * 7 + batch) % len(lens)] for i in range(batch)]
    if batch == 1:
        kv_lens = [2049]
    max_pages = -(-max(kv_lens + [1]) // page) + 1
    pages = sum(-(-k // page) for k in kv_lens) + 2
    g = torch.Generator().manual_seed(30 + batch)
    perm = torch.randperm(pages, generator=g)
    slots_of_req = torch.randperm(batch + 3, generator=g)[:batch].tolist()
    bt = torch.full((batch + 3, max_pages), -1, dtype=torch.int32)
    used = 0
    for r, kl in enumerate(kv_lens):
        n = -(-kl // page)
        bt[slots_of_req[r], :n] = perm[used:used + n].int()
        used += n
    kp = rnd(pages, page, Hkv, D, seed=31, dtype=dtype)
    vp = rnd(pages, page, Hkv, D, seed=32, dtype=dtype)
    # slots never written hold NaN: the kernel must not read them
    written = torch.zeros(pages * page, dtype=torch.bool)
    for r, kl in enumerate(kv_lens):
        for p in range(kl):
            written[int(bt[slots_of_req[r], p // page]) * page + p % page] = True
    kp.view(-1, Hkv, D)[~written.cuda()] = float("nan")
    vp.view(-1, Hkv, D)[~written.cuda()] = float("nan")
    W = (Hq + 2 * Hkv) * D
    qkv = rnd(batch, W, seed=33, dtype=dtype)
    cu = torch.arange(batch + 1, dtype=torch.int32).cuda()
    token_req = torch.arange(batch, dtype=torch.int32).cuda()
    out = torch.full((batch, Hq * D), 9.0, dtype=dtype, device="cuda")
    scale = D ** -0.5
    ctx = _DecodeCtx(batch)
    old = K().use_balanced_decode, K().use_tcgen05_decode
    old_cluster = K().decode_cluster_merge
    K().use_balanced_decode, K().use_tcgen05_decode = balanced, mode == "tcgen05"
    K().set_decode_cluster_merge(mode == "split")
    try:
        K().paged_attention(qkv, out, kp, vp, bt.cuda(), torch.tensor(slots_of_req, dtype=torch.int32).cuda(), cu,
                            torch.tensor(kv_lens, dtype=torch.int32).cuda(), token_req, Hq, Hkv, D, page, window,
                            scale, ctx)
    finally:
        K().use_balanced_decode, K().use_tcgen05_decode = old
        K().set_decode_cluster_merge(old_cluster)
    K().raise_on_status()
    assert K().attention_path == {"split": "decode", "split-merge-kernel": "decode", "balanced": "decode_balanced",
                                  "tcgen05": "decode_tcgen05"}[mode]
    if mode == "split" and batch * Hkv < 400:  # several splits: they met inside a cluster
        assert K().lib.ullm_decode_attention_last_used_cluster() == 1
    if mode == "split-merge-kernel":
        assert K().lib.ullm_decode_attention_last_used_cluster() == 0
    live = [r for r, kl in enumerate(kv_lens) if kl > 0]
    ref = attention_reference(qkv[:, : Hq * D].float().cpu().view(batch, Hq, D)[live],
                              torch.nan_to_num(kp.float().cpu()).view(-1, Hkv, D),
                              torch.nan_to_num(vp.float().cpu()).view(-1, Hkv, D), bt.long(),
                              [slots_of_req[r] for r in live], [1] * len(live), [kv_lens[r] for r in live], Hq, Hkv, D,
                              page, window, scale)
    got = out.view(batch, Hq, D).float().cpu()
    assert torch.isfinite(got).all()
    close(got[live], ref, dtype)
    for r, kl in enumerate(kv_lens):
        if kl == 0:
            assert (got[r] == 0).all()


class _MixedCtx(_DecodeCtx):
    def __init__(self, batch):
        super().__init__(batch)
        self.decode_only = False


@pytest.mark.parametrize("Hq,Hkv,D,page,window", [
    (32, 8, 128, 16, 0), (8, 8, 128, 16, 0), (16, 1, 64, 16, 0), (9, 3, 64, 8, 0), (6, 2, 128, 32, 0),
    (8, 2, 128, 16, 100), (4, 2, 64, 4, 37), (12, 4, 128, 1, 0), (5, 1, 64, 16, 0),
])
def test_prefill_attention_bf16_mixed_batch(Hq, Hkv, D, page, window):
    """The tensor-core kernel for batches with prompt portions: whole prompts,
    portions that continue a long context, two-token portions, single decoded
    tokens, lengths around tile edges (64 keys, 128 rows / group tokens)."""
    dtype = torch.bfloat16
    q_lens = [1, 37, 1, 2, 64, 129, 300, 31, 200]
    kv_lens = [150, 37, 1, 100, 130, 129, 700, 95, 200]
    B, T = len(q_lens), sum(q_lens)
    max_pages = -(-max(kv_lens) // page) + 1
    pages = sum(-(-k // page) for k in kv_lens) + 3
    g = torch.Generator().manual_seed(40)
    perm = torch.randperm(pages, generator=g)
    slots_of_req = torch.randperm(B + 2, generator=g)[:B].tolist()
    bt = torch.full((B + 2, max_pages), -1, dtype=torch.int32)
    used = 0
    written = torch.zeros(pages * page, dtype=torch.bool)
    for r, kl in enumerate(kv_lens):
        n = -(-kl // page)
        bt[slots_of_req[r], :n] = perm[used:used + n].int()
        for p in range(kl):
            written[int(perm[used + p // page]) * page + p % page] = True
        used += n
    kp = rnd(pages, page, Hkv, D, seed=41, dtype=dtype)
    vp = rnd(pages, page, Hkv, D, seed=42, dtype=dtype)
    kp.view(-1, Hkv, D)[~written.cuda()] = float("nan")
    vp.view(-1, Hkv, D)[~written.cuda()] = float("nan")
    qkv = rnd(T, (Hq + 2 * Hkv) * D, seed=43, dtype=dtype)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32).cuda()
    token_req = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(q_lens)]).cuda()
    out = torch.full((T, Hq * D), 9.0, dtype=dtype, device="cuda")
    scale = D ** -0.5
    old = K().use_tcgen05_attention
    K().use_tcgen05_attention = False  # this test is about the mma.sync kernel
    try:
        K().paged_attention(qkv, out, kp, vp, bt.cuda(), torch.tensor(slots_of_req, dtype=torch.int32).cuda(), cu,
                            torch.tensor(kv_lens, dtype=torch.int32).cuda(), token_req, Hq, Hkv, D, page, window, scale,
                            _MixedCtx(B))
    finally:
        K().use_tcgen05_attention = old
    K().raise_on_status()
    assert K().attention_path == "prefill"
    ref = attention_reference(qkv[:, : Hq * D].float().cpu().view(T, Hq, D),
                              torch.nan_to_num(kp.float().cpu()).view(-1, Hkv, D),
                              torch.nan_to_num(vp.float().cpu()).view(-1, Hkv, D), bt.long(), slots_of_req, q_lens,
                              kv_lens, Hq, Hkv, D, page, window, scale)
    got = out.view(T, Hq, D).float().cpu()
    assert torch.isfinite(got).all()
    close(got, ref, dtype)


@pytest.mark.parametrize("M,N,K", [
    (1, 128, 64), (8, 256, 128), (8, 4096, 4096), (8, 6144, 4096), (8, 4096, 12288), (3, 24576, 4096),
    (16, 1000, 520), (17, 331, 80), (64, 4096, 4096), (33, 777, 4104), (5, 151936, 1024), (48, 130, 72),
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_small_m_linear_tcgen05(M, N, K, out_dtype):
    """The tcgen05/TMA product for decode-sized batches against a float32 reference, with and without bias;
    sizes that are no multiple of the tile (128 rows, 64 columns); shapes whose tiles are shared by many blocks
    (few tiles, long K), by two, or owned whole; the second launch finds the tile counters reset."""
    x = rnd(M, K, seed=50, dtype=torch.bfloat16)
    w = rnd(N, K, seed=51, dtype=torch.bfloat16, scale=0.05)
    bias = rnd(N, seed=52, dtype=torch.bfloat16)
    ref = x.float() @ w.float().t()
    for b in (None, bias):
        out = torch.full((M, N), 7.0, dtype=out_dtype, device="cuda")
        took = K_().small_m_linear(x, w, out, b)
        K_().raise_on_status()
        assert took
        r = ref + (b.float() if b is not None else 0)
        err = (out.float() - r).abs().max().item() / max(r.abs().max().item(), 1e-6)
        assert err <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * K ** 0.5), f"max err {err:.3e} of scale"


def K_():
    return K()


@pytest.mark.parametrize("M,I,Kd,act", [
    (1, 64, 64, 0), (8, 12288, 4096, 0), (16, 200, 520, 1), (33, 331, 264, 0), (64, 1536, 2048, 0), (5, 96, 8192, 1),
])
def test_small_m_linear_with_fused_gate_activation(M, I, Kd, act):
    """act(x Wg^T) * (x Wu^T) in the product's epilogue, against float32; I no multiple of 64 (the last
    tile's gate box runs into the up rows and is masked), tiles split over many blocks (long K)."""
    x = rnd(M, Kd, seed=60, dtype=torch.bfloat16)
    w = rnd(2 * I, Kd, seed=61, dtype=torch.bfloat16, scale=0.05)
    bias = rnd(2 * I, seed=62, dtype=torch.bfloat16)
    for b in (None, bias):
        y = x.float() @ w.float().t() + (b.float() if b is not None else 0)
        g, u = y[:, :I], y[:, I:]
        ref = (g * torch.sigmoid(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")) * u
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((M, I), 7.0, dtype=out_dtype, device="cuda")
            assert K().small_m_linear(x, w, out, b, act)
            K().raise_on_status()
            err = (out.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
            assert err <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * Kd ** 0.5), f"max err {err:.3e} of scale"


@pytest.mark.parametrize("M,N,Kd", [
    (1, 16, 8), (1, 128, 64), (8, 4096, 4096), (8, 6144, 4096), (3, 4096, 12288), (16, 1000, 520), (17, 331, 80),
    (32, 777, 4104), (5, 151936, 1024), (24, 130, 72), (9, 24576, 4096),
])
def test_skinny_linear(M, N, Kd):
    """The streaming mma.sync product for decode-sized batches against a float32 reference, with and without
    bias, both output types; sizes that are no multiple of the 16-row tile or of the 32-wide k chunk, k ranges
    that divide unevenly over the warps."""
    x = rnd(M, Kd, seed=80, dtype=torch.bfloat16)
    w = rnd(N, Kd, seed=81, dtype=torch.bfloat16, scale=0.05)
    bias = rnd(N, seed=82, dtype=torch.bfloat16)
    ref = x.float() @ w.float().t()
    for b in (None, bias):
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((M, N), 7.0, dtype=out_dtype, device="cuda")
            assert K().skinny_linear(x, w, out, b)
            r = ref + (b.float() if b is not None else 0)
            err = (out.float() - r).abs().max().item() / max(r.abs().max().item(), 1e-6)
            assert err <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * Kd ** 0.5), f"max err {err:.3e} of scale"


@pytest.mark.parametrize("M,I,Kd,act", [
    (1, 16, 32, 0), (8, 12288, 4096, 0), (16, 200, 520, 1), (31, 331, 264, 0), (5, 96, 8192, 1),
])
def test_skinny_linear_with_fused_gate_activation(M, I, Kd, act):
    x = rnd(M, Kd, seed=90, dtype=torch.bfloat16)
    w = rnd(2 * I, Kd, seed=91, dtype=torch.bfloat16, scale=0.05)
    bias = rnd(2 * I, seed=92, dtype=torch.bfloat16)
    for b in (None, bias):
        y = x.float() @ w.float().t() + (b.float() if b is not None else 0)
        g, u = y[:, :I], y[:, I:]
        ref = (g * torch.sigmoid(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")) * u
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((M, I), 7.0, dtype=out_dtype, device="cuda")
            assert K().skinny_linear(x, w, out, b, act)
            err = (out.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
            assert err <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * Kd ** 0.5), f"max err {err:.3e} of scale"


@pytest.mark.parametrize("M,N,Kd", [
    (1, 16, 8), (1, 128, 64), (8, 4096, 4096), (8, 6144, 4096), (3, 4096, 12288), (16, 1000, 520), (17, 331, 80),
    (32, 777, 4104), (5, 151936, 1024), (24, 130, 72), (9, 24576, 4096), (16, 33, 256), (2, 4097, 776),
])
def test_stream_linear(M, N, Kd):
    """The weight-streaming TMA product for decode-sized batches against a float32 reference, with and without
    bias and residual, both output types; row counts that fill 1, 2 and 4 batch tiles, N that is no multiple of
    the 32-row unit (also fewer units than blocks and several units per block), K that is no multiple of the
    256-wide stage or of the 64-wide box."""
    x = rnd(M, Kd, seed=80, dtype=torch.bfloat16)
    w = rnd(N, Kd, seed=81, dtype=torch.bfloat16, scale=0.05)
    bias = rnd(N, seed=82, dtype=torch.bfloat16)
    res = rnd(M, N, seed=83, dtype=torch.bfloat16)
    ref = x.float() @ w.float().t()
    for b, rs in ((None, None), (bias, None), (None, res), (bias, res)):
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((M, N), 7.0, dtype=out_dtype, device="cuda")
            assert K().stream_linear(x, w, out, b, None, rs)
            K().raise_on_status()
            r = ref + (b.float() if b is not None else 0) + (rs.float() if rs is not None else 0)
            err = (out.float() - r).abs().max().item() / max(r.abs().max().item(), 1e-6)
            assert err <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * Kd ** 0.5), f"max err {err:.3e} of scale"
    # the residual may be the output itself (the residual stream updated in place)
    acc = res.clone()
    assert K().stream_linear(x, w, acc, None, None, acc)
    r = ref + res.float()
    assert (acc.float() - r).abs().max().item() / r.abs().max().item() <= 1e-2


@pytest.mark.parametrize("M,I,Kd,act", [
    (1, 16, 32, 0), (8, 12288, 4096, 0), (16, 200, 520, 1), (31, 331, 264, 0), (5, 96, 8192, 1), (12, 3072, 1024, 0),
])
def test_stream_linear_with_fused_gate_activation(M, I, Kd, act):
    x = rnd(M, Kd, seed=90, dtype=torch.bfloat16)
    w = rnd(2 * I, Kd, seed=91, dtype=torch.bfloat16, scale=0.05)
    bias = rnd(2 * I, seed=92, dtype=torch.bfloat16)
    for b in (None, bias):
        y = x.float() @ w.float().t() + (b.float() if b is not None else 0)
        g, u = y[:, :I], y[:, I:]
        ref = (g * torch.sigmoid(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")) * u
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((M, I), 7.0, dtype=out_dtype, device="cuda")
            assert K().stream_linear(x, w, out, b, act)
            K().raise_on_status()
            err = (out.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
            assert err <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * Kd ** 0.5), f"max err {err:.3e} of scale"


def test_stream_linear_is_deterministic_and_refuses_what_it_does_not_take():
    x = rnd(16, 4096, seed=70, dtype=torch.bfloat16)
    w = rnd(6144, 4096, seed=71, dtype=torch.bfloat16, scale=0.05)
    outs = []
    for bps in (1, 2, 1):  # one or two blocks per SM deal the units differently; the sums do not change
        K().lib.ullm_linear_stream_blocks_per_sm(bps)
        out = torch.empty(16, 6144, dtype=torch.float32, device="cuda")
        assert K().stream_linear(x, w, out)
        outs.append(out)
    one = torch.empty(1, 6144, dtype=torch.float32, device="cuda")
    assert K().stream_linear(x[:1].contiguous(), w, one)
    K().raise_on_status()
    assert torch.equal(outs[1], outs[0]) and torch.equal(outs[2], outs[0])
    assert torch.equal(one[0], outs[0][0]), "a row's result does not depend on the other rows of the batch"
    assert not K().stream_linear(rnd(40, 64, seed=1, dtype=torch.bfloat16), rnd(128, 64, seed=2, dtype=torch.bfloat16),
                                 torch.empty(40, 128, dtype=torch.bfloat16, device="cuda"))
    assert not K().stream_linear(rnd(4, 60, seed=1, dtype=torch.bfloat16), rnd(128, 60, seed=2, dtype=torch.bfloat16),
                                 torch.empty(4, 128, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("M,H,QD,I,act", [
    (8, 256, 256, 256, 0), (16, 512, 768, 1024, 0), (3, 4096, 4096, 12288, 0), (16, 1024, 2048, 3072, 1),
    (1, 256, 512, 256, 0), (11, 768, 256, 512, 1), (16, 5120, 8192, 25600, 0),
])
def test_fused_layer_tail(M, H, QD, I, act):
    """The second half of a decoder layer in one cooperative kernel (output projection + residual, RMSNorm, gated
    feed-forward, down projection + residual) against the same chain in float32 with the roundings of the separate
    kernels: row counts that fill one and two batch tiles, phases with and without split units, several items
    per block, three launches in a row on the same counters (tickets and grid barriers must come back), and the
    same bits every time."""
    assert K().lib.ullm_layer_tail_fused_supported(M, H, QD, I)
    bf = torch.bfloat16
    attn = rnd(M, QD, seed=200, dtype=bf)
    res0 = rnd(M, H, seed=201, dtype=bf)
    w_o = rnd(H, QD, seed=202, dtype=bf, scale=QD ** -0.5)
    w_gu = rnd(2 * I, H, seed=203, dtype=bf, scale=H ** -0.5)
    w_d = rnd(H, I, seed=204, dtype=bf, scale=I ** -0.5)
    norm_w = (1.0 + 0.1 * rnd(H, seed=205, dtype=torch.float32)).contiguous()
    eps = 1e-6
    s1 = res0.float() + attn.float() @ w_o.float().t()
    r1 = s1.to(bf)
    h = (s1 * torch.rsqrt(s1.pow(2).mean(-1, keepdim=True) + eps) * norm_w).to(bf)
    y = h.float() @ w_gu.float().t()
    g, u = y[:, :I], y[:, I:]
    a = ((g * torch.sigmoid(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")) * u).to(bf)
    ref = (r1.float() + a.float() @ w_d.float().t()).to(bf).float()
    outs = []
    for _ in range(3):
        res = res0.clone()
        work = torch.full((M, I), 7.0, dtype=bf, device="cuda")
        K().fused_layer_tail(attn, res, work, w_o, w_gu, w_d, norm_w, eps, act)
        K().raise_on_status()
        err = (res.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
        assert err <= 2e-2, f"residual after the layer: max err {err:.3e} of scale"
        aerr = (work.float() - a.float()).abs().max().item() / max(a.float().abs().max().item(), 1e-6)
        assert aerr <= 2e-2, f"activation: max err {aerr:.3e} of scale"
        outs.append(res)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("M,H,QD,I,act", [
    (8, 256, 256, 256, 0), (16, 520, 776, 1000, 0), (3, 4096, 4096, 12288, 0), (1, 1024, 2048, 3072, 1), (11, 80, 72, 176, 1),
])
def test_stream_products_with_the_norm_folded_between_them(M, H, QD, I, act):
    """Three stream products as a block chains them in small steps: the output projection adds the residual and
    leaves r * w and the units' sums of squares, the gate / up product multiplies its sums by the rows' 1 / rms
    before the activation, the down projection adds the residual; against the same chain in float32 with the
    roundings of the separate kernels.  Sizes with clusters (narrow outputs) and without, K and N that are no
    multiples of the tiles."""
    bf = torch.bfloat16
    attn = rnd(M, QD, seed=210, dtype=bf)
    res0 = rnd(M, H, seed=211, dtype=bf)
    w_o = rnd(H, QD, seed=212, dtype=bf, scale=QD ** -0.5)
    w_gu = rnd(2 * I, H, seed=213, dtype=bf, scale=H ** -0.5)
    w_d = rnd(H, I, seed=214, dtype=bf, scale=I ** -0.5)
    norm_w = (1.0 + 0.1 * rnd(H, seed=215, dtype=torch.float32)).contiguous()
    eps = 1e-6
    s1 = res0.float() + attn.float() @ w_o.float().t()
    r1 = s1.to(bf)
    h = (s1 * torch.rsqrt(s1.pow(2).mean(-1, keepdim=True) + eps) * norm_w).to(bf)
    y = h.float() @ w_gu.float().t()
    g, u = y[:, :I], y[:, I:]
    a = ((g * torch.sigmoid(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")) * u).to(bf)
    ref = (r1.float() + a.float() @ w_d.float().t()).to(bf).float()
    res = res0.clone()
    operand = torch.empty(M, H, dtype=bf, device="cuda")
    sq = torch.full((K().stream_sq_floats(H),), float("nan"), device="cuda")
    work = torch.empty(M, I, dtype=bf, device="cuda")
    assert K().stream_linear(attn, w_o, res, None, None, res, norm_behind=(norm_w, operand, sq))
    assert K().stream_linear(operand, w_gu, work, None, act, norm_in_front=(sq, H, eps))
    # the down projection prepares the NEXT norm the same way (a product that splits K over a cluster when its
    # output is narrow), and a product with a bias behind that norm applies 1 / rms before the bias
    norm_w2 = (1.0 + 0.1 * rnd(H, seed=216, dtype=torch.float32)).contiguous()
    operand2 = torch.empty(M, H, dtype=bf, device="cuda")
    sq2 = torch.full((K().stream_sq_floats(H),), float("nan"), device="cuda")
    assert K().stream_linear(work, w_d, res, None, None, res, norm_behind=(norm_w2, operand2, sq2))
    w_n = rnd(96, H, seed=217, dtype=bf, scale=H ** -0.5)
    b_n = rnd(96, seed=218, dtype=bf)
    nxt = torch.empty(M, 96, dtype=bf, device="cuda")
    assert K().stream_linear(operand2, w_n, nxt, b_n, None, None, norm_in_front=(sq2, H, eps))
    K().raise_on_status()
    s2 = r1.float() + a.float() @ w_d.float().t()
    h2 = (s2 * torch.rsqrt(s2.pow(2).mean(-1, keepdim=True) + eps) * norm_w2).to(bf)
    want_n = h2.float() @ w_n.float().t() + b_n.float()
    nerr = (nxt.float() - want_n).abs().max().item() / max(want_n.abs().max().item(), 1e-6)
    assert nerr <= 2e-2, f"product behind the next norm: max err {nerr:.3e} of scale"
    assert torch.allclose(sq2.view(-1, 16).sum(0)[:M].cpu(), s2.pow(2).sum(-1).cpu(), rtol=2e-2)
    assert torch.equal(res0.float() + 0, res0.float())  # (inputs untouched)
    aerr = (work.float() - a.float()).abs().max().item() / max(a.float().abs().max().item(), 1e-6)
    assert aerr <= 2e-2, f"activation: max err {aerr:.3e} of scale"
    err = (res.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
    assert err <= 2e-2, f"residual after the layer: max err {err:.3e} of scale"
    # the sums of squares add up to the rows' sums
    got = sq.view(-1, 16).sum(0)[:M].cpu()
    want = s1.pow(2).sum(-1).cpu()
    assert torch.allclose(got, want, rtol=2e-2), (got, want)


def test_skinny_linear_is_deterministic_and_refuses_what_it_does_not_take():
    x = rnd(16, 4096, seed=70, dtype=torch.bfloat16)
    w = rnd(512, 4096, seed=71, dtype=torch.bfloat16, scale=0.05)
    outs = []
    for _ in range(3):
        out = torch.empty(16, 512, dtype=torch.float32, device="cuda")
        assert K().skinny_linear(x, w, out)
        outs.append(out)
    one = torch.empty(1, 512, dtype=torch.float32, device="cuda")
    assert K().skinny_linear(x[:1].contiguous(), w, one)
    assert torch.equal(outs[1], outs[0]) and torch.equal(outs[2], outs[0])
    assert torch.equal(one[0], outs[0][0]), "a row's result does not depend on the other rows of the batch"
    assert not K().skinny_linear(rnd(40, 64, seed=1, dtype=torch.bfloat16), rnd(128, 64, seed=2, dtype=torch.bfloat16),
                                 torch.empty(40, 128, dtype=torch.bfloat16, device="cuda"))
    assert not K().skinny_linear(rnd(4, 60, seed=1, dtype=torch.bfloat16), rnd(128, 60, seed=2, dtype=torch.bfloat16),
                                 torch.empty(4, 128, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("M,N,Kd", [
    (128, 256, 64), (2048, 4096, 4096), (300, 1000, 520), (65, 331, 80), (1, 128, 64), (513, 777, 4104),
    (2048, 6144, 1024), (129, 130, 72),
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("variant", [1, 2])
def test_large_linear_tcgen05(M, N, Kd, out_dtype, variant):
    """The persistent tcgen05 product for many rows against a float32 reference, with and without bias, with
    tiles of 128 rows (variant 1) and of 256 rows (variant 2): sizes that are no multiple of the tile or of the
    64-wide k block, more tiles than blocks (several tiles per block through both accumulators), fewer tiles
    than blocks."""
    x = rnd(M, Kd, seed=150, dtype=torch.bfloat16)
    w = rnd(N, Kd, seed=151, dtype=torch.bfloat16, scale=0.05)
    bias = rnd(N, seed=152, dtype=torch.bfloat16)
    ref = x.float() @ w.float().t()
    for b in (None, bias):
        out = torch.full((M, N), 7.0, dtype=out_dtype, device="cuda")
        assert K().large_linear(x, w, out, b, None, variant)
        K().raise_on_status()
        r = ref + (b.float() if b is not None else 0)
        err = (out.float() - r).abs().max().item() / max(r.abs().max().item(), 1e-6)
        assert err <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * Kd ** 0.5), f"max err {err:.3e} of scale"


@pytest.mark.parametrize("M,I,Kd,act", [(128, 128, 64, 0), (2048, 3072, 1024, 0), (300, 200, 520, 1), (77, 331, 264, 0),
                                          (1100, 20000, 136, 0)])
@pytest.mark.parametrize("variant", [1, 2])
def test_large_linear_tcgen05_with_fused_gate_activation(M, I, Kd, act, variant):
    x = rnd(M, Kd, seed=160, dtype=torch.bfloat16)
    w = rnd(2 * I, Kd, seed=161, dtype=torch.bfloat16, scale=0.05)
    bias = rnd(2 * I, seed=162, dtype=torch.bfloat16)
    for b in (None, bias):
        y = x.float() @ w.float().t() + (b.float() if b is not None else 0)
        g, u = y[:, :I], y[:, I:]
        ref = (g * torch.sigmoid(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")) * u
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((M, I), 7.0, dtype=out_dtype, device="cuda")
            assert K().large_linear(x, w, out, b, act, variant)
            K().raise_on_status()
            err = (out.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
            assert err <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * Kd ** 0.5), f"max err {err:.3e} of scale"


def test_small_m_linear_is_deterministic_and_independent_of_other_rows():
    """Partial sums of a tile are added in block order whoever arrives last: repeated launches give the same
    bits; a row's result does not depend on how many other rows the batch has."""
    x = rnd(16, 4096, seed=70, dtype=torch.bfloat16)
    w = rnd(512, 4096, seed=71, dtype=torch.bfloat16, scale=0.05)
    outs = []
    for _ in range(5):
        out = torch.empty(16, 512, dtype=torch.float32, device="cuda")
        assert K().small_m_linear(x, w, out)
        outs.append(out)
    one = torch.empty(1, 512, dtype=torch.float32, device="cuda")
    assert K().small_m_linear(x[:1].contiguous(), w, one)
    K().raise_on_status()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    assert torch.equal(one[0], outs[0][0])


def test_small_m_linear_refuses_what_it_does_not_take():
    x = rnd(70, 64, seed=1, dtype=torch.bfloat16)
    w = rnd(128, 64, seed=2, dtype=torch.bfloat16)
    assert not K().small_m_linear(x, w, torch.empty(70, 128, dtype=torch.bfloat16, device="cuda"))
    x = rnd(4, 60, seed=1, dtype=torch.bfloat16)  # rows of 120 bytes: no 16-byte stride for TMA
    w = rnd(128, 60, seed=2, dtype=torch.bfloat16)
    assert not K().small_m_linear(x, w, torch.empty(4, 128, dtype=torch.bfloat16, device="cuda"))
    xf = rnd(4, 64, seed=1)
    assert not K().small_m_linear(xf, rnd(128, 64, seed=2), torch.empty(4, 128, device="cuda"))


@pytest.mark.parametrize("mode", ["pair", "single"])
@pytest.mark.parametrize("Hq,Hkv,page,window", [(32, 8, 16, 0), (8, 8, 16, 0), (16, 1, 16, 0), (8, 2, 32, 0),
                                                 (4, 2, 8, 0), (8, 2, 16, 100), (4, 1, 64, 37), (8, 4, 128, 0),
                                                 (4, 4, 16, 300)])
def test_prefill_attention_tcgen05_mixed_batch(Hq, Hkv, page, window, mode):
    """The two tcgen05/TMA attention kernels (head size 128; two query tiles per block, and one) on the same ragged
    batch as the mma.sync kernel: whole prompts, portions that continue a context, two-token portions, single
    tokens, requests of one to six key tiles; unwritten slots of the pool hold NaN."""
    if mode == "single" and page == 128:
        pytest.skip("the one-tile kernel takes pages of at most 64 tokens")
    dtype, D = torch.bfloat16, 128
    q_lens = [1, 37, 1, 2, 64, 129, 300, 31, 200]
    kv_lens = [150, 37, 1, 100, 130, 129, 700, 95, 200]
    B, T = len(q_lens), sum(q_lens)
    max_pages = -(-max(kv_lens) // page) + 1
    pages = sum(-(-k // page) for k in kv_lens) + 3
    g = torch.Generator().manual_seed(60)
    perm = torch.randperm(pages, generator=g)
    slots_of_req = torch.randperm(B + 2, generator=g)[:B].tolist()
    bt = torch.full((B + 2, max_pages), -1, dtype=torch.int32)
    used = 0
    written = torch.zeros(pages * page, dtype=torch.bool)
    for r, kl in enumerate(kv_lens):
        n = -(-kl // page)
        bt[slots_of_req[r], :n] = perm[used:used + n].int()
        for p in range(kl):
            written[int(perm[used + p // page]) * page + p % page] = True
        used += n
    kp = rnd(pages, page, Hkv, D, seed=61, dtype=dtype)
    vp = rnd(pages, page, Hkv, D, seed=62, dtype=dtype)
    kp.view(-1, Hkv, D)[~written.cuda()] = float("nan")
    vp.view(-1, Hkv, D)[~written.cuda()] = float("nan")
    qkv = rnd(T, (Hq + 2 * Hkv) * D, seed=63, dtype=dtype)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32).cuda()
    token_req = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(q_lens)]).cuda()
    out = torch.full((T, Hq * D), 9.0, dtype=dtype, device="cuda")
    scale = D ** -0.5
    k = K()
    old = k.use_tcgen05_attention, k.tc_attention_mode
    k.use_tcgen05_attention, k.tc_attention_mode = True, mode
    try:
        k.paged_attention(qkv, out, kp, vp, bt.cuda(), torch.tensor(slots_of_req, dtype=torch.int32).cuda(), cu,
                          torch.tensor(kv_lens, dtype=torch.int32).cuda(), token_req, Hq, Hkv, D, page, window, scale,
                          _MixedCtx(B))
        torch.cuda.synchronize()
        k.raise_on_status()
    finally:
        k.use_tcgen05_attention, k.tc_attention_mode = old
    assert k.attention_path == "prefill_tcgen05" and k.prefill_attention_kernel == mode
    ref = attention_reference(qkv[:, : Hq * D].float().cpu().view(T, Hq, D),
                              torch.nan_to_num(kp.float().cpu()).view(-1, Hkv, D),
                              torch.nan_to_num(vp.float().cpu()).view(-1, Hkv, D), bt.long(), slots_of_req, q_lens,
                              kv_lens, Hq, Hkv, D, page, window, scale)
    got = out.view(T, Hq, D).float().cpu()
    assert torch.isfinite(got).all()
    close(got, ref, dtype)


@pytest.mark.parametrize("M,N,Kd", [(1, 64, 64), (16, 6144, 4096), (16, 200, 520), (64, 1000, 136), (256, 777 * 8, 264),
                                     (5, 96, 8192)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_library_product_with_timed_choice(M, N, Kd, out_dtype):
    """`lt_linear`: the vendor library's product through cuBLASLt, the algorithm chosen by timing the library's
    candidates once per shape.  Whatever it chooses computes x W^T; the second call (no timing) gives the same
    bits as the first (the choice is kept)."""
    x = rnd(M, Kd, seed=170, dtype=torch.bfloat16)
    w = rnd(N, Kd, seed=171, dtype=torch.bfloat16, scale=0.05)
    ref = x.float() @ w.float().t()
    out = torch.full((M, N), 7.0, dtype=out_dtype, device="cuda")
    assert K().lt_linear(x, w, out)
    err = (out.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
    assert err <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * Kd ** 0.5), f"max err {err:.3e} of scale"
    again = torch.full((M, N), 3.0, dtype=out_dtype, device="cuda")
    assert K().lt_linear(x, w, again)
    assert torch.equal(out, again)
    ch = K().lt_last_choice()
    assert 0 <= ch["chosen"] < max(ch["candidates"], 1)


def test_library_product_with_timed_choice_refuses_what_it_cannot_take():
    x = rnd(4, 60, seed=1, dtype=torch.bfloat16)  # rows of 120 bytes: no 16-byte pieces
    assert not K().lt_linear(x, rnd(16, 60, seed=2, dtype=torch.bfloat16), torch.empty(4, 16, dtype=torch.bfloat16, device="cuda"))
    xf = rnd(4, 64, seed=1)  # float32 operands stay with the 32-bit path
    assert not K().lt_linear(xf, rnd(16, 64, seed=2), torch.empty(4, 16, device="cuda"))


def test_library_product_inside_a_stream_capture_takes_an_untimed_shape_without_timing():
    """A shape first seen while a CUDA graph is being recorded cannot be timed (timing synchronises): it takes the
    library's first candidate, the recording holds that launch, and the shape is timed at its next eager call."""
    x = rnd(24, 320, seed=180, dtype=torch.bfloat16)
    w = rnd(264, 320, seed=181, dtype=torch.bfloat16, scale=0.05)
    out = torch.zeros(24, 264, dtype=torch.bfloat16, device="cuda")
    ref = x.float() @ w.float().t()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g):
            assert K().lt_linear(x, w, out)
    assert (24, 264, 320, 0) not in K()._lt_tuned
    g.replay()
    torch.cuda.synchronize()
    assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()
    out.zero_()
    assert K().lt_linear(x, w, out)
    assert (24, 264, 320, 0) in K()._lt_tuned
    assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()


@pytest.mark.parametrize("Hq,Hkv,D,page,window,with_norm", [
    (32, 8, 128, 16, 0, True), (8, 8, 128, 16, 0, True), (12, 3, 64, 8, 0, True), (6, 2, 128, 32, 40, False),
    (16, 1, 64, 16, 0, True),
])
@pytest.mark.parametrize("batch", [1, 3, 40])
def test_decode_attention_that_prepares_q_k_and_v_itself(Hq, Hkv, D, page, window, with_norm, batch):
    """The per-request decode kernel with the q/k norm, the rotation and the cache write inside it, against the
    two-kernel way (`qk_norm_rope_store`, then the attention): the same attention output, the same new key and
    value in the cache (to a rounding of bfloat16: the sums of squares are added in another order); rows of
    length 0 write nothing; every split count, with the cluster merge and with the merge kernel."""
    dtype = torch.bfloat16
    lens = [1, 15, 16, 17, 63, 64, 65, 300, 1000, 2049, 0, 33, 129, 511, 77, 5]
    kv_lens = [lens[(i * 5 + batch) % len(lens)] for i in range(batch)]
    max_pages = -(-max(kv_lens + [1]) // page) + 1
    pages = sum(-(-k // page) for k in kv_lens) + 2
    g = torch.Generator().manual_seed(90 + batch)
    perm = torch.randperm(pages, generator=g)
    bt = torch.full((batch, max_pages), -1, dtype=torch.int32)
    used = 0
    for r, kl in enumerate(kv_lens):
        n = -(-kl // page)
        bt[r, :n] = perm[used:used + n].int()
        used += n
    slot_mapping = torch.tensor([int(bt[r, (kl - 1) // page]) * page + (kl - 1) % page if kl > 0 else -1
                                 for r, kl in enumerate(kv_lens)], dtype=torch.int32, device="cuda")
    positions = torch.tensor([max(kl - 1, 0) for kl in kv_lens], dtype=torch.int32, device="cuda")
    kp0 = rnd(pages, page, Hkv, D, seed=91, dtype=dtype)
    vp0 = rnd(pages, page, Hkv, D, seed=92, dtype=dtype)
    qkv0 = rnd(batch, (Hq + 2 * Hkv) * D, seed=93, dtype=dtype)
    q_w = (1 + 0.1 * rnd(D, seed=94)) if with_norm else None
    k_w = (1 + 0.1 * rnd(D, seed=95)) if with_norm else None
    pos = torch.arange(2100, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    cos, sin = torch.cos(pos[:, None] * inv).cuda().contiguous(), torch.sin(pos[:, None] * inv).cuda().contiguous()
    slots = torch.arange(batch, dtype=torch.int32, device="cuda")
    cu = torch.arange(batch + 1, dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    scale = D ** -0.5
    old = K().use_balanced_decode, K().use_tcgen05_decode, K().decode_cluster_merge, K().decode_split_target
    K().use_balanced_decode, K().use_tcgen05_decode = False, False
    try:
        for cluster, target in ((True, 400), (False, 400), (False, 4000), (True, 1)):
            K().set_decode_cluster_merge(cluster)
            K().decode_split_target = target
            res = []
            for fused in (False, True):
                qkv, kp, vp = qkv0.clone(), kp0.clone(), vp0.clone()
                out = torch.full((batch, Hq * D), 9.0, dtype=dtype, device="cuda")
                ctx = _DecodeCtx(batch)
                fuse = None
                if fused:
                    assert K().decode_fusion_applies(ctx, qkv, Hq, Hkv, D, page, D, cos)
                    fuse = dict(q_w=q_w, k_w=k_w, eps=1e-6, cos=cos, sin=sin, positions=positions, slot_mapping=slot_mapping)
                else:
                    K().qk_norm_rope_store(qkv, Hq, Hkv, D, q_w, k_w, 1e-6, cos, sin, D, positions, slot_mapping, kp, vp)
                K().paged_attention(qkv, out, kp, vp, bt.cuda(), slots, cu, kvl, slots, Hq, Hkv, D, page, window, scale,
                                    ctx, **({"fuse": fuse} if fused else {}))
                K().raise_on_status()
                res.append((out.float(), kp.float(), vp.float()))
            (o0, k0, v0), (o1, k1, v1) = res
            assert torch.equal(v0, v1)
            assert (k0 - k1).abs().max().item() <= 2 ** -7 * max(k0.abs().max().item(), 1.0)
            assert (k0 != kp0.float()).any() or all(kl == 0 for kl in kv_lens)  # the new keys were written
            live = [r for r, kl in enumerate(kv_lens) if kl > 0]
            scale_o = max(o0[live].abs().max().item(), 1e-6)
            assert (o0[live] - o1[live]).abs().max().item() <= 2e-2 * scale_o, (cluster, target)
            assert (o1[[r for r in range(batch) if r not in live]] == 0).all()
    finally:
        K().use_balanced_decode, K().use_tcgen05_decode = old[0], old[1]
        K().set_decode_cluster_merge(old[2])
        K().decode_split_target = old[3]
