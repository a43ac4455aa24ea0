"""A stand-in for ullm_b200.csrc.ops.Kernels written in plain torch, so that the
host-side logic of the engine (block tables, slot mappings, batching, windows,
scheduling) can be exercised without a GPU.  It is a test double: nothing in
the package imports it, and on a GPU the real kernels run.  It follows the
kernels' contracts (in-place updates, -1 slots skipped, padding rows zero)."""

from __future__ import annotations

import math

import torch


class CpuKernels:
    def __init__(self):
        self.status = torch.zeros(4, dtype=torch.int32)
        self.timer = None
        self.calls = {}

    def _count(self, name):
        self.calls[name] = self.calls.get(name, 0) + 1

    def raise_on_status(self):
        pass

    def linear(self, x, weight, out, bias=None):
        self._count("linear")
        y = x.float() @ weight.float().t()
        if bias is not None:
            y = y + bias.float()
        out.copy_(y.to(out.dtype))
        return out

    def linear_act_mul(self, x, weight, out, gate_up, act=0):
        self.linear(x, weight, gate_up)
        self.act_mul(gate_up, out, act)
        return out

    def linear_f32_out(self, x, weight, out):
        self._count("linear")
        out.copy_(x.float() @ weight.float().t())
        return out

    def embedding(self, ids, table, out, last_tokens=None, token_req=None, req_slots=None):
        self._count("embedding")
        idx = ids[: out.shape[0]].long().clone()
        if last_tokens is not None:
            for t in (idx < 0).nonzero().flatten().tolist():
                b = int(token_req[t])
                idx[t] = int(last_tokens[int(req_slots[b])]) if b >= 0 else 0
        out.copy_(table[idx])

    def gather_rows(self, src, rows, out):
        self._count("gather_rows")
        out.copy_(src[rows[: out.shape[0]].long()])

    def add_rmsnorm(self, x, residual, weight, eps, out):
        self._count("add_rmsnorm")
        s = x.float()
        if residual is not None:
            s = s + residual.float()
            residual.copy_(s.to(residual.dtype))
        y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * weight
        out.copy_(y.to(out.dtype))

    def act_mul(self, gate_up, out, act=0):
        self._count("act_mul")
        I = out.shape[1]
        g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
        a = g * torch.sigmoid(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")
        out.copy_((a * u).to(out.dtype))

    def layer_tail_applies(self, *args, **kwargs):
        return False

    def stream_chain_applies(self, *args, **kwargs):
        return False

    def decode_fusion_applies(self, *args, **kwargs):
        return False  # the stand-in always prepares q and k in a step of their own

    def qk_norm_rope_store(self, qkv, num_q, num_kv, D, q_w, k_w, eps, cos, sin, rotary_dim, positions,
                           slot_mapping, k_pages, v_pages):
        self._count("qk_norm_rope_store")
        T = qkv.shape[0]
        x = qkv.float().clone().view(T, num_q + 2 * num_kv, D)
        q, k, v = x[:, :num_q], x[:, num_q:num_q + num_kv], x[:, num_q + num_kv:]

        def norm(t, w):
            if w is None:
                return t
            return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w

        def rope(t):
            if rotary_dim == 0:
                return t
            half = rotary_dim // 2
            c = cos[positions[:T].long()][:, None, :]
            s = sin[positions[:T].long()][:, None, :]
            x1, x2, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
            return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), -1)

        q = rope(norm(q, q_w))
        k = rope(norm(k, k_w))
        qkv[:, : num_q * D] = q.reshape(T, num_q * D).to(qkv.dtype)
        if slot_mapping is not None:
            kf = k_pages.view(-1, num_kv, D)
            vf = v_pages.view(-1, num_kv, D)
            sm = slot_mapping[:T].long()
            ok = sm >= 0
            kf[sm[ok]] = k[ok].to(kf.dtype)
            vf[sm[ok]] = v[ok].to(vf.dtype)

    def qk_norm_in_place(self, qkv, num_q, num_kv, D, q_w, k_w, eps):
        T = qkv.shape[0]
        x = qkv.float().clone().view(T, num_q + 2 * num_kv, D)
        for lo, hi, w in ((0, num_q, q_w), (num_q, num_q + num_kv, k_w)):
            if w is not None:
                t = x[:, lo:hi]
                x[:, lo:hi] = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w
        qkv.copy_(x.view(T, -1).to(qkv.dtype))

    def paged_attention(self, qkv, out, k_pages, v_pages, block_table, req_slots, cu_q, kv_len, token_req,
                        num_q, num_kv, D, page_size, window, scale, ctx=None, ragged=False):
        self._count("paged_attention")
        T = out.shape[0]
        kf = k_pages.view(-1, num_kv, D).float()
        vf = v_pages.view(-1, num_kv, D).float()
        q = qkv[:T, : num_q * D].float().view(T, num_q, D)
        group = num_q // num_kv
        o = torch.zeros(T, num_q, D)
        for t in range(T):
            r = int(token_req[t])
            if r < 0:
                continue
            qlen = int(cu_q[r + 1] - cu_q[r])
            kvl = int(kv_len[r])
            pos = kvl - qlen + (t - int(cu_q[r]))
            if qlen <= 0 or kvl <= 0 or pos < 0:
                continue
            lo = max(0, pos - window + 1) if window > 0 else 0
            keys = torch.arange(lo, pos + 1)
            pages = block_table[int(req_slots[r])][(keys // page_size).long()].long()
            assert (pages >= 0).all(), "attention touched a page that was given back"
            slots = pages * page_size + keys % page_size
            for h in range(num_q):
                kh = h // group
                s = (kf[slots, kh] @ q[t, h]) * scale
                p = torch.softmax(s, 0)
                o[t, h] = p @ vf[slots, kh]
        out.copy_(o.reshape(T, num_q * D).to(out.dtype))

    def argmax(self, logits, out):
        out[: logits.shape[0]] = torch.argmax(logits, -1).to(torch.int32)

    def sample(self, logits, temperature, top_k, top_p, min_p, uniform, out, probs_out=None, row_slots=None,
               last_tokens=None):
        import plain_model as pm

        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t <= 0:
                out[r] = int(torch.argmax(logits[r]))
            else:
                probs = pm.filtered_distribution(logits[r], t, int(top_k[r]), float(top_p[r]), float(min_p[r]))
                out[r] = pm.inverse_cdf_draw(probs, float(uniform[r]))
                if probs_out is not None:
                    probs_out[r] = probs
            if row_slots is not None and last_tokens is not None and int(row_slots[r]) >= 0:
                last_tokens[int(row_slots[r])] = out[r]
