"""Runs izmttk/ullm's own Qwen3 model code on the CPU (float32) on the tiny
random models A and B and stores its logits, so that the plain implementation
in tests/plain_model.py can be compared with the reference once.

Usage (dev time, needs the reference tree):

    python tests/golden/make_golden.py /path/to/izmttk-ullm

Only two things of the reference are substituted, because they are GPU
libraries and not reference code: the FlashInfer paged-attention wrapper and
the Triton KV store (ullm/layers/attention.py:282-309).  A few lines of plain
torch stand in for them; every other formula that runs is the reference's own
(ullm/models/qwen3.py, ullm/layers/*.py).  The attention core of the plain
implementation therefore rests on the formulas, not on this comparison.

Writes tests/golden/ref_logits_<A|B>.pt: {"prompts": [...], "logits": [...]}
(logits at every prompt position, float32) and the Sampler's filtered
distributions on fixed logits (ullm/layers/sampler.py run on the CPU).
"""

from __future__ import annotations

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from plain_model import random_weights  # noqa: E402
from tiny_configs import ALL  # noqa: E402


class FakeKV:
    def __init__(self, L, n, Hkv, D):
        self.k = torch.zeros(L, n, Hkv, D)
        self.v = torch.zeros(L, n, Hkv, D)

    def set_kv_cache(self, layer, idx, k, v):
        m = idx >= 0
        self.k[layer, idx[m]] = k[m]
        self.v[layer, idx[m]] = v[m]

    def get_kv_cache(self, layer):
        return self.k[layer], self.v[layer]


class FakeWrapper:
    """Stands in for FlashInfer's paged prefill wrapper: gathers by slot list,
    right-aligned causal softmax, grouped heads."""

    def __init__(self, qo, kvp, kvi, Hq, Hkv):
        self.qo, self.kvp, self.kvi = qo, kvp, kvi
        self.Hq, self.Hkv = Hq, Hkv
        self._sm_scale = None

    def run(self, q, kv):
        kc, vc = kv
        kc, vc = kc[:, 0], vc[:, 0]
        out = torch.zeros_like(q)
        for r in range(len(self.qo) - 1):
            qs, qe = self.qo[r], self.qo[r + 1]
            idx = self.kvi[self.kvp[r]:self.kvp[r + 1]]
            K, V = kc[idx], vc[idx]
            ql, kl = qe - qs, len(idx)
            for h in range(self.Hq):
                kh = h // (self.Hq // self.Hkv)
                sc = (q[qs:qe, h] @ K[:, kh].T) * self._sm_scale
                ii = torch.arange(ql)[:, None]
                jj = torch.arange(kl)[None, :]
                sc = sc.masked_fill(jj > (kl - ql + ii), float("-inf"))
                out[qs:qe, h] = torch.softmax(sc, -1) @ V[:, kh]
        return out


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from transformers.models.qwen3 import Qwen3Config
    from ullm.core.common import ForwardMode
    from ullm.distributed import init_distributed_environment, initialize_model_parallel
    from ullm.layers.attention import AttentionMetadata, attention_context
    from ullm.layers.sampler import _apply_min_p, _apply_top_k_top_p
    from ullm.models.qwen3 import Qwen3ForCausalLM

    init_distributed_environment(1, 0, backend="gloo", init_method="tcp://127.0.0.1:29641")
    initialize_model_parallel(1, 1, 0, 0)
    torch.set_default_dtype(torch.float32)

    for tag in ("A", "B"):
        cfgd, init, _page = ALL[tag]
        keys = ("num_hidden_layers hidden_size num_attention_heads num_key_value_heads head_dim "
                "intermediate_size vocab_size rms_norm_eps attention_bias tie_word_embeddings "
                "use_sliding_window max_position_embeddings").split()
        cfg = Qwen3Config(**{k: cfgd[k] for k in keys})
        cfg.rope_theta = cfgd["rope_theta"]  # transformers 5 keeps it elsewhere; the reference reads this attribute
        model = Qwen3ForCausalLM(cfg).eval()
        w = random_weights(cfgd, **init)
        wl = dict(w)
        if "lm_head.weight" not in wl:  # tied: the reference needs the tensor in the file
            wl["lm_head.weight"] = wl["model.embed_tokens.weight"].clone()
        padded = {}
        if cfgd["vocab_size"] % 64:
            # The reference's own loader cannot take a vocabulary that is no
            # multiple of 64 (vocab_parallel_embedding.py:99 narrows the file's
            # tensor to the padded row count and raises).  Do by hand what it
            # intends (:100-101): rows [0, V) from the file, pad rows zero.
            for name in ("model.embed_tokens.weight", "lm_head.weight"):
                padded[name] = wl.pop(name)
        model.load_weights(iter(wl.items()))
        params = dict(model.named_parameters())
        for name, t in padded.items():
            params[name].data[: t.shape[0]].copy_(t)
            params[name].data[t.shape[0]:].zero_()
        L, Hq, Hkv, D = (cfgd["num_hidden_layers"], cfgd["num_attention_heads"],
                         cfgd["num_key_value_heads"], cfgd["head_dim"])
        g = torch.Generator().manual_seed(100 + ord(tag))
        prompts, logits = [], []
        for n in (1, 5, 17, 40):
            ids = torch.randint(0, cfgd["vocab_size"], (n,), generator=g)
            slots = torch.randperm(64, generator=g)[:n]
            kv = FakeKV(L, 64, Hkv, D)
            md = AttentionMetadata(
                forward_mode=ForwardMode.PREFILL, kv_cache=kv,
                wrapper=FakeWrapper([0, n], [0, n], slots, Hq, Hkv),
                output_kv_indices=slots,
            )
            with torch.no_grad(), attention_context(md):
                hs = model(ids, torch.arange(n))
                lg = model.compute_logits(hs)
            prompts.append(ids.tolist())
            logits.append(lg.clone())
        # the Sampler's filters on fixed logits
        fl = torch.randn(4, cfgd["vocab_size"], generator=g) * 2.0
        cases = [(0.7, 20, 0.95, 0.0), (1.0, -1, 0.5, 0.0), (1.3, 5, 1.0, 0.1), (0.5, -1, 1.0, 0.3)]
        dists = []
        for row, (t, k, p, mp) in zip(fl, cases):
            x = (row.clone().float() / t)[None]
            x = _apply_top_k_top_p(x, torch.tensor([p]), torch.tensor([k]))
            x = _apply_min_p(x, torch.tensor([mp]))
            dists.append(torch.softmax(x, -1)[0])
        torch.save(
            {"prompts": prompts, "logits": logits, "sampler_logits": fl,
             "sampler_cases": cases, "sampler_dists": dists},
            os.path.join(HERE, f"ref_logits_{tag}.pt"),
        )
        print(tag, "ok", [tuple(l.shape) for l in logits])


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/izmttk-ullm")
    main(sys.argv[1])
