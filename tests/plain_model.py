"""Plain, slow implementation of the Qwen3 dense decoder, written from the
reference's formulas.  Whole sequences, no cache, one function for each part.

It shares no code with the engine: it takes a plain dict of HF-named tensors
and a plain dict of config.json keys.  Every function cites the reference file
and lines (paths inside izmttk/ullm) whose arithmetic it restates.

All arithmetic runs in the dtype of the weights given (float32 in the tests,
optionally float64 for a tighter oracle); the rotary table is always built in
float32 first, as the reference builds it.
"""

from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather, ullm/layers/vocab_parallel_embedding.py:117 (tp=1 path)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ullm/layers/layernorm.py:20-34: mean of squares over the last dim,
    rsqrt(var + eps), then times the weight."""
    var = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def rope_table(head_dim: int, theta: float, max_pos: int) -> tuple[torch.Tensor, torch.Tensor]:
    """ullm/layers/rotary_embedding.py:58-75: inv_freq_i = 1/theta^(2i/D),
    angle[p, i] = p * inv_freq_i, all in float32.  Returns (cos, sin), each
    [max_pos, D/2] float32."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    return freqs.cos(), freqs.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """ullm/layers/rotary_embedding.py:5-24.  x [T, heads, D]; cos/sin [T, D/2].
    x1/x2 are the two halves of the head; o1 = x1 cos - x2 sin,
    o2 = x2 cos + x1 sin.  The reference interleaves (o1, o2) in its output;
    the same permutation is applied to q and k, so q.k is unchanged by keeping
    the halves contiguous as done here."""
    cos = cos.unsqueeze(-2).to(x.dtype)
    sin = sin.unsqueeze(-2).to(x.dtype)
    x1, x2 = torch.chunk(x, 2, dim=-1)
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


def causal_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: float,
    window: int | None = None,
) -> torch.Tensor:
    """Scores, mask, softmax, weighted sum for one whole sequence.
    q [T, Hq, D], k/v [T, Hkv, D] -> [T, Hq, D].

    ullm/models/qwen3.py:81 (scale = D^-0.5), ullm/layers/attention.py:66-91
    (causal, grouped heads: query head h reads kv head h // (Hq/Hkv)).  With a
    window w, query p sees keys p-w+1 .. p."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    out = torch.empty_like(q)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    hidden = j > i
    if window is not None:
        hidden = hidden | (j <= i - window)
    for h in range(Hq):
        kh = h // group
        s = (q[:, h] @ k[:, kh].T) * scale
        s = s.masked_fill(hidden, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h] = p @ v[:, kh]
    return out


def attention_block(
    h: torch.Tensor,
    w: dict[str, torch.Tensor],
    prefix: str,
    cfg: dict,
    positions: torch.Tensor,
    window: int | None = None,
    shared_kv: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> tuple[torch.Tensor, tuple[torch.Tensor, torch.Tensor]]:
    """ullm/models/qwen3.py:113-130: qkv projection, per-head q/k RMSNorm,
    rotation, attention, output projection.  Returns (output, (k, v)) so that a
    later layer can read this layer's keys and values."""
    T = h.shape[0]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = h @ w[prefix + "q_proj.weight"].T
    k = h @ w[prefix + "k_proj.weight"].T
    v = h @ w[prefix + "v_proj.weight"].T
    if prefix + "q_proj.bias" in w:
        q = q + w[prefix + "q_proj.bias"]
        k = k + w[prefix + "k_proj.bias"]
        v = v + w[prefix + "v_proj.bias"]
    q = rms_norm(q.view(T, Hq, D), w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k.view(T, Hkv, D), w[prefix + "k_norm.weight"], eps)
    v = v.view(T, Hkv, D)
    cos, sin = rope_table(D, cfg["rope_theta"], int(positions.max()) + 1)
    q = apply_rope(q, cos[positions], sin[positions])
    k = apply_rope(k, cos[positions], sin[positions])
    if shared_kv is not None:
        k, v = shared_kv
    a = causal_attention(q, k, v, D ** -0.5, window)
    return a.reshape(T, Hq * D) @ w[prefix + "o_proj.weight"].T, (k, v)


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """ullm/layers/activation.py:16-18: silu(gate) * up."""
    return gate * torch.sigmoid(gate) * up


def gated_mlp(h: torch.Tensor, w: dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """ullm/models/qwen3.py:42-46."""
    g = h @ w[prefix + "gate_proj.weight"].T
    u = h @ w[prefix + "up_proj.weight"].T
    return silu_mul(g, u) @ w[prefix + "down_proj.weight"].T


def layer_window(cfg: dict, layer: int) -> int | None:
    """Window of a layer from the config.json keys use_sliding_window,
    sliding_window and max_window_layers (the reference never reads them,
    ullm/models/qwen3.py:136-157; layers from max_window_layers on are
    windowed when the switch is on)."""
    if cfg.get("use_sliding_window") and cfg.get("sliding_window"):
        if layer >= cfg.get("max_window_layers", 0):
            return int(cfg["sliding_window"])
    return None


def decoder_layer(
    x: torch.Tensor,
    w: dict[str, torch.Tensor],
    layer: int,
    cfg: dict,
    positions: torch.Tensor,
    shared_kv=None,
):
    """ullm/models/qwen3.py:160-178 with the residual written out: the stream
    x carries hidden + residual of the reference's fused add-and-norm form."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    a, kv = attention_block(
        h, w, p + "self_attn.", cfg, positions, layer_window(cfg, layer), shared_kv
    )
    x = x + a
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + gated_mlp(h, w, p + "mlp.")
    return x, kv


def lm_head(h: torch.Tensor, w: dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """ullm/models/qwen3.py:284-286.  A tied model reads the embedding table
    (the reference never ties; a tied checkpoint only works there when the file
    carries lm_head.weight)."""
    if "lm_head.weight" in w:
        return h @ w["lm_head.weight"].T
    if not cfg.get("tie_word_embeddings", False):
        raise KeyError("lm_head.weight")
    return h @ w["model.embed_tokens.weight"].T


def forward_logits(
    ids,
    w: dict[str, torch.Tensor],
    cfg: dict,
    schedule: list[tuple[int, int | None]] | None = None,
) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence.
    ullm/models/qwen3.py:228-255 then compute_logits.

    `schedule` lists (layer, position in the schedule whose keys and values to
    read, or None); the default runs every layer once, in order."""
    cfg = normalized(cfg)
    ids = torch.as_tensor(ids)
    T = ids.shape[0]
    positions = torch.arange(T)
    x = embed(ids, w["model.embed_tokens.weight"])
    if schedule is None:
        schedule = [(l, None) for l in range(cfg["num_hidden_layers"])]
    kvs = []
    for layer, share in schedule:
        x, kv = decoder_layer(
            x, w, layer, cfg, positions, None if share is None else kvs[share]
        )
        kvs.append(kv)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    return lm_head(x, w, cfg)


def normalized(cfg: dict) -> dict:
    """Defaults the reference applies: head_dim = H // Hq
    (ullm/models/qwen3.py:77), rope_theta 1e6 (qwen3.py:144)."""
    cfg = dict(cfg)
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    if cfg.get("head_dim") is None:
        cfg["head_dim"] = cfg["hidden_size"] // cfg["num_attention_heads"]
    cfg.setdefault("rope_theta", 1000000.0)
    cfg.setdefault("rms_norm_eps", 1e-6)
    return cfg


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------
def filtered_distribution(
    logits: torch.Tensor,
    temperature: float,
    top_k: int,
    top_p: float,
    min_p: float,
) -> torch.Tensor:
    """Probabilities after temperature, top-k, top-p and min-p, for one row.
    ullm/layers/sampler.py:39-52 and :59-107, restated without the sort's
    scatter: top-k keeps values >= the k-th largest (ties kept); top-p removes,
    on the ascending order, every entry whose running mass is <= 1 - p (never
    the largest); min-p removes probabilities below min_p * max."""
    x = logits.to(torch.float32).clone()
    V = x.shape[-1]
    if temperature > 0:
        x = x / temperature
    k = V if top_k <= 0 else min(top_k, V)
    srt, idx = torch.sort(x, descending=False, stable=True)
    thresh = srt[V - k]
    srt = srt.masked_fill(srt < thresh, float("-inf"))
    p = 1.0 if top_p <= 0 else top_p
    probs = torch.softmax(srt, dim=-1)
    cum = torch.cumsum(probs, dim=-1)
    mask = cum <= 1 - p
    mask[-1] = False
    srt = srt.masked_fill(mask, float("-inf"))
    x = torch.empty_like(srt).scatter_(0, idx, srt)
    probs = torch.softmax(x, dim=-1)
    x = x.masked_fill(probs < min_p * probs.max(), float("-inf"))
    return torch.softmax(x, dim=-1)


def greedy(logits: torch.Tensor) -> int:
    """ullm/layers/sampler.py:35-36 (argmax); lowest index on ties."""
    return int(torch.argmax(logits.to(torch.float32)))


def inverse_cdf_draw(probs: torch.Tensor, u: float) -> int:
    """First index whose running sum of probabilities exceeds u * total."""
    c = torch.cumsum(probs.double(), 0)
    target = u * float(c[-1])
    return int(min(int(torch.searchsorted(c, torch.tensor(target, dtype=c.dtype), right=True)), probs.numel() - 1))


def greedy_generate(prompt, w, cfg, n_new: int, schedule=None) -> list[int]:
    """Greedy continuation by re-running the whole sequence for every token."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        lg = forward_logits(ids, w, cfg, schedule)
        nxt = greedy(lg[-1])
        out.append(nxt)
        ids.append(nxt)
    return out


# --------------------------------------------------------------------------
# random weights for the tests (independent of the engine's generator)
# --------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    cfg = normalized(cfg)
    H, Hq, Hkv, D = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    I, V = cfg["intermediate_size"], cfg["vocab_size"]
    shapes: dict[str, tuple[int, ...]] = {"model.embed_tokens.weight": (V, H)}
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        shapes[p + "input_layernorm.weight"] = (H,)
        shapes[p + "post_attention_layernorm.weight"] = (H,)
        shapes[p + "self_attn.q_proj.weight"] = (Hq * D, H)
        shapes[p + "self_attn.k_proj.weight"] = (Hkv * D, H)
        shapes[p + "self_attn.v_proj.weight"] = (Hkv * D, H)
        if cfg.get("attention_bias", False):
            shapes[p + "self_attn.q_proj.bias"] = (Hq * D,)
            shapes[p + "self_attn.k_proj.bias"] = (Hkv * D,)
            shapes[p + "self_attn.v_proj.bias"] = (Hkv * D,)
        shapes[p + "self_attn.o_proj.weight"] = (H, Hq * D)
        shapes[p + "self_attn.q_norm.weight"] = (D,)
        shapes[p + "self_attn.k_norm.weight"] = (D,)
        shapes[p + "mlp.gate_proj.weight"] = (I, H)
        shapes[p + "mlp.up_proj.weight"] = (I, H)
        shapes[p + "mlp.down_proj.weight"] = (H, I)
    shapes["model.norm.weight"] = (H,)
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (V, H)
    return shapes


def random_weights(cfg: dict, seed: int, std: float, norm_std: float, dtype=torch.float32):
    """Linears and embedding N(0, std); norm weights 1 + N(0, norm_std)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm.weight"):
            t = 1.0 + torch.randn(shape, generator=g) * norm_std
        else:
            t = torch.randn(shape, generator=g) * std
        w[name] = t.to(dtype)
    return w
