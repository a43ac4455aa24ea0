"""Each part alone against its plain counterpart, and a toy mixer with state of
its own that is registered, built and stepped without touching the framework."""

import pytest
import torch

import plain_model as pm
from conftest import device
from helpers import TOL, assert_close, errors, random_ids, weights_for, write_model_dir

pytestmark = pytest.mark.gpu


def runner_for(tmp_path, tag, dtype, **kw):
    from ullm_b200.engine import ModelRunner

    cfg, w, page = weights_for(tag, dtype)
    d = write_model_dir(str(tmp_path / f"m{tag}{dtype}"), cfg, w)
    r = ModelRunner(d, dtype=dtype, device=device(), page_size=page, num_pages=32, max_requests=4,
                    max_context=cfg["max_position_embeddings"], max_step_tokens=64, poison_cache=True, **kw)
    return r, cfg, {k: v.float() for k, v in w.items()}


def rand(shape, seed, dtype, scale=1.0):
    t = torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale
    return t.to(dtype).to(device())


def part_close(got, ref, dtype, what):
    mx, _ = errors(got, ref)
    assert mx <= (2e-5 if dtype == "float32" else 2e-2), f"{what}: max err {mx:.2e} of scale"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(tmp_path, dtype):
    r, cfg, w = runner_for(tmp_path, "B", dtype)
    norm = r.model.blocks[1].mixer_norm
    td = r.dtype
    x, res = rand((11, 80), 1, td), rand((11, 80), 2, td)
    s = x.float().cpu() + res.float().cpu()
    ref = pm.rms_norm(s, w["model.layers.1.input_layernorm.weight"], cfg["rms_norm_eps"])
    res2 = res.clone()
    out = norm.forward(x.clone(), res2)
    part_close(out, ref, dtype, "fused add + norm")
    assert torch.equal(res2.cpu(), s.to(td))
    part_close(norm.forward(x.clone()), pm.rms_norm(x.float().cpu(), w["model.layers.1.input_layernorm.weight"],
                                                   cfg["rms_norm_eps"]), dtype, "norm alone")


def test_position_part_tables():
    from ullm_b200.parts.position import RotaryPositions

    p = RotaryPositions(rotary_dim=48, theta=50000.0, max_positions=300)
    p.build_tables("cpu")
    cos, sin = pm.rope_table(48, 50000.0, 300)
    assert torch.equal(p.tables()["cos"], cos) and torch.equal(p.tables()["sin"], sin)
    with pytest.raises(ValueError):
        RotaryPositions(rotary_dim=7, theta=1.0, max_positions=4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_feed_forward_and_head_parts(tmp_path, dtype):
    from ullm_b200.engine.batch import Workspace

    r, cfg, w = runner_for(tmp_path, "C", dtype)
    td = r.dtype

    class Ctx:
        workspace = Workspace(r.device)

    ids = torch.tensor(random_ids(cfg["vocab_size"], 9, 3), dtype=torch.int32, device=r.device)
    emb = torch.empty(9, cfg["hidden_size"], dtype=td, device=r.device)
    r.model.embedding.forward(ids, emb)
    assert torch.equal(emb.float().cpu(), pm.embed(ids.cpu(), w["model.embed_tokens.weight"]))
    x = rand((13, cfg["hidden_size"]), 4, td)
    y = r.model.blocks[2].feed_forward.forward(x, Ctx())
    part_close(y, pm.gated_mlp(x.float().cpu(), w, "model.layers.2.mlp."), dtype, "gated mlp")
    lg = torch.empty(13, cfg["vocab_size"], dtype=torch.float32, device=r.device)
    r.model.head.forward(x, lg)
    part_close(lg, pm.lm_head(x.float().cpu(), w, cfg), dtype, "head")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [0, 3])
def test_attention_part_and_block_alone(tmp_path, dtype, layer):
    """The mixer and the whole block of one layer (layer 3 of C is windowed), fed
    with random activations in two steps: 40 tokens, then 9 more."""
    from ullm_b200.engine import StepEntry

    r, cfg, w = runner_for(tmp_path, "C", dtype)
    td, H = r.dtype, cfg["hidden_size"]
    x_all = rand((49, H), 5 + layer, td, 0.5)
    res_all = rand((49, H), 6 + layer, td, 0.5)
    pre = f"model.layers.{layer}."
    pos = torch.arange(49)
    # plain: attention over the whole 49 tokens, then the block
    ref_attn, _ = pm.attention_block(x_all.float().cpu(), w, pre + "self_attn.", pm.normalized(cfg), pos,
                                     pm.layer_window(cfg, layer))
    stream = x_all.float().cpu() + res_all.float().cpu()
    ref_stream, _ = pm.decoder_layer(stream, w, layer, pm.normalized(cfg), pos)
    got_attn, got_y, got_res = [], [], []
    ids = random_ids(cfg["vocab_size"], 49, 7)
    # the mixer alone and the whole block write different keys: each gets a request (pages) of its own
    for rid in ("mixer", "block"):
        r.add_request(rid)
        for a, b in ((0, 40), (40, 49)):
            entries = [StepEntry(rid, ids[a:b], [])]
            ctx = r.prepare(entries)
            caches = r.cache.layer_caches(ctx.groups)
            if rid == "mixer":
                out = r.model.blocks[layer].mixer.forward(x_all[a:b].clone(), ctx, caches[layer])
                got_attn.append(out.float().cpu().clone())
            else:
                res = res_all[a:b].clone()
                y, res = r.model.blocks[layer].forward(x_all[a:b].clone(), res, ctx, caches[layer])
                got_y.append(y.float().cpu().clone())
                got_res.append(res.float().cpu().clone())
            r.commit(entries)
    r.check_device_status()
    part_close(torch.cat(got_attn), ref_attn, dtype, "attention part")
    part_close(torch.cat(got_y) + torch.cat(got_res), ref_stream, dtype, "block")


# ---------------------------------------------------------------------------------------
# a toy mixer with per-request state, defined here
# ---------------------------------------------------------------------------------------
def _register_toy():
    from ullm_b200.config import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                  ScheduleEntry, register_architecture)
    from ullm_b200.parts import Mixer, ParamDecl, StateNeed, register_mixer

    @register_mixer("running_mean")
    class RunningMean(Mixer):
        """out_t = mean(x_0 .. x_t) W^T.  State per request: the running sum (hidden floats) and the count."""

        def __init__(self, hidden_size: int):
            super().__init__()
            self.hidden_size = hidden_size

        def param_decls(self):
            return {"mix.weight": ParamDecl((self.hidden_size, self.hidden_size))}

        def state_need(self):
            return StateNeed((self.hidden_size + 1,), torch.float32)

        def forward(self, x, ctx, cache):
            H = self.hidden_size
            out = ctx.workspace.get("toy.out", x.shape[0], H, x.dtype)
            W = self.tensors["mix.weight"].float()
            for b in range(ctx.num_requests):
                lo, hi = ctx.cu_q_host[b], ctx.cu_q_host[b + 1]
                row = cache.state[ctx.req_slots_host[b]]
                sums = torch.cumsum(x[lo:hi].float(), 0) + row[:H]
                counts = row[H] + torch.arange(1, hi - lo + 1, device=x.device, dtype=torch.float32)
                out[lo:hi] = ((sums / counts[:, None]) @ W.t()).to(x.dtype)
                row[:H] = sums[-1]
                row[H] = counts[-1]
            return out

    def parse(d):
        return d

    def spec(d):
        H = d["hidden_size"]
        norm = NormSpec("rmsnorm", H, d["eps"])
        ff = FeedForwardSpec("gated_mlp", dict(hidden_size=H, intermediate_size=d["intermediate_size"], activation="silu"))
        names = dict(mixer="mixer.", feed_forward="mlp.", mixer_norm="norm1.", feed_forward_norm="norm2.")
        toy = LayerSpec("prenorm_residual", MixerSpec("running_mean", dict(hidden_size=H)), ff, norm, norm, names)
        att = LayerSpec("prenorm_residual", MixerSpec("paged_attention", dict(
            hidden_size=H, num_heads=d["heads"], num_kv_heads=d["kv_heads"], head_dim=d["head_dim"],
            qk_norm=NormSpec("rmsnorm", d["head_dim"], d["eps"]),
            position=PositionSpec("rope", d["head_dim"], d["theta"], d["max_positions"]))), ff, norm, norm, names)
        return ModelSpec(architecture="ToyForCausalLM", hidden_size=H, vocab_size=d["vocab_size"], layers=[toy, att, toy],
                         schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2)], final_norm=norm,
                         tie_embeddings=True, max_positions=d["max_positions"], dtype="float32",
                         embedding_name="emb.", layer_name="layers.{}.", final_norm_name="final_norm.", head_name="head.")

    register_architecture("ToyForCausalLM", parse, spec)


TOY = dict(architectures=["ToyForCausalLM"], hidden_size=48, intermediate_size=72, vocab_size=97, heads=4, kv_heads=2,
           head_dim=16, eps=1e-5, theta=10000.0, max_positions=128)


def toy_plain(ids, w):
    """Whole-sequence reference of the toy model."""
    T = len(ids)
    x = w["emb.weight"][torch.tensor(ids)]
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5, rope_theta=10000.0)
    for l in range(3):
        p = f"layers.{l}."
        h = pm.rms_norm(x, w[p + "norm1.weight"], 1e-5)
        if l == 1:
            a, _ = pm.attention_block(h, w, p + "mixer.", cfg, torch.arange(T))
        else:
            means = torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]
            a = means @ w[p + "mixer.mix.weight"].T
        x = x + a
        h = pm.rms_norm(x, w[p + "norm2.weight"], 1e-5)
        x = x + pm.gated_mlp(h, w, p + "mlp.")
    return pm.rms_norm(x, w["final_norm.weight"], 1e-5) @ w["emb.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_registers_builds_and_steps(dtype):
    from ullm_b200.config import ARCHITECTURES
    from ullm_b200.engine import ModelRunner, StepEntry
    from ullm_b200.parts import MIXERS

    _register_toy()
    try:
        r = ModelRunner(config=TOY, dtype=dtype, device=device(), page_size=8, num_pages=16, max_requests=3,
                        max_context=128, max_step_tokens=64, load_format="random", seed=3, random_std=0.2,
                        random_norm_std=0.1)
        assert r.cache.tree is None, "prefix reuse is off for a model with per-request state"
        assert sorted(r.cache.states) == [0, 2] and r.cache.states[0].shape == (3, 49)
        w = {n: t.float().cpu() for n, t in r.model.all_tensors().items()}
        a, b = random_ids(97, 60, 1), random_ids(97, 41, 2)
        ra, rb = toy_plain(a, w), toy_plain(b, w)
        r.add_request("a")
        r.add_request("b")
        got_a, got_b = [], []
        # portions of a beside portions and single tokens of b
        plan = [(7, 2), (2, 30), (20, 1), (1, 1), (30, 7)]
        ia = ib = 0
        for na, nb in plan:
            lg = r.step([StepEntry("a", a[ia:ia + na], list(range(na))), StepEntry("b", b[ib:ib + nb], list(range(nb)))])
            got_a.append(lg[:na].float().cpu().clone())
            got_b.append(lg[na:].float().cpu().clone())
            ia += na
            ib += nb
        r.check_device_status()
        assert_close(torch.cat(got_a), ra[:ia], dtype, "toy a")
        assert_close(torch.cat(got_b), rb[:ib], dtype, "toy b")
        # a slot that is handed out again starts from zeroed state
        r.end_request("a")
        r.add_request("c")
        lg = r.step([StepEntry("c", a[:10], list(range(10)))])
        assert_close(lg.float().cpu(), ra[:10], dtype, "toy c on a reused slot")
    finally:
        ARCHITECTURES.pop("ToyForCausalLM", None)
        MIXERS.pop("running_mean", None)


# ---------------------------------------------------------------------------------------
# a toy feed-forward with routing and a toy position encoding, defined here
# ---------------------------------------------------------------------------------------
def _register_toy_routing():
    from ullm_b200.config import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                  ScheduleEntry, register_architecture)
    from ullm_b200.parts import (FeedForward, ParamDecl, PositionEncoding, register_feed_forward,
                                 register_position_encoding)

    @register_position_encoding("slow_partial_rope")
    class SlowPartialRope(PositionEncoding):
        """Rotates the first `rotary_dim` elements of a head only, with positions divided by `factor`."""

        def __init__(self, rotary_dim, theta, max_positions, factor=1.0):
            super().__init__()
            self.rotary_dim, self.theta, self.max_positions, self.factor = rotary_dim, theta, max_positions, factor
            self._tables = {}

        def build_tables(self, device):
            inv = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim))
            ang = (torch.arange(self.max_positions, dtype=torch.float32) / self.factor)[:, None] * inv[None, :]
            self._tables = {"cos": ang.cos().contiguous().to(device), "sin": ang.sin().contiguous().to(device)}

        def tables(self):
            return self._tables

    @register_feed_forward("top1_experts")
    class Top1Experts(FeedForward):
        """Each token goes to the expert whose router logit (32-bit) is largest; experts are small gated MLPs."""

        def __init__(self, hidden_size, intermediate_size, num_experts):
            super().__init__()
            self.H, self.I, self.E = hidden_size, intermediate_size, num_experts

        def param_decls(self):
            d = {"router.weight": ParamDecl((self.E, self.H))}
            for e in range(self.E):
                d[f"experts.{e}.gate_up.weight"] = ParamDecl((2 * self.I, self.H))
                d[f"experts.{e}.down.weight"] = ParamDecl((self.H, self.I))
            return d

        def forward(self, x, ctx):
            out = ctx.workspace.get("toy.ffn_out", x.shape[0], self.H, x.dtype)
            xf = x.float()
            choice = (xf @ self.tensors["router.weight"].float().t()).argmax(-1)
            for e in range(self.E):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                gu = xf[rows] @ self.tensors[f"experts.{e}.gate_up.weight"].float().t()
                act = torch.nn.functional.silu(gu[:, :self.I]) * gu[:, self.I:]
                out[rows] = (act.to(x.dtype).float() @ self.tensors[f"experts.{e}.down.weight"].float().t()).to(x.dtype)
            return out

    def spec(d):
        H = d["hidden_size"]
        norm = NormSpec("rmsnorm", H, d["eps"])
        names = dict(mixer="mixer.", feed_forward="mlp.", mixer_norm="norm1.", feed_forward_norm="norm2.")
        att = MixerSpec("paged_attention", dict(
            hidden_size=H, num_heads=d["heads"], num_kv_heads=d["kv_heads"], head_dim=d["head_dim"],
            qk_norm=NormSpec("rmsnorm", d["head_dim"], d["eps"]),
            position=PositionSpec("slow_partial_rope", d["rotary_dim"], d["theta"], d["max_positions"],
                                  dict(factor=d["factor"]))))
        routed = FeedForwardSpec("top1_experts", dict(hidden_size=H, intermediate_size=d["intermediate_size"],
                                                      num_experts=d["experts"]))
        dense = FeedForwardSpec("gated_mlp", dict(hidden_size=H, intermediate_size=d["intermediate_size"],
                                                  activation="silu"))
        layers = [LayerSpec("prenorm_residual", att, routed, norm, norm, names),
                  LayerSpec("prenorm_residual", att, dense, norm, norm, names)]
        return ModelSpec(architecture="ToyRoutedForCausalLM", hidden_size=H, vocab_size=d["vocab_size"], layers=layers,
                         schedule=[ScheduleEntry(0), ScheduleEntry(1)], final_norm=norm, tie_embeddings=True,
                         max_positions=d["max_positions"], dtype="float32", embedding_name="emb.",
                         layer_name="layers.{}.", final_norm_name="final_norm.", head_name="head.")

    register_architecture("ToyRoutedForCausalLM", lambda d: d, spec)


TOY_ROUTED = dict(architectures=["ToyRoutedForCausalLM"], hidden_size=40, intermediate_size=56, vocab_size=83, heads=4,
                  kv_heads=1, head_dim=16, rotary_dim=8, factor=4.0, experts=3, eps=1e-5, theta=100.0, max_positions=96)


def toy_routed_plain(ids, w, round_to=None):
    """Whole-sequence reference of the routed toy model.  `round_to`: the engine's dtype, applied where the toy
    feed-forward itself rounds (its activation), so that routing ties are the only thing left to differ."""
    d = TOY_ROUTED
    T, D, r = len(ids), d["head_dim"], d["rotary_dim"]
    x = w["emb.weight"][torch.tensor(ids)]
    inv = 1.0 / (d["theta"] ** (torch.arange(0, r, 2, dtype=torch.float32) / r))
    ang = (torch.arange(T, dtype=torch.float32) / d["factor"])[:, None] * inv[None, :]

    def rot(t):  # [T, heads, D]: the first r elements rotate, the rest pass
        return torch.cat((pm.apply_rope(t[..., :r], ang.cos(), ang.sin()), t[..., r:]), -1)

    for l in range(2):
        p = f"layers.{l}."
        h = pm.rms_norm(x, w[p + "norm1.weight"], d["eps"])
        m = p + "mixer."
        q = pm.rms_norm((h @ w[m + "q_proj.weight"].T).view(T, d["heads"], D), w[m + "q_norm.weight"], d["eps"])
        k = pm.rms_norm((h @ w[m + "k_proj.weight"].T).view(T, d["kv_heads"], D), w[m + "k_norm.weight"], d["eps"])
        v = (h @ w[m + "v_proj.weight"].T).view(T, d["kv_heads"], D)
        a = pm.causal_attention(rot(q), rot(k), v, D ** -0.5, None)
        x = x + a.reshape(T, -1) @ w[m + "o_proj.weight"].T
        h = pm.rms_norm(x, w[p + "norm2.weight"], d["eps"])
        if l == 0:
            choice = (h @ w[p + "mlp.router.weight"].T).argmax(-1)
            y = torch.zeros_like(h)
            for t in range(T):
                e = int(choice[t])
                gu = h[t] @ w[p + f"mlp.experts.{e}.gate_up.weight"].T
                act = pm.silu_mul(gu[:d["intermediate_size"]], gu[d["intermediate_size"]:])
                y[t] = act @ w[p + f"mlp.experts.{e}.down.weight"].T
            x = x + y
        else:
            x = x + pm.gated_mlp(h, w, p + "mlp.")
    return pm.rms_norm(x, w["final_norm.weight"], d["eps"]) @ w["emb.weight"].T


def test_toy_routed_feed_forward_and_another_position_encoding_register_build_and_step():
    """A feed-forward that routes tokens to experts and a position encoding with a constant of its own
    (positions divided by a factor, part of the head rotated), both defined here, are registered, built from a
    specification and stepped (whole, and in portions beside another request) without a change to the package."""
    from ullm_b200.config import ARCHITECTURES
    from ullm_b200.engine import ModelRunner, StepEntry
    from ullm_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS

    _register_toy_routing()
    try:
        r = ModelRunner(config=TOY_ROUTED, dtype="float32", device=device(), page_size=8, num_pages=24, max_requests=3,
                        max_context=96, max_step_tokens=64, load_format="random", seed=5, random_std=0.3,
                        random_norm_std=0.1)
        w = {n: t.float().cpu() for n, t in r.model.all_tensors().items()}
        a, b = random_ids(83, 50, 3), random_ids(83, 33, 4)
        ra, rb = toy_routed_plain(a, w), toy_routed_plain(b, w)
        r.add_request("whole")
        lg = r.step([StepEntry("whole", a, list(range(len(a))))])
        assert_close(lg.float().cpu(), ra, "float32", "routed toy, whole")
        r.end_request("whole")
        r.add_request("a")
        r.add_request("b")
        got_a, got_b = [], []
        ia = ib = 0
        for na, nb in [(9, 2), (2, 20), (25, 1), (1, 1), (13, 9)]:
            lg = r.step([StepEntry("a", a[ia:ia + na], list(range(na))), StepEntry("b", b[ib:ib + nb], list(range(nb)))])
            got_a.append(lg[:na].float().cpu().clone())
            got_b.append(lg[na:].float().cpu().clone())
            ia += na
            ib += nb
        r.check_device_status()
        assert_close(torch.cat(got_a), ra[:ia], "float32", "routed toy a")
        assert_close(torch.cat(got_b), rb[:ib], "float32", "routed toy b")
    finally:
        ARCHITECTURES.pop("ToyRoutedForCausalLM", None)
        FEED_FORWARDS.pop("top1_experts", None)
        POSITION_ENCODINGS.pop("slow_partial_rope", None)


# ---------------------------------------------------------------------------------------------------------
# a position encoding that is no rotation by tables: it changes queries and keys with code of its own
# ---------------------------------------------------------------------------------------------------------
TOY_GAIN = dict(architectures=["ToyGainForCausalLM"], hidden_size=48, intermediate_size=64, vocab_size=97, heads=6,
                kv_heads=2, head_dim=16, eps=1e-5, gain=0.03, drift=0.2, max_positions=128)


def _register_toy_gain():
    from ullm_b200.config import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                  ScheduleEntry, register_architecture)
    from ullm_b200.parts import PositionEncoding, register_position_encoding

    @register_position_encoding("position_gain")
    class PositionGain(PositionEncoding):
        """Queries grow with their position, keys get a position-dependent offset: no rotation, no tables."""

        def __init__(self, rotary_dim, theta, max_positions, gain=0.0, drift=0.0):
            super().__init__()
            self.gain, self.drift, self.max_positions = gain, drift, max_positions

        def transforms_qk(self):
            return True

        def apply(self, q, k, positions):
            pos = positions.to(torch.float32)
            q.mul_((1.0 + self.gain * pos)[:, None, None].to(q.dtype))
            k.add_((self.drift * torch.sin(0.1 * pos))[:, None, None].to(k.dtype))

    def spec(d):
        H = d["hidden_size"]
        norm = NormSpec("rmsnorm", H, d["eps"])
        names = dict(mixer="mixer.", feed_forward="mlp.", mixer_norm="norm1.", feed_forward_norm="norm2.")
        att = MixerSpec("paged_attention", dict(
            hidden_size=H, num_heads=d["heads"], num_kv_heads=d["kv_heads"], head_dim=d["head_dim"],
            qk_norm=NormSpec("rmsnorm", d["head_dim"], d["eps"]),
            position=PositionSpec("position_gain", 0, 0.0, d["max_positions"], dict(gain=d["gain"], drift=d["drift"]))))
        dense = FeedForwardSpec("gated_mlp", dict(hidden_size=H, intermediate_size=d["intermediate_size"], activation="silu"))
        layers = [LayerSpec("prenorm_residual", att, dense, norm, norm, names) for _ in range(2)]
        return ModelSpec(architecture="ToyGainForCausalLM", hidden_size=H, vocab_size=d["vocab_size"], layers=layers,
                         schedule=[ScheduleEntry(0), ScheduleEntry(1)], final_norm=norm, tie_embeddings=True,
                         max_positions=d["max_positions"], dtype="float32", embedding_name="emb.",
                         layer_name="layers.{}.", final_norm_name="final_norm.", head_name="head.")

    register_architecture("ToyGainForCausalLM", lambda d: d, spec)


def toy_gain_plain(ids, w):
    d = TOY_GAIN
    T, D = len(ids), d["head_dim"]
    x = w["emb.weight"][torch.tensor(ids)]
    pos = torch.arange(T, dtype=torch.float32)
    for l in range(2):
        p = f"layers.{l}."
        h = pm.rms_norm(x, w[p + "norm1.weight"], d["eps"])
        m = p + "mixer."
        q = pm.rms_norm((h @ w[m + "q_proj.weight"].T).view(T, d["heads"], D), w[m + "q_norm.weight"], d["eps"])
        k = pm.rms_norm((h @ w[m + "k_proj.weight"].T).view(T, d["kv_heads"], D), w[m + "k_norm.weight"], d["eps"])
        v = (h @ w[m + "v_proj.weight"].T).view(T, d["kv_heads"], D)
        q = q * (1.0 + d["gain"] * pos)[:, None, None]
        k = k + (d["drift"] * torch.sin(0.1 * pos))[:, None, None]
        a = pm.causal_attention(q, k, v, D ** -0.5, None)
        x = x + a.reshape(T, -1) @ w[m + "o_proj.weight"].T
        h = pm.rms_norm(x, w[p + "norm2.weight"], d["eps"])
        x = x + pm.gated_mlp(h, w, p + "mlp.")
    return pm.rms_norm(x, w["final_norm.weight"], d["eps"]) @ w["emb.weight"].T


def test_a_position_encoding_with_code_of_its_own_registers_builds_and_steps():
    """An encoding that is no rotation by tables (queries scaled and keys shifted by functions of the position,
    written here with plain tensor operations) is registered, built from a specification and stepped: whole, one
    token at a time and in portions, against the plain computation; the keys it changed are the keys the cache
    holds."""
    from ullm_b200.config import ARCHITECTURES
    from ullm_b200.engine import ModelRunner, StepEntry
    from ullm_b200.parts.registry import POSITION_ENCODINGS

    _register_toy_gain()
    try:
        runner = ModelRunner(config=TOY_GAIN, dtype="float32", device=device(), page_size=8, num_pages=24,
                             max_requests=2, max_context=96, max_step_tokens=64, load_format="random", seed=5,
                             random_std=0.2, random_norm_std=0.1, poison_cache=True)
        w = {n: t.float().cpu() for n, t in runner.model.all_tensors().items()}
        ids = random_ids(TOY_GAIN["vocab_size"], 60, 3)
        ref = toy_gain_plain(ids, w)
        assert not torch.allclose(ref, toy_gain_plain(ids[:30] + ids[30:][::-1], w)[:60], atol=1e-3)
        for cuts in ([60], [28] + [1] * 32, [7, 2, 5, 3, 16, 2, 1, 9, 15]):
            runner.add_request("a")
            outs, i = [], 0
            for n in cuts:
                outs.append(runner.step([StepEntry("a", ids[i:i + n], list(range(n)))]).float().cpu().clone())
                i += n
            runner.end_request("a")
            runner.check_device_status()
            assert_close(torch.cat(outs), ref, "float32", f"position gain, cuts {cuts[:3]}")
    finally:
        ARCHITECTURES.pop("ToyGainForCausalLM", None)
        POSITION_ENCODINGS.pop("position_gain", None)
