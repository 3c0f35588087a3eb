"""Each part of a layer alone (norm, position encoding, attention mixer, feed-forward, block,
embedding and head), and that layers are data: another mixer with state of its own, defined here,
is registered, built and stepped without a change to the library; a schedule may name a layer
twice or let a layer read another layer's cache."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_llama as plain
from helpers import TINY, TOL_BF16, TOL_F32, make_model_dir, plain_model, random_ids, rel_err

pytestmark = pytest.mark.gpu
TOL = {"float32": TOL_F32, "bfloat16": TOL_BF16}


def f64(t):
    return t.detach().cpu().to(torch.float64)


def engine_with_context(tmp_path, name, dtype, lens, pos0):
    """An engine on a tiny model whose sequences already hold pos0 tokens, and the context of a
    step that brings `lens` more: the place in which a part can be run alone."""
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    raw, seed = TINY[name]
    d = make_model_dir(tmp_path / "model", raw, seed)
    eng = Engine.from_folder(d, dtype, max_tokens=2048, use_graphs=False)
    seqs, olds = [], []
    for b, p in enumerate(pos0):
        s = eng.open()
        old = random_ids(p, raw["vocab_size"], 300 + b)
        if p:
            eng.step([StepEntry(s, old, [])])
        seqs.append(s)
        olds.append(old)
    news = [random_ids(n, raw["vocab_size"], 400 + b) for b, n in enumerate(lens)]
    entries = [StepEntry(s, t) for s, t in zip(seqs, news)]
    eng.cache.reserve([(s.slot, n) for s, n in zip(seqs, lens)])
    ids = np.concatenate(news)
    ctx = eng._context(entries, ids, lens, pos0, [])
    return eng, ctx, d, olds, news


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_parts_alone(tmp_path, name, dtype):
    lens, pos0 = [9, 1, 40], [0, 70, 33]
    eng, ctx, d, olds, news = engine_with_context(tmp_path, name, dtype, lens, pos0)
    pm = plain_model(d)
    w, cfg = pm.w, pm.cfg
    tdt = eng.dtype
    T, hid = sum(lens), cfg["hidden_size"]
    g = torch.Generator().manual_seed(5)
    rnd = (lambda t: t) if dtype == "float32" else (lambda t: t.bfloat16().float())
    block = eng.model.blocks[1]
    p = "model.layers.1."

    # embedding
    x0 = eng.model.embedding.forward(ctx.token_ids, ctx)
    assert torch.equal(f64(x0), w["model.embed_tokens.weight"][torch.as_tensor(np.concatenate(news))])

    # norm (with the residual sum)
    res = torch.randn(T, hid, generator=g).cuda()
    delta = rnd(torch.randn(T, hid, generator=g)).to(tdt).cuda()
    r2 = res.clone()
    n = block.mixer_norm.forward(r2, delta, ctx)
    want_res = f64(res) + f64(delta)
    assert rel_err(f64(r2), want_res) < 1e-6
    assert rel_err(f64(n), plain.rms_norm(want_res, w[p + "input_layernorm.weight"], pm.eps)) < TOL[dtype]

    # position encoding: the table is cos/sin of position * frequency, rescaled as configured
    enc = block.mixer.position
    inv = plain.rope_inv_freq(enc.rotary_dim, cfg["rope_theta"], cfg.get("rope_scaling"))
    assert np.allclose(enc.inv_freq, inv.numpy(), rtol=1e-12)
    pos = torch.arange(enc.max_positions, dtype=torch.float64)[:, None] * inv[None]
    assert rel_err(f64(enc.cos_sin[..., 0]), torch.cos(pos)) < 1e-6 and rel_err(f64(enc.cos_sin[..., 1]), torch.sin(pos)) < 1e-6

    # feed-forward
    x = rnd(torch.randn(T, hid, generator=g)).to(tdt).cuda()
    y = block.feed_forward.forward(x, ctx)
    y = y.sum(0) if y.dim() == 3 else y
    hmid = plain.swiglu(plain.linear(f64(x), w[p + "mlp.gate_proj.weight"]), plain.linear(f64(x), w[p + "mlp.up_proj.weight"]))
    assert rel_err(f64(y), plain.linear(hmid, w[p + "mlp.down_proj.weight"])) < TOL[dtype]

    # attention mixer on top of what the cache holds for unit 1: the new rows' outputs equal the
    # plain attention over [keys of the old tokens as the engine computed them] + [new keys]
    old_hidden = []                                                       # layer-1 inputs of the cached tokens
    for b in range(len(lens)):
        if pos0[b]:
            xs = w["model.embed_tokens.weight"][torch.as_tensor(olds[b])]
            kv = {}
            xs = pm.block(0, xs, torch.arange(pos0[b]), kv, 0, True)
            old_hidden.append(plain.rms_norm(xs, w[p + "input_layernorm.weight"], pm.eps))
        else:
            old_hidden.append(torch.zeros(0, hid, dtype=torch.float64))
    a = block.mixer.forward(x, ctx, 1, True)
    a = a.sum(0) if a.dim() == 3 else a
    H, G, hd = pm.H, pm.G, pm.hd
    row, want = 0, []
    for b, nb in enumerate(lens):
        xn = torch.cat([old_hidden[b], f64(x[row:row + nb])])
        positions = torch.arange(pos0[b] + nb)
        q = plain.apply_rope(plain.linear(xn, w[p + "self_attn.q_proj.weight"]).view(-1, H, hd), positions, pm.inv_freq, pm.pairing)
        k = plain.apply_rope(plain.linear(xn, w[p + "self_attn.k_proj.weight"]).view(-1, G, hd), positions, pm.inv_freq, pm.pairing)
        v = plain.linear(xn, w[p + "self_attn.v_proj.weight"]).view(-1, G, hd)
        o = plain.attention(q[pos0[b]:], k, v, positions[pos0[b]:], positions, pm.window).reshape(nb, H * hd)
        want.append(plain.linear(o, w[p + "self_attn.o_proj.weight"]))
        row += nb
    assert rel_err(f64(a), torch.cat(want)) < TOL[dtype]

    # final norm on chosen rows + head
    rows = torch.tensor([T - 1, 0, 5], dtype=torch.int32).cuda()
    nf = eng.model.final_norm.forward(res.clone(), None, ctx, rows=rows)
    lg = eng.model.head.forward(nf, ctx)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    want = plain.linear(plain.rms_norm(f64(res)[[T - 1, 0, 5]], w["model.norm.weight"], pm.eps), head)
    assert lg.dtype == torch.float32 and rel_err(f64(lg), want) < TOL[dtype]


# --------------------------------------------------------------------------- a toy mixer with state
def register_toy():
    """A causal running mean: y_t = mean(x_0..x_t) W^T. Its per-sequence state (the running sum
    and the count) has a fixed size, unlike keys and values; it needs no cache pages."""
    from scriptling_llm_lib_b200.cache import StateNeed
    from scriptling_llm_lib_b200.config import ConfigError, register_architecture
    from scriptling_llm_lib_b200.engine.layout import ModelLayout, sequential_schedule
    from scriptling_llm_lib_b200.parts import MIXERS, Linear, Mixer, PartSpec, linear_head, pre_norm_layer, token_embedding

    class RunningMean(Mixer):
        def __init__(self, hidden, w_name):
            self.hidden = hidden
            self.proj = Linear([w_name], [hidden], hidden)

        def tensor_specs(self):
            return self.proj.tensor_specs()

        def bind(self, tensors, dtype, device):
            self.proj.bind(tensors, dtype, device)

        def state_need(self):
            return StateNeed((self.hidden + 1,), torch.float32)         # running sum, count

        def forward(self, x, ctx, unit, writes):
            state = ctx.unit_state(unit)
            starts = ctx.seq_start.tolist()
            slots = ctx.slots.tolist()
            out = torch.empty_like(x, dtype=torch.float32)
            for b, slot in enumerate(slots):
                seg = x[starts[b]:starts[b + 1]].float()
                sums = state[slot, :-1] + torch.cumsum(seg, dim=0)
                counts = state[slot, -1] + torch.arange(1, seg.shape[0] + 1, device=x.device)
                out[starts[b]:starts[b + 1]] = sums / counts[:, None]
                state[slot, :-1] = sums[-1]
                state[slot, -1] = counts[-1]
            return self.proj.forward(out.to(x.dtype), ctx)

    MIXERS.register("running_mean", RunningMean, replace=True)

    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int
        vocab_size: int
        intermediate_size: int
        max_position_embeddings: int

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            try:
                return cls(raw["hidden_size"], raw["vocab_size"], raw["intermediate_size"], raw["max_position_embeddings"])
            except KeyError as e:
                raise ConfigError(f"{where}: required key {e} is missing") from None

        def to_json_dict(self):
            return {"architectures": ["ToyMeanForCausalLM"], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                    "intermediate_size": self.intermediate_size, "max_position_embeddings": self.max_position_embeddings}

    def layout(cfg):
        def norm(name):
            return PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=1e-5, weight_name=name))
        rotary = PartSpec("rotary", dict(head_dim=16, rotary_dim=16, theta=10000.0, scaling=None, pairing="half"))
        attn = PartSpec("attention", dict(hidden=cfg.hidden_size, n_heads=2, n_kv_heads=1, head_dim=16, position=rotary,
                                          q_name="l1.q", k_name="l1.k", v_name="l1.v", o_name="l1.o"))
        ffn = lambda i: PartSpec("swiglu", dict(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                                                gate_name=f"l{i}.gate", up_name=f"l{i}.up", down_name=f"l{i}.down"))
        layers = (pre_norm_layer(PartSpec("running_mean", dict(hidden=cfg.hidden_size, w_name="l0.mean")), ffn(0), norm("l0.n1"), norm("l0.n2")),
                  pre_norm_layer(attn, ffn(1), norm("l1.n1"), norm("l1.n2")))       # different mixers in different layers
        return ModelLayout(cfg.vocab_size, cfg.hidden_size, cfg.max_position_embeddings,
                           token_embedding(cfg.vocab_size, cfg.hidden_size, "embed"), layers, sequential_schedule(2), norm("final"),
                           linear_head(cfg.vocab_size, cfg.hidden_size, "head"))

    register_architecture("ToyMeanForCausalLM", ToyConfig, layout, replace=True)
    return ToyConfig, layout


def toy_plain_logits(w, ids, hidden):
    """The toy model in plain float64, whole sequence."""
    x = w["embed"][torch.as_tensor(ids)]
    S = len(ids)
    pos = torch.arange(S)
    n = plain.rms_norm(x, w["l0.n1"], 1e-5)
    mean = torch.cumsum(n, 0) / torch.arange(1, S + 1, dtype=torch.float64)[:, None]
    x = x + plain.linear(mean, w["l0.mean"])
    n = plain.rms_norm(x, w["l0.n2"], 1e-5)
    x = x + plain.linear(plain.swiglu(plain.linear(n, w["l0.gate"]), plain.linear(n, w["l0.up"])), w["l0.down"])
    n = plain.rms_norm(x, w["l1.n1"], 1e-5)
    inv = plain.rope_inv_freq(16, 10000.0)
    q = plain.apply_rope(plain.linear(n, w["l1.q"]).view(S, 2, 16), pos, inv, "half")
    k = plain.apply_rope(plain.linear(n, w["l1.k"]).view(S, 1, 16), pos, inv, "half")
    v = plain.linear(n, w["l1.v"]).view(S, 1, 16)
    x = x + plain.linear(plain.attention(q, k, v, pos, pos).reshape(S, 32), w["l1.o"])
    n = plain.rms_norm(x, w["l1.n2"], 1e-5)
    x = x + plain.linear(plain.swiglu(plain.linear(n, w["l1.gate"]), plain.linear(n, w["l1.up"])), w["l1.down"])
    return plain.linear(plain.rms_norm(x, w["final"], 1e-5), w["head"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    from scriptling_llm_lib_b200.weights import write_random_model
    ToyConfig, layout = register_toy()
    cfg = ToyConfig(hidden_size=40, vocab_size=97, intermediate_size=72, max_position_embeddings=256)
    d = write_random_model(cfg, DecoderModel(layout(cfg)).tensor_specs(), 3, tmp_path / "toy")
    eng = Engine.from_folder(d, dtype, max_tokens=1024, max_seqs=3)
    assert not eng.use_graphs                                           # the toy mixer reads the host: no replay
    assert list(eng.cache.state) == [0] and eng.cache.state[0].shape == (3 + 1, 41)
    assert len(eng.cache.groups) == 1 and eng.cache.groups[0].units == [1]       # only the attention layer has pages
    w = plain.read_safetensors(d / "model.safetensors")
    reqs = [random_ids(n, 97, 500 + n) for n in (50, 7, 90, 33)]
    want = [toy_plain_logits(w, r, 40) for r in reqs]
    tol = TOL[dtype]
    for r, wl in zip(reqs, want):                                       # whole
        s = eng.open()
        assert rel_err(f64(eng.step([StepEntry(s, r, list(range(len(r))))])), wl) < tol
        s.close()
    # a batch of unequal prompts, then token by token; the fourth request reuses the slot (and the
    # state, which must start at zero again) of the first to end
    seqs = [eng.open() for _ in range(3)]
    plens = [20, 7, 1]
    got = {i: [] for i in range(4)}
    out = eng.step([StepEntry(s, reqs[i][:plens[i]], list(range(plens[i]))) for i, s in enumerate(seqs)])
    off = 0
    for i in range(3):
        got[i].append(f64(out[off:off + plens[i]]))
        off += plens[i]
    live = {0: seqs[0], 2: seqs[2]}
    seqs[1].close()                                                     # request 1 was whole in its prompt
    pos = {0: 20, 2: 1}
    started4 = False
    while live:
        if not started4 and len(live) < 3:
            s4 = eng.open()
            assert s4.slot == seqs[1].slot
            got[3].append(f64(eng.step([StepEntry(s4, reqs[3][:10], list(range(10)))])))
            live[3], pos[3], started4 = s4, 10, True
        order = sorted(live)
        out = eng.step([StepEntry(live[i], [reqs[i][pos[i]]], [0]) for i in order])
        for j, i in enumerate(order):
            got[i].append(f64(out[j:j + 1]))
            pos[i] += 1
            if pos[i] == len(reqs[i]):
                live.pop(i).close()
    for i in range(4):
        assert rel_err(torch.cat(got[i]), want[i]) < tol, f"request {i}"
    assert eng.cache.slots.n_free == 3


# --------------------------------------------------------------------------- the schedule is data
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_names_a_layer_twice_and_shares_a_cache(tmp_path, dtype):
    from scriptling_llm_lib_b200.config import LlamaConfig, register_architecture
    from scriptling_llm_lib_b200.engine.layout import ScheduleEntry
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    from scriptling_llm_lib_b200.models.llama import llama_layout
    import dataclasses
    # layer 0, layer 1, layer 0 again (a cache unit of its own), layer 1 reading the unit it wrote before
    order = (ScheduleEntry(0, 0, True), ScheduleEntry(1, 1, True), ScheduleEntry(0, 2, True), ScheduleEntry(1, 1, False))

    def looped(cfg):
        return dataclasses.replace(llama_layout(cfg), schedule=order)
    register_architecture("LoopedLlamaForCausalLM", LlamaConfig, looped, replace=True)
    raw = dict(TINY["A"][0], architectures=["LoopedLlamaForCausalLM"])
    d = make_model_dir(tmp_path / "looped", raw, 4)
    pm = plain_model(d, schedule=[(e.layer, e.cache_unit, e.writes_cache) for e in order])
    eng = Engine.from_folder(d, dtype, max_tokens=512)
    assert sorted(eng.cache.group_of_unit) == [0, 1, 2]
    ids = random_ids(90, 256, 9)
    want = pm.logits(ids)
    assert rel_err(want, plain_model(d).logits(ids)) > 1e-3              # the order matters
    s = eng.open()
    rows = [f64(eng.step([StepEntry(s, ids[:50], list(range(50)))]))]
    for t in ids[50:]:
        rows.append(f64(eng.step([StepEntry(s, [t], [0])])))
    s.close()
    assert rel_err(torch.cat(rows), want) < TOL[dtype]


# --------------------------------------------------------------------------- a routed feed-forward and another position encoding
def register_routed_toy():
    """Two more parts defined here and registered without a change to the library: a feed-forward
    that sends each token to the one expert (of three dense SiLU-gated ones) its router scores
    highest, weighted by that score's sigmoid; and a position encoding that rotates by the angle
    f_i * log(1 + position) instead of f_i * position (its own table, the library's kernels)."""
    from scriptling_llm_lib_b200.config import ConfigError, register_architecture
    from scriptling_llm_lib_b200.engine.layout import ModelLayout, sequential_schedule
    from scriptling_llm_lib_b200.parts import (FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, Linear, PartSpec, PositionEncoding,
                                               linear_head, pre_norm_layer, token_embedding)
    from scriptling_llm_lib_b200.parts.feedforward import SwiGLU

    class TopOneExperts(FeedForward):
        graph_safe = False                       # the routing decision is read on the host

        def __init__(self, hidden, intermediate, n_experts, prefix):
            self.hidden = hidden
            self.router = Linear([prefix + "router"], [n_experts], hidden)
            self.experts = [SwiGLU(hidden, intermediate, f"{prefix}e{e}.gate", f"{prefix}e{e}.up", f"{prefix}e{e}.down")
                            for e in range(n_experts)]

        def tensor_specs(self):
            return self.router.tensor_specs() + [s for e in self.experts for s in e.tensor_specs()]

        def bind(self, tensors, dtype, device):
            self.router.bind(tensors, dtype, device)
            for e in self.experts:
                e.bind(tensors, dtype, device)

        def forward(self, x, ctx):
            scores = self.router.forward(x, ctx, out_dtype=torch.float32)          # router logits in 32-bit
            choice = scores.argmax(dim=1)
            gate = torch.sigmoid(scores.gather(1, choice[:, None]))
            out = torch.zeros((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
            for e, expert in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    y = expert.forward(x[rows].contiguous(), ctx)
                    y = y.float().sum(0) if y.dim() == 3 else y.float()
                    out[rows] = y * gate[rows]
            return out.to(x.dtype)

    class LogRotary(PositionEncoding):
        def __init__(self, head_dim, theta):
            self.head_dim, self.theta = head_dim, theta
            self.cos_sin = None

        def prepare(self, max_positions, device):
            inv = 1.0 / np.power(self.theta, 2.0 * np.arange(self.head_dim // 2, dtype=np.float64) / self.head_dim)
            ang = np.log1p(np.arange(max_positions, dtype=np.float64))[:, None] * inv[None, :]
            self.cos_sin = torch.from_numpy(np.stack([np.cos(ang), np.sin(ang)], -1).astype(np.float32)).to(device)

        def rotation(self):                      # a rotation by a table of its own: the library's kernels do the rest
            return self.cos_sin, self.head_dim, False

    FEED_FORWARDS.register("top_one_experts", TopOneExperts, replace=True)
    POSITION_ENCODINGS.register("log_rotary", LogRotary, replace=True)

    @dataclass(frozen=True)
    class RoutedConfig:
        hidden_size: int
        vocab_size: int
        intermediate_size: int
        max_position_embeddings: int

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            try:
                return cls(raw["hidden_size"], raw["vocab_size"], raw["intermediate_size"], raw["max_position_embeddings"])
            except KeyError as e:
                raise ConfigError(f"{where}: required key {e} is missing") from None

        def to_json_dict(self):
            return {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                    "intermediate_size": self.intermediate_size, "max_position_embeddings": self.max_position_embeddings}

    def layout(cfg):
        def norm(name):
            return PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=1e-6, weight_name=name))
        pos = PartSpec("log_rotary", dict(head_dim=32, theta=100.0))
        attn = lambda i: PartSpec("attention", dict(hidden=cfg.hidden_size, n_heads=3, n_kv_heads=1, head_dim=32, position=pos,
                                                    q_name=f"l{i}.q", k_name=f"l{i}.k", v_name=f"l{i}.v", o_name=f"l{i}.o"))
        dense = PartSpec("swiglu", dict(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                                        gate_name="l0.gate", up_name="l0.up", down_name="l0.down"))
        routed = PartSpec("top_one_experts", dict(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size, n_experts=3, prefix="l1."))
        layers = (pre_norm_layer(attn(0), dense, norm("l0.n1"), norm("l0.n2")),
                  pre_norm_layer(attn(1), routed, norm("l1.n1"), norm("l1.n2")))      # different feed-forwards in different layers
        return ModelLayout(cfg.vocab_size, cfg.hidden_size, cfg.max_position_embeddings,
                           token_embedding(cfg.vocab_size, cfg.hidden_size, "embed"), layers, sequential_schedule(2), norm("final"),
                           linear_head(cfg.vocab_size, cfg.hidden_size, "head"))

    register_architecture("ToyRoutedForCausalLM", RoutedConfig, layout, replace=True)
    return RoutedConfig, layout


def routed_plain_logits(w, ids, act_round):
    """The routed toy model in plain float64, whole sequence; `act_round` rounds where the engine's
    activations are stored (identity in 32-bit), so that a near-tie between two experts' scores is
    decided on the same numbers."""
    S = len(ids)
    pos = torch.arange(S)
    logpos = torch.log1p(pos.to(torch.float64))
    inv = plain.rope_inv_freq(32, 100.0)
    x = w["embed"][torch.as_tensor(ids)]
    margins = []
    for i in range(2):
        n = act_round(plain.rms_norm(x, w[f"l{i}.n1"], 1e-6))
        q = plain.apply_rope(act_round(plain.linear(n, w[f"l{i}.q"])).view(S, 3, 32), logpos, inv, "half")
        k = plain.apply_rope(act_round(plain.linear(n, w[f"l{i}.k"])).view(S, 1, 32), logpos, inv, "half")
        v = act_round(plain.linear(n, w[f"l{i}.v"])).view(S, 1, 32)
        a = act_round(plain.attention(act_round(q), act_round(k), v, pos, pos).reshape(S, 96))
        x = x + plain.linear(a, w[f"l{i}.o"])
        n = act_round(plain.rms_norm(x, w[f"l{i}.n2"], 1e-6))
        if i == 0:
            h = act_round(plain.swiglu(plain.linear(n, w["l0.gate"]), plain.linear(n, w["l0.up"])))
            x = x + plain.linear(h, w["l0.down"])
        else:
            scores = plain.linear(n, w["l1.router"])
            top2 = scores.topk(2, dim=1).values
            margins.append((top2[:, 0] - top2[:, 1]).min())
            choice = scores.argmax(dim=1)
            y = torch.zeros_like(x)
            for e in range(3):
                rows = (choice == e).nonzero().flatten()
                h = act_round(plain.swiglu(plain.linear(n[rows], w[f"l1.e{e}.gate"]), plain.linear(n[rows], w[f"l1.e{e}.up"])))
                y[rows] = plain.linear(h, w[f"l1.e{e}.down"]) * torch.sigmoid(scores[rows, e])[:, None]
            x = x + y
    return plain.linear(plain.rms_norm(x, w["final"], 1e-6), w["head"]), min(margins)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path, dtype):
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    from scriptling_llm_lib_b200.weights import write_random_model
    RoutedConfig, layout = register_routed_toy()
    cfg = RoutedConfig(hidden_size=48, vocab_size=101, intermediate_size=40, max_position_embeddings=256)
    d = write_random_model(cfg, DecoderModel(layout(cfg)).tensor_specs(), 11, tmp_path / "routed")
    from scriptling_llm_lib_b200.weights import write_safetensors
    w = plain.read_safetensors(d / "model.safetensors")
    w["l1.router"] = w["l1.router"] * 40.0                          # routing decisions that do not hang on rounding
    write_safetensors(d / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    eng = Engine.from_folder(d, dtype, max_tokens=1024, max_seqs=3)
    assert not eng.use_graphs                                       # the routed feed-forward reads the host: no replay
    w = plain.read_safetensors(d / "model.safetensors")
    act_round = (lambda t: t) if dtype == "float32" else (lambda t: t.to(torch.bfloat16).to(torch.float64))
    reqs = [random_ids(n, 101, 730 + n) for n in (60, 9, 35)]           # seeds with routing margins above 0.06
    want, margins = zip(*[routed_plain_logits(w, r, act_round) for r in reqs])
    tol = TOL[dtype]
    # whole; then a batch of unequal prompts followed by single tokens
    for r, wl in zip(reqs, want):
        s = eng.open()
        assert rel_err(f64(eng.step([StepEntry(s, r, list(range(len(r))))])), wl) < tol
        s.close()
    seqs = [eng.open() for _ in reqs]
    plens = [30, 9, 1]
    got = {i: [] for i in range(3)}
    out = eng.step([StepEntry(s, reqs[i][:plens[i]], list(range(plens[i]))) for i, s in enumerate(seqs)])
    off = 0
    for i in range(3):
        got[i].append(f64(out[off:off + plens[i]]))
        off += plens[i]
    pos = dict(enumerate(plens))
    live = {i: s for i, s in enumerate(seqs) if pos[i] < len(reqs[i])}
    while live:
        order = sorted(live)
        out = eng.step([StepEntry(live[i], [reqs[i][pos[i]]], [0]) for i in order])
        for j, i in enumerate(order):
            got[i].append(f64(out[j:j + 1]))
            pos[i] += 1
            if pos[i] == len(reqs[i]):
                live.pop(i).close()
    for i in range(3):
        assert rel_err(torch.cat(got[i]), want[i]) < tol, f"request {i}"
    assert min(margins) > 0.05                                       # no routing decision hung on rounding


# --------------------------------------------------------------------------- another architecture's surroundings
def register_capped_toy():
    """What another architecture could bring without a change to the library, all defined here: an
    embedding scaled by sqrt(hidden), a head whose logits are capped (cap * tanh(logit / cap)) and
    that is tied to the embedding, a block of one mixer and no feed-forward ("mixer_only"), a layer
    whose attention has no position encoding at all, and a position encoding that is no rotation
    (it adds position * slope to the first dimension of every query and key head, in place)."""
    import math
    from scriptling_llm_lib_b200.config import ConfigError, register_architecture
    from scriptling_llm_lib_b200.engine.layout import ModelLayout, sequential_schedule
    from scriptling_llm_lib_b200.parts import (ARRANGEMENTS, EMBEDDINGS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, LayerSpec,
                                               OutputHead, PartSpec, PositionEncoding, TokenEmbedding, pre_norm_layer)

    class ScaledEmbedding(TokenEmbedding):
        def forward(self, ids, ctx):
            return super().forward(ids, ctx) * math.sqrt(self.width)

    class CappedHead(OutputHead):
        def __init__(self, cap, **kw):
            super().__init__(**kw)
            self.cap = cap

        def forward(self, normed, ctx):
            return self.cap * torch.tanh(super().forward(normed, ctx) / self.cap)

    class MixerOnlyBlock(Block):
        """x += mixer(norm(x)); nothing else."""

        def __init__(self, spec):
            self.norm = NORMS.build(spec.parts["norm"])
            self.mixer = MIXERS.build(spec.parts["mixer"])

        def parts(self):
            return [self.norm, self.mixer]

        def forward(self, residual, delta, ctx, unit, writes):
            return self.mixer.forward(self.norm.forward(residual, delta, ctx), ctx, unit, writes)

    class FirstDimRamp(PositionEncoding):
        graph_safe = True

        def __init__(self, slope):
            self.slope = slope

        def transform(self, qkv, ctx, n_heads, n_kv_heads, head_dim):
            ramp = (ctx.tok_pos.to(torch.float32) * self.slope).to(qkv.dtype)
            cols = torch.arange(n_heads + n_kv_heads, device=qkv.device) * head_dim
            qkv[:, cols] = (qkv[:, cols].float() + ramp.float()[:, None]).to(qkv.dtype)

    EMBEDDINGS.register("scaled_embedding", ScaledEmbedding, replace=True)
    HEADS.register("capped_head", CappedHead, replace=True)
    ARRANGEMENTS.register("mixer_only", MixerOnlyBlock, replace=True)
    POSITION_ENCODINGS.register("first_dim_ramp", FirstDimRamp, replace=True)

    @dataclass(frozen=True)
    class CappedConfig:
        hidden_size: int
        vocab_size: int
        intermediate_size: int
        max_position_embeddings: int

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            try:
                return cls(raw["hidden_size"], raw["vocab_size"], raw["intermediate_size"], raw["max_position_embeddings"])
            except KeyError as e:
                raise ConfigError(f"{where}: required key {e} is missing") from None

        def to_json_dict(self):
            return {"architectures": ["ToyCappedForCausalLM"], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                    "intermediate_size": self.intermediate_size, "max_position_embeddings": self.max_position_embeddings}

    def layout(cfg):
        def norm(name):
            return PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=1e-5, weight_name=name))
        attn = lambda i, pos: PartSpec("attention", dict(hidden=cfg.hidden_size, n_heads=4, n_kv_heads=2, head_dim=16, position=pos,
                                                         q_name=f"l{i}.q", k_name=f"l{i}.k", v_name=f"l{i}.v", o_name=f"l{i}.o"))
        ffn = PartSpec("swiglu", dict(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                                      gate_name="l1.gate", up_name="l1.up", down_name="l1.down"))
        layers = (LayerSpec("mixer_only", dict(norm=norm("l0.n"), mixer=attn(0, None))),                   # no positions, no feed-forward
                  pre_norm_layer(attn(1, PartSpec("first_dim_ramp", dict(slope=0.05))), ffn, norm("l1.n1"), norm("l1.n2")))
        return ModelLayout(cfg.vocab_size, cfg.hidden_size, cfg.max_position_embeddings,
                           PartSpec("scaled_embedding", dict(vocab=cfg.vocab_size, width=cfg.hidden_size, name="embed")), layers,
                           sequential_schedule(2), norm("final"),
                           PartSpec("capped_head", dict(cap=3.0, vocab=cfg.vocab_size, width=cfg.hidden_size, weight_name="embed", tied=True)))

    register_architecture("ToyCappedForCausalLM", CappedConfig, layout, replace=True)
    return CappedConfig, layout


def capped_plain_logits(w, ids, hidden, act_round):
    S = len(ids)
    pos = torch.arange(S)
    x = w["embed"][torch.as_tensor(ids)] * (hidden ** 0.5)

    def attn(i, n, ramp):
        q = act_round(plain.linear(n, w[f"l{i}.q"])).view(S, 4, 16).clone()
        k = act_round(plain.linear(n, w[f"l{i}.k"])).view(S, 2, 16).clone()
        v = act_round(plain.linear(n, w[f"l{i}.v"])).view(S, 2, 16)
        if ramp:
            r = act_round((pos.to(torch.float32) * 0.05).to(torch.float64))
            q[:, :, 0] = act_round(q[:, :, 0] + r[:, None])
            k[:, :, 0] = act_round(k[:, :, 0] + r[:, None])
        return plain.linear(act_round(plain.attention(q, k, v, pos, pos).reshape(S, 64)), w[f"l{i}.o"])

    x = x + attn(0, act_round(plain.rms_norm(x, w["l0.n"], 1e-5)), False)
    x = x + attn(1, act_round(plain.rms_norm(x, w["l1.n1"], 1e-5)), True)
    n = act_round(plain.rms_norm(x, w["l1.n2"], 1e-5))
    x = x + plain.linear(act_round(plain.swiglu(plain.linear(n, w["l1.gate"]), plain.linear(n, w["l1.up"]))), w["l1.down"])
    return 3.0 * torch.tanh(plain.linear(act_round(plain.rms_norm(x, w["final"], 1e-5)), w["embed"]) / 3.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_its_own_embedding_head_block_and_positions(tmp_path, dtype):
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    from scriptling_llm_lib_b200.weights import write_random_model
    CappedConfig, layout = register_capped_toy()
    cfg = CappedConfig(hidden_size=48, vocab_size=83, intermediate_size=56, max_position_embeddings=256)
    model = DecoderModel(layout(cfg))
    names = [s.name for s in model.tensor_specs()]
    assert names.count("embed") == 1 and "head" not in names           # the tied head asks for nothing of its own
    assert model.elements_read_per_step() == sum(int(np.prod(s.shape)) for s in model.tensor_specs())   # table counted once, as the head
    d = write_random_model(cfg, model.tensor_specs(), 5, tmp_path / "capped")
    eng = Engine.from_folder(d, dtype, max_tokens=1024, max_seqs=3)
    assert eng.use_graphs and len(eng.cache.groups) == 1 and eng.cache.groups[0].units == [0, 1]
    w = plain.read_safetensors(d / "model.safetensors")
    act_round = (lambda t: t) if dtype == "float32" else (lambda t: t.to(torch.float32).to(torch.bfloat16).to(torch.float64))
    reqs = [random_ids(n, 83, 830 + n) for n in (70, 9, 33)]
    want = [capped_plain_logits(w, r, 48, act_round) for r in reqs]
    tol = TOL[dtype]
    for r, wl in zip(reqs, want):                                       # whole
        s = eng.open()
        assert rel_err(f64(eng.step([StepEntry(s, r, list(range(len(r))))])), wl) < tol
        s.close()
    seqs = [eng.open() for _ in reqs]                                   # unequal prompts, then one by one (captured steps)
    plens = [40, 9, 1]
    got = {i: [] for i in range(3)}
    out = eng.step([StepEntry(s, reqs[i][:plens[i]], list(range(plens[i]))) for i, s in enumerate(seqs)])
    off = 0
    for i in range(3):
        got[i].append(f64(out[off:off + plens[i]]))
        off += plens[i]
    pos = dict(enumerate(plens))
    live = {i: s for i, s in enumerate(seqs) if pos[i] < len(reqs[i])}
    while live:
        order = sorted(live)
        out = eng.step([StepEntry(live[i], [reqs[i][pos[i]]], [0]) for i in order])
        for j, i in enumerate(order):
            got[i].append(f64(out[j:j + 1]))
            pos[i] += 1
            if pos[i] == len(reqs[i]):
                live.pop(i).close()
    for i in range(3):
        assert rel_err(torch.cat(got[i]), want[i]) < tol, f"request {i}"
    assert float(torch.cat(got[0]).abs().max()) <= 3.0                  # the cap holds
