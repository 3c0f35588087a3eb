"""The plain implementation itself: hand-computable cases of the kind the reference's own op tests
use (float32_ops_test.go:16-118), invariants, and the samplers (no GPU)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as plain
from helpers import TINY, make_model_dir, plain_model, random_ids, rel_err


def test_rms_norm_by_hand():
    x = torch.tensor([[0.5, -0.3, 0.8]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 0.5], dtype=torch.float64)
    inv = 1.0 / math.sqrt((0.25 + 0.09 + 0.64) / 3 + 1e-5)
    assert torch.allclose(plain.rms_norm(x, w, 1e-5), torch.tensor([[0.5 * inv, -0.6 * inv, 0.4 * inv]], dtype=torch.float64))


def test_rope_by_hand_both_pairings_and_partial_width():
    f = plain.rope_inv_freq(4, 10000.0)
    assert torch.allclose(f, torch.tensor([1.0, 0.01], dtype=torch.float64))
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 9.0, 9.5]]], dtype=torch.float64)          # hd 6, rotary width 4
    pos = torch.tensor([5])
    c0, s0, c1, s1 = math.cos(5.0), math.sin(5.0), math.cos(0.05), math.sin(0.05)
    inter = plain.apply_rope(x, pos, f, "interleaved")[0, 0]
    assert torch.allclose(inter, torch.tensor([1 * c0 - 2 * s0, 1 * s0 + 2 * c0, 3 * c1 - 4 * s1, 3 * s1 + 4 * c1, 9.0, 9.5],
                                              dtype=torch.float64))
    half = plain.apply_rope(x, pos, f, "half")[0, 0]
    assert torch.allclose(half, torch.tensor([1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 1 * s0 + 3 * c0, 2 * s1 + 4 * c1, 9.0, 9.5],
                                             dtype=torch.float64))
    assert torch.equal(plain.apply_rope(x, torch.tensor([0]), f, "half"), x)            # position 0 rotates nothing


def test_llama3_scaling_leaves_fast_frequencies_and_divides_slow_ones():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    f, g = plain.rope_inv_freq(16, 1e5), plain.rope_inv_freq(16, 1e5, sc)
    wl = 2 * math.pi / f
    assert torch.equal(g[wl < 16], f[wl < 16]) and torch.allclose(g[wl > 64], f[wl > 64] / 8)
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and ((g[mid] < f[mid]) & (g[mid] > f[mid] / 8)).all()


def test_attention_by_hand_two_keys_causal_gqa_and_window():
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 2.0]]], dtype=torch.float64)                 # S=2, H=1, hd=2
    k = torch.tensor([[[1.0, 1.0]], [[3.0, -1.0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0, 10.0]], [[2.0, 20.0]]], dtype=torch.float64)
    pos = torch.arange(2)
    out = plain.attention(q, k, v, pos, pos)
    assert torch.allclose(out[0, 0], v[0, 0])                                           # row 0 sees key 0 only
    s = torch.tensor([2.0, -2.0], dtype=torch.float64) / math.sqrt(2.0)
    p = torch.softmax(s, 0)
    assert torch.allclose(out[1, 0], p[0] * v[0, 0] + p[1] * v[1, 0])
    assert torch.allclose(plain.attention(q, k, v, pos, pos, window=1)[1, 0], v[1, 0])  # window 1: own key only
    # grouped heads: query heads 0,1 read kv head 0; heads 2,3 read kv head 1
    g = torch.Generator().manual_seed(0)
    q4 = torch.randn(5, 4, 8, generator=g, dtype=torch.float64)
    k2, v2 = torch.randn(5, 2, 8, generator=g, dtype=torch.float64), torch.randn(5, 2, 8, generator=g, dtype=torch.float64)
    pos = torch.arange(5)
    full = plain.attention(q4, k2, v2, pos, pos)
    for h in range(4):
        one = plain.attention(q4[:, h:h + 1], k2[:, h // 2:h // 2 + 1], v2[:, h // 2:h // 2 + 1], pos, pos)
        assert torch.allclose(full[:, h], one[:, 0])


def test_swiglu_and_linear_by_hand():
    g, u = torch.tensor([0.0, 1.0, -2.0], dtype=torch.float64), torch.tensor([3.0, 2.0, 1.0], dtype=torch.float64)
    want = [0.0, 1.0 / (1 + math.exp(-1.0)) * 2.0, -2.0 / (1 + math.exp(2.0))]
    assert torch.allclose(plain.swiglu(g, u), torch.tensor(want, dtype=torch.float64))
    x = torch.tensor([[1.0, 2.0]], dtype=torch.float64)
    w = torch.tensor([[1.0, 0.0], [0.5, 0.5], [-1.0, 2.0]], dtype=torch.float64)      # [out, in]
    assert torch.equal(plain.linear(x, w), torch.tensor([[1.0, 1.5, 3.0]], dtype=torch.float64))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_model_is_causal_and_window_matters(tmp_path, name):
    raw, seed = TINY[name]
    m = plain_model(make_model_dir(tmp_path, raw, seed))
    ids = random_ids(60, raw["vocab_size"], 3)
    full = m.logits(ids)
    assert full.shape == (60, raw["vocab_size"]) and torch.isfinite(full).all()
    assert rel_err(m.logits(ids[:33]), full[:33]) < 1e-12                               # later tokens change nothing earlier
    other = list(ids)
    other[2] = (other[2] + 1) % raw["vocab_size"]
    changed = (m.logits(other) - full).abs().amax(dim=-1)
    assert float(changed[:2].max()) == 0.0 and float(changed[2]) > 0
    if name == "C":                                                                      # window 24, 2 layers: reach < 48
        assert float(changed[2 + 2 * 24:].max()) < 1e-12 and float(changed[10]) > 0
    else:
        assert float(changed[-1]) > 0


def test_philox_known_answers():
    assert plain.philox4x32([0, 0, 0, 0], [0, 0]) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert plain.philox4x32([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    us = [plain.uniform_for(3, i) for i in range(200)]
    assert all(0.0 <= u < 1.0 for u in us) and 0.35 < sum(us) / 200 < 0.65 and len(set(us)) == 200
    assert plain.uniform_for(3, 5) != plain.uniform_for(4, 5)


def test_samplers():
    lg = np.array([0.1, 2.0, 2.0, -1.0, 0.5])
    assert plain.sample(lg, "greedy") == 1                                              # first of equal maxima
    p = plain.softmax_t(lg, 0.7)
    assert abs(p.sum() - 1) < 1e-12 and p[1] == p[2] > p[4] > p[0] > p[3]
    assert plain.weighted_pick([0.2, 0.3, 0.5], 0.0) == 0 and plain.weighted_pick([0.2, 0.3, 0.5], 0.2) == 0
    assert plain.weighted_pick([0.2, 0.3, 0.5], 0.21) == 1 and plain.weighted_pick([0.2, 0.3, 0.5], 0.999) == 2
    assert plain.weighted_pick([0.2, 0.3, 0.4], 0.95) == 2                              # short sum: last index
    assert plain.sample(lg, "temperature", temperature=1.0, u=0.0) == 0
    assert {plain.sample(lg, "top_k", 1.0, top_k=2, u=u) for u in np.linspace(0, 0.999, 50)} == {1, 2}
    assert {plain.sample(lg, "top_k", 1.0, top_k=3, u=u) for u in np.linspace(0, 0.999, 200)} == {1, 2, 4}
    assert {plain.sample(lg, "top_p", 1.0, top_p=0.5, u=u) for u in np.linspace(0, 0.999, 50)} == {1, 2}
    assert {plain.sample(lg, "top_p", 1.0, top_p=1.0, u=u) for u in np.linspace(0, 0.9999, 2000)} == {0, 1, 2, 3, 4}
    pen = plain.apply_repeat_penalty([2.0, -2.0, 3.0, 1.0], [0, 1, 0, 9, -1], 2.0, 64)
    assert list(pen) == [1.0, -4.0, 3.0, 1.0]                                           # once per distinct token
    assert list(plain.apply_repeat_penalty([2.0, -2.0, 3.0], [0, 1, 2], 2.0, 1)) == [2.0, -2.0, 1.5]


def test_generate_semantics(tmp_path):
    raw, seed = TINY["A"]
    m = plain_model(make_model_dir(tmp_path, raw, seed))
    prompt = random_ids(9, 256, 1)
    out = plain.generate(m, prompt, 6)
    assert len(out) == 6
    assert plain.generate(m, prompt, 1) == out[:1]                                      # at least one token, counted
    stop_at = out[2]
    first = out.index(stop_at)
    assert plain.generate(m, prompt, 6, stop_ids=(stop_at,)) == out[:first + 1]         # stop token kept
    t1 = plain.generate(m, prompt, 8, "temperature", temperature=0.8, seed=5)
    assert t1 == plain.generate(m, prompt, 8, "temperature", temperature=0.8, seed=5)
    assert t1 != plain.generate(m, prompt, 8, "temperature", temperature=0.8, seed=6)
    assert plain.generate(m, prompt, 6, "temperature", temperature=0.0) == out          # T = 0 is greedy


def test_llama3_scaling_by_hand_and_the_librarys_table():
    """The reference has no frequency rescaling, so nothing of its pins this rule; three values
    worked out by hand do (theta 500000, 64 pairs, factor 8, low 1, high 4, original length 8192:
    pair 27 has a wavelength of 1594 < 8192/4 and stays; pair 35 has 8219 > 8192/1 and is divided
    by 8; pair 30 has 2948.3, in between, period count 8192/2948.3 = 2.77855, smooth =
    (2.77855 - 1)/(4 - 1) = 0.592849, scale = (1 - 0.592849)/8 + 0.592849 = 0.643743) and so does a
    second statement of the rule, the table builder of the library's rotary part."""
    from scriptling_llm_lib_b200.config.llama import RopeScaling
    from scriptling_llm_lib_b200.parts.rotary import inverse_frequencies
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
    f, g = plain.rope_inv_freq(128, 500000.0), plain.rope_inv_freq(128, 500000.0, sc)
    assert abs(2 * math.pi / f[30].item() - 2948.3026) < 1e-3
    assert g[27].item() == f[27].item() and abs(g[35].item() / f[35].item() - 0.125) < 1e-15
    assert abs(g[30].item() / f[30].item() - 0.6437431331) < 1e-9
    for scaling in (None, sc, dict(sc, factor=32.0), {"rope_type": "linear", "factor": 4.0}):
        for dim, theta in ((128, 500000.0), (64, 130000.0), (16, 10000.0)):
            lib = inverse_frequencies(dim, theta, RopeScaling(**scaling) if scaling else None)
            assert np.allclose(lib, plain.rope_inv_freq(dim, theta, scaling).numpy(), rtol=1e-13, atol=0)


def test_half_pairing_is_the_references_rotation_under_a_permutation_of_rows(tmp_path):
    """The reference rotates adjacent pairs (float32_ops.go:174-188); checkpoints of the family pair
    dimension i with i + width/2 instead. The two are one rotation seen through a permutation of the
    query and key projections' rows inside each head (pairs 0,1 | 2,3 | ... -> first halves, then second
    halves): a model with interleaved pairing and the same model with permuted rows and half pairing
    give the same logits, which ties the half pairing to the formula the reference does have. Scores
    are sums over a head's dimensions, so the order inside a head does not matter otherwise."""
    raw, seed = TINY["A"]                                                # interleaved, full rotary width
    assert raw["rope_pairing"] == "interleaved"
    cfg, w = plain.load_folder(make_model_dir(tmp_path, raw, seed))
    hd = cfg["head_dim"]
    perm_in_head = list(range(0, hd, 2)) + list(range(1, hd, 2))
    w2 = dict(w)
    for i in range(cfg["num_hidden_layers"]):
        for name, heads in (("q_proj", cfg["num_attention_heads"]), ("k_proj", cfg["num_key_value_heads"])):
            key = f"model.layers.{i}.self_attn.{name}.weight"
            rows = torch.tensor([h * hd + j for h in range(heads) for j in perm_in_head])
            w2[key] = w[key][rows]
    ids = random_ids(50, cfg["vocab_size"], 12)
    a = plain.PlainLlama(cfg, w).logits(ids)
    b = plain.PlainLlama(dict(cfg, rope_pairing="half"), w2).logits(ids)
    assert rel_err(b, a) < 1e-12
    assert rel_err(plain.PlainLlama(dict(cfg, rope_pairing="half"), w).logits(ids), a) > 1e-3    # without the permutation it is another model


def test_tied_head_is_the_embedding_matrix_as_stored(tmp_path):
    """With tie_word_embeddings the logits are the final norm times the embedding matrix itself
    (model_f32.go:147-162 falls back to it; its re-quantisation of that matrix to 8 bits is a storage
    choice of the reference's and is not reproduced): a tied model equals the untied model whose
    lm_head.weight is a copy of the embedding."""
    raw, seed = TINY["A"]
    cfg, w = plain.load_folder(make_model_dir(tmp_path, raw, seed))
    assert cfg["tie_word_embeddings"] and "lm_head.weight" not in w
    ids = random_ids(20, cfg["vocab_size"], 4)
    untied = plain.PlainLlama(dict(cfg, tie_word_embeddings=False), dict(w, **{"lm_head.weight": w["model.embed_tokens.weight"].clone()}))
    assert torch.equal(untied.logits(ids), plain.PlainLlama(cfg, w).logits(ids))
