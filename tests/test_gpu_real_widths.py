"""The SmolLM2-1.7B layer sizes (hidden 2048, 32 heads of 64, intermediate 8192, vocabulary 49152,
theta 130000, tied head) and a Llama-3 style shape (grouped queries, heads of 128, rescaled rotary
frequencies), each with two layers and random weights: the widths at which the tensor-core
kernels of the bfloat16 path and the tiled kernels of the 32-bit path are actually used, whole
prompt, then token by token, in a batch of unequal lengths, against the plain implementation."""
import pytest
import torch

from helpers import MEASURED, check_logits, make_model_dir, plain_model, plain_model_bf16, random_ids

pytestmark = pytest.mark.gpu

REAL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 49152, "rope_theta": 130000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 8192, "hidden_act": "silu",
}


# Llama-3 style: grouped queries (4 query heads per key/value head), heads of 128, rescaled rotary
# frequencies, a head of its own, a vocabulary that is no multiple of 128
GROUPED = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 1024,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 2816,
    "vocab_size": 32003, "rope_theta": 500000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 8192, "hidden_act": "silu",
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 256},
}


@pytest.fixture(scope="module", params=["mha64", "gqa128"])
def real_model(request, tmp_path_factory):
    raw = REAL if request.param == "mha64" else GROUPED
    d = make_model_dir(tmp_path_factory.mktemp("real"), raw, 7)
    pm, pm16 = plain_model(d), plain_model_bf16(d)
    reqs = [random_ids(n, raw["vocab_size"], 900 + n) for n in (300, 70, 1)]
    return d, reqs, [pm.logits(r) for r in reqs], [pm16.logits(r) for r in reqs]


def report(what):
    if MEASURED:
        print(f"\n[{what}] largest error against the rounding / the unrounded plain implementation: "
              f"{max(m[1] for m in MEASURED):.3g} / {max(m[2] for m in MEASURED):.3g}")
        MEASURED.clear()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_widths(real_model, dtype):
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    d, reqs, want, want16 = real_model
    eng = Engine.from_folder(d, dtype, max_tokens=1024)
    # whole, alone
    for i, r in enumerate(reqs):
        s = eng.open()
        got = eng.step([StepEntry(s, r, list(range(len(r))))]).cpu().double()
        s.close()
        check_logits(got, want[i], want16[i], dtype, f"request {i} whole")
    # the longest prompt in two portions, the second (200 rows: the two-SM product whose epilogue rotates
    # and fills the cache) onto 100 cached tokens; and in three, the last of 129 rows onto 171
    for cuts in ([100], [64, 171]):
        s = eng.open()
        edges = [0] + cuts + [len(reqs[0])]
        got = torch.cat([eng.step([StepEntry(s, reqs[0][a:b], list(range(b - a)))]) for a, b in zip(edges, edges[1:])]).cpu().double()
        s.close()
        check_logits(got, want[0], want16[0], dtype, f"request 0 in portions cut at {cuts}")
    # a batch of unequal prompts, then 12 tokens one by one
    seqs = [eng.open() for _ in reqs]
    heads = [max(1, len(r) - 12) for r in reqs]
    out = eng.step([StepEntry(s, r[:h], list(range(h))) for s, r, h in zip(seqs, reqs, heads)]).cpu().double()
    rows, off = [[] for _ in reqs], 0
    for i, h in enumerate(heads):
        rows[i].append(out[off:off + h])
        off += h
    pos = list(heads)
    while any(p < len(r) for p, r in zip(pos, reqs)):
        live = [i for i, r in enumerate(reqs) if pos[i] < len(r)]
        out = eng.step([StepEntry(seqs[i], [reqs[i][pos[i]]], [0]) for i in live]).cpu().double()
        for j, i in enumerate(live):
            rows[i].append(out[j:j + 1])
            pos[i] += 1
    for i in range(len(reqs)):
        check_logits(torch.cat(rows[i]), want[i], want16[i], dtype, f"request {i} in a batch, then one by one")
    assert int(eng.err_flag) == 0
    report(f"real widths {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", [20, 64, 100])
def test_many_sequences_decode_together(real_model, dtype, n):
    """Decode steps of 20, 64 and 100 rows (the few-rows tensor-core products up to 64 rows replayed as a
    graph, the one-SM product beyond; in 32-bit the 64- and 128-row register tiles): unequal short
    prompts in one step, then a few tokens each, every row against the plain implementation."""
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    d, _, _, _ = real_model
    pm, pm16 = plain_model(d), plain_model_bf16(d)
    V = pm.cfg["vocab_size"]
    n_dec = 6 if n == 20 else 3
    span = 38 if n == 20 else 9
    reqs = [random_ids(3 + (7 * i) % span + n_dec, V, 1200 + i) for i in range(n)]
    eng = Engine.from_folder(d, dtype, max_tokens=n * 64, max_seqs=n)
    seqs = [eng.open() for _ in reqs]
    heads = [len(r) - n_dec for r in reqs]
    out = eng.step([StepEntry(s, r[:h], [h - 1]) for s, r, h in zip(seqs, reqs, heads)]).cpu().double()
    rows = [[out[i:i + 1]] for i in range(n)]
    for t in range(n_dec):
        out = eng.step([StepEntry(s, [r[h + t]], [0]) for s, r, h in zip(seqs, reqs, heads)]).cpu().double()
        for i in range(n):
            rows[i].append(out[i:i + 1])
    for i, (r, h) in enumerate(zip(reqs, heads)):
        check_logits(torch.cat(rows[i]), pm.logits(r)[h - 1:], pm16.logits(r)[h - 1:], dtype, f"request {i} of {n}")
    assert int(eng.err_flag) == 0
    report(f"{n} rows {dtype}")


def test_norms_folded_into_the_decode_products(real_model, monkeypatch):
    """In a bfloat16 decode step of few rows the norms between two products have no kernel of their own
    (the product before adds to the residual stream and prepares, the product behind scales its rows).
    The same steps with every norm as a kernel give the same logits up to where bfloat16 rounds, and
    take three launches more for these two layers (the first norm of the first layer and the final
    norm are never folded)."""
    from scriptling_llm_lib_b200.csrc import bindings
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    from scriptling_llm_lib_b200.parts import block
    d, reqs, want, want16 = real_model
    eng = Engine.from_folder(d, "bfloat16", max_tokens=1024)
    eng.use_graphs = False                                   # count the launches of the steps themselves
    runs = {}
    for folded in (True, False):
        monkeypatch.setattr(block, "_NO_FOLD", not folded)
        seqs = [eng.open() for _ in reqs[:2]]
        eng.step([StepEntry(s, r[:40], []) for s, r in zip(seqs, reqs)])
        rows, n0 = [], bindings.LAUNCHES[0]
        for t in range(40, 46):
            rows.append(eng.step([StepEntry(s, [r[t]], [0]) for s, r in zip(seqs, reqs)]).cpu().double())
        runs[folded] = (torch.stack(rows), (bindings.LAUNCHES[0] - n0) // 6)
        for s in seqs:
            s.close()
    (a, n_a), (b, n_b) = runs[True], runs[False]
    assert n_b - n_a == 3
    for i in range(2):
        check_logits(a[:, i], want[i][40:46], want16[i][40:46], "bfloat16", f"request {i}, norms folded")
        check_logits(b[:, i], want[i][40:46], want16[i][40:46], "bfloat16", f"request {i}, norms as kernels")
    assert int(eng.err_flag) == 0
