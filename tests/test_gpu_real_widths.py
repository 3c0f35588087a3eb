"""The SmolLM2-1.7B layer sizes (hidden 2048, 32 heads of 64, intermediate 8192, vocabulary 49152,
theta 130000, tied head) and a Llama-3 style shape (grouped queries, heads of 128, rescaled rotary
frequencies), each with two layers and random weights: the widths at which the tensor-core
kernels of the bfloat16 path and the tiled kernels of the 32-bit path are actually used, whole
prompt, then token by token, in a batch of unequal lengths, against the plain implementation."""
import pytest
import torch

from helpers import TOL_BF16, TOL_F32, make_model_dir, plain_model, random_ids, rel_err

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
    pm = plain_model(d)
    reqs = [random_ids(n, raw["vocab_size"], 900 + n) for n in (300, 70, 1)]
    return d, reqs, [pm.logits(r) for r in reqs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_widths(real_model, dtype):
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    d, reqs, want = real_model
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    eng = Engine.from_folder(d, dtype, max_tokens=1024)
    # whole, alone
    for r, w in zip(reqs, want):
        s = eng.open()
        got = eng.step([StepEntry(s, r, list(range(len(r))))]).cpu().double()
        s.close()
        assert rel_err(got, w) < tol
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
    for i, w in enumerate(want):
        assert rel_err(torch.cat(rows[i]), w) < tol, f"request {i}"
    assert int(eng.err_flag) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_twenty_sequences_decode_together(real_model, dtype):
    """A decode step of 20 rows (the few-rows tensor-core products, replayed as a graph): unequal short
    prompts in one step, then six tokens each, every row against the plain implementation."""
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    d, _, _ = real_model
    pm = plain_model(d)
    V = pm.cfg["vocab_size"]
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    reqs = [random_ids(3 + (7 * i) % 38 + 6, V, 1200 + i) for i in range(20)]
    want = [pm.logits(r) for r in reqs]
    eng = Engine.from_folder(d, dtype, max_tokens=20 * 64, max_seqs=20)
    seqs = [eng.open() for _ in reqs]
    heads = [len(r) - 6 for r in reqs]
    out = eng.step([StepEntry(s, r[:h], [h - 1]) for s, r, h in zip(seqs, reqs, heads)]).cpu().double()
    rows = [[out[i:i + 1]] for i in range(20)]
    for t in range(6):
        out = eng.step([StepEntry(s, [r[h + t]], [0]) for s, r, h in zip(seqs, reqs, heads)]).cpu().double()
        for i in range(20):
            rows[i].append(out[i:i + 1])
    for i, (w, h) in enumerate(zip(want, heads)):
        assert rel_err(torch.cat(rows[i]), w[h - 1:]) < tol, f"request {i}"
    assert int(eng.err_flag) == 0
