"""Generation on the GPU through the Python entry point and the command line: greedy and sampled
tokens against the plain implementation, unequal batches with stop tokens, batch after batch on
reused slots, long decoding, the first tokens of a sequence, stale cache contents."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_llama as plain
from helpers import MEASURED, TINY, TOL_BF16, check_logits, make_model_dir, plain_model, plain_model_bf16, random_ids

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(autouse=True)
def fresh_model_cache():
    from scriptling_llm_lib_b200 import llm
    llm.unload()
    yield
    llm.unload()


def near_maximum(model, prompt, out, tol):
    """Every generated token is a maximum of the plain logits on the generated path, within rounding."""
    for i, t in enumerate(out):
        lg = model.logits(list(prompt) + list(out[:i]))[-1]
        if float(lg.max() - lg[t]) > tol * float(lg.abs().max()):
            return False
    return True


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_greedy_through_the_entry_point(tmp_path, name):
    from scriptling_llm_lib_b200 import llm
    raw, seed = TINY[name]
    d = make_model_dir(tmp_path / "m", raw, seed)
    pm = plain_model(d)
    V = raw["vocab_size"]
    prompts = [random_ids(n, V, 10 + n) for n in (5, 17, 31, 1)]
    want = [plain.generate(pm, p, 12, stop_ids=()) for p in prompts]
    got = llm.generate(d, prompts, 12, "greedy", temperature=0.0, stop_ids=[], dtype="float32")
    assert got == want
    one = llm.generate(d, prompts[1], 12, "greedy", temperature=0.0, stop_ids=[], dtype="float32")
    assert one == want[1]                                                # alone == in the batch; a flat list in, a flat list out
    got16 = llm.generate(d, prompts, 12, "greedy", temperature=0.0, stop_ids=[], dtype="bfloat16")
    assert all(len(g) == 12 and near_maximum(pm, p, g, TOL_BF16) for p, g in zip(prompts, got16))


def test_stop_tokens_unequal_ends_and_batches_on_reused_slots(tmp_path):
    from scriptling_llm_lib_b200 import llm
    raw, seed = TINY["A"]
    d = make_model_dir(tmp_path / "m", raw, seed)
    pm = plain_model(d)
    prompts = [random_ids(n, 256, 30 + n) for n in (5, 17, 31, 9, 2, 40, 3)]
    # greedy on random weights soon repeats one token, so sample (seeded; request i draws from stream seed + i)
    kw = dict(strategy="temperature", temperature=1.0, repeat_penalty=0.0)
    free_run = [plain.generate(pm, p, 16, stop_ids=(), seed=3 + i, **kw) for i, p in enumerate(prompts)]

    def lengths(stop):   # a stop token cuts a run short and changes nothing before it
        return [next((i + 1 for i, t in enumerate(r) if t in stop), len(r)) for r in free_run]
    tokens = sorted({t for r in free_run for t in r})
    stops = max(([a, b] for a in tokens for b in tokens if a < b), key=lambda st: len(set(lengths(st))))
    want = [plain.generate(pm, p, 16, stop_ids=stops, seed=3 + i, **kw) for i, p in enumerate(prompts)]
    assert [len(w) for w in want] == lengths(stops) and len({len(w) for w in want}) > 2
    got, st = llm.generate(d, prompts, 16, kw["strategy"], temperature=1.0, repeat_penalty=0.0, seed=3, stop_ids=stops,
                           dtype="float32", max_batch=3, stats=True)
    assert got == want                                                   # three batches on three slots
    assert st["generated_tokens"] == [len(w) for w in want] and st["prompt_tokens"] == [len(p) for p in prompts]
    assert st["finish_reason"] == ["stop" if w[-1] in stops else "length" for w in want]
    eng, _ = llm.load(d, "float32")
    assert eng.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in eng.cache.groups)
    # greedy: config.json's eos id (7) is the default stop set; max_tokens counts the first token
    dflt = llm.generate(d, prompts[:2], 16, dtype="float32")
    assert dflt == [plain.generate(pm, p, 16, stop_ids=(7,)) for p in prompts[:2]]
    assert llm.generate(d, prompts[0], 1, dtype="float32") == plain.generate(pm, prompts[0], 1)


def test_sampling_strategies_match_the_plain_samplers_in_32_bit(tmp_path):
    from scriptling_llm_lib_b200 import llm
    raw, seed = TINY["B"]
    d = make_model_dir(tmp_path / "m", raw, seed)
    pm = plain_model(d)
    prompts = [random_ids(n, 384, 50 + n) for n in (1, 8, 40, 63)]
    for kw in [dict(strategy="temperature", temperature=0.8), dict(strategy="top_k", temperature=1.0, top_k=20),
               dict(strategy="top_p", temperature=0.9, top_p=0.8),
               dict(strategy="temperature", temperature=0.8, repeat_penalty=1.3, repeat_last_n=16)]:
        strategy = kw.pop("strategy")
        kw.setdefault("repeat_penalty", 0.0)
        got = llm.generate(d, prompts, 10, strategy, seed=11, stop_ids=[], dtype="float32", **kw)
        for i, p in enumerate(prompts):
            want = plain.generate(pm, p, 10, strategy, stop_ids=(), seed=11 + i, **kw)
            assert got[i] == want, f"{strategy} {kw} request {i}"
        alone = llm.generate(d, [prompts[2]], 10, strategy, seed=11, stop_ids=[], dtype="float32", **kw)
        again = llm.generate(d, prompts[:1] + [prompts[2]], 10, strategy, seed=11, stop_ids=[], dtype="float32", **kw)
        # a request's stream is (seed + its index in the call): alone, prompt 2 is request 0 and draws what
        # the plain implementation draws for seed 11 + 0
        assert alone[0] == plain.generate(pm, prompts[2], 10, strategy, stop_ids=(), seed=11, **kw)
        assert again[0] == got[0]                                        # same request index, same seed: same tokens
    a = llm.generate(d, prompts[3], 10, "temperature", temperature=0.8, seed=1, stop_ids=[], dtype="float32")
    b = llm.generate(d, prompts[3], 10, "temperature", temperature=0.8, seed=2, stop_ids=[], dtype="float32")
    assert a != b


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(tmp_path, dtype):
    """A prompt of one token (positions 0, 1, 2, ... all decoded), then a long run past several page
    boundaries; every step's logits against the plain implementation."""
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    raw = dict(TINY["B"][0], max_position_embeddings=512)
    d = make_model_dir(tmp_path / "m", raw, 1)
    ids = random_ids(300, 384, 77)
    want, want16 = plain_model(d).logits(ids), plain_model_bf16(d).logits(ids)
    eng = Engine.from_folder(d, dtype, max_tokens=1024)
    s, other = eng.open(), eng.open()
    eng.step([StepEntry(other, random_ids(130, 384, 78))])               # a neighbour in the cache
    rows = [eng.step([StepEntry(s, [t], [0])]).cpu().to(torch.float64) for t in ids]
    got = torch.cat(rows)
    check_logits(got[:8], want[:8], want16[:8], dtype, "the first tokens of a sequence")
    check_logits(got, want, want16, dtype, "300 tokens one by one")
    MEASURED.clear()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_the_width_of_a_captured_step(tmp_path, dtype):
    """A captured decode step is sized for a block table of 8, 16, 32, ... pages: a sequence that grows
    from 500 to 530 tokens leaves the step captured for 8 pages (512 tokens) for the one of 16, while
    a short neighbour decodes beside it; every step's logits against the plain implementation."""
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    raw = dict(TINY["D"][0], max_position_embeddings=2048, sliding_window=None)
    d = make_model_dir(tmp_path / "m", raw, 3)
    V = raw["vocab_size"]
    long_ids, short_ids = random_ids(530, V, 81), random_ids(40, V, 82)
    pm, pm16 = plain_model(d), plain_model_bf16(d)
    eng = Engine.from_folder(d, dtype, max_tokens=2048, max_seqs=4)
    a, b = eng.open(), eng.open()
    eng.step([StepEntry(a, long_ids[:500], []), StepEntry(b, short_ids[:10], [])])
    rows_a, rows_b = [], []
    for t in range(30):
        out = eng.step([StepEntry(a, [long_ids[500 + t]], [0]), StepEntry(b, [short_ids[10 + t]], [0])]).cpu().double()
        rows_a.append(out[0:1])
        rows_b.append(out[1:2])
    if eng.use_graphs:
        assert sorted(w for _, w in eng.decode_graphs.graphs) == [8, 16]
    check_logits(torch.cat(rows_a), pm.logits(long_ids)[500:], pm16.logits(long_ids)[500:], dtype, "the long sequence")
    check_logits(torch.cat(rows_b), pm.logits(short_ids)[10:], pm16.logits(short_ids)[10:], dtype, "its short neighbour")
    MEASURED.clear()
    assert int(eng.err_flag) == 0


def test_one_sequence_ends_by_capacity_while_others_go_on(tmp_path):
    """The generation loop launches the next decode step before it has read the last one's tokens,
    for the sequences that cannot end by count. With 128 positions a prompt of 120 tokens ends after
    its ninth token for want of room while two shorter requests run to their length and a third to
    its stop token: every request's tokens equal the plain implementation's."""
    from scriptling_llm_lib_b200 import llm
    raw, seed = TINY["A"]                                                # 128 positions
    d = make_model_dir(tmp_path / "m", raw, seed)
    pm = plain_model(d)
    prompts = [random_ids(n, 256, 130 + n) for n in (120, 20, 5, 64)]
    kw = dict(strategy="temperature", temperature=1.0, repeat_penalty=0.0)
    free = [plain.generate(pm, p, 30, stop_ids=(), seed=9 + i, **kw) for i, p in enumerate(prompts)]
    stop = free[2][11]                                                   # request 2 stops at its 12th token at the latest
    want = [plain.generate(pm, p, 30, stop_ids=(stop,), seed=9 + i, **kw)[:128 - len(p) + 1] for i, p in enumerate(prompts)]
    got, st = llm.generate(d, prompts, 30, "temperature", temperature=1.0, repeat_penalty=0.0, seed=9, stop_ids=[stop],
                           dtype="float32", stats=True)
    assert got == want
    reasons = ["stop" if w[-1] == stop else ("capacity" if len(p) + len(w) - 1 >= 128 else "length") for p, w in zip(prompts, want)]
    assert st["finish_reason"] == reasons and reasons[0] == "capacity" and "length" in reasons
    eng, _ = llm.load(d, "float32")
    assert eng.use_graphs and eng.cache.slots.n_held == 0


def test_stale_cache_contents_change_nothing(tmp_path):
    """Pages and slots that are used again hold the last owner's keys; fill all cache memory with
    NaN between two runs: the tokens are the same."""
    from scriptling_llm_lib_b200 import llm
    raw, seed = TINY["C"]
    d = make_model_dir(tmp_path / "m", raw, seed)
    prompts = [random_ids(n, 1003, 90 + n) for n in (70, 3, 129)]
    for dtype in ("float32", "bfloat16"):
        first = llm.generate(d, prompts, 20, stop_ids=[], dtype=dtype)
        eng, _ = llm.load(d, dtype)
        for g in eng.cache.groups:
            g.k.fill_(float("nan"))
            g.v.fill_(float("nan"))
        assert llm.generate(d, prompts, 20, stop_ids=[], dtype=dtype) == first
        assert llm.generate(d, prompts[::-1], 20, stop_ids=[], dtype=dtype) == first[::-1]


def test_errors_before_anything_runs(tmp_path):
    from scriptling_llm_lib_b200.cache import CacheFull
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry, StepError
    raw, seed = TINY["A"]
    d = make_model_dir(tmp_path / "m", raw, seed)
    eng = Engine.from_folder(d, "float32", max_tokens=128, max_seqs=2)
    s = eng.open()
    with pytest.raises(StepError, match="vocabulary"):
        eng.step([StepEntry(s, [1, 256])])
    with pytest.raises(StepError, match="no tokens"):
        eng.step([StepEntry(s, [])])
    with pytest.raises(StepError, match="twice"):
        eng.step([StepEntry(s, [1]), StepEntry(s, [2])])
    with pytest.raises(StepError, match="outside the entry"):
        eng.step([StepEntry(s, [1, 2], [2])])
    with pytest.raises(StepError, match="at most"):
        eng.step([StepEntry(s, [1] * 129)])
    assert s.length == 0
    s2 = eng.open()
    with pytest.raises(CacheFull):
        eng.open()
    eng.step([StepEntry(s, [1] * 100)])
    with pytest.raises(CacheFull):
        eng.step([StepEntry(s2, [1] * 30)])                              # 2 pages hold 128 tokens: 1 page is left
    assert s2.length == 0 and s.length == 100
    s.close()
    with pytest.raises(StepError, match="closed"):
        eng.step([StepEntry(s, [1])])
    with pytest.raises(StepError, match="CUDA"):
        Engine.from_folder(d, "float32", max_tokens=128, device="cpu")


def test_command_line(tmp_path):
    raw, seed = TINY["A"]
    d = make_model_dir(tmp_path / "m", raw, seed)
    pm = plain_model(d)
    p = random_ids(9, 256, 5)
    want = plain.generate(pm, p, 6, stop_ids=(7,))
    run = subprocess.run([sys.executable, str(ROOT / "bin" / "sllm-b200"), "-model", str(d), "-prompt",
                          ",".join(map(str, p)), "-tokens", "6", "-dtype", "float32"], capture_output=True, text=True)
    assert run.returncode == 0, run.stderr
    assert [int(t) for t in run.stdout.split()] == want
    assert "prefill" in run.stderr and "decode" in run.stderr and "t/s" in run.stderr
    bad = subprocess.run([sys.executable, str(ROOT / "bin" / "sllm-b200"), "-prompt", "1,2"], capture_output=True, text=True)
    assert bad.returncode == 1 and "-model is required" in bad.stderr


@pytest.mark.parametrize("stored", [torch.bfloat16, torch.float32])
def test_random_mode_on_the_device_equals_the_written_folder(tmp_path, stored):
    """The fill kernel and the host statement of the generator give the same bits: every tensor of
    a model drawn on the device equals the tensor in the folder that random-weights mode writes,
    in bfloat16 and in 32-bit storage, odd sizes and norm weights included."""
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    from scriptling_llm_lib_b200.config.registry import architecture_for
    from scriptling_llm_lib_b200.weights.random_init import draw_device, draw_host, random_tensors
    from scriptling_llm_lib_b200.weights.spec import TensorSpec
    raw, _ = TINY["C"]                                                   # vocabulary 1003, hidden 144: nothing a power of two
    arch = architecture_for(raw["architectures"][0])
    specs = DecoderModel(arch.layout(arch.config_class.from_dict(raw, "test"))).tensor_specs()
    host = random_tensors(specs, 11, stored, "cpu")
    devt = random_tensors(specs, 11, stored, "cuda:0")
    for s in specs:
        assert devt[s.name].dtype == stored and torch.equal(devt[s.name].cpu(), host[s.name]), s.name
    # a larger matrix (more than one pass of the host's chunks is not needed: 3 million elements), an odd
    # element count, a seed with a high word, an integer table
    for spec, seed, index in [(TensorSpec("w", (1501, 2003)), 2 ** 40 + 3, 77), (TensorSpec("w", (7,)), 5, 0),
                              (TensorSpec("t", (1001,), init="integer_table"), 9, 3)]:
        a, b = draw_host(spec, seed, index, stored), draw_device(spec, seed, index, stored, "cuda:0").cpu()
        assert torch.equal(a, b), spec


def test_random_model_spec_runs_like_its_folder(tmp_path):
    """`random:<config.json>:seed` through the entry point, trace replay and the command line gives what
    the written folder of the same configuration and seed gives."""
    import json
    from scriptling_llm_lib_b200 import llm
    raw, _ = TINY["B"]
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(raw))
    d = llm.random_model(raw, 21, tmp_path / "folder")
    prompts = [random_ids(n, raw["vocab_size"], 70 + n) for n in (9, 30)]
    for dtype in ("float32", "bfloat16"):
        want = llm.generate(d, prompts, 10, "greedy", stop_ids=[], dtype=dtype)
        got = llm.generate(f"random:{cfg_path}:21", prompts, 10, "greedy", stop_ids=[], dtype=dtype)
        assert got == want
    other = llm.generate(f"random:{cfg_path}:22", prompts, 10, "greedy", stop_ids=[], dtype="float32")
    assert other != llm.generate(d, prompts, 10, "greedy", stop_ids=[], dtype="float32")
    # trace replay takes the spec where it takes a folder
    from helpers import Replay, replay_whole
    ids = random_ids(40, raw["vocab_size"], 5)
    outs = []
    for model in (str(d), f"random:{cfg_path}:21"):
        rp = Replay(model, "float32", tmp_path / ("out" + str(len(outs))), 64, raw["vocab_size"])
        outs.append(replay_whole(rp, "a", ids))
        assert rp.close() == 0
    assert (outs[0] == outs[1]).all()
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "sllm-b200"), "-model", f"random:{cfg_path}:21", "-prompt",
                        " ".join(map(str, prompts[0])), "-tokens", "10", "-stop", "", "-dtype", "float32"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == llm.generate(d, prompts[0], 10, "greedy", stop_ids=[], dtype="float32")


def test_state_record_on_the_device_follows_the_generation(tmp_path, monkeypatch):
    """Every sequence has a fixed-size record on the device (tokens held, tokens generated, last
    token, finished flag, sampling key and draw counter) that the sampling kernel reads and
    advances: a sampled run packs and uploads no parameters per step, and after the run the records
    hold what the host's bookkeeping says."""
    from scriptling_llm_lib_b200 import llm
    from scriptling_llm_lib_b200.cache.store import (SEQ_COUNTER, SEQ_FLAG_FINISHED, SEQ_FLAGS, SEQ_GENERATED, SEQ_KEY,
                                                     SEQ_LAST_TOKEN, SEQ_POS)
    from scriptling_llm_lib_b200.sampling.sampler import Sampler
    raw, seed = TINY["B"]
    d = make_model_dir(tmp_path / "m", raw, seed)
    pm = plain_model(d)
    prompts = [random_ids(n, 384, 60 + n) for n in (8, 40, 3)]
    kw = dict(strategy="top_k", temperature=0.9, top_k=30, repeat_penalty=0.0)
    free = [plain.generate(pm, p, 14, stop_ids=(), seed=2 ** 33 + 5 + i, **kw) for i, p in enumerate(prompts)]
    stop = free[1][6]
    want = [plain.generate(pm, p, 14, stop_ids=(stop,), seed=2 ** 33 + 5 + i, **kw) for i, p in enumerate(prompts)]

    def no_upload(self, options, seeds, draws):
        raise AssertionError("sampling parameters were packed on the host for a step")
    monkeypatch.setattr(Sampler, "_params", no_upload)
    got = llm.generate(d, prompts, 14, "top_k", temperature=0.9, top_k=30, repeat_penalty=0.0, seed=2 ** 33 + 5, stop_ids=[stop],
                       dtype="float32")
    assert got == want
    eng, _ = llm.load(d, "float32")
    rec = eng.cache.seq_state.cpu().numpy().astype("int64") & 0xFFFFFFFF
    for slot, (p, out) in enumerate(zip(prompts, got)):                  # one batch: request i ran in slot i
        r = rec[slot]
        assert r[SEQ_GENERATED] == len(out) and r[SEQ_LAST_TOKEN] == out[-1]
        assert r[SEQ_POS] == len(p) + len(out) - 1                       # the last sampled token is not fed back
        assert bool(r[SEQ_FLAGS] & SEQ_FLAG_FINISHED) == (out[-1] == stop)
        assert r[SEQ_KEY] == 5 + slot and r[SEQ_KEY + 1] == 2 and r[SEQ_COUNTER] == len(out) and r[SEQ_COUNTER + 1] == 0
    # a slot that is opened again starts from a zeroed record
    s = eng.open()
    assert int(eng.cache.seq_state[s.slot].abs().sum()) == 0
    s.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_batches_of_prompts_go_through_in_portions(tmp_path, dtype):
    """The generation loop keeps a prompt step under a number of rows: with room for 64 rows a step,
    prompts of 120, 30, 75 and 200 tokens take seven steps, each portion landing on what the ones
    before left in the cache; logits of the last places and generated tokens are those of one step."""
    from scriptling_llm_lib_b200 import llm
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    raw, seed = TINY["D"]
    d = make_model_dir(tmp_path / "m", raw, seed)
    pm, pm16 = plain_model(d), plain_model_bf16(d)
    prompts = [random_ids(n, raw["vocab_size"], 640 + n) for n in (120, 30, 75, 200)]
    eng = Engine.from_folder(d, dtype, max_tokens=1024, max_seqs=4)
    seqs = [eng.open() for _ in prompts]
    steps_before = []
    orig_step = eng.step
    eng.step = lambda entries: (steps_before.append(sum(len(e.tokens) for e in entries)), orig_step(entries))[1]
    logits, index = eng.prompt_step([StepEntry(s, p) for s, p in zip(seqs, prompts)], max_tokens_per_step=64)
    assert steps_before == [64, 64, 64, 64, 64, 64, 41] and index.slots.tolist() == [s.slot for s in seqs]
    assert index.pos_after.tolist() == [len(p) for p in prompts] == [s.length for s in seqs]
    for i, p in enumerate(prompts):
        check_logits(logits[i:i + 1].cpu().double(), pm.logits(p)[-1:], pm16.logits(p)[-1:], dtype, f"prompt {i} in portions")
    MEASURED.clear()
    for s in seqs:
        s.close()
    if dtype == "float32":
        gen_eng, _ = llm.load(d, "float32")
        gen_eng.PROMPT_TOKENS_PER_STEP = 64
        got = llm.generate(d, prompts, 6, "greedy", stop_ids=[], dtype="float32")
        assert got == [plain.generate(pm, p, 6, stop_ids=()) for p in prompts]


def test_no_garbage_collection_while_a_step_is_captured(tmp_path):
    """Graphs of an engine that is no longer in use hang in reference cycles; were the collector to
    run while another engine captures a step, destroying them would invalidate that capture. So the
    collector runs before a capture and is off during it (and on again afterwards)."""
    import gc
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    raw, seed = TINY["D"]
    d = make_model_dir(tmp_path / "m", raw, seed)
    eng = Engine.from_folder(d, "bfloat16", max_tokens=256)
    assert eng.use_graphs
    seen = []
    forward = eng._forward

    def watched(ctx, want):
        if torch.cuda.is_current_stream_capturing():
            seen.append(gc.isenabled())
        return forward(ctx, want)

    eng._forward = watched
    assert gc.isenabled()
    s = eng.open()
    eng.step([StepEntry(s, random_ids(5, raw["vocab_size"], 3), [])])
    eng.step([StepEntry(s, [7], [0])])                      # the first decode step of this shape: captured here
    s.close()
    assert seen == [False] and gc.isenabled()
