"""The generation loop's decisions, driven by a scripted step function (no GPU)."""
import pytest
import torch

from scriptling_llm_lib_b200.engine.generate import BatchState, Generator, plan_batches
from scriptling_llm_lib_b200.sampling.sampler import SamplingOptions, pack_params


def test_plan_batches_respects_slots_and_pages():
    assert plan_batches([5, 17, 31], 16, 8, 100, 128) == [[0, 1, 2]]
    assert plan_batches([5, 17, 31, 2, 9], 16, 2, 100, 128) == [[0, 1], [2, 3], [4]]
    # 100 + 29 = 129 tokens -> 3 pages each; 7 pages hold two such requests
    assert plan_batches([100, 100, 100], 30, 8, 7, 4096) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="cache pages"):
        plan_batches([1000], 30, 8, 7, 4096)
    assert plan_batches([], 4, 2, 2, 64) == []


def test_batch_state_stop_length_capacity():
    st = BatchState([10, 11, 12], [[1, 2, 3], [4], [5, 6]], max_tokens=3, stop_ids=[9], max_positions=64)
    assert st.live() == [0, 1, 2]
    ended = st.accept([0, 1, 2], [3, 1, 2], [7, 9, 8])
    assert ended == [1] and st.seqs[1].reason == "stop" and st.seqs[1].out == [9]      # stop token kept and counted
    assert st.live() == [0, 2]
    assert st.accept([0, 2], [1, 1], [7, 7]) == []
    assert st.accept([0, 2], [1, 1], [7, 9]) == [0, 2]
    assert st.seqs[0].reason == "length" and st.seqs[0].out == [7, 7, 7]
    assert st.seqs[2].reason == "stop" and st.seqs[2].held == 4                         # last token not fed back
    assert st.live() == []
    cap = BatchState([0], [[1] * 100], max_tokens=50, stop_ids=(), max_positions=8)
    assert cap.seqs[0].prompt == [1] * 8                                                # the prompt keeps its tail
    assert cap.accept([0], [8], [3]) == [0] and cap.seqs[0].reason == "capacity"
    with pytest.raises(ValueError):
        BatchState([0], [[]], 3, (), 8)
    with pytest.raises(ValueError):
        BatchState([0], [[1]], 0, (), 8)


class _Seq:
    def __init__(self, eng, slot):
        self.eng, self.slot, self.closed = eng, slot, False

    def close(self):
        assert not self.closed
        self.closed = True
        self.eng.free.append(self.slot)
        self.eng.closed += 1


class _Layout:
    stop_ids = (0,)


class _Cache:
    def __init__(self, n):
        self.n_slots, self.n_pages = n, 64


class _Event:
    def record(self): pass
    def synchronize(self): pass
    def elapsed_time(self, other): return 1.0


class ScriptedEngine:
    """Counts up: the 'logits' row of a sequence is (sum of everything it was fed) as a one-hot id
    source; the scripted sampler turns that into the next token."""

    def __init__(self, n_slots):
        self.cache, self.layout, self.max_positions = _Cache(n_slots), _Layout(), 1000
        self.free = list(range(n_slots))[::-1]
        self.sums, self.opened, self.closed, self.steps = {}, 0, 0, []

    def open(self):
        slot = self.free.pop()
        self.sums[slot] = 0
        self.opened += 1
        return _Seq(self, slot)

    def new_event(self):
        return _Event()

    def step(self, entries):
        self.steps.append([(e.sequence.slot, len(e.tokens)) for e in entries])
        rows = []
        for e in entries:
            assert not e.sequence.closed
            self.sums[e.sequence.slot] += sum(e.tokens)
            rows.append(self.sums[e.sequence.slot])
        return torch.tensor(rows)


class ScriptedSampler:
    """next token = (sum so far) % 7, so every request's output is known in closed form."""

    def sample(self, logits, options, seeds, draws, recent=None):
        self.last_draws = list(draws)
        return logits % 7


def expected(prompt, max_tokens, stop=(0,)):
    out, s = [], sum(prompt)
    for _ in range(max_tokens):
        t = s % 7
        out.append(t)
        if t in stop:
            break
        s += t
    return out


def test_generator_batches_stops_and_reuses_slots():
    prompts = [[1, 2], [3], [6, 6, 6, 5], [2, 2], [1], [4, 4, 4]]
    eng = ScriptedEngine(n_slots=2)
    res = Generator(eng, ScriptedSampler()).generate(prompts, max_tokens=6, options=SamplingOptions())
    for p, r in zip(prompts, res):
        assert r.tokens == expected(p, 6) and r.prompt_tokens == len(p)
        assert r.finish_reason == ("stop" if r.tokens[-1] == 0 else "length")
    assert eng.opened == 6 and eng.closed == 6 and sorted(eng.free) == [0, 1]           # three batches on two slots
    # the first step of each batch carries whole prompts, later steps one token per live sequence
    assert eng.steps[0] == [(0, 2), (1, 1)]
    assert all(n == 1 for step in eng.steps[1:3] for _, n in step)
    # requests run alone give the same tokens
    for p, r in zip(prompts, res):
        alone = Generator(ScriptedEngine(1), ScriptedSampler()).generate([p], 6, SamplingOptions())
        assert alone[0].tokens == r.tokens


class PipelinedEngine(ScriptedEngine):
    """An engine that can take the sampled ids from the device: the loop then launches a step before
    it has read the last tokens."""
    use_graphs = True

    def __init__(self, n_slots):
        super().__init__(n_slots)
        self.device_steps = 0

    def decode_step_device(self, sequences, ids):
        self.device_steps += 1
        from scriptling_llm_lib_b200.engine.step import StepEntry
        return self.step([StepEntry(s, [int(t)]) for s, t in zip(sequences, ids.tolist())])


def test_generator_pipelined_steps_give_the_same_tokens():
    prompts = [[1, 2], [3], [6, 6, 6, 5], [2, 2], [1], [4, 4, 4], [5]]
    for max_tokens in (1, 2, 6):
        eng = PipelinedEngine(n_slots=3)
        res = Generator(eng, ScriptedSampler()).generate(prompts, max_tokens=max_tokens, options=SamplingOptions())
        for p, r in zip(prompts, res):
            assert r.tokens == expected(p, max_tokens)
            assert r.finish_reason == ("stop" if r.tokens[-1] == 0 else "length")
        assert eng.opened == len(prompts) and eng.closed == len(prompts) and sorted(eng.free) == [0, 1, 2]
        assert (eng.device_steps > 0) == (max_tokens > 1)
    # with the repeat penalty the host needs the tokens first: no step is launched ahead
    eng = PipelinedEngine(n_slots=3)
    Generator(eng, ScriptedSampler()).generate(prompts, 4, SamplingOptions("temperature", repeat_penalty=1.2))
    assert eng.device_steps == 0


def test_generator_no_stop_ids_and_cancel():
    eng = ScriptedEngine(3)
    res = Generator(eng, ScriptedSampler()).generate([[1, 2], [5, 2]], 5, SamplingOptions(), stop_ids=())
    assert [len(r.tokens) for r in res] == [5, 5] and all(r.finish_reason == "length" for r in res)
    seen = []
    res = Generator(eng, ScriptedSampler()).generate([[1, 2], [3, 3]], 50, SamplingOptions(), stop_ids=(),
                                                     on_step=lambda i, toks: seen.append((i, dict(toks))) or i >= 2)
    assert [len(r.tokens) for r in res] == [3, 3] and all(r.finish_reason == "cancelled" for r in res)
    assert [i for i, _ in seen] == [0, 1, 2] and set(seen[0][1]) == {0, 1}
    assert eng.closed == eng.opened


def test_sampling_options_and_params():
    with pytest.raises(ValueError):
        SamplingOptions("beam")
    with pytest.raises(ValueError):
        SamplingOptions("top_p", top_p=0.0)
    assert SamplingOptions("temperature", temperature=0.0).is_greedy
    assert not SamplingOptions("greedy", repeat_penalty=1.3).penalises               # greedy ignores the penalty
    assert SamplingOptions("top_k", repeat_penalty=1.3).penalises and not SamplingOptions("top_k", repeat_penalty=1.0).penalises
    p = pack_params(SamplingOptions("top_p", 0.5, 40, 0.75), [0x1_0000_0002, 5], [3, 1 << 33])
    assert p.shape == (2, 8) and p[0, 0] == 3 and p[0, 2] == 40
    assert p[0, 4] == 2 and p[0, 5] == 1 and p[0, 6] == 3 and p[1, 7] == 2
    assert p[:, 1].view("float32")[0] == 0.5 and p[:, 3].view("float32")[0] == 0.75
