"""Trace replay on the GPU: the same requests whole, with the last 32 tokens one by one, and in
batches of unequal lengths one after another on reused slots, in 32-bit and in bfloat16, all
against the plain implementation."""
import pytest

import numpy as np
import torch

from helpers import (MEASURED, TINY, TOL_BF16, TOL_F32, Replay, check_logits, make_model_dir, plain_model, plain_model_bf16,
                     random_ids, rel_err, replay_batch, replay_tail_stepwise, replay_whole)

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 33, 5, 64, 1, 100, 47], "B": [40, 63, 1, 8, 129, 65, 200], "C": [90, 33, 150, 64, 17, 230, 128],
           "D": [300, 33, 150, 129, 17, 260, 128], "E": [40, 280, 1, 8, 160, 65, 200]}
PROMPTS = [0.5, 1.0, 0.2, 0.9, 1.0, 0.33, 0.01]       # share of a request that is its prompt in the batched replay


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_replay_cuttings(tmp_path, name, dtype):
    raw, seed = TINY[name]
    d = make_model_dir(tmp_path / "model", raw, seed)
    V = raw["vocab_size"]
    reqs = {f"r{i}": random_ids(n, V, 100 + i) for i, n in enumerate(LENGTHS[name])}
    want = {r: plain_model(d).logits(ids).numpy() for r, ids in reqs.items()}
    want16 = {r: plain_model_bf16(d).logits(ids).numpy() for r, ids in reqs.items()} if dtype == "bfloat16" else want
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    # cache: just enough pages for the largest batch of three, so later batches reuse slots and pages
    names = list(reqs)
    batches = [names[0:3], names[3:6], names[6:]]
    need = max(sum(-(-len(reqs[r]) // 64) * 64 for r in b) for b in batches)
    rp = Replay(d, dtype, tmp_path / "out", need, V)
    try:
        whole = {r: replay_whole(rp, r, ids) for r, ids in reqs.items()}
        for r in reqs:
            check_logits(whole[r], want[r], want16[r], dtype, f"{name} {r} whole")
        for r, ids in reqs.items():
            got = replay_tail_stepwise(rp, r, ids, 32)
            check_logits(got, want[r], want16[r], dtype, f"{name} {r} last 32 one by one")
            assert rel_err(got, whole[r]) < (1e-5 if dtype == "float32" else tol), f"{r} stepwise vs whole"
        for r, ids in reqs.items():
            # the prompt in two portions: the second, of 130 tokens where the request is long enough
            # (more rows than the few-rows products take), lands on a cache that is not empty
            head = len(ids) - 130 if len(ids) >= 194 else len(ids) // 3
            if head < 1:
                continue
            first = rp.step([(r, ids[:head], list(range(head)))])
            second = rp.step([(r, ids[head:], list(range(len(ids) - head)))], end=[r])
            got = np.concatenate([first, second])
            check_logits(got, want[r], want16[r], dtype, f"{name} {r} in two portions ({head} + {len(ids) - head})")
            assert rel_err(got, whole[r]) < (1e-5 if dtype == "float32" else tol), f"{r} two portions vs whole"
        for b in batches:
            plens = {r: max(1, int(len(reqs[r]) * PROMPTS[names.index(r)])) for r in b}
            got = replay_batch(rp, {r: reqs[r] for r in b}, plens)
            for r in b:
                check_logits(got[r], want[r], want16[r], dtype, f"{name} {r} in batch {b}")
                assert rel_err(got[r], whole[r]) < (1e-5 if dtype == "float32" else tol), f"{r} batch vs whole"
        assert rp.step([("x", [1, 2, 3], [])], end=["x"]) is None           # nothing wanted: no file
    finally:
        assert rp.close() == 0
    if MEASURED:
        print(f"\n[{name} {dtype}] largest error against the rounding / the unrounded plain implementation: "
              f"{max(m[1] for m in MEASURED):.3g} / {max(m[2] for m in MEASURED):.3g}")
        MEASURED.clear()


def test_replay_refuses_more_than_the_cache_holds(tmp_path):
    raw, seed = TINY["A"]
    d = make_model_dir(tmp_path / "model", raw, seed)
    rp = Replay(d, "float32", tmp_path / "out", 64, 256)
    with pytest.raises(AssertionError):
        rp.step([("a", random_ids(65, 256, 0), [0])])
    assert rp.close() != 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_a_step_may_mix_prompts_and_single_tokens(tmp_path, name, dtype):
    """The step function takes entries of any lengths: one sequence goes on by one token while
    another brings its whole prompt and a third a further portion of its prompt. Replay never
    drives such a step, generation never does; the engine accepts it, so it has to be right."""
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    raw, seed = TINY[name]
    d = make_model_dir(tmp_path / "model", raw, seed)
    V = raw["vocab_size"]
    a, b, c = random_ids(90, V, 301), random_ids(41, V, 302), random_ids(100, V, 303)
    pm, pm16 = plain_model(d), plain_model_bf16(d)
    eng = Engine.from_folder(d, dtype, max_tokens=512)
    sa, sb, sc = eng.open(), eng.open(), eng.open()
    eng.step([StepEntry(sa, a[:70], []), StepEntry(sc, c[:64], [])])
    got_a, got_b, got_c = [], [], []
    out = eng.step([StepEntry(sa, [a[70]], [0]), StepEntry(sb, b, list(range(len(b)))), StepEntry(sc, c[64:90], [0, 25])])
    got_a.append(out[0:1]); got_b.append(out[1:1 + len(b)]); got_c.append(out[1 + len(b):])
    out = eng.step([StepEntry(sc, c[90:], [9]), StepEntry(sa, a[71:], list(range(19)))])
    got_c.append(out[0:1]); got_a.append(out[1:])
    for got, ids, rows, what in [(got_a, a, list(range(70, 90)), "a"), (got_b, b, list(range(len(b))), "b"),
                                 (got_c, c, [64, 89, 99], "c")]:
        g = torch.cat(got).cpu().double()
        check_logits(g, pm.logits(ids)[rows], pm16.logits(ids)[rows], dtype, f"{name} mixed step, request {what}")
    MEASURED.clear()
    assert int(eng.err_flag) == 0
