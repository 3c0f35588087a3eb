"""Trace replay on the GPU: the same requests whole, with the last 32 tokens one by one, and in
batches of unequal lengths one after another on reused slots, in 32-bit and in bfloat16, all
against the plain implementation."""
import pytest

from helpers import (TINY, TOL_BF16, TOL_F32, Replay, make_model_dir, plain_model, random_ids, rel_err, replay_batch,
                     replay_tail_stepwise, replay_whole)

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
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    # cache: just enough pages for the largest batch of three, so later batches reuse slots and pages
    names = list(reqs)
    batches = [names[0:3], names[3:6], names[6:]]
    need = max(sum(-(-len(reqs[r]) // 64) * 64 for r in b) for b in batches)
    rp = Replay(d, dtype, tmp_path / "out", need, V)
    try:
        whole = {r: replay_whole(rp, r, ids) for r, ids in reqs.items()}
        for r in reqs:
            assert rel_err(whole[r], want[r]) < tol, f"{r} whole"
        for r, ids in reqs.items():
            got = replay_tail_stepwise(rp, r, ids, 32)
            assert rel_err(got, want[r]) < tol, f"{r} last 32 one by one"
            assert rel_err(got, whole[r]) < (1e-5 if dtype == "float32" else tol), f"{r} stepwise vs whole"
        for b in batches:
            plens = {r: max(1, int(len(reqs[r]) * PROMPTS[names.index(r)])) for r in b}
            got = replay_batch(rp, {r: reqs[r] for r in b}, plens)
            for r in b:
                assert rel_err(got[r], want[r]) < tol, f"{r} in batch {b}"
                assert rel_err(got[r], whole[r]) < (1e-5 if dtype == "float32" else tol), f"{r} batch vs whole"
        assert rp.step([("x", [1, 2, 3], [])], end=["x"]) is None           # nothing wanted: no file
    finally:
        assert rp.close() == 0


def test_replay_refuses_more_than_the_cache_holds(tmp_path):
    raw, seed = TINY["A"]
    d = make_model_dir(tmp_path / "model", raw, seed)
    rp = Replay(d, "float32", tmp_path / "out", 64, 256)
    with pytest.raises(AssertionError):
        rp.step([("a", random_ids(65, 256, 0), [0])])
    assert rp.close() != 0
