"""The C++ statement of the decoder (tests/plain_cpp/plain_llama.cpp: the reference's float32
arithmetic with its float64 islands, sequential sums) against the Python one (float64 throughout):
two statements of the same formulas, written apart, agree on every tiny configuration to the
rounding of float32 (no GPU)."""
import pytest

from helpers import TINY, cpp_logits, cpp_plain_binary, make_model_dir, plain_model, random_ids, rel_err

pytestmark = pytest.mark.skipif(cpp_plain_binary() is None, reason="no g++ here")


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_cpp_and_python_statements_agree(tmp_path, name):
    raw, seed = TINY[name]
    d = make_model_dir(tmp_path / "m", raw, seed)
    ids = random_ids(70, raw["vocab_size"], 21)
    got = cpp_logits(d, ids, tmp_path / "cpp")
    want = plain_model(d).logits(ids)
    assert rel_err(got, want) < 2e-5
    # and it is a statement of this model: another token changes the rows from its place on
    other = list(ids)
    other[30] = (other[30] + 1) % raw["vocab_size"]
    changed = cpp_logits(d, other, tmp_path / "cpp2")
    assert (changed[:30] == got[:30]).all() and rel_err(changed[30:], want[30:]) > 1e-3
