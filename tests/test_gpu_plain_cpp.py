"""The 32-bit engine against the C++ statement of the decoder, which computes in the reference's own
arithmetic (float32 with sequential sums and float64 islands): whole prompts and the last tokens one
by one, every tiny configuration."""
import pytest
import torch

from helpers import TINY, TOL_F32, cpp_logits, cpp_plain_binary, make_model_dir, random_ids, rel_err

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(cpp_plain_binary() is None, reason="no g++ here")]


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_32_bit_engine_agrees_with_the_cpp_statement(tmp_path, name):
    from scriptling_llm_lib_b200.engine.step import Engine, StepEntry
    raw, seed = TINY[name]
    d = make_model_dir(tmp_path / "m", raw, seed)
    ids = random_ids(100, raw["vocab_size"], 31)
    want = cpp_logits(d, ids, tmp_path / "cpp")
    eng = Engine.from_folder(d, "float32", max_tokens=256)
    s = eng.open()
    whole = eng.step([StepEntry(s, ids, list(range(len(ids))))]).cpu().double()
    s.close()
    assert rel_err(whole, want) < TOL_F32
    s = eng.open()
    rows = [eng.step([StepEntry(s, ids[:80], list(range(80)))])] + [eng.step([StepEntry(s, [t], [0])]) for t in ids[80:]]
    s.close()
    assert rel_err(torch.cat(rows).cpu().double(), want) < TOL_F32
