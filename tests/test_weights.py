"""Safetensors reading/writing, the loader's one error, random-weights mode (no GPU)."""
import json
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, make_model_dir
import plain_llama as plain
from scriptling_llm_lib_b200 import models  # noqa: F401
from scriptling_llm_lib_b200.config import LlamaConfig
from scriptling_llm_lib_b200.engine.model import DecoderModel
from scriptling_llm_lib_b200.models.llama import llama_layout
from scriptling_llm_lib_b200.weights.spec import TensorSpec
from scriptling_llm_lib_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights,
                                              write_safetensors)


def specs_of(raw):
    return DecoderModel(llama_layout(LlamaConfig.from_dict(raw))).tensor_specs()


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32),
         "c": torch.randn(2, 2, 2), "empty": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", t, {"note": "hi"})
    with SafetensorsFile(tmp_path / "x.safetensors") as f:
        assert set(f.names()) == set(t)
        assert f.metadata["note"] == "hi"
        for k, v in t.items():
            got = f.tensor(k).clone()
            assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    # the plain implementation's own parse reads the same numbers
    other = plain.read_safetensors(tmp_path / "x.safetensors")
    assert torch.equal(other["a"], t["a"].double()) and torch.equal(other["c"], t["c"].double())


def test_malformed_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="claims bytes"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                      "v": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="overlap"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 1]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0")
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(p)


def test_random_mode_writes_a_loadable_folder_and_is_seeded(tmp_path):
    d0 = make_model_dir(tmp_path / "a0", TINY_A, 0)
    d0b = make_model_dir(tmp_path / "a0b", TINY_A, 0)
    d1 = make_model_dir(tmp_path / "a1", TINY_A, 1)
    assert (d0 / "config.json").is_file() and (d0 / "model.safetensors").is_file()
    assert LlamaConfig.from_dict(json.loads((d0 / "config.json").read_text())) == LlamaConfig.from_dict(TINY_A)
    w0 = load_weights(d0, specs_of(TINY_A), "cpu", torch.bfloat16)
    w0b = load_weights(d0b, specs_of(TINY_A), "cpu", torch.bfloat16)
    w1 = load_weights(d1, specs_of(TINY_A), "cpu", torch.bfloat16)
    assert set(w0) == {s.name for s in specs_of(TINY_A)} and "lm_head.weight" not in w0    # tied
    for k in w0:
        assert w0[k].dtype == torch.bfloat16 and torch.equal(w0[k], w0b[k])
    assert not torch.equal(w0["model.layers.0.mlp.up_proj.weight"], w1["model.layers.0.mlp.up_proj.weight"])
    q = w0["model.layers.1.self_attn.q_proj.weight"].float()
    assert q.shape == (64, 64) and abs(float(q.std()) - 0.02) < 0.003 and abs(float(q.mean())) < 0.002
    n = w0["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.02                                               # 1 + N(0, 0.02)


def test_precision_kept_as_stored(tmp_path):
    d = make_model_dir(tmp_path / "f", TINY_B, 1, dtype=torch.float32)
    w = load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)
    assert all(t.dtype == torch.float32 for t in w.values())           # stored in 32-bit: stays so
    d = make_model_dir(tmp_path / "b", TINY_B, 1, dtype=torch.bfloat16)
    w16 = load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)
    w32 = load_weights(d, specs_of(TINY_B), "cpu", torch.float32)
    for k in w16:
        assert w16[k].dtype == torch.bfloat16 and w32[k].dtype == torch.float32
        assert torch.equal(w16[k].float(), w32[k])                     # widening is exact


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    d = make_model_dir(tmp_path / "m", TINY_B, 1)
    with SafetensorsFile(d / "model.safetensors") as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["model.layers.2.mlp.down_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 95, dtype=torch.bfloat16)
    tensors["model.layers.9.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    write_safetensors(d / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)
    err = e.value
    assert set(err.missing) == {"model.layers.2.mlp.down_proj.weight", "lm_head.weight"}
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.misshapen == [("model.layers.0.self_attn.k_proj.weight", (32, 95), (32, 96))]
    assert err.bad_dtype == [("model.norm.weight", "int32")]
    msg = str(err)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "is [32, 95], expected [32, 96]",
                 "model.layers.9.extra.weight", "lm_head.weight"):
        assert word in msg


def test_tied_model_tolerates_a_head_in_the_file_and_missing_file_is_an_error(tmp_path):
    d = make_model_dir(tmp_path / "t", TINY_A, 0)
    with SafetensorsFile(d / "model.safetensors") as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(d / "model.safetensors", tensors)
    layout = llama_layout(LlamaConfig.from_dict(TINY_A))
    w = load_weights(d, specs_of(TINY_A), "cpu", torch.bfloat16, ignore=layout.ignorable_tensors)
    assert "lm_head.weight" not in w
    (d / "model.safetensors").unlink()
    with pytest.raises(WeightError, match="missing tensors"):
        load_weights(d, specs_of(TINY_A), "cpu", torch.bfloat16)


def test_weights_spread_over_several_files(tmp_path):
    """A folder whose tensors lie in several safetensors files named by model.safetensors.index.json
    loads to the same tensors; a tensor in two files, or an index that names a file outside the
    folder or a missing one, is an error; a tensor missing from all files is listed as missing."""
    from scriptling_llm_lib_b200.weights import SafetensorsError
    d = make_model_dir(tmp_path / "s", TINY_B, 1)
    want = load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)
    with SafetensorsFile(d / "model.safetensors") as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    (d / "model.safetensors").unlink()
    names = sorted(tensors)
    parts = {"model-00001-of-00003.safetensors": names[0::3], "model-00002-of-00003.safetensors": names[1::3],
             "model-00003-of-00003.safetensors": names[2::3]}
    for fn, ns in parts.items():
        write_safetensors(d / fn, {n: tensors[n] for n in ns})
    index = {"metadata": {}, "weight_map": {n: fn for fn, ns in parts.items() for n in ns}}
    (d / "model.safetensors.index.json").write_text(json.dumps(index))
    got = load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)
    assert set(got) == set(want) and all(torch.equal(got[k], want[k]) for k in want)
    # one tensor absent from every file
    write_safetensors(d / "model-00003-of-00003.safetensors", {n: tensors[n] for n in names[2::3][1:]})
    with pytest.raises(WeightError) as e:
        load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)
    assert e.value.missing == [names[2]]
    # the same tensor in two files
    write_safetensors(d / "model-00003-of-00003.safetensors", {n: tensors[n] for n in names[2::3] + names[:1]})
    with pytest.raises(SafetensorsError, match="two files"):
        load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)
    # an index that names a file that is not there, or not in the folder
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {names[0]: "nowhere.safetensors"}}))
    with pytest.raises(SafetensorsError, match="not in the model folder"):
        load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {names[0]: "../x.safetensors"}}))
    with pytest.raises(SafetensorsError, match="not in the model folder"):
        load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)
    (d / "model.safetensors.index.json").write_text("[1, 2")
    with pytest.raises(SafetensorsError, match="not an index"):
        load_weights(d, specs_of(TINY_B), "cpu", torch.bfloat16)


def test_random_model_through_the_python_entry_point(tmp_path):
    """llm.random_model writes a folder from a config (a dict or a file) and a seed; the same seed gives
    the same bytes, an unknown architecture is named in the error."""
    from scriptling_llm_lib_b200 import llm
    from scriptling_llm_lib_b200.config import ConfigError
    d1 = llm.random_model(TINY_A, 5, tmp_path / "r1")
    (tmp_path / "cfg.json").write_text(json.dumps(TINY_A))
    d2 = llm.random_model(tmp_path / "cfg.json", 5, tmp_path / "r2")
    assert (d1 / "model.safetensors").read_bytes() == (d2 / "model.safetensors").read_bytes()
    assert json.loads((d1 / "config.json").read_text())["hidden_size"] == 64
    assert llm.random_model(TINY_A, 6, tmp_path / "r3").joinpath("model.safetensors").read_bytes() != (d1 / "model.safetensors").read_bytes()
    with pytest.raises(ConfigError, match="not registered"):
        llm.random_model(dict(TINY_A, architectures=["NoSuchModel"]), 0, tmp_path / "r4")


def test_random_generator_is_the_stated_one():
    """The host statement of random-weights mode: Philox4x32-10 keyed by (seed, tensor number),
    a counter per four elements, Box-Muller with series for the logarithm and the sine/cosine whose
    values agree with the library functions to a few units in the last place of a double."""
    import numpy as np
    from scriptling_llm_lib_b200.weights import random_init as ri
    # the block function against the scalar statement beside the plain implementation
    c = [7, 1, 0x89ABCDEF, 0]
    w = ri.philox4x32_10(np.array([c[0]]), np.array([c[1]]), np.array([c[2]]), np.array([c[3]]), 0x12345678, 42)
    assert [int(x[0]) for x in w] == plain.philox4x32(c, [0x12345678, 42])
    # the normal pair against numpy's own functions
    a = np.array([0, 1, 2 ** 31, 2 ** 32 - 1, 12345678, 3000000000], dtype=np.uint64)
    b = np.array([0, 2 ** 30, 2 ** 31 + 5, 2 ** 32 - 1, 987654321, 2 ** 29 + 1], dtype=np.uint64)
    z0, z1 = ri._normal_pair(a, b)
    u1, u2 = (a.astype(np.float64) + 0.5) / 2 ** 32, b.astype(np.float64) / 2 ** 32
    r = np.sqrt(-2 * np.log(u1))
    assert np.abs(z0 - r * np.cos(2 * np.pi * u2)).max() < 1e-14 and np.abs(z1 - r * np.sin(2 * np.pi * u2)).max() < 1e-14
    # a tensor's values depend on (seed, number, element) only: a longer tensor starts with the shorter one
    short = ri.draw_host(TensorSpec("t", (10, 7)), 3, 5, torch.float32)
    longer = ri.draw_host(TensorSpec("t", (30, 7)), 3, 5, torch.float32)
    assert torch.equal(short, longer[:10])
    assert not torch.equal(short, ri.draw_host(TensorSpec("t", (10, 7)), 3, 6, torch.float32))
    assert not torch.equal(short, ri.draw_host(TensorSpec("t", (10, 7)), 3 + 2 ** 32, 5, torch.float32))   # the seed's high word counts
    big = ri.draw_host(TensorSpec("t", (400, 500)), 1, 0, torch.float32).double() / ri.MATRIX_STD
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01 and float(big.abs().max()) < 6.0
    assert abs(float((big ** 4).mean()) - 3.0) < 0.1                   # a normal's fourth moment
    ints = ri.draw_host(TensorSpec("t", (1000,), init="integer_table"), 1, 0, torch.float32)
    assert ints.dtype == torch.int32 and int(ints.min()) >= 0 and int(ints.max()) < 2 ** 15 and len(set(ints.tolist())) > 900


def test_init_laws_are_a_registry():
    from scriptling_llm_lib_b200.weights import random_init as ri
    with pytest.raises(ValueError, match="unknown init law"):
        ri.draw_host(TensorSpec("t", (4,), init="no_such_law"), 0, 0, torch.float32)
    ri.register_init("test_wide", ri.Normal(5.0, 2.0), replace=True)
    t = ri.draw_host(TensorSpec("t", (5000,), init="test_wide"), 0, 0, torch.float32)
    assert abs(float(t.mean()) - 5.0) < 0.1 and abs(float(t.std()) - 2.0) < 0.1
    with pytest.raises(ValueError, match="already registered"):
        ri.register_init("matrix", ri.Normal(0.0, 1.0))
    plain_norm = ri.draw_host(TensorSpec("n", (5000,), init="norm_weight"), 0, 0, torch.float32, norm_init="plain")
    assert abs(float(plain_norm.mean())) < 0.01


def test_random_model_spec_is_parsed():
    from scriptling_llm_lib_b200.weights.random_init import RandomSpec, is_random_spec, parse_random_spec
    assert parse_random_spec("random:/a/b.json") == RandomSpec("/a/b.json", 0, torch.bfloat16)
    assert parse_random_spec("random:cfg.json:7") == RandomSpec("cfg.json", 7, torch.bfloat16)
    assert parse_random_spec("random:c:/x/cfg.json:7:float32") == RandomSpec("c:/x/cfg.json", 7, torch.float32)
    assert is_random_spec("random:x") and not is_random_spec("/a/random:x") and not is_random_spec(None)
    with pytest.raises(ValueError):
        parse_random_spec("random:")
    with pytest.raises(ValueError):
        parse_random_spec("/a/folder")
