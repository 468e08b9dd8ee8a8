"""Safetensors reading and writing, the one error that lists every misfit, and the
random-weights folder."""

from __future__ import annotations

import json
import os

import numpy as np
import pytest
import torch

from borrowed_compute_b200.config import WeightsError
from borrowed_compute_b200.engine.model import expected_tensors_for_config
from borrowed_compute_b200.parts.base import Runtime, TensorSpec
from borrowed_compute_b200.weights import (SafetensorsFile, TensorSource, check_tensors, load_tensors, random_tensors,
                                           write_model_folder, write_safetensors)
from conftest import TINY_A, TINY_B, make_weights, write_folder


def test_roundtrip_keeps_bits_and_types(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "d": torch.zeros(0, 4), "e": torch.tensor([1, 2], dtype=torch.int64)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t, metadata={"k": "v"})
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(t) and f.metadata == {"k": "v"}
    for k, v in t.items():
        got = f.tensor(k)
        assert got.dtype == v.dtype and tuple(got.shape) == tuple(v.shape) and torch.equal(got, v)


def test_a_library_reader_agrees(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(4, 4).to(torch.bfloat16), "n": torch.ones(4)}
    path = str(tmp_path / "y.safetensors")
    write_safetensors(path, t)
    back = st.load_file(path)
    assert all(torch.equal(back[k], t[k]) for k in t)
    st.save_file(t, str(tmp_path / "z.safetensors"))
    ours = SafetensorsFile(str(tmp_path / "z.safetensors"))
    assert all(torch.equal(ours.tensor(k), t[k]) for k in t)


def test_broken_files_are_refused(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(WeightsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightsError, match="header length"):
        SafetensorsFile(str(p))
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 8)
    with pytest.raises(WeightsError, match="spans"):
        SafetensorsFile(str(p))
    with pytest.raises(WeightsError, match="neither"):
        TensorSource(str(tmp_path / "nowhere"))


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    w = make_weights(TINY_A, 1)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.q_proj.bias"] = np.zeros(64, dtype=np.float32)
    w["model.layers.0.self_attn.k_proj.weight"] = np.zeros((16, 64), dtype=np.float32)
    folder = write_folder(str(tmp_path / "m"), TINY_A, w, "float32")
    expected = expected_tensors_for_config(TINY_A)
    with pytest.raises(WeightsError) as e:
        load_tensors(expected, TensorSource(folder), Runtime(torch.device("cpu"), torch.float32))
    msg = str(e.value)
    assert "missing (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected (1)" in msg and "q_proj.bias" in msg
    assert "wrong shape or type (1)" in msg and "expected [32, 64], found [16, 64]" in msg


def test_roles_decide_the_type_on_the_device(tmp_path):
    folder = write_folder(str(tmp_path / "m"), TINY_B, make_weights(TINY_B, 2), "bfloat16")
    expected = expected_tensors_for_config(TINY_B)
    for dtype in (torch.bfloat16, torch.float32):
        got = load_tensors(expected, TensorSource(folder), Runtime(torch.device("cpu"), dtype))
        assert got["model.layers.0.mlp.gate_proj.weight"].dtype == dtype
        assert got["model.norm.weight"].dtype == torch.float32          # vectors are float32 on both paths
        assert "lm_head.weight" not in got                               # tied and absent
    check_tensors({"t": TensorSpec((2,), role="index")}, {"t": (torch.int64, (2,))}, "x")
    with pytest.raises(WeightsError, match="role 'index'"):
        check_tensors({"t": TensorSpec((2,), role="index")}, {"t": (torch.float32, (2,))}, "x")


def test_a_stored_head_is_tolerated_when_tied(tmp_path):
    w = make_weights(TINY_B, 2)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].copy()
    folder = write_folder(str(tmp_path / "m"), TINY_B, w, "bfloat16")
    load_tensors(expected_tensors_for_config(TINY_B), TensorSource(folder), Runtime(torch.device("cpu"), torch.bfloat16))


def test_random_folder_is_a_function_of_config_and_seed(tmp_path):
    a = write_model_folder(str(tmp_path / "a"), TINY_A, seed=4)
    b = write_model_folder(str(tmp_path / "b"), TINY_A, seed=4)
    c = write_model_folder(str(tmp_path / "c"), TINY_A, seed=5)
    sa, sb, sc = TensorSource(a), TensorSource(b), TensorSource(c)
    assert sorted(sa.names()) == sorted(expected_tensors_for_config(TINY_A))
    assert json.load(open(os.path.join(a, "config.json")))["hidden_size"] == 64
    name = "model.layers.1.self_attn.v_proj.weight"
    assert torch.equal(sa.tensor(name), sb.tensor(name)) and not torch.equal(sa.tensor(name), sc.tensor(name))
    assert sa.info(name) == (torch.bfloat16, (32, 64))
    w = sa.tensor(name).float()
    assert abs(float(w.std()) - 0.02) < 0.003 and abs(float(w.mean())) < 0.003
    assert torch.equal(sa.tensor("model.norm.weight").float(), torch.ones(64))
    # a tensor's values depend on its own name and the seed only
    one = random_tensors({name: expected_tensors_for_config(TINY_A)[name]}, 4, torch.bfloat16)
    assert torch.equal(one[name], sa.tensor(name))
    tied = TensorSource(write_model_folder(str(tmp_path / "t"), TINY_B, seed=1, dtype=torch.float32))
    assert "lm_head.weight" not in tied.names() and tied.info("model.norm.weight")[0] == torch.float32
