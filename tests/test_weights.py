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


def test_random_values_are_a_function_of_seed_name_and_index_alone():
    from borrowed_compute_b200.weights.random_init import normal_deviates, tensor_key

    key = tensor_key(7, "model.layers.0.mlp.up_proj.weight")
    assert key != tensor_key(8, "model.layers.0.mlp.up_proj.weight") and key != tensor_key(7, "model.layers.0.mlp.gate_proj.weight")
    z = normal_deviates(key, 200_000)
    assert z.dtype == np.float32 and np.isfinite(z).all()
    # a standard normal: moments, and the mass inside one and two deviations
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01
    assert abs(((z - z.mean()) ** 4).mean() / z.var() ** 2 - 3.0) < 0.1
    assert abs((np.abs(z) < 1).mean() - 0.6827) < 0.005 and abs((np.abs(z) < 2).mean() - 0.9545) < 0.003
    # any cut of the index range gives the same values
    cut = np.concatenate([normal_deviates(key, 1, 0), normal_deviates(key, 4095, 1), normal_deviates(key, 5000, 4096)])
    assert np.array_equal(cut, z[:9096])
    # the polynomials stand in for log, cos and sin: against the float64 formula on the same draws
    h = []
    for i in range(1, 513):
        x = (key + i * 0x9E3779B97F4A7C15) & ((1 << 64) - 1)
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & ((1 << 64) - 1)
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & ((1 << 64) - 1)
        h.append(x ^ (x >> 31))
    u = np.array([((v >> 40) + 1) / 2.0 ** 24 for v in h])
    ang = np.array([2.0 * np.pi * ((v >> 16) & 0xFFFFFF) / 2.0 ** 24 for v in h])
    want = np.sqrt(-2.0 * np.log(u)) * np.cos(ang)
    assert np.abs(z[:512] - want).max() < 2e-6


def test_a_sharded_folder_reads_like_a_single_file(tmp_path):
    w = make_weights(TINY_A, 3)
    single = write_folder(str(tmp_path / "single"), TINY_A, w, "bfloat16")
    sharded = str(tmp_path / "sharded")
    os.makedirs(sharded)
    json.dump(TINY_A, open(os.path.join(sharded, "config.json"), "w"))
    names = sorted(w)
    parts = {"model-00001-of-00002.safetensors": names[: len(names) // 2], "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for fname, mine in parts.items():
        write_safetensors(os.path.join(sharded, fname), {k: torch.from_numpy(w[k]).to(torch.bfloat16) for k in mine})
    json.dump({"metadata": {}, "weight_map": {k: f for f, mine in parts.items() for k in mine}},
              open(os.path.join(sharded, "model.safetensors.index.json"), "w"))
    a, b = TensorSource(single), TensorSource(sharded)
    assert sorted(a.names()) == sorted(b.names()) == names
    for k in names:
        assert a.info(k) == b.info(k) and torch.equal(a.tensor(k), b.tensor(k))
    rt = Runtime(torch.device("cpu"), torch.bfloat16)
    la = load_tensors(expected_tensors_for_config(TINY_A), a, rt)
    lb = load_tensors(expected_tensors_for_config(TINY_A), b, rt)
    assert all(torch.equal(la[k], lb[k]) for k in la)
    # a shard that the index names but the folder lacks is one clear error
    os.remove(os.path.join(sharded, "model-00002-of-00002.safetensors"))
    with pytest.raises(WeightsError):
        TensorSource(sharded)
