"""Safetensors reading and writing, the by-name loader and its one error, random
weights (no device needed)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from tiny import CONFIGS, TINY_A, make_model_dir, read_weights_numpy
from torchless_rs_b200.config import config_from_dict
from torchless_rs_b200.engine.model import expected_tensors
from torchless_rs_b200.weights import (SafetensorsFile, SafetensorsFormatError, TensorSpec,
                                       WeightsMismatchError, load_checked, random_tensor,
                                       storage_dtype, write_random_model, write_safetensors)


def test_expected_names_are_the_reference_names():
    names = expected_tensors(config_from_dict(TINY_A).model_spec())
    assert len(names) == 3 + 9 * 2
    assert names["model.embed_tokens.weight"].shape == (256, 64)
    assert names["lm_head.weight"].shape == (256, 64)
    assert names["model.norm.weight"].shape == (64,)
    assert names["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert names["model.layers.0.mlp.down_proj.weight"].shape == (64, 176)
    assert names["model.layers.0.post_attention_layernorm.weight"].shape == (64,)


def test_written_file_reads_back_with_the_safetensors_package(tmp_path):
    d = make_model_dir(CONFIGS["C"], 3, torch.bfloat16, str(tmp_path))
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    theirs = read_weights_numpy(d)
    spec = expected_tensors(config_from_dict(CONFIGS["C"]).model_spec())
    ours, src = load_checked(d, spec)
    assert set(theirs) == set(ours) == set(spec)
    for k in ours:
        assert ours[k].dtype == torch.bfloat16
        assert np.array_equal(ours[k].float().numpy(), theirs[k])
    src.close()


def test_storage_rule(tmp_path):
    assert storage_dtype(torch.float16) == torch.bfloat16
    assert storage_dtype(torch.float16, torch.float32) == torch.float32   # widened exactly for the 32-bit path
    assert storage_dtype(torch.bfloat16) == torch.bfloat16
    assert storage_dtype(torch.float32) == torch.float32     # stored in 32-bit stays so
    assert storage_dtype(torch.float64) == torch.float32
    assert storage_dtype(torch.int64) == torch.int32         # integer tables
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, [("a", torch.ones(2, 3, dtype=torch.float32)),
                          ("b", torch.ones(4, dtype=torch.float16)),
                          ("c", torch.arange(5, dtype=torch.int64))])
    got, src = load_checked(str(tmp_path), {"a": TensorSpec((2, 3)), "b": TensorSpec((4,)),
                                            "c": TensorSpec((5,), integer=True)})
    assert (got["a"].dtype, got["b"].dtype, got["c"].dtype) == (torch.float32, torch.bfloat16, torch.int32)
    src.close()
    # a float16 value that bfloat16 cannot hold survives on the 32-bit path
    fine = torch.tensor([1.0 + 2.0 ** -10] * 4, dtype=torch.float16)
    write_safetensors(p, [("b", fine)])
    got, src = load_checked(str(tmp_path), {"b": TensorSpec((4,))}, torch.float32)
    assert got["b"].dtype == torch.float32 and torch.equal(got["b"], fine.float())
    src.close()
    got, src = load_checked(str(tmp_path), {"b": TensorSpec((4,))}, torch.bfloat16)
    assert got["b"].dtype == torch.bfloat16 and torch.equal(got["b"], fine.to(torch.bfloat16))
    src.close()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(TINY_A)
    spec = expected_tensors(cfg.model_spec())
    tensors = {n: torch.zeros(s.shape, dtype=torch.bfloat16) for n, s in spec.items()}
    del tensors["lm_head.weight"]
    del tensors["model.layers.1.mlp.up_proj.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64, dtype=torch.bfloat16)
    tensors["model.norm.weight"] = torch.zeros(65, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros((64, 32), dtype=torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), list(tensors.items()))
    with pytest.raises(WeightsMismatchError) as ei:
        load_checked(str(tmp_path), spec)
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert sorted(n for n, _, _ in e.wrong_shape) == ["model.layers.0.self_attn.k_proj.weight",
                                                      "model.norm.weight"]
    msg = str(e)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (2)", "expected [32, 64] got [64, 32]"):
        assert word in msg


def test_sharded_folder_and_its_errors(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), [("a", torch.ones(2))])
    write_safetensors(str(tmp_path / "s2.safetensors"), [("b", torch.ones(3))])
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    got, src = load_checked(str(tmp_path), {"a": TensorSpec((2,)), "b": TensorSpec((3,))})
    assert got["b"].shape == (3,)
    src.close()
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"a": "s1.safetensors", "b": "gone.safetensors"}}))
    with pytest.raises(SafetensorsFormatError, match="gone.safetensors"):
        load_checked(str(tmp_path), {})
    with pytest.raises(FileNotFoundError):
        load_checked(str(tmp_path / "empty"), {})


def test_malformed_files_are_refused(tmp_path):
    def write(name, header: bytes, data: bytes = b"", hlen=None):
        p = tmp_path / name
        p.write_bytes(struct.pack("<Q", len(header) if hlen is None else hlen) + header + data)
        return str(p)
    with pytest.raises(SafetensorsFormatError, match="too small"):
        (tmp_path / "tiny").write_bytes(b"abc")
        SafetensorsFile(str(tmp_path / "tiny"))
    with pytest.raises(SafetensorsFormatError, match="header size"):
        SafetensorsFile(write("h", b"{}", hlen=10 ** 9))
    with pytest.raises(SafetensorsFormatError, match="JSON"):
        SafetensorsFile(write("j", b"{not json}"))
    hdr = json.dumps({"a": {"dtype": "Q4", "shape": [1], "data_offsets": [0, 1]}}).encode()
    with pytest.raises(SafetensorsFormatError, match="unknown dtype"):
        SafetensorsFile(write("d", hdr, b"\0"))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with pytest.raises(SafetensorsFormatError, match="beyond"):
        SafetensorsFile(write("b", hdr, b"\0" * 8))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}).encode()
    with pytest.raises(SafetensorsFormatError, match="needs 12"):
        SafetensorsFile(write("s", hdr, b"\0" * 16))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                      "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    with pytest.raises(SafetensorsFormatError, match="overlap"):
        SafetensorsFile(write("o", hdr, b"\0" * 12))
    with pytest.raises(SafetensorsFormatError, match="twice"):
        SafetensorsFile(write("t", b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},'
                                   b'"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}', b"\0" * 4))


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    s = TensorSpec((40, 30))
    a = random_tensor("x.weight", s, 5, torch.float32)
    assert torch.equal(a, random_tensor("x.weight", s, 5, torch.float32))
    assert not torch.equal(a, random_tensor("x.weight", s, 6, torch.float32))
    assert not torch.equal(a, random_tensor("y.weight", s, 5, torch.float32))
    assert abs(float(a.std()) - 0.02) < 0.003 and abs(float(a.mean())) < 0.003
    n = random_tensor("n.weight", TensorSpec((4000,)), 5, torch.float32)
    assert abs(float(n.mean()) - 1.0) < 0.01 and abs(float(n.std()) - 0.1) < 0.01
    d1 = write_random_model(config_from_dict(TINY_A), str(tmp_path / "a"), 9)
    d2 = write_random_model(config_from_dict(TINY_A), str(tmp_path / "b"), 9)
    w1, w2 = read_weights_numpy(d1), read_weights_numpy(d2)
    assert all(np.array_equal(w1[k], w2[k]) for k in w1)
    assert json.load(open(os.path.join(d1, "config.json")))["sliding_window"] == 16


def test_random_stream_is_a_function_of_key_and_index():
    """Any stretch of a tensor can be drawn by itself; the numbers are standard normal; the
    polynomials that stand in for ln, sin and cos agree with the library's to rounding."""
    from torchless_rs_b200.weights.random_init import _bits, standard_normals, tensor_key
    key = tensor_key(3, "model.layers.0.mlp.up_proj.weight")
    whole = standard_normals(key, 0, 5000)
    assert np.array_equal(whole[137:1500], standard_normals(key, 137, 1363))
    assert np.array_equal(whole[4001:], standard_normals(key, 4001, 999))
    z = standard_normals(key, 0, 400000)
    assert abs(z.mean()) < 5e-3 and abs(z.std() - 1) < 5e-3 and abs((z ** 4).mean() - 3) < 5e-2
    assert abs(np.corrcoef(z[0::2], z[1::2])[0, 1]) < 5e-3        # the two numbers of a pair
    # Box-Muller with the library's functions on the same bits
    i = np.arange(5000, dtype=np.uint64)
    bits = _bits(key, i >> np.uint64(1))
    u1 = ((bits >> np.uint64(32)).astype(np.float64) + 1.0) / 2.0 ** 32
    ang = 2.0 * np.pi * (bits & np.uint64(0xFFFFFFFF)).astype(np.float64) / 2.0 ** 32
    lib = np.sqrt(-2.0 * np.log(u1)) * np.where(i % 2 == 0, np.cos(ang), np.sin(ang))
    assert np.allclose(whole, lib, rtol=0, atol=1e-13)
