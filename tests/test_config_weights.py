"""Configuration, registry and weight loading: what is accepted, and the errors for what is not."""
from __future__ import annotations

import json
import struct

import pytest
import torch

from tiny_configs import TINY_A, TINY_B, TINY_C
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.models.llama_config import LlamaConfig
from tinyllama_inference_engine_b200.config import architecture_for, load_model_config, registered_architectures
from tinyllama_inference_engine_b200.errors import ConfigError, EngineError, FormatError, WeightError
from tinyllama_inference_engine_b200.models import expected_tensors
from tinyllama_inference_engine_b200.weights import SafetensorsFile, WeightStore, write_random_model, write_safetensors


def test_config_reads_its_own_keys_and_derives_sizes():
    a = LlamaConfig.from_dict(TINY_A)
    assert (a.head_dim, a.kv_dim, a.q_dim, a.query_groups) == (16, 32, 64, 2)
    c = LlamaConfig.from_dict(TINY_C)
    assert c.head_dim == 48 and c.q_dim == 144 and c.query_groups == 1  # head_dim given, not hidden / heads
    minimal = {k: TINY_A[k] for k in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "max_position_embeddings", "vocab_size", "rms_norm_eps")}
    m = LlamaConfig.from_dict(minimal)
    assert m.num_key_value_heads == 4 and m.rope_theta == 10000.0 and not m.tie_word_embeddings
    assert LlamaConfig.from_dict(a.to_dict()) == a
    tinyllama = dict(TINY_A, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, max_position_embeddings=2048, vocab_size=32000)
    t = LlamaConfig.from_dict(tinyllama)
    assert len(expected_tensors(architecture_for(tinyllama).build_spec(t))) == 22 * 9 + 3  # src/model_config.cpp:80


@pytest.mark.parametrize("change,match", [
    ({"hidden_size": None}, "lacks required keys"),
    ({"model_type": "mistral"}, "model_type must be llama"),
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"hidden_size": 66}, "no head_dim"),
    ({"head_dim": 15}, "multiple of 16"),
    ({"head_dim": 40}, "multiple of 16"),
    ({"head_dim": 272}, "up to 256"),
    ({"hidden_act": "gelu"}, "silu"),
    ({"attention_bias": True}, "biases"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"rms_norm_eps": 0.0}, "positive"),
    ({"vocab_size": 0}, ">= 1"),
    ({"num_hidden_layers": "2"}, "integer"),
])
def test_config_refuses(change, match):
    data = dict(TINY_A)
    for key, value in change.items():
        if value is None:
            data.pop(key)
        else:
            data[key] = value
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict(data)


def test_registry_chooses_by_name(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    assert architecture_for({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    assert architecture_for({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError, match="no registered architecture"):
        architecture_for({"architectures": ["SomethingElse"], "model_type": "llama"})
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="invalid model config JSON"):
        load_model_config(tmp_path)
    with pytest.raises(EngineError, match="unable to open"):
        load_model_config(tmp_path / "nowhere")


def test_engine_config():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16"
    assert EngineConfig(page_size=32, max_cache_tokens=100).num_pages == 3
    for bad in (dict(dtype="float16"), dict(page_size=24), dict(page_size=64, max_cache_tokens=10), dict(max_requests=0)):
        with pytest.raises(ConfigError):
            EngineConfig(**bad)


def test_random_mode_is_seeded_and_keeps_bfloat16(tmp_path):
    config = LlamaConfig.from_dict(TINY_B)
    one = write_random_model(tmp_path / "one", config, seed=2)
    two = write_random_model(tmp_path / "two", config, seed=2)
    three = write_random_model(tmp_path / "three", config, seed=3)
    assert (one / "model.safetensors").read_bytes() == (two / "model.safetensors").read_bytes()
    assert (one / "model.safetensors").read_bytes() != (three / "model.safetensors").read_bytes()
    assert json.loads((one / "config.json").read_text())["tie_word_embeddings"] is True
    architecture, loaded = load_model_config(one)
    spec = architecture.build_spec(loaded)
    store = WeightStore.load(one, expected_tensors(spec))
    assert not store.has("lm_head.weight")  # tied: the head has no tensor of its own
    w = store.get("model.layers.2.mlp.down_proj.weight")
    assert w.dtype == torch.bfloat16 and tuple(w.shape) == (192, 512)
    assert abs(float(w.float().std()) - 0.02) < 0.002
    n = store.get("model.norm.weight", torch.float32)
    assert n.dtype == torch.float32 and abs(float(n.mean()) - 1.0) < 0.05


def test_storage_rule_32_bit_stays_and_integers_become_int32(tmp_path):
    from tinyllama_inference_engine_b200.parts.spec import TensorSpec

    write_safetensors(tmp_path / "model.safetensors", {
        "half": torch.ones(2, 3, dtype=torch.float16), "brain": torch.ones(2, 3, dtype=torch.bfloat16),
        "single": torch.ones(4, dtype=torch.float32), "table": torch.arange(5, dtype=torch.int64),
    })
    store = WeightStore.load(tmp_path, [TensorSpec("half", (2, 3)), TensorSpec("brain", (2, 3)), TensorSpec("single", (4,)), TensorSpec("table", (5,), integer=True)])
    assert store.get("half").dtype == torch.float16 and store.get("brain").dtype == torch.bfloat16   # each as the file has it
    assert store.get("half", torch.float32).dtype == torch.float32
    assert store.get("single").dtype == torch.float32 and store.get("table").dtype == torch.int32


def test_a_float16_checkpoint_widens_exactly_for_the_32_bit_engine(tmp_path):
    """A float16 value has three more mantissa bits than bfloat16 keeps: the store must hand the 32-bit path the value itself
    (the reference's GPU checkpoints are float16, scripts/convert_model_fp16.py:23-67)."""
    folder = write_random_model(tmp_path / "half", TINY_A, seed=0, storage_dtype="float16")
    architecture, loaded = load_model_config(folder)
    store = WeightStore.load(folder, expected_tensors(architecture.build_spec(loaded)))
    file = SafetensorsFile(folder / "model.safetensors")
    name = "model.layers.0.self_attn.q_proj.weight"
    raw = file.tensor(name).clone()
    file.close()
    assert raw.dtype == torch.float16
    assert torch.equal(store.get(name, torch.float32), raw.float())
    assert not torch.equal(raw.float(), raw.bfloat16().float())          # so rounding to bfloat16 would have been visible
    assert torch.equal(store.get(name, torch.bfloat16), raw.bfloat16())  # the bfloat16 engine rounds, once


def test_a_tied_checkpoint_may_store_the_head_as_well(tmp_path):
    folder = write_random_model(tmp_path / "tied", TINY_B, seed=2)
    file = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: file.tensor(name).clone() for name in file.names()}
    file.close()
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(folder / "model.safetensors", tensors)
    architecture, loaded = load_model_config(folder)
    store = WeightStore.load(folder, expected_tensors(architecture.build_spec(loaded)))   # not "unexpected"
    assert store.has("lm_head.weight")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = LlamaConfig.from_dict(TINY_A)
    folder = write_random_model(tmp_path / "m", config, seed=0)
    file = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: file.tensor(name).clone() for name in file.names()}
    file.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)
    write_safetensors(folder / "model.safetensors", tensors)
    spec = architecture_for(TINY_A).build_spec(config)
    with pytest.raises(WeightError) as caught:
        WeightStore.load(folder, expected_tensors(spec))
    message = str(caught.value)
    assert "missing (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in message
    assert "unexpected (1): model.layers.0.self_attn.q_proj.bias" in message
    assert "model.layers.0.self_attn.k_proj.weight: file has [64, 64], model needs [32, 64]" in message


def test_malformed_files_are_refused(tmp_path):
    path = tmp_path / "model.safetensors"
    with pytest.raises(EngineError, match="no model.safetensors"):
        WeightStore.load(tmp_path, [])
    path.write_bytes(b"\x01\x02")
    with pytest.raises(FormatError, match="truncated"):
        SafetensorsFile(path)
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(FormatError, match="exceeds the file"):
        SafetensorsFile(path)
    path.write_bytes(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(FormatError, match="malformed JSON"):
        SafetensorsFile(path)
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(FormatError, match="outside the file"):
        SafetensorsFile(path)
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(FormatError, match="its shape needs 16"):
        SafetensorsFile(path)
    header = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}, "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 12)
    with pytest.raises(FormatError, match="overlap"):
        SafetensorsFile(path)
    header = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 4)
    with pytest.raises(EngineError, match="unsupported dtype"):
        SafetensorsFile(path)


def test_weights_can_be_pinned_by_their_sha256(tmp_path):
    """The reference refuses a checkpoint whose digest differs from the pinned one with checksum_mismatch (src/weight_store.cpp:150-190)."""
    import hashlib

    from tinyllama_inference_engine_b200.weights import verify_weights, weights_sha256

    folder = write_random_model(tmp_path / "m", TINY_A, seed=0)
    digest = hashlib.sha256((folder / "model.safetensors").read_bytes()).hexdigest()
    assert weights_sha256(folder) == digest and verify_weights(folder, digest.upper()) == digest
    with pytest.raises(EngineError, match="expected") as caught:
        verify_weights(folder, "0" * 64)
    assert caught.value.code == "checksum_mismatch"
    with pytest.raises(EngineError, match="64 hexadecimal"):
        verify_weights(folder, "abc")
    with pytest.raises(EngineError, match="no model.safetensors"):
        weights_sha256(tmp_path)
    # a sharded folder: the digest of the shards' digests, in the order of their names
    file = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: file.tensor(name).clone() for name in file.names()}
    file.close()
    names = sorted(tensors)
    shards = {"model-00001-of-00002.safetensors": names[: len(names) // 2], "model-00002-of-00002.safetensors": names[len(names) // 2 :]}
    sharded = tmp_path / "sharded"
    sharded.mkdir()
    (sharded / "config.json").write_text((folder / "config.json").read_text())
    for shard, members in shards.items():
        write_safetensors(sharded / shard, {name: tensors[name] for name in members})
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {name: shard for shard, members in shards.items() for name in members}}))
    combined = hashlib.sha256(b"".join(hashlib.sha256((sharded / shard).read_bytes()).digest() for shard in sorted(shards))).hexdigest()
    assert weights_sha256(sharded) == combined
