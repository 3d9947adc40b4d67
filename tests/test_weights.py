"""SafeTensors reading and writing, lookup by name, and the one error that lists what is wrong (no GPU)."""
import json
import os
import struct

import pytest
import torch

import helpers
from llama_rs_metal_b200.engine.model import DecoderModel
from llama_rs_metal_b200.errors import InvalidError, UnsupportedError, WeightError
from llama_rs_metal_b200.registry import find_architecture
from llama_rs_metal_b200.runtime import Runtime
from llama_rs_metal_b200.weights import (load_tensors, open_checkpoint, random_tensors,
                                         write_model_folder, write_safetensors)

CPU = Runtime(torch.device("cpu"), torch.float32)


def specs_of(name):
    root = helpers.TINY[name]["config"]
    arch = find_architecture(root)
    plan = arch.plan(arch.config_class.from_dict(root))
    return plan, DecoderModel(plan, CPU).tensor_specs()


def test_random_mode_writes_a_folder_the_safetensors_library_reads(model_dirs):
    from safetensors import safe_open
    plan, specs = specs_of("B")
    with safe_open(os.path.join(model_dirs["B"], "model.safetensors"), framework="pt") as handle:
        assert set(handle.keys()) == set(specs)
        for name, spec in specs.items():
            t = handle.get_tensor(name)
            assert tuple(t.shape) == spec.shape and t.dtype == torch.bfloat16
    with open(os.path.join(model_dirs["B"], "config.json")) as handle:
        assert json.load(handle)["num_hidden_layers"] == 3


def test_own_reader_agrees_with_the_library(model_dirs):
    from safetensors import safe_open
    entries = open_checkpoint(model_dirs["A"])
    with safe_open(os.path.join(model_dirs["A"], "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            assert torch.equal(entries[name].load(), handle.get_tensor(name))


def test_random_tensors_do_not_depend_on_order_or_company():
    _, specs = specs_of("A")
    full = random_tensors(specs, seed=5)
    name = "model.layers.1.mlp.up_proj.weight"
    alone = random_tensors({name: specs[name]}, seed=5)
    assert torch.equal(full[name], alone[name])
    assert not torch.equal(full[name], random_tensors({name: specs[name]}, seed=6)[name])
    assert torch.all(full["model.norm.weight"] == 1.0)


def test_storage_precision_is_kept(tmp_path):
    _, specs = specs_of("A")
    tensors = random_tensors(specs, seed=1)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()  # one tensor stored in 32-bit
    write_model_folder(str(tmp_path), helpers.TINY["A"]["config"], tensors)
    loaded = load_tensors(str(tmp_path), specs)
    assert loaded["model.norm.weight"].dtype == torch.float32
    assert loaded["model.embed_tokens.weight"].dtype == torch.bfloat16
    widened = load_tensors(str(tmp_path), specs, float32=True)
    assert all(t.dtype == torch.float32 for t in widened.values())
    assert torch.equal(widened["model.embed_tokens.weight"], tensors["model.embed_tokens.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    _, specs = specs_of("A")
    tensors = random_tensors(specs, seed=1)
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    write_model_folder(str(tmp_path), helpers.TINY["A"]["config"], tensors)
    with pytest.raises(WeightError) as info:
        load_tensors(str(tmp_path), specs)
    err = info.value
    assert err.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert err.wrong_shape == [("model.layers.1.self_attn.k_proj.weight", (32, 64), (16, 64))]
    text = str(err)
    assert "missing tensors: model.layers.0.mlp.up_proj.weight, model.norm.weight" in text
    assert "unexpected tensors: model.layers.0.self_attn.q_norm.weight" in text
    assert "model.layers.1.self_attn.k_proj.weight: expected [32, 64], got [16, 64]" in text


def test_tied_model_ignores_a_saved_head(tmp_path):
    plan, specs = specs_of("A")  # tied
    tensors = random_tensors(specs, seed=1)
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    write_model_folder(str(tmp_path), helpers.TINY["A"]["config"], tensors)
    loaded = load_tensors(str(tmp_path), specs, ignored=plan.ignored_names)
    assert "lm_head.weight" not in loaded and loaded.unexpected == ()
    with pytest.raises(WeightError):
        load_tensors(str(tmp_path), specs, strict=True)  # without the plan's ignore list it is unexpected


def test_unknown_tensors_are_skipped_and_listed(tmp_path):
    """A stored name no part asked for is no error by itself (crates/model-format/src/mlx/mod.rs:41-43
    skips unknown names, e.g. the other towers of a multimodal export): it is left on disk and
    reported; `strict` turns it into the one error."""
    _, specs = specs_of("A")
    tensors = {"language_model." + n: t for n, t in random_tensors(specs, seed=1).items()}
    tensors["vision_tower.patch_embed.weight"] = torch.zeros(8, 3, dtype=torch.bfloat16)
    tensors["language_model.model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    write_model_folder(str(tmp_path), helpers.TINY["A"]["config"], tensors)
    loaded = load_tensors(str(tmp_path), specs)
    assert set(loaded) == set(specs)
    assert loaded.unexpected == ("model.layers.0.self_attn.rotary_emb.inv_freq", "vision_tower.patch_embed.weight")
    with pytest.raises(WeightError) as info:
        load_tensors(str(tmp_path), specs, strict=True)
    assert info.value.unexpected == list(loaded.unexpected) and not info.value.missing


def test_language_model_prefixes_are_stripped(tmp_path):
    _, specs = specs_of("A")
    tensors = {"language_model." + n: t for n, t in random_tensors(specs, seed=1).items()}
    write_model_folder(str(tmp_path), helpers.TINY["A"]["config"], tensors)
    assert set(load_tensors(str(tmp_path), specs)) == set(specs)


def test_sharded_checkpoint_and_its_errors(tmp_path):
    _, specs = specs_of("A")
    tensors = random_tensors(specs, seed=1)
    names = sorted(tensors)
    halves = {"model-00001-of-00002.safetensors": names[:7], "model-00002-of-00002.safetensors": names[7:]}
    weight_map = {}
    for shard, members in halves.items():
        write_safetensors(str(tmp_path / shard), {n: tensors[n] for n in members})
        weight_map.update({n: shard for n in members})
    index = tmp_path / "model.safetensors.index.json"
    index.write_text(json.dumps({"weight_map": weight_map}))
    (tmp_path / "config.json").write_text(json.dumps(helpers.TINY["A"]["config"]))
    loaded = load_tensors(str(tmp_path), specs)
    assert all(torch.equal(loaded[n], tensors[n]) for n in names)

    bad = dict(weight_map)
    bad[names[0]] = "model-00002-of-00002.safetensors"  # the index assigns it to the wrong shard
    index.write_text(json.dumps({"weight_map": bad}))
    with pytest.raises(InvalidError, match="not assigned to this shard"):
        open_checkpoint(str(tmp_path))
    bad = dict(weight_map, ghost="model-00001-of-00002.safetensors")
    index.write_text(json.dumps({"weight_map": bad}))
    with pytest.raises(InvalidError, match="missing from shards"):
        open_checkpoint(str(tmp_path))
    for unsafe in ("../evil.safetensors", "sub/x.safetensors", "model.bin"):
        index.write_text(json.dumps({"weight_map": {names[0]: unsafe}}))
        with pytest.raises(InvalidError, match="unsafe shard name"):
            open_checkpoint(str(tmp_path))


def test_truncated_and_missing_files(tmp_path):
    with pytest.raises(InvalidError, match="neither model.safetensors"):
        open_checkpoint(str(tmp_path))
    path = tmp_path / "model.safetensors"
    write_safetensors(str(path), {"x": torch.ones(8, 8)})
    blob = path.read_bytes()
    path.write_bytes(blob[:-16])
    with pytest.raises(InvalidError, match="truncated"):
        open_checkpoint(str(tmp_path))
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(InvalidError, match="truncated or oversized"):
        open_checkpoint(str(tmp_path))
    path.write_bytes(b"\x01\x02")
    with pytest.raises(InvalidError, match="truncated"):
        open_checkpoint(str(tmp_path))


def test_unsupported_dtype_is_named(tmp_path):
    header = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 4)
    with pytest.raises(UnsupportedError, match="F8_E4M3"):
        open_checkpoint(str(tmp_path))
