"""Weights: the safetensors container, loading by name, the one error for every mismatch, and
the random-weights mode."""
import json
import os

import pytest
import torch

import helpers
import vipera_rs_b200  # noqa: F401
from vipera_rs_b200 import errors, parts  # noqa: F401
from vipera_rs_b200.config import load_config
from vipera_rs_b200.engine.loader import write_random_model
from vipera_rs_b200.parts import model_schema
from vipera_rs_b200.weights import (RandomSource, SafetensorsFile, SafetensorsSource, check_source, to_run_dtype,
                                    write_safetensors)


def test_container_round_trip_and_agrees_with_the_safetensors_library(tmp_path):
    tensors = {
        "a": torch.randn(3, 5),
        "b.bf16": torch.randn(7).bfloat16(),
        "table": torch.arange(12, dtype=torch.int32).view(3, 4),
        "half": torch.randn(2, 2).half(),
    }
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors.items(), metadata={"note": "t"})
    mine = SafetensorsFile(path)
    assert sorted(mine.names()) == sorted(tensors)
    for name, tensor in tensors.items():
        assert mine.shape(name) == tuple(tensor.shape) and mine.dtype(name) == tensor.dtype
        assert torch.equal(mine.get(name), tensor)
    from safetensors.torch import load_file, save_file

    theirs = load_file(path)                       # our writer, their reader
    for name, tensor in tensors.items():
        assert torch.equal(theirs[name], tensor)
    other = str(tmp_path / "y.safetensors")
    save_file(tensors, other)                      # their writer, our reader
    for name, tensor in tensors.items():
        assert torch.equal(SafetensorsFile(other).get(name), tensor)


def test_malformed_files_are_parse_errors(tmp_path):
    short = tmp_path / "short.safetensors"
    short.write_bytes(b"abc")
    with pytest.raises(errors.ParseError):
        SafetensorsFile(str(short))
    lying = tmp_path / "lying.safetensors"
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 400]}}).encode()
    lying.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 16)
    with pytest.raises(errors.ParseError):
        SafetensorsFile(str(lying))
    with pytest.raises(errors.IoError):
        SafetensorsFile(str(tmp_path / "absent.safetensors"))


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    folder = str(tmp_path / "m")
    write_random_model(folder, helpers.TINY_B, seed=3, dtype="bfloat16")
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    arch, config = load_config(folder)
    schema = model_schema(arch.model_spec(config))
    source = SafetensorsSource(folder)
    check_source(schema, source)                   # nothing missing, nothing extra, shapes right
    assert source.stored_dtype("model.layers.0.self_attn.q_proj.weight") == torch.bfloat16
    assert source.stored_dtype("model.norm.weight") == torch.float32   # norms are stored in 32-bit
    norm = source.get("model.norm.weight")
    assert abs(float(norm.mean()) - 1.0) < 0.01 and 0.005 < float(norm.std()) < 0.02
    weight = source.get("model.layers.1.mlp.down_proj.weight").float()
    assert abs(float(weight.mean())) < 1e-3 and 0.018 < float(weight.std()) < 0.022
    # the same seed gives the same values whatever the order of asking; another seed does not
    again = RandomSource(schema, 3, torch.bfloat16)
    assert torch.equal(again.get("lm_head.weight"), source.get("lm_head.weight"))
    assert not torch.equal(RandomSource(schema, 4, torch.bfloat16).get("lm_head.weight"), source.get("lm_head.weight"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = str(tmp_path / "m")
    write_random_model(folder, helpers.TINY_A, seed=1, dtype="float32")
    source = SafetensorsSource(folder)
    tensors = {name: source.get(name) for name in source.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.layers.0.self_attn.k_proj.bias"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(32)
    tensors["lm_head.weight"] = torch.zeros(512, 256)              # tied model: an output matrix is unexpected
    tensors["model.norm.weight"] = torch.zeros(255)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
    arch, config = load_config(folder)
    with pytest.raises(errors.UnsupportedError) as info:
        check_source(model_schema(arch.model_spec(config)), SafetensorsSource(folder))
    error = info.value
    assert error.missing == ["model.layers.0.self_attn.k_proj.bias", "model.layers.1.mlp.up_proj.weight"]
    assert error.unexpected == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(error.wrong_shape) == 1 and "model.norm.weight" in error.wrong_shape[0] and "[255]" in error.wrong_shape[0]
    text = str(error)
    assert "missing (2)" in text and "unexpected (2)" in text and "wrong shape (1)" in text
    assert error.exit_code == 2


def test_the_references_tensor_names_are_accepted(tmp_path):
    """A file that names its tensors as the reference's files do (token_embd.weight,
    blk.3.attn_q.bias, ...) loads like one with the usual names; a name that is neither still
    shows up as unexpected."""
    from vipera_rs_b200.weights import AliasedSource

    folder = str(tmp_path / "m")
    write_random_model(folder, helpers.TINY_B, seed=5, dtype="float32")
    source = SafetensorsSource(folder)
    renames = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
               "lm_head.weight": "output.weight"}
    layer = {"input_layernorm.weight": "attn_norm.weight", "self_attn.q_proj.weight": "attn_q.weight",
             "self_attn.q_proj.bias": "attn_q.bias", "self_attn.k_proj.weight": "attn_k.weight",
             "self_attn.k_proj.bias": "attn_k.bias", "self_attn.v_proj.weight": "attn_v.weight",
             "self_attn.v_proj.bias": "attn_v.bias", "self_attn.o_proj.weight": "attn_output.weight",
             "post_attention_layernorm.weight": "ffn_norm.weight", "mlp.gate_proj.weight": "ffn_gate.weight",
             "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight"}
    tensors = {}
    for name in source.names():
        new = renames.get(name)
        if new is None:
            _, _, index, tail = name.split(".", 3)
            new = f"blk.{index}.{layer[tail]}"
        tensors[new] = source.get(name)
    tensors["blk.0.attn_sinks"] = torch.zeros(3)
    renamed = str(tmp_path / "renamed")
    os.makedirs(renamed)
    with open(os.path.join(folder, "config.json")) as src, open(os.path.join(renamed, "config.json"), "w") as dst:
        dst.write(src.read())
    write_safetensors(os.path.join(renamed, "model.safetensors"), tensors.items())
    arch, config = load_config(renamed)
    schema = model_schema(arch.model_spec(config))
    seen = AliasedSource(SafetensorsSource(renamed), arch.tensor_alias)
    with pytest.raises(errors.UnsupportedError) as info:
        check_source(schema, seen)
    assert info.value.missing == [] and info.value.wrong_shape == [] and info.value.unexpected == ["blk.0.attn_sinks"]
    assert torch.equal(seen.get("model.layers.2.self_attn.k_proj.bias"), source.get("model.layers.2.self_attn.k_proj.bias"))
    assert torch.equal(seen.get("lm_head.weight"), source.get("lm_head.weight"))


def test_run_dtypes():
    assert to_run_dtype(torch.zeros(2, dtype=torch.bfloat16), torch.bfloat16).dtype == torch.bfloat16
    assert to_run_dtype(torch.zeros(2, dtype=torch.float16), torch.bfloat16).dtype == torch.bfloat16
    assert to_run_dtype(torch.zeros(2, dtype=torch.float32), torch.bfloat16).dtype == torch.float32  # 32-bit stays
    assert to_run_dtype(torch.zeros(2, dtype=torch.bfloat16), torch.float32).dtype == torch.float32
    assert to_run_dtype(torch.zeros(2, dtype=torch.int64), torch.bfloat16).dtype == torch.int32


def test_no_device_means_a_loud_failure():
    """There is no CPU path: asking the engine to run without a CUDA device raises."""
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from vipera_rs_b200.kernels import ops

    with pytest.raises(errors.InternalError):
        ops.embed(torch.zeros(4, 8), torch.zeros(2, dtype=torch.int32), torch.zeros(2, 8))
