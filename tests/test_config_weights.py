"""Configuration, registry, safetensors container, weight checking and the
random-weights mode.  No GPU."""

from __future__ import annotations

import json
import struct

import pytest
import torch

from conftest import TINY
from litinfer_b200.config import (ConfigError, Qwen2Config, config_from_dict, load_config, register_architecture,
                                  supported_architectures)
from litinfer_b200.models import DecoderModel, declared_params
from litinfer_b200.weights import (ParamSpec, SafetensorsError, WeightError, iter_tensors, load_tensors, random_tensor,
                                   read_header, write_file, write_model_folder)


# --------------------------------------------------------------------------
# configuration
# --------------------------------------------------------------------------

def test_keys_and_defaults_follow_the_reference_loader():
    # defaults of python/llaisys/models/qwen2.py:266-282
    c = Qwen2Config.from_dict(dict(architectures=["Qwen2ForCausalLM"], hidden_size=96, num_attention_heads=3, num_hidden_layers=2,
                                   intermediate_size=64, vocab_size=50, max_position_embeddings=32))
    assert c.num_key_value_heads == 3 and c.head_dim == 32
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.eos_token_ids == () and not c.tie_word_embeddings and c.sliding_window is None
    c = Qwen2Config.from_dict(dict(TINY["B"], eos_token_id=[7, 9]))
    assert c.eos_token_ids == (7, 9)
    assert Qwen2Config.from_dict(dict(TINY["B"], eos_token_id=5)).eos_token_ids == (5,)


def test_every_size_comes_from_the_configuration():
    for name, cfg in TINY.items():
        c = config_from_dict(cfg)
        spec = c.to_model_spec()
        assert len(spec.blocks) == cfg["num_hidden_layers"] and spec.vocab_size == cfg["vocab_size"]
        m = spec.blocks[0].part("mixer")
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"])
        assert m["position"]["theta"] == cfg["rope_theta"]
        assert spec.blocks[0].part("mixer_norm")["eps"] == cfg["rms_norm_eps"]
        assert spec.blocks[0].part("feed_forward")["intermediate_size"] == cfg["intermediate_size"]
        assert spec.tie_word_embeddings == cfg["tie_word_embeddings"]
    # the window applies from max_window_layers on
    spec = config_from_dict(TINY["B"]).to_model_spec()
    assert [b.part("mixer")["window"] for b in spec.blocks] == [None, 24, 24]


@pytest.mark.parametrize("change,fragment", [
    (dict(num_key_value_heads=2), "not a multiple"),
    (dict(head_dim=15), "even"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"type": "linear", "factor": 2}), "rope_scaling"),
    (dict(vocab_size=0), "vocab_size"),
    (dict(use_sliding_window=True, sliding_window=None), "sliding_window"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
])
def test_bad_configurations_are_refused(change, fragment):
    with pytest.raises(ConfigError, match=fragment):
        config_from_dict(dict(TINY["B"], **change))


def test_registry_names_what_it_supports(tmp_path):
    assert "Qwen2ForCausalLM" in supported_architectures()
    with pytest.raises(ConfigError, match="LlamaForCausalLM.*supported.*Qwen2ForCausalLM"):
        config_from_dict(dict(TINY["A"], architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY["A"].items() if k != "architectures"})
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path)

    class Other(Qwen2Config):
        ARCHITECTURE = "ToyForCausalLM"

    register_architecture("ToyForCausalLM", Other)
    try:
        assert isinstance(config_from_dict(dict(TINY["A"], architectures=["ToyForCausalLM"])), Other)
    finally:
        from litinfer_b200.config import registry
        registry._ARCHITECTURES.pop("ToyForCausalLM")
    with pytest.raises(TypeError):
        register_architecture("Broken", object)


# --------------------------------------------------------------------------
# safetensors container
# --------------------------------------------------------------------------

def test_container_round_trip_of_every_kept_dtype(tmp_path):
    tensors = {
        "a.f32": torch.randn(3, 5),
        "b.bf16": torch.randn(4, 2).to(torch.bfloat16),
        "c.f16": torch.randn(7).to(torch.float16),
        "d.i32": torch.arange(6, dtype=torch.int32).reshape(2, 3),
        "e.i64": torch.arange(4, dtype=torch.int64),
    }
    write_file(tmp_path / "t.safetensors", tensors)
    header, base = read_header(tmp_path / "t.safetensors")
    assert list(header) == list(tensors) and base % 8 == 0
    back = dict(iter_tensors(tmp_path / "t.safetensors"))
    for k, v in tensors.items():
        assert back[k].dtype == v.dtype and torch.equal(back[k], v)


def test_corrupt_containers_are_refused(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        read_header(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        read_header(p)
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="JSON"):
        read_header(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="data_offsets"):
        read_header(p)
    hdr = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="dtype"):
        read_header(p)


# --------------------------------------------------------------------------
# weights
# --------------------------------------------------------------------------

def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_model_folder(tmp_path / "m", dict(TINY["B"], attention_bias=True), seed=3)     # the key given: biases are required
    tensors = dict(iter_tensors(d / "model.safetensors"))
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(5, 7)
    tensors["model.layers.9.extra.weight"] = torch.zeros(2)
    tensors["model.embed_tokens.weight"] = torch.zeros(389, 96, dtype=torch.int32)
    write_file(d / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        DecoderModel.from_dir(d, "float32", "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.mlp.gate_proj.weight", (5, 7), (272, 96))]
    assert [n for n, _, _ in err.wrong_dtype] == ["model.embed_tokens.weight"]
    msg = str(err)
    for part in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "is [5, 7], expected [272, 96]"):
        assert part in msg


def test_the_head_follows_the_file(tmp_path):
    """LitInfer uses a stored lm_head and ties to the embedding when there is none, whatever config.json says
    (python/llaisys/models/qwen2.py:143-146, 196-199)."""
    cfg = dict(TINY["A"])                                  # tied: random mode writes no lm_head
    d = write_model_folder(tmp_path / "m", cfg, seed=3)
    tensors = dict(iter_tensors(d / "model.safetensors"))
    assert "lm_head.weight" not in tensors
    m = DecoderModel.from_dir(d, "float32", "cpu")
    assert m.lm_head is m.embedding and m.head_is_tied     # the table itself
    # a config that says "untied" over a file without a head: tied all the same
    cfg["tie_word_embeddings"] = False
    (d / "config.json").write_text(json.dumps(cfg))
    m = DecoderModel.from_dir(d, "float32", "cpu")
    assert m.lm_head is m.embedding and m.head_is_tied
    # a tied config over a file that stores a head: the stored one is used
    cfg["tie_word_embeddings"] = True
    (d / "config.json").write_text(json.dumps(cfg))
    head = torch.randn(cfg["vocab_size"], cfg["hidden_size"])
    write_file(d / "model.safetensors", dict(tensors, **{"lm_head.weight": head}))
    m = DecoderModel.from_dir(d, "float32", "cpu")
    assert torch.equal(m.lm_head, head) and not m.head_is_tied
    # a head of the wrong shape is still an error
    write_file(d / "model.safetensors", dict(tensors, **{"lm_head.weight": head[:, :5].contiguous()}))
    with pytest.raises(WeightError, match="wrong shapes.*lm_head.weight"):
        DecoderModel.from_dir(d, "float32", "cpu")


def test_the_other_names_of_litinfers_loader_are_accepted(tmp_path):
    """transformer.wte.weight, model.lm_head.weight, transformer.ln_f.weight (python/llaisys/models/qwen2.py:139-149)."""
    d = write_model_folder(tmp_path / "m", dict(TINY["B"]), seed=3)
    tensors = dict(iter_tensors(d / "model.safetensors"))
    want = DecoderModel.from_dir(d, "float32", "cpu")
    renamed = {"model.embed_tokens.weight": "transformer.wte.weight", "lm_head.weight": "model.lm_head.weight",
               "model.norm.weight": "transformer.ln_f.weight"}
    write_file(d / "model.safetensors", {renamed.get(k, k): v for k, v in tensors.items()})
    got = DecoderModel.from_dir(d, "float32", "cpu")
    assert torch.equal(got.embedding, want.embedding) and torch.equal(got.lm_head, want.lm_head)
    assert torch.equal(got.final_norm.weight, want.final_norm.weight)
    # both names of one tensor at once: the second is unexpected
    write_file(d / "model.safetensors", dict(tensors, **{"transformer.wte.weight": tensors["model.embed_tokens.weight"]}))
    with pytest.raises(WeightError, match="unexpected tensors.*transformer.wte.weight"):
        DecoderModel.from_dir(d, "float32", "cpu")


def test_biases_follow_the_file_when_the_config_does_not_say(tmp_path):
    """Qwen2's config.json has no attention_bias key and LitInfer's loader does not require the q/k/v biases
    (python/llaisys/models/qwen2.py:220-230); a missing bias is none (src/llaisys/ops.cc:27-29)."""
    cfg = dict(TINY["B"])
    assert "attention_bias" not in cfg
    d = write_model_folder(tmp_path / "m", cfg, seed=3)
    tensors = dict(iter_tensors(d / "model.safetensors"))
    assert "model.layers.1.self_attn.k_proj.bias" in tensors                  # random mode makes them
    full = DecoderModel.from_dir(d, "float32", "cpu")
    nh, nkv, dh = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    # one bias gone: zeros in its place, the others kept
    write_file(d / "model.safetensors", {k: v for k, v in tensors.items() if k != "model.layers.1.self_attn.k_proj.bias"})
    m = DecoderModel.from_dir(d, "float32", "cpu")
    b = m.blocks[1].mixer.qkv.bias
    assert torch.equal(b[:nh * dh], full.blocks[1].mixer.qkv.bias[:nh * dh])
    assert torch.count_nonzero(b[nh * dh:(nh + nkv) * dh]) == 0
    # all gone: no bias at all
    write_file(d / "model.safetensors", {k: v for k, v in tensors.items() if not k.endswith("_proj.bias")})
    m = DecoderModel.from_dir(d, "float32", "cpu")
    assert all(blk.mixer.qkv.bias is None for blk in m.blocks)
    # attention_bias false in the config: a stored bias is unexpected
    (d / "config.json").write_text(json.dumps(dict(cfg, attention_bias=False)))
    write_file(d / "model.safetensors", tensors)
    with pytest.raises(WeightError, match="unexpected tensors"):
        DecoderModel.from_dir(d, "float32", "cpu")


def test_device_dtypes_by_role(tmp_path):
    d = write_model_folder(tmp_path / "m", dict(TINY["A"]), seed=3, store_dtype="bfloat16")
    m = DecoderModel.from_dir(d, "bfloat16", "cpu")
    att = m.blocks[0].mixer
    assert m.embedding.dtype == torch.bfloat16 and att.qkv.weight.dtype == torch.bfloat16
    assert att.qkv.bias.dtype == torch.float32 and m.final_norm.weight.dtype == torch.float32     # vectors are 32-bit
    assert att.qkv.weight.shape == ((4 + 2 * 2) * 16, 64)                                           # q | k | v fused
    m32 = DecoderModel.from_dir(d, "float32", "cpu")
    assert m32.embedding.dtype == torch.float32
    assert torch.equal(m32.embedding, m.embedding.float())
    # integer tables become int32; a tensor stored in 32-bit and marked keep stays as stored
    write_file(tmp_path / "t.safetensors", {"ids": torch.arange(4, dtype=torch.int64), "k": torch.ones(2, dtype=torch.float32)})
    (tmp_path / "t").mkdir()
    (tmp_path / "t.safetensors").rename(tmp_path / "t" / "model.safetensors")
    got = load_tensors(tmp_path / "t", [ParamSpec("ids", (4,), role="table"), ParamSpec("k", (2,), role="keep")], torch.bfloat16, "cpu")
    assert got["ids"].dtype == torch.int32 and got["k"].dtype == torch.float32


def test_random_weights_mode(tmp_path):
    d1 = write_model_folder(tmp_path / "a", dict(TINY["B"]), seed=11)
    d2 = write_model_folder(tmp_path / "b", dict(TINY["B"]), seed=11)
    d3 = write_model_folder(tmp_path / "c", dict(TINY["B"]), seed=12)
    t1, t2, t3 = (dict(iter_tensors(d / "model.safetensors")) for d in (d1, d2, d3))
    assert sorted(t1) == sorted(p.name for p in declared_params(config_from_dict(TINY["B"]).to_model_spec()))
    assert all(torch.equal(t1[k], t2[k]) for k in t1)
    assert not torch.equal(t1["lm_head.weight"], t3["lm_head.weight"])
    w = t1["model.layers.0.mlp.down_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    g = t1["model.layers.2.input_layernorm.weight"]
    assert abs(float(g.mean()) - 1.0) < 0.05 and 0.05 < float(g.std()) < 0.15
    assert json.loads((d1 / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]
    # a tensor's values depend on the seed and its own name only
    p = ParamSpec("model.layers.0.mlp.down_proj.weight", tuple(w.shape))
    assert torch.equal(random_tensor(p, 11), w)
    # the folder loads back through the name path
    m = DecoderModel.from_dir(d1, "float32", "cpu")
    assert torch.equal(m.blocks[0].feed_forward.down.weight, w)


def test_the_generator_of_random_weights_against_its_plain_restatement():
    """The package's NumPy path (what writes model folders) gives, bit for bit, what the element-at-a-time restatement in
    tests/plain_random.py gives; the series inside it are accurate; a tensor depends on the seed and its own name only."""
    import numpy as np

    import plain_random as PR
    from litinfer_b200.weights.random_init import tensor_key

    assert tensor_key(11, "model.norm.weight") == PR.tensor_key(11, "model.norm.weight")
    for name, shape, init, std in (("a.weight", (7, 9), "normal", 0.02), ("b.weight", (64,), "ones_normal", 0.02), ("c", (1001,), "normal", 0.5)):
        got = random_tensor(ParamSpec(name, shape, init=init, std=std), 11).numpy().reshape(-1)
        mean, sd = (1.0, 0.1) if init == "ones_normal" else (0.0, std)
        want = PR.normal(PR.tensor_key(11, name), got.size, mean, sd)
        assert got.dtype == np.float32 and np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
    ids = random_tensor(ParamSpec("t", (33,), role="table", init="randint"), 11)
    assert ids.dtype == torch.int32 and np.array_equal(ids.numpy(), PR.randint(PR.tensor_key(11, "t"), 33, 1 << 15))
    # a large tensor is drawn in slabs on several threads: the same values as in one piece
    from litinfer_b200.weights.random_init import _host_normal, normal_pairs

    n = (1 << 20) + 3
    whole = _host_normal(5, n, 0.0, 1.0).numpy()
    piece = normal_pairs(5, 0, (n + 1) // 2).reshape(-1)[:n]
    assert np.array_equal(whole, piece)
    assert abs(float(whole.mean())) < 0.005 and abs(float(whole.std()) - 1.0) < 0.005 and 4.0 < float(np.abs(whole).max()) < 6.5
    assert abs(float((np.abs(whole) > 2.0).mean()) - 0.0455) < 0.002
    worst_ln, worst_sc = PR.series_errors()
    assert worst_ln < 2e-6 and worst_sc < 3e-7, (worst_ln, worst_sc)
