"""Configuration, registry and weight loading (CPU)."""
import json
import struct

import pytest
import torch

from jllm_serve_b200.config import (ConfigError, Decoder, GqaAttentionSpec, load_config, parse_config,
                                    register_architecture, supported_architectures, unregister_architecture)
from jllm_serve_b200.engine.model import DecoderModel
from jllm_serve_b200.weights import (SafetensorsError, TensorSource, WeightError, compare, load_checked,
                                     write_model_folder, write_safetensors)
from tests.tiny import TINY_A, TINY_B, TINY_C


def test_qwen3_fields_come_from_config_json():
    d = parse_config(TINY_B)
    assert isinstance(d, Decoder)
    assert (d.core.dim, d.core.layers, d.core.vocab, d.core.tied, d.core.norm_eps) == (96, 3, 1000, False, 1e-5)
    a = d.layers[0].mixer
    assert isinstance(a, GqaAttentionSpec)
    assert (a.heads, a.kv_heads, a.head_dim, a.qk_norm, a.bias, a.out_bias, a.window) == (8, 2, 32, True, False, False, 0)
    assert abs(a.scale - 32 ** -0.5) < 1e-9
    assert d.layers[0].feed_forward.hidden == 200 and d.rope_tables[0].theta == 1e6 and d.rope_tables[0].rotary_dim == 32
    assert "heads=8/2 headDim=32" in d.core.description


def test_defaults_follow_the_reference():
    c = dict(model_type="qwen3", hidden_size=64, num_hidden_layers=1, vocab_size=10, num_attention_heads=4,
             intermediate_size=8)
    d = parse_config(c)
    a = d.layers[0].mixer
    assert (a.kv_heads, a.head_dim) == (4, 16)                       # kv heads = heads, head_dim = dim / heads
    assert d.core.norm_eps == 1e-6 and d.rope_tables[0].theta == 10000.0 and d.core.max_positions == 4096
    assert d.core.tied is False and d.core.bos == -1 and d.core.eos == ()
    assert parse_config(dict(c, eos_token_id=[5, 7])).core.eos == (5, 7)
    assert parse_config(dict(c, eos_token_id=5)).core.eos == (5,)


def test_window_rule_and_bias_and_partial_rotary():
    d = parse_config(TINY_C)
    assert [l.mixer.window for l in d.layers] == [0, 40, 40, 40]      # from max_window_layers on
    assert d.layers[0].mixer.bias and d.layers[0].mixer.out_bias      # attention_bias: q, k, v and o_proj
    assert d.rope_tables[0].rotary_dim == 24 and d.rope_tables[0].scaling.kind == "linear"
    no = parse_config(dict(TINY_C, use_sliding_window=False))
    assert all(l.mixer.window == 0 for l in no.layers)                 # sliding_window alone does nothing


@pytest.mark.parametrize("change, word", [
    (dict(num_key_value_heads=3), "num_key_value_heads"), (dict(hidden_act="gelu"), "hidden_act"),
    (dict(mlp_bias=True), "mlp_bias"), (dict(hidden_size=0), "hidden_size"), (dict(head_dim=0), "head_dim"),
    (dict(vocab_size="many"), "vocab_size"), (dict(rope_scaling={"rope_type": "llama3"}), "llama3"),
    (dict(partial_rotary_factor=0.01), "partial_rotary_factor"), (dict(architectures=["LlamaForCausalLM"]), "Llama"),
    (dict(num_experts=8), "num_experts"), (dict(rms_norm_eps="tiny"), "rms_norm_eps"),
    (dict(tie_word_embeddings="yes"), "tie_word_embeddings"), (dict(intermediate_size=0), "intermediate_size"),
])
def test_bad_configs_are_refused_by_key(change, word):
    with pytest.raises(ConfigError, match=word):
        parse_config(dict(TINY_A, **change))


def test_missing_key_and_unknown_architecture():
    c = dict(TINY_A)
    del c["num_hidden_layers"]
    with pytest.raises(ConfigError, match="num_hidden_layers"):
        parse_config(c)
    with pytest.raises(ConfigError, match="supported: .*qwen3"):
        parse_config(dict(TINY_A, model_type="mamba"))
    assert "qwen3" in supported_architectures()


def test_registry_takes_another_architecture():
    def parse(values):
        return parse_config(dict(values, model_type="qwen3"))
    register_architecture("qwen3_twin", parse)
    try:
        assert parse_config(dict(TINY_A, model_type="qwen3_twin")).core.dim == 64
        with pytest.raises(ValueError):
            register_architecture("qwen3_twin", parse)
    finally:
        unregister_architecture("qwen3_twin")


def test_a_dense_family_is_a_few_switches_on_the_shared_reader():
    """The reference's families are a shared draft plus switches (model/Families.java:166-171,611-733): a family
    with biases on q, k, v always, no q/k norm, the window on every layer and tied embeddings by default."""
    from jllm_serve_b200.config import DecoderDraft

    def parse_toy(values):
        d = DecoderDraft(values, "toy_dense", "ToyDenseForCausalLM")
        d.bias, d.qk_norm, d.window, d.tied_default, d.theta_default = "always", False, "all", True, 5e5
        return d.build()

    register_architecture("toy_dense", parse_toy)
    try:
        c = dict(model_type="toy_dense", hidden_size=64, num_hidden_layers=2, vocab_size=50, num_attention_heads=4,
                 num_key_value_heads=2, intermediate_size=24, sliding_window=9)
        d = parse_config(c)
        a = d.layers[1].mixer
        assert (a.bias, a.out_bias, a.qk_norm, a.window) == (True, False, False, 9)
        assert d.core.tied and d.rope_tables[0].theta == 5e5 and d.core.architecture == "ToyDenseForCausalLM"
        wants = DecoderModel.wants(d)
        assert "model.layers.0.self_attn.q_proj.bias" in wants and "model.layers.0.self_attn.o_proj.bias" not in wants
        assert "model.layers.0.self_attn.q_norm.weight" not in wants and "lm_head.weight" not in wants
        with pytest.raises(ConfigError, match="ToyDenseForCausalLM"):
            parse_config(dict(c, architectures=["Qwen3ForCausalLM"]))
        # newer configs nest the rope keys; the top-level key wins when both are there
        nested = parse_config(dict(c, rope_parameters={"rope_theta": 123.0, "rope_type": "linear", "factor": 2.0}))
        assert nested.rope_tables[0].theta == 123.0 and nested.rope_tables[0].scaling.kind == "linear"
        assert parse_config(dict(c, rope_theta=7.0, rope_parameters={"rope_theta": 123.0})).rope_tables[0].theta == 7.0
    finally:
        unregister_architecture("toy_dense")

    def parse_strict(values):          # the default switches are Llama's: attention_bias is not a key of the family
        return DecoderDraft(values, "toy_strict", "ToyStrictForCausalLM").build()

    register_architecture("toy_strict", parse_strict)
    try:
        c = dict(model_type="toy_strict", hidden_size=64, num_hidden_layers=1, vocab_size=50, num_attention_heads=4,
                 intermediate_size=24, sliding_window=9)
        assert parse_config(c).layers[0].mixer.window == 0 and not parse_config(c).layers[0].mixer.qk_norm
        with pytest.raises(ConfigError, match="attention_bias"):
            parse_config(dict(c, attention_bias=True))
    finally:
        unregister_architecture("toy_strict")


def test_the_reference_reads_qwen3_this_way():
    """The cases of the reference's own test (src/test/java/org/robomiri/jllm/SmokeTest.java:844-846): a qwen3
    config gets the q/k norm, and attention_bias biases q, k, v AND o_proj."""
    plain = parse_config(dict(TINY_A)).layers[0].mixer
    assert plain.qk_norm and not plain.bias and not plain.out_bias
    biased = parse_config(dict(TINY_A, attention_bias=True)).layers[0].mixer
    assert biased.qk_norm and biased.bias and biased.out_bias


def test_schedule_is_data():
    d = parse_config(TINY_A)
    assert [(r.layer, r.cache_of) for r in d.schedule] == [(0, None), (1, None)]
    twice = d.with_schedule([(0, None), (1, None), (1, None), (0, 0)])
    assert len(twice.schedule) == 4
    with pytest.raises(ConfigError):
        d.with_schedule([(0, 1), (1, None)])           # reads a cache that has not been written yet
    with pytest.raises(ConfigError):
        d.with_schedule([(0, None), (5, None)])


def test_yarn_parameters():
    d = parse_config(dict(TINY_B, rope_scaling={"rope_type": "yarn", "factor": 4.0,
                                                 "original_max_position_embeddings": 128}))
    s = d.rope_tables[0].scaling
    assert (s.kind, s.factor, s.original_max_positions, s.beta_fast, s.beta_slow) == ("yarn", 4.0, 128, 32.0, 1.0)
    # the frequencies and the amplitude themselves are checked against the reference's own numbers in
    # tests/test_reference_literals.py


# ---- weights ------------------------------------------------------------------------------------------------

def test_model_folder_round_trip(tmp_path):
    folder = write_model_folder(TINY_B, 3, tmp_path / "m")
    spec, raw = load_config(folder)
    assert raw["hidden_size"] == 96
    wants = DecoderModel.wants(spec)
    src = TensorSource(folder)
    assert set(src.names()) == set(wants)
    t = load_checked(src, wants, torch.bfloat16, "cpu")
    assert t["lm_head.weight"].dtype == torch.bfloat16 and t["lm_head.weight"].shape == (1000, 96)
    assert t["model.layers.2.self_attn.q_norm.weight"].shape == (32,)
    again = write_model_folder(TINY_B, 3, tmp_path / "n")
    assert torch.equal(TensorSource(again).tensor("model.norm.weight"), src.tensor("model.norm.weight"))
    other = write_model_folder(TINY_B, 4, tmp_path / "o")
    assert not torch.equal(TensorSource(other).tensor("model.norm.weight"), src.tensor("model.norm.weight"))
    gains = src.tensor("model.layers.0.input_layernorm.weight").float()
    assert abs(float(gains.mean()) - 1.0) < 0.1                      # norm gains are 1 + N(0, 0.1)
    assert float(src.tensor("model.embed_tokens.weight").float().std()) < 0.03


def test_tied_model_has_no_head_tensor(tmp_path):
    folder = write_model_folder(TINY_A, 1, tmp_path / "m")
    assert not TensorSource(folder).has("lm_head.weight")


def test_precision_policy(tmp_path):
    folder = write_model_folder(TINY_A, 1, tmp_path / "m", torch.bfloat16, vector_dtype=torch.float32)
    spec, _ = load_config(folder)
    wants = DecoderModel.wants(spec)
    bf = load_checked(TensorSource(folder), wants, torch.bfloat16, "cpu")
    assert bf["model.embed_tokens.weight"].dtype == torch.bfloat16       # kept in bfloat16
    assert bf["model.norm.weight"].dtype == torch.float32                # a tensor stored in 32-bit stays so
    f32 = load_checked(TensorSource(folder), wants, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in f32.values())
    assert torch.equal(f32["model.embed_tokens.weight"], bf["model.embed_tokens.weight"].float())  # exact widening


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_model_folder(TINY_A, 1, tmp_path / "m")
    src = TensorSource(folder)
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    write_safetensors(folder / "model.safetensors", tensors)
    spec, _ = load_config(folder)
    with pytest.raises(WeightError) as e:
        load_checked(TensorSource(folder), DecoderModel.wants(spec), torch.bfloat16, "cpu")
    msg = str(e.value)
    assert "missing (2): model.layers.1.mlp.down_proj.weight, model.norm.weight" in msg
    assert "unexpected (1): model.layers.0.self_attn.rotary_emb.inv_freq" in msg
    assert "model.layers.0.self_attn.k_proj.weight is [16, 64], config wants [32, 64]" in msg
    assert e.value.missing and e.value.unexpected and e.value.wrong_shape


def test_untied_model_without_head_uses_the_embedding(tmp_path):
    """`lmHead = file.has("lm_head.weight") ? that : embed` (model/ModelWeights.java:37 of the reference)."""
    from jllm_serve_b200.parts import Runtime
    folder = write_model_folder(TINY_B, 1, tmp_path / "m")
    src = TensorSource(folder)
    tensors = {n: src.tensor(n).clone() for n in src.names() if n != "lm_head.weight"}
    write_safetensors(folder / "model.safetensors", tensors)
    spec, _ = load_config(folder)
    loaded = load_checked(TensorSource(folder), DecoderModel.wants(spec), torch.float32, "cpu")
    assert "lm_head.weight" not in loaded
    rt = Runtime(torch.device("cpu"), torch.float32, 64, 8, 4)
    model = DecoderModel(spec, loaded, rt)
    assert model.head.weight is model.embedding and any("embedding serves as the head" in n for n in rt.notes)


def test_tensors_the_model_does_not_ask_for_are_noted_not_refused(tmp_path):
    """A tied checkpoint that still ships lm_head.weight, an old one with rotary_emb.inv_freq: read what is needed,
    note the rest; `strict` turns them into the error."""
    folder = write_model_folder(TINY_A, 1, tmp_path / "m")
    src = TensorSource(folder)
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    write_safetensors(folder / "model.safetensors", tensors)
    spec, _ = load_config(folder)
    notes = []
    loaded = load_checked(TensorSource(folder), DecoderModel.wants(spec), torch.bfloat16, "cpu", notes)
    assert "lm_head.weight" not in loaded and set(loaded) == set(DecoderModel.wants(spec))
    assert len(notes) == 1 and "2 tensors" in notes[0] and "rotary_emb.inv_freq" in notes[0]
    with pytest.raises(WeightError, match=r"unexpected \(2\)"):
        load_checked(TensorSource(folder), DecoderModel.wants(spec), torch.bfloat16, "cpu", strict=True)


def test_multimodal_prefixes_are_dropped(tmp_path):
    """`model.language_model.X` and `language_model.model.X` are read as `model.X` (model/ModelConverter.java:977-988
    of the reference); a vision tower beside them is left alone."""
    folder = write_model_folder(TINY_B, 1, tmp_path / "m")
    src = TensorSource(folder)
    plain = {n: src.tensor(n).clone() for n in src.names()}
    spec, _ = load_config(folder)
    want = load_checked(TensorSource(folder), DecoderModel.wants(spec), torch.float32, "cpu")
    for prefix, head in (("model.language_model.", "lm_head."), ("language_model.model.", "language_model.lm_head.")):
        renamed = {(prefix + n[len("model."):] if n.startswith("model.") else head + n[len("lm_head."):]): t
                   for n, t in plain.items()}
        renamed["model.visual.patch_embed.weight"] = torch.zeros(4, 4)
        write_safetensors(folder / "model.safetensors", renamed)
        notes = []
        got = load_checked(TensorSource(folder), DecoderModel.wants(spec), torch.float32, "cpu", notes)
        assert set(got) == set(want) and all(torch.equal(got[n], want[n]) for n in want)
        assert any("model.visual.patch_embed.weight" in n for n in notes)
    both = dict(plain)
    both["model.language_model.norm.weight"] = plain["model.norm.weight"].clone()
    write_safetensors(folder / "model.safetensors", both)
    with pytest.raises(WeightError, match="are both 'model.norm.weight'"):
        load_checked(TensorSource(folder), DecoderModel.wants(spec), torch.float32, "cpu")


def _raw_file(path, header: dict, data: bytes):
    text = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(text)) + text + data)


def test_safetensors_checks(tmp_path):
    (tmp_path / "a").mkdir()
    f = tmp_path / "a" / "model.safetensors"
    _raw_file(f, {"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 8 bytes"):
        TensorSource(tmp_path / "a")
    _raw_file(f, {"x": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        TensorSource(tmp_path / "a")
    _raw_file(f, {"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                  "y": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="overlap"):
        TensorSource(tmp_path / "a")
    f.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        TensorSource(tmp_path / "a")
    f.write_bytes(struct.pack("<Q", 30) + b'{"x":{"dtype":"F32"},"x":{}}  ')
    with pytest.raises(SafetensorsError, match="duplicate"):
        TensorSource(tmp_path / "a")
    with pytest.raises(SafetensorsError, match="neither"):
        TensorSource(tmp_path)


def test_sharded_checkpoint(tmp_path):
    write_safetensors(tmp_path / "s1.safetensors", {"a": torch.ones(2)})
    write_safetensors(tmp_path / "s2.safetensors", {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    src = TensorSource(tmp_path)
    assert src.tensor("a").tolist() == [1.0, 1.0] and src.meta("b")[1] == (3,)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../s1.safetensors"}}))
    with pytest.raises(SafetensorsError, match="plain file name"):
        TensorSource(tmp_path)
