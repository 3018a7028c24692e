"""Configuration, registry and weight loading (no GPU)."""
import json
import os

import pytest
import torch

from helpers import CONFIG_A, CONFIG_B, TinyModel
from transformers_neuronx_b200.config import (ConfigError, EngineConfig, OPTConfig, canonical_dtype, load_config,
                                              resolve_architecture)
from transformers_neuronx_b200.models import opt as opt_arch
from transformers_neuronx_b200.models.decoder import DecoderModel
from transformers_neuronx_b200.weights import (TensorSpec, WeightError, load_tensors, match_tensors,
                                               save_safetensors, SafetensorsFile)


def test_config_reads_its_keys():
    cfg = OPTConfig.from_dict(dict(CONFIG_B, some_unknown_key=3))
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim) == (96, 3, 32)
    assert cfg.word_embed_proj_dim == 48 and cfg.has_projection
    assert not cfg.do_layer_norm_before and not cfg.has_final_layer_norm
    assert cfg.layer_norm_eps == 1e-6 and not cfg.enable_bias
    a = OPTConfig.from_dict({k: v for k, v in CONFIG_A.items() if k != "word_embed_proj_dim"})
    assert a.word_embed_proj_dim == a.hidden_size and not a.has_projection and a.has_final_layer_norm


def test_config_errors():
    with pytest.raises(ConfigError, match="ffn_dim"):
        OPTConfig.from_dict({k: v for k, v in CONFIG_A.items() if k != "ffn_dim"})
    with pytest.raises(ConfigError, match="multiple"):
        OPTConfig.from_dict(dict(CONFIG_A, num_attention_heads=5))
    with pytest.raises(ConfigError):
        OPTConfig.from_dict(dict(CONFIG_A, vocab_size=-1))


def test_registry():
    assert resolve_architecture({"architectures": ["OPTForCausalLM"]}).name == "OPTForCausalLM"
    assert resolve_architecture({"model_type": "opt"}).name == "OPTForCausalLM"
    with pytest.raises(KeyError, match="OPTForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})


def test_dtype_names():
    assert canonical_dtype("f32") == "float32" and canonical_dtype("bf16") == "bfloat16"
    assert canonical_dtype(torch.bfloat16) == "bfloat16"
    assert canonical_dtype("f16") == "float16" and canonical_dtype(torch.float16) == "float16"   # dtypes.py:18-35
    with pytest.raises(ValueError, match="f32, f16, bf16"):
        canonical_dtype("f8")
    with pytest.raises(ValueError):
        EngineConfig(page_size=24)


def test_spec_follows_config():
    for c in (CONFIG_A, CONFIG_B):
        cfg = OPTConfig.from_dict(c)
        spec = opt_arch.build_spec(cfg)
        assert len(spec.layers) == cfg.num_hidden_layers == len(spec.schedule)
        l0 = spec.layers[0]
        assert l0.block == ("pre_norm" if cfg.do_layer_norm_before else "post_norm")
        assert l0.mixer.n_heads == cfg.num_attention_heads and l0.mixer.head_dim == cfg.head_dim
        assert l0.norm1.eps == cfg.layer_norm_eps
        assert (l0.mixer.q.bias is not None) == cfg.enable_bias
        assert (l0.norm1.weight is not None) == cfg.layer_norm_elementwise_affine
        assert (spec.embedding.project_in is not None) == cfg.has_projection
        assert (spec.head.final_norm is not None) == cfg.has_final_layer_norm
        assert spec.embedding.position.rows == cfg.max_position_embeddings + 2
        names = [s.name for s in DecoderModel(spec).tensor_specs()]
        assert len(names) == len(set(names))
        assert ("model.decoder.project_in.weight" in names) == cfg.has_projection


def test_random_weights_are_seeded_and_roundtrip(tmp_path):
    m1, m2, m3 = TinyModel("A", seed=5), TinyModel("A", seed=5), TinyModel("A", seed=6)
    k = "model.decoder.layers.1.fc1.weight"
    assert torch.equal(m1.tensors[k], m2.tensors[k]) and not torch.equal(m1.tensors[k], m3.tensors[k])
    assert m1.tensors[k].dtype == torch.bfloat16
    assert m1.tensors["model.decoder.layers.0.final_layer_norm.weight"].dtype == torch.float32   # stays 32-bit
    assert m1.tensors["lm_head.weight"] is m1.tensors["model.decoder.embed_tokens.weight"]        # tied
    arch, cfg = load_config(m1.folder)
    assert arch.name == "OPTForCausalLM" and cfg == m1.cfg
    assert sorted(os.listdir(m1.folder)) == ["config.json", "model.safetensors"]


def _specs():
    return [TensorSpec("model.a.weight", (4, 3)), TensorSpec("model.a.bias", (4,), "bias"),
            TensorSpec("head.weight", (4, 3), tied_to="model.a.weight")]


def test_one_error_lists_everything():
    avail = {"model.a.weight": (torch.bfloat16, (4, 5)), "stray": (torch.float32, (1,)),
             "other.stray": (torch.float32, (2,))}
    with pytest.raises(WeightError) as ei:
        match_tensors(_specs() + [TensorSpec("model.b.weight", (2, 2))], avail, "mem")
    e = ei.value
    assert set(e.missing) == {"model.a.bias", "model.b.weight"}
    assert set(e.unexpected) == {"stray", "other.stray"}
    assert [w[0] for w in e.wrong_shape][:1] == ["model.a.weight"]
    msg = str(e)
    for word in ("missing", "unexpected", "wrong shape", "model.b.weight", "stray", "[4, 5]"):
        assert word in msg


def test_prefix_and_tie(tmp_path):
    # a checkpoint of the bare decoder lacks 'model.'; the tied head is absent
    t = {"a.weight": torch.randn(4, 3).bfloat16(), "a.bias": torch.randn(4).half()}
    save_safetensors(t, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text("{}")
    out = load_tensors(str(tmp_path), _specs())
    assert out["head.weight"] is out["model.a.weight"]
    assert out["model.a.bias"].dtype == torch.float16 and torch.equal(out["model.a.bias"], t["a.bias"])   # kept as stored
    # a stored head that differs from the table it is tied to is an error
    t["head.weight"] = torch.randn(4, 3).bfloat16()
    save_safetensors(t, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError, match="tied"):
        load_tensors(str(tmp_path), _specs())
    t["head.weight"] = t["a.weight"].clone()
    save_safetensors(t, str(tmp_path / "model.safetensors"))
    assert torch.equal(load_tensors(str(tmp_path), _specs())["head.weight"], t["a.weight"])


def test_dtypes_kept(tmp_path):
    t = {"w32": torch.randn(3, 3), "wb": torch.randn(3, 3).bfloat16(), "i64": torch.arange(4), "i32": torch.arange(4, dtype=torch.int32)}
    save_safetensors(t, str(tmp_path / "model.safetensors"))
    specs = [TensorSpec("w32", (3, 3)), TensorSpec("wb", (3, 3)), TensorSpec("i64", (4,), "int_table"), TensorSpec("i32", (4,), "int_table")]
    out = load_tensors(str(tmp_path), specs)
    assert out["w32"].dtype == torch.float32 and torch.equal(out["w32"], t["w32"])
    assert out["wb"].dtype == torch.bfloat16
    assert out["i64"].dtype == torch.int32 and out["i32"].dtype == torch.int32


def test_missing_files(tmp_path):
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_tensors(str(tmp_path), _specs())
    with pytest.raises(FileNotFoundError, match="config.json"):
        load_config(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(b"\x00\x01")
    with pytest.raises(ValueError):
        SafetensorsFile(str(tmp_path / "model.safetensors"))


def test_sharded_index(tmp_path):
    a = {"model.a.weight": torch.randn(4, 3).bfloat16()}
    b = {"model.a.bias": torch.randn(4)}
    save_safetensors(a, str(tmp_path / "s1.safetensors"))
    save_safetensors(b, str(tmp_path / "s2.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"model.a.weight": "s1.safetensors", "model.a.bias": "s2.safetensors"}}))
    out = load_tensors(str(tmp_path), _specs())
    assert torch.equal(out["model.a.bias"], b["model.a.bias"])


def test_the_reference_s_torch_saved_layouts(tmp_path):
    """The folders that the reference itself writes and reads besides safetensors
    (src/transformers_neuronx/module.py:30-50 writer, :434-460 reader): a directory pytorch_model.bin/
    with one torch-saved tensor per file and key_to_filename.json, one pytorch_model.bin state dict,
    and shards with pytorch_model.bin.index.json.  The files are laid out here as that writer lays them
    out ('p<index>.<key>'); the model's tensors come back the same from each, the tied head included."""
    m = TinyModel("B", seed=4)
    specs = DecoderModel(opt_arch.build_spec(m.cfg)).tensor_specs()
    want = load_tensors(m.folder, specs)
    stored = {k: v for k, v in m.plain_tensors.items()}
    config = open(os.path.join(m.folder, "config.json")).read()

    def check(folder):
        got = load_tensors(str(folder), specs)
        assert sorted(got) == sorted(want)
        for k in want:
            assert got[k].dtype == want[k].dtype and torch.equal(got[k], want[k]), k
        assert got["lm_head.weight"] is got["model.decoder.embed_tokens.weight"]

    split = tmp_path / "split"
    (split / "pytorch_model.bin").mkdir(parents=True)
    (split / "config.json").write_text(config)
    names = {k: f"p{i}.{k}" for i, k in enumerate(stored)}
    (split / "pytorch_model.bin" / "key_to_filename.json").write_text(json.dumps(names, indent=2))
    for k, t in stored.items():
        torch.save(t, str(split / "pytorch_model.bin" / names[k]))
    check(split)

    single = tmp_path / "single"
    single.mkdir()
    (single / "config.json").write_text(config)
    torch.save(stored, str(single / "pytorch_model.bin"))
    check(single)

    shards = tmp_path / "shards"
    shards.mkdir()
    (shards / "config.json").write_text(config)
    keys = list(stored)
    parts = {"pytorch_model-00001-of-00002.bin": keys[: len(keys) // 2], "pytorch_model-00002-of-00002.bin": keys[len(keys) // 2:]}
    for fn, ks in parts.items():
        torch.save({k: stored[k] for k in ks}, str(shards / fn))
    (shards / "pytorch_model.bin.index.json").write_text(json.dumps(
        {"metadata": {}, "weight_map": {k: fn for fn, ks in parts.items() for k in ks}}))
    check(shards)

    # one error that lists everything, as for safetensors
    os.remove(str(split / "pytorch_model.bin" / names[keys[3]]))
    del names[keys[3]]
    names["stray.weight"] = "p999.stray.weight"
    torch.save(torch.zeros(2), str(split / "pytorch_model.bin" / "p999.stray.weight"))
    (split / "pytorch_model.bin" / "key_to_filename.json").write_text(json.dumps(names))
    with pytest.raises(WeightError) as ei:
        load_tensors(str(split), specs)
    assert keys[3] in ei.value.missing and "stray.weight" in ei.value.unexpected


def test_compiled_kernels_can_be_kept_in_a_folder(tmp_path):
    """export_libraries / import_libraries (model.save / model.load): libraries carry the digest of
    their source in their names; a file of another version or of another origin is not taken."""
    from transformers_neuronx_b200.kernels import build as kb
    out = kb.export_libraries(["embedding"], str(tmp_path))
    assert [os.path.basename(p) for p in out] == [os.path.basename(kb.library_path("embedding"))]
    (tmp_path / "embedding.0000000000000000.so").write_bytes(b"stale")
    (tmp_path / "notes.txt").write_text("x")
    assert kb.import_libraries(str(tmp_path)) == ["embedding"]
    try:
        kb.import_libraries(str(tmp_path / "missing"))
    except kb.KernelBuildError:
        pass
    else:
        raise AssertionError("a missing folder was accepted")


def test_files_agree_with_the_safetensors_package_in_both_directions(tmp_path):
    """The engine has a reader and a writer of its own; a mistake that both share (header padding,
    dtype tags, offsets) would be invisible to a test that only ever feeds one to the other.  So:
    a file written by the `safetensors` package is read by the engine's reader, a file written by the
    engine's writer is read by the package, in every type the engine stores, and a sharded folder
    with an index as the package's users write it."""
    import json
    from safetensors import safe_open
    from safetensors.torch import load_file, save_file
    from transformers_neuronx_b200.weights import SafetensorsFile, open_model_files
    g = torch.Generator().manual_seed(3)
    t = {"w.bf16": torch.randn(7, 5, generator=g).bfloat16(), "w.f16": torch.randn(3, 11, generator=g).half(),
         "w.f32": torch.randn(2, 3, 4, generator=g), "i.i32": torch.arange(6, dtype=torch.int32).view(2, 3),
         "i.i64": torch.arange(5), "scalar": torch.tensor(1.5), "empty": torch.zeros(0, 4)}
    theirs, ours = str(tmp_path / "theirs.safetensors"), str(tmp_path / "ours.safetensors")
    save_file(t, theirs, metadata={"format": "pt"})
    f = SafetensorsFile(theirs)
    assert sorted(f.keys()) == sorted(t)
    for k, v in t.items():
        got = f.tensor(k)
        assert got.dtype == v.dtype and tuple(got.shape) == tuple(v.shape) and torch.equal(got, v), k
        assert f.info(k) == (v.dtype, tuple(v.shape))
    f.close()
    save_safetensors(t, ours, metadata={"format": "pt", "seed": 3})
    back = load_file(ours)
    assert sorted(back) == sorted(t)
    for k, v in t.items():
        assert back[k].dtype == v.dtype and torch.equal(back[k], v), k
    with safe_open(ours, framework="pt") as fp:
        assert fp.metadata()["format"] == "pt" and fp.metadata()["seed"] == "3"
    # a sharded folder: two files and model.safetensors.index.json
    folder = tmp_path / "sharded"
    folder.mkdir()
    names = sorted(t)
    save_file({k: t[k] for k in names[:3]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({k: t[k] for k in names[3:]}, str(folder / "model-00002-of-00002.safetensors"))
    index = {"metadata": {}, "weight_map": {k: ("model-00001-of-00002.safetensors" if k in names[:3]
                                                 else "model-00002-of-00002.safetensors") for k in names}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    files = open_model_files(str(folder))
    seen = {}
    for fl in files:
        for k in fl.keys():
            seen[k] = fl.tensor(k).clone()
        fl.close()
    assert sorted(seen) == names and all(torch.equal(seen[k], t[k]) for k in names)


def test_entry_point_small_parity_methods(tmp_path):
    """is_compiled() and update_generation_config(), which the reference's base class offers
    (src/transformers_neuronx/base.py:143-151, :761-762), work without a GPU."""
    from transformers_neuronx_b200 import GenerationConfig
    from transformers_neuronx_b200.kernels import build as kb
    from transformers_neuronx_b200.opt.model import OPTForSampling
    tiny = TinyModel("A", seed=2)
    m = OPTForSampling.from_pretrained(tiny.folder, batch_size=2, amp="bf16", n_positions=32)
    have = all(os.path.isfile(kb.library_path(n)) for n in ("gemm_tc", "gemv", "layernorm", "embedding", "kv_cache",
                                                              "attention_decode", "attention_prefill", "attention_prefill_tc",
                                                              "gemm_simt", "attention_simt"))
    assert m.is_compiled() == have
    m.update_generation_config(GenerationConfig(do_sample=True, top_k=7))
    assert m.neuron_config.on_device_generation.top_k == 7
    with pytest.raises(TypeError):
        m.update_generation_config({"top_k": 3})


def test_auto_class_picks_the_entry_point_by_config(tmp_path):
    """NeuronAutoModelForCausalLM.from_pretrained (modeling_auto.py:5-47): the folder's model_type chooses the class."""
    from transformers_neuronx_b200 import NeuronAutoModelForCausalLM, OPTForSampling
    tiny = TinyModel("B", seed=3)
    m = NeuronAutoModelForCausalLM.from_pretrained(tiny.folder, batch_size=2, amp="f32", n_positions=32)
    assert isinstance(m, OPTForSampling) and m.batch_size == 2 and m.config == tiny.cfg
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["NobodyForCausalLM"], "model_type": "nobody"}))
    with pytest.raises(Exception, match="nobody|Nobody"):
        NeuronAutoModelForCausalLM.from_pretrained(str(tmp_path))
    with pytest.raises(FileNotFoundError):
        NeuronAutoModelForCausalLM.from_pretrained("facebook/opt-125m")
