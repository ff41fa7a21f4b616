"""Safetensors reading and writing, name maps, strictness, random weights."""

import json

import pytest
import torch

from helpers import TINY, TINY_A, TINY_B, make_tensors, write_model_folder
from plain_llama import PlainModel
from torch_ops import TorchOps
from torchllms_b200.models.llama_config import LlamaConfig
from torchllms_b200.engine.loading import load_model
from torchllms_b200.models.llama import interleave_rotary_rows, split_rotary_rows
from torchllms_b200.weights.loader import WeightError
from torchllms_b200.weights.random_init import write_random_model
from torchllms_b200.weights.safetensors_io import SafetensorsError, TensorSource, write_safetensors

OPS = TorchOps()


def load(folder, dtype="float32"):
    return load_model(folder, dtype=dtype, device="cpu", ops=OPS)


def test_own_writer_and_reader_agree_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    tensors = {"a": torch.randn(3, 5), "b.c": torch.randn(7).to(torch.bfloat16), "i": torch.arange(6, dtype=torch.int64).view(2, 3),
               "empty": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "mine.safetensors", tensors, metadata={"format": "pt"})
    theirs = load_file(str(tmp_path / "mine.safetensors"))
    for k, v in tensors.items():
        assert theirs[k].dtype == v.dtype and torch.equal(theirs[k], v)
    save_file(tensors, str(tmp_path / "theirs.safetensors"))
    src = TensorSource(tmp_path / "theirs.safetensors")
    assert sorted(src.names()) == sorted(tensors)
    for k, v in tensors.items():
        got = src.get(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)


def test_sharded_folder_and_broken_files(tmp_path):
    t = make_tensors(TINY_A, 0)
    names = list(t)
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {k: t[k] for k in names[:7]})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {k: t[k] for k in names[7:]})
    index = {"weight_map": {k: ("model-00001-of-00002.safetensors" if i < 7 else "model-00002-of-00002.safetensors")
                            for i, k in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    _, _, model = load(tmp_path)
    assert torch.equal(model.embedding, t["tok_embeddings.weight"])
    (tmp_path / "bad.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{not json")
    with pytest.raises(SafetensorsError):
        TensorSource(tmp_path / "bad.safetensors")
    with pytest.raises(FileNotFoundError):
        TensorSource(tmp_path / "nowhere")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    t = make_tensors(TINY_A, 0)
    del t["layers.1.ffn_norm.weight"], t["output.weight"]
    t["layers.0.attention.wq.weight"] = torch.zeros(64, 32)
    t["layers.0.feed_forward.w2.weight"] = torch.zeros(192, 64)       # transposed
    t["layers.0.attention.bias_k"] = torch.zeros(3)
    t["extra.weight"] = torch.zeros(1)
    folder = write_model_folder(tmp_path, TINY_A, t)
    with pytest.raises(WeightError) as e:
        load(folder)
    err = e.value
    assert sorted(err.missing) == ["layers.1.ffn_norm.weight", "output.weight"]
    assert sorted(err.unexpected) == ["extra.weight", "layers.0.attention.bias_k"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["layers.0.attention.wq.weight", "layers.0.feed_forward.w2.weight"]
    text = str(err)
    for needle in ("missing", "unexpected", "wrong shapes", "layers.1.ffn_norm.weight", "extra.weight", "[64, 64]", "[64, 32]"):
        assert needle in text


def test_integer_tensor_where_a_float_belongs(tmp_path):
    t = make_tensors(TINY_A, 0)
    t["norm.weight"] = torch.ones(64, dtype=torch.int32)
    with pytest.raises(WeightError, match="floating"):
        load(write_model_folder(tmp_path, TINY_A, t))


def test_tied_head(tmp_path):
    t = make_tensors(TINY_B, 1)
    assert "output.weight" not in t
    _, _, model = load(write_model_folder(tmp_path / "a", TINY_B, t))
    assert model.head is model.embedding
    t2 = dict(t, **{"output.weight": t["tok_embeddings.weight"].clone()})        # the same table twice is harmless
    load(write_model_folder(tmp_path / "b", TINY_B, t2))
    t3 = dict(t, **{"output.weight": t["tok_embeddings.weight"] + 1})
    with pytest.raises(WeightError, match="ties"):
        load(write_model_folder(tmp_path / "c", TINY_B, t3))


def hf_named(cfg, t):
    """The same weights under Hugging Face names, q/k rows in the half-split order."""
    hd = cfg["head_dim"]
    out = {}
    ren = {"attention.wq.weight": "self_attn.q_proj.weight", "attention.wk.weight": "self_attn.k_proj.weight",
           "attention.wv.weight": "self_attn.v_proj.weight", "attention.wo.weight": "self_attn.o_proj.weight",
           "feed_forward.w1.weight": "mlp.gate_proj.weight", "feed_forward.w3.weight": "mlp.up_proj.weight",
           "feed_forward.w2.weight": "mlp.down_proj.weight", "attention_norm.weight": "input_layernorm.weight",
           "ffn_norm.weight": "post_attention_layernorm.weight"}
    for name, v in t.items():
        if name.startswith("layers."):
            _, i, rest = name.split(".", 2)
            if rest in ("attention.wq.weight", "attention.wk.weight"):
                v = split_rotary_rows(v, v.shape[0] // hd, hd)
            out[f"model.layers.{i}.{ren[rest]}"] = v
        else:
            out[{"tok_embeddings.weight": "model.embed_tokens.weight", "norm.weight": "model.norm.weight",
                 "output.weight": "lm_head.weight"}[name]] = v
    return out


@pytest.mark.parametrize("name", ["A", "B"])
def test_hugging_face_names_load_to_the_same_model(tmp_path, name):
    cfg, seed, _ = TINY[name]
    t = make_tensors(cfg, seed)
    hf = hf_named(cfg, t)
    hf["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(cfg["head_dim"] // 2)   # dropped silently
    a = load(write_model_folder(tmp_path / "native", cfg, t))[2]
    b = load(write_model_folder(tmp_path / "hf", cfg, hf))[2]
    for x, y in zip(a.blocks, b.blocks):
        assert torch.equal(x.mixer.wqkv, y.mixer.wqkv) and torch.equal(x.feed_forward.w13, y.feed_forward.w13)
    # and the plain implementation, with its own name map and permutation, sees the same model
    toks = list(range(5, 25))
    pa = PlainModel(tmp_path / "native").logits(toks)
    pb = PlainModel(tmp_path / "hf").logits(toks)
    assert torch.equal(pa, pb)


def test_rotary_row_permutation_is_a_bijection():
    w = torch.arange(4 * 8 * 3, dtype=torch.float32).view(32, 3)
    assert torch.equal(split_rotary_rows(interleave_rotary_rows(w, 4, 8), 4, 8), w)
    v = interleave_rotary_rows(torch.arange(8.0).view(8, 1), 1, 8).flatten().tolist()
    assert v == [0, 4, 1, 5, 2, 6, 3, 7]       # row s*hd/2 + i -> row 2i + s


def test_dtypes_kept_as_stored_then_cast_by_the_model(tmp_path):
    t = make_tensors(TINY_A, 0)
    mixed = {k: (v if "norm" in k else v.to(torch.bfloat16)) for k, v in t.items()}
    from safetensors.torch import save_file
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    save_file(mixed, str(tmp_path / "model.safetensors"))
    src = TensorSource(tmp_path)
    assert src.dtype("norm.weight") == torch.float32 and src.dtype("tok_embeddings.weight") == torch.bfloat16
    _, _, m16 = load(tmp_path, "bfloat16")
    assert m16.embedding.dtype == torch.bfloat16 and m16.final_norm.weight.dtype == torch.float32
    assert m16.blocks[0].mixer.wqkv.dtype == torch.bfloat16
    _, _, m32 = load(tmp_path, "float32")
    assert m32.embedding.dtype == torch.float32 and m32.blocks[0].feed_forward.w2.dtype == torch.float32


def test_random_weights_mode_writes_a_loadable_reproducible_folder(tmp_path):
    cfg = LlamaConfig.from_hf(TINY_B)
    a = write_random_model(tmp_path / "a", cfg, seed=5)
    b = write_random_model(tmp_path / "b", cfg, seed=5)
    c = write_random_model(tmp_path / "c", cfg, seed=6)
    assert (a / "config.json").is_file() and (a / "model.safetensors").is_file()
    sa, sb, sc = TensorSource(a), TensorSource(b), TensorSource(c)
    assert all(torch.equal(sa.get(n), sb.get(n)) for n in sa.names())
    assert not torch.equal(sa.get("norm.weight"), sc.get("norm.weight"))
    w = sa.get("layers.0.feed_forward.w1.weight")
    assert abs(w.std().item() - 0.02) < 0.002 and abs(sa.get("norm.weight").mean().item() - 1) < 0.05
    arch, cfg2, model = load(a)
    assert cfg2 == cfg and "output.weight" not in sa.names()
    w16 = write_random_model(tmp_path / "d", cfg, seed=5, dtype=torch.bfloat16)
    assert TensorSource(w16).dtype("tok_embeddings.weight") == torch.bfloat16


def test_later_paths_override_earlier_ones(tmp_path):
    t = make_tensors(TINY_A, 0)
    base = write_model_folder(tmp_path / "base", TINY_A, t)
    write_safetensors(tmp_path / "patch.safetensors", {"norm.weight": torch.full((64,), 2.0)})
    _, _, model = load_model([base, tmp_path / "patch.safetensors"], dtype="float32", device="cpu", ops=OPS)
    assert torch.equal(model.final_norm.weight, torch.full((64,), 2.0))


def test_random_weights_command_line_writes_a_loadable_folder(tmp_path):
    """``python -m torchllms_b200.weights.random_init``: configuration + seed -> model folder."""
    import json
    import subprocess
    import sys

    from torch_ops import TorchOps
    from torchllms_b200.engine.loading import load_model
    cfg_file = tmp_path / "some_config.json"
    cfg_file.write_text(json.dumps(TINY_B))
    outs = []
    for seed, name in ((3, "a"), (3, "b"), (4, "c")):
        run = subprocess.run([sys.executable, "-m", "torchllms_b200.weights.random_init", "--config", str(cfg_file),
                              "--seed", str(seed), "--out", str(tmp_path / name), "--dtype", "float32"],
                             capture_output=True, text=True)
        assert run.returncode == 0, run.stderr
        assert sorted(p.name for p in (tmp_path / name).iterdir()) == ["config.json", "model.safetensors"]
        outs.append((tmp_path / name / "model.safetensors").read_bytes())
    assert outs[0] == outs[1] and outs[0] != outs[2]            # the seed decides, and nothing else
    _, config, model = load_model(tmp_path / "a", dtype="float32", device="cpu", ops=TorchOps())
    assert config.n_layers == TINY_B["num_hidden_layers"] and config.vocab_size == TINY_B["vocab_size"]


def test_the_references_own_checkpoint_folder_loads(tmp_path):
    """``params.json`` beside ``consolidated.00.pth`` (what the reference's converter writes and its
    loader reads, torchllms/models/utils.py:42-43, :107-111): same model as the safetensors folder,
    same strict check."""
    cfg, seed, _ = TINY["A"]
    t = make_tensors(cfg, seed)
    native = load(write_model_folder(tmp_path / "st", cfg, t))[2]
    folder = tmp_path / "pth"
    folder.mkdir()
    (folder / "params.json").write_text(json.dumps({
        "dim": 64, "n_layers": 2, "n_heads": 4, "n_kv_heads": 2, "head_dim": 16, "vocab_size": 512, "multiple_of": 192,
        "ffn_dim_multiplier": 3.0 - 1e-9, "norm_eps": 1e-5, "rope_theta": 10000.0, "max_seq_len": 128}))
    torch.save({k: v.to(torch.bfloat16) for k, v in t.items()}, str(folder / "consolidated.00.pth"))
    for path in (folder, folder / "consolidated.00.pth"):
        got = load(path)[2]
        for a, b in zip(native.blocks, got.blocks):
            assert torch.equal(a.mixer.wqkv.to(torch.bfloat16), b.mixer.wqkv.to(torch.bfloat16))
        assert torch.equal(native.head.to(torch.bfloat16), got.head.to(torch.bfloat16))
    broken = dict(t)
    del broken["norm.weight"]
    torch.save(broken, str(folder / "consolidated.00.pth"))
    with pytest.raises(WeightError) as e:
        load(folder)
    assert e.value.missing == ["norm.weight"]
    (folder / "consolidated.00.pth").write_bytes(b"not a checkpoint")
    with pytest.raises(Exception, match="not a checkpoint"):
        load(folder)
