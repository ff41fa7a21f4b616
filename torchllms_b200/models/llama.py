"""The Llama-3 dense decoder as an :class:`~torchllms_b200.config.registry.Architecture`.

Reference: the base ``Transformer`` of torchllms/models/networks.py:778-1049 with
every optional flag off (role embeddings :125, OLMo-2 :127, gpt-oss :128, q/k
norm :133, projection bias :122).  This module only *describes* that model:
it maps the configuration to a spec of generic parts, names the tensors, and
knows the two naming conventions a checkpoint may use.
"""

from __future__ import annotations

import re
from typing import Any, Dict, Iterator, Mapping, Tuple

import torch

from .llama_config import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, RunEntry, part
from ..weights.loader import LazyTensor


def parse_config(raw: Mapping[str, Any], source: str) -> LlamaConfig:
    if source.endswith("params.json"):
        return LlamaConfig.from_params_json(raw, source)
    return LlamaConfig.from_hf(raw, source)


def build_spec(cfg: LlamaConfig) -> ModelSpec:
    """Every layer is the same here; the spec still spells each one out."""
    position = part("rope", head_dim=cfg.head_dim, theta=cfg.rope_theta,
                    scaling=cfg.rope_scaling.to_dict(), pairing="interleaved")
    mixer = part("attention", dim=cfg.dim, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads,
                 head_dim=cfg.head_dim, scale=cfg.head_dim ** -0.5, position=position, window=None)
    ffn = part("swiglu", dim=cfg.dim, hidden=cfg.ffn_hidden)
    norm = part("rmsnorm", dim=cfg.dim, eps=cfg.norm_eps)
    block = part("prenorm", mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=norm,
                 mixer_prefix="attention", ffn_prefix="feed_forward",
                 mixer_norm_prefix="attention_norm", ffn_norm_prefix="ffn_norm")
    layers = tuple(LayerSpec(name=f"layers.{i}", block=block) for i in range(cfg.n_layers))
    return ModelSpec(
        dim=cfg.dim,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_seq_len,
        embedding_tensor="tok_embeddings.weight",
        layers=layers,
        run_order=tuple(RunEntry(i) for i in range(cfg.n_layers)),
        final_norm=norm,
        final_norm_prefix="norm",
        head_tensor="output.weight",
        tie_head=cfg.tie_word_embeddings,
    )


# Hugging Face name -> native (torchllms) name, torchllms/models/checkpoint_converter.py:124-141
_HF_TOP = {
    "model.embed_tokens.weight": "tok_embeddings.weight",
    "model.norm.weight": "norm.weight",
    "lm_head.weight": "output.weight",
}
_HF_LAYER = {
    "self_attn.q_proj.weight": "attention.wq.weight",
    "self_attn.k_proj.weight": "attention.wk.weight",
    "self_attn.v_proj.weight": "attention.wv.weight",
    "self_attn.o_proj.weight": "attention.wo.weight",
    "mlp.gate_proj.weight": "feed_forward.w1.weight",
    "mlp.up_proj.weight": "feed_forward.w3.weight",
    "mlp.down_proj.weight": "feed_forward.w2.weight",
    "input_layernorm.weight": "attention_norm.weight",
    "post_attention_layernorm.weight": "ffn_norm.weight",
}
_HF_LAYER_RE = re.compile(r"^model\.layers\.(\d+)\.(.+)$")
_DROPPED_RE = re.compile(r"^model\.layers\.\d+\.self_attn\.rotary_emb\.inv_freq$")


def interleave_rotary_rows(w: torch.Tensor, n_heads: int, head_dim: int) -> torch.Tensor:
    """Hugging Face keeps a head's rotary lanes as [first halves | second halves];
    the engine rotates adjacent lanes.  Row ``h*hd + s*hd/2 + i`` moves to row
    ``h*hd + 2i + s`` (torchllms/models/checkpoint_converter.py:96-102, :172-178)."""
    rest = w.shape[1:]
    return w.reshape(n_heads, 2, head_dim // 2, *rest).transpose(1, 2).reshape(n_heads * head_dim, *rest)


def split_rotary_rows(w: torch.Tensor, n_heads: int, head_dim: int) -> torch.Tensor:
    """Inverse of :func:`interleave_rotary_rows` (torchllms/models/checkpoint_converter.py:199-211)."""
    rest = w.shape[1:]
    return w.reshape(n_heads, head_dim // 2, 2, *rest).transpose(1, 2).reshape(n_heads * head_dim, *rest)


def adapt_tensors(cfg: LlamaConfig, found: Dict[str, LazyTensor]) -> Dict[str, LazyTensor]:
    """Bring a checkpoint's tensors to native names.  Hugging Face names are
    renamed, their q/k rows permuted; native names pass through; anything else
    keeps its name, so the strict check reports it as unexpected."""
    out: Dict[str, LazyTensor] = {}
    for name, t in found.items():
        if _DROPPED_RE.match(name):
            continue
        new, fix = name, None
        if name in _HF_TOP:
            new = _HF_TOP[name]
        else:
            m = _HF_LAYER_RE.match(name)
            if m and m.group(2) in _HF_LAYER:
                new = f"layers.{m.group(1)}.{_HF_LAYER[m.group(2)]}"
                if m.group(2) == "self_attn.q_proj.weight":
                    fix = cfg.n_heads
                elif m.group(2) == "self_attn.k_proj.weight":
                    fix = cfg.n_kv_heads
        if fix is not None and len(t.shape) == 2 and t.shape[0] == fix * cfg.head_dim:
            t = t.mapped(lambda w, n=fix: interleave_rotary_rows(w, n, cfg.head_dim))
        if new in out:
            raise ValueError(f"checkpoint provides tensor {new!r} under two names")
        out[new] = t
    return out


def tensor_shapes(cfg: LlamaConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """``(name, shape, init)`` of every tensor in the fixed order random weights are drawn in."""
    q, kv = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    yield "tok_embeddings.weight", (cfg.vocab_size, cfg.dim), "matrix"
    for i in range(cfg.n_layers):
        p = f"layers.{i}"
        yield f"{p}.attention.wq.weight", (q, cfg.dim), "matrix"
        yield f"{p}.attention.wk.weight", (kv, cfg.dim), "matrix"
        yield f"{p}.attention.wv.weight", (kv, cfg.dim), "matrix"
        yield f"{p}.attention.wo.weight", (cfg.dim, q), "matrix"
        yield f"{p}.feed_forward.w1.weight", (cfg.ffn_hidden, cfg.dim), "matrix"
        yield f"{p}.feed_forward.w2.weight", (cfg.dim, cfg.ffn_hidden), "matrix"
        yield f"{p}.feed_forward.w3.weight", (cfg.ffn_hidden, cfg.dim), "matrix"
        yield f"{p}.attention_norm.weight", (cfg.dim,), "norm"
        yield f"{p}.ffn_norm.weight", (cfg.dim,), "norm"
    yield "norm.weight", (cfg.dim,), "norm"
    if not cfg.tie_word_embeddings:
        yield "output.weight", (cfg.vocab_size, cfg.dim), "matrix"


def random_tensors(cfg: LlamaConfig, seed: int, *, device="cpu", dtype: torch.dtype = torch.float32,
                   matrix_std: float = 0.02, norm_std: float = 0.1) -> Iterator[Tuple[str, torch.Tensor]]:
    """Seeded random weights: matrices ``N(0, matrix_std)`` as the reference's ``init_module``
    draws them (torchllms/models/utils.py:197-214); norm weights ``1 + N(0, norm_std)`` rather than
    the reference's ones (torchllms/models/networks.py:192-193) so that a fault in a norm shows.
    One generator, one fixed order, drawn in float32 and then cast."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    for name, shape, init in tensor_shapes(cfg):
        t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        t = t * matrix_std if init == "matrix" else 1.0 + t * norm_std
        yield name, t.to(dtype)


LLAMA = register_architecture(Architecture(
    name="LlamaForCausalLM",
    parse_config=parse_config,
    build_spec=build_spec,
    adapt_tensors=adapt_tensors,
    random_tensors=random_tensors,
    chat_template="llama3_instruct",
))
