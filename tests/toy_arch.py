"""A toy architecture that lives outside the package: its own configuration class with its own
``config.json`` keys, a block kind with four norms (one before and one after the mixer, one
before and one after the feed-forward), a block kind without a feed-forward, and a registry
entry.  Nothing under ``torchllms_b200/`` knows of it.  It is no model of anyone's: it exists so
that the tests can show that new parts and a registry entry are all that another architecture
takes.  Importing this module registers it (``TORCHLLMS_B200_PLUGINS=toy_arch`` does that for
the command-line programs).

The plain forward at the end is the oracle: whole sequence, no cache, written with the plain
functions of ``tests/plain_llama.py``.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, Iterator, Mapping, Tuple

import torch

import plain_llama
from torchllms_b200.config.model_config import ConfigError, ModelConfig, require_key, typed_value
from torchllms_b200.config.registry import Architecture, register_architecture
from torchllms_b200.parts.base import (FEED_FORWARDS, MIXERS, NORMS, Block, BuildEnv, Residual, register_block)
from torchllms_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry, part

NAME = "ToyFourNormForCausalLM"


# ------------------------------------------------------------------------------- configuration

@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    architecture: str
    depth: int
    width: int
    heads: int
    kv_heads: int
    head_width: int
    inner: int
    vocab: int
    eps: float
    theta: float
    bare_layers: Tuple[int, ...] = ()       # layers that have a mixer and no feed-forward
    max_seq_len: int = 256

    def validate(self, where: str = "config") -> "ToyConfig":
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}: 'toy_heads' must be a multiple of 'toy_kv_heads'")
        if any(not 0 <= i < self.depth for i in self.bare_layers):
            raise ConfigError(f"{where}: 'toy_bare_layers' names a layer outside 0..{self.depth - 1}")
        return self

    @classmethod
    def parse(cls, raw: Mapping[str, Any], where: str) -> "ToyConfig":
        return cls(
            architecture=NAME,
            depth=require_key(raw, "toy_depth", int, where), width=require_key(raw, "toy_width", int, where),
            heads=require_key(raw, "toy_heads", int, where), kv_heads=require_key(raw, "toy_kv_heads", int, where),
            head_width=require_key(raw, "toy_head_width", int, where), inner=require_key(raw, "toy_inner", int, where),
            vocab=require_key(raw, "toy_vocab", int, where), eps=require_key(raw, "toy_eps", float, where),
            theta=require_key(raw, "toy_theta", float, where),
            bare_layers=tuple(typed_value(i, "toy_bare_layers", int, where) for i in raw.get("toy_bare_layers", [])),
            max_seq_len=typed_value(raw.get("toy_max_len", 256), "toy_max_len", int, where),
        ).validate(where)

    def to_hf(self) -> Dict[str, Any]:
        return {"architectures": [NAME], "toy_depth": self.depth, "toy_width": self.width, "toy_heads": self.heads,
                "toy_kv_heads": self.kv_heads, "toy_head_width": self.head_width, "toy_inner": self.inner,
                "toy_vocab": self.vocab, "toy_eps": self.eps, "toy_theta": self.theta,
                "toy_bare_layers": list(self.bare_layers), "toy_max_len": self.max_seq_len}


# -------------------------------------------------------------------------------------- blocks

class _SubParts(Block):
    """Shared plumbing: sub-parts under their tensor prefixes."""

    def _adopt(self, subparts):
        self._subparts = tuple(subparts)
        self.graph_safe = all(p.graph_safe for _prefix, p in self._subparts)

    def expected_tensors(self):
        return {f"{prefix}.{name}": e for prefix, p in self._subparts for name, e in p.expected_tensors().items()}

    def load(self, tensors):
        for prefix, p in self._subparts:
            p.load({name: tensors[f"{prefix}.{name}"] for name in p.expected_tensors()})

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.mixer.state_need()

    def _normed_alone(self, norm, y, like):
        """``norm(y)`` for a part's output (``[T, dim]``, or partial sums of a split product): a
        norm folds a pending delta into a stream, so the output is laid on a stream of zeros."""
        return norm.forward(Residual(torch.zeros_like(like), y))


@register_block("toy_four_norm")
class FourNormBlock(_SubParts):
    """``h = x + post1(mixer(pre1(x))); out = h + post2(ffn(pre2(h)))``."""

    def __init__(self, env: BuildEnv, *, mixer: PartSpec, feed_forward: PartSpec, pre1: PartSpec, post1: PartSpec,
                 pre2: PartSpec, post2: PartSpec):
        self.mixer = MIXERS.build(mixer, env)
        self.ffn = FEED_FORWARDS.build(feed_forward, env)
        self.pre1, self.post1, self.pre2, self.post2 = (NORMS.build(s, env) for s in (pre1, post1, pre2, post2))
        self._adopt((("mix", self.mixer), ("ff", self.ffn), ("pre1", self.pre1), ("post1", self.post1),
                     ("pre2", self.pre2), ("post2", self.post2)))

    def forward(self, residual: Residual, ctx, cache) -> None:
        x = self.pre1.forward(residual)
        residual.delta = self._normed_alone(self.post1, self.mixer.forward(x, ctx, cache), residual.h)
        x = self.pre2.forward(residual)
        residual.delta = self._normed_alone(self.post2, self.ffn.forward(x, ctx), residual.h)


@register_block("toy_bare")
class BareBlock(_SubParts):
    """A layer without a feed-forward: ``out = x + mixer(pre(x))``."""

    def __init__(self, env: BuildEnv, *, mixer: PartSpec, pre: PartSpec):
        self.mixer = MIXERS.build(mixer, env)
        self.pre = NORMS.build(pre, env)
        self._adopt((("mix", self.mixer), ("pre", self.pre)))

    def forward(self, residual: Residual, ctx, cache) -> None:
        x = self.pre.forward(residual)
        residual.delta = self.mixer.forward(x, ctx, cache)


# ------------------------------------------------------------------------------ the architecture

def build_spec(cfg: ToyConfig) -> ModelSpec:
    rope = part("rope", head_dim=cfg.head_width, theta=cfg.theta, scaling=None, pairing="interleaved")
    mixer = part("attention", dim=cfg.width, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads, head_dim=cfg.head_width,
                 scale=cfg.head_width ** -0.5, position=rope, window=None)
    norm = part("rmsnorm", dim=cfg.width, eps=cfg.eps)
    ffn = part("swiglu", dim=cfg.width, hidden=cfg.inner)
    layers = []
    for i in range(cfg.depth):
        if i in cfg.bare_layers:
            layers.append(LayerSpec(f"stack.{i}", part("toy_bare", mixer=mixer, pre=norm)))
        else:
            layers.append(LayerSpec(f"stack.{i}", part("toy_four_norm", mixer=mixer, feed_forward=ffn, pre1=norm,
                                                      post1=norm, pre2=norm, post2=norm)))
    return ModelSpec(dim=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_seq_len, embedding_tensor="table.weight",
                     layers=tuple(layers), run_order=tuple(RunEntry(i) for i in range(cfg.depth)), final_norm=norm,
                     final_norm_prefix="last_norm", head_tensor="table.weight", tie_head=True)


def tensor_shapes(cfg: ToyConfig) -> Iterator[Tuple[str, Tuple[int, ...]]]:
    q, kv = cfg.heads * cfg.head_width, cfg.kv_heads * cfg.head_width
    yield "table.weight", (cfg.vocab, cfg.width)
    for i in range(cfg.depth):
        p = f"stack.{i}"
        for name, rows, cols in (("wq", q, cfg.width), ("wk", kv, cfg.width), ("wv", kv, cfg.width), ("wo", cfg.width, q)):
            yield f"{p}.mix.{name}.weight", (rows, cols)
        if i in cfg.bare_layers:
            yield f"{p}.pre.weight", (cfg.width,)
            continue
        yield f"{p}.ff.w1.weight", (cfg.inner, cfg.width)
        yield f"{p}.ff.w2.weight", (cfg.width, cfg.inner)
        yield f"{p}.ff.w3.weight", (cfg.inner, cfg.width)
        for n in ("pre1", "post1", "pre2", "post2"):
            yield f"{p}.{n}.weight", (cfg.width,)
    yield "last_norm.weight", (cfg.width,)


def random_tensors(cfg: ToyConfig, seed: int, *, device="cpu", dtype=torch.float32):
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    for name, shape in tensor_shapes(cfg):
        t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        if len(shape) == 1:
            t = 1.0 + 0.1 * t
        elif ".wq." in name or ".wk." in name:
            t = 0.2 * t                      # peaked attention: one wrong key changes the logits
        else:
            t = 0.06 * t
        yield name, t.to(dtype)


TOY = register_architecture(Architecture(
    name=NAME,
    parse_config=lambda raw, source: ToyConfig.parse(raw, source),
    build_spec=build_spec,
    adapt_tensors=lambda cfg, found: dict(found),
    random_tensors=random_tensors,
))


# ------------------------------------------------------------------------------ the plain forward

def plain_logits(folder, tokens, stored=lambda t: t) -> torch.Tensor:
    """[len(tokens), vocab] float32.  ``stored`` rounds wherever the engine keeps an intermediate
    in its activation dtype."""
    from safetensors import safe_open
    raw = json.loads((folder / "config.json").read_text())
    H, KV, hd, eps, bare = raw["toy_heads"], raw["toy_kv_heads"], raw["toy_head_width"], raw["toy_eps"], raw["toy_bare_layers"]
    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        w = {k: f.get_tensor(k).float() for k in f.keys()}
    S = len(tokens)
    cos, sin = plain_llama.rope_angles(plain_llama.rope_frequencies(hd, raw["toy_theta"], None), torch.arange(S))
    norm = lambda x, name: stored(plain_llama.rms_norm(x, w[name], eps))
    x = w["table.weight"][torch.tensor(list(tokens))]
    for i in range(raw["toy_depth"]):
        p = f"stack.{i}"
        n = norm(x, f"{p}.pre.weight" if i in bare else f"{p}.pre1.weight")
        q = stored(plain_llama.apply_rope(stored(n @ w[f"{p}.mix.wq.weight"].T).view(S, H, hd), cos, sin))
        k = stored(plain_llama.apply_rope(stored(n @ w[f"{p}.mix.wk.weight"].T).view(S, KV, hd), cos, sin))
        v = stored(n @ w[f"{p}.mix.wv.weight"].T).view(S, KV, hd)
        mixed = stored(stored(plain_llama.causal_attention(q, k, v)) @ w[f"{p}.mix.wo.weight"].T)
        if i in bare:
            x = x + mixed
            continue
        h = x + norm(mixed, f"{p}.post1.weight")
        m = norm(h, f"{p}.pre2.weight")
        act = stored(torch.nn.functional.silu(stored(m @ w[f"{p}.ff.w1.weight"].T)) * stored(m @ w[f"{p}.ff.w3.weight"].T))
        x = h + norm(stored(act @ w[f"{p}.ff.w2.weight"].T), f"{p}.post2.weight")
    return norm(x, "last_norm.weight") @ w["table.weight"].T
