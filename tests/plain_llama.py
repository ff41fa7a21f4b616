"""A plain, slow implementation of the Llama-3 dense decoder: the oracle of the tests.

Whole sequences, no cache, no batching, one function per part, float32 unless
told otherwise.  It is written from the reference's formulas (each function
cites torchllms file:line) and shares no code with ``torchllms_b200``: it reads
``config.json`` with ``json`` and ``model.safetensors`` with the ``safetensors``
package.  ``tests/golden/make_golden.py`` compared it once with the reference's
own ``Transformer`` on CPU; ``tests/golden/*.json`` holds that run's outputs.
"""

from __future__ import annotations

import json
import math
import re
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


# ----------------------------------------------------------------------------- parts

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """torchllms/models/networks.py:195-200: normalise in float32, cast back, times weight."""
    xf = x.float()
    normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).type_as(x)
    return normed * weight


def rope_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """torchllms/models/networks.py:253-279: base frequencies and the llama3 three-band rescaling."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type", "default"))
    if kind == "llama3":
        factor = scaling["factor"]
        low = scaling["low_freq_factor"]
        high = scaling["high_freq_factor"]
        old_len = scaling["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv                      # of the unscaled frequencies (:263)
        low_band = wavelen > old_len / low               # long waves: divided by factor (:266)
        high_band = wavelen < old_len / high             # short waves: untouched (:264)
        smooth = (old_len / wavelen - low) / (high - low)
        blended = (1 - smooth) * inv / factor + smooth * inv
        inv = torch.where(low_band, inv / factor, torch.where(high_band, inv, blended))
    elif kind != "default":
        raise ValueError(kind)
    return inv


def rope_angles(inv_freq: torch.Tensor, positions: torch.Tensor):
    """torchllms/models/networks.py:284-297: cos and sin of position * frequency, in float32."""
    ang = positions.float()[:, None] * inv_freq[None, :].float()
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """torchllms/models/networks.py:332-352: rotate adjacent lanes (2i, 2i+1) in float32.
    x: [S, heads, head_dim]; cos, sin: [S, head_dim / 2]."""
    xf = x.float()
    even, odd = xf[..., 0::2], xf[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    out = torch.empty_like(xf)
    out[..., 0::2] = even * c - odd * s
    out[..., 1::2] = odd * c + even * s
    return out.type_as(x)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """torchllms/models/networks.py:355-397 (eager form): query head h uses kv head h // (H / KV)
    (repeat_interleave :371-374), scores / sqrt(head_dim) (:386), causal mask, softmax, times v.
    q: [S, H, hd]; k, v: [S, KV, hd] -> [S, H * hd].  ``window`` (not in the reference) keeps only
    the last ``window`` keys of each query, itself included."""
    S, H, hd = q.shape
    KV = k.shape[1]
    rep = H // KV
    out = torch.zeros(S, H, hd, dtype=torch.float32)
    for h in range(H):
        kh, vh = k[:, h // rep, :].float(), v[:, h // rep, :].float()
        scores = (q[:, h, :].float() @ kh.T) / math.sqrt(hd)
        i = torch.arange(S)[:, None]
        j = torch.arange(S)[None, :]
        hidden = j > i
        if window is not None:
            hidden = hidden | (j <= i - window)
        scores = scores.masked_fill(hidden, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ vh
    return out.reshape(S, H * hd).type_as(q)


def swiglu_ffn(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor) -> torch.Tensor:
    """torchllms/models/networks.py:604-605: w2(silu(w1 x) * w3 x)."""
    return (torch.nn.functional.silu(x @ w1.T) * (x @ w3.T)) @ w2.T


def _same(t: torch.Tensor) -> torch.Tensor:
    return t


def to_bfloat16_and_back(t: torch.Tensor) -> torch.Tensor:
    """What storing an activation in bfloat16 between two kernels does to it."""
    return t.to(torch.bfloat16).to(t.dtype)


def attention_layer(x, wq, wk, wv, wo, cfg, cos, sin, stored=_same, scale=None):
    """torchllms/models/networks.py:513-558: project, view as heads, rope q and k, attend, project.
    ``stored`` is applied wherever the engine keeps an intermediate in its activation dtype.
    ``scale`` ([S, 1], see :func:`weighted_rows`): ``x`` is not normalised yet and the projections
    are multiplied by it."""
    S = x.shape[0]
    q, k, v = stored(x @ wq.T), stored(x @ wk.T), stored(x @ wv.T)
    if scale is not None:
        q, k, v = q * scale, k * scale, stored(v * scale)
    q, k, v = (q.view(S, cfg["n_heads"], cfg["head_dim"]), k.view(S, cfg["n_kv_heads"], cfg["head_dim"]),
               v.view(S, cfg["n_kv_heads"], cfg["head_dim"]))
    q, k = stored(apply_rope(q, cos, sin)), stored(apply_rope(k, cos, sin))
    return stored(stored(causal_attention(q, k, v)) @ wo.T)


def weighted_rows(x: torch.Tensor, weight: torch.Tensor, eps: float):
    """The same norm (torchllms/models/networks.py:195-200) in the order the engine's bfloat16 mode
    takes it when a matrix product follows: the rows are stored as ``x * weight`` and the factor
    ``rsqrt(mean(x^2) + eps)`` is applied to the product instead (a product is linear in its input).
    Returns the weighted rows and the factor ``[S, 1]``."""
    xf = x.float()
    return xf * weight, torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)


def block(x, w: Dict[str, torch.Tensor], prefix: str, cfg, cos, sin, stored=_same):
    """torchllms/models/networks.py:635-644: pre-norm residual block.  With a ``stored`` that rounds
    (the emulation of the engine's bfloat16 mode) the two norms are taken in the engine's order
    (:func:`weighted_rows`); in float32 both orders are the same numbers up to rounding and the
    reference's is kept."""
    g = lambda n: w[f"{prefix}.{n}"]
    if stored is _same:
        h = x + attention_layer(rms_norm(x, g("attention_norm.weight"), cfg["eps"]),
                                g("attention.wq.weight"), g("attention.wk.weight"),
                                g("attention.wv.weight"), g("attention.wo.weight"), cfg, cos, sin)
        n = rms_norm(h, g("ffn_norm.weight"), cfg["eps"])
        return h + swiglu_ffn(n, g("feed_forward.w1.weight"), g("feed_forward.w2.weight"), g("feed_forward.w3.weight"))
    n, scale = weighted_rows(x, g("attention_norm.weight"), cfg["eps"])
    h = x + attention_layer(stored(n), g("attention.wq.weight"), g("attention.wk.weight"),
                            g("attention.wv.weight"), g("attention.wo.weight"), cfg, cos, sin, stored, scale)
    n, scale = weighted_rows(h, g("ffn_norm.weight"), cfg["eps"])
    n = stored(n)
    gate, up = stored(n @ g("feed_forward.w1.weight").T) * scale, stored(n @ g("feed_forward.w3.weight").T) * scale
    act = stored(torch.nn.functional.silu(gate) * up)           # :604-605
    return h + stored(act @ g("feed_forward.w2.weight").T)


def forward_logits(w: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int], stored=_same,
                   rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """torchllms/models/networks.py:1017-1047: embed, blocks, final norm, head (tied :806-809).
    Returns [len(tokens), vocab] logits for the whole sequence (with ``rows``: the head is applied
    to those positions only, :1030-1045 keeps rows the same way).

    With ``stored=to_bfloat16_and_back`` (and bfloat16-valued weights) this is the arithmetic of
    the engine's bfloat16 mode: float32 residual stream, norms, rotation, softmax and sums, with
    every intermediate that crosses from one kernel to the next rounded to bfloat16."""
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["tok_embeddings.weight"][ids]
    inv = rope_frequencies(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
    cos, sin = rope_angles(inv, torch.arange(len(ids)))
    for i in range(cfg["n_layers"]):
        x = block(x, w, f"layers.{i}", cfg, cos, sin, stored)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    x = stored(rms_norm(x, w["norm.weight"], cfg["eps"]))
    head = w["tok_embeddings.weight"] if cfg["tie"] else w["output.weight"]
    return x @ head.T


# ------------------------------------------------------------------ reading a model folder

_HF_LAYER = {
    "self_attn.q_proj.weight": "attention.wq.weight", "self_attn.k_proj.weight": "attention.wk.weight",
    "self_attn.v_proj.weight": "attention.wv.weight", "self_attn.o_proj.weight": "attention.wo.weight",
    "mlp.gate_proj.weight": "feed_forward.w1.weight", "mlp.up_proj.weight": "feed_forward.w3.weight",
    "mlp.down_proj.weight": "feed_forward.w2.weight", "input_layernorm.weight": "attention_norm.weight",
    "post_attention_layernorm.weight": "ffn_norm.weight",
}


def read_config(folder) -> dict:
    """Hugging Face keys -> the numbers above (torchllms/models/checkpoint_converter.py:359-397)."""
    raw = json.loads((Path(folder) / "config.json").read_text())
    heads = raw["num_attention_heads"]
    return {
        "n_layers": raw["num_hidden_layers"], "dim": raw["hidden_size"], "n_heads": heads,
        "n_kv_heads": raw.get("num_key_value_heads", heads),
        "head_dim": raw.get("head_dim") or raw["hidden_size"] // heads,
        "vocab": raw["vocab_size"], "eps": raw["rms_norm_eps"], "rope_theta": raw["rope_theta"],
        "rope_scaling": raw.get("rope_scaling"), "tie": raw.get("tie_word_embeddings", False),
    }


def read_weights(folder, cfg: dict, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Tensors by torchllms name; Hugging Face names are mapped and their q/k rows permuted to the
    adjacent-lane order (torchllms/models/checkpoint_converter.py:96-108, :124-141, :172-178)."""
    out: Dict[str, torch.Tensor] = {}
    with safe_open(str(Path(folder) / "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            t = f.get_tensor(name).to(dtype)
            m = re.match(r"^model\.layers\.(\d+)\.(.+)$", name)
            if m and m.group(2) in _HF_LAYER:
                new = f"layers.{m.group(1)}.{_HF_LAYER[m.group(2)]}"
                if m.group(2).startswith("self_attn.q_proj") or m.group(2).startswith("self_attn.k_proj"):
                    hd = cfg["head_dim"]
                    n = t.shape[0] // hd
                    t = t.view(n, 2, hd // 2, t.shape[1]).transpose(1, 2).reshape(n * hd, t.shape[1])
                out[new] = t
            elif name == "model.embed_tokens.weight":
                out["tok_embeddings.weight"] = t
            elif name == "model.norm.weight":
                out["norm.weight"] = t
            elif name == "lm_head.weight":
                out["output.weight"] = t
            else:
                out[name] = t
    return out


class PlainModel:
    def __init__(self, folder, dtype=torch.float32):
        self.cfg = read_config(folder)
        self.weights = read_weights(folder, self.cfg, dtype)

    @torch.no_grad()
    def logits(self, tokens: Sequence[int], stored=_same, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
        return forward_logits(self.weights, self.cfg, tokens, stored, rows).float()

    @torch.no_grad()
    def greedy(self, prompt: Sequence[int], n_new: int) -> List[int]:
        seq = list(prompt)
        for _ in range(n_new):
            seq.append(int(torch.argmax(self.logits(seq)[-1])))
        return seq[len(prompt):]
