"""The Python entry point: load a model, generate for prompts or conversations.

Reference: ``LLM`` (torchllms/inference/llm.py:80-1152).  Argument names and meanings follow
its ``__init__`` (:95-109: ``ckpt_paths, template_config, eos_ids, max_len, max_bsz, device,
precision, model_kwargs, batched, prefix_cache, page_size, kv_memory_gb``) and ``generate`` (:693-700, :1074-1083:
``prompts`` or ``conversations``, ``temperature``, ``max_new_tokens``, ``batch_size``,
``disable_tqdm``), and results are its ``GenerationResult`` (:63-77).  Differences: every call
runs through the continuous-batching scheduler (the reference's ``batched`` switch chose between
a one-by-one loop and static batches), token ids may be given directly, and sampling takes a
seed.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from ..engine.loading import load_model, model_dir_of, parse_dtype, random_model
from ..engine.scheduler import Request, Scheduler
from ..engine.step import Engine
from ..kernels import get_ops
from ..sampling.sampler import Sampler, SamplingParams
from .template import ChatTemplate, get_template


@dataclass
class GenerationResult:
    """``token_ids`` includes the stop token when generation stopped on a stop id; ``text`` is
    decoded without special tokens (empty when the model folder has no tokenizer);
    ``stop_reason`` is the stop id that fired, or ``None`` when the token budget or the length
    limit ended the request (torchllms/inference/llm.py:63-77).  ``error`` is set when the request
    could not run at all."""

    text: str
    token_ids: List[int]
    stop_reason: Optional[int]
    error: Optional[str] = None


class LLM:
    def __init__(
        self,
        ckpt_paths: Union[str, Path, Sequence[Union[str, Path]], None] = None,
        template_config: Optional[str] = None,
        eos_ids: Optional[List[int]] = None,
        max_len: int = 4096,
        max_bsz: int = 4,
        device: str = "cuda",
        precision: Optional[str] = "bfloat16",
        model_kwargs: Optional[Dict[str, Any]] = None,
        batched: bool = True,
        prefix_cache: Any = None,
        page_size: int = 16,
        kv_memory_gb: Optional[float] = None,
        kv_memory_fraction: Optional[float] = None,
        *,
        max_num_batched_tokens: int = 2048,
        prefill_chunk: Optional[int] = None,
        seed: int = 0,
        look_ahead: bool = True,
        config=None,
        random_seed: Optional[int] = None,
        ops=None,
    ):
        """``ckpt_paths``: a model folder (``config.json`` + ``model.safetensors``), a file in
        one, or a list of them loaded in order, later tensors overriding earlier ones (the
        configuration is read beside the first).  Alternatively ``config`` and ``random_seed``
        build a model with random weights on the device.  ``max_bsz`` is the number of requests
        that may run at once; the cache holds ``max_bsz * max_len`` tokens unless ``kv_memory_fraction``
        (a share of the device memory that is free once the weights are loaded) or ``kv_memory_gb``
        gives its size in GiB (torchllms/models/networks.py:872-884)."""
        if prefix_cache is not None:
            # the reference's argument at its place in the list; this engine keeps no cache of prefixes
            raise ValueError("prefix_cache: this engine has no prefix cache; leave it None")
        ops = ops or get_ops()
        precision = precision or "bfloat16"
        self.dtype = parse_dtype(precision)
        ops.prepare(self.dtype)
        if ckpt_paths is not None:
            paths = [ckpt_paths] if isinstance(ckpt_paths, (str, Path)) else list(ckpt_paths)
            self.model_dir: Optional[Path] = model_dir_of(paths[0])
            self.arch, self.config, self.model = load_model(
                paths, dtype=self.dtype, device=device, overrides=model_kwargs, max_positions=max_len, ops=ops)
        elif config is not None:
            self.model_dir = None
            config = config.with_overrides(model_kwargs)
            self.arch, self.config, self.model = random_model(
                config, random_seed or 0, dtype=self.dtype, device=device, max_positions=max_len, ops=ops)
        else:
            raise ValueError("give ckpt_paths (a model folder) or config and random_seed")
        self.max_len = int(max_len)
        self.max_bsz = int(max_bsz)
        self.device = device
        self.seed = int(seed)
        self.batched = batched
        bytes_per_token = sum(g_need.n_kv_heads * g_need.head_dim * 2 * n_runs for g_need, n_runs in self._kv_layout())
        bytes_per_token *= torch.empty((), dtype=self.dtype).element_size()
        if kv_memory_gb is not None and kv_memory_fraction is not None:
            raise ValueError("give kv_memory_gb or kv_memory_fraction, not both")
        if kv_memory_fraction is not None:
            # a share of what the device has free now that the weights are on it
            if not 0.0 < float(kv_memory_fraction) <= 1.0:
                raise ValueError(f"kv_memory_fraction must lie in (0, 1], got {kv_memory_fraction}")
            if self.model.device.type != "cuda":
                raise ValueError("kv_memory_fraction needs a CUDA device to ask for its free memory")
            free_bytes, _total = torch.cuda.mem_get_info(self.model.device)
            pool_tokens = max(int(float(kv_memory_fraction) * free_bytes) // max(bytes_per_token, 1), page_size)
        elif kv_memory_gb is None:
            pool_tokens = self.max_bsz * self.max_len
        else:
            pool_tokens = max(int(kv_memory_gb * (1 << 30)) // max(bytes_per_token, 1), page_size)
        self.engine = Engine(self.model, page_size=page_size, pool_tokens=pool_tokens, max_num_seqs=self.max_bsz,
                             max_len=self.max_len, max_step_tokens=max(max_num_batched_tokens, 1))
        self.sampler = Sampler(ops, self.model.device)
        self.max_num_batched_tokens = max_num_batched_tokens
        self.look_ahead = bool(look_ahead)      # launch a decode step before the one before it is read back
        self.prefill_chunk = prefill_chunk

        self.template: Optional[ChatTemplate] = get_template(template_config) if template_config else None
        self._tokenizer = None
        if self.template is not None and self.template.stop_token_ids:
            eos_ids = list(self.template.stop_token_ids)           # the template's stop ids win (:188-189)
        elif self.template is None and self.arch.chat_template and self._load_tokenizer(required=False) is not None:
            # no template named: a folder with a tokenizer gets its architecture's; the caller's stop ids stand
            self.template = get_template(self.arch.chat_template)
            if eos_ids is None and self.template.stop_token_ids:
                eos_ids = list(self.template.stop_token_ids)
        if eos_ids is None:
            tok = self._load_tokenizer(required=False)
            eos_ids = [tok.eos_token_id] if tok is not None and tok.eos_token_id is not None else []
        self.eos_ids = list(eos_ids)
        self.eos_set = set(self.eos_ids)
        self.last_stats = None
        self.last_trace = None

    def warmup(self, batch_sizes: Optional[Sequence[int]] = None, context_lengths: Optional[Sequence[int]] = None) -> int:
        """Record the CUDA graphs of decode steps for these numbers of running requests (default:
        every number up to ``max_bsz``) before the first request arrives; returns how many exist.
        A step of few requests plans its attention for the power of two that holds its longest
        context, so for those there is one graph per such bound: all of them are recorded, or only
        those that ``context_lengths`` names (the others then the second time they occur)."""
        sizes = list(batch_sizes) if batch_sizes is not None else list(range(1, self.max_bsz + 1))
        return self.engine.capture_decode_graphs(sizes, context_lengths)

    def _kv_layout(self):
        needs: Dict[Any, int] = {}
        for need, _state, cache_of in self.model.run_needs():
            if need is not None and cache_of is None:
                needs[need] = needs.get(need, 0) + 1
        return list(needs.items())

    # ---------------------------------------------------------------- text <-> ids
    def _load_tokenizer(self, required: bool = True):
        if self._tokenizer is None and self.model_dir is not None:
            has = any((self.model_dir / n).is_file() for n in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json"))
            if has:
                from transformers import AutoTokenizer
                self._tokenizer = AutoTokenizer.from_pretrained(str(self.model_dir))
        if self._tokenizer is None and required:
            raise ValueError("this model folder has no tokenizer: pass prompt_token_ids instead of text")
        return self._tokenizer

    def tokenize_conversation(self, conversation: Sequence[Dict[str, str]]) -> List[int]:
        if self.template is None:
            raise ValueError("conversations need a template (template_config='llama3_instruct')")
        tok = self._load_tokenizer()
        return tok(self.template.render(conversation), add_special_tokens=False).input_ids

    # -------------------------------------------------------------------- generate
    @torch.no_grad()
    def generate(
        self,
        prompts: Optional[List[str]] = None,
        conversations: Optional[List[List[Dict[str, str]]]] = None,
        temperature: float = 0.0,
        max_new_tokens: Optional[int] = None,
        batch_size: int = 0,
        disable_tqdm: bool = False,
        *,
        prompt_token_ids: Optional[List[List[int]]] = None,
        top_k: Optional[int] = None,
        seed: Optional[int] = None,
    ) -> List[GenerationResult]:
        """One result per input, in input order.  ``temperature`` 0 is greedy.  ``batch_size``
        bounds how many requests run at once (0: ``max_bsz``).  Unless ``disable_tqdm``, a progress
        bar on standard error counts the finished requests (torchllms/inference/llm.py:1126-1130; there it counts static batches)."""
        given = [x is not None for x in (prompts, conversations, prompt_token_ids)]
        if sum(given) != 1:
            raise ValueError("give exactly one of prompts, conversations and prompt_token_ids")
        if conversations is not None:
            encoded = [self.tokenize_conversation(c) for c in conversations]
        elif prompts is not None:
            tok = self._load_tokenizer()
            encoded = [list(ids) for ids in tok(prompts, add_special_tokens=False).input_ids]
        else:
            encoded = [list(map(int, ids)) for ids in prompt_token_ids]
        sampling = SamplingParams(float(temperature), top_k, self.seed if seed is None else int(seed))
        requests = []
        for i, ids in enumerate(encoded):
            budget = self.max_len - len(ids)
            if max_new_tokens is not None:
                budget = min(budget, int(max_new_tokens))
            requests.append(Request(index=i, prompt=ids, budget=budget, sampling=sampling))
        scheduler = Scheduler(self.engine, self.sampler,
                              max_num_seqs=min(batch_size, self.max_bsz) if batch_size else self.max_bsz,
                              max_num_batched_tokens=self.max_num_batched_tokens,
                              prefill_chunk=self.prefill_chunk, eos_ids=self.eos_set, look_ahead=self.look_ahead)
        bar = None
        if not disable_tqdm and len(requests) > 1:
            try:
                from tqdm import tqdm
                bar = tqdm(total=len(requests), desc="generate", unit="req")
            except ImportError:
                bar = None
        try:
            for r in requests:
                scheduler.add(r)
            if bar is not None:
                bar.update(sum(1 for r in requests if r.finished))      # nothing to generate, or refused
            while scheduler.has_work():
                done = scheduler.step()
                if bar is not None and done:
                    bar.update(len(done))
        finally:
            if bar is not None:
                bar.close()
            for r in requests:                      # whatever happened, give the pages back
                if r.handle is not None:
                    self.engine.release(r.handle)
                    r.handle = None
        self.last_stats = scheduler.stats
        self.last_trace = scheduler.trace          # per step: (request's place in the call, tokens it brought)
        tok = self._load_tokenizer(required=False)
        out = []
        for r in requests:
            text = tok.decode(r.generated, skip_special_tokens=True) if tok is not None else ""
            out.append(GenerationResult(text=text, token_ids=list(r.generated), stop_reason=r.stop_reason, error=r.error))
        return out
