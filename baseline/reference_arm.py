#!/usr/bin/env python3
"""The reference arm of ``bench.py``: the unmodified normster/torchllms, installed under
``baseline/_ref``, driven through its own public API on the headline workload.

    python baseline/reference_arm.py --steps K --warmup W [--batch 8] [--layers 32]

Nothing of ``torchllms_b200`` is imported here: the only code on the path is the reference's
(``from torchllms.inference import LLM``) and the libraries it calls (FlashInfer for paged
attention, cuBLAS through ``nn.Linear``).  What the reference's ``LLM`` wants and an offline box
does not have is made in a temporary folder first:

``params.json``
    the Llama-3.1-8B shape in the reference's own keys (torchllms/models/networks.py:110-157).
``consolidated.00.pth``
    every parameter of the reference's ``Transformer`` drawn as its ``init_module`` draws them
    (N(0, 0.02); torchllms/models/utils.py:197-214) in bfloat16, norm weights one.
``tokenizer.json``
    a word-level tokenizer with the words ``t0 .. t<vocab-1>``, so that the text ``"t17 t9"``
    is the token ids 17, 9: the reference's ``generate`` takes text only
    (torchllms/inference/llm.py:1103-1110).

Then ``LLM(ckpt_paths=[...], batched=True, max_bsz=B, max_len=8192).generate(prompts=...,
temperature=0.0, max_new_tokens=n)`` runs its stock path: one flat-packed prefill of the whole
batch, then one forward per decoded token with a host read-back each (torchllms/inference/llm.py:
946-981).  A decode step's time is the difference between a run that generates ``1 + W + K``
tokens and one that generates ``1 + W``, divided by K, so the prefill and the first W steps drop
out; it is taken with CUDA events (``value``) and with the host clock (``e2e``): the reference
reads every step's tokens back, so the two agree.  Both of the reference's ways of decoding are
measured: its default (eager) and its opt-in ``LLM.enable_decode_compile()`` (``torch.compile`` of
the one-token forward with CUDA graphs, torchllms/inference/llm.py:202-243); the faster one is the
line's ``value``, both stand under ``decode_ways``.  One JSON line is printed.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

PROMPT_LEN = 2048
CONTEXT = 8192
PARAMS_8B = {
    "dim": 4096, "n_layers": 32, "n_heads": 32, "n_kv_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "multiple_of": 256, "ffn_dim_multiplier": 3.5,          # int(3.5 * 4096) = 14336
    "norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": False, "max_seq_len": CONTEXT,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}


def say(msg: str) -> None:
    print(f"[reference arm] {msg}", file=sys.stderr, flush=True)


def scratch_dir(need_bytes: int) -> Path:
    for base in (tempfile.gettempdir(), "/dev/shm"):
        try:
            if shutil.disk_usage(base).free > need_bytes * 1.1:
                return Path(tempfile.mkdtemp(prefix="torchllms_ref_", dir=base))
        except OSError:
            continue
    raise RuntimeError(f"no temporary folder with {need_bytes / 2**30:.0f} GiB free for the reference's checkpoint")


def write_tokenizer(folder: Path, vocab: int) -> None:
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit
    tok = Tokenizer(WordLevel({f"t{i}": i for i in range(vocab)}, unk_token="t0"))
    tok.pre_tokenizer = WhitespaceSplit()
    tok.save(str(folder / "tokenizer.json"))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": f"t{vocab - 1}", "unk_token": "t0",
         "model_max_length": 1 << 20}))


def write_checkpoint(folder: Path, params: dict) -> int:
    """Every parameter of the reference's own model class, by its own names and shapes."""
    import torch
    from torchllms.models.networks import ModelParams, Transformer
    with torch.device("meta"):
        meta = Transformer.from_params(ModelParams(**params))
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    state, total = {}, 0
    for name, p in meta.named_parameters():
        if p.dim() == 1:                                   # RMSNorm weights: ones (torchllms/models/networks.py:192-193)
            t = torch.ones(p.shape, dtype=torch.bfloat16)
        else:                                              # Linear and Embedding: N(0, 0.02) (torchllms/models/utils.py:202-207)
            t = (torch.randn(p.shape, generator=gen, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()
        state[name] = t
        total += t.numel() * 2
    torch.save(state, str(folder / "consolidated.00.pth"))
    return total


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=PARAMS_8B["n_layers"])
    ap.add_argument("--no-decode-compile", action="store_true",
                    help="measure the reference's default (eager) decoding only; without this flag its opt-in "
                         "LLM.enable_decode_compile() is measured too and the faster of the two is the headline")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    sys.path.insert(0, str(REF))
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    import torch
    import torchllms
    assert Path(torchllms.__file__).resolve().is_relative_to(REF.resolve()), "not the install under baseline/_ref"
    from torchllms.inference import LLM

    params = dict(PARAMS_8B, n_layers=args.layers)
    n_weights = args.layers * (4096 * 128 * (2 * 32 + 2 * 8) + 3 * 4096 * 14336) + 2 * 128256 * 4096
    folder = scratch_dir(2 * n_weights)
    level = "LLM.generate (batched)"
    try:
        say(f"writing params.json, tokenizer and a {2 * n_weights / 2**30:.1f} GiB checkpoint to {folder}")
        (folder / "params.json").write_text(json.dumps(params))
        write_tokenizer(folder, params["vocab_size"])
        t0 = time.time()
        write_checkpoint(folder, params)
        say(f"checkpoint written in {time.time() - t0:.0f} s; loading the reference's LLM")
        kw = dict(ckpt_paths=[str(folder / "consolidated.00.pth")], template_config=None, eos_ids=[], max_len=CONTEXT,
                  max_bsz=args.batch, device="cuda", precision="bfloat16", model_kwargs={"max_seq_len": CONTEXT},
                  page_size=16)
        try:
            llm = LLM(batched=True, **kw)
        except AttributeError as e:
            # torchllms/inference/llm.py:181-186 names AttentionImpl.FLEX, which the enum
            # (torchllms/models/networks.py:104-107) does not have, so batched=True cannot be
            # constructed.  The constructor's only other use of the flag is to store it: set it after.
            say(f"LLM(batched=True) raised {type(e).__name__}: {e}; constructing with batched=False and setting llm.batched")
            llm = LLM(batched=False, **kw)
            llm.batched = True
            level = "LLM.generate (batched flag set after construction: LLM(batched=True) raises AttributeError on AttentionImpl.FLEX)"
    finally:
        # the weights are on the device now (torch.load(mmap=True) + assign kept no file open that matters)
        pass

    gen = torch.Generator().manual_seed(1234)

    def prompts(n, length):
        ids = torch.randint(0, params["vocab_size"], (n, length), generator=gen).tolist()
        return [" ".join(f"t{i}" for i in row) for row in ids]

    def run(texts, n_new):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.time()
        a.record()
        out = llm.generate(prompts=texts, temperature=0.0, max_new_tokens=n_new, disable_tqdm=True)
        b.record()
        torch.cuda.synchronize()
        t1 = time.time()
        assert all(len(r.token_ids) == n_new for r in out), [len(r.token_ids) for r in out]
        return a.elapsed_time(b), (t1 - t0) * 1e3, t0, t1

    say("warming up (the attention library compiles its kernels at first use)")
    t0 = time.time()
    run(prompts(args.batch, 64), 4)
    say(f"first call took {time.time() - t0:.0f} s")
    batch = prompts(args.batch, PROMPT_LEN)

    def decode_step_ms():
        """(device ms, wall ms, start, end) of one decode step: generate(1 + W + K) minus generate(1 + W), over K;
        the median of three runs on either side.  None when the difference is not positive: the K steps
        were lost in the run-to-run spread of the prefill then, and nothing was measured."""
        for _ in range(2):
            run(batch, 1 + args.warmup)
        short = sorted(run(batch, 1 + args.warmup)[:2] for _ in range(3))[1]
        long_ = sorted((run(batch, 1 + args.warmup + args.steps) for _ in range(3)), key=lambda r: r[0])[1]
        dev_ms, wall_ms, t_start, t_end = long_
        if dev_ms <= short[0] or wall_ms <= short[1]:
            return None
        return (dev_ms - short[0]) / args.steps, (wall_ms - short[1]) / args.steps, t_start, t_end

    ways = {"eager": decode_step_ms()}
    one = prompts(1, PROMPT_LEN)
    run(one, 1)
    pre_ms = sorted(run(one, 1)[0] for _ in range(5))[2]
    if not args.no_decode_compile:
        # the reference's own faster way of decoding, opt-in through its public API
        # (torchllms/inference/llm.py:202-243: torch.compile of the one-token forward with CUDA graphs)
        try:
            say("enable_decode_compile(): compiling the decode step")
            t0 = time.time()
            llm.enable_decode_compile()
            run(prompts(args.batch, 64), 8)
            say(f"compiled in {time.time() - t0:.0f} s")
            ways["decode_compile"] = decode_step_ms()
        except Exception as e:      # the compiler is the reference's to get right; its default stands then
            say(f"enable_decode_compile() failed: {type(e).__name__}: {str(e)[:200]}")
            llm.disable_decode_compile()
    lost = sorted(k for k, v in ways.items() if v is None)
    ways = {k: v for k, v in ways.items() if v is not None}
    if not ways:
        shutil.rmtree(folder, ignore_errors=True)
        print(json.dumps({"impl": "reference", "unavailable": f"{args.steps} decode steps were lost in the spread of the prefill's time: give more --steps"}))
        return 0
    best = min(ways, key=lambda k: ways[k][0])
    ms_dev, ms_wall, t_start, t_end = ways[best]
    level += f"; decoding: {best}" + ("" if len(ways) == 1 else f" (the faster of {' and '.join(sorted(ways))})")
    shutil.rmtree(folder, ignore_errors=True)
    print(json.dumps({
        "impl": "reference",
        "metric": f"decode tok/s at batch {args.batch} (Llama-3.1-8B shape, {PROMPT_LEN:,}-token prompts)",
        "value": round(args.batch / (ms_dev / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_dev, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights N(0, 0.02))",
        "config": {"model": "llama-3.1-8b-shape", "n_layers": args.layers, "n_layers_full": PARAMS_8B["n_layers"],
                   "dim": 4096, "n_heads": 32, "n_kv_heads": 8, "head_dim": 128, "ffn_hidden": 14336,
                   "vocab_size": 128256, "global_batch": args.batch, "seq_len": PROMPT_LEN, "context": CONTEXT,
                   "page_size": 16, "parallelism": "single-gpu", "level": level,
                   "timing": "generate(1+W+K tokens) minus generate(1+W tokens), over K",
                   "l2": "inputs larger than L2 (16 GB of weights per step)"},
        "e2e": {"value": round(args.batch / (ms_wall / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 8 * args.batch, "d2h_bytes_per_step": 8 * args.batch},
        "prefill": {"value": round(PROMPT_LEN / (pre_ms / 1e3), 1), "tokens": PROMPT_LEN, "ms": round(pre_ms, 3),
                    "note": "generate() of one 2,048-token prompt and one new token: prefill, sampling and read-back"},
        "decode_ways_unmeasured": lost,
        "decode_ways": {k: {"ms_per_step": round(v[0], 4), "tokens_per_s": round(args.batch / (v[0] / 1e3), 1),
                            "e2e_tokens_per_s": round(args.batch / (v[1] / 1e3), 1)} for k, v in ways.items()},
        "timed_window": [t_start, t_end],
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
