#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
    python bench.py --workload serve_1b | long_3b      (secondary: whole serving runs, a JSON line each)

The workload is the Llama-3.1-8B shape (32 layers, dim 4096, 32 heads, 8 kv heads, head_dim 128,
SwiGLU hidden 14336, vocabulary 128256, llama3 rope scaling, untied head) in bfloat16 with random
weights and synthetic token ids: requests with 2,048-token prompts decode with a batch of 8
(headline ``value``), of 1 and of 64 (``points``), and one 2,048-token prompt is prefilled
(``prefill``).  A step is one decode step.  One JSON line is printed.

``value`` times K decode steps on the device with CUDA events (engine step plus the sampling
kernel; the tokens fed are host lists prepared beforehand, so the device never waits for a
read-back).  ``e2e`` is the same batch through ``LLM.generate``: scheduler, upload of each step's
index data from pinned memory, sampling, and the read-back of the sampled tokens every step
(the batch's prompts are prefilled together in one step, as the reference's static batches are,
so that all of them decode side by side for the whole timed part; the scheduler puts a step on
the device before it has read the tokens of the step before, which the read-back then overlaps).
Every decode step streams all weights (16 GB, far more than the 126 MB L2), so no L2 flush is
needed between timed iterations.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPE_8B = dict(n_layers=32, dim=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn_hidden=14336,
                vocab_size=128256, norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=False)
ROPE_8B = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
               original_max_position_embeddings=8192)
PROMPT_LEN = 2048
CONTEXT = 8192
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                    "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines = []
        self.proc = None
        self.window = None      # (start, end) of the timed region, host clock

    def mark(self, start: float, end: float):
        self.window = (start, end)

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0],
                 f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, max_mhz, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        import datetime
        rows = []
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((stamp, int(float(parts[1])), int(float(parts[2])), parts[3:7]))
            except ValueError:
                continue
        inside = rows
        if self.window is not None:
            for slack in (0.0, 0.25, 1.0):      # a short region may fall between two samples
                inside = [r for r in rows if self.window[0] - slack <= r[0] <= self.window[1] + slack]
                if inside:
                    break
        for _stamp, sm, sm_max, flags in inside:
            mhz.append(sm)
            max_mhz = max(max_mhz, sm_max)
            for name, flag in zip(names, flags):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max_mhz or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def reference_arm(args):
    """The unmodified reference through its own public API, installed under baseline/_ref
    (pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <reference>, plus its
    data folder torchllms/messages/configs, which the wheel leaves out).  It runs in a process of its
    own (``baseline/reference_arm.py``) so that nothing of this package is on its path; this process
    only samples the clocks meanwhile and passes the line on.  Anything that keeps it from running is
    reported as ``unavailable``."""
    ref = ROOT / "baseline" / "_ref"
    script = ROOT / "baseline" / "reference_arm.py"
    if not (ref / "torchllms").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "reference not installed under baseline/_ref"}))
        return 0
    if not (ref / "torchllms" / "messages" / "configs").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "installed reference lacks torchllms/messages/configs (data the wheel leaves out)"}))
        return 0
    cmd = [sys.executable, str(script), "--steps", str(args.steps), "--warmup", str(args.warmup),
           "--batch", str(args.batch), "--layers", str(args.layers)]
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    with ClockSampler() as clocks:
        try:
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=env, cwd=str(ROOT / "baseline"))
        except subprocess.TimeoutExpired:
            print(json.dumps({"impl": "reference", "unavailable": "the reference run did not finish within 1500 s"}))
            return 0
        time.sleep(0.15)
    sys.stderr.write(proc.stderr[-4000:])
    line = None
    for text in reversed(proc.stdout.strip().splitlines()):
        if text.startswith("{"):
            try:
                line = json.loads(text)
                break
            except ValueError:
                continue
    if proc.returncode != 0 or line is None or "value" not in line:
        tail = " | ".join(l.strip() for l in proc.stderr.strip().splitlines()[-3:])[-300:]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference run exited {proc.returncode}: {tail}"}))
        return 0
    window = line.pop("timed_window", None)
    if window:
        clocks.mark(window[0], window[1])
    line["clocks"] = clocks.summary()
    line["gpu_launches"] = 0          # this arm launches none of this repository's kernels
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------- secondary serving workloads
SERVE = {
    # 64 requests at once, prompts uniform in 128..4096, 256 new tokens each, greedy: chunked prefill beside decoding
    "serve_1b": dict(shape=dict(n_layers=16, dim=2048, n_heads=32, n_kv_heads=8, head_dim=64, ffn_hidden=8192,
                                vocab_size=128256, norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True),
                     rope=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                               original_max_position_embeddings=8192),
                     requests=64, prompt=(128, 4096), new_tokens=256, temperature=0.0, name="llama-3.2-1b-shape"),
    # 32 requests with 16,384-token prompts, 512 new tokens each at temperature 1
    "long_3b": dict(shape=dict(n_layers=28, dim=3072, n_heads=24, n_kv_heads=8, head_dim=128, ffn_hidden=8192,
                               vocab_size=128256, norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True),
                    rope=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                              original_max_position_embeddings=8192),
                    requests=32, prompt=(16384, 16384), new_tokens=512, temperature=1.0, name="llama-3.2-3b-shape"),
}


def serving_workload(args, peaks):
    """A whole serving run through ``LLM.generate`` (continuous batching, prompts cut into portions of
    2,048 tokens beside decoded tokens): the record with tokens per second, wall clock around the call
    (host token lists in, host token lists out), and how that compares with what the run's arithmetic
    and memory traffic take at the peaks: ``flop_seconds`` (every token through every weight, causal
    attention) at the sustained tensor-core peak, ``byte_seconds`` (every step reads the weights once
    and the cache of the requests it holds) at the copy bandwidth, ``roofline_frac`` the larger of the
    two over the measured seconds."""
    import random

    import torch
    from torchllms_b200.models.llama_config import LlamaConfig, RopeScaling
    from torchllms_b200.inference import LLM

    w = SERVE[args.workload]
    lo, hi = w["prompt"]
    max_len = hi + w["new_tokens"] + 16
    cfg = LlamaConfig(architecture="LlamaForCausalLM", rope_scaling=RopeScaling(**w["rope"]), max_seq_len=max_len, **w["shape"])
    llm = LLM(config=cfg, random_seed=0, precision="bfloat16", max_len=max_len, max_bsz=w["requests"],
              max_num_batched_tokens=2048 + w["requests"], prefill_chunk=2048, page_size=16)
    llm.warmup()
    rng = random.Random(0)
    gen = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (rng.randint(lo, hi),), generator=gen).tolist() for _ in range(w["requests"])]
    llm.generate(prompt_token_ids=[p[:64] for p in prompts[:4]], max_new_tokens=4, disable_tqdm=True)      # warm the path
    ops = llm.model.ops
    launches0 = ops.launches
    with ClockSampler() as clocks:
        torch.cuda.synchronize()
        t0 = time.time()
        out = llm.generate(prompt_token_ids=prompts, max_new_tokens=w["new_tokens"], temperature=w["temperature"], seed=1, disable_tqdm=True)
        torch.cuda.synchronize()
        t1 = time.time()
        clocks.mark(t0, t1)
        time.sleep(0.15)
    st = llm.last_stats
    ops.check_status()
    n_prompt = sum(len(p) for p in prompts)
    n_new = sum(len(o.token_ids) for o in out)
    secs = t1 - t0
    # what the run had to compute and to read, from the steps the scheduler took
    per_token_flops = 2 * (cfg.n_layers * (cfg.dim * cfg.head_dim * (2 * cfg.n_heads + 2 * cfg.n_kv_heads) + 3 * cfg.dim * cfg.ffn_hidden))
    kv_bytes_per_token = cfg.n_layers * 2 * cfg.n_kv_heads * cfg.head_dim * 2
    weight_bytes = llm.model.weight_bytes()
    held, flops, byts = {}, 0.0, 0.0
    for step in llm.last_trace:
        byts += weight_bytes
        for idx, n in step:
            before = held.get(idx, 0)
            held[idx] = before + n
            flops += n * per_token_flops + 4 * cfg.n_layers * cfg.n_heads * cfg.head_dim * (n * before + n * (n + 1) / 2)
            byts += (before + n) * kv_bytes_per_token
        flops += 2 * cfg.dim * cfg.vocab_size * sum(1 for _ in step)          # the head, on one row per request at most
    flop_s = flops / (peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * 1e12)
    byte_s = byts / (peaks["hbm_gbs"] * 1e9)
    return ({
        "metric": f"tokens/s through LLM.generate, {args.workload} (prompt and generated tokens)",
        "value": round((n_prompt + n_new) / secs, 1), "unit": "tokens/s", "n_gpus": 1, "steps": st.steps, "warmup": 1,
        "ms_per_step": round(secs * 1e3 / max(st.steps, 1), 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights N(0, 0.02))",
        "generated_tokens_per_s": round(n_new / secs, 1), "seconds": round(secs, 3),
        "config": {"model": w["name"], "n_layers": cfg.n_layers, "dim": cfg.dim, "n_heads": cfg.n_heads,
                   "n_kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim, "ffn_hidden": cfg.ffn_hidden,
                   "vocab_size": cfg.vocab_size, "global_batch": w["requests"], "prompt_min": lo, "prompt_max": hi,
                   "new_tokens": w["new_tokens"], "temperature": w["temperature"], "prefill_chunk": 2048,
                   "page_size": 16, "prompt_tokens": n_prompt, "parallelism": "single-gpu"},
        "gpu_launches": ops.launches - launches0, "preemptions": st.preemptions, "clocks": clocks.summary(),
        "flop_seconds": round(flop_s, 3), "byte_seconds": round(byte_s, 3), "roofline_frac": round(max(flop_s, byte_s) / secs, 4),
        "peaks": peaks["source"],
    })


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=SHAPE_8B["n_layers"], help="fewer layers than the shape has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch and the prefill")
    ap.add_argument("--workload", default="decode_8b", choices=["decode_8b"] + sorted(SERVE),
                    help="decode_8b: the headline (default); serve_1b, long_3b: whole serving runs through LLM.generate")
    ap.add_argument("--context-len", type=int, default=PROMPT_LEN,
                    help="prompt length of the decode measurements (the headline is 2,048; the prefill figure stays at 2,048)")
    ap.add_argument("--long-contexts", type=lambda t: [int(x) for x in t.split(",") if x], default=[8192, 32768],
                    help="context lengths of the extra batch-8 decode points (comma separated; empty: none)")
    ap.add_argument("--with-secondary", action="store_true",
                    help="also run the two secondary serving workloads and put their figures under 'secondary'")
    ap.add_argument("--timeline", action="store_true",
                    help="also print, on standard error, start and end of every kernel of one decode step in place")
    ap.add_argument("--profile", action="store_true",
                    help="also print, on standard error, per-kernel times of one prefill and one decode step")
    args = ap.parse_args()
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload != "decode_8b":
        print(json.dumps(serving_workload(args, load_peaks())))
        return 0
    args.warmup = max(args.warmup, 3)

    import torch
    from torchllms_b200.models.llama_config import LlamaConfig, RopeScaling
    from torchllms_b200.engine.step import StepEntry
    from torchllms_b200.inference import LLM

    peaks = load_peaks()
    shape = dict(SHAPE_8B, n_layers=args.layers)
    ctx_len = args.context_len
    max_len = max(CONTEXT, -(-(ctx_len + args.warmup + args.steps + 64) // 16) * 16)
    cfg = LlamaConfig(architecture="LlamaForCausalLM", rope_scaling=RopeScaling(**ROPE_8B), max_seq_len=max_len, **shape)
    max_b = 64 if not args.skip_points else args.batch
    llm = LLM(config=cfg, random_seed=0, precision="bfloat16", max_len=max_len, max_bsz=max(max_b, args.batch),
              max_num_batched_tokens=args.batch * ctx_len, page_size=16)   # the e2e batch's prompts go in one step
    engine, ops = llm.engine, llm.model.ops
    gen = torch.Generator().manual_seed(1234)

    def prompts(n, length=PROMPT_LEN):
        return torch.randint(0, cfg.vocab_size, (n, length), generator=gen).tolist()

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ------------------------------------------------------------------ prefill, 2,048 tokens
    def prefill_once():
        h = engine.claim()
        toks = prompts(1)[0]
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        engine.step([StepEntry(h, toks, [PROMPT_LEN - 1])])
        b.record()
        torch.cuda.synchronize()
        engine.release(h)
        return a.elapsed_time(b)

    for _ in range(3):
        prefill_once()
    pre_ms = sorted(prefill_once() for _ in range(5))[2]
    ops.check_status()
    # 2 flops per weight per token; q, k, v, o projections: dim * hd * (2 H + 2 KV) weights; gate, up, down:
    # 3 * dim * hidden; the head runs on one row; causal attention: QK^T and PV, each 2 * H * hd * T^2 / 2
    lin = PROMPT_LEN * (args.layers * (2 * cfg.dim * cfg.head_dim * (2 * cfg.n_heads + 2 * cfg.n_kv_heads)
                                        + 6 * cfg.dim * cfg.ffn_hidden)) + 2 * cfg.dim * cfg.vocab_size
    attn = args.layers * 2 * cfg.n_heads * cfg.head_dim * PROMPT_LEN * PROMPT_LEN
    pre_flops = lin + attn
    prefill = {"value": round(PROMPT_LEN / (pre_ms / 1e3), 1), "tokens": PROMPT_LEN, "ms": round(pre_ms, 3),
               "frac": round(pre_flops / (pre_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}

    # ------------------------------------------------------------------ decode at a batch size
    kv_bytes_per_token = args.layers * 2 * cfg.n_kv_heads * cfg.head_dim * 2

    def decode_run(batch, steps, warmup, with_clocks=False, llm=llm, ctx_len=ctx_len):
        engine = llm.engine
        clocks = ClockSampler() if with_clocks else None
        if clocks:
            clocks.__enter__()
        handles = [engine.claim() for _ in range(batch)]
        ps = prompts(batch, ctx_len)
        chunk = min(engine.max_step_tokens, 8192)
        for h, p in zip(handles, ps):                       # prefill, one prompt after the other, in portions
            for i in range(0, len(p), chunk):
                engine.step([StepEntry(h, p[i:i + chunk], [])])
        feed = torch.randint(0, cfg.vocab_size, (warmup + steps, batch), generator=gen).tolist()
        for i in range(warmup):
            logits = engine.step([StepEntry(h, [t]) for h, t in zip(handles, feed[i])])
            ops.sample(logits)
        torch.cuda.synchronize()
        launches0 = ops.launches
        a, b = ev(), ev()
        t_start = time.time()
        a.record()
        for i in range(warmup, warmup + steps):
            logits = engine.step([StepEntry(h, [t]) for h, t in zip(handles, feed[i])])
            ops.sample(logits)
        b.record()
        torch.cuda.synchronize()
        if clocks:
            clocks.mark(t_start, time.time())
            time.sleep(0.15)
            clocks.__exit__()
        ops.check_status()                                  # a kernel that gave up a wait has said so by now
        if not bool(torch.isfinite(logits).all()):
            raise RuntimeError(f"decode at batch {batch}: the last step's logits are not finite")
        ms = a.elapsed_time(b) / steps
        for h in handles:
            engine.release(h)
        mean_ctx = ctx_len + warmup + steps / 2
        step_bytes = llm.model.weight_bytes() + batch * mean_ctx * kv_bytes_per_token
        return {"ms": ms, "tok_s": batch / (ms / 1e3), "bytes": step_bytes, "launches": ops.launches - launches0,
                "clocks": clocks.summary() if clocks else None}

    head = decode_run(args.batch, args.steps, args.warmup, with_clocks=True)
    points, point_fracs = {}, {}
    if not args.skip_points:
        for b in (1, 64):
            run = decode_run(b, max(args.steps // 2, 8), 3)
            points[f"decode_b{b}"] = round(run["tok_s"], 1)
            point_fracs[f"decode_b{b}"] = round(run["bytes"] / (run["ms"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
    achieved = head["bytes"] / (head["ms"] / 1e3) / 1e9

    if args.profile:
        def table(title, prof):
            total = sum(ms for _n, ms in prof.values())
            print(f"-- {title}: {total:.3f} ms in kernels", file=sys.stderr)
            for name, (calls, ms) in sorted(prof.items(), key=lambda kv: -kv[1][1]):
                print(f"   {name:16s} {calls:5d} calls {ms:9.3f} ms {100 * ms / total:5.1f} %", file=sys.stderr)
        engine.use_graphs = False                      # per-kernel times need eager launches
        h = engine.claim()
        with ops.profile() as prof:
            engine.step([StepEntry(h, prompts(1)[0], [PROMPT_LEN - 1])])
        table("prefill of 2,048 tokens", prof)
        hs = [engine.claim() for _ in range(args.batch - 1)]
        for x in hs:
            engine.step([StepEntry(x, prompts(1)[0], [])])
        with ops.profile() as prof:
            logits = engine.step([StepEntry(x, [1]) for x in [h] + hs])
            ops.sample(logits)
        table(f"decode step, batch {args.batch}, context 2,048", prof)
        for x in [h] + hs:
            engine.release(x)
        engine.use_graphs = True

    if args.timeline:
        # Start and end of every kernel of one recorded decode step as the device ran it, kernels
        # overlapping where programmatic dependent launch lets them (CUPTI through torch.profiler; the
        # tracing stretches the step by a few per cent).  "+x" is the time from the end of the kernel
        # before it to its own end: what the kernel added to the step.
        from torch.profiler import ProfilerActivity, profile
        hs = [engine.claim() for _ in range(args.batch)]
        for x in hs:
            engine.step([StepEntry(x, prompts(1)[0], [])])

        def one():
            ops.sample(engine.step([StepEntry(x, [1]) for x in hs]))
        for _ in range(6):
            one()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                one()
            torch.cuda.synchronize()
        evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda e: e.time_range.start)
        last = evs[-(len(evs) // 3):]
        t0, prev = last[0].time_range.start, 0.0
        print(f"-- one decode step, batch {args.batch}, context 2,048, {args.layers} layers: kernels in place (us)", file=sys.stderr)
        for e in last:
            a, b = e.time_range.start - t0, e.time_range.end - t0
            name = e.name.replace("void ", "").replace("(anonymous namespace)::", "")
            print(f"   {name[:44]:44s} start {a:8.1f}  end {b:8.1f}  {b - prev:+7.1f}", file=sys.stderr)
            prev = b
        for x in hs:
            engine.release(x)

    # ------------------------------------------------------------------ end to end through LLM.generate
    n_new = args.warmup + args.steps
    llm.warmup(range(1, args.batch + 1))                                            # decode graphs, as at server start
    llm.generate(prompt_token_ids=prompts(args.batch, 64), max_new_tokens=4, disable_tqdm=True)        # warm the path
    e2e_prompts = prompts(args.batch, ctx_len)
    e2e_out = llm.generate(prompt_token_ids=e2e_prompts, max_new_tokens=n_new, disable_tqdm=True)
    st = llm.last_stats
    ops.check_status()
    # the timed run launches each decode step before it has read the tokens of the step before: the
    # step-by-step way must give the same greedy tokens
    llm.look_ahead = False
    n_check = min(8, n_new)
    check = llm.generate(prompt_token_ids=e2e_prompts, max_new_tokens=n_check, disable_tqdm=True)
    llm.look_ahead = True
    if [r.token_ids[:n_check] for r in e2e_out] != [r.token_ids for r in check] or any(r.error for r in e2e_out):
        raise RuntimeError(f"end to end: launching ahead and the step-by-step way disagree on the first {n_check} greedy tokens")
    e2e_tok_s = st.decode_step_tokens / st.decode_seconds if st.decode_seconds > 0 else None
    h2d = engine._buf.uploaded_bytes                 # the last decode step's one upload (positions, slots, block tables)
    e2e = {"value": round(e2e_tok_s, 1) if e2e_tok_s else None, "unit": "tokens/s",
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch}

    # ------------------------------------------------------------------ longer contexts, batch 8 (an engine of their own)
    if not args.skip_points and args.long_contexts:
        weight_bytes = llm.model.weight_bytes()
        del llm, engine
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        longest = max(args.long_contexts)
        long_len = -(-(longest + 3 + 64 + 64) // 16) * 16
        cfg_long = LlamaConfig(architecture="LlamaForCausalLM", rope_scaling=RopeScaling(**ROPE_8B), max_seq_len=long_len, **shape)
        llm_long = LLM(config=cfg_long, random_seed=0, precision="bfloat16", max_len=long_len, max_bsz=8,
                       max_num_batched_tokens=8192, page_size=16)
        for n_ctx in args.long_contexts:
            run = decode_run(8, 64, 3, llm=llm_long, ctx_len=n_ctx)
            points[f"decode_b8_ctx{n_ctx}"] = round(run["tok_s"], 1)
            point_fracs[f"decode_b8_ctx{n_ctx}"] = round(run["bytes"] / (run["ms"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        ops.check_status()
        del llm_long
        gc.collect()
        torch.cuda.empty_cache()

    secondary = None
    if args.with_secondary:
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        secondary = {}
        for name in sorted(SERVE):
            args.workload = name
            line = serving_workload(args, peaks)
            secondary[name] = {k: line[k] for k in ("value", "generated_tokens_per_s", "seconds", "roofline_frac", "flop_seconds", "byte_seconds")}
            gc.collect()
            torch.cuda.empty_cache()

    out = {
        "metric": f"decode tok/s at batch {args.batch} (Llama-3.1-8B shape, {ctx_len:,}-token prompts)",
        "value": round(head["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(head["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights N(0, 0.02))",
        "config": {"model": "llama-3.1-8b-shape", "n_layers": args.layers, "n_layers_full": SHAPE_8B["n_layers"],
                   "dim": cfg.dim, "n_heads": cfg.n_heads, "n_kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
                   "ffn_hidden": cfg.ffn_hidden, "vocab_size": cfg.vocab_size, "global_batch": args.batch,
                   "seq_len": ctx_len, "context": max_len, "page_size": 16, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (16 GB of weights per step)"},
        "e2e": e2e, "gpu_launches": head["launches"], "clocks": head["clocks"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
        "points": points, "point_roofline_fracs": point_fracs,
    }
    if secondary is not None:
        out["secondary"] = secondary
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
