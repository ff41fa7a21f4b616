"""Another architecture from outside the package: its own configuration class and ``config.json``
keys, a block kind with four norms, a layer without a feed-forward, one registry entry
(``tests/toy_arch.py``).  Everything of the framework is used as it is: the random-weights
folder writer, the loader's strict check, ``LLM(folder)``, the scheduler, the replay program and
its ``bin/trace_run`` (which learns of the module through ``TORCHLLMS_B200_PLUGINS``).  The
reference would need another boolean flag in ``ModelParams`` and another branch in
``Transformer.from_params`` (torchllms/models/networks.py:779-788) for each such variant."""

import os
import random
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

import toy_arch
import traces
from helpers import ROOT, run_trace
from plain_llama import to_bfloat16_and_back
from torch_ops import TorchOps
from torchllms_b200.config import ConfigError, get_architecture, load_config
from torchllms_b200.engine.replay import Replayer
from torchllms_b200.inference import LLM
from torchllms_b200.weights.loader import WeightError
from torchllms_b200.weights.random_init import write_random_model

CONFIG = toy_arch.ToyConfig(architecture=toy_arch.NAME, depth=3, width=80, heads=5, kv_heads=1, head_width=16, inner=112,
                            vocab=301, eps=1e-4, theta=5000.0, bare_layers=(1,), max_seq_len=192)
# heads of 64 and a feed-forward width the gated product takes: the tensor-core kernels' sizes
CONFIG_WIDE_HEADS = toy_arch.ToyConfig(architecture=toy_arch.NAME, depth=2, width=128, heads=2, kv_heads=2, head_width=64,
                                       inner=192, vocab=409, eps=1e-5, theta=10000.0, bare_layers=(0,), max_seq_len=512)


def requests_for(cfg, lengths, seed=1):
    rng = random.Random(seed)
    return {f"t{i}": [rng.randrange(cfg.vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def test_the_package_does_not_know_the_toy():
    out = subprocess.run(["grep", "-rIl", "-i", "toy", str(ROOT / "torchllms_b200"), "--include=*.py", "--include=*.cu",
                          "--include=*.cuh", "--include=*.h"], capture_output=True, text=True)
    assert out.stdout.strip() == ""


def test_registered_parsed_and_written_like_any_architecture(tmp_path):
    assert get_architecture(toy_arch.NAME) is toy_arch.TOY
    folder = write_random_model(tmp_path / "toy", CONFIG, seed=4)
    arch, cfg = load_config(folder)
    assert arch is toy_arch.TOY and cfg == CONFIG
    assert load_config(folder, {"max_seq_len": 64})[1].max_seq_len == 64
    with pytest.raises(ConfigError, match="toy_depth"):
        toy_arch.ToyConfig.parse({"architectures": [toy_arch.NAME]}, "somewhere")
    spec = arch.build_spec(cfg)
    assert [l.block.kind for l in spec.layers] == ["toy_four_norm", "toy_bare", "toy_four_norm"]
    assert "feed_forward" not in spec.layers[1].block.params and len([k for k in spec.layers[0].block.params if "p" in k[:2]]) == 4
    # the strict loader speaks of this architecture's tensors
    from safetensors.torch import load_file, save_file
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["stack.1.pre.weight"]
    tensors["stack.1.ff.w1.weight"] = torch.zeros(2, 2)
    broken = tmp_path / "broken"
    broken.mkdir()
    (broken / "config.json").write_text((folder / "config.json").read_text())
    save_file(tensors, str(broken / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        LLM(broken, device="cpu", precision="float32", ops=TorchOps())
    assert e.value.missing == ["stack.1.pre.weight"] and e.value.unexpected == ["stack.1.ff.w1.weight"]


def test_generates_and_replays_on_the_kernel_twins(tmp_path):
    folder = write_random_model(tmp_path / "toy", CONFIG, seed=4)
    llm = LLM(folder, device="cpu", precision="float32", ops=TorchOps(), max_len=192, max_bsz=3, page_size=8,
              max_num_batched_tokens=40, prefill_chunk=16)
    prompts = list(requests_for(CONFIG, (3, 50, 21, 1)).values())
    got = llm.generate(prompt_token_ids=prompts, max_new_tokens=5, disable_tqdm=True)
    for p, r in zip(prompts, got):
        seq = list(p)
        for tok in r.token_ids:
            assert tok == int(torch.argmax(toy_arch.plain_logits(folder, seq)[-1]))
            seq.append(tok)
    reqs = requests_for(CONFIG, (60, 9, 131, 33, 70), seed=2)
    ref = {rid: toy_arch.plain_logits(folder, t).numpy() for rid, t in reqs.items()}
    steps, places, peak = traces.mixed(reqs)
    rp = Replayer(folder, "float32", peak, page_size=8, device="cpu", ops=TorchOps())
    for s in steps:
        out = rp.run_step(s)
        rp.engine.cache.check_invariants()
        if s["step"] in places:
            want = np.stack([ref[rid][pos] for rid, pos in places[s["step"]]])
            assert np.abs(out - want).max() < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["odd", "wide_heads"])
def test_replays_through_trace_run_on_the_gpu(tmp_path, dtype, which):
    cfg = CONFIG if which == "odd" else CONFIG_WIDE_HEADS
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_random_model(tmp_path / "toy", cfg, seed=6, dtype=store)
    reqs = requests_for(cfg, (60, 9, 131, 33, 170) if which == "odd" else (300, 40, 131, 97, 210), seed=3)
    if dtype == "float32":
        ref, tol = {rid: toy_arch.plain_logits(folder, t).numpy() for rid, t in reqs.items()}, 1e-4
    else:
        ref = {rid: toy_arch.plain_logits(folder, t, stored=to_bfloat16_and_back).numpy() for rid, t in reqs.items()}
        tol = 0.5 * max(float(np.abs(ref[rid] - toy_arch.plain_logits(folder, t).numpy()).max()) for rid, t in reqs.items())
    env_before = dict(os.environ)
    os.environ["TORCHLLMS_B200_PLUGINS"] = "toy_arch"
    os.environ["PYTHONPATH"] = str(Path(__file__).resolve().parent) + os.pathsep + os.environ.get("PYTHONPATH", "")
    try:
        for mode, kw in (("whole", {}), ("portions", {}), ("mixed", dict(chunks=(2, 5, 24, 96, 150, 40)))):
            steps, places, peak = getattr(traces, mode)(reqs, **kw)
            got = run_trace(folder, dtype, steps, tmp_path / mode, max_tokens=peak, vocab=cfg.vocab)
            for step, rows in places.items():
                want = np.stack([ref[rid][pos] for rid, pos in rows])
                err = np.abs(got[step] - want).max(axis=1)
                assert (err <= tol).all(), (mode, step, rows[int(np.argmax(err))], float(err.max()), tol)
    finally:
        os.environ.clear()
        os.environ.update(env_before)


@pytest.mark.gpu
def test_generates_through_the_entry_point_on_the_gpu(tmp_path):
    folder = write_random_model(tmp_path / "toy", CONFIG, seed=4)
    llm = LLM(folder, precision="float32", max_len=192, max_bsz=3, page_size=8, max_num_batched_tokens=40, prefill_chunk=16)
    prompts = list(requests_for(CONFIG, (3, 50, 21, 1)).values())
    got = llm.generate(prompt_token_ids=prompts, max_new_tokens=8, disable_tqdm=True)
    for p, r in zip(prompts, got):
        seq = list(p)
        for tok in r.token_ids:
            assert tok == int(torch.argmax(toy_arch.plain_logits(folder, seq)[-1]))
            seq.append(tok)
    assert llm.engine.use_graphs is False or llm.engine.model.graph_safe
