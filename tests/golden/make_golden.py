"""Compare the plain implementation once with the reference's own model code, on the CPU.

    python tests/golden/make_golden.py --reference /path/to/torchllms-checkout

Builds the two tiny configurations as the reference's ``Transformer``
(torchllms/models/networks.py:778, eager attention, float32), loads the very tensors the tests
use (``helpers.make_tensors``, torchllms names, so no renaming is involved), runs whole prompts
without a cache, and writes ``tests/golden/tiny_<name>.json``: for every prompt position the
argmax and a few logits, plus the largest difference to ``plain_llama`` seen in this run.  The
test ``test_plain.py`` then holds the plain implementation to these numbers without needing the
reference.

A second run per configuration anchors the row order of Hugging Face checkpoints: the same random
tensors are given Hugging Face names *as they are* (their q and k rows then mean "first halves,
second halves" of each head), converted by the reference's own ``_from_hf``
(torchllms/models/checkpoint_converter.py:81-192, whose ``permute`` :96-108 interleaves the rows),
loaded into the reference's model and run on the same prompts: the ``"hf"`` entry of the record.
The plain implementation and the engine each read the Hugging Face names with a permutation of
their own; the tests hold both to this entry.
"""

import argparse
import json
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

KEEP = 24            # logits kept per position
PROMPT_SEED = 11
LENGTHS = {"A": [1, 19, 70], "B": [3, 33, 130]}


def prompts_for(name, vocab):
    import random
    rng = random.Random(PROMPT_SEED + ord(name))
    return [[rng.randrange(vocab) for _ in range(n)] for n in LENGTHS[name]]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    os.environ["HF_HUB_OFFLINE"] = "1"
    os.environ["TRANSFORMERS_OFFLINE"] = "1"
    sys.path.insert(0, args.reference)
    import tempfile

    import torch
    from torchllms.models.networks import AttentionImpl, ModelParams, Transformer

    from helpers import TINY, make_tensors, write_model_folder
    from plain_llama import PlainModel

    from torchllms.models.checkpoint_converter import _from_hf

    from helpers import hugging_face_names

    for name, (cfg, seed, _page) in TINY.items():
        if name not in LENGTHS:              # only the configurations whose records are committed
            continue
        hidden = cfg["intermediate_size"]
        params = ModelParams(
            dim=cfg["hidden_size"], head_dim=cfg["head_dim"], n_layers=cfg["num_hidden_layers"],
            n_heads=cfg["num_attention_heads"], n_kv_heads=cfg["num_key_value_heads"], vocab_size=cfg["vocab_size"],
            multiple_of=hidden, ffn_dim_multiplier=hidden / cfg["hidden_size"] - 1e-9,
            norm_eps=cfg["rms_norm_eps"], max_seq_len=cfg["max_position_embeddings"], rope_theta=cfg["rope_theta"],
            rope_scaling=cfg["rope_scaling"] or {}, tie_word_embeddings=cfg["tie_word_embeddings"],
            attention_impl=AttentionImpl.EAGER)
        tensors = make_tensors(cfg, seed, std=0.05, qk_std=0.25)

        def run(state, folder_tensors, tmp):
            model = Transformer.from_params(params).float().eval()
            assert model.layers[0].feed_forward.w1.weight.shape[0] == hidden
            missing, unexpected = model.load_state_dict(state, strict=False)
            assert not unexpected and all("rope" in m for m in missing), (missing, unexpected)
            plain = PlainModel(write_model_folder(tmp, cfg, folder_tensors))
            rec = {"prompts": [], "max_diff_to_plain": 0.0}
            for toks in prompts_for(name, cfg["vocab_size"]):
                with torch.no_grad():
                    ref, _ = model(torch.tensor([toks]))
                ref = ref[0].float()
                mine = plain.logits(toks)
                rec["max_diff_to_plain"] = max(rec["max_diff_to_plain"], float((ref - mine).abs().max()))
                rec["prompts"].append({
                    "tokens": toks,
                    "argmax": ref.argmax(-1).tolist(),
                    "logits_head": [[round(float(x), 7) for x in row[:KEEP]] for row in ref[[0, len(toks) // 2, -1]]],
                    "logit_sum": [float(x) for x in ref.double().sum(-1)],
                })
            return rec

        with tempfile.TemporaryDirectory() as tmp:
            record = {"config": cfg, "seed": seed, "std": 0.05, "qk_std": 0.25}
            record.update(run(tensors, tensors, Path(tmp) / "native"))
            hf = hugging_face_names(tensors)
            converted = _from_hf(dict(hf), cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["hidden_size"],
                                 "float32", head_dim=cfg["head_dim"])
            record["hf"] = run(converted, hf, Path(tmp) / "hf")
            assert record["hf"]["prompts"][-1]["argmax"] != record["prompts"][-1]["argmax"]   # the row order matters
        out = HERE / f"tiny_{name}.json"
        out.write_text(json.dumps(record))
        print(f"{out.name}: largest difference between the reference and plain_llama {record['max_diff_to_plain']:.3g}; "
              f"from Hugging Face names through the reference's converter {record['hf']['max_diff_to_plain']:.3g}")


if __name__ == "__main__":
    main()
