"""Interactive chat: ``python -m torchllms_b200.inference.chat --ckpt_paths DIR ...``.

Reference: torchllms/inference/chat.py:11-86: the same options (``--ckpt_paths``,
``--template_config``, ``--max_new_tokens``, ``--temperature``, ``--device``, ``--precision``,
``--model_kwargs``), an optional system line, then user lines; ``!!reset`` starts over.  A folder
without a tokenizer (random weights) chats in token ids: type integers separated by spaces.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

from . import LLM


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Interactive chat with a torchllms_b200 model.")
    p.add_argument("--ckpt_paths", nargs="+", type=Path, required=True,
                   help="Model folder(s) or weight files, loaded in order; the configuration is read beside the first.")
    p.add_argument("--template_config", type=str, default=None, help="Chat template name, e.g. llama3_instruct.")
    p.add_argument("--max_new_tokens", type=int, default=200, help="Maximum number of new tokens.")
    p.add_argument("--temperature", type=float, default=0.0, help="Temperature for sampling; 0 is greedy.")
    p.add_argument("--device", type=str, default="cuda", help="Device to use.")
    p.add_argument("--precision", type=str, default=None, help="bfloat16 (default) or float32.")
    p.add_argument("--model_kwargs", type=json.loads, default={}, help="JSON object of configuration overrides.")
    p.add_argument("--max_len", type=int, default=4096, help="Longest sequence (prompt and answer).")
    p.add_argument("--top_k", type=int, default=None, help="Sample among the k most likely tokens only.")
    p.add_argument("--seed", type=int, default=0, help="Seed of the sampling noise.")
    return p.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    print("Loading model and tokenizer...")
    llm = LLM(ckpt_paths=args.ckpt_paths, template_config=args.template_config, device=args.device,
              precision=args.precision, model_kwargs=args.model_kwargs, max_len=args.max_len, max_bsz=1)
    text_mode = llm._load_tokenizer(required=False) is not None and llm.template is not None
    kw = dict(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k, seed=args.seed)

    def read_system():
        if not text_mode:
            return []
        line = input("[system]: ").strip()
        return [{"role": "system", "content": line}] if line else []

    conversation = read_system()
    history = []
    while True:
        try:
            content = input("[user]: ").strip()
        except EOFError:
            print()
            return
        if content == "!!reset":
            conversation, history = read_system(), []
            continue
        if text_mode:
            conversation.append({"role": "user", "content": content})
            result = llm.generate(conversations=[conversation], **kw)[0]
            conversation.append({"role": "assistant", "content": result.text})
            print("[assistant]: " + result.text)
        else:
            try:
                history += [int(t) for t in content.split()]
            except ValueError:
                print("(no tokenizer in this folder: enter token ids separated by spaces)")
                continue
            result = llm.generate(prompt_token_ids=[history], **kw)[0]
            history += result.token_ids
            print("[assistant]: " + " ".join(map(str, result.token_ids)))


if __name__ == "__main__":
    main()
