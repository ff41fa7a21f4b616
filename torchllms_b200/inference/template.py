"""Chat templates: turning a conversation into the token ids a chat model expects.

Reference: ``TemplateConfig`` and ``tokenize_conversation``
(torchllms/messages/tokenization.py:103-130, :284) with the Llama-3 values of
torchllms/messages/configs/llama3_instruct.yaml:9-32: a begin-of-text token, each message
wrapped in ``<|start_header_id|>role<|end_header_id|>\\n\\n ... <|eot_id|>``, the assistant
header as generation prompt, content stripped of surrounding whitespace, and stop id 128009.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple


@dataclass(frozen=True)
class ChatTemplate:
    name: str
    bos: str
    envelopes: Dict[str, Tuple[str, str]]       # role -> (text before, text after the content)
    generation_prompt: str
    stop_token_ids: Tuple[int, ...]
    strip_whitespace: bool = True

    def render(self, conversation: Sequence[Dict[str, str]], add_generation_prompt: bool = True) -> str:
        parts: List[str] = [self.bos]
        for message in conversation:
            role, content = message["role"], message["content"]
            if role not in self.envelopes:
                raise ValueError(f"template {self.name!r} has no role {role!r}; roles: {sorted(self.envelopes)}")
            before, after = self.envelopes[role]
            parts += [before, content.strip() if self.strip_whitespace else content, after]
        if add_generation_prompt:
            parts.append(self.generation_prompt)
        return "".join(parts)


def _header(role: str) -> str:
    return f"<|start_header_id|>{role}<|end_header_id|>\n\n"


LLAMA3_INSTRUCT = ChatTemplate(
    name="llama3_instruct",
    bos="<|begin_of_text|>",
    envelopes={
        "system": (_header("system"), "<|eot_id|>"),
        "user": (_header("user"), "<|eot_id|>"),
        "assistant": (_header("assistant"), "<|eot_id|>"),
        "tool": (_header("ipython"), "<|eot_id|>"),
    },
    generation_prompt=_header("assistant"),
    stop_token_ids=(128009,),
)

TEMPLATES = {LLAMA3_INSTRUCT.name: LLAMA3_INSTRUCT}


def get_template(name: str) -> ChatTemplate:
    key = name[:-5] if name.endswith(".yaml") else name
    try:
        return TEMPLATES[key]
    except KeyError:
        raise ValueError(f"unknown template {name!r}; known: {sorted(TEMPLATES)}") from None
