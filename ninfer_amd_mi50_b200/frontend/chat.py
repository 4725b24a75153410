"""The ChatML prompt the reference's CLI builds (src/frontend/chat.cpp:5-22), without the
Qwen3 thinking marker (another architecture's)."""

from __future__ import annotations

from typing import List, Sequence, Tuple


def render_chatml_messages(messages: Sequence[Tuple[str, str]], add_generation_prompt: bool = True) -> str:
    out = ""
    for role, content in messages:
        out += f"<|im_start|>{role}\n{content}<|im_end|>\n"
    if add_generation_prompt:
        out += "<|im_start|>assistant\n"
    return out


def render_chatml(system: str, user: str) -> str:
    messages: List[Tuple[str, str]] = []
    if system:
        messages.append(("system", system))
    messages.append(("user", user))
    return render_chatml_messages(messages)
