"""Chat data: roles, messages, conversations, and rendering to token ids with a role per token.

A ``Conversation`` is a list of ``Message(role, content)``.  ``render_conversation`` lays the messages out with a template
(by default the ChatML frame ``<|im_start|>role\\ncontent<|im_end|>\\n``; a Hugging Face tokenizer's own ``chat_template``
when it has one) and returns the ids together with ``roles [len(ids)]``: the role each token belongs to, so an objective
can score the assistant's tokens only (``LMObjective(loss_role=Role.ASSISTANT)`` reads the batch's ``"roles"``).
``render_prompt`` ends with the opening of an assistant turn, for generation.

Reference: src/dew/data/chat.py (``Role`` :61, ``Message`` :221, ``Conversation`` :298, ``render_prompt`` :505,
``render_conversation`` :517, ``RenderChat`` :611).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import IntEnum
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch


class Role(IntEnum):
    PAD = 0          # not part of any message (padding, frame tokens that belong to nobody)
    SYSTEM = 1
    USER = 2
    ASSISTANT = 3
    TOOL = 4

    @classmethod
    def of(cls, raw: Any) -> "Role":
        if isinstance(raw, Role):
            return raw
        if isinstance(raw, str) and raw.upper() in cls.__members__ and raw.upper() != "PAD":
            return cls[raw.upper()]
        raise ValueError(f"a message's role is one of system, user, assistant, tool, not {raw!r}")


@dataclass(frozen=True)
class Message:
    role: Role
    content: str

    @classmethod
    def of(cls, raw: Any) -> "Message":
        if isinstance(raw, Message):
            return raw
        if not isinstance(raw, Mapping) or "role" not in raw or "content" not in raw:
            raise ValueError(f"a message is a mapping with 'role' and 'content', got {raw!r}")
        if not isinstance(raw["content"], str):
            raise ValueError("this renderer takes text content only")
        return cls(Role.of(raw["role"]), raw["content"])


@dataclass(frozen=True)
class Conversation:
    messages: Tuple[Message, ...]

    @classmethod
    def of(cls, raw: Any) -> "Conversation":
        if isinstance(raw, Conversation):
            return raw
        if isinstance(raw, Mapping):
            raw = raw.get("messages", raw.get("conversation"))
        if not isinstance(raw, Sequence) or isinstance(raw, str) or not raw:
            raise ValueError("a conversation is a non-empty list of messages")
        msgs = tuple(Message.of(m) for m in raw)
        for i, m in enumerate(msgs):
            if m.role == Role.SYSTEM and i != 0:
                raise ValueError("a system message comes first")
        return cls(msgs)

    @property
    def prompt(self) -> "Conversation":
        """The conversation up to (not including) its last assistant message."""
        for i in range(len(self.messages) - 1, -1, -1):
            if self.messages[i].role == Role.ASSISTANT:
                return Conversation(self.messages[:i])
        return self


@dataclass(frozen=True)
class ChatTemplate:
    """``open + role name + sep + content + close`` per message; the ids of ``open``/``close`` frames take ``frame_role``."""
    open: str = "<|im_start|>"
    sep: str = "\n"
    close: str = "<|im_end|>\n"
    names: Mapping[Role, str] = field(default_factory=lambda: {Role.SYSTEM: "system", Role.USER: "user", Role.ASSISTANT: "assistant", Role.TOOL: "tool"})
    score_close: bool = True     # an assistant turn's closing frame is the assistant's (the model must learn to stop)


def _encode(tokenizer, text: str) -> List[int]:
    if hasattr(tokenizer, "encode"):
        try:
            return list(tokenizer.encode(text, add_special_tokens=False))
        except TypeError:
            return list(tokenizer.encode(text))
    return list(tokenizer(text))


def render_conversation(tokenizer, conversation: Any, template: Optional[ChatTemplate] = None, *, generation_prompt: bool = False,
                        max_len: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """``{"tokens": ids, "roles": role per token}``.  Each message's header (``open + name + sep``) is nobody's (PAD role), its
    content is the speaker's, and an assistant's closing frame is the assistant's when ``template.score_close``."""
    conv = Conversation.of(conversation)
    tpl = template or ChatTemplate()
    ids: List[int] = []
    roles: List[int] = []
    for m in conv.messages:
        head = _encode(tokenizer, tpl.open + tpl.names[m.role] + tpl.sep)
        body = _encode(tokenizer, m.content)
        tail = _encode(tokenizer, tpl.close)
        ids += head + body + tail
        tail_role = m.role if (m.role == Role.ASSISTANT and tpl.score_close) else Role.PAD
        roles += [Role.PAD] * len(head) + [m.role] * len(body) + [tail_role] * len(tail)
    if generation_prompt:
        head = _encode(tokenizer, tpl.open + tpl.names[Role.ASSISTANT] + tpl.sep)
        ids += head
        roles += [Role.PAD] * len(head)
    if max_len is not None:
        ids, roles = ids[:max_len], roles[:max_len]
    return {"tokens": torch.tensor(ids, dtype=torch.long), "roles": torch.tensor([int(r) for r in roles], dtype=torch.long)}


def render_prompt(tokenizer, conversation: Any, template: Optional[ChatTemplate] = None) -> torch.Tensor:
    """Ids of the conversation's prompt part followed by the opening of an assistant turn."""
    return render_conversation(tokenizer, Conversation.of(conversation).prompt, template, generation_prompt=True)["tokens"]


def chat_batch(tokenizer, conversations: Sequence[Any], seq_len: int, pad_id: int = 0, template: Optional[ChatTemplate] = None) -> Dict[str, torch.Tensor]:
    """Rows of ``seq_len + 1`` ids (inputs and shifted targets) with their roles, right-padded with ``pad_id`` / ``Role.PAD``."""
    tokens = torch.full((len(conversations), seq_len + 1), pad_id, dtype=torch.long)
    roles = torch.zeros((len(conversations), seq_len + 1), dtype=torch.long)
    for i, c in enumerate(conversations):
        r = render_conversation(tokenizer, c, template, max_len=seq_len + 1)
        n = r["tokens"].shape[0]
        tokens[i, :n], roles[i, :n] = r["tokens"], r["roles"]
    return {"tokens": tokens, "roles": roles}
