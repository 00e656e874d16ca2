"""Conversation state (example-cli/src/session/mod.rs:11-145, history.rs:4-95, config.rs:4-60)."""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import List, Optional


@dataclass
class GenerationConfig:
    max_tokens: int = 512
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 40
    repetition_penalty: float = 1.0

    def validate(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be positive")
        if not 0.0 <= self.temperature <= 2.0:
            raise ValueError("temperature must be in [0, 2]")
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError("top_p must be in [0, 1]")
        if self.top_k < 1:
            raise ValueError("top_k must be positive")


@dataclass
class Message:
    role: str
    content: str
    timestamp: float = field(default_factory=time.time)

    @classmethod
    def new_user(cls, c: str) -> "Message":
        return cls("user", c)

    @classmethod
    def new_assistant(cls, c: str) -> "Message":
        return cls("assistant", c)

    @classmethod
    def new_system(cls, c: str) -> "Message":
        return cls("system", c)

    def is_user(self) -> bool:
        return self.role == "user"

    def is_assistant(self) -> bool:
        return self.role == "assistant"

    def is_system(self) -> bool:
        return self.role == "system"


class SessionHistory:
    def __init__(self, max_history: int = 1000):
        self._messages: List[Message] = []
        self.max_history = max_history

    def _add(self, m: Message) -> None:
        self._messages.append(m)
        if len(self._messages) > self.max_history:
            del self._messages[: len(self._messages) - self.max_history]

    def add_user_message(self, c: str) -> None:
        self._add(Message.new_user(c))

    def add_assistant_message(self, c: str) -> None:
        self._add(Message.new_assistant(c))

    def add_system_message(self, c: str) -> None:
        self._add(Message.new_system(c))

    def pop_last(self) -> None:
        if self._messages:
            self._messages.pop()

    def clear(self) -> None:
        self._messages.clear()

    def message_count(self) -> int:
        return len(self._messages)

    def messages(self) -> List[Message]:
        return list(self._messages)

    def last_message(self) -> Optional[Message]:
        return self._messages[-1] if self._messages else None

    def user_messages(self):
        return (m for m in self._messages if m.is_user())

    def assistant_messages(self):
        return (m for m in self._messages if m.is_assistant())


CHAT_TEMPLATES = ("plain", "llama3", "chatml", "llama2")
# tokens that end an assistant turn in the template's family (looked up in the tokenizer's added tokens)
TURN_END_TOKENS = {"plain": (), "llama3": ("<|eot_id|>", "<|end_of_text|>"), "chatml": ("<|im_end|>", "<|endoftext|>"), "llama2": ("</s>",)}


def detect_chat_template(tokenizer=None, metadata: Optional[dict] = None) -> str:
    """Names the chat layout a model was tuned on from what it carries: the ``tokenizer.chat_template`` text of a GGUF
    file or the marker tokens in the tokenizer's vocabulary.  ``plain`` (``User:`` / ``Assistant:`` lines, the reference's
    only layout) when nothing tells."""
    text = str((metadata or {}).get("tokenizer.chat_template", ""))
    known = set(getattr(tokenizer, "added", None) or ())
    if "<|start_header_id|>" in text or "<|start_header_id|>" in known:
        return "llama3"
    if "<|im_start|>" in text or "<|im_start|>" in known:
        return "chatml"
    if "[INST]" in text:
        return "llama2"
    return "plain"


class SessionManager:
    def __init__(self, generation_config: Optional[GenerationConfig] = None, backend_name: str = "cpu", model_name: str = "none",
                 max_history: int = 1000):
        self.history = SessionHistory(max_history)
        self._gen = generation_config or GenerationConfig()
        self._gen.validate()
        self._backend, self._model = backend_name, model_name
        self._system: Optional[str] = None
        self._auto_save: Optional[str] = None
        self.tokens_generated = 0
        self.chat_template = "plain"

    def set_chat_template(self, name: str) -> None:
        if name not in CHAT_TEMPLATES:
            raise ValueError(f"chat template '{name}' is not one of {CHAT_TEMPLATES}")
        self.chat_template = name

    def with_auto_save(self, path: str) -> "SessionManager":
        self._auto_save = path
        return self

    def add_user_message(self, c: str) -> None:
        self.history.add_user_message(c)

    def add_assistant_message(self, c: str) -> None:
        self.history.add_assistant_message(c)

    def drop_last_message(self) -> None:
        """Forget the newest message (a user turn whose reply could not be generated)."""
        self.history.pop_last()

    def clear_history(self) -> None:
        self.history.clear()

    def save_history(self, path: str) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        doc = {"model": self._model, "backend": self._backend, "system_prompt": self._system, "generation": asdict(self._gen),
               "messages": [asdict(m) for m in self.history.messages()]}
        with open(path, "w") as f:
            json.dump(doc, f, indent=2)

    def load_history(self, path: str) -> None:
        with open(path) as f:
            doc = json.load(f)
        self.history.clear()
        for m in doc.get("messages", []):
            self.history._add(Message(m["role"], m["content"], m.get("timestamp", 0.0)))
        if doc.get("system_prompt"):
            self._system = doc["system_prompt"]

    def auto_save(self) -> None:
        if self._auto_save:
            self.save_history(self._auto_save)

    def message_count(self) -> int:
        return self.history.message_count()

    def total_tokens(self) -> int:
        """Rough size of the conversation (whitespace-separated words), as the reference reports it."""
        return sum(len(m.content.split()) for m in self.history.messages())

    def backend_name(self) -> str:
        return self._backend

    def model_name(self) -> str:
        return self._model

    def set_backend_name(self, b: str) -> None:
        self._backend = b

    def set_model_name(self, m: str) -> None:
        self._model = m

    def generation_config(self) -> GenerationConfig:
        return self._gen

    def set_system_prompt(self, p: str) -> None:
        self._system = p

    def system_prompt(self) -> Optional[str]:
        return self._system

    def get_messages(self) -> List[Message]:
        return self.history.messages()

    def describe_config(self) -> str:
        g = self._gen
        return (f"model: {self._model}\nbackend: {self._backend}\nmax_tokens: {g.max_tokens}\ntemperature: {g.temperature}\n"
                f"top_p: {g.top_p}\ntop_k: {g.top_k}\nchat template: {self.chat_template}\nsystem prompt: {self._system or '(none)'}")

    def _turns(self):
        """``(role, text)`` of the system prompt and the history, in order."""
        out = [("system", self._system)] if self._system else []
        for m in self.history.messages():
            out.append(("system" if m.is_system() else "user" if m.is_user() else "assistant", m.content))
        return out

    def build_prompt(self) -> str:
        """The conversation as one prompt that ends with an open assistant turn.  ``plain``: system prompt, then ``User:`` /
        ``Assistant:`` lines; ``llama3`` / ``chatml`` / ``llama2``: the marker layouts those model families were tuned on
        (the start-of-text marker is the tokenizer's business, not part of the text)."""
        if self.chat_template == "llama3":
            return "".join(f"<|start_header_id|>{r}<|end_header_id|>\n\n{t}<|eot_id|>" for r, t in self._turns()) + \
                "<|start_header_id|>assistant<|end_header_id|>\n\n"
        if self.chat_template == "chatml":
            return "".join(f"<|im_start|>{r}\n{t}<|im_end|>\n" for r, t in self._turns()) + "<|im_start|>assistant\n"
        if self.chat_template == "llama2":
            out, system = [], None
            for r, t in self._turns():
                if r == "system":
                    system = t if system is None else system + "\n" + t
                elif r == "user":
                    body = f"<<SYS>>\n{system}\n<</SYS>>\n\n{t}" if system is not None else t
                    system = None
                    out.append(f"[INST] {body} [/INST]")
                else:
                    out.append(f" {t} </s><s>")
            return "".join(out)
        parts = [self._system + "\n"] if self._system else []
        for m in self.history.messages():
            if m.is_system():
                parts.append(m.content + "\n")
            else:
                parts.append(("User: " if m.is_user() else "Assistant: ") + m.content + "\n")
        parts.append("Assistant:")
        return "".join(parts)
