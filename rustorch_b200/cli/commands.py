"""Slash commands of the REPL (example-cli/src/cli/commands.rs:5-92)."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Optional


class CommandKind(Enum):
    """The REPL's slash commands (example-cli/src/cli/commands.rs)."""

    EXIT = "exit"
    HELP = "help"
    CLEAR = "clear"
    SAVE = "save"
    LOAD = "load"
    MODEL = "model"
    BACKEND = "backend"
    STATS = "stats"
    SYSTEM = "system"
    CONFIG = "config"
    TEMPLATE = "template"                # an addition: the reference has one prompt layout
    UNKNOWN = "unknown"


_ALIASES = {"exit": CommandKind.EXIT, "quit": CommandKind.EXIT, "q": CommandKind.EXIT, "help": CommandKind.HELP, "h": CommandKind.HELP,
            "?": CommandKind.HELP, "clear": CommandKind.CLEAR, "cls": CommandKind.CLEAR, "save": CommandKind.SAVE, "load": CommandKind.LOAD,
            "model": CommandKind.MODEL, "backend": CommandKind.BACKEND, "stats": CommandKind.STATS, "system": CommandKind.SYSTEM,
            "config": CommandKind.CONFIG, "template": CommandKind.TEMPLATE}
_NEEDS_ARG = {CommandKind.LOAD: "/load <path>", CommandKind.MODEL: "/model <path>", CommandKind.BACKEND: "/backend <name>",
              CommandKind.SYSTEM: "/system <prompt>"}

HELP_TEXT = """Commands:
  /help, /h, /?        show this help
  /exit, /quit, /q     leave
  /clear, /cls         clear the conversation
  /save [path]         save the conversation as JSON
  /load <path>         load a conversation
  /model <path>        load another model
  /backend <name>      switch backend (cpu, cuda)
  /stats               session and performance statistics
  /system <prompt>     set the system prompt
  /config              show the current configuration
  /template [name]     show or set the chat layout (auto, plain, llama3, chatml, llama2)"""


@dataclass
class Command:
    kind: CommandKind
    arg: Optional[str] = None

    @staticmethod
    def is_command(line: str) -> bool:
        return line.strip().startswith("/")

    @staticmethod
    def parse(line: str) -> "Command":
        body = line.strip()
        if not body.startswith("/"):
            raise ValueError("not a command")
        name, _, rest = body[1:].partition(" ")
        rest = rest.strip() or None
        kind = _ALIASES.get(name.lower())
        if kind is None:
            return Command(CommandKind.UNKNOWN, name)
        if kind in _NEEDS_ARG and rest is None:
            raise ValueError(f"usage: {_NEEDS_ARG[kind]}")
        return Command(kind, rest)
