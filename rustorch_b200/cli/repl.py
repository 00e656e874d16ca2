"""The interactive loop (example-cli/src/cli/repl.rs:12-457) and the program entry point (main.rs:9-184)."""
from __future__ import annotations

import os
import sys
from typing import Callable, List, Optional

from .args import Backend, CliArgs, parse_args
from .commands import HELP_TEXT, Command, CommandKind
from .config import Config
from .download import DownloadOptions, ModelDownloadManager, ModelIdentifier, ModelSource
from .engine import InferenceEngine, ModelLoader
from .session import TURN_END_TOKENS, GenerationConfig, SessionManager


class Repl:
    def __init__(self, session: SessionManager, engine: InferenceEngine, config: Optional[Config] = None,
                 out: Callable[[str], None] = None, stream: bool = True, show_metrics: bool = False):
        self.session, self.engine, self.config = session, engine, config or Config()
        self.out = out or (lambda s: (sys.stdout.write(s), sys.stdout.flush()))
        self.stream, self.show_metrics = stream, show_metrics
        self.running = True
        self.errors = 0                              # generations that failed in this session
        self.tokenizer_path: Optional[str] = None
        self.template_choice = "auto"                # "auto": follow what each loaded model's tokenizer points to
        self.detected_template = "plain"             # what the loaded model's tokenizer points to

    def apply_chat_template(self, detected: Optional[str] = None) -> None:
        if detected is not None:
            self.detected_template = detected
        name = self.detected_template if self.template_choice in (None, "auto") else self.template_choice
        self.session.set_chat_template(name)
        self.engine.set_stop_tokens(TURN_END_TOKENS[name])

    # -- one line of input -> True while the loop should go on
    def handle_line(self, line: str) -> bool:
        line = line.strip()
        if not line:
            return True
        if Command.is_command(line):
            try:
                self.handle_command(Command.parse(line))
            except (ValueError, OSError) as e:
                self.out(f"error: {e}\n")
            return self.running
        self.session.add_user_message(line)
        self.out("Assistant: ")
        try:
            reply = self.engine.generate(self.session.build_prompt(), on_token=self.out if self.stream else None)
        except KeyboardInterrupt:
            raise
        except Exception as e:  # noqa: BLE001  (a failed generation must not end the session; the turn is dropped)
            self.session.drop_last_message()
            self.errors += 1
            self.out(f"\nerror: {type(e).__name__}: {e}\n")
            return True
        if not self.stream:
            self.out(reply)
        self.out("\n")
        self.session.add_assistant_message(reply.strip())
        self.session.tokens_generated += self.engine.last_token_count
        if self.show_metrics:
            s = self.engine.stats()
            self.out(f"[{s['tokens']} tokens, TTFT {s['ttft_ms']:.0f} ms, {s['tokens_per_s']:.1f} tok/s]\n")
        return True

    def handle_command(self, cmd: Command) -> None:
        k = cmd.kind
        if k is CommandKind.EXIT:
            self.running = False
            self.session.auto_save()
            self.out("Goodbye!\n")
        elif k is CommandKind.HELP:
            self.out(HELP_TEXT + "\n")
        elif k is CommandKind.CLEAR:
            self.session.clear_history()
            self.out("Conversation cleared.\n")
        elif k is CommandKind.SAVE:
            path = cmd.arg or os.path.expanduser(self.config.session.history_file + ".json")
            self.session.save_history(path)
            self.out(f"Saved {self.session.message_count()} messages to {path}\n")
        elif k is CommandKind.LOAD:
            self.session.load_history(cmd.arg)
            self.out(f"Loaded {self.session.message_count()} messages from {cmd.arg}\n")
        elif k is CommandKind.MODEL:
            rt, tok, meta = ModelLoader.from_file(cmd.arg, self.engine.device, self.tokenizer_path)
            self.engine.runtime, self.engine.tokenizer = rt, tok
            self.session.set_model_name(meta.name)
            self.apply_chat_template(meta.chat_template)
            self.out(f"Loaded {meta.name} ({meta.format}, {meta.num_layers} layers, vocab {meta.vocab_size}, chat template {self.session.chat_template})\n")
        elif k is CommandKind.BACKEND:
            b = Backend(cmd.arg.lower())
            if not b.available():
                raise ValueError(f"backend '{b.value}' is not available here")
            self.session.set_backend_name(b.value)
            self.engine.device = b.device()
            self.out(f"Backend set to {b.value}; reload the model with /model to move it\n")
        elif k is CommandKind.STATS:
            s = self.engine.stats()
            self.out(f"messages: {self.session.message_count()}\nwords in history: {self.session.total_tokens()}\n"
                     f"tokens generated: {self.session.tokens_generated}\nlast reply: {s['tokens']} tokens, "
                     f"TTFT {s['ttft_ms']:.0f} ms, {s['tokens_per_s']:.1f} tok/s\n")
        elif k is CommandKind.SYSTEM:
            self.session.set_system_prompt(cmd.arg)
            self.out("System prompt set.\n")
        elif k is CommandKind.CONFIG:
            self.out(self.session.describe_config() + "\n")
        elif k is CommandKind.TEMPLATE:
            if cmd.arg:
                choice = cmd.arg.lower()
                if choice != "auto":
                    self.session.set_chat_template(choice)          # refuses unknown names before anything changes
                self.template_choice = choice
                self.apply_chat_template()
            self.out(f"chat template: {self.session.chat_template}" + (" (auto)" if self.template_choice in (None, "auto") else "") + "\n")
        else:
            self.out(f"Unknown command '/{cmd.arg}'. Type /help.\n")

    def run(self, read: Callable[[str], str] = input) -> None:
        self.out("RusTorch CLI - type /help for commands, /exit to quit\n")
        while self.running:
            try:
                line = read("You: ")
            except (EOFError, KeyboardInterrupt):
                self.handle_command(Command(CommandKind.EXIT))
                break
            self.handle_line(line)


def _run_download(a: CliArgs, out) -> int:
    mgr = ModelDownloadManager(a.output_dir)
    if a.command == "list":
        src = None if a.target in (None, "all") else ModelSource.from_prefix(a.target)
        models = mgr.list_models(src)
        out("\n".join(models) + "\n" if models else "no models downloaded\n")
        return 0
    try:
        ident = ModelIdentifier.parse(a.target)
    except ValueError as e:
        out(f"error: {e}\n")
        return 2
    if a.revision:
        ident.with_revision(a.revision)
    try:
        path = mgr.download(ident, DownloadOptions(a.output_dir, a.force, a.token),
                            None if a.no_progress else (lambda d, t: out(f"\r{d / 1e6:.1f} MB" + (f" / {t / 1e6:.1f} MB" if t else ""))))
    except (ConnectionError, FileNotFoundError, ValueError) as e:
        out(f"error: {e}\n")
        return 1
    out(f"\nsaved to {path}\n")
    return 0


def main(argv: Optional[List[str]] = None, read: Callable[[str], str] = input, out: Callable[[str], None] = None) -> int:
    out = out or (lambda s: (sys.stdout.write(s), sys.stdout.flush()))
    try:
        pre = parse_args(argv, Config())              # find --config first
        config = Config.load(pre.config) if pre.config else Config.load_or_default()
        a = parse_args(argv, config)
    except (ValueError, OSError) as e:
        out(f"error: {e}\n")
        return 2
    if a.command in ("download", "list"):
        return _run_download(a, out)
    device = a.backend.device()
    gen = GenerationConfig(a.max_tokens, a.temperature, a.top_p, a.top_k)
    runtime = tokenizer = None
    model_name, detected = "dummy", "plain"
    if a.model:
        try:
            runtime, tokenizer, meta = ModelLoader.from_file(a.model, device, a.tokenizer)
            model_name, detected = meta.name, meta.chat_template
        except (OSError, ValueError, KeyError) as e:
            out(f"error: cannot load model: {e}\n")
            return 1
    session = SessionManager(gen, a.backend.value, model_name, config.session.max_history)
    if config.session.auto_save and a.save_history:
        session.with_auto_save(a.save_history)
    if a.system_prompt:
        session.set_system_prompt(a.system_prompt)
    if a.load_history:
        session.load_history(a.load_history)
    engine = InferenceEngine(runtime, tokenizer, gen, device)
    repl = Repl(session, engine, config, out, config.ui.stream, config.ui.show_metrics)
    repl.tokenizer_path = a.tokenizer
    repl.template_choice = a.chat_template or "auto"
    repl.apply_chat_template(detected)
    if a.prompt is not None:
        repl.handle_line(a.prompt)
        if a.save_history:
            session.save_history(a.save_history)
        return 1 if repl.errors else 0
    repl.run(read)
    if a.save_history:
        session.save_history(a.save_history)
    return 0
