"""``rustorch-cli``: local LLM chat REPL (example-cli/src/main.rs:9-184, cli/args.rs:12-320, cli/repl.rs:12-457,
cli/commands.rs:5-92, model/inference.rs:58-331, model/loader.rs:6-156, session/*, utils/config.rs:11-261,
tokenizer/wrapper.rs:8-96, download/*).

``python -m rustorch_b200.cli --model x.gguf`` starts the REPL; ``download`` / ``list`` are the subcommands.
Unlike the reference (whose GGUF loader returns a dummy model and whose generation loop re-runs the whole
sequence per token), a GGUF file is really loaded into the quantised Llama runtime and decoded with a KV cache.
"""
from .args import Backend, CliArgs, build_parser, parse_args
from .commands import Command, CommandKind
from .config import BackendConfig, Config, GenerationSection, ModelConfig, SessionConfig, UiConfig
from .download import DownloadOptions, HuggingFaceClient, ModelDownloadManager, ModelIdentifier, ModelSource, OllamaClient
from .engine import InferenceEngine, ModelLoader, ModelMetadata
from .repl import Repl, main
from .session import GenerationConfig, Message, SessionHistory, SessionManager
from .tokenizer import ByteTokenizer, GGUFTokenizer, Tokenizer, load_tokenizer

__all__ = [n for n in dir() if not n.startswith("_")]
