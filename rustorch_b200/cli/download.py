"""Model sources and downloads (example-cli/src/download/mod.rs:9-130, huggingface.rs:11-200, ollama.rs, manager.rs:9-230).

``hf:<org>/<repo>[:<file>]`` and ``ollama:<name>[:<tag>]`` identifiers, cache directory layout, GGUF
recommendation by quantisation preference, resumable streaming download with a progress callback.  Network
access goes through ``urllib`` and fails with a clear error where there is none; everything else (parsing,
URL construction, cache listing, file choice) is offline logic.
"""
from __future__ import annotations

import json
import os
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, List, Optional


class ModelSource(Enum):
    HUGGINGFACE = "hf"
    OLLAMA = "ollama"

    @classmethod
    def from_prefix(cls, prefix: str) -> "ModelSource":
        p = prefix.lower()
        if p in ("hf", "huggingface"):
            return cls.HUGGINGFACE
        if p == "ollama":
            return cls.OLLAMA
        raise ValueError(f"unknown model source '{prefix}' (use hf: or ollama:)")


@dataclass
class ModelIdentifier:
    source: ModelSource
    repo_id: str
    filename: Optional[str] = None
    revision: Optional[str] = None

    @classmethod
    def parse(cls, text: str) -> "ModelIdentifier":
        if ":" not in text:
            raise ValueError("expected <source>:<model>, e.g. hf:TheBloke/Llama-2-7B-GGUF or ollama:llama2:7b")
        prefix, rest = text.split(":", 1)
        src = ModelSource.from_prefix(prefix)
        if not rest:
            raise ValueError("empty model name")
        if src is ModelSource.HUGGINGFACE:
            repo, _, fname = rest.partition(":")
            if repo.count("/") != 1:
                raise ValueError("HuggingFace models are <org>/<repo>")
            return cls(src, repo, fname or None)
        name, _, tag = rest.partition(":")
        return cls(src, name, None, tag or "latest")

    def with_filename(self, f: str) -> "ModelIdentifier":
        self.filename = f
        return self

    def with_revision(self, r: str) -> "ModelIdentifier":
        self.revision = r
        return self


@dataclass
class DownloadOptions:
    output_dir: Optional[str] = None
    force: bool = False
    token: Optional[str] = None
    quant_preference: List[str] = field(default_factory=lambda: ["Q4_0", "Q4_K_M", "Q8_0", "Q5_K_M"])

    @staticmethod
    def default_model_dir() -> str:
        return os.path.join(os.path.expanduser("~"), ".rustorch", "models")

    @staticmethod
    def get_hf_token() -> Optional[str]:
        return os.environ.get("HF_TOKEN") or os.environ.get("HUGGING_FACE_HUB_TOKEN")


@dataclass
class ModelFile:
    filename: str
    size: Optional[int] = None


def _stream(url: str, dest: str, headers: dict, progress: Optional[Callable[[int, Optional[int]], None]], force: bool) -> str:
    os.makedirs(os.path.dirname(os.path.abspath(dest)), exist_ok=True)
    part = dest + ".part"
    have = os.path.getsize(part) if os.path.exists(part) and not force else 0
    if os.path.exists(dest) and not force:
        return dest
    if have:
        headers = {**headers, "Range": f"bytes={have}-"}
    req = urllib.request.Request(url, headers=headers)
    try:
        with urllib.request.urlopen(req, timeout=30) as r, open(part, "ab" if have else "wb") as f:
            total = r.headers.get("Content-Length")
            total = int(total) + have if total else None
            done = have
            while True:
                chunk = r.read(1 << 20)
                if not chunk:
                    break
                f.write(chunk)
                done += len(chunk)
                if progress:
                    progress(done, total)
    except (urllib.error.URLError, OSError) as e:
        raise ConnectionError(f"download of {url} failed: {e}") from e
    os.replace(part, dest)
    return dest


class HuggingFaceClient:
    BASE = "https://huggingface.co"

    def __init__(self, token: Optional[str] = None):
        self.token = token or DownloadOptions.get_hf_token()

    def _headers(self) -> dict:
        return {"Authorization": f"Bearer {self.token}"} if self.token else {}

    def file_url(self, repo_id: str, filename: str, revision: Optional[str] = None) -> str:
        return f"{self.BASE}/{repo_id}/resolve/{revision or 'main'}/{filename}"

    def api_url(self, repo_id: str, revision: Optional[str] = None) -> str:
        return f"{self.BASE}/api/models/{repo_id}" + (f"/revision/{revision}" if revision else "")

    def list_files(self, repo_id: str, revision: Optional[str] = None) -> List[ModelFile]:
        req = urllib.request.Request(self.api_url(repo_id, revision), headers=self._headers())
        try:
            with urllib.request.urlopen(req, timeout=30) as r:
                doc = json.load(r)
        except (urllib.error.URLError, OSError) as e:
            raise ConnectionError(f"cannot list {repo_id}: {e}") from e
        return [ModelFile(s["rfilename"], s.get("size")) for s in doc.get("siblings", [])]

    @staticmethod
    def find_gguf_files(files: List[ModelFile]) -> List[ModelFile]:
        return [f for f in files if f.filename.lower().endswith(".gguf")]

    @staticmethod
    def recommend_gguf(files: List[ModelFile], preference: List[str]) -> Optional[ModelFile]:
        ggufs = HuggingFaceClient.find_gguf_files(files)
        for q in preference:
            for f in ggufs:
                if q.lower() in f.filename.lower():
                    return f
        return ggufs[0] if ggufs else None

    def download_file(self, repo_id: str, filename: str, dest_dir: str, revision=None, progress=None, force=False) -> str:
        return _stream(self.file_url(repo_id, filename, revision), os.path.join(dest_dir, filename), self._headers(), progress, force)


class OllamaClient:
    REGISTRY = "https://registry.ollama.ai"

    def manifest_url(self, name: str, tag: str = "latest") -> str:
        ns = name if "/" in name else f"library/{name}"
        return f"{self.REGISTRY}/v2/{ns}/manifests/{tag}"

    def blob_url(self, name: str, digest: str) -> str:
        ns = name if "/" in name else f"library/{name}"
        return f"{self.REGISTRY}/v2/{ns}/blobs/{digest}"

    @staticmethod
    def model_layer(manifest: dict) -> Optional[dict]:
        for layer in manifest.get("layers", []):
            if layer.get("mediaType", "").endswith("image.model"):
                return layer
        return None

    def download(self, name: str, tag: str, dest_dir: str, progress=None, force=False) -> str:
        try:
            with urllib.request.urlopen(self.manifest_url(name, tag), timeout=30) as r:
                manifest = json.load(r)
        except (urllib.error.URLError, OSError) as e:
            raise ConnectionError(f"cannot fetch the manifest of {name}:{tag}: {e}") from e
        layer = self.model_layer(manifest)
        if layer is None:
            raise ValueError("manifest has no model layer")
        return _stream(self.blob_url(name, layer["digest"]), os.path.join(dest_dir, f"{name.replace('/', '_')}-{tag}.gguf"), {}, progress, force)


class ModelDownloadManager:
    def __init__(self, model_dir: Optional[str] = None):
        self.model_dir = model_dir or DownloadOptions.default_model_dir()

    def target_dir(self, ident: ModelIdentifier, options: Optional[DownloadOptions] = None) -> str:
        base = (options.output_dir if options and options.output_dir else self.model_dir)
        return os.path.join(base, ident.source.value, ident.repo_id.replace("/", "--"))

    def download(self, ident: ModelIdentifier, options: Optional[DownloadOptions] = None, progress=None) -> str:
        options = options or DownloadOptions()
        dest = self.target_dir(ident, options)
        if ident.source is ModelSource.HUGGINGFACE:
            hf = HuggingFaceClient(options.token)
            fname = ident.filename
            if fname is None:
                pick = hf.recommend_gguf(hf.list_files(ident.repo_id, ident.revision), options.quant_preference)
                if pick is None:
                    raise FileNotFoundError(f"{ident.repo_id} has no GGUF file; name one with hf:{ident.repo_id}:<file>")
                fname = pick.filename
            return hf.download_file(ident.repo_id, fname, dest, ident.revision, progress, options.force)
        return OllamaClient().download(ident.repo_id, ident.revision or "latest", dest, progress, options.force)

    def list_models(self, source: Optional[ModelSource] = None) -> List[str]:
        out = []
        for src in ([source] if source else list(ModelSource)):
            root = os.path.join(self.model_dir, src.value)
            if not os.path.isdir(root):
                continue
            for repo in sorted(os.listdir(root)):
                for f in sorted(os.listdir(os.path.join(root, repo))):
                    if not f.endswith(".part"):
                        out.append(f"{src.value}:{repo.replace('--', '/')}:{f}")
        return out
