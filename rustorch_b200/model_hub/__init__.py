"""Model hub: registry of known models, verified downloads with retries and progress, an LRU disk cache with a
size cap, checksum / format verification (src/model_hub/mod.rs:20-160, registry.rs, downloader.rs:12-330,
cache.rs:12-260, verification.rs).  Network access fails with a clear error where there is none; registry, cache
and verification are offline logic.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import time
import zlib
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Tuple


@dataclass
class ModelInfo:
    name: str
    url: str
    architecture: str
    parameters: int = 0
    file_format: str = "safetensors"
    sha256: Optional[str] = None
    size_bytes: Optional[int] = None
    description: str = ""
    tags: List[str] = field(default_factory=list)


class ModelRegistry:
    def __init__(self):
        self.models: Dict[str, ModelInfo] = {}
        for m in (
            ModelInfo("resnet18", "https://download.pytorch.org/models/resnet18-f37072fd.pth", "resnet", 11_689_512, "pytorch",
                      description="ResNet-18 ImageNet classifier", tags=["vision", "classification"]),
            ModelInfo("resnet50", "https://download.pytorch.org/models/resnet50-0676ba61.pth", "resnet", 25_557_032, "pytorch",
                      description="ResNet-50 ImageNet classifier", tags=["vision", "classification"]),
            ModelInfo("gpt2", "https://huggingface.co/gpt2/resolve/main/model.safetensors", "gpt2", 124_439_808, "safetensors",
                      description="GPT-2 small language model", tags=["nlp", "generation"]),
            ModelInfo("bert-base-uncased", "https://huggingface.co/bert-base-uncased/resolve/main/model.safetensors", "bert", 109_482_240,
                      "safetensors", description="BERT base (uncased)", tags=["nlp", "encoder"]),
        ):
            self.models[m.name] = m

    def register_model(self, info: ModelInfo) -> None:
        self.models[info.name] = info

    def get_model_info(self, name: str) -> ModelInfo:
        if name not in self.models:
            raise KeyError(f"model '{name}' is not in the registry")
        return self.models[name]

    def list_models(self) -> List[str]:
        return sorted(self.models)

    def search(self, query: str = "", tag: Optional[str] = None, architecture: Optional[str] = None) -> List[ModelInfo]:
        q = query.lower()
        return [m for m in self.models.values() if (q in m.name.lower() or q in m.description.lower())
                and (tag is None or tag in m.tags) and (architecture is None or m.architecture == architecture)]

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({k: asdict(v) for k, v in self.models.items()}, f, indent=2)

    def load(self, path: str) -> None:
        with open(path) as f:
            for k, v in json.load(f).items():
                self.models[k] = ModelInfo(**v)


@dataclass
class DownloadProgress:
    downloaded: int
    total: Optional[int]
    elapsed_s: float

    def percentage(self) -> float:
        return 100.0 * self.downloaded / self.total if self.total else 0.0

    def format_speed(self) -> str:
        bps = self.downloaded / self.elapsed_s if self.elapsed_s > 0 else 0.0
        return f"{bps / 1e6:.1f} MB/s" if bps >= 1e6 else f"{bps / 1e3:.1f} KB/s"

    def format_size(self) -> str:
        return f"{self.downloaded / 1e6:.1f} MB" + (f" / {self.total / 1e6:.1f} MB" if self.total else "")


class DownloadError(RuntimeError):
    """A download failed after all retries, or its checksum did not match (src/model_hub/downloader.rs)."""


class ModelDownloader:
    def __init__(self, max_retries: int = 3, timeout_seconds: int = 30, opener: Optional[Callable] = None):
        self.max_retries, self.timeout = max_retries, timeout_seconds
        self._open = opener                            # injectable for tests: opener(url, offset) -> (file-like, total)

    def _default_open(self, url: str, offset: int):
        import urllib.request
        req = urllib.request.Request(url, headers={"Range": f"bytes={offset}-"} if offset else {})
        r = urllib.request.urlopen(req, timeout=self.timeout)
        n = r.headers.get("Content-Length")
        return r, (int(n) + offset if n else None)

    def download(self, url: str, dest: str, progress: Optional[Callable[[DownloadProgress], None]] = None) -> str:
        os.makedirs(os.path.dirname(os.path.abspath(dest)), exist_ok=True)
        part, last = dest + ".part", None
        t0 = time.time()
        for attempt in range(self.max_retries):
            offset = os.path.getsize(part) if os.path.exists(part) else 0
            try:
                src, total = (self._open or self._default_open)(url, offset)
                with open(part, "ab") as f:
                    done = offset
                    while True:
                        chunk = src.read(1 << 20)
                        if not chunk:
                            break
                        f.write(chunk)
                        done += len(chunk)
                        if progress:
                            progress(DownloadProgress(done, total, time.time() - t0))
                if total is not None and done < total:
                    raise IOError(f"connection closed after {done} of {total} bytes")
                os.replace(part, dest)
                return dest
            except Exception as e:  # noqa: BLE001  (retry on any transport error, resume from the partial file)
                last = e
                time.sleep(min(0.05 * 2 ** attempt, 2.0))
        raise DownloadError(f"download of {url} failed after {self.max_retries} attempts: {last}")


class ModelVerifier:
    @staticmethod
    def checksum(path: str, algo: str = "sha256") -> str:
        if algo == "crc32":
            c = 0
            with open(path, "rb") as f:
                for chunk in iter(lambda: f.read(1 << 20), b""):
                    c = zlib.crc32(chunk, c)
            return f"{c & 0xFFFFFFFF:08x}"
        h = hashlib.new(algo)
        with open(path, "rb") as f:
            for chunk in iter(lambda: f.read(1 << 20), b""):
                h.update(chunk)
        return h.hexdigest()

    @staticmethod
    def verify(path: str, expected: str, algo: str = "sha256") -> bool:
        return ModelVerifier.checksum(path, algo).lower() == expected.lower()

    @staticmethod
    def verify_format(path: str, expected_format: str) -> bool:
        from ..formats.safetensors import detect_format
        got = detect_format(path)
        return got == expected_format or (expected_format == "pytorch" and got in ("torch", "pth"))


@dataclass
class CacheConfig:
    max_size_bytes: int = 10 << 30
    max_entries: int = 100


@dataclass
class CacheEntry:
    name: str
    path: str
    size: int
    last_access: float


class ModelCache:
    """Files under ``cache_dir`` tracked in ``index.json``; least recently used entries are evicted to respect the
    size and entry caps."""

    def __init__(self, cache_dir: str, config: Optional[CacheConfig] = None):
        self.dir, self.config = cache_dir, config or CacheConfig()
        os.makedirs(cache_dir, exist_ok=True)
        self.entries: Dict[str, CacheEntry] = {}
        idx = os.path.join(cache_dir, "index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                for k, v in json.load(f).items():
                    if os.path.exists(v["path"]):
                        self.entries[k] = CacheEntry(**v)

    def _save(self) -> None:
        with open(os.path.join(self.dir, "index.json"), "w") as f:
            json.dump({k: asdict(v) for k, v in self.entries.items()}, f)

    def get_model_path(self, name: str) -> Optional[str]:
        e = self.entries.get(name)
        if e is None or not os.path.exists(e.path):
            self.entries.pop(name, None)
            return None
        e.last_access = time.time()
        self._save()
        return e.path

    def get_download_path(self, name: str, ext: str = "bin") -> str:
        return os.path.join(self.dir, f"{name.replace('/', '--')}.{ext}")

    def cache_model(self, name: str, src_path: str, now: Optional[float] = None) -> str:
        dest = self.get_download_path(name, os.path.splitext(src_path)[1].lstrip(".") or "bin")
        if os.path.abspath(src_path) != os.path.abspath(dest):
            shutil.copyfile(src_path, dest)
        self.entries[name] = CacheEntry(name, dest, os.path.getsize(dest), now if now is not None else time.time())
        self._evict(keep=name)
        self._save()
        return dest

    def _evict(self, keep: str) -> None:
        def over():
            return sum(e.size for e in self.entries.values()) > self.config.max_size_bytes or len(self.entries) > self.config.max_entries
        while over():
            victims = sorted((e for e in self.entries.values() if e.name != keep), key=lambda e: e.last_access)
            if not victims:
                break
            self.remove_model(victims[0].name)

    def remove_model(self, name: str) -> bool:
        e = self.entries.pop(name, None)
        if e is None:
            return False
        if os.path.exists(e.path):
            os.remove(e.path)
        self._save()
        return True

    def clear(self) -> None:
        for n in list(self.entries):
            self.remove_model(n)

    def stats(self) -> Tuple[int, int]:
        return len(self.entries), sum(e.size for e in self.entries.values())

    def list_cached_models(self) -> List[str]:
        return sorted(self.entries)


class ModelHub:
    def __init__(self, cache_dir: Optional[str] = None, downloader: Optional[ModelDownloader] = None):
        self.registry = ModelRegistry()
        self.cache = ModelCache(cache_dir or os.path.join(os.path.expanduser("~"), ".rustorch", "hub"))
        self.downloader = downloader or ModelDownloader()

    @classmethod
    def with_cache_dir(cls, d: str) -> "ModelHub":
        return cls(d)

    def list_models(self) -> List[str]:
        return self.registry.list_models()

    def get_model_info(self, name: str) -> ModelInfo:
        return self.registry.get_model_info(name)

    def download_model(self, name: str, progress=None, force: bool = False) -> str:
        info = self.registry.get_model_info(name)
        if not force:
            p = self.cache.get_model_path(name)
            if p:
                return p
        ext = {"pytorch": "pth", "safetensors": "safetensors", "gguf": "gguf", "onnx": "onnx"}.get(info.file_format, "bin")
        tmp = self.cache.get_download_path(name, ext)
        self.downloader.download(info.url, tmp, progress)
        if info.sha256 and not ModelVerifier.verify(tmp, info.sha256):
            os.remove(tmp)
            raise DownloadError(f"checksum mismatch for '{name}'")
        return self.cache.cache_model(name, tmp)

    def load_model(self, name: str, progress=None):
        """Download (or take from the cache) and import: returns an ``ImportedModel``."""
        from ..model_import import ModelImporter
        return ModelImporter().import_from_file(self.download_model(name, progress))
