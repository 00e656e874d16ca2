"""Model hub without a network: registry search, a download through an injected opener (with a dropped connection
that resumes), checksum verification and the LRU cache."""
import _path  # noqa: F401
import hashlib
import io
import os
import tempfile

from rustorch_b200 import model_hub as H

root = tempfile.mkdtemp()
blob = os.urandom(20000)
attempts = {"n": 0}


def opener(url, offset):
    attempts["n"] += 1
    data = blob[offset:]
    return io.BytesIO(data[:8000] if attempts["n"] == 1 else data), len(blob)      # first connection drops after 8000 bytes


hub = H.ModelHub(os.path.join(root, "hub"), H.ModelDownloader(max_retries=3, opener=opener))
print("registry:", len(hub.list_models()), "models;", "search 'bert' ->", [m.name for m in hub.registry.search("bert")][:3])
hub.registry.register_model(H.ModelInfo("toy-mlp", "http://example.invalid/toy.bin", "mlp", sha256=hashlib.sha256(blob).hexdigest(), file_format="bin"))
path = hub.download_model("toy-mlp")
print("downloaded", os.path.getsize(path), "bytes in", attempts["n"], "connections; verified:", H.ModelVerifier.verify(path, hashlib.sha256(blob).hexdigest()))
print("second request served from the cache:", hub.download_model("toy-mlp") == path and attempts["n"] == 2)
cache = H.ModelCache(os.path.join(root, "cache"), H.CacheConfig(max_size_bytes=50000, max_entries=10))
for i, name in enumerate(("a", "b", "c")):
    cache.cache_model(name, path, now=float(i))
print("cache of 50 kB after three 20 kB models keeps", cache.list_cached_models(), "->", cache.stats())
print("crc32 / md5:", H.ModelVerifier.checksum(path, "crc32"), H.ModelVerifier.checksum(path, "md5")[:8] + "...")
