"""Models that live outside the local file system (``file://``, ``s3://``, ``gs://`` ... URIs).

The weights of such a model are streamed from the source by the loader; the small files next to them
(configuration, tokenizer, generation defaults, custom code) must be on local disk of EVERY host, because
every rank re-reads them while it builds the model.  ``ensure_local_aux_files`` gives each host its own copy:

* the local directory is named by a hash of the URI, so all ranks of all hosts agree on it;
* ranks that share a host serialise on a file lock: one pulls, the others wait and then find the copy;
* completion is recorded by a sentinel written after the last file (the first file to arrive is usually
  ``config.json``, so its presence proves nothing), and a pull that died half-way leaves a "pulling" mark
  without the sentinel, which the next caller treats as "start over".

Fetchers are registered per scheme.  ``file://`` is built in; object stores need a fetcher that lists and
downloads (a deployment registers one around its own client; nothing here talks to a network).
(reference: src/vllm_torchtpu/worker/runai_repull.py:1-162 — the same repair for worker ranks of remote hosts)"""
from __future__ import annotations

import fcntl
import fnmatch
import hashlib
import os
import shutil
from typing import Callable, Optional
from urllib.parse import urlparse

from ..logger import init_logger

logger = init_logger(__name__)

AUX_PATTERNS = ("*.json", "*.txt", "*.model", "*.py", "*.jinja", "*.tiktoken", "tokenizer*", "*.md")
WEIGHT_PATTERNS = ("*.safetensors", "*.bin", "*.pt", "*.pth", "*.gguf")
_PULLING, _COMPLETE = ".b200_pulling", ".b200_aux_complete"

# scheme -> (list_files(uri) -> [relative names], fetch(uri, relative name, destination path))
_FETCHERS: dict = {}


def register_fetcher(scheme: str, list_files: Callable, fetch: Callable) -> None:
    _FETCHERS[scheme] = (list_files, fetch)


def _file_list(uri: str) -> list:
    root = urlparse(uri).path
    return sorted(f for f in os.listdir(root) if os.path.isfile(os.path.join(root, f)))


def _file_fetch(uri: str, name: str, dst: str) -> None:
    shutil.copyfile(os.path.join(urlparse(uri).path, name), dst)


register_fetcher("file", _file_list, _file_fetch)


def is_remote_uri(model: str) -> bool:
    return isinstance(model, str) and "://" in model


def is_aux_file(name: str) -> bool:
    if any(fnmatch.fnmatch(name, p) for p in WEIGHT_PATTERNS):
        return False
    return any(fnmatch.fnmatch(name, p) for p in AUX_PATTERNS)


def local_dir_for(uri: str, cache_root: Optional[str] = None) -> str:
    root = cache_root or os.path.join(os.path.expanduser("~"), ".cache", "vllm_torchtpu_b200", "model_source")
    return os.path.join(root, hashlib.sha256(uri.rstrip("/").encode()).hexdigest()[:32])


def is_complete(local_dir: str) -> bool:
    return os.path.exists(os.path.join(local_dir, _COMPLETE))


def ensure_local_aux_files(uri: str, cache_root: Optional[str] = None) -> str:
    """Local directory holding the non-weight files of ``uri``; pulled on this host if it is not there yet."""
    scheme = urlparse(uri).scheme
    if scheme not in _FETCHERS:
        raise ValueError(f"no fetcher is registered for {scheme}:// models (known: {sorted(_FETCHERS)})")
    list_files, fetch = _FETCHERS[scheme]
    local = local_dir_for(uri, cache_root)
    if is_complete(local):
        return local
    os.makedirs(os.path.dirname(local), exist_ok=True)
    with open(local + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)           # ranks of one host: one pulls, the others wait here
        try:
            if is_complete(local):
                return local
            if os.path.exists(os.path.join(local, _PULLING)):
                logger.warning("[aux-pull] %s holds a pull that did not finish: starting over", local)
                shutil.rmtree(local)
            os.makedirs(local, exist_ok=True)
            with open(os.path.join(local, _PULLING), "w") as f:
                f.write(uri)
            names = [n for n in list_files(uri) if is_aux_file(n)]
            if "config.json" not in names:
                raise FileNotFoundError(f"{uri} has no config.json")
            logger.info("[aux-pull] pulling %d aux files for %s on this host", len(names), uri)
            for n in names:
                fetch(uri, n, os.path.join(local, n))
            with open(os.path.join(local, _COMPLETE), "w") as f:
                f.write(uri)
            os.remove(os.path.join(local, _PULLING))
            return local
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def resolve_model(model: str, cache_root: Optional[str] = None) -> tuple:
    """(directory with configuration and tokenizer, place the weights are read from).  For a ``file://`` model
    the weights are read in place; for other schemes the weight source stays the URI and the loader needs a
    streaming reader for it."""
    if not is_remote_uri(model):
        return model, model
    local = ensure_local_aux_files(model, cache_root)
    if urlparse(model).scheme == "file":
        return local, urlparse(model).path
    return local, model
