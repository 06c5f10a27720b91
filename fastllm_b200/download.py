"""Model download with resume (reference: tools/fastllm_pytools/download.py; HF / ModelScope snapshot into a cache dir).
There is no network on air-gapped hosts: the function then reports that clearly instead of hanging."""
from __future__ import annotations

import os


def download(repo: str, cache_dir: str | None = None) -> str:
    if not repo:
        raise SystemExit("download: give a repository id, e.g. Qwen/Qwen3-0.6B")
    if os.path.isdir(repo):
        return repo
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:
        raise SystemExit(f"download needs the huggingface_hub package: {e}")
    try:
        return snapshot_download(repo, cache_dir=cache_dir, resume_download=True,
                                 allow_patterns=["*.json", "*.safetensors", "*.txt", "*.model", "*.jinja", "*.tiktoken"])
    except Exception as e:
        raise SystemExit(f"download of '{repo}' failed (offline host?): {e}")
