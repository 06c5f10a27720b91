"""Model download with resume (reference: tools/fastllm_pytools/download.py; HF / ModelScope snapshot into a cache dir).
There is no network on air-gapped hosts: the function then reports that clearly instead of hanging."""
from __future__ import annotations

import os


def download(repo: str, cache_dir: str | None = None, local_dir: str | None = None, revision: str | None = None,
             include: list | None = None, exclude: list | None = None, token: str | None = None, workers: int = 8,
             dataset: bool = False) -> str:
    """Snapshot a model repository (resumable).  ``include`` / ``exclude`` are glob patterns as in the reference's
    ``ftllm download --include ... --exclude ...``."""
    if not repo:
        raise SystemExit("download: give a repository id, e.g. Qwen/Qwen3-0.6B")
    if os.path.isdir(repo):
        return repo
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:
        raise SystemExit(f"download needs the huggingface_hub package: {e}")
    try:
        if dataset:
            return snapshot_download(repo, repo_type="dataset", cache_dir=cache_dir, local_dir=local_dir, revision=revision, token=token,
                                     max_workers=workers, allow_patterns=include or None, ignore_patterns=exclude or None)
        return snapshot_download(repo, cache_dir=cache_dir, local_dir=local_dir, revision=revision, token=token, max_workers=workers,
                                 allow_patterns=include or ["*.json", "*.safetensors", "*.txt", "*.model", "*.jinja", "*.tiktoken"],
                                 ignore_patterns=exclude or None)
    except Exception as e:
        raise SystemExit(f"download of '{repo}' failed (offline host?): {e}")
