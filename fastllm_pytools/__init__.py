"""The reference's second package name (`from fastllm_pytools import llm`, tools/fastllm_pytools): forwards to fastllm_b200."""
from fastllm_b200 import llm, util  # noqa: F401
from fastllm_b200.cli import main  # noqa: F401

from . import hf_model, torch2flm  # noqa: F401
