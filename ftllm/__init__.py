"""Drop-in package name of the reference (`from ftllm import llm`): forwards to fastllm_b200."""
from fastllm_b200 import llm, util  # noqa: F401
from fastllm_b200.cli import main  # noqa: F401
