"""``python -m ftllm.cli`` / the ``ftllm`` console entry of the reference."""
import sys

from fastllm_b200.cli import main  # noqa: F401

if __name__ == "__main__":
    sys.exit(main())
