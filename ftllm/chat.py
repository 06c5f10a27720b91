"""`python -m ftllm.chat ...` of the reference: forwards to the `chat` sub-command."""
import sys

from fastllm_b200.cli import main

if __name__ == "__main__":
    sys.exit(main(["chat", *sys.argv[1:]]))
