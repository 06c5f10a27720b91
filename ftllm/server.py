"""`python -m ftllm.server ...` of the reference: forwards to the `server` sub-command."""
import sys

from fastllm_b200.cli import main

if __name__ == "__main__":
    sys.exit(main(["server", *sys.argv[1:]]))
