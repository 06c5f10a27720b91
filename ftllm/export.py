"""`python -m ftllm.export ...` of the reference: forwards to the `export` sub-command."""
import sys

from fastllm_b200.cli import main

if __name__ == "__main__":
    sys.exit(main(["export", *sys.argv[1:]]))
