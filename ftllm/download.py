"""`python -m ftllm.download ...` of the reference: forwards to the `download` sub-command."""
import sys

from fastllm_b200.cli import main

if __name__ == "__main__":
    sys.exit(main(["download", *sys.argv[1:]]))
