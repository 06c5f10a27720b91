"""`python -m ftllm.benchmark ...` of the reference: forwards to the `bench` sub-command."""
import sys

from fastllm_b200.cli import main

if __name__ == "__main__":
    sys.exit(main(["bench", *sys.argv[1:]]))
