"""`python -m ftllm.webui ...` of the reference: forwards to the `webui` sub-command."""
import sys

from fastllm_b200.cli import main

if __name__ == "__main__":
    sys.exit(main(["webui", *sys.argv[1:]]))
