import sys

from fastllm_b200.cli import main

sys.exit(main())
