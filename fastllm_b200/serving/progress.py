"""Start-up progress events: one JSON object per line on stderr, prefixed ``FTLLM_PROGRESS`` (reference:
tools/fastllm_pytools/startup_progress.py, enabled by the ``FTLLM_PROGRESS`` environment variable)."""
import json
import os
import sys
import time

_t0 = time.time()


def emit(stage: str, current: int, total: int, **extra) -> None:
    if os.environ.get("FTLLM_PROGRESS", "0") in ("0", "", "false"):
        return
    ev = {"stage": stage, "current": current, "total": total, "elapsed_s": round(time.time() - _t0, 3)}
    ev.update(extra)
    sys.stderr.write("FTLLM_PROGRESS " + json.dumps(ev) + "\n")
    sys.stderr.flush()
