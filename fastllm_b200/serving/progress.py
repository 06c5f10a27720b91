"""Start-up progress events: one JSON object per line on stderr, prefixed ``FTLLM_PROGRESS`` (reference:
tools/fastllm_pytools/startup_progress.py, enabled by the ``FTLLM_PROGRESS`` environment variable)."""
import json
import os
import sys
import time

_t0 = time.time()


_callback = None


def set_callback(fn) -> None:
    """``fn(stage, current, total, completed_bytes, total_bytes)`` is called for every progress event (None: remove)."""
    global _callback
    _callback = fn


def emit(stage: str, current: int, total: int, **extra) -> None:
    if _callback is not None:
        try:
            _callback(stage, current, total, int(extra.get("completed_bytes", 0)), int(extra.get("total_bytes", 0)))
        except Exception:          # a failing observer must not stop the load
            pass
    if os.environ.get("FTLLM_PROGRESS", "0") in ("0", "", "false"):
        return
    ev = {"stage": stage, "current": current, "total": total, "elapsed_s": round(time.time() - _t0, 3)}
    ev.update(extra)
    sys.stderr.write("FTLLM_PROGRESS " + json.dumps(ev) + "\n")
    sys.stderr.flush()
