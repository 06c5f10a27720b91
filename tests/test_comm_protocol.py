"""Host-thread model of the counter / expect / ticket protocol of the fused tensor-parallel kernels: ranks x CTAs as threads
over atomics, random delays, many launches back to back; no slot or gathered row may be read stale and no wait may run out."""
import ctypes

import pytest

from fastllm_b200.ops import _lib


def _model():
    L = _lib.runtime()
    L.fbmodel_comm_protocol.argtypes = [ctypes.c_int] * 5 + [ctypes.c_uint]
    L.fbmodel_comm_protocol.restype = ctypes.c_int
    return L.fbmodel_comm_protocol


@pytest.mark.parametrize("tp,ctas,defer", [(2, 4, 0), (2, 3, 1), (4, 2, 0), (4, 2, 1), (8, 1, 1)])
def test_counter_protocol_holds_under_random_delays(tp, ctas, defer):
    assert _model()(tp, ctas, 300, defer, 3, 1234 + tp + ctas) == 0


def test_model_rejects_bad_arguments():
    assert _model()(0, 1, 1, 0, 1, 0) == -1


def test_model_notices_a_missing_consumer_wait():
    """The broken variant (deferred all-gather, consumer does not wait) must show stale rows: the model is sensitive."""
    assert any(_model()(4, 2, 400, 2, 3, seed) > 0 for seed in range(5))
