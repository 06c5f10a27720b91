"""Fused tensor-parallel kernels on 2 GPUs (skipped on boxes with fewer).  Runs with NVLS multicast and
with plain peer loads/stores."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("multicast", ["1", "0"])
def test_fused_tp_two_gpus(multicast):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, FB_TEST_MULTICAST=multicast)
    port = 29700 + os.getpid() % 100 + (1 if multicast == "1" else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "tp_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TP_GPU_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_layer_split_placement_two_gpus(tmp_path):
    """Layer-split device map: half the layers on each GPU, same greedy tokens as the single-GPU model."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from baseline import synth
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.loader import hf

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.bfloat16, std=0.05)
    prompts = [list(range(3, 90, 2)), list(range(5, 30))]
    outs = []
    for dm in (None, {"cuda:0": 1, "cuda:1": 1}):
        m = hf.load_model(d, device="cuda:0", device_map=dm)
        if dm:
            assert [str(x) for x in m.layer_devices] == ["cuda:0", "cuda:1"]
            assert m.layers[1].attn.qkv.w.device.index == 1 and m.lm_head.w.device.index == 1
        eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=256), num_pages=8)
        outs.append(eng.generate(prompts, GenerationConfig(max_new_tokens=6, ignore_eos=True)))
    assert outs[0] == outs[1]


def test_server_command_tp2_streams_on_two_gpus(tmp_path):
    """``ftllm server <model> --tp 2`` on two GPUs: rank 0 serves HTTP and schedules, the spawned rank 1 replays its step
    plans; the fused NVLink kernels run under CUDA graphs.  One streamed chat completion must arrive and finish."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from baseline import synth
    from tests.serve_tp_helper import run_server_and_stream

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.bfloat16, std=0.05)
    chunks, finish = run_server_and_stream(d, ["--tp", "2"])
    assert finish in ("length", "stop") and len(chunks) >= 1
