"""Tensor-parallel sharding logic on CPU ranks (gloo): a TP=2 group must reproduce the single-rank tokens."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _worker(rank, world, port, name, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.models import TPInfo, preset, random_init
    from fastllm_b200.parallel.tp import TPComm

    torch.manual_seed(0)
    cfg = preset(name)
    tp = TPInfo(rank, world, TPComm(rank, world, "cpu"))
    m = random_init(cfg, "cpu", torch.float32, tp=tp, std=0.05)
    eng = LLMEngine(m, EngineConfig(max_batch=8, max_context=1024, chunked_prefill_size=100), num_pages=64)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 130)]
    outs = eng.generate(prompts, GenerationConfig(max_new_tokens=6, ignore_eos=True))
    if rank == 0:
        q.put(outs)
    dist.barrier()
    dist.destroy_process_group()


def _single(name):
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.models import preset, random_init

    cfg = preset(name)
    m = random_init(cfg, "cpu", torch.float32, std=0.05)
    eng = LLMEngine(m, EngineConfig(max_batch=8, max_context=1024, chunked_prefill_size=100), num_pages=64)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 130)]
    return eng.generate(prompts, GenerationConfig(max_new_tokens=6, ignore_eos=True))


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-qwen3-moe", "tiny-deepseek-v3"])
def test_tp2_matches_single(name):
    ref = _single(name)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 200)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, name, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert out == ref
