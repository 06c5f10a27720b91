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


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-qwen3-moe", "tiny-deepseek-v3", "tiny-minimax-m1", "tiny-minimax-m2", "tiny-hy-v3", "tiny-pangu-moe", "tiny-minicpm3", "tiny-moss", "tiny-step3p5", "tiny-laguna", "tiny-deepseek-v32"])
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


# ---------------------------------------------------------------------------------------------------------
# control plane: only rank 0 schedules; the worker rank is a separate process replaying published step plans
# ---------------------------------------------------------------------------------------------------------
_SPEC = {"kind": "preset", "model": "tiny-llama", "dtype": "float32", "std": 0.05, "seed": 0, "num_pages": 6,
         "engine": {"max_batch": 4, "max_context": 512, "prefix_cache": False, "prefill_page_limit": 1.0,
                    "chunked_prefill_size": 100}}


def _scenario(eng):
    """Three requests through the public launch / fetch / abort calls, on a pool small enough to force an eviction."""
    from fastllm_b200.engine import GenerationConfig

    g = torch.Generator().manual_seed(7)
    vocab = eng.model.cfg.vocab_size
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (120, 125, 110, 90)]
    gen = GenerationConfig(max_new_tokens=40, ignore_eos=True)
    hs = [eng.launch(p, gen) for p in prompts[:3]]
    doomed = eng.launch(prompts[3], GenerationConfig(max_new_tokens=200, ignore_eos=True))
    reqs = [eng.requests[h] for h in hs]
    dreq = eng.requests[doomed]
    sampled = eng.launch(prompts[0][:30], GenerationConfig(max_new_tokens=5, ignore_eos=True, do_sample=True, top_k=5, temperature=0.8))
    sreq = eng.requests[sampled]
    steps = 0
    while not all(r.finished() for r in reqs + [dreq, sreq]):
        eng.step()
        steps += 1
        if steps == 6:
            eng.abort(doomed)
        assert steps < 5000
    return [r.output_ids for r in reqs], dreq.state.name, len(sreq.output_ids), eng.pm.num_free()


def _rank0_with_spawned_worker(q):
    from fastllm_b200.parallel.launcher import TPGroup

    group, eng, _ = TPGroup.launch(_SPEC, ["cpu", "cpu"])
    try:
        assert eng.control is not None and eng.model.tp.size == 2
        out = _scenario(eng)
        q.put((out, eng.control.published))
    finally:
        group.shutdown()
    assert all(p.returncode == 0 for p in group.procs)


def test_control_plane_spawned_worker_follows_rank0():
    from fastllm_b200.engine import EngineConfig, LLMEngine
    from fastllm_b200.models import preset, random_init

    m = random_init(preset("tiny-llama"), "cpu", torch.float32, std=0.05, seed=0)
    eng = LLMEngine(m, EngineConfig(**_SPEC["engine"]), num_pages=_SPEC["num_pages"])
    ref = _scenario(eng)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_rank0_with_spawned_worker, args=(q,))
    p.start()
    out, published = q.get(timeout=300)
    p.join(timeout=60)
    assert p.exitcode == 0
    assert out[0] == ref[0]                      # same tokens as one rank, through eviction + recompute
    assert out[1] == "ABORTED" and out[2] == 5   # the aborted request ended; the sampled one (logits gathered over ranks) finished
    assert out[3] == _SPEC["num_pages"]          # every page returned
    assert published > 40                        # the worker was driven by plans, one per forward pass


def _attached_rank(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from fastllm_b200.parallel.launcher import TPGroup

    group, eng, _ = TPGroup.attach(_SPEC, device="cpu")
    if group is None:                            # worker rank: attach() returned after rank 0 shut the group down
        q.put(("worker", eng.worker_loop.steps))
        return
    try:
        q.put(("rank0", _scenario(eng)))
    finally:
        group.shutdown()


def test_control_plane_attach_mode():
    """Ranks started by an outer launcher (what torchrun does): rank 0 schedules, rank 1 serves inside attach()."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29800 + (os.getpid() % 150)
    procs = [ctx.Process(target=_attached_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got["worker"] > 40 and got["rank0"][1] == "ABORTED" and got["rank0"][3] == _SPEC["num_pages"]


def _public_api_tp(path, q):
    from fastllm_b200 import llm

    llm.set_device_map("cpu")
    m = llm.model(path, tp=["cpu", "cpu"])                 # spawns the second rank
    try:
        assert m._group is not None and m.torch_model.tp.size == 2
        toks = list(m.stream_response_raw(list(range(3, 40)), max_length=8, do_sample=False))
        q.put(toks)
    finally:
        m.shutdown()


def test_llm_model_tp_argument_spawns_ranks(tmp_path):
    """``llm.model(path, tp=[...])`` -- the call ``ftllm server --tp N`` makes -- serves over two ranks."""
    from baseline import synth
    from fastllm_b200 import llm

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    llm.set_device_map("cpu")
    single = llm.model(d)
    ref = list(single.stream_response_raw(list(range(3, 40)), max_length=8, do_sample=False))
    single.shutdown()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_public_api_tp, args=(d, q))
    p.start()
    out = q.get(timeout=300)
    p.join(timeout=60)
    assert p.exitcode == 0 and out == ref and len(out) > 0


def test_server_command_with_tp_streams_a_chat_completion(tmp_path):
    """``ftllm server <model> --device cpu --tp 2``: the one command starts both ranks; an HTTP client streams a completion."""
    from baseline import synth
    from tests.serve_tp_helper import run_server_and_stream

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    chunks, finish = run_server_and_stream(d, ["--device", "cpu", "--tp", "2", "--dtype", "float32"])
    assert finish in ("length", "stop") and len(chunks) >= 1


_SPEC_MTP = {"kind": "preset", "model": "tiny-llama-mtp", "dtype": "float32", "std": 0.05, "seed": 0, "num_pages": 12,
             "engine": {"max_batch": 4, "max_context": 512, "prefix_cache": False, "chunked_prefill_size": 64,
                        "speculative": "mtp", "speculative_tokens": 2}}


def _mtp_prompts(vocab):
    g = torch.Generator().manual_seed(11)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (70, 33)]


def _rank0_mtp(q):
    from fastllm_b200.engine import GenerationConfig
    from fastllm_b200.parallel.launcher import TPGroup

    group, eng, _ = TPGroup.launch(_SPEC_MTP, ["cpu", "cpu"])
    try:
        assert eng.model.tp.size == 2 and eng.model.mtp is not None
        out = eng.generate(_mtp_prompts(eng.model.cfg.vocab_size), GenerationConfig(max_new_tokens=12, ignore_eos=True))
        q.put((out, eng.spec_proposed))
    finally:
        group.shutdown()
    assert all(p.returncode == 0 for p in group.procs)


def test_control_plane_carries_the_draft_head_passes():
    """Drafts from the multi-token-prediction head under tensor parallelism: the worker rank replays the decoder passes (keeping
    their hidden rows), the head's passes and the candidate exchanges from the published plans; tokens equal one rank's greedy
    output."""
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.models import preset, random_init

    m = random_init(preset("tiny-llama-mtp"), "cpu", torch.float32, std=0.05, seed=0)
    ref = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=12).generate(
        _mtp_prompts(m.cfg.vocab_size), GenerationConfig(max_new_tokens=12, ignore_eos=True))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_rank0_mtp, args=(q,))
    p.start()
    out, proposed = q.get(timeout=300)
    p.join(timeout=60)
    assert p.exitcode == 0
    assert out == ref and proposed > 0


_SPEC_MM = {"kind": "preset", "model": "tiny-qwen3", "dtype": "float32", "std": 0.05, "seed": 0, "num_pages": 8,
            "config_raw": {"rope_parameters": {"mrope_section": [24, 20, 20]}},
            "engine": {"max_batch": 4, "max_context": 512, "prefix_cache": False, "chunked_prefill_size": 16}}


def _mm_case(cfg):
    from fastllm_b200.engine.engine import MultimodalContext
    from fastllm_b200.models import vision as V

    ids = [5, 6, 7] + [9] * 12 + [8, 10, 11, 12]
    pos3, delta = V.mrope_positions(ids, 9, [(1, 6, 8)], 2)
    emb = torch.randn(12, cfg.hidden_size, generator=torch.Generator().manual_seed(1)) * 0.05
    return ids, MultimodalContext(emb, [i for i, t in enumerate(ids) if t == 9], pos3, delta)


def _rank0_mm(q):
    from fastllm_b200.engine import GenerationConfig
    from fastllm_b200.parallel.launcher import TPGroup

    group, eng, _ = TPGroup.launch(_SPEC_MM, ["cpu", "cpu"])
    try:
        assert eng.model.cfg.raw["rope_parameters"]["mrope_section"] == [24, 20, 20]
        ids, mm = _mm_case(eng.model.cfg)
        h = eng.launch(ids, GenerationConfig(max_new_tokens=6, ignore_eos=True), mm=mm)
        text = eng.launch([3, 4, 5, 6, 7, 8, 9, 10], GenerationConfig(max_new_tokens=4, ignore_eos=True))
        reqs = [eng.requests[h], eng.requests[text]]
        while not all(r.finished() for r in reqs):
            eng.step()
        q.put([r.output_ids for r in reqs])
    finally:
        group.shutdown()
    assert all(p.returncode == 0 for p in group.procs)


def test_control_plane_carries_image_prompts():
    """A prompt with image tokens under tensor parallelism: rank 0 hands the embeddings and 3-D rotary positions to the worker
    rank, whose replayed chunks refer to them; tokens equal one rank's output (a text request runs alongside)."""
    from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
    from fastllm_b200.models import preset, random_init

    m = random_init(preset("tiny-qwen3"), "cpu", torch.float32, std=0.05, seed=0)
    m.cfg.raw["rope_parameters"] = {"mrope_section": [24, 20, 20]}
    eng = LLMEngine(m, EngineConfig(**_SPEC_MM["engine"]), num_pages=8)
    ids, mm = _mm_case(m.cfg)
    h = eng.launch(ids, GenerationConfig(max_new_tokens=6, ignore_eos=True), mm=mm)
    t = eng.launch([3, 4, 5, 6, 7, 8, 9, 10], GenerationConfig(max_new_tokens=4, ignore_eos=True))
    reqs = [eng.requests[h], eng.requests[t]]
    while not all(r.finished() for r in reqs):
        eng.step()
    ref = [r.output_ids for r in reqs]
    plain = LLMEngine(m, EngineConfig(**_SPEC_MM["engine"]), num_pages=8).generate([ids], GenerationConfig(max_new_tokens=6, ignore_eos=True))[0]
    assert plain != ref[0]                      # the image embeddings and positions matter for this prompt
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_rank0_mm, args=(q,))
    p.start()
    out = q.get(timeout=300)
    p.join(timeout=60)
    assert p.exitcode == 0 and out == ref
