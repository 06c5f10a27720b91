"""Engine behaviour on CPU with tiny models: cache consistency, prefix reuse, chunked prefill, eviction + recompute,
abort, sampling, page manager, export round trip (quantised HF)."""
import pytest
import torch

from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
from fastllm_b200.engine.kv_cache import PageManager
from fastllm_b200.models import preset, random_init


def _model(name="tiny-llama"):
    torch.manual_seed(0)
    return random_init(preset(name), "cpu", torch.float32, std=0.05)


def _prompts(vocab, lens, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def test_paged_chunked_matches_full_recompute():
    for name in ("tiny-llama", "tiny-qwen3", "tiny-qwen3-moe", "tiny-deepseek-v3"):
        m = _model(name)
        eng = LLMEngine(m, EngineConfig(max_batch=8, max_context=1024, chunked_prefill_size=100), num_pages=64)
        prompts = _prompts(m.cfg.vocab_size, (5, 130, 260))
        outs = eng.generate(prompts, GenerationConfig(max_new_tokens=5, ignore_eos=True))
        eng2 = LLMEngine(m, EngineConfig(max_batch=8, max_context=1024, prefix_cache=False), num_pages=64)
        for p, o in zip(prompts, outs):
            seq = list(p)
            for k in range(5):
                t = eng2.generate([seq], GenerationConfig(max_new_tokens=1, ignore_eos=True))[0][0]
                assert t == o[k], (name, k)
                seq.append(t)


def test_prefix_cache_reuses_pages_and_keeps_output():
    m = _model()
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=1024), num_pages=32)
    p = _prompts(m.cfg.vocab_size, (300,))[0]
    a = eng.generate([p], GenerationConfig(max_new_tokens=4, ignore_eos=True))[0]
    h = eng.launch(p + [7, 8, 9], GenerationConfig(max_new_tokens=4, ignore_eos=True))
    req = eng.requests[h]
    while not req.finished():
        eng.step()
    assert req.stats.cached_tokens == 256          # two whole pages came from the trie
    b = eng.generate([p], GenerationConfig(max_new_tokens=4, ignore_eos=True))[0]
    assert a == b


def test_eviction_recompute_gives_same_tokens():
    m = _model()
    prompts = _prompts(m.cfg.vocab_size, (120, 125, 110))
    gen = GenerationConfig(max_new_tokens=40, ignore_eos=True)
    ref = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, prefix_cache=False), num_pages=32).generate(prompts, gen)
    small = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, prefix_cache=False, prefill_page_limit=1.0), num_pages=4)
    out = small.generate(prompts, gen)          # 3 requests x 2 pages do not fit in 4 pages: someone is evicted and recomputed
    assert out == ref


def test_eviction_of_a_request_later_in_the_batch():
    """A short request admitted first crosses a page boundary while a longer one, later in the batch, holds the
    remaining pages: the longer one is evicted on the short one's behalf and must then be skipped by the same
    page-allocation loop; both finish with the tokens of an unconstrained run and the pool ends fully free."""
    m = _model()
    p_short, p_long = _prompts(m.cfg.vocab_size, (100, 180), seed=3)
    gen = GenerationConfig(max_new_tokens=40, ignore_eos=True)
    ref = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, prefix_cache=False), num_pages=32).generate([p_short, p_long], gen)
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, prefix_cache=False, prefill_page_limit=1.0), num_pages=3)
    h0 = eng.launch(p_short, gen)
    eng.step()                                   # the short request is admitted and prefilled alone
    h1 = eng.launch(p_long, gen)
    reqs = [eng.requests[h0], eng.requests[h1]]
    for _ in range(2000):
        if all(r.finished() for r in reqs):
            break
        eng.step()
    assert [r.output_ids for r in reqs] == ref
    assert all(r.finish_reason == "length" for r in reqs)
    assert eng.pm.num_free() == 3


def test_engine_loop_survives_a_failed_step():
    """A step that raises ends the requests in flight with reason "error"; the background loop keeps serving."""
    m = _model()
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, prefix_cache=False), num_pages=16)
    real = eng.runner.decode
    state = {"fail": True}

    def flaky(*a, **k):
        if state["fail"]:
            state["fail"] = False
            raise RuntimeError("injected step failure")
        return real(*a, **k)

    eng.runner.decode = flaky
    eng.start()
    try:
        gen = GenerationConfig(max_new_tokens=4, ignore_eos=True)
        h = eng.launch(_prompts(m.cfg.vocab_size, (20,))[0], gen)
        toks = []
        while (t := eng.fetch(h)) >= 0:
            toks.append(t)
        assert len(toks) <= 1                       # at most the prefill's token came out before the failure
        assert isinstance(eng.error, RuntimeError) and not eng.dead
        h2 = eng.launch(_prompts(m.cfg.vocab_size, (20,))[0], gen)
        toks = []
        while (t := eng.fetch(h2)) >= 0:
            toks.append(t)
        assert len(toks) == 4
    finally:
        eng.stop()


def test_abort_releases_pages():
    m = _model()
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, prefix_cache=False), num_pages=16)
    h = eng.launch(_prompts(m.cfg.vocab_size, (200,))[0], GenerationConfig(max_new_tokens=100, ignore_eos=True))
    for _ in range(3):
        eng.step()
    eng.abort(h)
    eng.step()
    assert eng.requests[h].state.name == "ABORTED" and eng.pm.num_free() == 16
    assert eng.fetch(h) >= 0 or True
    while eng.fetch(h) >= 0:
        pass


def test_sampling_top_k_top_p():
    from fastllm_b200.engine import sampling

    torch.manual_seed(0)
    logits = torch.tensor([[0.0, 5.0, 4.9, -3.0]] * 200)
    t = sampling.sample(logits, [2] * 200, [1.0] * 200, [1.0] * 200)
    assert set(t.tolist()) <= {1, 2} and len(set(t.tolist())) == 2
    t = sampling.sample(logits, [4] * 200, [0.3] * 200, [1.0] * 200)
    assert set(t.tolist()) == {1}
    t = sampling.sample(logits, [0] * 200, [1.0] * 200, [1.0] * 200)          # top_k <= 0: top-k is off, not greedy
    assert len(set(t.tolist())) > 1
    lg = sampling.apply_repeat_penalty(torch.tensor([[2.0, -2.0, 1.0]]), [[0, 1]], [2.0])
    assert lg.tolist() == [[1.0, -4.0, 1.0]]


def test_page_manager_trie():
    pm = PageManager(8, 4)
    pages = pm.alloc(3)
    toks = list(range(12))
    pm.record(toks, pages)
    pm.release(pages)
    assert pm.num_free() == 5 and pm.num_available() == 8
    got = pm.query(toks + [99])
    assert got == pages                                  # whole-page prefix, references taken
    assert pm.query(toks) == pages[:2]                   # the page holding the last token is never matched
    pm.release(got)
    pm.release(pages[:2])
    assert pm.alloc(8) is not None                       # cached pages are evicted when the free list runs dry
    assert pm.stats()["cached"] == 0


def test_quantised_export_roundtrip(tmp_path):
    from baseline import synth
    from fastllm_b200.loader import hf
    from fastllm_b200.loader.export import export_quantized_hf

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    export_quantized_hf(d, str(tmp_path / "q"), "int8")
    a = hf.load_model(d, device="cpu", dtype=torch.float32, wdtype="int8")
    b = hf.load_model(str(tmp_path / "q"), device="cpu", dtype=torch.float32)
    wa, wb = a.layers[0].attn.qkv.dequant(torch.float32), b.layers[0].attn.qkv.dequant(torch.float32)
    assert (wa - wb).abs().max() < 2e-3


def test_engine_recovers_from_device_kernel_error():
    """Host-side fault injection: one forward raises the error a failed bounded wait produces.  The requests in flight end
    with reason "error", later requests are served, nothing hangs."""
    from fastllm_b200.models.config import preset
    from fastllm_b200.models.decoder import random_init
    from fastllm_b200.ops import _lib

    m = random_init(preset("tiny-llama"), "cpu", torch.float32, std=0.05)
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=256), num_pages=8)
    good = eng.generate([list(range(3, 20))], GenerationConfig(max_new_tokens=4, ignore_eos=True))[0]
    h = eng.launch(list(range(3, 20)), GenerationConfig(max_new_tokens=8, ignore_eos=True))
    eng.step()                          # prefill
    orig = eng.runner.decode
    calls = {"n": 0}

    def failing(*a, **k):
        calls["n"] += 1
        if calls["n"] == 2:
            raise _lib.DeviceKernelError("kernel 7 site 1: wait ran out (injected)")
        return orig(*a, **k)

    eng.runner.decode = failing
    for _ in range(6):
        eng.step()
    r = eng.requests[h]
    assert r.finished() and r.finish_reason == "error" and eng.device_errors == 1
    eng.runner.decode = orig
    again = eng.generate([list(range(3, 20))], GenerationConfig(max_new_tokens=4, ignore_eos=True))[0]
    assert again == good
    assert eng.pm.stats()["free"] + eng.pm.stats()["cached"] == 8      # no page leaked by the failed request


def test_add_cache_populates_prefix_cache(tmp_path):
    from baseline import synth
    from fastllm_b200 import llm

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    llm.set_device_map("cpu")
    m = llm.model(d, device="cpu")
    prefix = list(range(3, 3 + 300))                      # two full 128-token pages + a tail
    assert m.add_cache(prefix) == 300
    h = m.launch_stream_response(prefix + [7, 8, 9], max_length=2, do_sample=False)
    req = m.engine.requests[h]
    while m.engine.fetch(h) >= 0:
        pass
    assert req.stats.as_dict()["cached_tokens"] >= 256
    m.release_memory()


def test_llm_model_adapter_switching(tmp_path):
    import pytest

    """``load_adapter`` / ``set_adapter`` / ``disable_adapter`` on a loaded model change (and restore) what it generates."""
    import json

    from baseline import synth
    from fastllm_b200 import llm
    from fastllm_b200.loader.safetensors import save_file

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    llm.set_device_map("cpu")
    m = llm.model(d, device="cpu")
    c = m.engine.model.cfg
    torch.manual_seed(2)
    t = {}
    for i in range(c.num_layers):
        t[f"base_model.model.model.layers.{i}.mlp.down_proj.lora_A.weight"] = torch.randn(4, c.intermediate_size) * 0.3
        t[f"base_model.model.model.layers.{i}.mlp.down_proj.lora_B.weight"] = torch.randn(c.hidden_size, 4) * 0.3
    ad = tmp_path / "ad"
    ad.mkdir()
    (ad / "adapter_config.json").write_text(json.dumps({"r": 4, "lora_alpha": 8}))
    save_file(t, ad / "adapter_model.safetensors")
    prompt = list(range(5, 40))

    def run():
        h = m.launch_stream_response(prompt, max_length=6, do_sample=False)
        out = []
        while True:
            tok = m.engine.fetch(h)
            if tok < 0:
                return out
            out.append(tok)

    base = run()
    with pytest.raises(KeyError):
        m.set_adapter("a")
    assert m.load_adapter("a", str(ad)) == c.num_layers
    try:
        m.set_adapter("a")
        tuned = run()
        assert tuned != base
    finally:
        m.disable_adapter()
    assert run() == base
    m.release_memory()


def test_fp8_kv_cache(tmp_path):
    """``kv_cache_dtype="fp8_e4m3"``: e4m3 pages (half the bytes), generation close to the 16/32-bit cache."""
    from baseline import synth
    from fastllm_b200 import llm

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    llm.set_device_map("cpu")
    prompt = list(range(5, 150))
    outs, logits = [], []
    for kvd in ("auto", "fp8_e4m3"):
        m = llm.model(d, device="cpu", kv_cache_dtype=kvd)
        k_pool = m.engine.runner.kv.pools[0][0]
        assert (k_pool.dtype == torch.float8_e4m3fn) == (kvd != "auto")
        logits.append(torch.as_tensor(m.response_logits(prompt)).float())
        h = m.launch_stream_response(prompt, max_length=4, do_sample=False)
        toks = []
        while True:
            t = m.engine.fetch(h)
            if t < 0:
                break
            toks.append(t)
        outs.append(toks)
        m.release_memory()
    assert len(outs[1]) == 4
    assert torch.nn.functional.cosine_similarity(logits[0].flatten(), logits[1].flatten(), dim=0) > 0.99


def test_module_level_switches(tmp_path, capsys):
    """The reference's module-level helpers exist and behave: device probes, progress callback, graph-node helpers, settings."""
    from baseline import synth
    from fastllm_b200 import llm

    assert llm.has_device("cpu") and not llm.has_device("tfacc")
    assert abs(float(llm.softmax([1.0, 2.0, 3.0]).sum()) - 1.0) < 1e-9
    assert llm.GraphNode("x") == {"name": "x", "type": "data"}
    assert llm.FloatGraphNode(2)["type"] == "constant.float" and llm.IntGraphNode(3.0)["value"] == 3
    llm.set_cpu_kvcache(True)
    assert llm.get_cpu_kvcache()
    llm.set_cpu_kvcache(False)
    llm.set_cpu_low_mem(True)
    assert llm.get_cpu_low_mem()
    llm.set_cpu_low_mem(False)
    for f, a in ((llm.set_cuda_embedding, True), (llm.set_cuda_slab, 64), (llm.set_enable_amx, False), (llm.set_cuda_shared_expert, True),
                 (llm.set_moe_device_layers, -1)):
        f(a)
    llm.disable_cuda_malloc()
    llm.print_ins_info()
    assert "cpu backend" in capsys.readouterr().out
    events = []
    llm.set_model_load_progress_callback(lambda stage, cur, tot, cb, tb: events.append((stage, cur, tot)))
    try:
        d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
        llm.set_device_map("cpu")
        m = llm.model(d, device="cpu")
        n = m.engine.model.cfg.num_layers
        assert ("load_weights", n, n) in events
        llm.report_model_load_progress("custom", 1, 2)
        assert events[-1] == ("custom", 1, 2)
        m.release_memory()
    finally:
        llm.set_model_load_progress_callback(None)


def test_model_convenience_methods(tmp_path):
    """``generate`` / ``chat`` / ``stream_chat`` / token helpers / run-time setters of the reference's ``model`` class."""
    import pytest

    from baseline import synth
    from fastllm_b200 import llm

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    llm.set_device_map("cpu")
    m = llm.model(d, device="cpu")
    assert m.eval() is m
    prompt = list(range(5, 25))
    outs = m.generate([prompt, prompt[:7]], max_length=5, do_sample=False)
    assert outs[0][:len(prompt)] == prompt and len(outs[0]) == len(prompt) + 5 and len(outs[1]) == 7 + 5
    again = m.generate(torch.tensor([prompt]), max_length=5, do_sample=False)
    assert again[0] == outs[0]
    text, hist = m.chat(None, "hello", history=[], max_length=4, do_sample=False)
    assert hist == [("hello", text)]
    last = None
    for last in m.stream_chat(None, "hello", history=[], max_length=4, do_sample=False):
        pass
    assert (last[0] if last is not None else "") == text
    n = m.get_input_token_len([{"role": "user", "content": [{"type": "text", "text": "hello"}]}])
    assert n == m.get_input_token_len([{"role": "user", "content": "hello"}]) > 0
    ids = m.tokenizer_encode_string("hello world")
    assert b"".join(m.tokenizer_decode_token(i) for i in ids).decode("utf-8", errors="ignore").strip() == m.decode(ids).strip()
    m.set_max_batch(3)
    assert m.get_max_batch() == 3
    m.set_chunked_prefill_size(256)
    m.set_max_context_length(512)
    m.set_kv_cache_limit("2G")
    assert m.kv_cache_limit_bytes == 2 << 30
    have = str(m.torch_model.dtype).replace("torch.", "")
    m.set_atype(have)
    with pytest.raises(ValueError):
        m.set_atype("float16" if have != "float16" else "float32")
    with pytest.raises(RuntimeError):
        m.set_kv_cache_dtype("fp8_e4m3")
    m.release_memory()


def test_decode_rides_along_with_prefill_chunks():
    """A request that is decoding keeps producing one token per scheduler step while a long prompt is prefilled in chunks, and
    both end with the tokens of an unmixed run."""
    m = _model()
    short, long_ = _prompts(m.cfg.vocab_size, (20, 700), seed=5)
    gen = GenerationConfig(max_new_tokens=12, ignore_eos=True)
    ref = LLMEngine(m, EngineConfig(max_batch=4, max_context=1024, prefix_cache=False, mixed_prefill_decode=False),
                    num_pages=32).generate([short, long_], gen)
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=1024, prefix_cache=False, chunked_prefill_size=128), num_pages=32)
    h0 = eng.launch(short, gen)
    eng.step()                                      # prefill of the short request -> its first token
    r0 = eng.requests[h0]
    assert len(r0.output_ids) == 1
    h1 = eng.launch(long_, gen)
    r1 = eng.requests[h1]
    per_step = []
    while r1.state.name in ("WAITING", "PREFILL"):
        before = len(r0.output_ids)
        eng.step()
        per_step.append(len(r0.output_ids) - before)
    assert len(per_step) >= 5 and all(n == 1 for n in per_step[:5])     # never stalled by the 700-token prompt
    while not (r0.finished() and r1.finished()):
        eng.step()
    assert [r0.output_ids, r1.output_ids] == ref


@pytest.mark.parametrize("preset_name", ["tiny-qwen3-next", "tiny-minimax-m1"])
def test_hybrid_linear_attention_engine_consistency(preset_name):
    """Hybrid stacks (Gated DeltaNet of Qwen3-Next, lightning attention of MiniMax-M1): chunked prefill + stateful decode
    (per-request state slots) reproduces token-by-token recomputation; eviction restarts a request from empty state; slots
    are returned."""
    m = _model(preset_name)
    assert m.cfg.has_linear_attn and m.layers[0].lin is not None and m.layers[1].lin is None
    prompts = _prompts(m.cfg.vocab_size, (5, 130, 70))
    gen = GenerationConfig(max_new_tokens=6, ignore_eos=True)
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, chunked_prefill_size=48), num_pages=32)
    outs = eng.generate(prompts, gen)
    assert sorted(eng.state_free) == [0, 1, 2, 3] and not eng.cfg.prefix_cache
    eng2 = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=32)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for k in range(6):
            t = eng2.generate([seq], GenerationConfig(max_new_tokens=1, ignore_eos=True))[0][0]
            assert t == o[k], k
            seq.append(t)
    # a pool too small for all three: someone is evicted, recomputed from scratch (state reset) and still matches
    small = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, prefill_page_limit=1.0), num_pages=3)
    assert small.generate(prompts, GenerationConfig(max_new_tokens=30, ignore_eos=True)) == \
        LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=32).generate(prompts, GenerationConfig(max_new_tokens=30, ignore_eos=True))


def test_ngram_speculative_decoding_keeps_greedy_output():
    """Prompt-lookup drafts verified in one forward pass: same tokens as plain greedy decoding, in fewer steps when the
    text repeats itself."""
    m = _model()
    base = _prompts(m.cfg.vocab_size, (24,), seed=9)[0]
    prompts = [base * 5, _prompts(m.cfg.vocab_size, (40,), seed=10)[0]]          # one very repetitive, one random
    gen = GenerationConfig(max_new_tokens=40, ignore_eos=True)
    plain = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=32)
    ref = plain.generate(prompts, gen)
    spec = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, speculative="ngram", speculative_tokens=4), num_pages=32)
    out = spec.generate(prompts, gen)
    assert out == ref
    assert spec.spec_proposed > 0 and 0 <= spec.spec_accepted <= spec.spec_proposed
    assert spec.pm.num_available() == 32
    # a greedy model that has entered a cycle repeats it: the drafts are then accepted and steps are saved
    if spec.spec_accepted > 0:
        assert spec.decode_steps < plain.decode_steps


def test_candidate_sampling_matches_whole_row_sampling():
    """Vocab-sharded sampling on per-shard top-k candidates: with repetition penalties the chosen token equals the penalised
    whole-row arg-max (greedy) and lies in the penalised whole-row top-k (sampling), for shards split at any point."""
    from types import SimpleNamespace

    from fastllm_b200.engine import sampling

    m = _model()
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=256), num_pages=8)
    g = torch.Generator().manual_seed(5)
    V, R = 512, 6
    for trial in range(8):
        logits = torch.randn(R, V, generator=g) * 3
        reqs = []
        for r in range(R):
            recent = torch.randint(0, V, (40,), generator=g).tolist() + logits[r].topk(3).indices.tolist()    # the best tokens are penalised
            gen = GenerationConfig(max_new_tokens=4, do_sample=(r % 2 == 1), top_k=5, top_p=1.0, temperature=0.7, repeat_penalty=1.8)
            reqs.append(SimpleNamespace(gen=gen, all_ids=recent, output_ids=[]))
        k = eng._candidate_width(reqs)
        assert k >= 5 + 1 and (k & (k - 1)) == 0
        cut = [100, 256, 400, 37][trial % 4]
        vals, ids = [], []
        for lo, hi in ((0, cut), (cut, V)):
            v, i = logits[:, lo:hi].topk(min(k, hi - lo), dim=-1)
            pad = k - v.shape[1]
            if pad > 0:
                v = torch.cat([v, torch.full((R, pad), float("-inf"))], dim=1)
                i = torch.cat([i, torch.zeros((R, pad), dtype=torch.long)], dim=1)
            vals.append(v); ids.append(i + lo)
        got = eng._sample_candidates(reqs, torch.cat(vals, 1), torch.cat(ids, 1))
        full = logits.clone()
        sampling.apply_repeat_penalty(full, [r.all_ids for r in reqs], [1.8] * R)
        for r in range(R):
            if r % 2 == 0:
                assert got[r] == int(full[r].argmax())
            else:
                assert got[r] in full[r].topk(5).indices.tolist()
    # whole rows are needed for log-probabilities / returned logits / logits processors
    reqs[0].gen.logprobs = 3
    assert eng._candidate_width(reqs) == 0


def _mtp_model(identity_layers: bool):
    from fastllm_b200.models import preset, random_init

    m = random_init(preset("tiny-llama-mtp"), "cpu", torch.float32, seed=3, std=0.05)
    assert m.mtp is not None and len(m.layers) == 2
    if identity_layers:
        # every decoder layer (the draft head's too) adds nothing to the residual stream: the next token then depends on the
        # current token alone, and a head whose fusion keeps the embedding half predicts exactly what the decoder will say
        H = m.cfg.hidden_size
        for lw in list(m.layers) + [m.mtp.layer]:
            lw.attn.o.w.zero_()
            lw.mlp.down.w.zero_()
        m.mtp.fc.w.zero_()
        m.mtp.fc.w[:, :H] = torch.eye(H)
    return m


@pytest.mark.parametrize("k", [1, 3])
def test_mtp_speculative_matches_greedy(k):
    """Drafts from the multi-token-prediction head never change the output: with random head weights (drafts mostly rejected)
    and chunked prefill, several requests at once, the tokens equal plain greedy decoding."""
    m = _mtp_model(False)
    prompts = _prompts(m.cfg.vocab_size, (40, 150, 9))
    gen = GenerationConfig(max_new_tokens=12, ignore_eos=True)
    ref = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=16).generate(prompts, gen)
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, chunked_prefill_size=64, speculative="mtp", speculative_tokens=k),
                    num_pages=16)
    out = eng.generate(prompts, gen)
    assert out == ref
    assert eng.spec_proposed > 0


def test_mtp_head_that_predicts_the_decoder_is_accepted():
    """With decoder layers that add nothing and a head that keeps the embedding half of its fused input, every draft is what
    the decoder says next: all drafts are accepted and a step yields speculative_tokens + 1 tokens."""
    m = _mtp_model(True)
    prompts = _prompts(m.cfg.vocab_size, (30, 70))
    gen = GenerationConfig(max_new_tokens=16, ignore_eos=True)
    ref = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=16).generate(prompts, gen)
    for k in (1, 3):
        eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, chunked_prefill_size=32, speculative="mtp", speculative_tokens=k),
                        num_pages=16)
        assert eng.generate(prompts, gen) == ref
        assert eng.spec_proposed > 0 and eng.spec_accepted == eng.spec_proposed
        assert eng.decode_steps <= 2 * (16 // (k + 1) + 2)


@pytest.mark.parametrize("algo", ["ngram", "mtp"])
def test_speculative_decoding_on_a_hybrid_model(algo):
    """Gated-DeltaNet hybrid: a rejected draft has advanced the recurrent state, which is put back from a snapshot and rebuilt
    from the accepted tokens -- the output equals plain greedy decoding for prompt-lookup drafts and for the draft head."""
    import dataclasses

    from fastllm_b200.models import preset, random_init

    cfg = dataclasses.replace(preset("tiny-qwen3-next"), mtp_layers=1)
    m = random_init(cfg, "cpu", torch.float32, seed=5, std=0.05)
    assert m.mtp is not None and m.cfg.has_linear_attn
    base = [3, 9, 4, 7, 11, 5]
    prompts = [base * 6, _prompts(cfg.vocab_size, (50,))[0]]
    gen = GenerationConfig(max_new_tokens=14, ignore_eos=True)
    ref = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=16).generate(prompts, gen)
    eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, chunked_prefill_size=32, speculative=algo, speculative_tokens=3),
                    num_pages=16)
    assert eng.generate(prompts, gen) == ref
    assert eng.spec_proposed > 0 and eng.spec_accepted < eng.spec_proposed       # some drafts were rejected and rolled back


@pytest.mark.parametrize("same", [False, True])
def test_draft_model_speculative_matches_greedy(same):
    """A separate draft model never changes the output.  ``same``: the draft is a copy of the target, so every draft is what the
    target says next (all accepted, k + 1 tokens per step); otherwise a smaller model with other weights (drafts mostly
    rejected).  Chunked prefill, several requests, prefix reuse between two requests, page pools shared by page id."""
    import dataclasses

    from fastllm_b200.models import preset, random_init

    cfg = preset("tiny-llama")
    m = random_init(cfg, "cpu", torch.float32, seed=3, std=0.05)
    if same:
        d = random_init(cfg, "cpu", torch.float32, seed=3, std=0.05)
    else:
        d = random_init(dataclasses.replace(cfg, num_layers=1), "cpu", torch.float32, seed=11, std=0.05)
    prompts = _prompts(cfg.vocab_size, (40, 150, 9))
    prompts.append(prompts[1][:140] + [5, 6, 7])           # shares a whole-page prefix with the second prompt
    gen = GenerationConfig(max_new_tokens=13, ignore_eos=True)
    ref = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=16).generate(prompts, gen)
    for k in (1, 3):
        eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512, chunked_prefill_size=64, speculative="draft", speculative_tokens=k),
                        num_pages=16, draft_model=d)
        assert eng.generate(prompts, gen) == ref
        assert eng.spec_proposed > 0
        if same:
            assert eng.spec_accepted == eng.spec_proposed
            assert eng.decode_steps <= 13 // (k + 1) + 3
        # a later request whose prompt is cached: the draft model reads the shared pages under the same page ids
        again = eng.generate([prompts[1]], gen)
        assert again == [ref[1]]
    with pytest.raises(ValueError):
        LLMEngine(m, EngineConfig(speculative="draft"), num_pages=16,
                  draft_model=random_init(dataclasses.replace(cfg, vocab_size=cfg.vocab_size + 8), "cpu", torch.float32, seed=1))


def test_draft_model_through_llm_model(tmp_path):
    """``--speculative_algorithm draft --speculative_draft_model_path DIR``: the option parser sets the draft path, ``llm.model``
    loads the draft beside the target, and the replies equal those without speculation."""
    import sys

    sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parent.parent))
    from baseline import synth
    from fastllm_b200 import llm, util

    big = synth.write_model("tiny-llama", str(tmp_path / "big"), dtype=torch.float32, std=0.05)
    small = synth.write_model("tiny-llama", str(tmp_path / "small"), dtype=torch.float32, std=0.05, seed=9)
    llm.set_device_map("cpu")
    keep = dict(llm._settings)
    try:
        plain = llm.model(big, device="cpu", dtype="float32")
        want = list(plain.stream_response_raw([5, 6, 7, 8, 9, 10], max_length=12, do_sample=False))
        plain.release_memory()
        args = util.make_normal_parser().parse_args([big, "--device", "cpu", "--dtype", "float32", "--speculative_algorithm", "draft",
                                              "--speculative_draft_model_path", small, "--speculative_dspark_block_size", "3"])
        m = util.make_normal_llm_model(args)
        try:
            assert m.engine.draft is not None and m.engine.cfg.speculative == "draft" and m.engine.cfg.speculative_tokens == 3
            assert list(m.stream_response_raw([5, 6, 7, 8, 9, 10], max_length=12, do_sample=False)) == want
            assert m.engine.spec_proposed > 0
        finally:
            m.release_memory()
    finally:
        llm._settings.clear()
        llm._settings.update(keep)
