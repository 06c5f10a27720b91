"""ComputeGraph custom models: a Llama described operator by operator (the reference's example/python/qwen2.py pattern)
generates the same tokens as the built-in decoder, the graph serialises to JSON, and a model file with ``__model__`` loads."""
import json
import math
import textwrap

import torch

from fastllm_b200.engine import EngineConfig, GenerationConfig, LLMEngine
from fastllm_b200.graph import ComputeGraph, load_custom_file, load_graph_model
from fastllm_b200.loader import hf

MODEL_FILE = textwrap.dedent('''
    import math
    from fastllm_b200.llm import ComputeGraph

    class TinyLlama(ComputeGraph):
        def build(self):
            weight, data, config = self.weight, self.data, self.config
            config["max_positions"] = config["max_position_embeddings"]
            head_dim = config["head_dim"]
            self.Embedding(data["inputIds"], weight["model.embed_tokens.weight"], data["hiddenStates"])
            self.DataTypeAs(data["hiddenStates"], data["atype"])
            for i in range(config["num_hidden_layers"]):
                layer = weight["model.layers."][i]
                self.RMSNorm(data["hiddenStates"], layer[".input_layernorm.weight"], config["rms_norm_eps"], data["attenInput"])
                for n in "qkv":
                    self.Linear(data["attenInput"], layer[".self_attn." + n + "_proj.weight"], None, data[n])
                    self.ExpandHead(data[n], head_dim)
                self.LlamaRotatePosition2D(data["q"], data["positionIds"], data["sin"], data["cos"], head_dim // 2)
                self.LlamaRotatePosition2D(data["k"], data["positionIds"], data["sin"], data["cos"], head_dim // 2)
                self.FusedAttention(data["q"], data["pastKey."][i], data["pastValue."][i], data["k"], data["v"], data["attenInput"],
                                    data["attentionMask"], data["attenOutput"], data["seqLens"], 1.0 / math.sqrt(head_dim))
                self.Linear(data["attenOutput"], layer[".self_attn.o_proj.weight"], None, data["attenLastOutput"])
                self.AddTo(data["hiddenStates"], data["attenLastOutput"])
                self.RMSNorm(data["hiddenStates"], layer[".post_attention_layernorm.weight"], config["rms_norm_eps"], data["attenInput"])
                self.Linear(data["attenInput"], layer[".mlp.gate_proj.weight"], None, data["w1"])
                self.Linear(data["attenInput"], layer[".mlp.up_proj.weight"], None, data["w3"])
                self.Silu(data["w1"], data["w1"])
                self.MulTo(data["w1"], data["w3"])
                self.Linear(data["w1"], layer[".mlp.down_proj.weight"], None, data["w2"])
                self.AddTo(data["hiddenStates"], data["w2"])
            self.SplitLastTokenStates(data["hiddenStates"], data["seqLens"], data["lastTokensStates"])
            self.RMSNorm(data["lastTokensStates"], weight["model.norm.weight"], config["rms_norm_eps"], data["lastTokensStates"])
            self.Linear(data["lastTokensStates"], weight["lm_head.weight"], None, data["logits"])

    __model__ = TinyLlama
''')


def test_custom_graph_model_matches_builtin(tmp_path):
    from baseline import synth

    d = synth.write_model("tiny-llama", str(tmp_path / "m"), dtype=torch.float32, std=0.05)
    f = tmp_path / "tiny_llama_graph.py"
    f.write_text(MODEL_FILE)
    cls = load_custom_file(str(f))
    assert issubclass(cls, ComputeGraph)
    gm = load_graph_model(d, cls, device="cpu", dtype=torch.float32)
    ref = hf.load_model(d, device="cpu", dtype=torch.float32)
    prompts = [list(range(3, 70, 2)), list(range(9, 20))]
    outs = []
    for m in (ref, gm):
        eng = LLMEngine(m, EngineConfig(max_batch=4, max_context=512), num_pages=16)
        outs.append(eng.generate(prompts, GenerationConfig(max_new_tokens=6, ignore_eos=True)))
    assert outs[0] == outs[1]
    g = cls(json.loads((tmp_path / "m" / "config.json").read_text()))
    g.build()
    js = json.loads(g.to_json())
    assert js["graph"][0]["type"] == "Embedding" and js["graph"][0]["nodes"]["weight"] == "weight:model.embed_tokens.weight"
    assert any(op["type"] == "FusedAttention" and abs(op["floatParams"]["scale"] - 1 / math.sqrt(128)) < 1e-9 for op in js["graph"])
