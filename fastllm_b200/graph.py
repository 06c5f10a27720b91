"""ComputeGraph: describe a model that the framework has no built-in class for as a list of operators, in Python.

A custom model file subclasses ``ComputeGraph``, implements ``build()`` with the operator methods below and ends with
``__model__ = MyModel``; ``llm.model(path, graph=MyModel)`` (or ``--custom file.py`` on the command line) then runs it through
the same paged-KV engine as the built-in models.  The recorded graph is a JSON-serialisable list of
``{"type", "nodes": {...}, "floatParams", "intParams"}`` entries.

Reference: include/graph.h, src/graph.cpp (RunComputeGraph), Python DSL tools/fastllm_pytools/llm.py:2825-2932,
docs/custom.md, example/python/qwen2.py.  Inputs available in ``data``: inputIds, positionIds, attentionMask, sin, cos, atype,
seqLens, pastKey.[i], pastValue.[i].
"""
from __future__ import annotations

import json
import math

import torch

from .models.config import ModelConfig, from_hf_dict
from .models.decoder import DecoderModel, ForwardBatch, TPInfo
from .ops import attention as A
from .ops import basic as B


class _Sym:
    """A named graph value.  ``sym["suffix"]`` / ``sym[i]`` extend the name, so ``weight["model.layers."][3][".x"]`` works."""

    def __init__(self, kind: str, name: str = ""):
        self.kind, self.name = kind, name

    def __getitem__(self, key):
        return _Sym(self.kind, self.name + str(key))

    def __repr__(self):
        return f"{self.kind}:{self.name}"


class ComputeGraph:
    def __init__(self, config: dict | None = None):
        self.weight = _Sym("weight")
        self.data = _Sym("data")
        self.config = dict(config or {})
        self.graph: list[dict] = []

    # ---- recording ------------------------------------------------------------------------------
    def _op(self, type_: str, nodes: dict, floats: dict | None = None, ints: dict | None = None):
        self.graph.append({"type": type_, "nodes": {k: repr(v) for k, v in nodes.items() if v is not None},
                           "floatParams": dict(floats or {}), "intParams": dict(ints or {})})

    def build(self):          # pragma: no cover - implemented by the model file
        raise NotImplementedError

    def to_json(self) -> str:
        return json.dumps({"config": self.config, "graph": self.graph})

    # ---- operators (names and argument order of the reference DSL) ---------------------------------
    def Print(self, input):
        self._op("Print", {"input": input})

    def Exit(self):
        self._op("Exit", {})

    def AddTo(self, input0, input1, alpha=1.0):
        self._op("AddTo", {"input0": input0, "input1": input1}, {"alpha": float(alpha)})

    def MulTo(self, input0, input1):
        self._op("MulTo", {"input0": input0, "input1": input1})

    def DataTypeAs(self, input, input1):
        self._op("DataTypeAs", {"input": input, "input1": input1})

    def Embedding(self, input, weight, output):
        self._op("Embedding", {"input": input, "weight": weight, "output": output})

    def ExpandHead(self, input, headDim):
        self._op("ExpandHeads", {"input": input}, ints={"headDim": int(headDim)})

    def FusedAttention(self, q, k, v, curk, curv, original, mask, output, seqLens, scale, maskType=0, unitLen=128):
        self._op("FusedAttention", {"q": q, "k": k, "v": v, "curk": curk, "curv": curv, "original": original, "mask": mask,
                                    "output": output, "seqLens": seqLens}, {"scale": float(scale)},
                 {"maskType": int(maskType), "unitLen": int(unitLen)})

    def Linear(self, input, weight, bias, output):
        self._op("Linear", {"input": input, "weight": weight, "bias": bias, "output": output})

    def LlamaRotatePosition2D(self, input, positionIds, sin, cos, rotaryDim):
        self._op("LlamaRotatePosition2D", {"input": input, "positionIds": positionIds, "sin": sin, "cos": cos},
                 ints={"rotaryDim": int(rotaryDim)})

    def RMSNorm(self, input, weight, eps, output):
        self._op("RMSNorm", {"input": input, "weight": weight, "output": output}, {"eps": float(eps)})

    def LayerNorm(self, input, gamma, beta, output, eps=1e-5):
        self._op("LayerNorm", {"input": input, "gamma": gamma, "beta": beta, "output": output}, {"eps": float(eps)})

    def Silu(self, input, output):
        self._op("Silu", {"input": input, "output": output})

    def Gelu(self, input, output):
        self._op("Gelu", {"input": input, "output": output})

    def Swiglu(self, input, output):
        self._op("Swiglu", {"input": input, "output": output})

    def Split(self, input, axis, start, end, output):
        self._op("Split", {"input": input, "output": output}, ints={"axis": int(axis), "start": int(start), "end": int(end)})

    def Cat(self, input0, input1, axis, output):
        self._op("Cat", {"input0": input0, "input1": input1, "output": output}, ints={"axis": int(axis)})

    def SplitLastTokenStates(self, input, seqLens, output):
        self._op("SplitLastTokenStates", {"input": input, "seqLens": seqLens, "output": output})


class GraphModel(DecoderModel):
    """Executes a recorded ComputeGraph on the paged-KV engine (one tensor-parallel rank only)."""

    def __init__(self, graph: ComputeGraph, weights: dict, device, dtype=torch.bfloat16):
        c = graph.config
        cfg = from_hf_dict(dict(c))
        if "max_positions" in c:
            cfg.max_position = int(c["max_positions"])
        super().__init__(cfg, device, dtype, TPInfo())
        self.ops = graph.graph
        self.weights = {k: (v.to(self.device, dtype) if v.is_floating_point() else v.to(self.device)) for k, v in weights.items()}
        self.general_attn = True          # interpreted op by op: decode stays out of CUDA graphs
        self.head_dims: dict = {}

    def _get(self, env, ref):
        if ref is None:
            return None
        kind, name = ref.split(":", 1)
        return self.weights.get(name) if kind == "weight" else env.get(name)

    @torch.no_grad()
    def forward(self, fb: ForwardBatch, kv_caches) -> torch.Tensor:
        cos, sin = self.rope_tables()
        env = {"inputIds": fb.ids, "positionIds": fb.positions, "sin": sin, "cos": cos, "atype": self.dtype, "seqLens": fb.kv_lens,
               "attentionMask": None}
        for i, (k, v) in enumerate(kv_caches):
            env[f"pastKey.{i}"], env[f"pastValue.{i}"] = k, v
        hd = {}
        for op in self.ops:
            t, n, fp, ip = op["type"], op["nodes"], op["floatParams"], op["intParams"]
            g = lambda key: self._get(env, n.get(key))
            out = n.get("output", "data:").split(":", 1)[1]
            if t == "Embedding":
                env[out] = B.embedding(g("input"), g("weight"))
            elif t == "DataTypeAs":
                name = n["input"].split(":", 1)[1]
                env[name] = env[name].to(self.dtype)
            elif t == "RMSNorm":
                env[out] = B.rmsnorm(g("input"), g("weight"), fp["eps"])
            elif t == "LayerNorm":
                x = g("input")
                env[out] = torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), g("gamma").float(), g("beta").float(), fp["eps"]).to(x.dtype)
            elif t == "Linear":
                env[out] = B.linear(g("input"), g("weight"), g("bias"))
            elif t == "ExpandHeads":
                hd[n["input"].split(":", 1)[1]] = ip["headDim"]
            elif t == "LlamaRotatePosition2D":
                name = n["input"].split(":", 1)[1]
                x, D = env[name], hd[name]
                T = x.shape[0]
                env[name] = A.apply_rope_ref(x.reshape(T, -1, D), g("positionIds"), g("cos"), g("sin"), A.ROPE_NEOX,
                                             2 * ip["rotaryDim"]).reshape(T, -1)
            elif t == "FusedAttention":
                q, ck, cv = g("q"), g("curk"), g("curv")
                k_pool, v_pool = g("k"), g("v")
                D = hd[n["q"].split(":", 1)[1]]
                Hq, Hkv = q.shape[1] // D, ck.shape[1] // D
                valid = fb.slots >= 0
                sl = fb.slots[valid].long()
                k_pool.view(-1, Hkv, D)[sl] = ck.reshape(-1, Hkv, D)[valid].to(k_pool.dtype)
                v_pool.view(-1, Hkv, D)[sl] = cv.reshape(-1, Hkv, D)[valid].to(v_pool.dtype)
                if fb.is_decode:
                    o = A.attn_decode(q.contiguous(), k_pool, v_pool, fb.page_table, fb.kv_lens, fp["scale"], Hq, Hkv, D)
                else:
                    o = A.attn_prefill(q.contiguous(), k_pool, v_pool, fb.page_table, fb.kv_lens, fb.cu_q, fp["scale"], Hq, Hkv, D,
                                       cu_q_host=fb.cu_q_host)
                env[out] = o
            elif t == "AddTo":
                name = n["input0"].split(":", 1)[1]
                env[name] = env[name] + g("input1") * fp.get("alpha", 1.0) if fp.get("alpha", 1.0) != 1.0 else env[name] + g("input1")
            elif t == "MulTo":
                name = n["input0"].split(":", 1)[1]
                env[name] = env[name] * g("input1")
            elif t == "Silu":
                env[out] = torch.nn.functional.silu(g("input").float()).to(g("input").dtype)
            elif t == "Gelu":
                env[out] = torch.nn.functional.gelu(g("input").float()).to(g("input").dtype)
            elif t == "Swiglu":
                env[out] = B.silu_mul(g("input"))
            elif t == "Split":
                env[out] = g("input").narrow(ip["axis"], ip["start"], ip["end"] - ip["start"])
            elif t == "Cat":
                env[out] = torch.cat([g("input0"), g("input1")], dim=ip["axis"])
            elif t == "SplitLastTokenStates":
                x = g("input")
                env[out] = x.index_select(0, fb.logit_rows) if fb.logit_rows is not None else x
            elif t == "Print":
                print(n.get("input"), g("input"))
            elif t == "Exit":
                break
            else:
                raise ValueError(f"ComputeGraph operator '{t}' is not supported")
        return env["logits"].float()

    def kv_cache_shape(self, num_pages: int):
        c = self.cfg
        s = (num_pages, A.PAGE_LEN, c.num_kv_heads, c.head_dim)
        return s, s


def load_graph_model(path: str, graph_cls, device="cuda", dtype=None) -> GraphModel:
    """Build ``graph_cls`` against the checkpoint folder ``path`` (weights are addressed by their names in the checkpoint)."""
    from pathlib import Path

    from .loader.safetensors import open_model_dir

    cfg = json.loads((Path(path) / "config.json").read_text())
    g = graph_cls(cfg)
    g.build()
    files, _where = open_model_dir(path)
    weights = {}
    for f in files:
        for k in f.keys():
            weights[k] = f.get(k).clone()
        f.close()
    if cfg.get("tie_word_embeddings") and "lm_head.weight" not in weights and "model.embed_tokens.weight" in weights:
        weights["lm_head.weight"] = weights["model.embed_tokens.weight"]
    if dtype is None:
        dtype = torch.float32 if str(device) == "cpu" else torch.bfloat16
    return GraphModel(g, weights, device, dtype)


def load_custom_file(py_file: str):
    """Import a custom model file and return its ``__model__`` class."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("fastllm_custom_model", py_file)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.__model__
