"""BERT / XLM-RoBERTa encoders for ``/v1/embed`` and ``/v1/rerank`` (reference: src/models/bert.cpp,
src/models/xlmroberta.cpp).  Post-LayerNorm encoder, CLS pooling + L2 normalisation for embeddings, classification
head for rerank scores.  Runs as plain PyTorch ops on the model's device (not a decode hot path)."""
from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.nn.functional as F

from ..loader import safetensors as st


class BertModel:
    def __init__(self, path: str, device="cpu", dtype=torch.float32):
        p = Path(path)
        self.cfg = json.loads((p / "config.json").read_text())
        self.device, self.dtype = torch.device(device), dtype
        files, where = st.open_model_dir(p)
        self.w = {}
        for k, fi in where.items():
            name = k
            for pre in ("bert.", "roberta.", "model."):
                if name.startswith(pre):
                    name = name[len(pre):]
            self.w[name] = files[fi].get(k).to(self.device, dtype)
        for f in files:
            f.close()
        self.heads = self.cfg["num_attention_heads"]
        self.layers = self.cfg["num_hidden_layers"]
        self.eps = self.cfg.get("layer_norm_eps", 1e-12)
        self.is_roberta = self.cfg.get("model_type", "bert") in ("xlm-roberta", "roberta")
        self.pad_id = self.cfg.get("pad_token_id", 1 if self.is_roberta else 0)

    def _ln(self, x, prefix):
        return F.layer_norm(x, (x.shape[-1],), self.w[prefix + ".weight"], self.w[prefix + ".bias"], self.eps)

    def _lin(self, x, prefix):
        return F.linear(x, self.w[prefix + ".weight"], self.w.get(prefix + ".bias"))

    @torch.no_grad()
    def hidden(self, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """ids, mask: [B, T] -> last hidden state [B, T, H]"""
        B, T = ids.shape
        if self.is_roberta:
            pos = (torch.cumsum(mask, 1) * mask + self.pad_id).long()
        else:
            pos = torch.arange(T, device=ids.device)[None].expand(B, T)
        e = self.w["embeddings.word_embeddings.weight"][ids] + self.w["embeddings.position_embeddings.weight"][pos]
        if "embeddings.token_type_embeddings.weight" in self.w:
            e = e + self.w["embeddings.token_type_embeddings.weight"][torch.zeros_like(ids)]
        x = self._ln(e, "embeddings.LayerNorm")
        bias = (1.0 - mask[:, None, None, :].to(x.dtype)) * torch.finfo(x.dtype).min
        H = self.heads
        for i in range(self.layers):
            p = f"encoder.layer.{i}."
            q = self._lin(x, p + "attention.self.query").view(B, T, H, -1).transpose(1, 2)
            k = self._lin(x, p + "attention.self.key").view(B, T, H, -1).transpose(1, 2)
            v = self._lin(x, p + "attention.self.value").view(B, T, H, -1).transpose(1, 2)
            a = torch.softmax(q @ k.transpose(-1, -2) / (q.shape[-1] ** 0.5) + bias, dim=-1) @ v
            a = a.transpose(1, 2).reshape(B, T, -1)
            x = self._ln(self._lin(a, p + "attention.output.dense") + x, p + "attention.output.LayerNorm")
            h = F.gelu(self._lin(x, p + "intermediate.dense"))
            x = self._ln(self._lin(h, p + "output.dense") + x, p + "output.LayerNorm")
        return x

    def embed(self, ids, mask, normalize=True):
        cls = self.hidden(ids, mask)[:, 0]
        return F.normalize(cls, dim=-1) if normalize else cls

    def classify(self, ids, mask):
        x = self.hidden(ids, mask)
        if "classifier.dense.weight" in self.w:         # roberta head
            h = torch.tanh(self._lin(x[:, 0], "classifier.dense"))
            return self._lin(h, "classifier.out_proj").squeeze(-1)
        pooled = torch.tanh(self._lin(x[:, 0], "pooler.dense")) if "pooler.dense.weight" in self.w else x[:, 0]
        return self._lin(pooled, "classifier").squeeze(-1)
