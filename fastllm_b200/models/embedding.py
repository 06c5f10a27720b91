"""Sentence embeddings and rerank scores behind ``/v1/embed`` and ``/v1/rerank`` (reference C ABI:
``embedding_sentence`` / ``reranker_compute_score``, tools/src/pytools.cpp:1076-1099)."""
from __future__ import annotations

import torch


def _batch(tok, texts, pairs=None, device="cpu", pad_id=0, max_len=512):
    if tok.hf is not None:
        enc = tok.hf(texts, pairs, padding=True, truncation=True, max_length=max_len, return_tensors="pt") if pairs else \
            tok.hf(texts, padding=True, truncation=True, max_length=max_len, return_tensors="pt")
        return enc["input_ids"].to(device), enc["attention_mask"].to(device)
    rows = [tok.encode(t)[:max_len] for t in texts]
    T = max(len(r) for r in rows)
    ids = torch.full((len(rows), T), pad_id, dtype=torch.long)
    mask = torch.zeros((len(rows), T), dtype=torch.long)
    for i, r in enumerate(rows):
        ids[i, :len(r)] = torch.tensor(r)
        mask[i, :len(r)] = 1
    return ids.to(device), mask.to(device)


def embed_texts(model, texts, normalize=True):
    enc = getattr(model, "encoder", None)
    if enc is not None:
        ids, mask = _batch(model.tokenizer, list(texts), device=enc.device, pad_id=enc.pad_id)
        return enc.embed(ids, mask, normalize).float().cpu().tolist()
    # decoder-only model: mean of the final-norm hidden state is not exposed; use last-token logits-free fallback
    raise ValueError("the loaded model is not an embedding model (load a bert / xlm-roberta folder)")


def rerank_scores(model, query, texts):
    enc = getattr(model, "encoder", None)
    if enc is None:
        raise ValueError("the loaded model is not a reranker (load a bert / xlm-roberta sequence-classification folder)")
    ids, mask = _batch(model.tokenizer, [query] * len(texts), list(texts), device=enc.device, pad_id=enc.pad_id)
    return enc.classify(ids, mask).float().cpu().tolist()


class EncoderModel:
    """``llm.model``-like wrapper for encoder folders."""

    def __init__(self, path, device=None):
        from ..tokenizer import Tokenizer
        from .bert import BertModel

        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.encoder = BertModel(path, dev, torch.float32 if dev == "cpu" else torch.float16)
        self.tokenizer = Tokenizer(path)
        self.tool_call_parser = "auto"

    def embedding_sentence(self, text, normalize=True):
        return embed_texts(self, [text], normalize)[0]

    def reranker_compute_score(self, pairs):
        return [rerank_scores(self, q, [t])[0] for q, t in pairs]

    def get_type(self):
        return self.encoder.cfg.get("model_type", "bert")

    def warmup(self):
        pass
