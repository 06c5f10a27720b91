"""`hf_model.create(model, tokenizer, dtype=...)`: a served model from an in-memory Hugging Face model
(reference: tools/fastllm_pytools/hf_model.py:create)."""
from fastllm_b200 import llm


def create(model, tokenizer, pre_prompt=None, user_role=None, bot_role=None, history_sep=None, dtype="float16", **_ignored):
    """The prompt-format arguments of the reference's signature are accepted and unused: the chat template of the tokenizer
    decides the prompt format here."""
    return llm.from_hf(model, tokenizer, dtype=dtype)
