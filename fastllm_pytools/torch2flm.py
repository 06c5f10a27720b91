"""`torch2flm.tofile(path, model, tokenizer, dtype=...)`: write an in-memory Hugging Face model as a `.flm` file
(reference: tools/fastllm_pytools/torch2flm.py:tofile).  The model and tokenizer are saved to a temporary folder in the
Hugging Face layout and exported from there by the `.flm` writer of `fastllm_b200.loader.flm`."""
import tempfile


def tofile(exportPath, model, tokenizer=None, pre_prompt=None, user_role=None, bot_role=None, history_sep=None, eos_id=None,
           dtype="float16", **_ignored):
    from fastllm_b200.loader import flm

    with tempfile.TemporaryDirectory(prefix="torch2flm_") as d:
        model.save_pretrained(d, safe_serialization=True)
        if tokenizer is not None:
            tokenizer.save_pretrained(d)
        flm.export_hf_to_flm(d, exportPath, dtype)
