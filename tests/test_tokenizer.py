"""Native byte-level BPE vs the Hugging Face `tokenizers` implementation, chat template rendering, streaming decode."""
import pytest

from fastllm_b200.chat_template import render
from fastllm_b200.tokenizer import NativeBPE, StreamDecoder, Tokenizer

CORPUS = ["Hello world, this is a test of the tokenizer. It's working!",
          "The quick brown fox jumps over 12345 lazy dogs.\n\nNew paragraph here.",
          "def foo(x):\n    return x + 1  # comment", "多语言 テスト 한국어 émoji 🙂 mixed text"]


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    tk = pytest.importorskip("tokenizers")
    from tokenizers import decoders, models, pre_tokenizers, trainers

    tok = tk.Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    tok.decoder = decoders.ByteLevel()
    tr = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(CORPUS * 50, tr)
    p = tmp_path_factory.mktemp("tok") / "tokenizer.json"
    tok.save(str(p))
    return tok, p


def test_native_bpe_matches_hf(trained):
    tok, p = trained
    nb = NativeBPE(p)
    for s in CORPUS + ["It's 2024!  Two  spaces", "a<|endoftext|>b", " leading space", "tabs\tand\nnewlines\n", ""]:
        assert nb.encode(s) == tok.encode(s).ids, s
        assert nb.decode(nb.encode(s), skip_special_tokens=False) == s


def test_stream_decoder_holds_back_partial_utf8(trained):
    _, p = trained
    t = Tokenizer(None)
    t.native = NativeBPE(p)
    ids = t.native.encode("héllo 🙂 wörld")
    sd = StreamDecoder(t)
    out = "".join(sd.push(i) for i in ids)
    assert out == "héllo 🙂 wörld"


def test_chat_template_render():
    tpl = "{% for m in messages %}<|{{ m['role'] }}|>{{ m['content'] }}</s>{% endfor %}{% if add_generation_prompt %}<|assistant|>{% endif %}"
    s = render(tpl, [{"role": "user", "content": "hi"}], add_generation_prompt=True)
    assert s == "<|user|>hi</s><|assistant|>"
    assert "<|im_start|>user" in render(None, [{"role": "user", "content": "hi"}])


def test_native_unigram_matches_hf_tokenizers(tmp_path):
    """The C++ Unigram core against the Hugging Face ``tokenizers`` implementation on the same model file."""
    import json

    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer as HFTok, decoders, models, pre_tokenizers

    from fastllm_b200.tokenizer import NativeUnigram, native_tokenizer

    pieces = [("<unk>", 0.0), ("<s>", 0.0)] + [(f"<0x{b:02X}>", -20.0) for b in range(256)]
    words = ["▁the", "▁", "the", "▁hello", "hello", "he", "llo", "▁world", "wor", "ld", "world", "▁a", "an", "b", "c", "d", "e",
             "h", "l", "o", "r", "t", "w", "a", "n", "▁to", "ken", "iz", "er", "▁tokenizer", "s", "é", "▁caf"]
    for i, w in enumerate(words):
        pieces.append((w, -1.0 - 0.37 * (i % 7) - 0.01 * len(w)))
    tok = HFTok(models.Unigram(pieces, unk_id=0, byte_fallback=True))
    tok.pre_tokenizer = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme="always")
    tok.decoder = decoders.Sequence([decoders.Metaspace(replacement="▁", prepend_scheme="always"), decoders.ByteFallback(), decoders.Fuse()])
    path = tmp_path / "tokenizer.json"
    tok.save(str(path))
    nat = native_tokenizer(path)
    assert isinstance(nat, NativeUnigram) and nat.vocab_size == len(pieces)
    for text in ["hello world", "the tokenizers are here", "a b c", "café 中 hello", "hello  world", "x"]:
        want = tok.encode(text, add_special_tokens=False).ids
        got = nat.encode(text)
        assert got == want, (text, got, want)
        assert nat.decode(got) == tok.decode(want), text
