"""Tokenizers of the decode path's callers: the reference's own known-answer fixtures
(Tests/ModelSupportTests/TokenizerTests.swift) restated, plus a cross-check of the byte-level BPE against the
HuggingFace `tokenizers` implementation on a vocabulary trained here."""
import json
import struct

import pytest

from espresso_b200 import tokenizers as tk

B2U = tk.byte_to_unicode()
NEWLINE, SPACE = B2U[10], B2U[32]
VOCAB = {"Hello": 0, ",": 1, f"{SPACE}world": 2, "!": 3, NEWLINE: 4}
MERGES = ["H e", "He l", "Hel l", "Hell o", f"{SPACE} w", f"{SPACE}w o", f"{SPACE}wo r", f"{SPACE}wor l", f"{SPACE}worl d"]


def gpt2_fixture(tmp_path):
    (tmp_path / "vocab.json").write_text(json.dumps(VOCAB, sort_keys=True), encoding="utf-8")
    (tmp_path / "merges.txt").write_text("\n".join(["#version: 0.2"] + MERGES), encoding="utf-8")
    return str(tmp_path / "vocab.json"), str(tmp_path / "merges.txt")


def tokenizer_json_fixture(tmp_path):
    payload = {
        "added_tokens": [{"id": 5, "content": "<|begin_of_text|>", "special": True, "single_word": False, "lstrip": False,
                          "rstrip": False, "normalized": False}],
        "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
            {"type": "Split", "pattern": {"Regex": tk.DEFAULT_PRETOKENIZER}, "behavior": "Isolated", "invert": False}]},
        "post_processor": {"type": "Sequence", "processors": [{"type": "TemplateProcessing", "single": [
            {"SpecialToken": {"id": "<|begin_of_text|>", "ids": [5], "tokens": ["<|begin_of_text|>"]}},
            {"Sequence": {"id": "A", "type_id": 0}}]}]},
        "model": {"type": "BPE", "vocab": VOCAB, "merges": MERGES},
    }
    p = tmp_path / "tokenizer.json"
    p.write_text(json.dumps(payload, sort_keys=True), encoding="utf-8")
    return str(p)


def sentencepiece_fixture(tmp_path):
    pieces = [("▁", 0.0), ("H", 0.0), ("e", 0.0), ("l", 0.0), ("o", 0.0), (",", 0.0), ("w", 0.0), ("r", 0.0), ("d", 0.0), ("!", 0.0),
              ("▁H", 1.0), ("▁He", 2.0), ("▁Hel", 3.0), ("▁Hell", 4.0), ("▁Hello", 5.0), ("▁w", 1.0), ("▁wo", 2.0), ("▁wor", 3.0),
              ("▁worl", 4.0), ("▁world", 5.0), ("<0x0A>", 0.0)]
    blob = struct.pack("<i", 16)
    for piece, score in pieces:
        raw = piece.encode("utf-8")
        blob += struct.pack("<fi", score, len(raw)) + raw
    p = tmp_path / "tokenizer.model"
    p.write_bytes(blob)
    return str(p)


def test_gpt2_round_trips_hello_world_and_non_printable_bytes(tmp_path):
    t = tk.GPT2BPETokenizer.from_vocab_and_merges(*gpt2_fixture(tmp_path))
    enc = t.encode("Hello, world!")
    assert enc == [0, 1, 2, 3] and t.decode(enc) == "Hello, world!"
    assert t.encode("\n") == [4] and t.decode([4]) == "\n"
    assert t.vocab_size == 5


def test_tokenizer_json_round_trips_and_skips_special_tokens(tmp_path):
    t = tk.GPT2BPETokenizer.from_tokenizer_json(tokenizer_json_fixture(tmp_path))
    enc = t.encode("Hello, world!")
    assert enc == [5, 0, 1, 2, 3] and t.decode(enc) == "Hello, world!"
    assert t.encode("\n") == [5, 4] and t.decode([5, 4]) == "\n"


def test_sentencepiece_round_trips_hello_world_and_byte_fallback(tmp_path):
    t = tk.SentencePieceTokenizer(sentencepiece_fixture(tmp_path))
    enc = t.encode("Hello, world!")
    assert enc == [14, 5, 19, 9]  # ▁Hello , ▁world !
    assert t.decode(enc) == "Hello, world!"
    nl = t.encode("\n")
    assert nl == [0, 20] and t.decode(nl) == "\n"


def test_error_kinds(tmp_path):
    (tmp_path / "vocab.json").write_text('["not","a","map"]')
    (tmp_path / "merges.txt").write_text("#version: 0.2\n")
    with pytest.raises(tk.TokenizerError) as e:
        tk.GPT2BPETokenizer.from_vocab_and_merges(str(tmp_path / "vocab.json"), str(tmp_path / "merges.txt"))
    assert e.value.kind == "malformedVocabulary"
    (tmp_path / "vocab.json").write_text(json.dumps({"a": 0, "b": 2}))
    with pytest.raises(tk.TokenizerError) as e:
        tk.GPT2BPETokenizer.from_vocab_and_merges(str(tmp_path / "vocab.json"), str(tmp_path / "merges.txt"))
    assert e.value.kind == "nonContiguousTokenIDs" and "expectedCount=2 actualMaxTokenID=2" in e.value.detail
    (tmp_path / "tokenizer.json").write_text(json.dumps({"model": {"type": "WordPiece", "vocab": {"a": 0}, "merges": []}}))
    with pytest.raises(tk.TokenizerError) as e:
        tk.GPT2BPETokenizer.from_tokenizer_json(str(tmp_path / "tokenizer.json"))
    assert e.value.kind == "unsupportedTokenizerModel" and e.value.detail == "WordPiece"
    (tmp_path / "tokenizer.model").write_bytes(bytes([1, 2]))
    with pytest.raises(tk.TokenizerError) as e:
        tk.SentencePieceTokenizer(str(tmp_path / "tokenizer.model"))
    assert e.value.kind == "truncatedModel"
    (tmp_path / "tokenizer.model").write_bytes(struct.pack("<ifi", 8, 0.0, 4) + b"ab")
    with pytest.raises(tk.TokenizerError) as e:
        tk.SentencePieceTokenizer(str(tmp_path / "tokenizer.model"))
    assert e.value.kind == "truncatedEntry" and e.value.detail == "index=0"


def test_file_search_order(tmp_path):
    with pytest.raises(FileNotFoundError):
        tk.load_tokenizer("llama", str(tmp_path))
    gpt2_fixture(tmp_path)
    assert isinstance(tk.load_tokenizer("llama", str(tmp_path)), tk.GPT2BPETokenizer)  # Qwen-style fallback
    assert isinstance(tk.load_tokenizer("gpt2", str(tmp_path)), tk.GPT2BPETokenizer)
    tokenizer_json_fixture(tmp_path)
    assert tk.load_tokenizer("llama", str(tmp_path)).prefix_token_ids == [5]
    sentencepiece_fixture(tmp_path)
    assert isinstance(tk.load_tokenizer("llama", str(tmp_path)), tk.SentencePieceTokenizer)


def test_byte_level_bpe_matches_huggingface_tokenizers(tmp_path):
    hf = pytest.importorskip("tokenizers")
    import random

    rnd = random.Random(5)
    words = ["decode", "token", "cache", "layer", "head", "norm", "über", "naïve", "日本語", "42", "3.14", "don't", "we'll", "α+β"]
    corpus = [" ".join(rnd.choice(words) for _ in range(rnd.randint(3, 12))) + rnd.choice([".", "!", "\n", "  ", "?"]) for _ in range(400)]
    tok = hf.Tokenizer(hf.models.BPE())
    # the reference's pattern (no "\\s+(?!\\S)" alternative) as an explicit Split, so both sides cut the text alike
    tok.pre_tokenizer = hf.pre_tokenizers.Sequence([
        hf.pre_tokenizers.Split(hf.Regex(tk.DEFAULT_PRETOKENIZER), behavior="isolated"),
        hf.pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = hf.decoders.ByteLevel()
    tok.train_from_iterator(corpus, hf.trainers.BpeTrainer(vocab_size=400, initial_alphabet=hf.pre_tokenizers.ByteLevel.alphabet(), show_progress=False))
    path = str(tmp_path / "tokenizer.json")
    tok.save(path)
    mine = tk.GPT2BPETokenizer.from_tokenizer_json(path)
    assert mine.vocab_size == tok.get_vocab_size()
    probes = corpus[:60] + ["Hello, world!", "  leading and trailing  ", "tabs\tand\nnewlines\r\n", "emoji 🙂 and 日本語 mixed 123abc", ""]
    for text in probes:
        want = tok.encode(text).ids
        assert mine.encode(text) == want, text
        assert mine.decode(want) == tok.decode(want), text


@pytest.mark.gpu
def test_generate_text_round_trip(tmp_path, tmp_models):
    """Text in, text out through the engine: ids from the tokenizer, greedy decode, ids back to text."""
    from espresso_b200 import runtime as rt
    from espresso_b200.model_config import tiny_llama

    t = tk.GPT2BPETokenizer.from_tokenizer_json(tokenizer_json_fixture(tmp_path))
    cfg = tiny_llama(vocab=t.vocab_size, max_seq=32, n_layer=1)
    eng = rt.DecodeEngine.build(tmp_models(cfg))
    text, res = eng.generate_text(t, "Hello, world!", 8)
    assert len(res.tokens) == 8 and text == t.decode([int(x) for x in res.tokens])
    assert list(res.tokens) == list(eng.generate(t.encode("Hello, world!"), 8).tokens)
    empty = tk.GPT2BPETokenizer({"a": 0}, [])
    with pytest.raises(rt.RealModelInferenceError):
        eng.generate_text(empty, "zzz", 4)  # nothing of the prompt is in the vocabulary: invalidPrompt
    eng.close()
