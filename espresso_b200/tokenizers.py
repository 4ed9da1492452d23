"""Text <-> token ids for the decode path's callers: byte-level BPE (GPT-2 ``vocab.json`` + ``merges.txt`` or a
HuggingFace ``tokenizer.json``) and the llama2.c ``tokenizer.bin`` SentencePiece layout.

Behaviour follows the reference's host-side tokenizers:

* ``GPT2BPETokenizer`` (Sources/ModelSupport/GPT2BPETokenizer.swift:13-110, 166-230): pre-tokeniser regex, bytes mapped
  to printable code points, lowest-rank pair merged first (every occurrence, left to right), pieces missing from the
  vocabulary dropped; ``tokenizer.json``: ``added_tokens`` extend the vocabulary (special ones are skipped when
  decoding), the pre-tokeniser regex and the BOS prefix come from the file (:46-75, 278-374).
* ``SentencePieceTokenizer`` (Sources/ModelSupport/SentencePieceTokenizer.swift:19-150): i32 max_token_length, then
  per piece f32 score, i32 byte length, UTF-8 bytes; "▁" + text with spaces replaced by "▁", one piece per character
  with ``<0xNN>`` byte fallback, then repeatedly the best-scoring adjacent pair (first of equals) is merged.
* ``load_tokenizer`` picks the files in the reference's order (RealModelInferenceEngine.swift:7558-7613).

Host-side only; nothing here touches the GPU.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Iterable, Optional, Protocol

import regex  # \p{L} / \p{N} classes of the pre-tokeniser pattern

DEFAULT_PRETOKENIZER = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+"
BOS_NAME = "<|begin_of_text|>"


class TokenizerError(ValueError):
    """Carries the reference's error case name in ``kind`` (``malformedVocabulary``, ``truncatedEntry`` ...)."""

    def __init__(self, kind: str, detail: str = ""):
        super().__init__(f"{kind}{': ' + detail if detail else ''}")
        self.kind = kind
        self.detail = detail


class Tokenizer(Protocol):
    vocab_size: int

    def encode(self, text: str) -> list[int]: ...

    def decode(self, tokens: Iterable[int]) -> str: ...


def byte_to_unicode() -> list[str]:
    """GPT-2's byte -> printable code point table: printable Latin-1 bytes map to themselves, the rest to 256.."""
    direct = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table = [""] * 256
    for b in direct:
        table[b] = chr(b)
    nxt = 256
    for b in range(256):
        if not table[b]:
            table[b] = chr(nxt)
            nxt += 1
    return table


class GPT2BPETokenizer:
    def __init__(self, encoder: dict[str, int], merges: list[str], pattern: str = DEFAULT_PRETOKENIZER,
                 prefix_token_ids: Optional[list[int]] = None, skipped_token_ids: Optional[set[int]] = None):
        if not encoder:
            raise TokenizerError("emptyVocabulary")
        top = max(encoder.values())
        if top < 0:
            raise TokenizerError("emptyVocabulary")
        if top + 1 != len(encoder):
            raise TokenizerError("nonContiguousTokenIDs", f"expectedCount={len(encoder)} actualMaxTokenID={top}")
        self.encoder = encoder
        self.decoder = [""] * (top + 1)
        for piece, i in encoder.items():
            if 0 <= i <= top:
                self.decoder[i] = piece
        self.vocab_size = len(self.decoder)
        self.prefix_token_ids = list(prefix_token_ids or [])
        self.skipped_token_ids = set(skipped_token_ids or ())
        self.ranks: dict[tuple[str, str], int] = {}
        for line in merges:
            if not line or line.startswith("#"):
                continue
            parts = line.split()
            if len(parts) != 2:
                continue
            self.ranks[(parts[0], parts[1])] = len(self.ranks)
        self._b2u = byte_to_unicode()
        self._u2b = {u: b for b, u in enumerate(self._b2u)}
        try:
            self._pre = regex.compile(pattern)
        except regex.error as e:
            raise TokenizerError("invalidPreTokenizerPattern", pattern) from e
        self._cache: dict[str, list[str]] = {}

    # ---- construction from files -------------------------------------------------------------------------
    @classmethod
    def from_vocab_and_merges(cls, vocab_path: str, merges_path: str) -> "GPT2BPETokenizer":
        with open(vocab_path, "r", encoding="utf-8") as f:
            raw = json.load(f)
        with open(merges_path, "r", encoding="utf-8") as f:
            merges = f.read().split("\n")
        return cls(_parse_vocabulary(raw), merges)

    @classmethod
    def from_tokenizer_json(cls, path: str) -> "GPT2BPETokenizer":
        with open(path, "r", encoding="utf-8") as f:
            root = json.load(f)
        model = root.get("model") if isinstance(root, dict) else None
        if not isinstance(model, dict):
            raise TokenizerError("malformedTokenizerJSON")
        kind = model.get("type", "unknown")
        if kind != "BPE":
            raise TokenizerError("unsupportedTokenizerModel", str(kind))
        if not isinstance(model.get("vocab"), dict):
            raise TokenizerError("malformedTokenizerJSON")
        encoder = _parse_vocabulary(model["vocab"])
        skipped = set()
        for tok in root.get("added_tokens") or []:
            if isinstance(tok, dict) and isinstance(tok.get("id"), int) and isinstance(tok.get("content"), str):
                encoder[tok["content"]] = tok["id"]
                if tok.get("special") is True:
                    skipped.add(tok["id"])
        raw_merges = model.get("merges")
        if raw_merges is None:
            raise TokenizerError("malformedTokenizerJSON")
        if all(isinstance(m, str) for m in raw_merges):
            merges = list(raw_merges)
        elif all(isinstance(m, list) for m in raw_merges):
            merges = [f"{m[0]} {m[1]}" for m in raw_merges if len(m) == 2]
        else:
            raise TokenizerError("malformedTokenizerJSON")
        pattern = _find_regex(root.get("pre_tokenizer")) or DEFAULT_PRETOKENIZER
        return cls(encoder, merges, pattern, _prefix_ids(root, encoder), skipped)

    # ---- encode / decode ------------------------------------------------------------------------------------
    def _bpe(self, token: str) -> list[str]:
        hit = self._cache.get(token)
        if hit is not None:
            return hit
        word = list(token)
        while len(word) > 1:
            best_rank, best = None, None
            for pair in zip(word, word[1:]):
                r = self.ranks.get(pair)
                if r is not None and (best_rank is None or r < best_rank):
                    best_rank, best = r, pair
            if best is None:
                break
            merged, i = [], 0
            while i < len(word):
                if i + 1 < len(word) and word[i] == best[0] and word[i + 1] == best[1]:
                    merged.append(best[0] + best[1])
                    i += 2
                else:
                    merged.append(word[i])
                    i += 1
            word = merged
        self._cache[token] = word
        return word

    def encode(self, text: str) -> list[int]:
        out = list(self.prefix_token_ids)
        for match in self._pre.finditer(text):
            chunk = match.group(0)
            mapped = "".join(self._b2u[b] for b in chunk.encode("utf-8"))
            for piece in self._bpe(mapped):
                i = self.encoder.get(piece)
                if i is not None:
                    out.append(i)
        return out

    def decode(self, tokens: Iterable[int]) -> str:
        data = bytearray()
        for t in tokens:
            if not 0 <= t < len(self.decoder) or t in self.skipped_token_ids:
                continue
            for ch in self.decoder[t]:
                b = self._u2b.get(ch)
                if b is not None:
                    data.append(b)
                else:
                    data.extend(ch.encode("utf-8"))
        return data.decode("utf-8", errors="replace")


def _parse_vocabulary(raw) -> dict[str, int]:
    if not isinstance(raw, dict):
        raise TokenizerError("malformedVocabulary")
    if not raw:
        raise TokenizerError("emptyVocabulary")
    out = {}
    for piece, value in raw.items():
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise TokenizerError("malformedVocabulary")
        out[piece] = int(value)
    return out


def _find_regex(pre) -> Optional[str]:
    if not isinstance(pre, dict):
        return None
    pattern = pre.get("pattern")
    if isinstance(pattern, dict) and isinstance(pattern.get("Regex"), str):
        return pattern["Regex"]
    for entry in pre.get("pretokenizers") or []:
        found = _find_regex(entry)
        if found:
            return found
    return None


def _prefix_in(processor) -> Optional[list[int]]:
    if not isinstance(processor, dict):
        return None
    for entry in processor.get("processors") or []:
        found = _prefix_in(entry)
        if found is not None:
            return found
    special = processor.get("special_tokens")
    if isinstance(special, dict) and isinstance(special.get(BOS_NAME), dict):
        ids = [i for i in special[BOS_NAME].get("ids") or [] if isinstance(i, int)]
        if ids:
            return ids
    single = processor.get("single")
    if not isinstance(single, list):
        return None
    prefix: list[int] = []
    for item in single:
        if isinstance(item, dict) and isinstance(item.get("SpecialToken"), dict):
            prefix.extend(i for i in item["SpecialToken"].get("ids") or [] if isinstance(i, int))
            continue
        if isinstance(item, dict) and "Sequence" in item:
            break
    return prefix


def _prefix_ids(root: dict, encoder: dict[str, int]) -> list[int]:
    found = _prefix_in(root.get("post_processor"))
    if found:
        return found
    return [encoder[BOS_NAME]] if BOS_NAME in encoder else []


class SentencePieceTokenizer:
    def __init__(self, model_path: str):
        with open(model_path, "rb") as f:
            data = f.read()
        if len(data) < 4:
            raise TokenizerError("truncatedModel")
        (self.max_token_length,) = struct.unpack_from("<i", data, 0)
        if self.max_token_length <= 0:
            raise TokenizerError("invalidMaxTokenLength", str(self.max_token_length))
        cur = 4
        self.pieces: list[str] = []
        self.scores: list[float] = []
        self.piece_to_id: dict[str, int] = {}
        while cur < len(data):
            index = len(self.pieces)
            if cur + 8 > len(data):
                raise TokenizerError("truncatedEntry", f"index={index}")
            score, length = struct.unpack_from("<fi", data, cur)
            cur += 8
            if length < 0 or cur + length > len(data):
                raise TokenizerError("truncatedEntry", f"index={index}")
            try:
                piece = data[cur:cur + length].decode("utf-8")
            except UnicodeDecodeError as e:
                raise TokenizerError("invalidUTF8Entry", f"index={index}") from e
            cur += length
            self.pieces.append(piece)
            self.scores.append(score)
            self.piece_to_id[piece] = index  # a repeated piece keeps its last id, as a dictionary assignment does
        if not self.pieces:
            raise TokenizerError("emptyVocabulary")
        self.vocab_size = len(self.pieces)

    def encode(self, text: str) -> list[int]:
        tokens: list[int] = []
        for ch in "▁" + text.replace(" ", "▁"):
            i = self.piece_to_id.get(ch)
            if i is not None:
                tokens.append(i)
                continue
            for b in ch.encode("utf-8"):
                j = self.piece_to_id.get(f"<0x{b:02X}>")
                if j is not None:
                    tokens.append(j)
        while len(tokens) >= 2:
            best_score, best_at, best_id = None, -1, -1
            for k in range(len(tokens) - 1):
                merged = self.pieces[tokens[k]] + self.pieces[tokens[k + 1]]
                if len(merged.encode("utf-8")) > self.max_token_length:
                    continue
                i = self.piece_to_id.get(merged)
                if i is None:
                    continue
                if best_score is None or self.scores[i] > best_score:
                    best_score, best_at, best_id = self.scores[i], k, i
            if best_at < 0:
                break
            tokens[best_at:best_at + 2] = [best_id]
        return tokens

    def decode(self, tokens: Iterable[int]) -> str:
        text, pending = [], bytearray()
        for t in tokens:
            if not 0 <= t < len(self.pieces):
                continue
            piece = self.pieces[t]
            if piece.startswith("<0x") and piece.endswith(">") and len(piece) == 6:
                try:
                    pending.append(int(piece[3:5], 16))
                    continue
                except ValueError:
                    pass
            if pending:
                text.append(pending.decode("utf-8", errors="replace"))
                pending = bytearray()
            text.append(piece)
        if pending:
            text.append(pending.decode("utf-8", errors="replace"))
        restored = "".join(text).replace("▁", " ")
        return restored[1:] if restored.startswith(" ") else restored


def load_tokenizer(architecture: str, tokenizer_dir: str):
    """The reference's file search: GPT-2 needs vocab.json + merges.txt; llama tries tokenizer.model, tokenizer.bin,
    tokenizer.json, then vocab.json + merges.txt."""
    def p(name: str) -> str:
        return os.path.join(tokenizer_dir, name)

    if architecture == "gpt2":
        for name in ("vocab.json", "merges.txt"):
            if not os.path.exists(p(name)):
                raise FileNotFoundError(p(name))
        return GPT2BPETokenizer.from_vocab_and_merges(p("vocab.json"), p("merges.txt"))
    for name in ("tokenizer.model", "tokenizer.bin"):
        if os.path.exists(p(name)):
            return SentencePieceTokenizer(p(name))
    if os.path.exists(p("tokenizer.json")):
        return GPT2BPETokenizer.from_tokenizer_json(p("tokenizer.json"))
    if os.path.exists(p("vocab.json")) and os.path.exists(p("merges.txt")):
        return GPT2BPETokenizer.from_vocab_and_merges(p("vocab.json"), p("merges.txt"))
    raise FileNotFoundError(f"No tokenizer found in {tokenizer_dir} — tried tokenizer.model, tokenizer.bin, tokenizer.json, vocab.json+merges.txt")
