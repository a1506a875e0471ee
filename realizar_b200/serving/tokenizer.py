"""Tokenizers: byte-level BPE (with merges, or greedy longest-match over a bare vocabulary as
found in GGUF files that ship no merges), SentencePiece-style unigram (Viterbi over scores), and
construction from GGUF / APR metadata.

Behavioural parity with the reference (``BPETokenizer`` src/tokenizer.rs:24-478: GPT-2 byte
mapping ``Ġ``/``Ċ``, greedy longest match of up to 32 characters, ``<0xNN>`` byte fallback;
``SentencePieceTokenizer`` src/tokenizer_sentence_piece.rs:13-300; special tokens matched
atomically, src/apr/tokenizer.rs).
"""
from __future__ import annotations

import math
import re
from functools import lru_cache
from typing import Dict, Iterable, List, Optional, Sequence, Tuple


class TokenizerError(ValueError):
    pass


@lru_cache(maxsize=1)
def bytes_to_unicode() -> Dict[int, str]:
    """GPT-2's reversible byte <-> printable-character table (space -> ``Ġ``, newline -> ``Ċ``)."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


@lru_cache(maxsize=1)
def unicode_to_bytes() -> Dict[str, int]:
    return {v: k for k, v in bytes_to_unicode().items()}


_PRETOKENIZE = re.compile(r"'s|'t|'re|'ve|'m|'ll|'d| ?[^\W\d_]+| ?\d+| ?[^\s\w]+|\s+(?!\S)|\s+", re.UNICODE)
_SPECIAL_RE = re.compile(r"^<\|.*\|>$|^<s>$|^</s>$|^<unk>$|^<pad>$|^\[INST\]$|^\[/INST\]$")


class Vocabulary:
    def __init__(self, tokens: Sequence[str]):
        if not tokens:
            raise TokenizerError("vocabulary is empty")
        self.tokens = list(tokens)
        self.index: Dict[str, int] = {}
        for i, t in enumerate(self.tokens):
            self.index.setdefault(t, i)

    def __len__(self): return len(self.tokens)
    def id(self, token: str) -> Optional[int]: return self.index.get(token)
    def token(self, i: int) -> Optional[str]: return self.tokens[i] if 0 <= i < len(self.tokens) else None


class BPETokenizer:
    def __init__(self, vocab: Sequence[str], merges: Optional[Iterable] = None, special_tokens: Optional[Iterable[str]] = None,
                 bos_token_id: Optional[int] = None, eos_token_id: Optional[int] = None, add_bos: bool = False, unk_token: str = "<unk>"):
        self.vocab = Vocabulary(vocab)
        self.ranks: Dict[Tuple[str, str], int] = {}
        if merges:
            for i, m in enumerate(merges):
                a, _, b = m.partition(" ") if isinstance(m, str) else (m[0], " ", m[1])
                self.ranks[(a, b)] = i
        sp = set(special_tokens or [])
        sp.update(t for t in self.vocab.tokens if _SPECIAL_RE.match(t))
        self.special = sorted(sp & set(self.vocab.index), key=len, reverse=True)
        self._special_re = re.compile("(" + "|".join(re.escape(s) for s in self.special) + ")") if self.special else None
        self.bos_token_id, self.eos_token_id, self.add_bos = bos_token_id, eos_token_id, add_bos
        self.unk_id = self.vocab.id(unk_token)
        self.max_piece = min(32, max(len(t) for t in self.vocab.tokens))
        self._cache: Dict[str, List[int]] = {}

    @property
    def vocab_size(self) -> int:
        return len(self.vocab)

    # -- encoding --------------------------------------------------------------------------
    def _bpe(self, word: str) -> List[str]:
        parts = list(word)
        while len(parts) > 1:
            best, best_rank = None, None
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best is None:
                break
            parts[best: best + 2] = [parts[best] + parts[best + 1]]
        return parts

    def _greedy(self, word: str) -> List[int]:
        out, i = [], 0
        b2u = unicode_to_bytes()
        while i < len(word):
            for L in range(min(self.max_piece, len(word) - i), 0, -1):
                tid = self.vocab.id(word[i: i + L])
                if tid is not None:
                    out.append(tid)
                    i += L
                    break
            else:                                            # unknown character: byte fallback, then <unk>
                ch = word[i]
                raw = bytes([b2u[ch]]) if ch in b2u else ch.encode("utf-8")
                for byte in raw:
                    tid = self.vocab.id(f"<0x{byte:02X}>")
                    if tid is None:
                        tid = self.unk_id
                    if tid is not None:
                        out.append(tid)
                i += 1
        return out

    def _encode_chunk(self, text: str) -> List[int]:
        if text in self._cache:
            return self._cache[text]
        b2u = bytes_to_unicode()
        ids: List[int] = []
        for piece in _PRETOKENIZE.findall(text):
            word = "".join(b2u[b] for b in piece.encode("utf-8"))
            if self.ranks:
                for part in self._bpe(word):
                    tid = self.vocab.id(part)
                    ids.extend([tid] if tid is not None else self._greedy(part))
            else:
                ids.extend(self._greedy(word))
        if len(self._cache) < 4096:
            self._cache[text] = ids
        return ids

    def encode(self, text: str, add_bos: Optional[bool] = None) -> List[int]:
        ids: List[int] = []
        if (self.add_bos if add_bos is None else add_bos) and self.bos_token_id is not None:
            ids.append(self.bos_token_id)
        chunks = self._special_re.split(text) if self._special_re else [text]
        for c in chunks:
            if not c:
                continue
            if c in self.special:
                ids.append(self.vocab.index[c])
            else:
                ids.extend(self._encode_chunk(c))
        return ids

    # -- decoding --------------------------------------------------------------------------
    def token_bytes(self, tid: int) -> bytes:
        t = self.vocab.token(tid)
        if t is None:
            return b""
        if t in self.special:
            return t.encode()
        m = re.fullmatch(r"<0x([0-9A-Fa-f]{2})>", t)
        if m:
            return bytes([int(m.group(1), 16)])
        u2b = unicode_to_bytes()
        out = bytearray()
        for ch in t:
            if ch in u2b:
                out.append(u2b[ch])
            else:
                out.extend(ch.encode("utf-8"))
        return bytes(out)

    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        buf = bytearray()
        for i in ids:
            t = self.vocab.token(int(i))
            if t is None or (skip_special and t in self.special):
                continue
            buf.extend(self.token_bytes(int(i)))
        return buf.decode("utf-8", "replace")


class StreamDecoder:
    """Incremental detokenisation for streaming: holds back bytes until they form whole UTF-8 characters."""

    def __init__(self, tokenizer):
        self.tok, self.pending = tokenizer, b""

    def push(self, token_id: int) -> str:
        self.pending += self.tok.token_bytes(token_id)
        for cut in range(len(self.pending), max(len(self.pending) - 4, -1), -1):
            try:
                text = self.pending[:cut].decode("utf-8")
                self.pending = self.pending[cut:]
                return text
            except UnicodeDecodeError:
                continue
        return ""

    def flush(self) -> str:
        text, self.pending = self.pending.decode("utf-8", "replace"), b""
        return text


class SentencePieceTokenizer:
    """Unigram model: Viterbi segmentation maximising the sum of piece scores; ``▁`` marks spaces."""
    SPACE = "▁"

    def __init__(self, pieces: Sequence[str], scores: Sequence[float], unk_id: int = 0, bos_token_id: Optional[int] = None,
                 eos_token_id: Optional[int] = None, add_bos: bool = True, special_tokens: Optional[Iterable[str]] = None):
        if len(pieces) != len(scores):
            raise TokenizerError("pieces and scores differ in length")
        self.vocab = Vocabulary(pieces)
        self.scores = list(scores)
        self.unk_id, self.bos_token_id, self.eos_token_id, self.add_bos = unk_id, bos_token_id, eos_token_id, add_bos
        self.max_piece = max(len(p) for p in pieces)
        sp = set(special_tokens or [])
        sp.update(t for t in pieces if _SPECIAL_RE.match(t))
        self.special = sorted(sp & set(self.vocab.index), key=len, reverse=True)
        self._special_re = re.compile("(" + "|".join(re.escape(s) for s in self.special) + ")") if self.special else None

    @property
    def vocab_size(self): return len(self.vocab)

    def _viterbi(self, s: str) -> List[int]:
        n = len(s)
        best = [-math.inf] * (n + 1)
        back: List[Tuple[int, int]] = [(0, self.unk_id)] * (n + 1)
        best[0] = 0.0
        for i in range(n):
            if best[i] == -math.inf:
                continue
            matched = False
            for L in range(1, min(self.max_piece, n - i) + 1):
                tid = self.vocab.id(s[i: i + L])
                if tid is not None and s[i: i + L] not in self.special:
                    sc = best[i] + self.scores[tid]
                    if sc > best[i + L]:
                        best[i + L], back[i + L] = sc, (i, tid)
                    matched = True
            if not matched or best[i + 1] == -math.inf:
                sc = best[i] - 20.0                           # unknown character penalty
                if sc > best[i + 1]:
                    best[i + 1], back[i + 1] = sc, (i, -1)
        ids, i = [], n
        while i > 0:
            j, tid = back[i]
            if tid == -1:                                      # byte fallback pieces, else <unk>
                raw = s[j:i].encode("utf-8")
                fb = [self.vocab.id(f"<0x{b:02X}>") for b in raw]
                ids.extend(reversed(fb if all(f is not None for f in fb) else [self.unk_id]))
            else:
                ids.append(tid)
            i = j
        return ids[::-1]

    def encode(self, text: str, add_bos: Optional[bool] = None) -> List[int]:
        ids: List[int] = []
        if (self.add_bos if add_bos is None else add_bos) and self.bos_token_id is not None:
            ids.append(self.bos_token_id)
        chunks = self._special_re.split(text) if self._special_re else [text]
        first = True
        for c in chunks:
            if not c:
                continue
            if c in self.special:
                ids.append(self.vocab.index[c])
            else:
                s = c.replace(" ", self.SPACE)
                if first and not s.startswith(self.SPACE):
                    s = self.SPACE + s
                ids.extend(self._viterbi(s))
            first = False
        return ids

    def token_bytes(self, tid: int) -> bytes:
        t = self.vocab.token(tid)
        if t is None:
            return b""
        m = re.fullmatch(r"<0x([0-9A-Fa-f]{2})>", t)
        return bytes([int(m.group(1), 16)]) if m else t.replace(self.SPACE, " ").encode("utf-8")

    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        buf = bytearray()
        for i in ids:
            t = self.vocab.token(int(i))
            if t is None or (skip_special and t in self.special):
                continue
            buf.extend(self.token_bytes(int(i)))
        text = buf.decode("utf-8", "replace").replace(self.SPACE, " ")     # a byte-fallback "▁" is a space too
        return text[1:] if text.startswith(" ") else text


def tokenizer_from_gguf(g):
    """Build the tokenizer described by ``tokenizer.ggml.*`` metadata; None if the file has no vocabulary."""
    toks = g.get("tokenizer.ggml.tokens")
    if not toks:
        return None
    model = g.get("tokenizer.ggml.model", "gpt2")
    bos, eos = g.get("tokenizer.ggml.bos_token_id"), g.get("tokenizer.ggml.eos_token_id")
    add_bos = bool(g.get("tokenizer.ggml.add_bos_token", model == "llama"))
    ttype = g.get("tokenizer.ggml.token_type") or []
    special = [t for t, ty in zip(toks, ttype) if ty in (3, 4)]   # control / user-defined
    if model == "llama" and g.get("tokenizer.ggml.scores"):
        return SentencePieceTokenizer(toks, g.get("tokenizer.ggml.scores"), unk_id=g.get("tokenizer.ggml.unknown_token_id", 0) or 0,
                                      bos_token_id=bos, eos_token_id=eos, add_bos=add_bos, special_tokens=special)
    return BPETokenizer(toks, g.get("tokenizer.ggml.merges"), special, bos, eos, add_bos)


class ByteTokenizer:
    """Fallback for checkpoints without a vocabulary: token id = byte value (ids above 255 print as ``<id>``)."""

    def __init__(self, vocab_size: int = 256, eos_token_id: Optional[int] = None):
        self.vocab_size, self.eos_token_id, self.bos_token_id = vocab_size, eos_token_id, None

    def encode(self, text: str, add_bos=None) -> List[int]:
        return [b % self.vocab_size for b in text.encode("utf-8")]

    def token_bytes(self, tid: int) -> bytes:
        return bytes([tid]) if 0 <= tid < 256 else f"<{tid}>".encode()

    def decode(self, ids, skip_special: bool = False) -> str:
        return b"".join(self.token_bytes(int(i)) for i in ids).decode("utf-8", "replace")
