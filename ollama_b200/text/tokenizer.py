"""Tokenizers built from GGUF metadata: byte-level BPE, SentencePiece-style and WordPiece.

The reference delegates tokenisation to its engine subprocess; its two readable Go tokenizers are the
behavioural spec used here: tokenizer/bytepairencoding.go (special-token pre-split :129-160, regex
split :78-110, byte->rune map :172-186, merge loop :224-262, decode :299-367) and
tokenizer/sentencepiece.go:55-249.  Selection is by ``tokenizer.ggml.model`` and the pre-tokenizer id
``tokenizer.ggml.pre`` (convert/tokenizer.go:83-112).  BOS is added when ``tokenizer.ggml.add_bos_token``
is set (llm/llama_server.go:257-277).
"""
from __future__ import annotations

import functools
from typing import Iterable, Sequence

import regex

TOKEN_NORMAL, TOKEN_UNKNOWN, TOKEN_CONTROL, TOKEN_USER, TOKEN_UNUSED, TOKEN_BYTE = 1, 2, 3, 4, 5, 6

_CONTRACTIONS = r"(?:'[sS]|'[tT]|'[rR][eE]|'[vV][eE]|'[mM]|'[lL][lL]|'[dD])"
PRETOKENIZERS: dict[str, list[str]] = {
    "default": [r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"],
    "gpt-2": [r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"],
    "llama-bpe": [_CONTRACTIONS + r"|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"],
    "qwen2": [_CONTRACTIONS + r"|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"],
    "gpt-4o": [
        r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?"
        r"|[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?"
        r"|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+"],
    "tekken": [
        r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+"
        r"|[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*"
        r"|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+"],
    "deepseek-llm": [r"[\r\n]", r"\s?\p{L}+", r"\s?\p{P}+", r"[\u4e00-\u9fa5\u0800-\u4e00\uac00-\ud7ff]+", r"\p{N}+"],
    "deepseek-coder": [r"[\r\n]", r"\s?\p{L}+", r"\s?\p{P}+", r"[\u4e00-\u9fa5\u0800-\u4e00\uac00-\ud7ff]+", r"\p{N}"],
}
PRETOKENIZERS["llama3"] = PRETOKENIZERS["llama-bpe"]
PRETOKENIZERS["smaug-bpe"] = PRETOKENIZERS["llama-bpe"]
PRETOKENIZERS["qwen35"] = PRETOKENIZERS["qwen2"]
PRETOKENIZERS["deepseek-r1-qwen"] = PRETOKENIZERS["qwen2"]


@functools.lru_cache(maxsize=1)
def _byte_to_unicode() -> dict[int, str]:
    """GPT-2 reversible byte <-> printable code point table."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


@functools.lru_cache(maxsize=1)
def _unicode_to_byte() -> dict[str, int]:
    return {v: k for k, v in _byte_to_unicode().items()}


class Tokenizer:
    """Common surface: ``encode``, ``decode``, ``token_bytes`` and the special-token bookkeeping."""

    model = "none"

    def __init__(self, tokens: Sequence[str], types: Sequence[int] | None, *, bos: int = -1, eos: int = -1,
                 eos_ids: Iterable[int] = (), add_bos: bool = False, add_eos: bool = False, unk: int = -1, pad: int = -1):
        self.tokens = list(tokens)
        self.types = list(types) if types is not None and len(types) == len(tokens) else [TOKEN_NORMAL] * len(tokens)
        self.vocab = {t: i for i, t in enumerate(self.tokens)}
        self.bos, self.eos, self.unk, self.pad = int(bos), int(eos), int(unk), int(pad)
        self.add_bos, self.add_eos = bool(add_bos), bool(add_eos)
        self.eog = {int(e) for e in eos_ids if int(e) >= 0}
        if self.eos >= 0:
            self.eog.add(self.eos)
        for name in ("<|eot_id|>", "<|im_end|>", "<|end|>", "<end_of_turn>", "<|endoftext|>", "<|return|>", "<|call|>", "<|eom_id|>", "<EOT>"):
            i = self.vocab.get(name)
            if i is not None and self.types[i] in (TOKEN_CONTROL, TOKEN_USER) and name not in ("<|end|>",):
                self.eog.add(i)
        self.special = {i for i, t in enumerate(self.types) if t in (TOKEN_CONTROL, TOKEN_USER)}
        # special tokens are matched verbatim, longest first, so that "<|eot_id|>" wins over any prefix of it;
        # lookups go through a set per length (a vocabulary may carry tens of thousands of them)
        self._special_set = {self.tokens[i] for i in self.special if self.tokens[i]}
        self._special_lens = sorted({len(s) for s in self._special_set}, reverse=True)
        self._special_first = {s[0] for s in self._special_set}

    @property
    def n_vocab(self) -> int:
        return len(self.tokens)

    def is_eog(self, tok: int) -> bool:
        return tok in self.eog

    # -- to be provided by subclasses -------------------------------------------------------------
    def _encode_piece(self, text: str) -> list[int]:
        raise NotImplementedError

    def token_bytes(self, tok: int) -> bytes:
        raise NotImplementedError

    # -- shared ----------------------------------------------------------------------------------
    def encode(self, text: str, add_special: bool = True, parse_special: bool = True) -> list[int]:
        out: list[int] = []
        if add_special and self.add_bos and self.bos >= 0:
            out.append(self.bos)
        first = True
        for is_special, frag in self._split_special(text, parse_special):
            if is_special:
                out.append(self.vocab[frag])
            elif frag:
                out.extend(self._encode_fragment(frag, first))
            first = False
        if add_special and self.add_eos and self.eos >= 0:
            out.append(self.eos)
        return out

    def _encode_fragment(self, frag: str, first: bool) -> list[int]:
        return self._encode_piece(frag)

    def _split_special(self, text: str, parse_special: bool):
        if not parse_special or not self._special_set:
            yield False, text
            return
        pos, i, n = 0, 0, len(text)
        first, lens, sset = self._special_first, self._special_lens, self._special_set
        while i < n:
            if text[i] in first:
                hit = 0
                for ln in lens:
                    if text[i:i + ln] in sset and i + ln <= n:
                        hit = ln
                        break
                if hit:
                    if i > pos:
                        yield False, text[pos:i]
                    yield True, text[i:i + hit]
                    i += hit
                    pos = i
                    continue
            i += 1
        if pos < n:
            yield False, text[pos:]

    def decode_bytes(self, ids: Iterable[int], skip_special: bool = False) -> bytes:
        out = bytearray()
        for t in ids:
            if t < 0 or t >= len(self.tokens):
                continue
            if skip_special and self.types[t] == TOKEN_CONTROL:
                continue
            out += self.token_bytes(t)
        return bytes(out)

    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        return self.decode_bytes(ids, skip_special).decode("utf-8", errors="replace")


class BPETokenizer(Tokenizer):
    model = "gpt2"

    def __init__(self, tokens, types, merges: Sequence[str], pre: str = "default", **kw):
        super().__init__(tokens, types, **kw)
        self.ranks: dict[tuple[str, str], int] = {}
        for i, m in enumerate(merges):
            a, _, b = m.partition(" ")
            self.ranks[(a, b)] = i
        pats = PRETOKENIZERS.get(pre) or PRETOKENIZERS["default"]
        self.pre = pre
        self._pats = [regex.compile(p) for p in pats]
        self._cache: dict[str, list[int]] = {}
        self._native = None       # (library, table handle, byte -> symbol id) once built; False: not usable

    def _pretokenize(self, text: str) -> list[str]:
        pieces = [text]
        for pat in self._pats:
            nxt: list[str] = []
            for p in pieces:
                pos = 0
                for m in pat.finditer(p):
                    if m.start() > pos:
                        nxt.append(p[pos:m.start()])
                    if m.group(0):
                        nxt.append(m.group(0))
                    pos = m.end()
                if pos < len(p):
                    nxt.append(p[pos:])
            pieces = nxt
            if len(self._pats) == 1:
                break
        return pieces

    def _bpe(self, word: str) -> list[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        parts = list(word)
        ranks = self.ranks
        while len(parts) > 1:
            best, best_i = None, -1
            for i in range(len(parts) - 1):
                r = ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, best_i = r, i
            if best is None:
                break
            a, b = parts[best_i], parts[best_i + 1]
            merged: list[str] = []
            i = 0
            while i < len(parts):
                if i < len(parts) - 1 and parts[i] == a and parts[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(parts[i])
                    i += 1
            parts = merged
        out: list[int] = []
        for p in parts:
            i = self.vocab.get(p)
            if i is not None:
                out.append(i)
            else:  # unknown piece: fall back to its single characters / byte tokens
                for ch in p:
                    j = self.vocab.get(ch)
                    if j is None:
                        j = self.vocab.get(f"<0x{_unicode_to_byte().get(ch, 0):02X}>", self.unk)
                    if j >= 0:
                        out.append(j)
        if len(self._cache) < 1 << 16:
            self._cache[word] = out
        return out

    def _native_table(self):
        """Merge table of the C++ merge loop (native/bpe.cpp), or None: no library, a byte symbol missing from the
        vocabulary, or a merge whose result is not a token (the Python loop then splits such pieces again)."""
        if self._native is not None:
            return self._native or None
        self._native = False
        from ..utils import hostlib
        L = hostlib.lib()
        if L is None or not hasattr(L, "b2h_bpe_new"):
            return None
        import ctypes as C

        import numpy as np
        b2u = _byte_to_unicode()
        byte_ids = np.array([self.vocab.get(b2u[b], -1) for b in range(256)], dtype=np.int32)
        triples = np.empty((len(self.ranks), 3), dtype=np.int32)
        for (a, b), r in self.ranks.items():
            ia, ib, im = self.vocab.get(a), self.vocab.get(b), self.vocab.get(a + b)
            if ia is None or ib is None or im is None:
                return None
            triples[r] = (ia, ib, im)
        L.b2h_bpe_new.restype = C.c_void_p
        L.b2h_bpe_new.argtypes = [C.c_void_p, C.c_int32]
        L.b2h_bpe_encode.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]
        h = L.b2h_bpe_new(triples.ctypes.data, len(triples)) if len(triples) == len({tuple(t[:2]) for t in triples.tolist()}) else None
        if not h:
            return None
        self._native = (L, h, byte_ids)
        return self._native

    def _encode_piece(self, text: str) -> list[int]:
        words = self._pretokenize(text)
        tab = self._native_table() if len(words) >= 8 else None
        if tab is not None:
            import numpy as np
            L, h, byte_ids = tab
            enc = [w.encode("utf-8") for w in words]
            syms = byte_ids[np.frombuffer(b"".join(enc), dtype=np.uint8)]
            if syms.size and int(syms.min()) >= 0:
                off = np.zeros(len(enc) + 1, dtype=np.int64)
                np.cumsum([len(e) for e in enc], out=off[1:])
                out = np.empty(syms.size, dtype=np.int32)
                out_off = np.empty(len(enc) + 1, dtype=np.int64)
                syms = np.ascontiguousarray(syms, dtype=np.int32)
                if L.b2h_bpe_encode(h, syms.ctypes.data, off.ctypes.data, len(enc), out.ctypes.data, out_off.ctypes.data) == 0:
                    return out[:int(out_off[-1])].tolist()
        b2u = _byte_to_unicode()
        out: list[int] = []
        for w in words:
            out.extend(self._bpe("".join(b2u[b] for b in w.encode("utf-8"))))
        return out

    def token_bytes(self, tok: int) -> bytes:
        s = self.tokens[tok]
        if tok in self.special:
            return s.encode("utf-8")
        u2b = _unicode_to_byte()
        out = bytearray()
        for ch in s:
            b = u2b.get(ch)
            if b is None:
                out += ch.encode("utf-8")
            else:
                out.append(b)
        return bytes(out)


class SPMTokenizer(Tokenizer):
    """SentencePiece-style: whitespace becomes U+2581, greedy highest-score bigram merges, byte fallback."""

    model = "llama"
    SPACE = "▁"

    def __init__(self, tokens, types, scores: Sequence[float] | None, add_space_prefix: bool = True, **kw):
        super().__init__(tokens, types, **kw)
        self.scores = list(scores) if scores is not None and len(scores) == len(tokens) else [0.0] * len(tokens)
        self.add_space_prefix = add_space_prefix
        self._byte_tok = {}
        for i, (t, ty) in enumerate(zip(self.tokens, self.types)):
            if ty == TOKEN_BYTE and len(t) == 6 and t.startswith("<0x"):
                self._byte_tok[int(t[3:5], 16)] = i

    def _encode_fragment(self, frag: str, first: bool) -> list[int]:
        if first and self.add_space_prefix:
            frag = " " + frag
        return self._encode_piece(frag.replace(" ", self.SPACE))

    def _encode_piece(self, text: str) -> list[int]:
        import heapq
        syms = list(text)
        n = len(syms)
        if n == 0:
            return []
        prev = list(range(-1, n - 1))
        nxt = list(range(1, n + 1))
        nxt[-1] = -1
        alive = [True] * n
        heap: list[tuple[float, int, int, str]] = []

        def push(i: int) -> None:
            j = nxt[i]
            if i < 0 or j < 0:
                return
            s = syms[i] + syms[j]
            tid = self.vocab.get(s)
            if tid is not None:
                heapq.heappush(heap, (-self.scores[tid], i, j, s))

        for i in range(n - 1):
            push(i)
        while heap:
            _, i, j, s = heapq.heappop(heap)
            if not (alive[i] and alive[j]) or nxt[i] != j or syms[i] + syms[j] != s:
                continue
            syms[i] = s
            alive[j] = False
            nxt[i] = nxt[j]
            if nxt[j] >= 0:
                prev[nxt[j]] = i
            if prev[i] >= 0:
                push(prev[i])
            push(i)
        out: list[int] = []
        i = 0
        while i >= 0:
            tid = self.vocab.get(syms[i])
            if tid is not None:
                out.append(tid)
            else:
                for b in syms[i].encode("utf-8"):
                    bt = self._byte_tok.get(b)
                    out.append(bt if bt is not None else max(self.unk, 0))
            i = nxt[i]
        return out

    def token_bytes(self, tok: int) -> bytes:
        ty = self.types[tok]
        s = self.tokens[tok]
        if ty == TOKEN_BYTE and len(s) == 6 and s.startswith("<0x"):
            return bytes([int(s[3:5], 16)])
        if ty in (TOKEN_CONTROL, TOKEN_USER):
            return s.encode("utf-8")
        return s.replace(self.SPACE, " ").encode("utf-8")

    def decode_bytes(self, ids, skip_special: bool = False) -> bytes:
        b = super().decode_bytes(ids, skip_special)
        return b


class WPMTokenizer(Tokenizer):
    """BERT WordPiece: lower-cased whitespace/punctuation split, greedy longest match with ``##`` continuations."""

    model = "bert"

    def __init__(self, tokens, types, lowercase: bool = True, **kw):
        super().__init__(tokens, types, **kw)
        self.lowercase = lowercase
        self.cls = self.vocab.get("[CLS]", self.bos)
        self.sep = self.vocab.get("[SEP]", self.eos)
        # GGUF stores word-initial pieces with a leading U+2581 and continuations bare
        self.ggml_style = any(t.startswith("▁") for t in self.tokens[:2000])

    def encode(self, text: str, add_special: bool = True, parse_special: bool = True) -> list[int]:
        ids = self._encode_piece(text)
        if add_special:
            ids = ([self.cls] if self.cls >= 0 else []) + ids + ([self.sep] if self.sep >= 0 else [])
        return ids

    def _encode_piece(self, text: str) -> list[int]:
        if self.lowercase:
            text = text.lower()
        words = regex.findall(r"[\p{L}\p{N}\p{M}]+|[^\s\p{L}\p{N}\p{M}]", text)
        out: list[int] = []
        for w in words:
            start, pieces = 0, []
            while start < len(w):
                end, cur = len(w), None
                while end > start:
                    sub = w[start:end]
                    if self.ggml_style:
                        cand = ("▁" + sub) if start == 0 else sub
                    else:
                        cand = sub if start == 0 else "##" + sub
                    if cand in self.vocab:
                        cur = self.vocab[cand]
                        break
                    end -= 1
                if cur is None:
                    pieces = [max(self.unk, 0)]
                    break
                pieces.append(cur)
                start = end
            out.extend(pieces)
        return out

    def token_bytes(self, tok: int) -> bytes:
        s = self.tokens[tok]
        if s.startswith("##"):
            return s[2:].encode()
        if s.startswith("▁"):
            return (" " + s[1:]).encode()
        return s.encode() if self.ggml_style else (" " + s).encode()


def tokenizer_from_gguf(kv: dict) -> Tokenizer:
    """Instantiate the tokenizer described by the ``tokenizer.ggml.*`` block of a GGUF."""
    model = str(kv.get("tokenizer.ggml.model", "gpt2"))
    tokens = kv.get("tokenizer.ggml.tokens")
    if tokens is None:
        raise ValueError("the model has no tokenizer.ggml.tokens")
    types = kv.get("tokenizer.ggml.token_type")
    types = [int(t) for t in types] if types is not None else None
    eos_ids = kv.get("tokenizer.ggml.eos_token_ids")
    common = dict(
        bos=int(kv.get("tokenizer.ggml.bos_token_id", -1)), eos=int(kv.get("tokenizer.ggml.eos_token_id", -1)),
        eos_ids=[int(x) for x in eos_ids] if eos_ids is not None else [],
        unk=int(kv.get("tokenizer.ggml.unknown_token_id", -1)), pad=int(kv.get("tokenizer.ggml.padding_token_id", -1)),
        add_eos=bool(kv.get("tokenizer.ggml.add_eos_token", False)),
    )
    pre = str(kv.get("tokenizer.ggml.pre", "default"))
    if model == "gpt2":
        add_bos = bool(kv.get("tokenizer.ggml.add_bos_token", False))
        merges = kv.get("tokenizer.ggml.merges") or []
        return BPETokenizer(tokens, types, merges, pre, add_bos=add_bos, **common)
    if model in ("llama", "gemma4"):
        add_bos = bool(kv.get("tokenizer.ggml.add_bos_token", True)) or model == "gemma4"
        scores = kv.get("tokenizer.ggml.scores")
        scores = [float(s) for s in scores] if scores is not None else None
        return SPMTokenizer(tokens, types, scores, bool(kv.get("tokenizer.ggml.add_space_prefix", True)), add_bos=add_bos, **common)
    if model == "bert":
        return WPMTokenizer(tokens, types, add_bos=True, **common)
    raise NotImplementedError(f"unsupported tokenizer model {model!r}")
