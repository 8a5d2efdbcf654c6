"""Tokenizers read from the GGUF header: GPT-2 byte-level BPE (``tokenizer.ggml.model`` =
``gpt2``, with the pre-tokenizer program named by ``tokenizer.ggml.pre``), llama
SentencePiece (score-driven bigram merges with byte fallback), and a byte tokenizer for
fixtures without a vocabulary.  Counterpart of ``crates/tokenizer`` (``lib.rs:1-17``,
``bpe.rs``, ``spm.rs``, ``pretok.rs``, ``guard.rs``).

Guard marks: text that came from the client is encoded with ``parse_special=False`` so it can
never spell a control token; only the template's own markup may (``crates/serve/src/guard.rs``).
"""
from __future__ import annotations

import heapq
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import regex

# ggml token types
T_NORMAL, T_UNKNOWN, T_CONTROL, T_USER, T_UNUSED, T_BYTE = 1, 2, 3, 4, 5, 6

PRETOK = {
    "default": r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""",
    "gpt-2": r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""",
    "llama-bpe": r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+""",
    "qwen2": r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+""",
    "deepseek-v3": r"""\p{N}{1,3}|[一-龥぀-ゟ゠-ヿ]+|[!"#$%&'()*+,\-./:;<=>?@\[\\\]^_`{|}~][A-Za-z]+|[^\r\n\p{L}\p{P}\p{S}]?[\p{L}\p{M}]+| ?[\p{P}\p{S}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+""",
}
PRETOK["llama3"] = PRETOK["llama-bpe"]
PRETOK["deepseek-llm"] = PRETOK["llama-bpe"]
PRETOK["kimi-k2"] = PRETOK["deepseek-v3"]


def _byte_unicode() -> Tuple[Dict[int, str], Dict[str, int]]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    b2u = {b: chr(c) for b, c in zip(bs, cs)}
    return b2u, {v: k for k, v in b2u.items()}


B2U, U2B = _byte_unicode()


class Tokenizer:
    """Common surface: encode / decode / special ids / streaming-safe detokenisation."""

    n_vocab = 0
    bos_id = eos_id = eot_id = -1
    add_bos = False

    def encode(self, text: str, parse_special: bool = True, add_bos: Optional[bool] = None) -> List[int]:
        raise NotImplementedError

    def token_bytes(self, tid: int) -> bytes:
        raise NotImplementedError

    def is_control(self, tid: int) -> bool:
        return False

    def is_eog(self, tid: int) -> bool:
        return tid in (self.eos_id, self.eot_id) and tid >= 0

    def decode(self, ids: Iterable[int], skip_special: bool = True) -> str:
        return self.decode_bytes(ids, skip_special).decode("utf-8", errors="replace")

    def decode_bytes(self, ids: Iterable[int], skip_special: bool = True) -> bytes:
        out = bytearray()
        for t in ids:
            if skip_special and self.is_control(t):
                continue
            out += self.token_bytes(t)
        return bytes(out)

    def encode_marked(self, segments: Sequence[Tuple[str, bool]], add_bos: Optional[bool] = None) -> List[int]:
        """Segments are (text, trusted).  Untrusted (client) text never yields control tokens."""
        ids: List[int] = []
        if (self.add_bos if add_bos is None else add_bos) and self.bos_id >= 0:
            ids.append(self.bos_id)
        for text, trusted in segments:
            if text:
                ids += self.encode(text, parse_special=trusted, add_bos=False)
        return ids


class StreamDecoder:
    """Turns a stream of token ids into text pieces that never split a UTF-8 sequence."""

    def __init__(self, tok: Tokenizer, skip_special: bool = True):
        self.tok, self.skip = tok, skip_special
        self.pending = b""

    def push(self, tid: int) -> str:
        if self.skip and self.tok.is_control(tid):
            return ""
        buf = self.pending + self.tok.token_bytes(tid)
        # longest prefix that is complete UTF-8
        cut = len(buf)
        for back in range(1, min(4, len(buf)) + 1):
            b = buf[-back]
            if b & 0xC0 == 0x80:
                continue
            need = 1 if b < 0x80 else 2 if b >> 5 == 0b110 else 3 if b >> 4 == 0b1110 else 4 if b >> 3 == 0b11110 else 1
            if need > back:
                cut = len(buf) - back
            break
        self.pending = buf[cut:]
        return buf[:cut].decode("utf-8", errors="replace")

    def flush(self) -> str:
        s = self.pending.decode("utf-8", errors="replace")
        self.pending = b""
        return s


class ByteTokenizer(Tokenizer):
    """ids 0..255 are bytes; 256 = BOS, 257 = EOS.  Used by fixtures and the mock engine."""

    def __init__(self, n_vocab: int = 258):
        self.n_vocab = max(258, n_vocab)
        self.bos_id, self.eos_id, self.eot_id = 256, 257, 257

    def encode(self, text, parse_special=True, add_bos=None):
        ids = list(text.encode("utf-8"))
        return ([self.bos_id] if add_bos else []) + ids

    def token_bytes(self, tid):
        return bytes([tid]) if 0 <= tid < 256 else b""

    def is_control(self, tid):
        return tid >= 256


class BpeTokenizer(Tokenizer):
    def __init__(self, tokens: Sequence[str], merges: Sequence[str], types: Optional[Sequence[int]] = None,
                 pre: str = "default", bos_id: int = -1, eos_id: int = -1, eot_id: int = -1, add_bos: bool = False):
        self.tokens = list(tokens)
        self.n_vocab = len(self.tokens)
        self.id_of = {t: i for i, t in enumerate(self.tokens)}
        self.rank = {tuple(m.split(" ", 1)): i for i, m in enumerate(merges)}
        self.types = list(types) if types is not None else [T_NORMAL] * self.n_vocab
        self.bos_id, self.eos_id, self.eot_id, self.add_bos = bos_id, eos_id, eot_id, add_bos
        self.re = regex.compile(PRETOK.get(pre, PRETOK["default"]))
        special = [t for i, t in enumerate(self.tokens) if self.types[i] in (T_CONTROL, T_USER) and t]
        special.sort(key=len, reverse=True)
        self.special_re = regex.compile("|".join(regex.escape(t) for t in special)) if special else None
        self._cache: Dict[str, List[int]] = {}
        if self.eot_id < 0:
            for name in ("<|im_end|>", "<|eot_id|>", "<|end|>", "<end_of_turn>", "<|endoftext|>"):
                if name in self.id_of:
                    self.eot_id = self.id_of[name]
                    break

    def _bpe(self, word: str) -> List[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        parts = list(word)
        while len(parts) > 1:
            best, best_i = None, -1
            for i in range(len(parts) - 1):
                r = self.rank.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, best_i = r, i
            if best is None:
                break
            parts[best_i:best_i + 2] = [parts[best_i] + parts[best_i + 1]]
        ids = []
        for p in parts:
            t = self.id_of.get(p)
            if t is None:            # unknown piece: fall back to its single characters
                ids += [self.id_of[c] for c in p if c in self.id_of]
            else:
                ids.append(t)
        if len(self._cache) < 65536:
            self._cache[word] = ids
        return ids

    def _encode_plain(self, text: str) -> List[int]:
        ids: List[int] = []
        for m in self.re.finditer(text):
            ids += self._bpe("".join(B2U[b] for b in m.group(0).encode("utf-8")))
        return ids

    def encode(self, text, parse_special=True, add_bos=None):
        ids: List[int] = []
        if (self.add_bos if add_bos is None else add_bos) and self.bos_id >= 0:
            ids.append(self.bos_id)
        if parse_special and self.special_re is not None:
            pos = 0
            for m in self.special_re.finditer(text):
                if m.start() > pos:
                    ids += self._encode_plain(text[pos:m.start()])
                ids.append(self.id_of[m.group(0)])
                pos = m.end()
            if pos < len(text):
                ids += self._encode_plain(text[pos:])
        else:
            ids += self._encode_plain(text)
        return ids

    def token_bytes(self, tid):
        if not 0 <= tid < self.n_vocab:
            return b""
        t = self.tokens[tid]
        if self.types[tid] in (T_CONTROL, T_USER):
            return t.encode("utf-8")
        return bytes(U2B.get(c, ord("?") if ord(c) > 255 else ord(c)) for c in t)

    def is_control(self, tid):
        return 0 <= tid < self.n_vocab and self.types[tid] == T_CONTROL


class SpmTokenizer(Tokenizer):
    """llama SentencePiece: merge the adjacent pair whose union is a token of the highest score."""

    def __init__(self, tokens: Sequence[str], scores: Sequence[float], types: Sequence[int], bos_id=1, eos_id=2,
                 add_bos=True, add_space_prefix=True):
        self.tokens, self.scores, self.types = list(tokens), list(scores), list(types)
        self.n_vocab = len(self.tokens)
        self.id_of = {t: i for i, t in enumerate(self.tokens)}
        self.bos_id, self.eos_id, self.eot_id, self.add_bos = bos_id, eos_id, eos_id, add_bos
        self.space_prefix = add_space_prefix
        self.byte_id = {}
        for i, (t, ty) in enumerate(zip(self.tokens, self.types)):
            if ty == T_BYTE and len(t) == 6 and t.startswith("<0x"):
                self.byte_id[int(t[3:5], 16)] = i
        special = [t for i, t in enumerate(self.tokens) if self.types[i] in (T_CONTROL, T_USER) and t]
        special.sort(key=len, reverse=True)
        self.special_re = regex.compile("|".join(regex.escape(t) for t in special)) if special else None

    def _encode_plain(self, text: str) -> List[int]:
        if not text:
            return []
        text = text.replace(" ", "▁")
        syms = list(text)
        n = len(syms)
        prev = list(range(-1, n - 1))
        nxt = list(range(1, n + 1))
        nxt[-1] = -1
        alive = [True] * n
        heap = []

        def try_add(i, j):
            if i < 0 or j < 0:
                return
            t = self.id_of.get(syms[i] + syms[j])
            if t is not None:
                heapq.heappush(heap, (-self.scores[t], i, j, syms[i] + syms[j]))

        for i in range(n - 1):
            try_add(i, i + 1)
        while heap:
            _, i, j, merged = heapq.heappop(heap)
            if not (alive[i] and alive[j]) or syms[i] + syms[j] != merged or nxt[i] != j:
                continue
            syms[i] = merged
            alive[j] = False
            nxt[i] = nxt[j]
            if nxt[j] >= 0:
                prev[nxt[j]] = i
            try_add(prev[i], i)
            try_add(i, nxt[i])
        ids = []
        i = 0
        while i >= 0:
            t = self.id_of.get(syms[i])
            if t is not None:
                ids.append(t)
            else:
                for b in syms[i].encode("utf-8"):
                    ids.append(self.byte_id.get(b, 0))
            i = nxt[i]
        return ids

    def encode(self, text, parse_special=True, add_bos=None):
        ids: List[int] = []
        if (self.add_bos if add_bos is None else add_bos) and self.bos_id >= 0:
            ids.append(self.bos_id)
        first = True
        segs = []
        if parse_special and self.special_re is not None:
            pos = 0
            for m in self.special_re.finditer(text):
                if m.start() > pos:
                    segs.append((text[pos:m.start()], False))
                segs.append((m.group(0), True))
                pos = m.end()
            if pos < len(text):
                segs.append((text[pos:], False))
        else:
            segs.append((text, False))
        for s, is_special in segs:
            if is_special:
                ids.append(self.id_of[s])
            else:
                ids += self._encode_plain((" " + s) if (first and self.space_prefix) else s)
            first = False
        return ids

    def token_bytes(self, tid):
        if not 0 <= tid < self.n_vocab:
            return b""
        ty, t = self.types[tid], self.tokens[tid]
        if ty == T_BYTE:
            return bytes([int(t[3:5], 16)])
        return t.replace("▁", " ").encode("utf-8")

    def is_control(self, tid):
        return 0 <= tid < self.n_vocab and self.types[tid] == T_CONTROL


def from_gguf(g, fallback_vocab: int = 0) -> Tokenizer:
    """Build the tokenizer a GGUF header describes; a header without one gives bytes."""
    model = g.get("tokenizer.ggml.model")
    tokens = g.get("tokenizer.ggml.tokens")
    if not model or tokens is None:
        return ByteTokenizer(fallback_vocab)
    types = g.get("tokenizer.ggml.token_type")
    types = [int(t) for t in types] if types is not None else [T_NORMAL] * len(tokens)
    bos = int(g.get("tokenizer.ggml.bos_token_id", -1))
    eos = int(g.get("tokenizer.ggml.eos_token_id", -1))
    eot = int(g.get("tokenizer.ggml.eot_token_id", -1))
    add_bos = bool(g.get("tokenizer.ggml.add_bos_token", model == "llama"))
    if model == "gpt2":
        return BpeTokenizer(tokens, g.get("tokenizer.ggml.merges") or [], types, str(g.get("tokenizer.ggml.pre", "default")),
                            bos, eos, eot, add_bos)
    if model == "llama":
        scores = g.get("tokenizer.ggml.scores")
        scores = [float(s) for s in scores] if scores is not None else [0.0] * len(tokens)
        return SpmTokenizer(tokens, scores, types, bos, eos, add_bos, bool(g.get("tokenizer.ggml.add_space_prefix", True)))
    raise ValueError(f"tokenizer model {model!r} is not supported")


def from_folder(path: str, fallback_vocab: int = 0) -> Tokenizer:
    """Tokenizer of a checkpoint folder: ``tokenizer.json`` (byte-level BPE: vocab, merges, added tokens) with
    ids of BOS/EOS from ``tokenizer_config.json`` / ``config.json``; a folder without one gives bytes."""
    import json
    import os
    tj = os.path.join(path, "tokenizer.json")
    if not os.path.exists(tj):
        return ByteTokenizer(fallback_vocab)
    doc = json.load(open(tj, encoding="utf-8"))
    model = doc.get("model") or {}
    if str(model.get("type", "BPE")) != "BPE":
        raise ValueError(f"tokenizer.json model type {model.get('type')!r} is not supported")
    vocab = model.get("vocab") or {}
    n = max(list(vocab.values()) + [a["id"] for a in doc.get("added_tokens", [])] + [-1]) + 1
    n = max(n, fallback_vocab)
    tokens = [f"[unused{i}]" for i in range(n)]
    types = [T_UNUSED if "T_UNUSED" in globals() else T_NORMAL] * n
    for tok, i in vocab.items():
        tokens[i], types[i] = tok, T_NORMAL
    for a in doc.get("added_tokens", []):
        tokens[a["id"]] = a["content"]
        types[a["id"]] = T_CONTROL if a.get("special") else T_USER if "T_USER" in globals() else T_NORMAL
    merges = [m if isinstance(m, str) else " ".join(m) for m in model.get("merges", [])]
    ids = {t: i for i, t in enumerate(tokens)}
    cfg = {}
    for fn in ("tokenizer_config.json", "config.json"):
        fp = os.path.join(path, fn)
        if os.path.exists(fp):
            for k, v in json.load(open(fp, encoding="utf-8")).items():
                cfg.setdefault(k, v)

    def tid(key: str) -> int:
        v = cfg.get(key + "_id", cfg.get(key))
        if isinstance(v, dict):
            v = v.get("content")
        if isinstance(v, list):
            v = v[0] if v else None
        if isinstance(v, int):
            return v
        return ids.get(v, -1) if isinstance(v, str) else -1

    pre = "default"
    blob = json.dumps(doc.get("pre_tokenizer") or {})
    if "\\p{N}{1,3}" in blob:
        pre = "llama-bpe"
    elif "\\p{N}" in blob and "(?i:'s|'t|'re|'ve|'m|'ll|'d)" in blob:
        pre = "qwen2"
    return BpeTokenizer(tokens, merges, types, pre, tid("bos_token"), tid("eos_token"), -1, bool(cfg.get("add_bos_token", False)))
