"""Tokenizers (native: ``libtfb_tokenizer``): trainable byte-pair, unigram (Viterbi, SentencePiece TSV)
and byte-level BPE loaded from a Hugging Face ``vocab.json`` + ``merges.txt`` (Qwen-style, with the
ChatML chat template).

Interface parity with the reference's ``Tokenizer`` (include/quant/tokenizer.h:10-57): ``encode``,
``decode``, ``vocab_size``, ``bos_id`` (1), ``eos_id`` (2), ``train``, ``save``, ``load``."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        p = Path(__file__).resolve().parent.parent / "lib" / "libtfb_tokenizer.so"
        if not p.exists():
            from .. import build
            build.build_host_lib("tfb_tokenizer", "tokenizer")
        L = C.CDLL(str(p))
        L.tfb_tok_new.restype = C.c_void_p
        L.tfb_tok_new.argtypes = [C.c_int]
        L.tfb_tok_free.argtypes = [C.c_void_p]
        L.tfb_tok_train.argtypes = [C.c_void_p, C.c_char_p, C.c_longlong, C.c_int]
        for n in ("tfb_tok_vocab_size", "tfb_tok_bos", "tfb_tok_eos"):
            getattr(L, n).argtypes = [C.c_void_p]
        L.tfb_tok_encode.restype = C.c_longlong
        L.tfb_tok_encode.argtypes = [C.c_void_p, C.c_char_p, C.c_longlong, C.c_void_p, C.c_longlong]
        L.tfb_tok_decode.restype = C.c_longlong
        L.tfb_tok_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_longlong]
        L.tfb_tok_save.argtypes = [C.c_void_p, C.c_char_p]
        L.tfb_tok_load.argtypes = [C.c_void_p, C.c_char_p]
        L.tfb_tok_token_to_id.argtypes = [C.c_void_p, C.c_char_p]
        _LIB = L
    return _LIB


class Tokenizer:
    KIND = 0

    def __init__(self):
        self._h = _lib().tfb_tok_new(self.KIND)

    def __del__(self):
        if getattr(self, "_h", None):
            _lib().tfb_tok_free(self._h)
            self._h = None

    def train(self, texts, vocab_size=32000):
        data = ("\n".join(texts) if not isinstance(texts, str) else texts).encode("utf-8", "ignore")
        if _lib().tfb_tok_train(self._h, data, len(data), vocab_size) != 0:
            raise ValueError("this tokenizer is not trainable")
        return self

    def encode(self, text: str, add_bos=False, add_eos=False):
        data = text.encode("utf-8", "ignore")
        cap = len(data) + 16
        buf = (C.c_int * cap)()
        n = _lib().tfb_tok_encode(self._h, data, len(data), buf, cap)
        ids = list(buf[: min(n, cap)])
        if add_bos and self.bos_id >= 0:
            ids = [self.bos_id] + ids
        if add_eos and self.eos_id >= 0:
            ids = ids + [self.eos_id]
        return ids

    def decode(self, ids) -> str:
        ids = [int(i) for i in ids]
        arr = (C.c_int * max(1, len(ids)))(*ids)
        cap = 64 * len(ids) + 64
        buf = C.create_string_buffer(cap)
        n = _lib().tfb_tok_decode(self._h, arr, len(ids), buf, cap)
        return buf.raw[: min(n, cap)].decode("utf-8", "replace")

    @property
    def vocab_size(self):
        return _lib().tfb_tok_vocab_size(self._h)

    @property
    def bos_id(self):
        return _lib().tfb_tok_bos(self._h)

    @property
    def eos_id(self):
        return _lib().tfb_tok_eos(self._h)

    def save(self, path):
        if _lib().tfb_tok_save(self._h, str(path).encode()) != 0:
            raise IOError(f"cannot save tokenizer to {path}")

    def load(self, path):
        if _lib().tfb_tok_load(self._h, str(path).encode()) != 0:
            raise IOError(f"cannot load tokenizer from {path}")
        return self

    def token_to_id(self, tok: str) -> int:
        return _lib().tfb_tok_token_to_id(self._h, tok.encode())

    def id_to_token(self, i: int) -> str:
        L = _lib()
        L.tfb_tok_id_to_token.restype = C.c_longlong
        L.tfb_tok_id_to_token.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_longlong]
        buf = C.create_string_buffer(512)
        n = L.tfb_tok_id_to_token(self._h, int(i), buf, 512)
        if n < 0:
            raise IndexError(i)
        return buf.raw[: min(n, 512)].decode("utf-8", "replace")

    def is_special(self, i: int) -> bool:
        L = _lib()
        L.tfb_tok_is_special.argtypes = [C.c_void_p, C.c_int]
        return bool(L.tfb_tok_is_special(self._h, int(i)))


class BPETokenizer(Tokenizer):
    KIND = 0


class UnigramTokenizer(Tokenizer):
    KIND = 1
    MARK = "\u2581"                       # the word-start marker of SentencePiece

    load_sentencepiece_tsv = Tokenizer.load
    save_sentencepiece_tsv = Tokenizer.save

    # ---- SentencePiece-flavoured verbs (reference: UnigramTokenizer, include/quant/bpe_tokenizer.h)
    def _set_special(self, which: int, i: int):
        L = _lib()
        L.tfb_tok_set_special.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.tfb_tok_set_special.restype = None
        L.tfb_tok_set_special(self._h, which, int(i))
        setattr(self, ("_unk", "_bos", "_eos")[which], int(i))

    def set_unk_id(self, i: int): self._set_special(0, i)
    def set_bos_id(self, i: int): self._set_special(1, i)
    def set_eos_id(self, i: int): self._set_special(2, i)

    @property
    def unk_id(self): return getattr(self, "_unk", 0)

    @property
    def bos_id(self): return getattr(self, "_bos", 1)

    @property
    def eos_id(self): return getattr(self, "_eos", 2)

    def piece_score(self, i: int) -> float:
        L = _lib()
        L.tfb_tok_piece_score.restype = C.c_double
        L.tfb_tok_piece_score.argtypes = [C.c_void_p, C.c_int]
        return float(L.tfb_tok_piece_score(self._h, int(i)))

    @classmethod
    def sentencepiece_normalize(cls, text: str) -> str:
        """Whitespace runs become one word-start marker each, and the text starts with one: "a  b" -> "\u2581a\u2581b"."""
        return cls.MARK + cls.MARK.join(text.split()) if text.split() else ""

    @classmethod
    def sentencepiece_join(cls, pieces) -> str:
        """Pieces back to text: markers become spaces, the leading one is dropped."""
        return "".join(pieces).replace(cls.MARK, " ").lstrip(" ")

    encode_sentencepiece = Tokenizer.encode

    def decode_sentencepiece(self, ids) -> str:
        return self.sentencepiece_join(self.id_to_token(i) for i in ids if i not in (self.bos_id, self.eos_id))

    def encode_with_scores(self, text: str):
        """(ids, log-probability of each piece) of the best segmentation."""
        L = _lib()
        L.tfb_tok_encode_scores.restype = C.c_longlong
        L.tfb_tok_encode_scores.argtypes = [C.c_void_p, C.c_char_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_longlong]
        data = text.encode("utf-8", "ignore")
        cap = len(data) + 16
        ids, sc = (C.c_int * cap)(), (C.c_double * cap)()
        n = L.tfb_tok_encode_scores(self._h, data, len(data), ids, sc, cap)
        return list(ids[:n]), list(sc[:n])

    def encode_nbest(self, text: str, n: int = 5):
        """The ``n`` most probable segmentations, best first, as lists of ids (k-best Viterbi over the piece lattice)."""
        s = self.sentencepiece_normalize(text)
        if not s:
            return [[]]
        pieces = {}
        for i in range(self.vocab_size):
            t = self.id_to_token(i)
            if t and i not in (self.unk_id, self.bos_id, self.eos_id):
                pieces[t] = (i, self.piece_score(i))
        max_len = max((len(t) for t in pieces), default=1)
        L_ = len(s)
        best = [[] for _ in range(L_ + 1)]          # best[j]: up to n (score, ids) ending at character j
        best[0] = [(0.0, [])]
        for j in range(1, L_ + 1):
            cand = []
            for i in range(max(0, j - max_len), j):
                if not best[i]:
                    continue
                hit = pieces.get(s[i:j])
                if hit is None and j - i == 1:
                    hit = (self.unk_id, -20.0)       # unknown character
                if hit is not None:
                    cand += [(sc + hit[1], ids + [hit[0]]) for sc, ids in best[i]]
            cand.sort(key=lambda c: -c[0])
            best[j] = cand[:n]
        return [ids for _, ids in best[L_]] or [self.encode(text)]


class Qwen35Tokenizer(Tokenizer):
    """Byte-level BPE from a model directory; ``apply_chat_template`` builds the ChatML prompt."""
    KIND = 2

    @classmethod
    def load_from_dir(cls, path):
        return cls().load(path)

    def im_start_id(self) -> int: return self.token_to_id("<|im_start|>")
    def im_end_id(self) -> int: return self.token_to_id("<|im_end|>")

    def apply_chat_template(self, messages, add_generation_prompt=True) -> str:
        out = []
        for m in messages:
            out.append(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n")
        if add_generation_prompt:
            out.append("<|im_start|>assistant\n")
        return "".join(out)


class ByteTokenizer:
    """Dependency-free fallback: UTF-8 bytes shifted past the three special ids."""
    bos_id, eos_id, vocab_size = 1, 2, 259

    def encode(self, text, add_bos=False, add_eos=False):
        ids = [b + 3 for b in text.encode("utf-8", "ignore")]
        return ([1] if add_bos else []) + ids + ([2] if add_eos else [])

    def decode(self, ids):
        return bytes(i - 3 for i in ids if 3 <= i < 259).decode("utf-8", "replace")


class WordPieceTokenizer:
    """Greedy longest-match-first sub-word tokenizer with "##" continuation pieces (the BERT scheme).  Training grows the
    vocabulary by merging the adjacent pair with the highest score count(ab) / (count(a) count(b)).  Reference:
    WordPieceTokenizer, include/quant/bpe_tokenizer.h."""

    def __init__(self):
        self.unk, self.cls, self.sep, self.pad, self.mask = "[UNK]", "[CLS]", "[SEP]", "[PAD]", "[MASK]"
        self.vocab, self.index = [], {}
        self._set_vocab([self.pad, self.unk, self.cls, self.sep, self.mask])

    def _set_vocab(self, vocab):
        self.vocab = list(vocab)
        self.index = {t: i for i, t in enumerate(self.vocab)}

    def set_special_tokens(self, unk, cls, sep, pad, mask):
        old = [self.pad, self.unk, self.cls, self.sep, self.mask]
        self.unk, self.cls, self.sep, self.pad, self.mask = unk, cls, sep, pad, mask
        rest = [t for t in self.vocab if t not in old]
        self._set_vocab([pad, unk, cls, sep, mask] + rest)

    @property
    def vocab_size(self): return len(self.vocab)

    @property
    def bos_id(self): return self.index[self.cls]

    @property
    def eos_id(self): return self.index[self.sep]

    @property
    def unk_id(self): return self.index[self.unk]

    @staticmethod
    def _words(text):
        import re
        return re.findall(r"\w+|[^\w\s]", text.lower())

    def train(self, corpus, vocab_size: int = 30000):
        from collections import Counter
        words = Counter(w for line in ([corpus] if isinstance(corpus, str) else corpus) for w in self._words(line))
        splits = {w: [c if i == 0 else "##" + c for i, c in enumerate(w)] for w in words}
        vocab = set(p for sp in splits.values() for p in sp)
        specials = [self.pad, self.unk, self.cls, self.sep, self.mask]
        while len(vocab) + len(specials) < vocab_size:
            pair, single = Counter(), Counter()
            for w, sp in splits.items():
                for p in sp:
                    single[p] += words[w]
                for a, b in zip(sp, sp[1:]):
                    pair[(a, b)] += words[w]
            if not pair:
                break
            (a, b), _ = max(pair.items(), key=lambda kv: (kv[1] / (single[kv[0][0]] * single[kv[0][1]]), kv[1], kv[0]))
            merged = a + b[2:]
            vocab.add(merged)
            for w, sp in splits.items():
                i, out = 0, []
                while i < len(sp):
                    if i + 1 < len(sp) and sp[i] == a and sp[i + 1] == b:
                        out.append(merged)
                        i += 2
                    else:
                        out.append(sp[i])
                        i += 1
                splits[w] = out
        self._set_vocab(specials + sorted(vocab))
        return self

    def encode(self, text: str, add_bos=False, add_eos=False):
        ids = []
        for w in self._words(text):
            start, piece_ids = 0, []
            while start < len(w):
                end, cur = len(w), None
                while end > start:
                    sub = ("##" if start else "") + w[start:end]
                    if sub in self.index:
                        cur = self.index[sub]
                        break
                    end -= 1
                if cur is None:
                    piece_ids = [self.unk_id]        # a word with an unknown part is unknown as a whole
                    break
                piece_ids.append(cur)
                start = end
            ids += piece_ids
        return ([self.bos_id] if add_bos else []) + ids + ([self.eos_id] if add_eos else [])

    def decode(self, ids) -> str:
        out = []
        for i in ids:
            t = self.vocab[i] if 0 <= i < len(self.vocab) else self.unk
            if t in (self.pad, self.cls, self.sep):
                continue
            if t.startswith("##") and out:
                out[-1] += t[2:]
            else:
                out.append(t)
        return " ".join(out)

    def save(self, path):
        with open(path, "w", encoding="utf-8") as f:
            f.write("\n".join(self.vocab) + "\n")

    def load(self, path):
        self._set_vocab([ln.rstrip("\n") for ln in open(path, encoding="utf-8") if ln.rstrip("\n")])
        self.pad, self.unk, self.cls, self.sep, self.mask = self.vocab[:5]
        return self
