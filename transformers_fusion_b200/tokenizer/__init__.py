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


class BPETokenizer(Tokenizer):
    KIND = 0


class UnigramTokenizer(Tokenizer):
    KIND = 1

    load_sentencepiece_tsv = Tokenizer.load
    save_sentencepiece_tsv = Tokenizer.save


class Qwen35Tokenizer(Tokenizer):
    """Byte-level BPE from a model directory; ``apply_chat_template`` builds the ChatML prompt."""
    KIND = 2

    @classmethod
    def load_from_dir(cls, path):
        return cls().load(path)

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
