"""Tokenizer handle: HF ``tokenizer.json`` (via the ``tokenizers`` package), a BPE tokenizer rebuilt from the
vocabulary and merges embedded in a GGUF file, or a byte-level fallback for synthetic models.

Reference parity: ``TokenizerHandle`` with ``encode / encode_pair / decode``, eos/bos resolution, GGUF rebuild
(src/tokenizer.rs:23-250).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import List, Optional, Sequence


class TokenizerHandle:
    def __init__(self, backend, bos_id: Optional[int] = None, eos_id: Optional[int] = None, pad_id: int = 0,
                 sep_id: Optional[int] = None, cls_id: Optional[int] = None):
        self._tk = backend
        self.bos_id, self.eos_id, self.pad_id, self.sep_id, self.cls_id = bos_id, eos_id, pad_id, sep_id, cls_id

    # ------------------------------------------------------------------------------------------
    @staticmethod
    def from_file(path, **kw) -> "TokenizerHandle":
        from tokenizers import Tokenizer
        tk = Tokenizer.from_file(str(path))
        h = TokenizerHandle(tk, **kw)
        d = Path(path).parent
        for name in ("tokenizer_config.json", "special_tokens_map.json", "generation_config.json", "config.json"):
            f = d / name
            if f.exists():
                try:
                    h._absorb_special(json.loads(f.read_text()))
                except Exception:
                    pass
        return h

    def _absorb_special(self, cfg: dict):
        def tok_id(v):
            if isinstance(v, int):
                return v
            if isinstance(v, dict):
                v = v.get("content")
            if isinstance(v, str):
                return self._tk.token_to_id(v)
            if isinstance(v, list) and v:
                return tok_id(v[0])
            return None
        for key, attr in (("eos_token", "eos_id"), ("bos_token", "bos_id"), ("pad_token", "pad_id"),
                          ("sep_token", "sep_id"), ("cls_token", "cls_id"), ("eos_token_id", "eos_id"),
                          ("bos_token_id", "bos_id"), ("pad_token_id", "pad_id")):
            if key in cfg and getattr(self, attr) in (None, 0):
                v = tok_id(cfg[key])
                if v is not None:
                    setattr(self, attr, v)

    @staticmethod
    def from_gguf(gguf) -> "TokenizerHandle":
        """Rebuild from ``tokenizer.ggml.tokens`` / ``merges`` (BPE models) or a unigram-free word-piece table."""
        tokens = gguf.tokenizer_tokens()
        if tokens is None:
            raise ValueError("the GGUF file has no embedded tokenizer")
        merges = gguf.tokenizer_merges() or []
        model = str(gguf.get("tokenizer.ggml.model", "gpt2"))
        vocab = {t: i for i, t in enumerate(tokens)}
        from tokenizers import Tokenizer, decoders, models, pre_tokenizers
        if model in ("gpt2", "llama-bpe", "bpe") or merges:
            pairs = [tuple(m.split(" ", 1)) for m in merges if " " in m]
            tk = Tokenizer(models.BPE(vocab=vocab, merges=pairs, fuse_unk=True))
            tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
            tk.decoder = decoders.ByteLevel()
        else:
            tk = Tokenizer(models.WordPiece(vocab=vocab, unk_token=tokens[int(gguf.get("tokenizer.ggml.unknown_token_id", 0))]))
            tk.pre_tokenizer = pre_tokenizers.BertPreTokenizer()
            tk.decoder = decoders.WordPiece()
        g = lambda k: (int(gguf.get(k)) if gguf.get(k) is not None else None)
        return TokenizerHandle(tk, bos_id=g("tokenizer.ggml.bos_token_id"), eos_id=g("tokenizer.ggml.eos_token_id"),
                               pad_id=g("tokenizer.ggml.padding_token_id") or 0,
                               sep_id=g("tokenizer.ggml.seperator_token_id"), cls_id=g("tokenizer.ggml.cls_token_id"))

    @staticmethod
    def byte_level(vocab_size: int = 256 + 3) -> "TokenizerHandle":
        return TokenizerHandle(_ByteTokenizer(vocab_size), bos_id=256, eos_id=257, pad_id=258)

    # ------------------------------------------------------------------------------------------
    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        enc = self._tk.encode(text, add_special_tokens=add_special_tokens)
        return list(enc.ids)

    def encode_pair(self, a: str, b: str) -> List[int]:
        """Cross-encoder input: ``[CLS] a [SEP] b [SEP]`` when the tokenizer defines those, else ``a b``."""
        if isinstance(self._tk, _ByteTokenizer):
            return self._tk.encode(a + " " + b).ids
        try:
            return list(self._tk.encode(a, b).ids)
        except Exception:
            ids = self.encode(a, False)
            if self.sep_id is not None:
                ids = ([self.cls_id] if self.cls_id is not None else []) + ids + [self.sep_id] + self.encode(b, False) + [self.sep_id]
            else:
                ids = ids + self.encode(" " + b, False)
            return ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return self._tk.decode([int(i) for i in ids], skip_special_tokens=skip_special_tokens)

    def token_to_id(self, tok: str) -> Optional[int]:
        return self._tk.token_to_id(tok)

    @property
    def vocab_size(self) -> int:
        return self._tk.get_vocab_size()

    def eos_ids(self, config_eos: Sequence[int] = ()) -> List[int]:
        """EOS resolution order of the reference: tokenizer -> config -> bos -> 0
        (src/engine/executor_compile.rs:480-495)."""
        if self.eos_id is not None:
            return sorted({self.eos_id, *config_eos})
        if config_eos:
            return list(config_eos)
        return [self.bos_id if self.bos_id is not None else 0]


class _Enc:
    def __init__(self, ids):
        self.ids = ids


class _ByteTokenizer:
    """UTF-8 bytes as tokens 0..255 (+ bos/eos/pad); tokens beyond the table decode to nothing."""

    def __init__(self, vocab_size):
        self.n = vocab_size

    def encode(self, text, pair=None, add_special_tokens=True):
        if pair is not None:
            text = text + " " + pair
        return _Enc(list(text.encode("utf-8")))

    def decode(self, ids, skip_special_tokens=True):
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", "replace")

    def token_to_id(self, tok):
        b = tok.encode("utf-8")
        return b[0] if len(b) == 1 else None

    def get_vocab_size(self):
        return self.n
