"""Tokenizers: a wrapper over a HF ``tokenizer.json`` directory and a byte-level fallback.

The fallback (``ByteTokenizer``) needs no files: ids 0..255 are bytes, followed by the special
tokens of the built-in chat template. It lets the server, the CLI and the tests run with
random-init weights. Reference counterpart: ``crates/models/src/tokenizer.rs``.
"""
from __future__ import annotations

import re


class ByteTokenizer:
    SPECIALS = ["<|im_start|>", "<|im_end|>", "<|endoftext|>", "<think>", "</think>", "<tool_call>", "</tool_call>",
                "<|image_pad|>", "<|vision_start|>", "<|vision_end|>"]

    def __init__(self, vocab_size: int = 512):
        self.vocab_size = vocab_size
        self.special_ids = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.id_special = {v: k for k, v in self.special_ids.items()}
        self.eos_ids = [self.special_ids["<|im_end|>"], self.special_ids["<|endoftext|>"]]
        self.image_pad_id = self.special_ids["<|image_pad|>"]
        self._split = re.compile("(" + "|".join(re.escape(x) for x in self.SPECIALS) + ")")

    def encode(self, text: str) -> list[int]:
        out = []
        for part in self._split.split(text):              # specials (leftmost first, list order on a tie) and the text between
            sid = self.special_ids.get(part)
            if sid is not None:
                out.append(sid)
            elif part:
                out.extend(part.encode("utf-8"))
        return out

    def decode(self, ids) -> str:
        buf, out = bytearray(), []
        for t in ids:
            if t < 256:
                buf.append(t)
            else:
                out.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
                out.append(self.id_special.get(t, ""))
        out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)


class HfTokenizer:
    def __init__(self, path: str):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path)
        self.vocab_size = len(self.tok)
        eos = self.tok.eos_token_id
        self.eos_ids = [eos] if isinstance(eos, int) else list(eos or [])
        self.image_pad_id = self.tok.convert_tokens_to_ids("<|image_pad|>")

    def encode(self, text: str) -> list[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def decode(self, ids) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=False)


class StreamDecoder:
    """Incremental detokenisation that never emits half of a multi-byte character.

    Each token decodes a short window of ids, not the whole answer: ``ids[prefix:read]`` is the part of the window whose text
    is already out, and the new text is what decoding ``ids[prefix:]`` adds to it (a tokenizer may render a token differently
    after its neighbours -- a leading space, a merged byte pair -- so the window keeps the previous emission as context).
    The window moves up only when text was emitted, so it always starts where a character ended; a long answer costs the
    same per token as a short one."""

    def __init__(self, tok):
        self.tok, self.ids = tok, []
        self.prefix = self.read = 0

    def push(self, token: int) -> str:
        self.ids.append(token)
        done = self.tok.decode(self.ids[self.prefix:self.read])
        full = self.tok.decode(self.ids[self.prefix:])
        if len(full) <= len(done) or full.endswith("\ufffd"):
            return ""                                   # nothing new yet, or the last character is still incomplete
        self.prefix, self.read = self.read, len(self.ids)
        return full[len(done):]
