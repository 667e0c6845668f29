"""Byte-level tokenizer used with model presets (no tokenizer files needed).

ids 0..255 are raw bytes; ids 256..vocab-2 map to single private code points so that text
round-trips through encode/decode; id vocab-1 is EOS.  It implements the small part of the
HuggingFace tokenizer interface the engine uses (encode, decode, apply_chat_template,
eos_token_id, all_special_ids, __len__).
"""
from __future__ import annotations

_BASE = 0xE000   # private-use area


class ByteTokenizer:
    def __init__(self, vocab_size: int = 1024):
        if vocab_size < 258:
            raise ValueError("vocab_size must be at least 258")
        self.vocab_size = vocab_size
        self.eos_token_id = vocab_size - 1
        self.eos_token = "<|eos|>"
        self.pad_token_id = self.eos_token_id
        self.all_special_ids = [self.eos_token_id]
        self._extra = min(vocab_size - 257, 0x1900)      # ids that have a private code point

    def __len__(self):
        return self.vocab_size

    def encode(self, text: str, add_special_tokens: bool = True) -> list:
        out = []
        for ch in text:
            cp = ord(ch)
            if _BASE <= cp < _BASE + self._extra:
                out.append(256 + cp - _BASE)
            else:
                out.extend(ch.encode("utf-8"))
        return out

    def __call__(self, text, **kw):
        return {"input_ids": self.encode(text)}

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        if isinstance(ids, int):
            ids = [ids]
        parts, buf = [], bytearray()

        def flush():
            if buf:
                parts.append(buf.decode("utf-8", errors="replace"))
                buf.clear()
        for i in ids:
            i = int(i)
            if 0 <= i < 256:
                buf.append(i)
                continue
            flush()
            if i == self.eos_token_id:
                if not skip_special_tokens:
                    parts.append(self.eos_token)
            elif 256 <= i < 256 + self._extra:
                parts.append(chr(_BASE + i - 256))
            else:
                parts.append("")
        flush()
        return "".join(parts)

    def convert_ids_to_tokens(self, ids):
        return [self.decode([i], skip_special_tokens=False) for i in ids]

    def apply_chat_template(self, messages, tokenize: bool = False, add_generation_prompt: bool = True, **kw):
        text = "".join(f"<|{m.get('role', 'user')}|>\n{m.get('content', '')}\n" for m in messages)
        if add_generation_prompt:
            text += "<|assistant|>\n"
        return self.encode(text) if tokenize else text


def load_tokenizer(config):
    """Tokenizer for a Config: byte-level for presets, AutoTokenizer for a local model directory."""
    import os
    spec = config.tokenizer
    if spec == "byte" or (spec == "auto" and not os.path.isdir(config.model)):
        return ByteTokenizer(config.model_config.vocab_size)
    from transformers import AutoTokenizer
    path = config.model if spec == "auto" else spec
    try:
        return AutoTokenizer.from_pretrained(path, trust_remote_code=False)
    except Exception:
        if spec == "auto":
            return ByteTokenizer(config.model_config.vocab_size)
        raise
