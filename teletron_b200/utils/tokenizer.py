"""Tokenizers the trainer can be asked for.  The example run uses ``--tokenizer-type NullTokenizer
--vocab-size 0`` (examples/wan/run_wan.sh:74-76): the DiT consumes embeddings, the real text
tokenizer lives with the text encoder (teletron/utils/tokenizer.py:49-91,1103-1134)."""
from __future__ import annotations


class NullTokenizer:
    """Whitespace-separated integers <-> ids; ``vocab_size`` ids plus one EOD."""

    def __init__(self, vocab_size: int):
        self._eod = int(vocab_size)
        self.vocab_size = self._eod + 1

    def tokenize(self, text: str):
        return [int(x) for x in text.split()]

    def detokenize(self, ids):
        return " ".join(str(int(i)) for i in ids)

    @property
    def eod(self):
        return self._eod

    @property
    def cls(self):
        return -1

    @property
    def sep(self):
        return -1

    @property
    def mask(self):
        return -1

    @property
    def pad(self):
        return -1


class HFTokenizerWrapper:
    def __init__(self, path: str):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path)
        self.vocab_size = len(self.tok)

    def tokenize(self, text):
        return self.tok(text).input_ids

    def detokenize(self, ids):
        return self.tok.decode(ids)

    @property
    def eod(self):
        return self.tok.eos_token_id


def build_tokenizer(args):
    kind = getattr(args, "tokenizer_type", "NullTokenizer")
    if kind == "NullTokenizer":
        tok = NullTokenizer(getattr(args, "vocab_size", 0) or 0)
    elif kind in ("HuggingFaceTokenizer", "PretrainedFromHF"):
        tok = HFTokenizerWrapper(args.tokenizer_model)
    else:
        raise NotImplementedError(f"tokenizer type {kind} is not provided; use NullTokenizer or HuggingFaceTokenizer")
    args.padded_vocab_size = tok.vocab_size
    return tok
