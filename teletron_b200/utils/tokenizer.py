"""Tokenizers the trainer can be asked for.  The example run uses ``--tokenizer-type NullTokenizer
--vocab-size 0`` (examples/wan/run_wan.sh:74-76): the DiT consumes embeddings, the real text
tokenizer lives with the text encoder (teletron/utils/tokenizer.py:49-91,1103-1134).  The other
Megatron tokenizer types of ``build_tokenizer`` are provided on top of ``sentencepiece`` and the
``transformers`` WordPiece / byte-level BPE implementations instead of re-implemented."""
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


class SentencePieceTokenizer:
    """SentencePiece model with the special tokens Megatron-style pipelines expect appended when the
    model lacks them (``<CLS> <SEP> <EOD> <MASK>``, pad / bos / eos, then ``vocab_extra_ids`` sentinels
    ``<extra_id_i>``), as the reference wrapper does (teletron/utils/tokenizer.py:847-1010).  ``legacy=False``
    gives the GPT flavour (:1013-1050): no added tokens, EOD = the model's eos."""

    def __init__(self, model_file: str, vocab_extra_ids: int = 0, legacy: bool = True):
        import sentencepiece

        self.sp = sentencepiece.SentencePieceProcessor(model_file=model_file)
        self.vocab = {self.sp.id_to_piece(i): i for i in range(len(self.sp))}
        self.special = {}
        if legacy:
            for name in ("<CLS>", "<SEP>", "<EOD>", "<MASK>"):
                self._add(name)
            self._add(self._piece(self.sp.pad_id(), "<PAD>"))
            self._add(self._piece(self.sp.bos_id(), "<BOS>"))
            self._add(self._piece(self.sp.eos_id(), "<EOS>"))
            for i in range(vocab_extra_ids):
                self._add(f"<extra_id_{i}>")
            self._ids = dict(cls=self.vocab["<CLS>"], sep=self.vocab["<SEP>"], eod=self.vocab["<EOD>"],
                             mask=self.vocab["<MASK>"], pad=self.vocab[self._piece(self.sp.pad_id(), "<PAD>")],
                             bos=self.vocab[self._piece(self.sp.bos_id(), "<BOS>")],
                             eos=self.vocab[self._piece(self.sp.eos_id(), "<EOS>")])
        else:
            self._ids = dict(cls=-1, sep=-1, mask=-1, pad=self.sp.pad_id(), bos=self.sp.bos_id(),
                             eos=self.sp.eos_id(), eod=self.sp.eos_id())
        self.inv_vocab = {i: t for t, i in self.vocab.items()}
        self.vocab_size = len(self.vocab)

    def _piece(self, idx: int, fallback: str) -> str:
        return self.sp.id_to_piece(idx) if 0 <= idx < len(self.sp) else fallback

    def _add(self, token: str):
        if token not in self.vocab:
            self.vocab[token] = len(self.vocab)
        self.special[token] = self.vocab[token]

    def tokenize(self, text: str):
        """Ids of ``text``; added special tokens written literally in the text map to their ids."""
        if not self.special:
            return self.sp.encode_as_ids(text)
        ids, pos = [], 0
        while pos < len(text):
            hits = [(text.find(t, pos), t) for t in self.special if text.find(t, pos) >= 0]
            if not hits:
                break
            at, tok = min(hits)
            ids += self.sp.encode_as_ids(text[pos:at]) + [self.special[tok]]
            pos = at + len(tok)
        return ids + self.sp.encode_as_ids(text[pos:])

    def detokenize(self, ids):
        parts, run = [], []
        for i in map(int, ids):
            if i < len(self.sp):
                run.append(i)
                continue
            if run:
                parts.append(self.sp.decode_ids(run))
                run = []
            parts.append(self.inv_vocab[i])             # an added token: written literally
        if run:
            parts.append(self.sp.decode_ids(run))
        return " ".join(parts)

    cls = property(lambda self: self._ids["cls"])
    sep = property(lambda self: self._ids["sep"])
    mask = property(lambda self: self._ids["mask"])
    pad = property(lambda self: self._ids["pad"])
    bos = property(lambda self: self._ids["bos"])
    eos = property(lambda self: self._ids["eos"])
    eod = property(lambda self: self._ids["eod"])


class Llama2Tokenizer(SentencePieceTokenizer):
    """SentencePiece without added tokens; ``tokenize(text, bos=True, eos=False)`` (:1053-1100)."""

    def __init__(self, model_file: str):
        super().__init__(model_file, legacy=False)

    def tokenize(self, text: str, bos: bool = True, eos: bool = False):
        ids = self.sp.encode_as_ids(text)
        return ([self.bos] if bos else []) + ids + ([self.eos] if eos else [])


class _HFVocabTokenizer:
    """WordPiece / byte-level BPE from vocabulary files, through the ``transformers`` implementations."""

    def __init__(self, tok, eod):
        self.tok, self._eod = tok, eod
        self.vocab_size = len(tok)

    def tokenize(self, text):
        return self.tok.convert_tokens_to_ids(self.tok.tokenize(text))

    def detokenize(self, ids):
        return self.tok.decode([int(i) for i in ids])

    cls = property(lambda self: self.tok.cls_token_id if self.tok.cls_token_id is not None else -1)
    sep = property(lambda self: self.tok.sep_token_id if self.tok.sep_token_id is not None else -1)
    mask = property(lambda self: self.tok.mask_token_id if self.tok.mask_token_id is not None else -1)
    pad = property(lambda self: self.tok.pad_token_id if self.tok.pad_token_id is not None else -1)
    eod = property(lambda self: self._eod)


def vocab_size_with_padding(orig_vocab_size: int, args) -> int:
    """Round the vocabulary up to a multiple of ``make_vocab_size_divisible_by x tensor-parallel size`` so an
    embedding table splits evenly (teletron/utils/tokenizer.py:33-46)."""
    mult = int(getattr(args, "make_vocab_size_divisible_by", 128) or 1) * \
        int(getattr(args, "tensor_model_parallel_size", 1) or 1)
    return (orig_vocab_size + mult - 1) // mult * mult


def build_tokenizer(args):
    kind = getattr(args, "tokenizer_type", "NullTokenizer")
    if kind == "NullTokenizer":
        tok = NullTokenizer(getattr(args, "vocab_size", 0) or 0)
    elif kind in ("HuggingFaceTokenizer", "PretrainedFromHF"):
        tok = HFTokenizerWrapper(args.tokenizer_model)
    elif kind == "SentencePieceTokenizer":
        tok = SentencePieceTokenizer(args.tokenizer_model, vocab_extra_ids=getattr(args, "vocab_extra_ids", 0) or 0)
    elif kind == "GPTSentencePieceTokenizer":
        tok = SentencePieceTokenizer(args.tokenizer_model, legacy=False)
    elif kind == "Llama2Tokenizer":
        tok = Llama2Tokenizer(args.tokenizer_model)
    elif kind in ("BertWordPieceLowerCase", "BertWordPieceCase"):
        from transformers import BertTokenizer

        bert = BertTokenizer(args.vocab_file, do_lower_case=kind.endswith("LowerCase"))
        tok = _HFVocabTokenizer(bert, eod=bert.sep_token_id)
    elif kind == "GPT2BPETokenizer":
        from transformers import GPT2Tokenizer

        gpt2 = GPT2Tokenizer(args.vocab_file, args.merge_file)
        tok = _HFVocabTokenizer(gpt2, eod=gpt2.convert_tokens_to_ids("<|endoftext|>"))
    else:
        raise NotImplementedError(f"unknown tokenizer type {kind}")
    args.padded_vocab_size = tok.vocab_size if kind == "NullTokenizer" else vocab_size_with_padding(tok.vocab_size, args)
    return tok
