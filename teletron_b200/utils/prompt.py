"""Caption / prompt normalisation before tokenisation.

``clean_prompt`` applies the web-caption rules of the reference (teletron/utils/prompt.py:9-140): URL and
@handle removal, CJK blocks, dash and quote unification, IP addresses, ids, file names, shop phrases,
size strings, punctuation runs.  Here the rules are data: two tables of pre-compiled ``(pattern,
replacement)`` pairs applied in order around the unicode / HTML repair step, so a caller can inspect,
extend or time them, and nothing is re-compiled per call.  ``basic_clean`` / ``whitespace_clean`` /
``canonicalize`` are the tokenizer-side cleaners of the Wan prompter (teletron/models/wan/encoder/
wan_prompter.py:13-35); ``apply_clean_mode`` selects among them by name as its tokenizer wrapper does
(wan_prompter.py:76-84).  ``ftfy`` is used when installed.
"""
from __future__ import annotations

import html
import re
import string
import urllib.parse
from typing import List, Optional, Tuple

_DOMAIN = r"[a-zA-Z0-9.\-]+[.](?:com|co|ru|net|org|edu|gov|it)[\w/-]*\b\/?(?!@)"
_MEDIA_EXT = r"(?:png|jpg|jpeg|bmp|webp|eps|pdf|apk|mp4)"
# unicode blocks dropped wholesale: CJK strokes, katakana extensions, enclosed CJK, CJK compatibility,
# ideograph extension A, hexagram symbols, unified ideographs
_CJK_BLOCKS = ("\u31c0-\u31ef", "\u31f0-\u31ff", "\u3200-\u32ff", "\u3300-\u33ff", "\u3400-\u4dbf",
               "\u4dc0-\u4dff", "\u4e00-\u9fff")
_DASHES = ("\u002D\u058A\u05BE\u1400\u1806\u2010-\u2015\u2E17\u2E1A\u2E3A\u2E3B\u2E40\u301C\u3030\u30A0"
           "\uFE31\uFE32\uFE58\uFE63\uFF0D")
_PUNCT_RUN = r"[#®•©™&@·º½¾¿¡§~\)\(\]\[\}\{\|\\\/\*]{1,}"


def _table(rules) -> List[Tuple[re.Pattern, str]]:
    return [(re.compile(p), r) for p, r in rules]


# applied in this order to the lower-cased, url-unquoted caption, before unicode / entity repair
_LEAD = _table(
    [("<person>", "person"),
     (r"\b((?:https?:(?:\/{1,3}|[a-zA-Z0-9%])|" + _DOMAIN + "))", ""),
     (r"\b((?:www:(?:\/{1,3}|[a-zA-Z0-9%])|" + _DOMAIN + "))", ""),
     (r"@[\w\d]+\b", "")])
_CJK = _table([(f"[{blk}]+", "") for blk in _CJK_BLOCKS])
_BEFORE_REPAIR = _table(
    [(f"[{_DASHES}]+", "-"),
     (r"[`´«»“”¨]", '"'),
     (r"[‘’]", "'"),
     (r"&quot;?", ""),
     (r"&amp", ""),
     (r"\d{1,3}\.\d{1,3}\.\d{1,3}\.\d{1,3}", " "),          # ip addresses
     (r"\d:\d\d\s+$", ""),                                    # trailing article ids
     (r"\\n", " "),
     (r"#\d{1,3}\b", ""),
     (r"#\d{5,}\b", ""),
     (r"\b\d{6,}\b", ""),
     (r"[\S]+\." + _MEDIA_EXT, ""),                           # file names
     (r"[\"\']{2,}", '"'),
     (r"[\.]{2,}", " "),
     (_PUNCT_RUN, " "),
     (r"\s+\.\s+", " ")])

# applied after the repair step
_AFTER_REPAIR = _table(
    [(r"\b[a-zA-Z]{1,3}\d{3,15}\b", ""),                        # jc6640
     (r"\b[a-zA-Z]+\d+[a-zA-Z]+\b", ""),                        # jc6640vc
     (r"\b\d+[a-zA-Z]+\d+\b", ""),                              # 6640vc231
     (r"(worldwide\s+)?(free\s+)?shipping", ""),
     (r"(free\s)?download(\sfree)?", ""),
     (r"\bclick\b\s(?:for|on)\s\w+", ""),
     (r"\b" + _MEDIA_EXT + r"(\simage[s]?)?", ""),
     (r"\bpage\s+\d+\b", ""),
     (r"\b\d*[a-zA-Z]+\d+[a-zA-Z]+\d+[a-zA-Z\d]*\b", " "),      # j2d1a2a...
     (r"\b\d+\.?\d*[xх×]\d+\.?\d*\b", ""),                      # 1920x1080
     (r"\b\s+\:\s+", ": "),
     (r"(\D[,\./])\b", r"\1 "),
     (r"\s+", " "),
     (r"^[\"\']([\w\W]+)[\"\']$", r"\1"),
     (r"^[\'\_,\-\:;]", ""),
     (r"[\'\_,\-\:\-\+]$", ""),
     (r"^\.\S+$", "")])

_WORD_JOINERS = re.compile(r"(?:\-|\_)")


def basic_clean(text: str) -> str:
    """Unicode repair (when ``ftfy`` is installed) and double HTML-entity unescape."""
    try:
        import ftfy

        text = ftfy.fix_text(text)
    except ImportError:
        pass
    return html.unescape(html.unescape(text)).strip()


def whitespace_clean(text: str) -> str:
    return re.sub(r"\s+", " ", text).strip()


def canonicalize(text: str, keep_punctuation_exact_string: Optional[str] = None) -> str:
    """Lower-case, underscores to spaces, punctuation dropped (except inside the given marker string)."""
    text = text.replace("_", " ")
    strip = str.maketrans("", "", string.punctuation)
    if keep_punctuation_exact_string:
        text = keep_punctuation_exact_string.join(p.translate(strip) for p in text.split(keep_punctuation_exact_string))
    else:
        text = text.translate(strip)
    return whitespace_clean(text.lower())


def apply_clean_mode(text: str, mode: Optional[str]) -> str:
    """``None`` (no change), ``"whitespace"``, ``"lower"`` or ``"canonicalize"``."""
    if mode is None:
        return text
    if mode == "whitespace":
        return whitespace_clean(basic_clean(text))
    if mode == "lower":
        return whitespace_clean(basic_clean(text)).lower()
    if mode == "canonicalize":
        return canonicalize(basic_clean(text))
    raise ValueError(f"unknown clean mode {mode!r}")


def clean_prompt(prompt, keep_cjk: bool = False) -> str:
    """Normalised caption.  ``keep_cjk`` leaves the CJK blocks in place (the reference always drops them,
    which empties Chinese prompts although umT5 is multilingual)."""
    c = urllib.parse.unquote_plus(str(prompt)).strip().lower()
    for pat, repl in _LEAD + ([] if keep_cjk else _CJK) + _BEFORE_REPAIR:
        c = pat.sub(repl, c)
    if len(_WORD_JOINERS.findall(c)) > 3:                       # this-is-my-cute-cat / this_is_my_cute_cat
        c = _WORD_JOINERS.sub(" ", c)
    c = basic_clean(c)
    for pat, repl in _AFTER_REPAIR:
        c = pat.sub(repl, c)
    return c.strip()


clean_caption = clean_prompt


def tokenize_long_prompt(tokenizer, prompt: str, max_length: Optional[int] = None):
    """Token ids of a prompt longer than the tokenizer's window as ``[n_chunks, window]`` rows (padded), for
    text encoders that are run once per window (teletron/models/wan/encoder/base_prompter.py:7-37)."""
    window = tokenizer.model_max_length if max_length is None else max_length
    saved = tokenizer.model_max_length
    tokenizer.model_max_length = 1 << 30                        # silence the over-length warning of the probe pass
    try:
        n_tok = tokenizer(prompt, return_tensors="pt").input_ids.shape[1]
    finally:
        tokenizer.model_max_length = saved
    total = (n_tok + window - 1) // window * window
    ids = tokenizer(prompt, return_tensors="pt", padding="max_length", max_length=total, truncation=True).input_ids
    return ids.reshape(total // window, window)
