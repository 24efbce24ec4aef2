"""Caption cleaning before tokenisation (URLs, HTML, @handles, CJK punctuation runs, IP addresses,
file names, shouting, repeated punctuation...), the normalisation the reference applies to prompts
(teletron/utils/prompt.py:9-140).  ``ftfy`` is used when installed."""
from __future__ import annotations

import html
import re
import urllib.parse

_BAD_PUNCT = re.compile(r"[#®•©™&@·º½¾¿¡§~\)\(\]\[\}\{\|\\/\*]{1,}")


def basic_clean(text: str) -> str:
    try:
        import ftfy

        text = ftfy.fix_text(text)
    except Exception:
        pass
    return html.unescape(html.unescape(text)).strip()


def whitespace_clean(text: str) -> str:
    return re.sub(r"\s+", " ", text).strip()


def clean_caption(caption: str) -> str:
    c = urllib.parse.unquote_plus(str(caption)).strip().lower()
    c = re.sub("<person>", "person", c)
    c = re.sub(r"\b((?:https?:(?:\/{1,3}|[a-zA-Z0-9%])|[a-zA-Z0-9.\-]+[.](?:com|co|ru|net|org|edu|gov|it)[\w/-]*\b\/?(?!@)))", "", c)
    c = re.sub(r"\b((?:www:(?:\/{1,3}|[a-zA-Z0-9%])|[a-zA-Z0-9.\-]+[.](?:com|co|ru|net|org|edu|gov|it)[\w/-]*\b\/?(?!@)))", "", c)
    c = re.sub(r"<[^>]+>", "", c)                       # html tags
    c = re.sub(r"@[\w\d]+\b", "", c)                    # @handles
    c = re.sub(r"[\u31c0-\u31ef\u31f0-\u31ff\u3200-\u32ff\u3300-\u33ff\u3400-\u4dbf\u4dc0-\u4dff]+", "", c)
    c = re.sub(r"[\u2012-\u2015\u2e3a\u2e3b\u2212]+", "-", c)      # dashes
    c = re.sub(r"[`´«»“”¨]", '"', c)
    c = re.sub(r"[‘’]", "'", c)
    c = re.sub(r"&quot;?", "", c)
    c = re.sub(r"&amp", "", c)
    c = re.sub(r"\d{1,3}\.\d{1,3}\.\d{1,3}\.\d{1,3}", " ", c)   # ip addresses
    c = re.sub(r"\d:\d\d\s+$", "", c)                   # trailing article ids
    c = re.sub(r"\\n", " ", c)
    c = re.sub(r"#\d{1,3}\b", "", c)
    c = re.sub(r"#\d{5,}\b", "", c)
    c = re.sub(r"\b\d{6,}\b", "", c)
    c = re.sub(r"[\S]+\.(?:png|jpg|jpeg|bmp|webp|eps|pdf|apk|mp4)", "", c)
    c = re.sub(r"[\"\']{2,}", '"', c)
    c = re.sub(r"[\.]{2,}", " ", c)
    c = _BAD_PUNCT.sub(" ", c)
    c = re.sub(r"\s+\.\s+", " ", c)
    if len(re.findall(r"[\-_]", c)) > 3:
        c = re.sub(r"[\-_]", " ", c)
    c = basic_clean(c)
    c = re.sub(r"\b[a-zA-Z]{1,3}\d{3,15}\b", "", c)
    c = re.sub(r"\b[a-zA-Z]+\d+[a-zA-Z]+\b", "", c)
    c = re.sub(r"\b\d+[a-zA-Z]+\d+\b", "", c)
    c = re.sub(r"(worldwide\s+)?(free\s+)?shipping", "", c)
    c = re.sub(r"(free\s)?download(\sfree)?", "", c)
    c = re.sub(r"\bclick\b\s(?:for|on)\s\w+", "", c)
    c = re.sub(r"\b(?:png|jpg|jpeg|bmp|webp|eps|pdf|apk|mp4)(\simage[s]?)?", "", c)
    c = re.sub(r"\bpage\s+\d+\b", "", c)
    c = re.sub(r"\b\d*[a-zA-Z]+\d+[a-zA-Z]+\d+[a-zA-Z\d]*\b", " ", c)
    c = re.sub(r"\b\d+\.?\d*[xх×]\d+\.?\d*\b", "", c)
    c = re.sub(r"\b\s+\:\s+", r": ", c)
    c = re.sub(r"(\D[,\./])\b", r"\1 ", c)
    c = whitespace_clean(c)
    c = re.sub(r"^[\"\']([\w\W]+)[\"\']$", r"\1", c)
    c = re.sub(r"^[\'\_,\-\:;]", "", c)
    c = re.sub(r"[\'\_,\-\:\-\+]$", "", c)
    c = re.sub(r"^\.\S+$", "", c)
    return c.strip()
