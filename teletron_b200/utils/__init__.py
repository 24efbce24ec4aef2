from .config import Config  # noqa: F401
from .flops import memory_report, theoretical_memory_gb, wan_flops_per_sample  # noqa: F401
from .prompt import apply_clean_mode, canonicalize, clean_caption, clean_prompt, tokenize_long_prompt  # noqa: F401
from .tokenizer import NullTokenizer, build_tokenizer  # noqa: F401
