from .config import Config  # noqa: F401
from .flops import memory_report, theoretical_memory_gb, wan_flops_per_sample  # noqa: F401
from .prompt import clean_caption  # noqa: F401
from .tokenizer import NullTokenizer, build_tokenizer  # noqa: F401
