from .config import Config, load_config  # noqa: F401
from .flops import (fit_activation_memory, max_trainable_frames, memory_report,  # noqa: F401
                    theoretical_memory_gb, wan_flops_per_sample)
from .prompt import apply_clean_mode, canonicalize, clean_caption, clean_prompt, tokenize_long_prompt  # noqa: F401
from .tokenizer import NullTokenizer, build_tokenizer  # noqa: F401
