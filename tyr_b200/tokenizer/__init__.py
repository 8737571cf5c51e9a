from .bpe import BPETokenizer, MergeRule, train_bpe, pretokenize, GPT4_SPLIT_PATTERN, DEFAULT_SPECIAL_TOKENS  # noqa: F401
from .hf import HFTokenizer, chatml_prompt, gemma_prompt, load_qwen3, load_qwen35, load_qwen36, load_laguna, load_gemma4  # noqa: F401
