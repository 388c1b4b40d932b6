"""Models and engine (exports follow ``python/triton_dist/models/__init__.py:32-56``)."""
from .config import ARCHS, ArchConfig, ModelConfig
from .engine import Engine
from .kv_cache import KV_Cache
from .qwen import Qwen3
from .utils import logger, sample_token, seed_everything


class AutoLLM:
    """``AutoLLM.from_pretrained(config, group)``: pick the model class for ``config.model_name``."""

    @staticmethod
    def from_pretrained(config: ModelConfig, group=None):
        arch = config.arch()
        if arch.num_experts:
            from .qwen_moe import Qwen3MoE
            return Qwen3MoE(config, group)
        return Qwen3(config, group)


class AutoTokenizer:
    """Tokenizers come from Hugging Face files; without a local copy there is nothing to load offline."""

    @staticmethod
    def from_pretrained(config: ModelConfig):
        import transformers
        path = config.checkpoint_dir or config.model_name
        return transformers.AutoTokenizer.from_pretrained(path, local_files_only=True)


__all__ = ["ARCHS", "ArchConfig", "ModelConfig", "AutoLLM", "AutoTokenizer", "Qwen3", "KV_Cache", "Engine",
           "sample_token", "seed_everything", "logger"]
