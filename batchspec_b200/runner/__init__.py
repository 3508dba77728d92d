from .runner import PREFILL_CHUNK_BY_BATCH, Runner, load_prompts, synthetic_prompts

__all__ = ["PREFILL_CHUNK_BY_BATCH", "Runner", "load_prompts", "synthetic_prompts"]
