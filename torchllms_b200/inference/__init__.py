from .llm import LLM, GenerationResult

__all__ = ["LLM", "GenerationResult"]
