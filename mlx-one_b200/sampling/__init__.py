from .options import GenerationChunk, GenerationResult, TextGenerationOptions

__all__ = ["GenerationChunk", "GenerationResult", "TextGenerationOptions"]
