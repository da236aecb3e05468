from .options import GenerationChunk, GenerationResult, TextGenerationOptions
from .sampler import Sampler

__all__ = ["GenerationChunk", "GenerationResult", "TextGenerationOptions", "Sampler"]
