"""mlx-one_b200: a small, whole inference engine for one B200.

From a model folder (config.json + safetensors) to generated tokens: typed configuration and
registry, weights by name, layers built from parts, a paged cache manager, one step function
for ragged mixed batches, a scheduler, sampling, a Python entry point and a command line.
Every forward kernel is hand-written CUDA for sm_100a.
"""

__version__ = "0.1.0"

from .engine import BatchingConfig, CacheConfig, Engine, load_model
from .sampling import GenerationChunk, GenerationResult, TextGenerationOptions
from .weights import write_random_model

__all__ = ["BatchingConfig", "CacheConfig", "Engine", "load_model", "GenerationChunk",
           "GenerationResult", "TextGenerationOptions", "write_random_model"]
