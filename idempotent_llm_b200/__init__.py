"""idempotent_llm_b200: a small, whole, single-GPU model library for the Qwen3 dense
decoder, the Lunulix decoder (attention and a state-space mixer side by side) and the Panodra
decoder (attention through a latent, experts by a table over token ids, looped layers) on NVIDIA
B200 (sm_100a): configuration and registry, weights by name, layers from parts, a paged
sequence cache with per-sequence state, one step function, a generation loop, sampling,
trace replay, and hand-written CUDA kernels in bfloat16 and in true 32-bit."""

from .api import LM, build_model, canonical_dtype, from_random, load
from .config import ConfigError, LunulixConfig, PanodraConfig, Qwen3Config
from .registry import read_config, register_architecture, registered_architectures

__all__ = ["LM", "build_model", "canonical_dtype", "from_random", "load", "ConfigError", "LunulixConfig", "PanodraConfig", "Qwen3Config",
           "read_config", "register_architecture", "registered_architectures"]
__version__ = "0.1.0"
