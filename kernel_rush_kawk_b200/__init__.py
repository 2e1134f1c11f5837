"""A small B200-native inference library for the Qwen3 dense decoder.

From a model folder (config.json + safetensors) or seeded random weights to
generated tokens on one GPU: typed configuration and registry, weights by
tensor name, layers put together from parts, a paged cache with slots, one step
function, a generation loop with greedy and temperature sampling, and trace
replay. All arithmetic of the model runs in this package's own CUDA kernels.
"""

from .config import ConfigError, Qwen3Config, read_config, register_architecture
from .engine import Engine, StepEntry
from .sampling import SamplingParams
from .weights import WeightError, write_model_folder

__version__ = "0.1.0"
__all__ = ["ConfigError", "Qwen3Config", "read_config", "register_architecture", "Engine", "StepEntry",
           "SamplingParams", "WeightError", "write_model_folder"]
