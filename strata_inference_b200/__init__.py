"""strata_inference_b200: a small, whole model library with generation of its
own for one B200 (sm_100a): typed configuration and an architecture
registry, safetensors weights by name (and a seeded random-weights mode),
decoder layers assembled from parts, a paged cache with a slot per sequence,
one step function, a generation loop, sampling, a command line and trace
replay, on hand-written CUDA kernels.

    from strata_inference_b200 import GenerationEngine, GenerationConfig, SamplingConfig
"""

from .config.registry import (known_architectures, read_config_json,  # noqa: F401
                              register_architecture, spec_from_config)
from .config.spec import (ConfigError, LayerSpec, ModelSpec, PartSpec,  # noqa: F401
                          ScheduleEntry)
from .sampling.sampler import SamplingConfig  # noqa: F401
from .engine.generate import GenerationConfig, GenerationOutput, generate  # noqa: F401
from .engine.engine import Engine  # noqa: F401
from .engine.api import GenerationEngine  # noqa: F401
from .weights.loader import TensorDecl, WeightError  # noqa: F401
from .weights.random_init import write_random_model  # noqa: F401

__version__ = "0.1.0"
