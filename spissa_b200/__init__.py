"""spissa_b200: a small model library with generation for one B200.

Everything between a request's tokens and its next token for the Llama dense GQA
decoder that Erik-cpu-create/spissa runs: typed configuration and an architecture
registry, safetensors weights by name (or seeded random weights), a model put
together from parts, a paged cache with a slot per sequence, one step function over
ragged batches, a generation loop with greedy and temperature sampling, and
hand-written CUDA kernels for sm_100a. There is no CPU path.

    from spissa_b200 import Engine, SamplingParams
    engine = Engine.from_folder("model_dir", dtype="bfloat16", max_tokens=8192)
    results, metrics = engine.generate([[1, 2, 3]], max_new_tokens=16)
"""
from .config import LlamaConfig, load_config, register_architecture
from .engine import Engine, StepEntry, StepError, generate
from .sampling import Sampler, SamplingParams
from .weights import WeightError, write_random_model

__version__ = "0.1.0"
__all__ = ["LlamaConfig", "load_config", "register_architecture", "Engine", "StepEntry", "StepError",
           "generate", "Sampler", "SamplingParams", "WeightError", "write_random_model"]
