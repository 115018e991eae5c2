"""infernum_b200: a small, whole inference engine for one NVIDIA B200.

From a model folder to tokens:

    import infernum_b200 as ib
    model = ib.load_model("path/to/model", dtype="bfloat16")
    engine = ib.Engine(model, ib.BatchConfig(max_batch_size=32, block_size=16, num_blocks=4096))
    tokens = engine.generate([1, 15043, 3186], ib.GenerateOptions(max_new_tokens=32))

``load_model`` picks the architecture by ``model_type`` in config.json.  All
compute runs in hand-written CUDA kernels for sm_100a (plus library matrix
products); there is no CPU path.
"""

from .engine import BatchConfig, Engine, FinishReason, GenerationEvent, RequestHandle
from .errors import (CacheError, ConfigError, InfernumError, KernelError, OutOfPagesError,
                     SchedulingError, UnsupportedModelError, WeightError)
from .loading import load_model, random_model
from .registry import register_architecture, resolve, supported_architectures
from .sampling import GenerateOptions, SamplingParams
from .weights.random_init import write_random_model

__version__ = "0.1.0"


def generate(model_dir: str, prompt_ids, options: GenerateOptions = None, dtype="bfloat16",
             config: BatchConfig = None):
    """One call from a model folder and prompt token ids to generated token
    ids.  The end-of-sequence id is taken from config.json when the options
    name none (infernum-runtime/src/runtime.rs:127-135)."""
    import dataclasses

    model = load_model(model_dir, dtype=dtype)
    options = options or GenerateOptions()
    if options.eos_token_id is None and model.spec.eos_token_id is not None:
        options = dataclasses.replace(options, eos_token_id=model.spec.eos_token_id)
    return Engine(model, config).generate(prompt_ids, options)
