"""nanoinfer_b200: a small, whole inference engine for one B200 GPU.

From a model folder (config.json + model.safetensors) to next-token logits and generated
tokens: typed configuration and an architecture registry, a safetensors loader, models put
together from parts, a paged cache manager, one step function over mixed batches, a
continuous-batching scheduler, sampling, and hand-written CUDA kernels for sm_100a.
"""
from . import parts as _parts  # registers the built-in parts  # noqa: F401
from .registry import architectures, get_architecture, load_config, register_architecture

__version__ = "0.1.0"
__all__ = ["architectures", "get_architecture", "load_config", "register_architecture", "load_model",
           "Engine", "SamplingParams"]


def __getattr__(name):
    # the engine pulls in the kernels; import it on demand so that configuration, weights and the
    # cache manager can be used where no GPU is present
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name == "SamplingParams":
        from .sampling.sampler import SamplingParams
        return SamplingParams
    raise AttributeError(name)


def load_model(model_dir: str, dtype="bfloat16", device="cuda"):
    """Build the model that ``model_dir/config.json`` names and load its weights."""
    import torch

    from .models.model import Model
    from .weights.loader import load_weights

    if isinstance(dtype, str):
        dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
                 "fp32": torch.float32}[dtype]
    config = load_config(model_dir)
    arch = get_architecture(config.architecture)
    model = Model(arch.build_spec(config), config)
    load_weights(model, model_dir, dtype, torch.device(device))
    return model
