"""Model assembly.  Importing this package registers the built-in architectures."""
from . import qwen3  # noqa: F401
from .decoder import DecoderModel


def build_model(config, dtype):
    """A ``DecoderModel`` (without weights) for a typed configuration: anything with ``model_spec()``."""
    return DecoderModel(config.model_spec(), dtype)
