from .engine_config import EngineConfig
from .model_config import ConfigError, read_config_json
from .registry import (ARCHITECTURES, BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, architecture_name,
                       config_from_dict, register_architecture)
from .specs import (BlockSpec, FeedForwardSpec, LayerCall, MixerSpec, ModelSpec, NormSpec, PositionSpec)
