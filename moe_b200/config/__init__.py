from .registry import (  # noqa: F401
    Architecture,
    ConfigError,
    architecture_name,
    lookup,
    parse_config,
    read_config_json,
    register_architecture,
    registered_architectures,
)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry  # noqa: F401
from .qwen2_moe import Qwen2MoeConfig  # noqa: F401  (registers the architecture)
