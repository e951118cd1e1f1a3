"""Parts of a layer.  Importing the package registers the built-in kinds."""
from .base import Activations, Part, Runtime, TensorSpec, make_part, register_part, registered_parts  # noqa: F401
from . import norm, rope, attention, feedforward, embedding  # noqa: F401  (registration)
from .block import PreNormBlock, make_block, register_block  # noqa: F401
