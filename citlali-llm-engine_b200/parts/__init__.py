from .base import (BuildContext, StepBatch, build_part, part_class, register_part, registered_parts,
                   unregister_part)
from . import rotary, norm, linear, attention, feed_forward, block   # registers the built-in parts
from .attention import GQAttention
from .block import PreNormResidualBlock
from .feed_forward import GatedSiluFeedForward
from .linear import DenseLinear
from .norm import RMSNorm
from .rotary import NoPosition, RotaryHalfSplit
