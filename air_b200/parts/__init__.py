from .spec import PartSpec, BlockSpec, ModelSpec, RunStep
from .base import (Runtime, CacheNeed, PagedKV, PagedKVView, SlotState, SlotStateView, HostBatch, Plan, Part, Mixer,
                   FeedForward, Norm, PositionEncoding)
from .registry import (register_mixer, register_feed_forward, register_norm, register_position_encoding,
                       register_block, register_architecture, architecture, architectures)
from . import norm, rope, attention, mlp, block  # registers the parts that ship with the engine
from .block import Block
