from .config import RWKV7Config, SimpleTrainConfig
from .model import Linear, RWKV7Block, RWKV7ChannelMix, RWKV7Model, RWKV7TimeMix
from .infctx_module import BlockState, BlockStateList, ChannelMixState, TimeMixState
from .model_infctx import RWKV7Infctx

__all__ = ["RWKV7Model", "RWKV7Block", "RWKV7TimeMix", "RWKV7ChannelMix", "RWKV7Config", "SimpleTrainConfig",
           "Linear", "BlockState", "BlockStateList", "ChannelMixState", "TimeMixState", "RWKV7Infctx"]
