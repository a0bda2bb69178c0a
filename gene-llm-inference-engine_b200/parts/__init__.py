from . import attention, block, feed_forward, norm, position  # noqa: F401  (registers the parts)
from .model import DecoderModel, LayerRun
from .registry import (BLOCKS, FEED_FORWARDS, LOGIT_TRANSFORMS, MIXERS, NORMS, POSITION_ENCODINGS, BuildContext, build_part,
                       register_block, register_feed_forward, register_logit_transform, register_mixer, register_norm,
                       register_position_encoding, sub_weights)

__all__ = ["DecoderModel", "LayerRun", "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
           "LOGIT_TRANSFORMS", "register_logit_transform", "BuildContext", "build_part", "register_block", "register_feed_forward", "register_mixer",
           "register_norm", "register_position_encoding", "sub_weights"]
