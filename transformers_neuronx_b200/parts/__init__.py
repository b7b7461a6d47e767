from . import spec
from .base import (FeedForward, Mixer, Norm, Part, PositionEncoding, StepContext, to_device)
from .registry import (build_block, build_part, register_block, register_feed_forward, register_mixer,
                       register_norm, register_position)
from .linear import Linear, linear_forward
from . import norm, position, attention, feedforward, block, embedding   # register the built-in kinds
from . import rotary_attention, retention, mingru, parallel, conv_attention   # noqa: F401  more built-in mixers
from . import moe   # noqa: F401  the feed-forward of routed experts
from . import latent_attention, delta_rule   # noqa: F401  attention through latents; the gated delta rule
from . import ssd, diff_attention   # noqa: F401  the selective state-space mixer; differential attention
from .embedding import Embedding, Head
