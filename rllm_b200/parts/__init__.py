from .base import (FeedForward, Junction, Mixer, Norm, PagedKVNeed, Part, PartError, Runtime, StateNeed,
                   build_part, part_class, register_part)
from . import (attention, block, chunked_attention, embedding, ffn, gated_attention, junction, latent_attention,
               mamba, mlstm, moe, norm, parallel, retention, rotary, rwkv)  # noqa: F401  (register the built-in kinds)

__all__ = ["FeedForward", "Junction", "Mixer", "Norm", "PagedKVNeed", "Part", "PartError", "Runtime", "StateNeed",
           "build_part", "part_class", "register_part"]
