"""The parts a model is put together from, each registered under a kind name.

Importing this package registers the built-in kinds: mixers ``attention``,
``latent_attention``, ``mamba2``, ``mlstm``, ``gated_linear_attention``, ``delta_rule``, ``talking_attention``
``side_by_side``, ``gated_attention`` and ``pooled_window_attention``; feed-forwards ``dense``, ``gated_dense``, ``experts``
and ``none``; norms ``layer_norm`` and ``rms_norm``; positions ``learned``, ``rotary`` and
``none``; blocks ``pre_norm``, ``parallel``, ``output_norm`` and ``sandwich_norm``; embedding ``token``; head
``linear``; side input ``token_gated``.
"""

from ayaka_b200.parts import (block, embedding, experts, feed_forward,  # noqa: F401
                              gated_attention, latent, mixer, norm, pooled_attention, recurrent,
                              side_by_side, token_input)
from ayaka_b200.parts.base import (BuildContext, CacheNeed, Part, StateNeed, build_part,
                                   register_part, registered_kinds)
from ayaka_b200.parts.context import GroupStep, LayerCache, StepContext, Workspace
from ayaka_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, Run

__all__ = [
    "BuildContext", "CacheNeed", "GroupStep", "LayerCache", "LayerSpec", "ModelSpec", "Part",
    "PartSpec", "Run", "StateNeed", "StepContext", "Workspace", "build_part", "register_part",
    "registered_kinds",
]
