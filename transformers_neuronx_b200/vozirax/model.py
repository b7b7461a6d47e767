"""The Python entry point of the Vozirax decoder, with the interface of every other model's:

    model = VoziraxForSampling.from_pretrained(folder, batch_size=4, amp='bf16', n_positions=2048)
    model.to_neuron()
    tokens = model.sample(input_ids, sequence_length=256)

Everything but the architecture's name is shared with the other entry points: the engine (scheduler, step
function, cache manager, sampler) behind it is the same.  The design has no end-of-sequence token and its
positions are computed, not looked up, so a row runs to ``sequence_length`` unless a generation configuration names an eos id, and
``n_positions`` only sizes the cache.
"""
from __future__ import annotations

from ..modeling_auto import register_model_class
from ..opt.model import OPTForSampling


class VoziraxForSampling(OPTForSampling):
    ARCHITECTURE = "Vozirax"


register_model_class("vozirax", VoziraxForSampling)
