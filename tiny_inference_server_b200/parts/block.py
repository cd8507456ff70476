"""A pre-norm block: norm, mixer, residual; norm, feed-forward, residual
(upstream ``Transformer_block``, main_models_new.py:139-152)."""
from __future__ import annotations

from .base import LayerBinding, Part
from .stream import ResidualStream


class Block(Part):
    def __init__(self, norm_mixer, mixer, norm_ffn, ffn, prefix: str = ""):
        super().__init__(prefix)
        self.norm_mixer = norm_mixer
        self.mixer = mixer
        self.norm_ffn = norm_ffn
        self.ffn = ffn

    def children(self):
        return (self.norm_mixer, self.mixer, self.norm_ffn, self.ffn)

    def forward(self, stream: ResidualStream, step, binding: LayerBinding) -> None:
        a = stream.normed(self.norm_mixer)
        stream.add(self.mixer.forward(a, step, binding))
        f = stream.normed(self.norm_ffn)
        stream.add(self.ffn.forward(f, step))
