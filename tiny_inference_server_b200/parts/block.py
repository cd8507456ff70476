"""A pre-norm block: norm, mixer, residual; norm, feed-forward, residual
(upstream ``Transformer_block``, main_models_new.py:139-152)."""
from __future__ import annotations

from typing import Optional

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

    def forward(self, stream: ResidualStream, step, binding: LayerBinding, following: Optional["Block"] = None) -> None:
        """``following``: the block that reads the stream after this one, if the caller knows it; its first
        norm can then be folded into this block's last product and that block's first one."""
        mixer, ffn = self.mixer, self.ffn
        a = stream.normed(self.norm_mixer, scaled=mixer.accepts_scaled_rows)
        if mixer.fuses_residual and ffn.accepts_scaled_rows:
            stream.add(mixer.forward(a, step, binding, residual=stream.sink(self.norm_ffn, a.dtype)))
        else:
            stream.add(mixer.forward(a, step, binding))
        f = stream.normed(self.norm_ffn, scaled=ffn.accepts_scaled_rows)
        if ffn.fuses_residual and following is not None and following.mixer.accepts_scaled_rows:
            stream.add(ffn.forward(f, step, residual=stream.sink(following.norm_mixer, f.dtype)))
        else:
            stream.add(ffn.forward(f, step))
