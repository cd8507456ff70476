"""The bias-free pre-norm GQA decoder with multi-token-prediction heads
(upstream ``Transformer``, main_models_new.py:174-226), put together from parts.

Tensor names are upstream's ``named_parameters()``::

    embedding.weight                                   (V, d)
    transformer_block_list.{l}.att.q_proj.weight       (d, H*hd)
    transformer_block_list.{l}.att.kv_proj.weight      (d, 2*KVH*hd)
    transformer_block_list.{l}.att.rms_norm_att.scale  (d,)
    transformer_block_list.{l}.att.linear_proj.weight  (H*hd, d)
    transformer_block_list.{l}.ffn.swig.linear1.weight (d, F)     gate
    transformer_block_list.{l}.ffn.swig.linear2.weight (d, F)     up
    transformer_block_list.{l}.ffn.fc.weight           (F, d)
    transformer_block_list.{l}.rms_norm_ffn.scale      (d,)
    rms_out.scale                                      (d,)
    mtp_heads_list.{i}.proj.weight                     (2d, d)
    mtp_heads_list.{i}.rms_embed.scale                 (d,)
    mtp_heads_list.{i}.rms_out.scale                   (d,)
    mtp_heads_list.{i}.trans_block.<the eight of a block>
    lm_head.weight                                     (V, d)     only when tie_word_embeddings is false
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.model_config import GqaMtpConfig
from ..kernels import ops
from ..parts.base import BuildContext, Part, StateSpec, WeightSpec
from ..parts.block import Block
from ..parts.embedding import Embedding, LMHead
from ..parts.stream import ResidualStream
from ..registry import part, register_architecture
from .base import Model, ScheduleEntry, StepOutput


def _make_block(cfg: GqaMtpConfig, prefix: str, layer_index: int, lag: int, mixer_type: str, ffn_type: str,
                position) -> Block:
    """One block of the architecture.  The parts are whatever classes the registries hold under
    the names the configuration gives; each reads its sizes and constants from ``cfg`` itself
    (``from_config``), so a part registered from outside is built the same way as a built-in one."""
    norm_cls = part("norm", cfg.norm_type)
    mixer = part("mixer", mixer_type).from_config(cfg, prefix=prefix + "att.", layer_index=layer_index, lag=lag,
                                                  position=position)
    ffn = part("ffn", ffn_type).from_config(cfg, prefix=prefix + "ffn.", layer_index=layer_index)
    return Block(
        norm_cls.from_config(cfg, prefix=prefix + "att.rms_norm_att."),
        mixer,
        norm_cls.from_config(cfg, prefix=prefix + "rms_norm_ffn."),
        ffn,
        prefix=prefix,
    )


class MtpHead(Part):
    """Head i (upstream ``mtp_head``, main_models_new.py:155-171): at position p it takes the
    previous stage's normalised output at p and the embedding of token p+1+i,
    ``u = cat[h, rms_embed(e)] @ proj``, runs one block at position p over its own cache,
    and normalises: ``g = rms_out(u)``.  It runs 1+i positions behind the trunk."""

    def __init__(self, cfg: GqaMtpConfig, index: int, embedding: Embedding, position):
        prefix = f"mtp_heads_list.{index}."
        super().__init__(prefix)
        norm_cls = part("norm", cfg.norm_type)
        self.index = index
        self.lag = 1 + index
        self.width = cfg.hidden_size
        self.embedding = embedding
        self.rms_embed = norm_cls.from_config(cfg, prefix=prefix + "rms_embed.")
        self.rms_out = norm_cls.from_config(cfg, prefix=prefix + "rms_out.")
        self.block = _make_block(cfg, prefix + "trans_block.", cfg.num_layers + index, self.lag, "gqa", "swiglu",
                                 position)
        self.w_proj: Optional[torch.Tensor] = None

    def children(self):
        return (self.rms_embed, self.rms_out, self.block)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"proj.weight": WeightSpec((2 * self.width, self.width))}

    def load(self, tensors, ctx: BuildContext) -> None:
        self.w_proj = tensors[self.prefix + "proj.weight"].to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, h_prev: torch.Tensor, pending_rows: torch.Tensor, step, entry: ScheduleEntry) -> torch.Tensor:
        """``h_prev``: the previous stage's output at this step's rows; ``pending_rows``
        ``[slots, width]``: per request, that stage's output at the last position fed."""
        n = h_prev.shape[0]
        trunk = step.stage(0)
        cat = torch.empty((n, 2 * self.width), dtype=h_prev.dtype, device=h_prev.device)
        ops.mtp_input(h_prev, pending_rows, trunk.row_slot, trunk.row_last, trunk.tokens, self.embedding.table,
                      self.rms_embed.scale, self.rms_embed.eps, cat)
        u = ops.gemm(cat, self.w_proj)
        stream = ResidualStream(torch.zeros((n, self.width), dtype=torch.float32, device=h_prev.device))
        stream.add(u)
        self.block.forward(stream, step.stage(self.lag), entry.binding)
        return stream.normed(self.rms_out)


class GqaMtpModel(Model):
    def __init__(self, cfg: GqaMtpConfig):
        super().__init__()
        self.config = cfg
        self.vocab_size = cfg.vocab_size
        self.max_positions = cfg.max_context
        self.position = part("position", cfg.position_type).from_config(cfg)
        self.embedding = Embedding(cfg.vocab_size, cfg.hidden_size)
        mixers = cfg.mixer_types or ["gqa"] * cfg.num_layers
        ffns = cfg.ffn_types or ["swiglu"] * cfg.num_layers
        self.blocks: List[Block] = [
            _make_block(cfg, f"transformer_block_list.{l}.", l, 0, mixers[l], ffns[l], self.position)
            for l in range(cfg.num_layers)
        ]
        norm_cls = part("norm", cfg.norm_type)
        self.rms_out = norm_cls.from_config(cfg, prefix="rms_out.")
        self.heads: List[MtpHead] = [MtpHead(cfg, i, self.embedding, self.position)
                                     for i in range(cfg.num_mtp_heads)]
        self.lm_head = LMHead(cfg.vocab_size, cfg.hidden_size, self.embedding if cfg.tie_word_embeddings else None)
        # the order in which layers run is data
        self.entries = [ScheduleEntry(self.blocks[l], source=src) for (l, src) in cfg.schedule()]
        self.n_trunk_entries = len(self.entries)
        self.entries += [ScheduleEntry(h.block) for h in self.heads]
        self._pending: List[torch.Tensor] = []

    def top_parts(self):
        return [self.embedding, self.position, *self.blocks, self.rms_out, *self.heads, self.lm_head]

    def extra_states(self, ctx: BuildContext) -> Dict[str, StateSpec]:
        # per MTP head: the previous stage's output row at the last position fed
        return {f"mtp_pending{i}": StateSpec((self.config.hidden_size,), ctx.dtype)
                for i in range(len(self.heads))}

    def bind(self, cache) -> None:
        super().bind(cache)
        self._pending = [cache.states[f"mtp_pending{i}"] for i in range(len(self.heads))]

    def forward(self, step, want_rows: torch.Tensor, aux: bool = False) -> StepOutput:
        """Trunk over the step's rows, then (``aux``) the MTP heads in order, each fed by the
        stage before it (server.py:328-359 upstream); logits only at the wanted rows."""
        stream = ResidualStream(self.embedding.forward(step.tokens))
        trunk = self.entries[: self.n_trunk_entries]
        for i, e in enumerate(trunk):
            e.block.forward(stream, step, e.binding, following=trunk[i + 1].block if i + 1 < len(trunk) else None)
        h = stream.normed(self.rms_out)
        # a step whose shape says that every row is wanted (a decode step) needs no gather
        pick = (lambda t: t) if getattr(step, "want_identity", False) else (lambda t: t.index_select(0, want_rows))
        if not (aux and self.heads):
            return StepOutput(main=self.lm_head.forward(pick(h)))
        # the heads' rows first (each is fed by the stage before it), then one product with the output matrix for
        # the trunk and all heads: the matrix, by far the largest, is read once a step
        rows, valid = [pick(h)], []
        prev = h
        for i, head in enumerate(self.heads):
            prev = head.forward(prev, self._pending[i], step, self.entries[self.n_trunk_entries + i])
            rows.append(pick(prev))
            valid.append(step.stage(head.lag).row_slot.index_select(0, want_rows) >= 0)
        n = rows[0].shape[0]
        logits = self.lm_head.forward(torch.cat(rows, dim=0))
        out = StepOutput(main=logits[:n])
        out.aux = [logits[(i + 1) * n:(i + 2) * n] for i in range(len(self.heads))]
        out.aux_valid = valid
        return out


def build(cfg: GqaMtpConfig) -> GqaMtpModel:
    return GqaMtpModel(cfg)


register_architecture(GqaMtpConfig.architecture, GqaMtpConfig, build)
