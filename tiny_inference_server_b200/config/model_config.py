"""Typed model configuration, read from ``config.json``.

The upstream project keeps its model constants in one dataclass shared with training
(``Config/config.py:5-23``: ``D_MODEL, VOCAB_SIZE, MAX_CONTEXT, MAX_FREQ, N_HEAD,
NUM_LAYERS, FFN_HIDDEN_DIM, NUM_GROUPS, MTP_HEADS``) and has no ``config.json``.  Here
every size and constant of the model comes from ``config.json``; the upstream names
are accepted as aliases of the lower-case keys.  No size is written into code.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, ClassVar, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a model; the message names every problem."""


# upstream Config field -> key of config.json  (Config/config.py:11-23)
UPSTREAM_ALIASES = {
    "D_MODEL": "hidden_size",
    "VOCAB_SIZE": "vocab_size",
    "MAX_CONTEXT": "max_context",
    "MAX_FREQ": "rope_theta",
    "N_HEAD": "num_heads",
    "NUM_LAYERS": "num_layers",
    "FFN_HIDDEN_DIM": "ffn_hidden",
    "MTP_HEADS": "num_mtp_heads",
}


@dataclass
class GqaMtpConfig:
    """Configuration of the bias-free pre-norm GQA decoder with MTP heads
    (``main_models_new.py:174-194``).

    Required keys have no default.  Defaults of the optional keys are the constants
    that the upstream code fixes: eps ``main_models_new.py:36``, RoPE base and table
    length ``Config/config.py:13-14``, end-of-sequence id ``server.py:12``.
    """

    architecture: ClassVar[str] = "gqa_mtp_transformer"

    vocab_size: int
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    ffn_hidden: int
    head_dim: Optional[int] = None            # default hidden_size // num_heads (main_models_new.py:91)
    rms_norm_eps: float = 2e-8
    rope_theta: float = 10000.0
    max_context: int = 8192
    tie_word_embeddings: bool = True
    num_mtp_heads: int = 0
    eos_token_id: Optional[int] = None
    # engine options that the upstream model does not have
    sliding_window: Optional[int] = None       # keys p-window+1..p instead of 0..p
    full_attention_layers: Optional[list] = None   # layers (0..L-1 trunk, L+i = MTP head i) exempt from the window
    layer_order: Optional[list] = None         # order in which trunk layers run; may name a layer twice
    cache_source: Optional[list] = None        # per entry of layer_order: None, or an earlier entry whose K/V it reads
    mixer_types: Optional[list] = None         # per trunk layer, a name of the mixer registry (default "gqa")
    ffn_types: Optional[list] = None           # per trunk layer, a name of the feed-forward registry (default "swiglu")
    norm_type: str = "rmsnorm_l2"
    position_type: str = "rope_half"
    torch_dtype: str = "bfloat16"              # dtype the weights are stored in

    def __post_init__(self):
        errs = []
        for name in ("vocab_size", "hidden_size", "num_layers", "num_heads", "num_kv_heads", "ffn_hidden"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                errs.append(f"{name} must be a positive integer, got {v!r}")
        if errs:
            raise ConfigError("; ".join(errs))
        if self.head_dim is None:
            if self.hidden_size % self.num_heads:
                errs.append(f"hidden_size {self.hidden_size} is not a multiple of num_heads {self.num_heads} "
                            f"and head_dim is not given")
            self.head_dim = self.hidden_size // self.num_heads
        if self.num_heads % self.num_kv_heads:
            errs.append(f"num_heads {self.num_heads} is not a multiple of num_kv_heads {self.num_kv_heads}")
        if self.head_dim % 2:
            errs.append(f"head_dim {self.head_dim} must be even for rotary position encoding")
        if not (self.rms_norm_eps >= 0):
            errs.append(f"rms_norm_eps must be >= 0, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            errs.append(f"rope_theta must be > 0, got {self.rope_theta}")
        if self.max_context <= 0:
            errs.append(f"max_context must be positive, got {self.max_context}")
        if self.num_mtp_heads < 0:
            errs.append(f"num_mtp_heads must be >= 0, got {self.num_mtp_heads}")
        if self.sliding_window is not None and self.sliding_window <= 0:
            errs.append(f"sliding_window must be positive or null, got {self.sliding_window}")
        n_all = self.num_layers + self.num_mtp_heads
        for l in self.full_attention_layers or []:
            if not (0 <= l < n_all):
                errs.append(f"full_attention_layers names layer {l}, outside 0..{n_all - 1}")
        order = self.layer_order if self.layer_order is not None else list(range(self.num_layers))
        for l in order:
            if not (isinstance(l, int) and 0 <= l < self.num_layers):
                errs.append(f"layer_order names layer {l!r}, outside 0..{self.num_layers - 1}")
        if self.cache_source is not None:
            if len(self.cache_source) != len(order):
                errs.append(f"cache_source has {len(self.cache_source)} entries, layer_order has {len(order)}")
            else:
                for e, s in enumerate(self.cache_source):
                    if s is None:
                        continue
                    if not (isinstance(s, int) and 0 <= s < e):
                        errs.append(f"cache_source[{e}]={s!r} must name an earlier entry")
                    elif self.cache_source[s] is not None:
                        errs.append(f"cache_source[{e}]={s} names an entry that has no cache of its own")
                    elif all(isinstance(l, int) and 0 <= l < self.num_layers for l in (order[e], order[s])):
                        # pages of the source's group are given back by the source's window: a reader
                        # that sees further back would walk pages that other requests hold by then
                        mine, theirs = self.window_of(order[e]), self.window_of(order[s])
                        if theirs is not None and (mine is None or mine > theirs):
                            errs.append(f"cache_source[{e}]={s}: layer {order[e]} sees "
                                        f"{'every key' if mine is None else f'{mine} keys'} but layer {order[s]}, "
                                        f"whose cache it reads, keeps only {theirs}")
        for key in ("mixer_types", "ffn_types"):
            v = getattr(self, key)
            if v is not None and len(v) != self.num_layers:
                errs.append(f"{key} has {len(v)} entries for {self.num_layers} layers")
        if self.torch_dtype not in ("bfloat16", "float32"):
            errs.append(f"torch_dtype must be bfloat16 or float32, got {self.torch_dtype!r}")
        if errs:
            raise ConfigError("; ".join(errs))

    # ---- derived ----
    @property
    def group_size(self) -> int:
        """Query heads per kv head (the upstream ``NUM_GROUPS``, Config/config.py:22)."""
        return self.num_heads // self.num_kv_heads

    def schedule(self):
        """[(layer index, entry whose cache is read or None)] in running order."""
        order = self.layer_order if self.layer_order is not None else list(range(self.num_layers))
        src = self.cache_source if self.cache_source is not None else [None] * len(order)
        return list(zip(order, src))

    def window_of(self, layer_index: int) -> Optional[int]:
        if self.sliding_window is None:
            return None
        if layer_index in (self.full_attention_layers or []):
            return None
        return int(self.sliding_window)

    # ---- (de)serialisation ----
    @classmethod
    def from_dict(cls, raw: dict) -> "GqaMtpConfig":
        d = {}
        for k, v in raw.items():
            d[UPSTREAM_ALIASES.get(k, k)] = v
        d.pop("architecture", None)
        if "NUM_GROUPS" in d:
            g = d.pop("NUM_GROUPS")
            if "num_heads" not in d:
                raise ConfigError("NUM_GROUPS given without N_HEAD / num_heads")
            if "num_kv_heads" not in d:
                if g <= 0 or d["num_heads"] % g:
                    raise ConfigError(f"N_HEAD {d['num_heads']} is not a multiple of NUM_GROUPS {g}")
                d["num_kv_heads"] = d["num_heads"] // g
        known = {f.name for f in dataclasses.fields(cls)}
        unknown = sorted(set(d) - known)
        required = [f.name for f in dataclasses.fields(cls)
                    if f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING]
        missing = [k for k in required if k not in d]
        if unknown or missing:
            parts = []
            if missing:
                parts.append("missing keys: " + ", ".join(missing))
            if unknown:
                parts.append("unknown keys: " + ", ".join(unknown))
            raise ConfigError(f"config for architecture {cls.architecture!r}: " + "; ".join(parts))
        return cls(**d)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture}
        for f in dataclasses.fields(self):
            d[f.name] = getattr(self, f.name)
        return d


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder!r}")
    with open(path) as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


def write_config_json(folder: str, cfg: Any) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f, indent=1)
