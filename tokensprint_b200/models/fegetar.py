"""Fegetar: its typed configuration and the architecture entry.

A decoder of post-normed layers (x <- x + Norm(f(x)), f reads x itself; norm weights stored as
their distance from one) around latent attention with an output gate per head, a feed-forward
that is absent, dense (two matrices around the tanh form of gelu) or a set of routed capped-GLU
experts with a shared one, and after it a gated input from a second token table (one slice of the
token's row per layer).  The embedding adds a row of a hashed table of token pairs.  Every size and
every constant that may differ between two models of the design comes from config.json:

    architecture, vocab, width, norm.eps
    embedding.bigram {buckets, mul_prev, mul_cur}          (optional)
    token_side {dim}                                        (optional)
    layers[i] {type: "latent_attention",
               mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}},
               mlp   null | {kind: "dense", ff}
                          | {kind: "moe", router {experts, top}, expert {ff, limit}, shared {ff, limit} | null}}

Tensor names: embed, bigram, side.embed, l<i>.norm1/.norm2, l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o},
l<i>.mlp.{up,down} or l<i>.mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down}},
l<i>.side.{gate,proj,norm}, final.norm, head.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional

from tokensprint_b200.config.model_config import ConfigError, read_config_json, require, write_config_json
from tokensprint_b200.config.registry import PRESET_DIR, register_architecture, register_preset
from tokensprint_b200.models.spec import ModelSpec
from tokensprint_b200.parts.base import PartSpec

ARCHITECTURE = "Fegetar"
EXPERT_ALPHA = 1.702  # the sigmoid's slope inside an expert's activation: fixed by the design
DEFAULT_MAX_POSITIONS = 32768  # the design sets no limit; what the engine plans for unless the file says otherwise


def _section(d: dict[str, Any], key: str, where: str) -> dict[str, Any]:
    value = d.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return value


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int  # unrotated query/key entries per head
    rot_dim: int  # rotated query/key entries per head (one key part for all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int  # how many of the rot_dim entries turn

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "LatentMixerConfig":
        rot = _section(d, "rot", where)
        c = cls(heads=require(d, "heads", int), dim=require(d, "dim", int), rot_dim=require(d, "rot_dim", int), vdim=require(d, "vdim", int),
                kv_rank=require(d, "kv_rank", int), scale=require(d, "scale", float), rot_base=require(rot, "base", float),
                rot_dims=require(rot, "dims", int))
        if min(c.heads, c.vdim, c.kv_rank) < 1 or c.dim < 0 or c.rot_dim < 0 or c.dim + c.rot_dim < 1:
            raise ConfigError(f"config.json: {where}mixer sizes must be positive")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.rot_dim or (c.rot_dims and c.rot_base <= 0):
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most rot_dim, rot.base positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str  # "dense" or "moe"
    ff: int  # dense: inner width; moe: an expert's inner width
    experts: int = 0
    top: int = 0
    limit: float = 0.0
    shared_ff: int = 0  # 0: no shared expert
    shared_limit: float = 0.0

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "FeedForwardConfig":
        kind = d.get("kind")
        if kind == "dense":
            c = cls(kind="dense", ff=require(d, "ff", int))
        elif kind == "moe":
            router, expert = _section(d, "router", where), _section(d, "expert", where)
            shared = d.get("shared")
            c = cls(kind="moe", ff=require(expert, "ff", int), experts=require(router, "experts", int), top=require(router, "top", int),
                    limit=require(expert, "limit", float), shared_ff=require(shared, "ff", int) if shared else 0,
                    shared_limit=require(shared, "limit", float) if shared else 0.0)
            if not 0 < c.top <= c.experts:
                raise ConfigError(f"config.json: {where}router.top must lie in 1..router.experts")
        else:
            raise ConfigError(f"config.json: {where}mlp.kind must be 'dense' or 'moe', got {kind!r}")
        if c.ff < 1 or c.shared_ff < 0:
            raise ConfigError(f"config.json: {where}mlp widths must be positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff, "limit": self.limit},
                "shared": {"ff": self.shared_ff, "limit": self.shared_limit} if self.shared_ff else None}


@dataclass(frozen=True)
class FegetarLayerConfig:
    mixer: LatentMixerConfig
    mlp: Optional[FeedForwardConfig]
    type: str = "latent_attention"


@dataclass(frozen=True)
class FegetarConfig:
    """All sizes and constants of one Fegetar model."""

    vocab: int
    width: int
    norm_eps: float
    layers: tuple[FegetarLayerConfig, ...]
    bigram_buckets: int = 0  # 0: no pair table
    bigram_mul_prev: int = 0
    bigram_mul_cur: int = 0
    side_dim: int = 0  # 0: no per-layer token input
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: int = -1
    extra: dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ConfigError("config.json: 'vocab', 'width' and the number of layers must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        if self.bigram_buckets < 0 or self.side_dim < 0:
            raise ConfigError("config.json: 'embedding.bigram.buckets' and 'token_side.dim' must not be negative")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "FegetarConfig":
        layers = []
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with an entry per layer")
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            kind = entry.get("type")
            if kind != "latent_attention":
                raise ConfigError(f"config.json: {where}type {kind!r} is no mixer of this design (known: 'latent_attention')")
            mlp = entry.get("mlp")
            layers.append(FegetarLayerConfig(
                mixer=LatentMixerConfig.from_dict(_section(entry, "mixer", where), where),
                mlp=None if mlp is None else FeedForwardConfig.from_dict(mlp, where)))
        bigram = (d.get("embedding") or {}).get("bigram")
        side = d.get("token_side")
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "layers", "embedding", "token_side",
                 "max_position_embeddings", "eos_token_id"}
        return cls(
            vocab=require(d, "vocab", int), width=require(d, "width", int), norm_eps=require(_section(d, "norm", ""), "eps", float),
            layers=tuple(layers),
            bigram_buckets=require(bigram, "buckets", int) if bigram else 0,
            bigram_mul_prev=require(bigram, "mul_prev", int) if bigram else 0,
            bigram_mul_cur=require(bigram, "mul_cur", int) if bigram else 0,
            side_dim=require(side, "dim", int) if side else 0,
            max_position_embeddings=int(d.get("max_position_embeddings") or DEFAULT_MAX_POSITIONS),
            eos_token_id=int(d["eos_token_id"]) if isinstance(d.get("eos_token_id"), int) else -1,
            extra={k: v for k, v in d.items() if k not in known})

    @classmethod
    def from_json(cls, path: str | Path) -> "FegetarConfig":
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers],
        }
        if self.bigram_buckets:
            d["embedding"] = {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev, "mul_cur": self.bigram_mul_cur}}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id >= 0:
            d["eos_token_id"] = self.eos_token_id
        return d

    def save(self, folder: str | Path) -> None:
        write_config_json(folder, self.to_dict())


def _capped_expert(prefix: str, width: int, ff: int, limit: float) -> PartSpec:
    return PartSpec("capped_glu", {"hidden_size": width, "intermediate_size": ff, "limit": limit, "alpha": EXPERT_ALPHA,
                                   "gate": prefix + "gate", "up": prefix + "up", "down": prefix + "down"})


@register_architecture(ARCHITECTURE, model_types=("fegetar",), config_from_dict=FegetarConfig.from_dict)
def build_fegetar_spec(config: FegetarConfig) -> ModelSpec:
    W, eps = config.width, config.norm_eps
    layers, ignorable = [], []

    def norm(name: str, offset: float) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": W, "eps": eps, "weight": name, "offset": offset})

    for i, layer in enumerate(config.layers):
        p, m = f"l{i}.", layer.mixer
        position = None
        if m.rot_dims:
            position = PartSpec("rotary", {"dim": m.rot_dims, "theta": m.rot_base, "pairing": "neighbours", "exact_frequencies": True})
        mixer = PartSpec("latent_attention", {
            "hidden_size": W, "num_heads": m.heads, "nope_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim, "kv_rank": m.kv_rank,
            "scale": m.scale, "norm_eps": eps, "position": position,
            "q": p + "mix.q", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk", "uv": p + "mix.uv",
            "gate": p + "mix.g", "o": p + "mix.o"})
        params: dict[str, Any] = {"mixer": mixer, "mixer_norm": norm(p + "norm1", 1.0)}
        f = layer.mlp
        if f is None:
            ignorable.append(p + "norm2")  # a layer without a feed-forward has no use for its norm
        else:
            if f.kind == "dense":
                ff = PartSpec("activated", {"hidden_size": W, "intermediate_size": f.ff, "activation": "gelu_tanh",
                                            "up": p + "mlp.up", "down": p + "mlp.down"})
            else:
                ff = PartSpec("routed_experts", {
                    "hidden_size": W, "num_experts": f.experts, "top": f.top, "intermediate_size": f.ff, "limit": f.limit,
                    "alpha": EXPERT_ALPHA, "renormalize": False, "weight_on": "input", "router": p + "mlp.router",
                    "expert_prefix": p + "mlp.e",
                    "shared": _capped_expert(p + "mlp.shared.", W, f.shared_ff, f.shared_limit) if f.shared_ff else None})
            params.update(feed_forward=ff, ffn_norm=norm(p + "norm2", 1.0))
        if config.side_dim:
            params.update(
                extra=PartSpec("token_gated_input", {
                    "hidden_size": W, "dim": config.side_dim, "table": "side.embed", "table_width": config.side_dim * len(config.layers),
                    "column0": i * config.side_dim, "vocab_size": config.vocab, "gate": p + "side.gate", "proj": p + "side.proj"}),
                extra_norm=norm(p + "side.norm", 0.0))
        layers.append(PartSpec("post_norm", params))
    pair = None
    if config.bigram_buckets:
        pair = PartSpec("pair_hash_embedding", {"table": "bigram", "buckets": config.bigram_buckets, "mul_prev": config.bigram_mul_prev,
                                                "mul_cur": config.bigram_mul_cur, "hidden_size": W, "vocab_size": config.vocab})
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=W, embedding="embed", layers=layers, final_norm=norm("final.norm", 1.0), lm_head="head",
        max_positions=config.max_position_embeddings, eos_token_id=config.eos_token_id, ignorable_tensors=tuple(ignorable),
        embedding_transform=pair)


# A named model of this design, so that the command lines can run it with random weights: four
# layers at a width of 2,048 (dense and routed feed-forwards in turn), the size bench.py --designs times.
for _path in sorted(PRESET_DIR.glob("fegetar-*.json")):
    register_preset("fegetar", _path.stem, _path)
