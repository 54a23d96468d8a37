"""Dazilix: its typed configuration and the architecture entry.

A decoder whose layers wrap each sublayer in two norms and a learned scale per channel
(x <- x + s * N_out(f(N_in(x)))).  A layer's mixer is one of two: a softmax attention that sees
only the keys of its own block of positions, with a sink in the softmax's denominator, q and k
normed over the whole projection, a rotation of the first entries of each head and the key
projection as values; or a gated linear attention with a decay per key channel whose state lives
in float32.  The feed-forward, where a layer has one, is a set of routed SwiGLU experts weighted by
the softmax over the chosen router logits.  A stretch of layers may run several times with the same
weights (each pass with caches and states of its own); every pass starts by adding a learned
vector to the stream, and every pass after the first the embedding rows as well.  Every size and
every constant that may differ between two models of the design comes from config.json:

    architecture, vocab, width, norm.eps, embedding.scale
    loop {start, stop, times}                                           (optional)
    layers[i] {type: "attention", mixer {heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size}},
               mlp null | {kind: "moe", router {experts, top}, expert {ff}}}
    layers[i] {type: "gla", mixer {heads, dim, vdim, tau, decay_rank (optional: else the tensors' own)},
               mlp as above}

Tensor names: embed, loop.step, l<i>.norm1/.norm1b/.norm2/.norm2b/.ls1/.ls2,
l<i>.mix.{q,k,q.norm,k.norm,o} or l<i>.mix.{q,k,v,g,o,norm,a1,a2,a2.b},
l<i>.mlp.{router,router.b,e<j>.{gate,up,down}}, final.norm, head.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional, Union

from tokensprint_b200.config.model_config import ConfigError, read_config_json, require, write_config_json
from tokensprint_b200.config.registry import PRESET_DIR, register_architecture, register_preset
from tokensprint_b200.models.spec import ModelSpec, RunSpec
from tokensprint_b200.parts.base import PartSpec

ARCHITECTURE = "Dazilix"
SINK_SCORE = 0.0  # the score of the softmax's sink: fixed by the design
DEFAULT_MAX_POSITIONS = 32768  # the design sets no limit; what the engine plans for unless the file says otherwise


def _section(d: dict[str, Any], key: str, where: str) -> dict[str, Any]:
    value = d.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return value


@dataclass(frozen=True)
class BlockAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    mask_size: int  # 0: no `mask` in the file, every earlier key is seen

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "BlockAttentionConfig":
        rot = d.get("rot") or {}
        c = cls(heads=require(d, "heads", int), kv_heads=require(d, "kv_heads", int), dim=require(d, "dim", int),
                vdim=require(d, "vdim", int), scale=require(d, "scale", float),
                rot_base=require(rot, "base", float) if rot else 1.0, rot_dims=require(rot, "dims", int) if rot else 0,
                mask_size=require(_section(d, "mask", where), "size", int) if d.get("mask") is not None else 0)
        if min(c.heads, c.kv_heads, c.dim) < 1 or c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a positive multiple of kv_heads, dim positive")
        if c.vdim != c.dim:
            raise ConfigError(f"config.json: {where}the values are the key projection, so vdim must equal dim")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.dim or (c.rot_dims and c.rot_base <= 0):
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim, rot.base positive")
        if c.mask_size < 0 or (d.get("mask") is not None and c.mask_size < 1):
            raise ConfigError(f"config.json: {where}mask.size must be positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.mask_size:
            d["mask"] = {"size": self.mask_size}
        return d


@dataclass(frozen=True)
class GatedLinearConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: Optional[int] = None  # None: the inner width of the decay's matrices is read from the tensors

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "GatedLinearConfig":
        c = cls(heads=require(d, "heads", int), dim=require(d, "dim", int), vdim=require(d, "vdim", int), tau=require(d, "tau", float),
                decay_rank=require(d, "decay_rank", int) if d.get("decay_rank") is not None else None)
        if min(c.heads, c.dim, c.vdim) < 1 or not c.tau > 0 or (c.decay_rank is not None and c.decay_rank < 1):
            raise ConfigError(f"config.json: {where}mixer sizes and tau must be positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        return d


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "ExpertsConfig":
        if d.get("kind") != "moe":
            raise ConfigError(f"config.json: {where}mlp.kind must be 'moe', got {d.get('kind')!r}")
        router, expert = _section(d, "router", where), _section(d, "expert", where)
        c = cls(experts=require(router, "experts", int), top=require(router, "top", int), ff=require(expert, "ff", int))
        if not 0 < c.top <= c.experts or c.ff < 1:
            raise ConfigError(f"config.json: {where}router.top must lie in 1..router.experts, expert.ff be positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}


MIXER_CONFIGS = {"attention": BlockAttentionConfig, "gla": GatedLinearConfig}


@dataclass(frozen=True)
class DazilixLayerConfig:
    type: str
    mixer: Union[BlockAttentionConfig, GatedLinearConfig]
    mlp: Optional[ExpertsConfig]


@dataclass(frozen=True)
class DazilixConfig:
    """All sizes and constants of one Dazilix model."""

    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[DazilixLayerConfig, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0  # 0: no stretch of layers repeats
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: int = -1
    extra: dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ConfigError("config.json: 'vocab', 'width' and the number of layers must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        if self.loop_times:
            if self.loop_times < 1 or not 0 <= self.loop_start < self.loop_stop <= len(self.layers):
                raise ConfigError("config.json: 'loop' needs times >= 1 and 0 <= start < stop <= the number of layers")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "DazilixConfig":
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with an entry per layer")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            kind = entry.get("type")
            if kind not in MIXER_CONFIGS:
                raise ConfigError(f"config.json: {where}type {kind!r} is no mixer of this design (known: {sorted(MIXER_CONFIGS)})")
            mlp = entry.get("mlp")
            layers.append(DazilixLayerConfig(type=kind, mixer=MIXER_CONFIGS[kind].from_dict(_section(entry, "mixer", where), where),
                                             mlp=None if mlp is None else ExpertsConfig.from_dict(mlp, where)))
        loop = d.get("loop")
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "layers", "embedding", "loop",
                 "max_position_embeddings", "eos_token_id"}
        return cls(
            vocab=require(d, "vocab", int), width=require(d, "width", int), norm_eps=require(_section(d, "norm", ""), "eps", float),
            embedding_scale=require(d["embedding"], "scale", float) if isinstance(d.get("embedding"), dict) else 1.0, layers=tuple(layers),
            loop_start=require(loop, "start", int) if loop else 0, loop_stop=require(loop, "stop", int) if loop else 0,
            loop_times=require(loop, "times", int) if loop else 0,
            max_position_embeddings=int(d.get("max_position_embeddings") or DEFAULT_MAX_POSITIONS),
            eos_token_id=int(d["eos_token_id"]) if isinstance(d.get("eos_token_id"), int) else -1,
            extra={k: v for k, v in d.items() if k not in known})

    @classmethod
    def from_json(cls, path: str | Path) -> "DazilixConfig":
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers],
        }
        if self.loop_times:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id >= 0:
            d["eos_token_id"] = self.eos_token_id
        return d

    def save(self, folder: str | Path) -> None:
        write_config_json(folder, self.to_dict())


def _run_order(config: DazilixConfig) -> tuple[list[RunSpec], list[PartSpec]]:
    """The runs of the layers and what stands before them: layers before the repeated stretch, the
    stretch `times` times (every pass opened by its entry: the pass's vector, and from the second
    pass on the embedding rows), the layers behind it.  Every run has a cache of its own."""
    n = len(config.layers)
    if not config.loop_times:
        return [RunSpec(layer=i) for i in range(n)], []
    runs = [RunSpec(layer=i) for i in range(config.loop_start)]
    entries = []
    for t in range(config.loop_times):
        entries.append(PartSpec("pass_entry", {"table": "loop.step", "rows": config.loop_times, "row": t, "hidden_size": config.width,
                                               "add_embedding": t > 0}))
        for i in range(config.loop_start, config.loop_stop):
            runs.append(RunSpec(layer=i, before=t if i == config.loop_start else None))
    runs += [RunSpec(layer=i) for i in range(config.loop_stop, n)]
    return runs, entries


@register_architecture(ARCHITECTURE, model_types=("dazilix",), config_from_dict=DazilixConfig.from_dict)
def build_dazilix_spec(config: DazilixConfig) -> ModelSpec:
    W, eps = config.width, config.norm_eps
    layers, ignorable = [], []

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": W, "eps": eps, "weight": name})

    for i, layer in enumerate(config.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "attention":
            position = PartSpec("rotary", {"dim": m.rot_dims, "theta": m.rot_base, "exact_frequencies": True}) if m.rot_dims else None
            mixer = PartSpec("attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "scale": m.scale,
                "qk_norm": "joint", "qk_norm_eps": eps, "values": "keys", "chunk": m.mask_size, "sink": SINK_SCORE, "position": position,
                "q": p + "mix.q", "k": p + "mix.k", "o": p + "mix.o", "q_norm": p + "mix.q.norm", "k_norm": p + "mix.k.norm"})
        else:
            mixer = PartSpec("gated_linear_attention", {
                "hidden_size": W, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "tau": m.tau, "norm_eps": eps,
                "decay_rank": m.decay_rank, "q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "gate": p + "mix.g", "o": p + "mix.o",
                "norm": p + "mix.norm", "decay_in": p + "mix.a1", "decay_out": p + "mix.a2", "decay_bias": p + "mix.a2.b"})
        params: dict[str, Any] = {"hidden_size": W, "mixer": mixer, "mixer_norm": norm(p + "norm1"), "mixer_out_norm": norm(p + "norm1b"),
                                  "mixer_scale": p + "ls1"}
        f = layer.mlp
        if f is None:
            ignorable += [p + "norm2", p + "norm2b", p + "ls2"]  # a layer without a feed-forward has no use for them
        else:
            params.update(
                feed_forward=PartSpec("routed_experts", {
                    "hidden_size": W, "num_experts": f.experts, "top": f.top, "intermediate_size": f.ff, "activation": "swiglu",
                    "score": "softmax_chosen", "weight_on": "output", "router": p + "mlp.router", "router_bias": p + "mlp.router.b",
                    "expert_prefix": p + "mlp.e"}),
                ffn_norm=norm(p + "norm2"), ffn_out_norm=norm(p + "norm2b"), ffn_scale=p + "ls2")
        layers.append(PartSpec("sandwich_norm", params))
    runs, entries = _run_order(config)
    if not config.loop_times:
        ignorable.append("loop.step")
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=W, embedding="embed", layers=layers, final_norm=norm("final.norm"), lm_head="head",
        run_order=runs, run_transforms=entries, embedding_scale=config.embedding_scale, max_positions=config.max_position_embeddings,
        eos_token_id=config.eos_token_id, ignorable_tensors=tuple(ignorable))


# Named models of this design, so that the command lines can run them with random weights.
for _path in sorted(PRESET_DIR.glob("dazilix-*.json")):
    register_preset("dazilix", _path.stem, _path)
