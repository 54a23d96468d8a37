"""The tests' own small Dazilix configurations and weights (no product code here).

The configurations differ from one another in every size and option: head counts and grouping,
head widths that are no multiple of 8, how much of a head turns (nothing, a part, all of it),
block lengths below, at and across the cache's page size, the order of the two mixers, layers
without a feed-forward, experts per token (one included), where the repeated stretch of layers
lies and how often it runs (not at all included).  Weights come from the tests' integer-hash
generator under the checkpoint's tensor names.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch

from tests.tiny_configs import seeded_normal


def _att(heads, kv_heads, dim, mask, rot_dims, base=10000.0, scale=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                                           "scale": float(dim) ** -0.5 if scale is None else scale,
                                           "rot": {"base": base, "dims": rot_dims}, "mask": {"size": mask}}}


def _gla(heads, dim, vdim, tau):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# both mixers; the stretch in the middle runs twice; a layer without a feed-forward; a third of a head turns
DAZ_A = {
    "architecture": "Dazilix", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer(_att(4, 2, 24, 16, 8), _moe(5, 2, 40)),
        _layer(_gla(3, 20, 28, 8.0), None),
        _layer(_att(4, 2, 24, 16, 8), _moe(5, 2, 40)),
        _layer(_gla(3, 20, 28, 8.0), _moe(7, 3, 24)),
    ],
}

# the recurrent mixer alone: one head with odd widths, many heads with narrow ones; one expert per token; nothing repeats
DAZ_B = {
    "architecture": "Dazilix", "vocab": 130, "width": 72, "norm": {"eps": 3e-6}, "embedding": {"scale": 1.0},
    "layers": [
        _layer(_gla(1, 7, 10, 3.5), _moe(3, 1, 20)),
        _layer(_gla(6, 36, 12, 24.0), _moe(4, 4, 16)),
    ],
}

# attention alone: every query head with its own keys, or all with one; whole heads turn, or nothing; blocks shorter than a
# page and blocks that no page size divides; the first two layers run three times
DAZ_C = {
    "architecture": "Dazilix", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        _layer(_att(6, 6, 16, 8, 16, base=500.0, scale=0.3), _moe(9, 3, 32)),
        _layer(_att(5, 1, 12, 40, 0), None),
        _layer(_att(2, 2, 64, 24, 32, base=123456.0), _moe(2, 1, 48)),
    ],
}

# heads of 128 (the widths at which prompt attention runs on the tcgen05 kernel), one key/value head for both query heads,
# blocks of 48 positions; a recurrent layer as wide; the first layer alone runs twice
DAZ_D = {
    "architecture": "Dazilix", "vocab": 180, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
    "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [
        _layer(_att(2, 1, 128, 48, 64), _moe(6, 2, 64)),
        _layer(_gla(2, 128, 64, 12.0), None),
    ],
}

# for one long request: blocks of 512 and 1,024 positions (a decoded token's keys are then split over several CTAs, a far key
# is hundreds of positions back), heads of 128 and of 64, two recurrent layers of different shapes, the middle stretch twice
DAZ_LONG = {
    "architecture": "Dazilix", "vocab": 500, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer(_att(8, 2, 128, 512, 64), _moe(8, 2, 96)),
        _layer(_gla(4, 32, 64, 16.0), _moe(8, 2, 96)),
        _layer(_att(4, 4, 64, 1024, 32, scale=0.2), None),
        _layer(_gla(2, 128, 128, 8.0), _moe(3, 1, 64)),
    ],
}

DAZ = {"a": DAZ_A, "b": DAZ_B, "c": DAZ_C, "d": DAZ_D}
DECAY_RANK = {"a": 6, "b": 5, "c": 0, "d": 8}  # the inner width of the decay's matrices: in no configuration key, only in the tensors


def tensor_shapes(cfg: dict, decay_rank: int) -> dict[str, tuple[int, ...]]:
    V, W = cfg["vocab"], cfg["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if cfg.get("loop"):
        shapes["loop.step"] = (cfg["loop"]["times"], W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes.update({p + "norm1": (W,), p + "norm1b": (W,), p + "ls1": (W,)})
        if layer["type"] == "attention":
            nq, nk = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            shapes.update({p + "mix.q": (nq, W), p + "mix.k": (nk, W), p + "mix.q.norm": (nq,), p + "mix.k.norm": (nk,), p + "mix.o": (W, nq)})
        else:
            hd, he = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            shapes.update({p + "mix.q": (hd, W), p + "mix.k": (hd, W), p + "mix.v": (he, W), p + "mix.g": (he, W), p + "mix.o": (W, he),
                           p + "mix.norm": (m["vdim"],), p + "mix.a1": (decay_rank, W), p + "mix.a2": (hd, decay_rank), p + "mix.a2.b": (hd,)})
        mlp = layer["mlp"]
        if mlp:
            shapes.update({p + "norm2": (W,), p + "norm2b": (W,), p + "ls2": (W,)})
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            shapes.update({p + "mlp.router": (E, W), p + "mlp.router.b": (E,)})
            for e in range(E):
                shapes.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
    return shapes


def dazilix_weights(cfg: dict, seed: int, *, decay_rank: int, sharp: float = 1.0, routed_share: float = 1.0) -> dict[str, torch.Tensor]:
    """Float32 weights whose values are all representable in bfloat16 (a bfloat16 run reads exactly
    what the plain model reads).  Matrices N(0, 1/fan_in), norm weights and scales around one,
    biases around zero (the decay's around two, so that states live for tens of tokens), the
    embedding and the passes' vectors N(0, 1).  `sharp` multiplies the query norm's weights: the
    softmax then picks few keys and one wrong key moves the logits far more than rounding does.
    `routed_share` multiplies the scale behind every feed-forward: a router is a step function of
    its input, so in a bfloat16 run a few tokens per hundred choose another expert than the float64
    model; with a small share such a choice moves the logits less than the tolerance."""
    out: dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        x = seeded_normal(shape, f"dazilix:{seed}:{name}")
        if name in ("embed", "loop.step"):
            pass
        elif name.endswith("router.b"):
            x = 0.5 * x
        elif name.endswith("a2.b"):
            x = 2.0 + x
        elif len(shape) == 1:
            x = 1.0 + 0.1 * x
            if name.endswith("q.norm"):
                x = x * sharp
            if name.endswith("ls2"):
                x = x * routed_share
        else:
            x = x / float(shape[1]) ** 0.5
            if name.endswith(("mix.a2", "mlp.router")):
                x = x * 2.0  # decays and routers that depend on the token
        out[name] = x.to(torch.bfloat16).to(torch.float32)
    return out


def write_dazilix_folder(folder: Path, cfg: dict, weights: dict[str, torch.Tensor], dtype: Optional[torch.dtype] = torch.bfloat16) -> Path:
    """config.json + model.safetensors, written with the safetensors package (not the engine's writer)."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: (v if dtype is None else v.to(dtype)).contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder


def random_ids(cfg: dict, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
