"""The tests' own small Fegetar configurations and weights (no product code here).

The configurations differ from one another in every size and option: head counts, value width
against key width, rotated part wider than what turns in it, latent rank, vocabulary, width, the
order of dense, routed and absent feed-forwards, experts per token, with and without a shared
expert, with and without the pair table and the per-layer token input.  Weights come from the
tests' integer-hash generator under the checkpoint's tensor names.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch

from tests.tiny_configs import seeded_normal


def _mixer(heads, dim, rot_dim, vdim, kv_rank, base, dims):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": float(dim + rot_dim) ** -0.5,
            "rot": {"base": base, "dims": dims}}


def _moe(experts, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


# three heads, values wider than the unrotated keys, only half of the rotated part turns, two experts per token
FEG_A = {
    "architecture": "Fegetar", "vocab": 211, "width": 96, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 5}},
    "token_side": {"dim": 12},
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(3, 24, 16, 40, 40, 10000.0, 8), "mlp": _moe(5, 2, 48, 1.5, (72, 0.75))},
        {"type": "latent_attention", "mixer": _mixer(3, 24, 16, 40, 40, 10000.0, 8), "mlp": {"kind": "dense", "ff": 160}},
        {"type": "latent_attention", "mixer": _mixer(3, 24, 16, 40, 40, 10000.0, 8), "mlp": None},
    ],
}

# one head, sizes that are no multiple of 8, no shared expert, no pair table, layers of different shapes
FEG_B = {
    "architecture": "Fegetar", "vocab": 130, "width": 72, "norm": {"eps": 3e-6},
    "token_side": {"dim": 7},
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(1, 20, 6, 28, 18, 500.0, 6), "mlp": {"kind": "dense", "ff": 100}},
        {"type": "latent_attention", "mixer": _mixer(5, 12, 10, 12, 26, 123456.0, 10), "mlp": _moe(7, 3, 20, 3.0)},
    ],
}

# many heads on a narrow latent, one expert per token, every expert small, no token input
FEG_C = {
    "architecture": "Fegetar", "vocab": 300, "width": 128, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 1000, "mul_prev": 1009, "mul_cur": 17}},
    "layers": [
        {"type": "latent_attention", "mixer": _mixer(8, 16, 16, 16, 32, 1000000.0, 16), "mlp": _moe(9, 1, 32, 2.5, (40, 1.25))},
        {"type": "latent_attention", "mixer": _mixer(8, 16, 16, 16, 32, 1000000.0, 16), "mlp": _moe(4, 4, 24, 0.5, (16, 4.0))},
    ],
}

FEG = {"a": FEG_A, "b": FEG_B, "c": FEG_C}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    V, W, L = cfg["vocab"], cfg["width"], len(cfg["layers"])
    shapes: dict[str, tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    pair = (cfg.get("embedding") or {}).get("bigram")
    if pair:
        shapes["bigram"] = (pair["buckets"] + 1, W)
    side = cfg.get("token_side")
    if side:
        shapes["side.embed"] = (V, L * side["dim"])
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, key = m["heads"], m["dim"] + m["rot_dim"]
        shapes.update({
            p + "norm1": (W,), p + "mix.q": (H * key, W), p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], W), p + "mix.dkv.norm": (m["kv_rank"],),
            p + "mix.uk": (H * m["dim"], m["kv_rank"]), p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.g": (H, W),
            p + "mix.o": (W, H * m["vdim"])})
        mlp = layer["mlp"]
        if mlp:
            shapes[p + "norm2"] = (W,)
            if mlp["kind"] == "dense":
                shapes.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                ff = mlp["expert"]["ff"]
                shapes[p + "mlp.router"] = (mlp["router"]["experts"], W)
                for e in range(mlp["router"]["experts"]):
                    shapes.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
                if mlp.get("shared"):
                    sf = mlp["shared"]["ff"]
                    shapes.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
        if side:
            shapes.update({p + "side.gate": (side["dim"], W), p + "side.proj": (W, side["dim"]), p + "side.norm": (W,)})
    return shapes


def fegetar_weights(cfg: dict, seed: int, *, sharp: float = 1.0, routed_share: float = 1.0, bf16_values: bool = True) -> dict[str, torch.Tensor]:
    """Float32 weights.  Matrices N(0, 1/sqrt(fan_in)) (so activations keep their size, gates and
    routers see both sides of their nonlinearities and the experts' limits bite), norm weights
    around zero (the model's norms) or around one (the latent's and the token input's), the
    tables N(0, 1).  `sharp` multiplies the query matrices: the softmax then picks few keys and one
    wrong key moves the logits far more than rounding does.  `routed_share` scales the norm behind
    every routed feed-forward (1 + w becomes about routed_share): a router is a step function of its
    input, so in a bfloat16 run a few tokens per hundred choose another expert than the float64
    model does; with a small share such a choice moves the logits less than the tolerance and
    every position stays comparable (the routed layer itself is held to the plain one in float32
    here and in both types on its own).  With `bf16_values` every value is
    representable in bfloat16, so a bfloat16 run reads exactly what the plain model reads."""
    routed_norms = {f"l{i}.norm2" for i, layer in enumerate(cfg["layers"]) if layer["mlp"] and layer["mlp"]["kind"] == "moe"}
    out: dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg).items():
        x = seeded_normal(shape, f"fegetar:{seed}:{name}")
        if name in ("embed", "bigram", "side.embed"):
            pass
        elif len(shape) == 1:
            x = 0.1 * x + (1.0 if name.endswith(("dkv.norm", "side.norm")) else 0.0)
            if name in routed_norms and routed_share != 1.0:
                x = routed_share * (1.0 + x) - 1.0
        else:
            x = x / float(shape[1]) ** 0.5
            if name.endswith("mix.q"):
                x = x * sharp
            if ".mlp." in name and name.endswith(("gate", "up")):
                x = x * 2.0  # pre-activations reach the limits
        out[name] = x.to(torch.bfloat16).to(torch.float32) if bf16_values else x
    return out


def write_fegetar_folder(folder: Path, cfg: dict, weights: dict[str, torch.Tensor], dtype: Optional[torch.dtype] = torch.bfloat16) -> Path:
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
