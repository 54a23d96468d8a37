"""Plain, slow Fegetar: whole sequences, no cache, one function per mechanism.

Fegetar is a decoder-only model of post-normed layers (the norm sits on a sublayer's output:
x <- x + N(f(x)), and f reads x itself) around latent attention (keys and values are rebuilt
from one low-rank row per token plus one shared rotated key part), a dense or a routed
feed-forward, and a per-layer gated input from a second token table; its embedding adds a row
of a hashed table of (previous token, token) pairs.

Everything here runs on whole sequences in one dtype (float64 by default) on the CPU and shares
no code with the engine under test.  `config` is the content of a config.json as a dict,
`weights` a dict of tensors under the checkpoint's names.
"""

from __future__ import annotations

import math
from typing import Mapping, Optional, Sequence

import torch

Weights = Mapping[str, torch.Tensor]


# ---------------------------------------------------------------------------
# small functions


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    """z/2 * (1 + tanh(sqrt(2/pi) * (z + 0.044715 z^3)))."""
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """Rows divided by their root mean square, eps under the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The model's norm: the stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


# ---------------------------------------------------------------------------
# embedding


def pair_rows(tokens: Sequence[int], mul_prev: int, mul_cur: int, buckets: int) -> list[int]:
    """Row of the pair table for every token: a hash of (token before, token); the first token
    of a sequence has nothing before it and takes the extra row behind the hashed ones."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def embed(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64) -> torch.Tensor:
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = weights["embed"].to(dtype)[ids]
    pair = (config.get("embedding") or {}).get("bigram")
    if pair:
        rows = pair_rows(tokens, int(pair["mul_prev"]), int(pair["mul_cur"]), int(pair["buckets"]))
        x = x + weights["bigram"].to(dtype)[torch.as_tensor(rows, dtype=torch.long)]
    return x


# ---------------------------------------------------------------------------
# rotation of neighbouring pairs


def rotate_pairs(x: torch.Tensor, positions: Sequence[int], base: float, dims: int) -> torch.Tensor:
    """x [T, ..., n]: entries (2i, 2i+1), i < dims/2, turn by the angle p * base^(-2i/dims);
    what lies behind `dims` stays."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = torch.as_tensor(base, dtype=torch.float64) ** (-2.0 * i / dims)
    ang = torch.as_tensor(list(positions), dtype=torch.float64)[:, None] * freq[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = ang.cos().to(x.dtype).view(shape), ang.sin().to(x.dtype).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ---------------------------------------------------------------------------
# latent attention


def latent_attention(h: torch.Tensor, positions: Sequence[int], weights: Weights, prefix: str, mixer: dict, eps: float,
                     probe: Optional[dict] = None) -> torch.Tensor:
    """h [T, width] -> [T, width].  Per token one latent row c (normed) and one rotated key part
    r, shared by all heads; head a's key is [U_k,a c ; r], its value U_v,a c."""
    dtype = h.dtype
    W = lambda name: weights[prefix + name].to(dtype)  # noqa: E731
    H, dn, dr, dv, rank = int(mixer["heads"]), int(mixer["dim"]), int(mixer["rot_dim"]), int(mixer["vdim"]), int(mixer["kv_rank"])
    rot = mixer["rot"]
    T = h.shape[0]
    q = (h @ W("q").T).view(T, H, dn + dr)
    down = h @ W("dkv").T
    c = norm_plain(down[:, :rank], W("dkv.norm"), eps)
    r = rotate_pairs(down[:, rank:], positions, float(rot["base"]), int(rot["dims"]))  # [T, dr]
    q_plain = q[..., :dn]
    q_rot = rotate_pairs(q[..., dn:], positions, float(rot["base"]), int(rot["dims"]))  # [T, H, dr]
    k_plain = (c @ W("uk").T).view(T, H, dn)
    v = (c @ W("uv").T).view(T, H, dv)
    scores = torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thd,sd->hts", q_rot, r)
    scores = scores * float(mixer["scale"])
    pos = torch.as_tensor(list(positions))
    hidden = pos[None, :] > pos[:, None]  # key s after query t
    scores = scores.masked_fill(hidden[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    if probe is not None:
        probe["weights"] = p
    o = torch.einsum("hts,shd->thd", p, v)
    gate = torch.sigmoid(h @ W("g").T)  # [T, H]
    o = o * gate[..., None]
    return o.reshape(T, H * dv) @ W("o").T


# ---------------------------------------------------------------------------
# feed-forward layers


def dense_ff(h: torch.Tensor, weights: Weights, prefix: str) -> torch.Tensor:
    dtype = h.dtype
    return gelu_tanh(h @ weights[prefix + "up"].to(dtype).T) @ weights[prefix + "down"].to(dtype).T


def capped_expert(h: torch.Tensor, weights: Weights, prefix: str, limit: float) -> torch.Tensor:
    """a = min(G h, limit), b = clamp(U h, -limit, limit); D (a sigmoid(1.702 a) (b + 1))."""
    dtype = h.dtype
    a = (h @ weights[prefix + "gate"].to(dtype).T).clamp(max=limit)
    b = (h @ weights[prefix + "up"].to(dtype).T).clamp(min=-limit, max=limit)
    return (a * torch.sigmoid(1.702 * a) * (b + 1.0)) @ weights[prefix + "down"].to(dtype).T


def route(h: torch.Tensor, weights: Weights, prefix: str, top: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Sigmoid scores; per token the `top` largest, with their scores as they are."""
    s = torch.sigmoid(h @ weights[prefix + "router"].to(h.dtype).T)
    w, e = torch.topk(s, top, dim=-1)
    return e, w


def routed_ff(h: torch.Tensor, weights: Weights, prefix: str, mlp: dict) -> torch.Tensor:
    """sum over the chosen experts of expert(score * h), plus the shared expert on h."""
    top = int(mlp["router"]["top"])
    chosen, score = route(h, weights, prefix, top)
    out = torch.zeros_like(h)
    limit = float(mlp["expert"]["limit"])
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(chosen[t, j])
            out[t] += capped_expert(score[t, j] * h[t : t + 1], weights, f"{prefix}e{e}.", limit)[0]
    if mlp.get("shared"):
        out = out + capped_expert(h, weights, prefix + "shared.", float(mlp["shared"]["limit"]))
    return out


# ---------------------------------------------------------------------------
# per-layer token input


def token_side(x: torch.Tensor, tokens: Sequence[int], layer: int, weights: Weights, prefix: str, dim: int, eps: float) -> torch.Tensor:
    """What is added to x: D (gelu(G x) * e), unit-normed and weighted; e is the layer's slice of
    the token's row in the second table."""
    dtype = x.dtype
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    e = weights["side.embed"].to(dtype)[ids][:, layer * dim : (layer + 1) * dim]
    g = gelu_tanh(x @ weights[prefix + "gate"].to(dtype).T) * e
    y = g @ weights[prefix + "proj"].to(dtype).T
    return norm_plain(y, weights[prefix + "norm"].to(dtype), eps)


# ---------------------------------------------------------------------------
# the model


def forward(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64,
            positions: Optional[Sequence[int]] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Logits [T, vocab] and the residual stream after every layer [layers, T, width]."""
    eps = float(config["norm"]["eps"])
    positions = list(range(len(tokens))) if positions is None else list(positions)
    x = embed(tokens, weights, config, dtype)
    side = config.get("token_side")
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] != "latent_attention":
            raise ValueError(f"unknown mixer {layer['type']}")
        m = latent_attention(x, positions, weights, p + "mix.", layer["mixer"], eps)
        x = x + norm_around_zero(m, weights[p + "norm1"].to(dtype), eps)
        mlp = layer.get("mlp")
        if mlp:
            f = dense_ff(x, weights, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(x, weights, p + "mlp.", mlp)
            x = x + norm_around_zero(f, weights[p + "norm2"].to(dtype), eps)
        if side:
            x = x + token_side(x, tokens, i, weights, p + "side.", int(side["dim"]), eps)
        after.append(x)
    logits = norm_around_zero(x, weights["final.norm"].to(dtype), eps) @ weights["head"].to(dtype).T
    return logits, torch.stack(after)
