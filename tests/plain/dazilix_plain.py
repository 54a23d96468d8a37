"""Plain, slow Dazilix: whole sequences, no cache, one function per mechanism.

Dazilix is a decoder-only model whose layers wrap each sublayer in two norms and a learned
per-channel scale (x <- x + s * N_out(f(N_in(x)))).  A layer's mixer is either a softmax
attention that sees only the keys of its own block of positions, has a sink in the softmax's
denominator and uses the unnormed, unrotated key projection as its values, or a gated linear
attention with a decay per key channel.  The feed-forward is a set of routed SwiGLU experts whose
weights are the softmax over the chosen router logits.  A run of layers may repeat with the same
weights; every repetition starts from the stream plus the embedding rows plus a learned vector.

Everything here runs on whole sequences in one dtype (float64 by default) on the CPU and shares
no code with the engine under test.  `config` is the content of a config.json as a dict,
`weights` a dict of tensors under the checkpoint's names.
"""

from __future__ import annotations

import math
from typing import Callable, Mapping, Optional, Sequence

import torch

Weights = Mapping[str, torch.Tensor]


# ---------------------------------------------------------------------------
# small functions


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """Rows divided by their root mean square, eps under the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ---------------------------------------------------------------------------
# embedding and the order of the layer runs


def embed(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64) -> torch.Tensor:
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    return weights["embed"].to(dtype)[ids] * float(config["embedding"]["scale"])


def run_plan(config: dict) -> list[tuple[int, Optional[int]]]:
    """(layer, pass number if this run opens a pass of the repeated stretch, else None), in run order."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or int(loop["times"]) < 1 or int(loop["stop"]) <= int(loop["start"]):
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    plan: list[tuple[int, Optional[int]]] = [(i, None) for i in range(a)]
    for t in range(times):
        plan += [(i, t if i == a else None) for i in range(a, b)]
    plan += [(i, None) for i in range(b, n)]
    return plan


def open_pass(x: torch.Tensor, x0: torch.Tensor, t: int, weights: Weights) -> torch.Tensor:
    """What happens right before the first layer of pass t: the embedding rows come back in (not in
    the first pass), then the pass's own vector is added."""
    if t > 0:
        x = x + x0
    return x + weights["loop.step"].to(x.dtype)[t]


# ---------------------------------------------------------------------------
# rotation (halves paired)


def rotate_halves(x: torch.Tensor, positions: Sequence[int], base: float, dims: int) -> torch.Tensor:
    """x [T, heads, n]: entry i < dims/2 is paired with entry i + dims/2 and the pair turns by
    position * base^(-2i/dims); entries from `dims` on stay."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.as_tensor(base, dtype=torch.float64) ** (-2.0 * i / dims)
    ang = torch.as_tensor(list(positions), dtype=torch.float64)[:, None] * freq[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------
# mixer: attention inside blocks of positions, with a sink


def sink_softmax(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    """exp(s_j) / (1 + sum over the visible j of exp(s_j)); rows [.., keys]."""
    e = torch.where(visible, torch.exp(scores), torch.zeros_like(scores))
    return e / (1.0 + e.sum(-1, keepdim=True))


def block_mask(positions: Sequence[int], size: int) -> torch.Tensor:
    """[T, T] True where key j is visible to query i: j <= i and both in the same block of `size` positions."""
    p = torch.as_tensor(list(positions), dtype=torch.long)
    return (p[None, :] <= p[:, None]) & ((p[None, :] // size) == (p[:, None] // size))


def attention_mixer(h: torch.Tensor, positions: Sequence[int], m: dict, prefix: str, weights: Weights, eps: float) -> torch.Tensor:
    T, dt = h.shape[0], h.dtype
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    w = lambda name: weights[prefix + name].to(dt)
    q_flat, k_flat = h @ w("q").T, h @ w("k").T
    values = k_flat.reshape(T, G, d)  # the key projection as it comes, before norm and rotation
    q = norm(q_flat, w("q.norm"), eps).reshape(T, H, d)  # one norm over all heads' entries together
    k = norm(k_flat, w("k.norm"), eps).reshape(T, G, d)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_halves(q, positions, float(rot["base"]), int(rot["dims"]))
    k = rotate_halves(k, positions, float(rot["base"]), int(rot["dims"]))
    visible = block_mask(positions, int(m["mask"]["size"]))
    out = torch.empty(T, H, d, dtype=dt)
    for head in range(H):
        g = head // (H // G)
        scores = (q[:, head] @ k[:, g].T) * float(m["scale"])
        out[:, head] = sink_softmax(scores, visible) @ values[:, g]
    return out.reshape(T, H * d) @ w("o").T


# ---------------------------------------------------------------------------
# mixer: gated linear attention


def gla_decay(h: torch.Tensor, m: dict, prefix: str, weights: Weights) -> torch.Tensor:
    """[T, heads * dim] decay per key channel: sigmoid(z)^(1/tau), z from two stacked matrices and a bias."""
    dt = h.dtype
    z = (h @ weights[prefix + "a1"].to(dt).T) @ weights[prefix + "a2"].to(dt).T + weights[prefix + "a2.b"].to(dt)
    return torch.exp(torch.nn.functional.logsigmoid(z) / float(m["tau"]))


def gla_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                   state: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """One head, token by token.  q, k, decay [T, d]; v [T, e]; state [d, e].  The row of the state
    that belongs to key channel c shrinks by decay[t, c] before k_t v_t^T is added; o_t = S_t^T q_t."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=q.dtype) if state is None else state.clone()
    out = torch.empty(T, v.shape[1], dtype=q.dtype)
    for t in range(T):
        S = decay[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out[t] = S.T @ q[t]
    return out, S


def gla_mixer(h: torch.Tensor, m: dict, prefix: str, weights: Weights, eps: float) -> torch.Tensor:
    T, dt = h.shape[0], h.dtype
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    w = lambda name: weights[prefix + name].to(dt)
    q = (h @ w("q").T).reshape(T, H, d) * d ** -0.5
    k = (h @ w("k").T).reshape(T, H, d)
    v = (h @ w("v").T).reshape(T, H, e)
    decay = gla_decay(h, m, prefix, weights).reshape(T, H, d)
    out = torch.empty(T, H, e, dtype=dt)
    for head in range(H):
        o, _ = gla_recurrence(q[:, head], k[:, head], v[:, head], decay[:, head])
        out[:, head] = norm(o, w("norm"), eps)  # one weight of size e for every head
    gated = out.reshape(T, H * e) * silu(h @ w("g").T)
    return gated @ w("o").T


# ---------------------------------------------------------------------------
# feed-forward: routed SwiGLU experts


def route(h: torch.Tensor, f: dict, prefix: str, weights: Weights) -> tuple[torch.Tensor, torch.Tensor]:
    """Chosen experts [T, top] (largest logits first) and their weights: softmax over the chosen logits."""
    dt = h.dtype
    logits = h @ weights[prefix + "router"].to(dt).T + weights[prefix + "router.b"].to(dt)
    top = torch.topk(logits, int(f["router"]["top"]), dim=-1)
    return top.indices, torch.softmax(top.values, dim=-1)


def expert(h: torch.Tensor, prefix: str, weights: Weights) -> torch.Tensor:
    dt = h.dtype
    return (silu(h @ weights[prefix + "gate"].to(dt).T) * (h @ weights[prefix + "up"].to(dt).T)) @ weights[prefix + "down"].to(dt).T


def routed_feed_forward(h: torch.Tensor, f: dict, prefix: str, weights: Weights) -> torch.Tensor:
    chosen, share = route(h, f, prefix, weights)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(chosen.shape[1]):
            out[t] += share[t, j] * expert(h[t:t + 1], f"{prefix}e{int(chosen[t, j])}.", weights)[0]
    return out


# ---------------------------------------------------------------------------
# a layer and the model


def layer(x: torch.Tensor, positions: Sequence[int], i: int, config: dict, weights: Weights) -> torch.Tensor:
    entry, eps, p, dt = config["layers"][i], float(config["norm"]["eps"]), f"l{i}.", x.dtype
    w = lambda name: weights[p + name].to(dt)
    h = norm(x, w("norm1"), eps)
    if entry["type"] == "attention":
        y = attention_mixer(h, positions, entry["mixer"], p + "mix.", weights, eps)
    elif entry["type"] == "gla":
        y = gla_mixer(h, entry["mixer"], p + "mix.", weights, eps)
    else:
        raise ValueError(f"unknown mixer {entry['type']!r}")
    x = x + norm(y, w("norm1b"), eps) * w("ls1")
    if entry.get("mlp") is not None:
        y = routed_feed_forward(norm(x, w("norm2"), eps), entry["mlp"], p + "mlp.", weights)
        x = x + norm(y, w("norm2b"), eps) * w("ls2")
    return x


def forward_stream(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64,
                   after_run: Optional[Callable[[int, torch.Tensor], None]] = None) -> torch.Tensor:
    positions = list(range(len(tokens)))
    x0 = embed(tokens, weights, config, dtype)
    x = x0
    for n, (i, opens) in enumerate(run_plan(config)):
        if opens is not None:
            x = open_pass(x, x0, opens, weights)
        x = layer(x, positions, i, config, weights)
        if after_run is not None:
            after_run(n, x)
    return x


def forward_logits(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64) -> torch.Tensor:
    x = forward_stream(tokens, weights, config, dtype)
    return norm(x, weights["final.norm"].to(dtype), float(config["norm"]["eps"])) @ weights["head"].to(dtype).T
