"""Gated linear attention as a mixer part: a recurrence with a decay per key channel, whose state
per request lives in a float32 state slot of the cache."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, CacheNeed, LayerCache, Mixer, StepContext, TensorSpec, register_part
from tokensprint_b200.parts.linear import linear


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    """Per head, with key width d and value width e, for the tokens of a sequence in order:

        q_t = W_q x_t * q_scale,  k_t = W_k x_t,  v_t = W_v x_t
        a_t = sigmoid(W_a2 (W_a1 x_t) + b)^(1/tau)       one decay per key channel, through a narrow
                                                          pair of matrices
        S_t = diag(a_t) S_(t-1) + k_t v_t^T               S [d, e], zero before the first token
        o_t = S_t^T q_t
        y_t = W_o ( concat over heads of  norm(o_t) * silu(W_g x_t) )

    where norm is an RMS norm over the e entries of a head with one weight [e] for all heads.

    Parameters: `hidden_size`, `num_heads`, `key_dim`, `value_dim`, `tau`, `q_scale` (default
    key_dim^-0.5), `norm_eps`, `decay_rank` (the inner width of the decay's pair of matrices; None:
    whatever the checkpoint's tensors have) and the tensors' names.  The projections of x that
    share its rows (q, k, v, the output gate, the decay's first matrix) are stacked at load into
    one product.  Decays, their logarithms, the state, the recurrence and the head norm are
    float32 whatever the compute dtype; the state is carried from step to step in the request's
    slot (`CacheNeed.state_shape` = [heads, key_dim, value_dim]), so prompts may be cut anywhere.
    """

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, tau: float, norm_eps: float,
                 q: str, k: str, v: str, gate: str, o: str, norm: str, decay_in: str, decay_out: str, decay_bias: Optional[str] = None,
                 decay_rank: Optional[int] = None, q_scale: Optional[float] = None) -> None:
        self.hidden_size, self.num_heads, self.key_dim, self.value_dim = int(hidden_size), int(num_heads), int(key_dim), int(value_dim)
        self.tau, self.norm_eps = float(tau), float(norm_eps)
        if min(self.num_heads, self.key_dim, self.value_dim) < 1 or not self.tau > 0:
            raise ValueError("gated linear attention: heads, key_dim, value_dim and tau must be positive")
        if self.key_dim > ops.GLA_MAX_KEY_DIM:
            raise ValueError(f"gated linear attention: key_dim {key_dim} exceeds the kernel's {ops.GLA_MAX_KEY_DIM}")
        self.q_scale = float(q_scale) if q_scale is not None else float(self.key_dim) ** -0.5
        self.decay_rank = None if decay_rank is None else int(decay_rank)
        self.names = {"q": q, "k": k, "v": v, "gate": gate, "o": o, "norm": norm, "decay_in": decay_in, "decay_out": decay_out,
                      "decay_bias": decay_bias}
        self.dtype = ctx.dtype
        self.in_weight: Optional[torch.Tensor] = None  # [q | k | v | gate | decay_in] stacked
        self.decay_out: Optional[torch.Tensor] = None
        self.decay_bias: Optional[torch.Tensor] = None
        self.norm_weight: Optional[torch.Tensor] = None
        self.o_weight: Optional[torch.Tensor] = None

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.in_weight

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", state_shape=(self.num_heads, self.key_dim, self.value_dim), state_dtype=torch.float32)

    def tensor_specs(self) -> list[TensorSpec]:
        W, n = self.hidden_size, self.names
        hd, he = self.num_heads * self.key_dim, self.num_heads * self.value_dim
        r = -1 if self.decay_rank is None else self.decay_rank
        specs = [TensorSpec(n["q"], (hd, W)), TensorSpec(n["k"], (hd, W)), TensorSpec(n["v"], (he, W)), TensorSpec(n["gate"], (he, W)),
                 TensorSpec(n["o"], (W, he)), TensorSpec(n["norm"], (self.value_dim,), "vector"),
                 TensorSpec(n["decay_in"], (r, W)), TensorSpec(n["decay_out"], (hd, r))]
        if n["decay_bias"] is not None:
            specs.append(TensorSpec(n["decay_bias"], (hd,), "vector"))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        decay_in, self.decay_out = tensors[n["decay_in"]], tensors[n["decay_out"]]
        if decay_in.shape[0] != self.decay_out.shape[1]:
            raise ValueError(f"gated linear attention: {n['decay_in']} has {decay_in.shape[0]} rows, {n['decay_out']} {self.decay_out.shape[1]} columns")
        self.rank = int(decay_in.shape[0])
        self.in_weight = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]], decay_in], dim=0).contiguous()
        self.decay_bias = tensors[n["decay_bias"]] if n["decay_bias"] is not None else None
        self.norm_weight, self.o_weight = tensors[n["norm"]], tensors[n["o"]]

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        if cache.state is None:
            raise ops.KernelError("gated linear attention: this mixer needs a state slot per request (none was bound to its run)")
        if not cache.writes:
            raise ops.KernelError("gated linear attention: a run cannot read another run's state")
        T, H, d, e = x.shape[0], self.num_heads, self.key_dim, self.value_dim
        hd, he = H * d, H * e
        proj = linear(x, self.in_weight, next_weight=self.decay_out)
        q, k, v = proj[:, :hd], proj[:, hd:2 * hd], proj[:, 2 * hd:2 * hd + he]
        gate, low = proj[:, 2 * hd + he:2 * hd + 2 * he], proj[:, 2 * hd + 2 * he:]
        z = linear(low, self.decay_out, next_weight=self.o_weight)
        o = torch.empty((T, he), device=x.device, dtype=torch.float32)
        ops.gla_scan(q, k, v, z, self.decay_bias, self.tau, self.q_scale, cache.state, step.state_slots, step.cu_seqlens_q, o,
                     step.num_seqs, H, d, e, max_seqlen=step.max_seqlen_q)
        y = torch.empty((T, he), device=x.device, dtype=x.dtype)
        ops.gla_norm_gate(o, gate, self.norm_weight, y, H, e, self.norm_eps)
        return linear(y, self.o_weight, next_weight=step.weight_after)
