"""Arrangements of mixer, feed-forward and norms in one layer."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import (
    Block,
    BuildContext,
    LayerCache,
    PartSpec,
    PreNormed,
    ResidualNorm,
    Rounded,
    StepContext,
    TensorSpec,
    build_part,
    register_part,
)


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """h = h + Mixer(Norm_a(h)); h = h + FeedForward(Norm_f(h))  (engine/nn/layers.py:111-121).

    The residual stream is float32.  Each branch output is handed on as `pending` and
    added by the next norm in the same pass that norms it, so a residual sum never costs
    a pass over memory of its own.
    """

    def __init__(self, ctx: BuildContext, *, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, ffn_norm: PartSpec) -> None:
        self.dtype = ctx.dtype
        self.mixer = build_part("mixer", mixer, ctx)
        self.feed_forward = build_part("feed_forward", feed_forward, ctx)
        self.mixer_norm = build_part("norm", mixer_norm, ctx)
        self.ffn_norm = build_part("norm", ffn_norm, ctx)
        self._parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)
        self.graph_safe = all(p.graph_safe for p in self._parts)
        # the block itself only hands tensors on; before a part that reads them by other means
        # than this package's ops, products that still wait in a chain are launched
        self.reads_through_ops = True

    def tensor_specs(self) -> list[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load(tensors)

    def entry_norm(self):
        return self.mixer_norm

    def forward(self, hidden, pending, step: StepContext, cache: LayerCache):
        """`pending`: None, the last branch output not yet added to `hidden`, or a PreNormed that
        stands for mixer_norm(hidden) (the part before prepared it; `hidden` is then complete).

        Where mixer and feed-forward offer it (`folds_norms`, and `can_fold` for this step), the
        norms and residual sums between them are folded into their products: the mixer's last
        product adds into `hidden` and prepares the feed-forward's input, the feed-forward's last
        product does the same for `step.norm_after`.  Otherwise every norm is a step of its own."""
        T = hidden.shape[0]
        if isinstance(pending, Rounded):  # the block before handed on rounded rows, no branch: nothing to add
            pending = None
        after_block, norm_after = step.weight_after, step.norm_after
        mixer_folds = self.mixer.folds_norms and self.mixer.can_fold(T, self.dtype)
        ffn_folds = self.feed_forward.folds_norms and self.feed_forward.can_fold(T, self.dtype)

        if isinstance(pending, PreNormed) and mixer_folds:
            x = pending
        else:
            x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
            self._before(self.mixer_norm)
            self.mixer_norm.forward(hidden, None if isinstance(pending, PreNormed) else pending, x)
        step.weight_after = self.feed_forward.first_weight()
        ffn_norm = self.ffn_norm.params()
        self._before(self.mixer)
        if mixer_folds and ffn_folds and ffn_norm is not None:
            x = self.mixer.forward(x, step, cache, fold=ResidualNorm(hidden, ffn_norm))
        else:
            mixed = self.mixer.forward(x, step, cache)
            x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
            self._before(self.ffn_norm)
            self.ffn_norm.forward(hidden, mixed, x)
        step.weight_after = after_block
        next_norm = norm_after.params() if norm_after is not None else None
        self._before(self.feed_forward)
        if ffn_folds and next_norm is not None:
            return self.feed_forward.forward(x, step, fold=ResidualNorm(hidden, next_norm))
        return self.feed_forward.forward(x, step)

    @staticmethod
    def _before(part) -> None:
        if not part.reads_through_ops:
            ops.flush_gemm_chain()

    def first_weight(self):
        return self.mixer.first_weight()


@register_part("block", "post_norm")
class PostNormBlock(Block):
    """h = h + Norm_a(Mixer(h)); h = h + Norm_f(FeedForward(h)); h = h + Norm_e(Extra(h)).

    The norm sits on each sublayer's output and the sublayers read the residual stream itself.
    `feed_forward` and `extra` (a second feed-forward-like sublayer, for instance a per-layer
    token input) may each be absent.  The residual stream is float32; a sublayer reads its rows
    rounded to the compute dtype, which the norm kernel of the sublayer before writes in the same
    pass that adds into the stream (`Norm.forward_branch`), and the last one hands them to the
    next block as a `Rounded`.
    """

    def __init__(self, ctx: BuildContext, *, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: Optional[PartSpec] = None,
                 ffn_norm: Optional[PartSpec] = None, extra: Optional[PartSpec] = None, extra_norm: Optional[PartSpec] = None) -> None:
        if (feed_forward is None) != (ffn_norm is None) or (extra is None) != (extra_norm is None):
            raise ValueError("post_norm block: a sublayer and its norm come together")
        self.dtype = ctx.dtype
        self.mixer = build_part("mixer", mixer, ctx)
        self.mixer_norm = build_part("norm", mixer_norm, ctx)
        self.feed_forward = None if feed_forward is None else build_part("feed_forward", feed_forward, ctx)
        self.ffn_norm = None if ffn_norm is None else build_part("norm", ffn_norm, ctx)
        self.extra = None if extra is None else build_part("feed_forward", extra, ctx)
        self.extra_norm = None if extra_norm is None else build_part("norm", extra_norm, ctx)
        self._parts = tuple(p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.ffn_norm, self.extra, self.extra_norm) if p is not None)
        self.graph_safe = all(p.graph_safe for p in self._parts)
        self.reads_through_ops = True

    def tensor_specs(self) -> list[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load(tensors)

    def first_weight(self):
        return self.mixer.first_weight()

    def _rows(self, hidden: torch.Tensor, pending) -> torch.Tensor:
        """The stream's rows in the compute dtype: the stream itself in a float32 run, else what the
        sublayer before left, else a rounding pass."""
        if self.dtype == torch.float32:
            return hidden
        if isinstance(pending, Rounded) and pending.x.dtype == self.dtype:
            return pending.x
        x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
        ops.round_rows(hidden, x)
        return x

    def _add(self, norm, branch: torch.Tensor, hidden: torch.Tensor):
        PreNormBlock._before(norm)
        if self.dtype == torch.float32:
            norm.forward_branch(branch, hidden)
            return hidden
        x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
        norm.forward_branch(branch, hidden, x)
        return x

    def forward(self, hidden, pending, step: StepContext, cache: LayerCache):
        if isinstance(pending, torch.Tensor):  # a branch that the block before did not add
            ops.residual_add(hidden, pending)
            pending = None
        x = self._rows(hidden, pending)
        after_block = step.weight_after
        step.weight_after = None
        PreNormBlock._before(self.mixer)
        x = self._add(self.mixer_norm, self.mixer.forward(x, step, cache), hidden)
        for part, norm in ((self.feed_forward, self.ffn_norm), (self.extra, self.extra_norm)):
            if part is None:
                continue
            PreNormBlock._before(part)
            branch = part.forward(x, step, residual=hidden) if part.wants_residual else part.forward(x, step)
            x = self._add(norm, branch, hidden)
        step.weight_after = after_block
        return None if self.dtype == torch.float32 else Rounded(x)
