"""Pre-norm residual block: h += mixer(norm1(h)); h += ffn(norm2(h))
(src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:14-36).  The residual stream h is
float32; the normed activations have the engine's compute type."""
from __future__ import annotations

from .base import PartSpec, Prenormed, build_part, register_part


class PreNormBlock:
    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, feed_forward: PartSpec):
        self.norm1 = build_part("norm", norm1)
        self.mixer = build_part("mixer", mixer)
        self.norm2 = build_part("norm", norm2)
        self.feed_forward = build_part("feed_forward", feed_forward)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    # -- what the model asks a block (never its parts): one entry per mixer it holds ---------------
    def cache_needs(self) -> list:
        return [self.mixer.cache_need()]

    def state_bytes(self) -> list:
        return [int(self.mixer.state_bytes())]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts())

    def tensors(self):
        t = {}
        for p in self.parts():
            t.update(p.tensors())
        return t

    def load(self, weights, device, dtype):
        for p in self.parts():
            p.load(weights, device, dtype)

    def first_norm(self):
        """The norm that this block applies to the residual first, if the part behind it can take a norm's output in
        two pieces (parts.base.Prenormed): the block before may then prepare it in its last product."""
        return self.norm1 if getattr(self.mixer, "takes_prenormed", False) else None

    def forward(self, residual, ctx, slots) -> None:
        x = self.norm1.forward(residual, ctx, ctx.dtype)      # what the block before left behind, or the norm's own kernel
        if isinstance(x, Prenormed) and not getattr(self.mixer, "takes_prenormed", False):
            x = x.materialize(ctx)
        # what the feed-forward streams first, for a mixer whose last kernel can ask for it ahead of time
        ctx.weights_ahead = getattr(self.feed_forward, "first_weights", lambda: None)()
        # the norm that comes next, for a mixer whose last product can prepare it
        ctx.norm_ahead = self.norm2 if getattr(self.feed_forward, "takes_prenormed", False) else None
        self.mixer.forward(x, residual, ctx, slots[0])
        ctx.weights_ahead = ctx.norm_ahead = None
        x = self.norm2.forward(residual, ctx, ctx.dtype)
        if isinstance(x, Prenormed) and not getattr(self.feed_forward, "takes_prenormed", False):
            x = x.materialize(ctx)
        ctx.norm_ahead = ctx.next_first_norm
        self.feed_forward.forward(x, residual, ctx)
        ctx.norm_ahead = None


register_part("block", "pre_norm", PreNormBlock)


class SandwichBlock:
    """A block with a norm before AND after each sublayer, and an optional short convolution in front of each:

        h = norm1(x);  h = h + conv1(h);  x += norm1b(mixer(h))
        h = norm2(x);  h = h + conv2(h);  x += norm2b(ff(h))          (no feed-forward: the second line is absent)

    The convolutions run over time on each channel (parts.conv.ShortConv); their last inputs are state of the
    sequence, which this block asks the model for beside its mixer's: cache_needs() / state_bytes() have the mixer's
    entry first, then one entry for each convolution it holds.  A sublayer's output is collected in a float32 buffer and
    joins the residual through the norm after it.  Mixers and feed-forwards add into what they are given, so the buffer
    starts from zeros; a part that says `can_store = True` takes `store=True` and overwrites it instead (no zeroing)."""

    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm1_after: PartSpec, norm2: PartSpec | None = None,
                 feed_forward: PartSpec | None = None, norm2_after: PartSpec | None = None, conv1: dict | None = None,
                 conv2: dict | None = None):
        from .conv import ShortConv
        self.norm1 = build_part("norm", norm1)
        self.mixer = build_part("mixer", mixer)
        self.norm1_after = build_part("norm", norm1_after)
        self.feed_forward = build_part("feed_forward", feed_forward) if feed_forward is not None else None
        self.norm2 = build_part("norm", norm2) if feed_forward is not None else None
        self.norm2_after = build_part("norm", norm2_after) if feed_forward is not None else None
        self.conv1 = ShortConv(add_input=True, **conv1) if conv1 is not None else None
        self.conv2 = ShortConv(add_input=True, **conv2) if conv2 is not None and feed_forward is not None else None

    def parts(self):
        return tuple(p for p in (self.norm1, self.conv1, self.mixer, self.norm1_after, self.norm2, self.conv2,
                                 self.feed_forward, self.norm2_after) if p is not None)

    def _convs(self):
        return [c for c in (self.conv1, self.conv2) if c is not None]

    def cache_needs(self) -> list:
        return [self.mixer.cache_need()] + [None for _ in self._convs()]

    def state_bytes(self) -> list:
        return [int(self.mixer.state_bytes())] + [c.state_bytes() for c in self._convs()]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts())

    def tensors(self):
        t = {}
        for p in self.parts():
            t.update(p.tensors())
        return t

    def load(self, weights, device, dtype):
        for p in self.parts():
            p.load(weights, device, dtype)

    def first_norm(self):
        return None   # what reads the residual first here is followed by a convolution, which wants the plain rows

    def forward(self, residual, ctx, slots) -> None:
        import torch
        conv_slots = list(slots[1:])
        ctx.weights_ahead = ctx.norm_ahead = None
        h = self.norm1.forward(residual, ctx, ctx.dtype, fresh=True)
        if self.conv1 is not None:
            h = self.conv1.forward(h, ctx, conv_slots.pop(0))
        if getattr(self.mixer, "can_store", False):
            branch = torch.empty_like(residual)
            self.mixer.forward(h, branch, ctx, slots[0], store=True)
        else:
            branch = torch.zeros_like(residual)
            self.mixer.forward(h, branch, ctx, slots[0])
        ctx.prenormed = None
        if self.feed_forward is None:
            self.norm1_after.add_into(branch, residual)
            return
        h = self.norm1_after.add_into_then(branch, residual, self.norm2, ctx.dtype)
        if self.conv2 is not None:
            h = self.conv2.forward(h, ctx, conv_slots.pop(0))
        if getattr(self.feed_forward, "can_store", False):
            self.feed_forward.forward(h, branch, ctx, store=True)
        else:
            branch.zero_()
            self.feed_forward.forward(h, branch, ctx)
        ctx.prenormed = None
        self.norm2_after.add_into(branch, residual)


register_part("block", "sandwich", SandwichBlock)
