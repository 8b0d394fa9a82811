"""Arrangement of a layer's parts.

parallel_residual (further down): x += mult * (Mixer(norm(x)) + FeedForward(norm(x))), with one norm for both
sublayers or one each.

pre_norm_residual (src/dense.rs:178-194):
    x += [post_norm](Mixer(norm(x)));  x += [post_norm](FeedForward(norm(x)))
The norms after the mixer and after the feed-forward are the reference's own lfm3 layout and
are present only when the layer names them.  The residual x is float and is added to in float.

In a decode step of a few bfloat16 rows a norm kernel costs more in launch latency than in work,
so there the block splits a norm between the product that wrote x last and the product that
reads norm(x) first (ops.kernels.SplitNorm), when both parts say they can (`split_norm`); in
every other case the norm runs as a kernel of its own.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import BLOCKS


@BLOCKS.register("pre_norm_residual")
class PreNormResidualBlock:
    def __init__(self, mixer, ffn, mixer_norm, ffn_norm, post_mixer_norm=None, post_ffn_norm=None):
        self.mixer, self.ffn = mixer, ffn
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.post_mixer_norm, self.post_ffn_norm = post_mixer_norm, post_ffn_norm

    def parts(self) -> dict[str, object]:
        p = {"mixer": self.mixer, "ffn": self.ffn, "mixer_norm": self.mixer_norm, "ffn_norm": self.ffn_norm}
        if self.post_mixer_norm is not None:
            p["post_mixer_norm"] = self.post_mixer_norm
        if self.post_ffn_norm is not None:
            p["post_ffn_norm"] = self.post_ffn_norm
        return p

    def first_reader(self):
        """(norm, part) that read the residual when this block starts: the block before may split that norm."""
        return self.mixer_norm, self.mixer

    def _offer(self, producer, norm, consumer, x, env, which: int):
        """Before `producer` adds into x: if `norm` (the next reader of x) can be split between it
        and `consumer`, asks the producer to leave its half.  Returns the split or None."""
        M, D = x.shape
        if not (getattr(norm, "splittable", False) and getattr(producer, "split_norm", False)
                and getattr(consumer, "split_norm", False)):
            return None
        reader = getattr(consumer, "split_reader_weight", None)
        if not kernels.split_norm_ok(M, env.dtype, reader() if callable(reader) else None):
            return None      # the product that would read the split's values could not scale its rows
        ws = env.workspace
        sp = kernels.SplitNorm(ws.get(f"block.split.values{which}", (M, D), torch.bfloat16),
                               ws.get(f"block.split.ssq{which}", (M, -(-D // 16)), torch.float32),
                               norm.weight, norm.eps)
        env.split_out = sp
        return sp

    def _normed(self, norm, x, pending, env):
        """norm(x) as the next part's input: the split's values (the part scales its first product),
        or the norm kernel's result."""
        env.split_in = env.split_out = None   # nothing is left over from a part that did not take its offer (or raised)
        if pending is not None and pending.filled and pending.weight is norm.weight:
            env.split_in = pending
            return pending.values
        M, D = x.shape
        h = env.workspace.get("block.h", (M, D), env.dtype)
        norm.forward(h, x)
        return h

    def forward(self, x: torch.Tensor, batch, cache, env, pending=None):
        """Runs the layer on the residual x.  `pending`: the split of this block's first norm that
        the block before left, if it did; returns the split of the next block's first norm
        (`env.next_block_norm`) if this block's feed-forward left one."""
        M, D = x.shape
        ws = env.workspace
        h = self._normed(self.mixer_norm, x, pending, env)
        if self.post_mixer_norm is None:
            mid = self._offer(self.mixer, self.ffn_norm, self.ffn, x, env, 0)
            self.mixer.forward(h, x, True, batch, cache, env)
        else:
            mid = None
            t = ws.get("block.t", (M, D), torch.float32)
            self.mixer.forward(h, t, False, batch, cache, env)
            self.post_mixer_norm.forward(x, t, add=True)
        env.split_in = None
        h = self._normed(self.ffn_norm, x, mid, env)
        if self.post_ffn_norm is None:
            nxt = env.next_block_norm
            last = None
            if nxt is not None:
                norm, consumer = nxt
                last = self._offer(self.ffn, norm, consumer, x, env, 1)
            self.ffn.forward(h, x, True, batch, env)
        else:
            last = None
            t = ws.get("block.t", (M, D), torch.float32)
            self.ffn.forward(h, t, False, batch, env)
            self.post_ffn_norm.forward(x, t, add=True)
        env.split_in = env.split_out = None
        return last if last is not None and last.filled else None


class NormedRows:
    """The norm of the residual stream as a block left it for the block after it."""

    filled = False      # not the half of a split norm: a block that splits norms passes it by

    def __init__(self, values: torch.Tensor, norm):
        self.values, self.norm = values, norm


@BLOCKS.register("gated_pre_norm_residual")
class GatedPreNormResidualBlock:
    """x += s1 * Mixer(h1), h1 = norm1(x);  x += s2 * FeedForward(h2), h2 = norm2(x), where each
    s = gate(h) is computed from the sublayer's own input (parts.gate) and multiplies the sublayer's
    result element by element; a gate that is absent leaves the plain sum.  A layer may have no
    feed-forward: it then ends after the first sum.  The residual and both sums are float.

    Fused steps: the kernel that adds a gated result into x also leaves the norm of the new x for the
    sublayer that follows (in this block, or the first of the next block when that is of this
    arrangement too and nothing is added to the stream in between), so a layer runs one norm kernel
    at most; and a mixer that can (`absorb_input_rows`) forms the gate's product R h in its own
    first product."""

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm, post_mixer_norm=None, post_ffn_norm=None,
                 mixer_gate=None, ffn_gate=None):
        if post_mixer_norm is not None or post_ffn_norm is not None:
            raise ValueError("the gated arrangement has no norms after its sublayers")
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together or not at all")
        self.mixer, self.ffn = mixer, ffn
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.mixer_gate, self.ffn_gate = mixer_gate, ffn_gate
        self._folded: bool | None = None      # whether the mixer forms its gate's product (decided at the first step)

    def parts(self) -> dict[str, object]:
        p = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.ffn is not None:
            p["ffn"], p["ffn_norm"] = self.ffn, self.ffn_norm
        if self.mixer_gate is not None:
            p["mixer_gate"] = self.mixer_gate
        if self.ffn_gate is not None and self.ffn is not None:
            p["ffn_gate"] = self.ffn_gate
        return p

    def first_reader(self):
        """(norm, reader) of the stream when this block starts; the reader is the block itself, so
        only a block of this arrangement leaves the norm's result for it."""
        return self.mixer_norm, self

    def _next(self, env):
        """The next block's first norm, if this block's last sum may leave its result."""
        nxt = env.next_block_norm
        if nxt is not None and isinstance(nxt[1], GatedPreNormResidualBlock):
            return nxt[0]
        return None

    def forward(self, x: torch.Tensor, batch, cache, env, pending=None):
        M, D = x.shape
        ws = env.workspace
        env.split_in = env.split_out = None
        if self._folded is None:
            self._folded = self.mixer_gate is not None and self.mixer_gate.give_rows_to(self.mixer)
        if isinstance(pending, NormedRows) and pending.norm is self.mixer_norm and pending.values.shape == (M, D):
            h = pending.values
        else:
            h = ws.get("block.h", (M, D), env.dtype)
            self.mixer_norm.forward(h, x)
        # the norm that reads x after each sum, and where its result goes (two buffers: h is still the gate's input)
        after_mixer = self.ffn_norm if self.ffn is not None else self._next(env)
        h2 = ws.get("block.h2" if h is ws.get("block.h", (M, D), env.dtype) else "block.h", (M, D), env.dtype)
        left = None
        if self.mixer_gate is None:
            self.mixer.forward(h, x, True, batch, cache, env)
            if self.ffn is not None:
                self.ffn_norm.forward(h2, x)
        else:
            y = ws.get("block.t", (M, D), torch.float32)
            self.mixer.forward(h, y, False, batch, cache, env)
            z = self.mixer.extra_out if self._folded else None
            self.mixer_gate.add_gated(x, y, h, env, z=z, next_norm=after_mixer, h_out=h2 if after_mixer is not None else None)
            if self.ffn is None and after_mixer is not None:
                left = NormedRows(h2, after_mixer)
        if self.ffn is None:
            return left
        after_ffn = self._next(env)
        if self.ffn_gate is None:
            self.ffn.forward(h2, x, True, batch, env)
            return None
        y = ws.get("block.t", (M, D), torch.float32)
        self.ffn.forward(h2, y, False, batch, env)
        self.ffn_gate.add_gated(x, y, h2, env, next_norm=after_ffn, h_out=h if after_ffn is not None else None)
        return NormedRows(h, after_ffn) if after_ffn is not None else None


@BLOCKS.register("parallel_residual")
class ParallelResidualBlock:
    """h = norm(x);  x += mult * (Mixer(h) + FeedForward(h)): both sublayers read the stream as it was before
    the layer, their results are summed in float and enter the stream together, times a constant.  With one
    norm both read its result; with `ffn_norm` the feed-forward reads a norm of its own (two layer norms of
    the same row share its mean and variance and are formed by one launch).  A layer may have no feed-forward.
    The kernel that adds the sum into x also leaves the norm (or the two norms) of the new x for the next block
    when that is of this arrangement too (with layer norms) and nothing is added to the stream in between, so a
    model runs one norm kernel, for its first layer."""

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm=None, post_mixer_norm=None, post_ffn_norm=None,
                 mult: float = 1.0):
        if post_mixer_norm is not None or post_ffn_norm is not None:
            raise ValueError("the parallel arrangement has its norms in front of the sublayers")
        if ffn_norm is not None and ffn is None:
            raise ValueError("a feed-forward's norm without a feed-forward")
        if ffn_norm is not None and (getattr(ffn_norm, "has_bias", True) or getattr(mixer_norm, "has_bias", True)
                                     or ffn_norm.eps != mixer_norm.eps):
            raise ValueError("two norms in front of parallel sublayers: layer norms without bias and with one eps")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self.mult = float(mult)

    def parts(self) -> dict[str, object]:
        p = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.ffn is not None:
            p["ffn"] = self.ffn
        if self.ffn_norm is not None:
            p["ffn_norm"] = self.ffn_norm
        return p

    def first_reader(self):
        return self.mixer_norm, self

    def forward(self, x: torch.Tensor, batch, cache, env, pending=None):
        from .norm import LayerNorm
        M, D = x.shape
        ws = env.workspace
        env.split_in = env.split_out = None
        two = self.ffn_norm is not None
        first_set = ("block.h", "block.hb")
        if (isinstance(pending, NormedRows) and pending.norm is self.mixer_norm and pending.values.shape == (M, D)
                and (not two or getattr(pending, "second_norm", None) is self.ffn_norm)):
            h = pending.values
            hf = pending.second if two else h
        else:
            h = ws.get(first_set[0], (M, D), env.dtype)
            if two:
                hf = ws.get(first_set[1], (M, D), env.dtype)
                kernels.layernorm_pair(h, hf, x, self.mixer_norm.weight, self.ffn_norm.weight, self.mixer_norm.eps)
            else:
                hf = h
                self.mixer_norm.forward(h, x)
        y = ws.get("block.t", (M, D), torch.float32)
        self.mixer.forward(h, y, False, batch, cache, env)
        if self.ffn is not None:
            self.ffn.forward(hf, y, True, batch, env)
        nxt = env.next_block_norm
        after = nxt[1] if nxt is not None and isinstance(nxt[1], ParallelResidualBlock) and isinstance(nxt[0], LayerNorm) \
            and not nxt[0].has_bias else None
        if after is None:
            kernels.scaled_residual(x, y, self.mult)
            return None
        names = ("block.h2", "block.hb2") if h is ws.get(first_set[0], (M, D), env.dtype) else first_set
        h2 = ws.get(names[0], (M, D), env.dtype)
        if after.ffn_norm is not None:
            hf2 = ws.get(names[1], (M, D), env.dtype)
            kernels.layernorm_pair(h2, hf2, x, after.mixer_norm.weight, after.ffn_norm.weight, after.mixer_norm.eps,
                                   y=y, mult=self.mult)
            left = NormedRows(h2, after.mixer_norm)
            left.second, left.second_norm = hf2, after.ffn_norm
            return left
        kernels.scaled_residual(x, y, self.mult, h=h2, norm_w=after.mixer_norm.weight, eps=after.mixer_norm.eps)
        return NormedRows(h2, after.mixer_norm)


class StreamRows:
    """The residual stream in the activation type, as a block left it for a block that reads the stream itself."""

    filled = False      # not the half of a split norm
    norm = None

    def __init__(self, values: torch.Tensor):
        self.values = values


@BLOCKS.register("post_norm_residual")
class PostNormResidualBlock:
    """x <- norm1(alpha x + Mixer(x));  x <- norm2(alpha x + FeedForward(x)): the sublayers read the stream
    itself and the norm comes after each sum, with a constant `alpha` on the stream's side of it.  A layer may
    have no feed-forward: it then ends after the first norm.  The stream, the sums and the norms are float; the
    sublayers get the stream in the activation type.  The kernel that norms a sum also leaves the new stream in
    the activation type for the sublayer that reads it next (in this block, or the first of the next block when
    that is of this arrangement too and nothing is added to the stream in between), so the stream is cast by a
    kernel of its own only in front of the model's first layer."""

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm=None, post_mixer_norm=None, post_ffn_norm=None,
                 alpha: float = 1.0):
        if post_mixer_norm is not None or post_ffn_norm is not None:
            raise ValueError("the post-norm arrangement names its two norms mixer_norm and ffn_norm")
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together or not at all")
        for n in (mixer_norm, ffn_norm):
            if n is not None and not hasattr(n, "bias"):
                raise ValueError("the post-norm arrangement takes layer norms")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self.alpha = float(alpha)

    def parts(self) -> dict[str, object]:
        p = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.ffn is not None:
            p["ffn"], p["ffn_norm"] = self.ffn, self.ffn_norm
        return p

    def first_reader(self):
        """(norm, reader): no norm stands in front of this block; the reader is the block itself, so a
        block of this arrangement before it leaves the stream in the activation type."""
        return None, self

    def forward(self, x: torch.Tensor, batch, cache, env, pending=None):
        M, D = x.shape
        ws = env.workspace
        env.split_in = env.split_out = None
        f32 = env.is_float32
        if f32:
            h = x        # the sublayers read the stream where it is; they write elsewhere
        elif isinstance(pending, StreamRows) and pending.values.shape == (M, D):
            h = pending.values
        else:
            h = ws.get("block.h", (M, D), env.dtype)
            kernels.cast_rows(h, x)
        other = None if f32 else ws.get("block.h2" if h is ws.get("block.h", (M, D), env.dtype) else "block.h", (M, D), env.dtype)
        nxt = env.next_block_norm
        feeds_next = (not f32) and nxt is not None and isinstance(nxt[1], PostNormResidualBlock)
        y = ws.get("block.t", (M, D), torch.float32)
        self.mixer.forward(h, y, False, batch, cache, env)
        n1 = self.mixer_norm
        if self.ffn is None:
            kernels.postnorm_residual(x, y, self.alpha, n1.weight, n1.bias, n1.eps, h=other if feeds_next else None)
            return StreamRows(other) if feeds_next else None
        kernels.postnorm_residual(x, y, self.alpha, n1.weight, n1.bias, n1.eps, h=other)
        h2 = x if f32 else other
        self.ffn.forward(h2, y, False, batch, env)
        n2 = self.ffn_norm
        kernels.postnorm_residual(x, y, self.alpha, n2.weight, n2.bias, n2.eps, h=h if feeds_next else None)
        return StreamRows(h) if feeds_next else None
