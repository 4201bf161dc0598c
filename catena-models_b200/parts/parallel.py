"""Arrangements for models whose residual stream is float32 whatever the activation dtype.

`SideBySide`: two mixers that read the same input; the result is a_scale * a + b_scale * b.  Each keeps
its own state (the layer's state spec is the pair of theirs).

`ParallelBlock`: one norm, and both sublayers read its output: with n = norm(h), h <- h + (mixer(n) +
feed_forward(n)); the feed-forward may be absent.  The sum of all terms, the float32 residual sum and the
norm of whatever runs next are one kernel (`residual_add_norm`), as the sandwich block's `add_norm` is.

`PreNormBlock`: the sequential arrangement on the same stream: a norm and a mixer, then a norm and a
feed-forward, each sum with a constant factor.

`PostNormBlock`: the norm behind each sum: h <- norm1(c h + mixer(h)), then h <- norm2(c h + feed_forward(h)); the
sublayers read the stream itself.  Optionally followed by an average over the depth of the stack: what the next layer
reads is a weighted sum of the embedding output and of every layer's result so far.

`LoopEntry`: the step between two passes of a looped stack: h <- W [h; h0] + step, h0 being the embedding
rows of the batch (the definition keeps them: `keep_embedding`) and `step` a learned row of the pass.  It
has no norm of its own and no state; the product's float32 result becomes the new residual stream, and the
row is added in the kernel that forms the next block's norm.

Sublayers hand their result over as a tensor or as `kernels.Terms` (pieces with a factor each), and a final
projection may leave its result in float32 (`out_dtype`): nothing is rounded between a projection and
the residual sum.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import CompositeStateSpec
from ..weights.loader import TensorSpec
from .base import Block, Mixer, register_part
from .linear import Linear


def _terms(y):
    return y if isinstance(y, kernels.Terms) else kernels.Terms([(y, 1.0, 1)])


class SideBySide(Mixer):
    prompt_capturable = True
    supports_append = True

    def __init__(self, a, b, a_scale=1.0, b_scale=1.0):
        self.a, self.b, self.a_scale, self.b_scale = a, b, float(a_scale), float(b_scale)

    def children(self):
        return [self.a, self.b]

    def state_spec(self):
        return CompositeStateSpec((self.a.state_spec(), self.b.state_spec()))

    def forward(self, rt, batch, x, state):
        out = kernels.Terms()
        for i, (mixer, scale) in enumerate(((self.a, self.a_scale), (self.b, self.b_scale))):
            view = state.views[i]
            view.owned, view.unit = state.owned, (state.unit, i)
            out += [(e[0], e[1] * scale, *e[2:]) for e in _terms(mixer.forward(rt, batch, x, view))]
        return out


class ParallelBlock(Block):
    prompt_capturable = True
    supports_append = True

    def __init__(self, mixer, feed_forward, input_norm):
        self.mixer, self.feed_forward, self.input_norm = mixer, feed_forward, input_norm

    def children(self):
        return [p for p in (self.input_norm, self.mixer, self.feed_forward) if p is not None]

    def state_spec(self):
        return self.mixer.state_spec()

    def forward(self, rt, batch, h, n, state, next_norm):
        if h.dtype != torch.float32:
            raise ValueError("ParallelBlock works on a float32 residual stream (ModelDefinition.residual_float32)")
        batch.partial_sums_ok = False
        terms = _terms(self.mixer.forward(rt, batch, n, state))
        if self.feed_forward is not None:
            terms = kernels.Terms(terms + _terms(self.feed_forward.forward(rt, batch, n)))
        return _sum_and_norm(rt, h, terms, None, next_norm)


def _sum_and_norm(rt, h, terms, bias, next_norm):
    """h += terms (+ bias); the next norm in the same kernel when it is an RMS norm or a dynamic tanh."""
    kind = getattr(next_norm, "fused_kind", None) if next_norm is not None else None
    fuse = kind in ("rms", "dyt")
    n_out = torch.empty(h.shape, dtype=rt.dtype, device=h.device) if fuse else None
    kernels.residual_add_norm(h, terms, n_out, next_norm.weight if fuse else None, next_norm.eps if fuse else 0.0, bias,
                              dyt=(next_norm.alpha, next_norm.shift) if kind == "dyt" else None)
    return h, n_out


class PreNormBlock(Block):
    """Two sublayers one after the other on a float32 stream, each behind a norm of its own and each added with
    the same constant factor: h <- h + c * mixer(norm1(h)), then h <- h + c * feed_forward(norm2(h)); the
    feed-forward (and its norm) may be absent.  Each sum forms the norm of whatever reads the stream next."""
    prompt_capturable = True
    supports_append = True

    def __init__(self, mixer, feed_forward, input_norm, ffn_norm, residual_scale=1.0):
        if (feed_forward is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer, self.feed_forward, self.input_norm, self.ffn_norm = mixer, feed_forward, input_norm, ffn_norm
        self.residual_scale = float(residual_scale)

    def children(self):
        return [p for p in (self.input_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None]

    def state_spec(self):
        return self.mixer.state_spec()

    def _scaled(self, y):
        return kernels.Terms([(e[0], e[1] * self.residual_scale, *e[2:]) for e in _terms(y)])

    def forward(self, rt, batch, h, n, state, next_norm):
        if h.dtype != torch.float32:
            raise ValueError("PreNormBlock works on a float32 residual stream (ModelDefinition.residual_float32)")
        batch.partial_sums_ok = False
        if n is None:
            n = self.input_norm.apply(rt, h)
        y = self._scaled(self.mixer.forward(rt, batch, n, state))
        if self.feed_forward is None:
            return _sum_and_norm(rt, h, y, None, next_norm)
        h, n2 = _sum_and_norm(rt, h, y, None, self.ffn_norm)
        if n2 is None:
            n2 = self.ffn_norm.apply(rt, h)
        return _sum_and_norm(rt, h, self._scaled(self.feed_forward.forward(rt, batch, n2)), None, next_norm)


class PostNormBlock(Block):
    """Two sublayers one after the other on a float32 stream, each followed by a norm over the sum:
    h <- norm1(c * h + mixer(h)), then h <- norm2(c * h + feed_forward(h)), c = `residual_scale`.  Both sublayers read
    the stream itself (in the activation dtype); the block has no input norm.  The feed-forward may be absent; its norm
    then still runs if it is given (over c * h alone).

    `depth_name` (a tensor of `depth_index + 2` numbers) adds an average over the depth: with X_0 the stream before the
    first block and X_(j+1) the result of block j (before this average), the block leaves sum_j depth[j] * X_j, j = 0 ..
    depth_index + 1, as the stream.  The X_j of a step are kept in StepBatch.shared["depth_history"] (float32
    [entries, rows, width]; entry 0 is filled by the model, ModelDefinition.depth_entries says how many there are).

    Each sum, its norm, the average and the rounding of the result for the next reader's products are one kernel
    (`postnorm_residual`).  A norm is anything with a float32 `weight` row and `eps` (an RMS norm)."""
    prompt_capturable = True
    supports_append = True

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, residual_scale=1.0, depth_name=None, depth_index=0):
        for norm in (mixer_norm, ffn_norm):
            if norm is not None and getattr(norm, "fused_kind", None) != "rms":
                raise ValueError("PostNormBlock: its norms are RMS norms")
        if mixer_norm is None or (feed_forward is not None and ffn_norm is None):
            raise ValueError("PostNormBlock: every sublayer is followed by a norm")
        self.mixer, self.feed_forward, self.mixer_norm, self.ffn_norm = mixer, feed_forward, mixer_norm, ffn_norm
        self.residual_scale = float(residual_scale)
        self.depth_name, self.depth_index = depth_name, int(depth_index)
        self.depth = None

    def children(self):
        return [p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.ffn_norm) if p is not None]

    def tensor_specs(self):
        return [TensorSpec(self.depth_name, (self.depth_index + 2,), "vector")] if self.depth_name else []

    def bind(self, tensors, rt):
        if self.depth_name:
            self.depth = tensors[self.depth_name].to(torch.float32).contiguous()
            self._bound = [self.depth]

    def state_spec(self):
        return self.mixer.state_spec()

    def _sum(self, rt, batch, h, terms, norm, last, cast):
        """h <- norm(c h + terms), then the depth average if this is the block's last sum; the rounded copy if asked."""
        history = None
        if last and self.depth is not None:
            history = batch.shared.get("depth_history")
            if history is None or history.shape[0] < self.depth_index + 2:
                raise ValueError("PostNormBlock: the step's depth history is missing or short (ModelDefinition.depth_entries)")
            history = history[:self.depth_index + 2]
        n_out = torch.empty(h.shape, dtype=rt.dtype, device=h.device) if cast and rt.dtype != torch.float32 else None
        kernels.postnorm_residual(h, terms, self.residual_scale, norm.weight, norm.eps, n_out=n_out, history=history,
                                  coef=self.depth if history is not None else None)
        if not cast:
            return None
        return h if rt.dtype == torch.float32 else n_out

    def forward(self, rt, batch, h, n, state, next_norm):
        if h.dtype != torch.float32:
            raise ValueError("PostNormBlock works on a float32 residual stream (ModelDefinition.residual_float32)")
        batch.partial_sums_ok = False
        if n is None:
            n = h if rt.dtype == torch.float32 else h.to(rt.dtype)
        # the caller forms next_norm itself when there is one (the final norm); else the next block reads the rounded stream
        cast_last = next_norm is None
        y = _terms(self.mixer.forward(rt, batch, n, state))
        if self.ffn_norm is None:
            return h, self._sum(rt, batch, h, y, self.mixer_norm, True, cast_last)
        n1 = self._sum(rt, batch, h, y, self.mixer_norm, False, self.feed_forward is not None)
        f = kernels.Terms()
        if self.feed_forward is not None:
            batch.shared["ff_input_f32"] = h            # a feed-forward that hands its input through takes it unrounded
            f = _terms(self.feed_forward.forward(rt, batch, n1))
            batch.shared.pop("ff_input_f32", None)
        return h, self._sum(rt, batch, h, f, self.ffn_norm, True, cast_last)


class LoopEntry(Block):
    prompt_capturable = True
    supports_append = True

    def __init__(self, in_name, step_name, hidden, passes, index):
        self.hidden, self.passes, self.index, self.step_name = hidden, passes, index, step_name
        self.proj = Linear(in_name, hidden, 2 * hidden)
        self.step = None

    def children(self):
        return [self.proj]

    def tensor_specs(self):
        return [TensorSpec(self.step_name, (self.passes, self.hidden), "vector")]

    def bind(self, tensors, rt):
        self.step = tensors[self.step_name].to(torch.float32)[self.index].contiguous()
        self._bound = [self.step]

    def forward(self, rt, batch, h, n, state, next_norm):
        both = torch.empty((h.shape[0], 2 * self.hidden), dtype=rt.dtype, device=h.device)
        kernels.concat_cast(both, h, batch.shared["embedding"])
        h = self.proj.apply(rt, both, out_dtype=torch.float32)
        return _sum_and_norm(rt, h, kernels.Terms(), self.step, next_norm)


register_part("mixer", "side_by_side", SideBySide)
register_part("block", "parallel", ParallelBlock)
register_part("block", "prenorm", PreNormBlock)
register_part("block", "postnorm", PostNormBlock)
register_part("block", "loop_entry", LoopEntry)
