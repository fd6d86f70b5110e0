"""How one layer arranges its parts.

``sandwich_residual``: a norm before and a norm after each sublayer,
``h += norm_b(mixer(norm_a(h))); h += norm_d(feed_forward(norm_c(h)))``; the
feed-forward may be absent.  ``embedding_mix_in``: no sublayers at all, ``h =
W [h; e]`` with ``e`` the embedding output of the step's tokens.

``parallel_residual``: one norm whose output both sublayers read,
``x = norm(h); h += mixer(x) + feed_forward(x)`` (the feed-forward may be
absent).  ``embedding_add``: no sublayers, ``h += e``.

``prenorm_residual``: ``h += mixer(norm_a(h)); h += feed_forward(norm_b(h))``
(src/alofa/model/arch/qwen.mojo:1367-1372, 1418-1510).  The residual stream
``h`` is fp32; the parts add into it."""
from __future__ import annotations

from ..csrc import ops
from .base import Part, TensorSpec, build_part, register_part
from .linear import STORE, Linear


class PrenormResidual(Part):
    family = "block"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer = build_part("mixer", self.param("mixer"), rt)
        self.feed_forward = build_part("feed_forward", self.param("feed_forward"), rt)
        self.mixer_norm = build_part("norm", self.param("mixer_norm"), rt)
        self.feed_forward_norm = build_part("norm", self.param("feed_forward_norm"), rt)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def tensors(self):
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, state):
        for part in self.parts():
            part.load(state)

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def scratch_row_bytes(self) -> int:
        return sum(getattr(part, "scratch_row_bytes", lambda: 0)() for part in self.parts())

    absorbs_pending = True  # its norms add partial sums owed to h; other readers get them flushed first

    def _norm(self, norm, ctx, h, reader):
        if not getattr(norm, "absorbs_pending", False):
            ctx.flush_pending()
            return norm.forward(ctx, h)
        # a reader that says so may get rows still to be made (the norm folded into its own product)
        if getattr(reader, "takes_normed_rows", False) and getattr(norm, "gives_normed_rows", False):
            return norm.forward(ctx, h, lazy=True)
        return norm.forward(ctx, h)

    def forward(self, ctx, h, cache, writes=True):
        x = self._norm(self.mixer_norm, ctx, h, self.mixer)
        self.mixer.forward(ctx, x, h, cache, writes)
        x = self._norm(self.feed_forward_norm, ctx, h, self.feed_forward)
        self.feed_forward.forward(ctx, x, h)


class SandwichResidual(Part):
    """Norms on both sides of each sublayer.  The sublayer's output goes to an
    fp32 buffer of its own (parts that say ``stores_output`` write it, any
    other part adds into a zeroed one); one kernel then normalises it, adds it
    to the stream and, for the mixer, also yields the normed input of the
    feed-forward."""

    family = "block"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer = build_part("mixer", self.param("mixer"), rt)
        self.mixer_norm = build_part("norm", self.param("mixer_norm"), rt)
        self.mixer_post = build_part("norm", self.param("mixer_post_norm"), rt)
        ff = self.params.get("feed_forward")
        self.feed_forward = build_part("feed_forward", ff, rt) if ff is not None else None
        self.feed_forward_norm = build_part("norm", self.param("feed_forward_norm"), rt) if ff is not None else None
        self.feed_forward_post = build_part("norm", self.param("feed_forward_post_norm"), rt) if ff is not None else None

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post, self.feed_forward_norm, self.feed_forward, self.feed_forward_post) if p is not None)

    def tensors(self):
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, state):
        for part in self.parts():
            part.load(state)

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def scratch_row_bytes(self) -> int:
        return 12 * self.mixer_norm.size + sum(getattr(part, "scratch_row_bytes", lambda: 0)() for part in self.parts())

    def _sublayer(self, ctx, part, x, h, *args):
        """The part's output for the rows ``x``, fp32, in a buffer of its own."""
        y = ctx.buf(tuple(h.shape), h.dtype)
        if getattr(part, "stores_output", False):
            part.forward(ctx, x, y, *args, store=True)
        else:
            y.zero_()
            part.forward(ctx, x, y, *args)
            ctx.flush_pending()
        return y

    def forward(self, ctx, h, cache, writes=True):
        x = self.mixer_norm.forward(ctx, h)
        y = self._sublayer(ctx, self.mixer, x, h, cache, writes)
        if self.feed_forward is None:
            ops.sandwich_norm(h, y, self.mixer_post.weight, self.mixer_post.eps)
            return
        x = ctx.buf(tuple(h.shape), self.rt.dtype)
        ops.sandwich_norm(h, y, self.mixer_post.weight, self.mixer_post.eps, x, self.feed_forward_norm.weight, self.feed_forward_norm.eps)
        y = self._sublayer(ctx, self.feed_forward, x, h)
        ops.sandwich_norm(h, y, self.feed_forward_post.weight, self.feed_forward_post.eps)


class EmbeddingMixIn(Part):
    """``h = W [h; e]``: the stream and the embedding output ``e`` of the same
    tokens, side by side, through one matrix [hidden, 2 * hidden] (the stream's
    columns first).  It keeps no cache; the model keeps ``e`` for the step."""

    family = "block"
    graph_safe = True
    needs_embedding_output = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.param("hidden_size"))
        self.name = self.prefix + str(self.params.get("weight_name", "weight"))
        self.linear = None

    def tensors(self):
        return {self.name: TensorSpec((self.hidden, 2 * self.hidden))}

    def load(self, state):
        self.linear = Linear(state[self.name], None, STORE)

    def cache_spec(self):
        return None

    def scratch_row_bytes(self) -> int:
        return 8 * self.hidden

    def forward(self, ctx, h, cache, writes=True):
        both = ctx.buf((h.shape[0], 2 * self.hidden), self.rt.dtype)
        ops.concat_rows(both, h, ctx.embedding_output)
        self.linear(h, both, buf=ctx.buf)


class ParallelResidual(Part):
    """One norm, and the mixer and the feed-forward side by side on its
    output; each adds what it makes into the fp32 stream."""

    family = "block"
    absorbs_pending = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.norm = build_part("norm", self.param("norm"), rt)
        self.mixer = build_part("mixer", self.param("mixer"), rt)
        ff = self.params.get("feed_forward")
        self.feed_forward = build_part("feed_forward", ff, rt) if ff is not None else None

    def parts(self):
        return tuple(p for p in (self.norm, self.mixer, self.feed_forward) if p is not None)

    def tensors(self):
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, state):
        for part in self.parts():
            part.load(state)

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def scratch_row_bytes(self) -> int:
        return sum(getattr(part, "scratch_row_bytes", lambda: 0)() for part in self.parts())

    def forward(self, ctx, h, cache, writes=True):
        if not getattr(self.norm, "absorbs_pending", False):
            ctx.flush_pending()
        x = self.norm.forward(ctx, h)
        # the feed-forward first: it adds into h itself, while the mixer's last product may leave sums for the next reader to add
        if self.feed_forward is not None:
            ctx.flush_pending()
            self.feed_forward.forward(ctx, x, h)
        self.mixer.forward(ctx, x, h, cache, writes)


class EmbeddingAdd(Part):
    """``h += e`` with ``e`` the embedding output of the step's tokens: what a
    stretch of layers that runs several times gets before each further pass."""

    family = "block"
    graph_safe = True
    needs_embedding_output = True

    def cache_spec(self):
        return None

    def forward(self, ctx, h, cache, writes=True):
        ctx.flush_pending()
        ops.add_rows(h, ctx.embedding_output)


register_part("block", "prenorm_residual", PrenormResidual)
register_part("block", "parallel_residual", ParallelResidual)
register_part("block", "embedding_add", EmbeddingAdd)
register_part("block", "sandwich_residual", SandwichResidual)
register_part("block", "embedding_mix_in", EmbeddingMixIn)
