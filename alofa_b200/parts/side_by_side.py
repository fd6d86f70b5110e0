"""Several mixers side by side on the same input: each makes its output in a
buffer of its own, each output is RMS-normed over the model width with a plain
weight of its own (``<prefix><name>.out``), and their mean is added into the
residual stream (two branches: half the sum).  The branches keep their own
caches (pages, state slots), so this mixer's cache is the tuple of theirs."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from .base import Part, TensorSpec, as_float32_vector, build_part, register_part


class SideBySide(Part):
    family = "mixer"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.param("hidden_size"))
        self.eps = float(self.param("eps"))
        self.names = [str(n) for n in self.param("names")]
        self.branches = [build_part("mixer", s, rt) for s in self.param("branches")]
        if len(self.names) != len(self.branches) or not self.branches:
            raise AlofaError("invalid_argument", "side_by_side needs a name for every branch", f"names={self.names}")
        self.weights = None

    @property
    def graph_safe(self):
        return all(b.graph_safe for b in self.branches)

    def cache_spec(self):
        return tuple(b.cache_spec() for b in self.branches)

    def scratch_row_bytes(self) -> int:
        return 4 * self.hidden * len(self.branches) + sum(getattr(b, "scratch_row_bytes", lambda: 0)() for b in self.branches)

    def tensors(self):
        t = {}
        for name, b in zip(self.names, self.branches):
            t.update(b.tensors())
            t[self.prefix + name + ".out"] = TensorSpec((self.hidden,), "ones")
        return t

    def load(self, state):
        for b in self.branches:
            b.load(state)
        self.weights = [as_float32_vector(state[self.prefix + name + ".out"]) for name in self.names]

    def forward(self, ctx, x, h, cache, writes=True):
        outs = []
        for b, c in zip(self.branches, cache):
            y = ctx.buf(tuple(h.shape), torch.float32)
            if getattr(b, "stores_output", False):
                b.forward(ctx, x, y, c, writes, store=True)
            else:
                ctx.flush_pending()
                y.zero_()
                b.forward(ctx, x, y, c, writes)
                ctx.flush_pending()
            outs.append(y)
        ctx.flush_pending()  # the sums below go into h itself
        scale = 1.0 / len(outs)
        for i in range(0, len(outs), 2):
            pair = outs[i : i + 2]
            ops.branch_norm_add(h, pair[0], self.weights[i], pair[1] if len(pair) > 1 else None, self.weights[i + 1] if len(pair) > 1 else None, self.eps, scale)


register_part("mixer", "side_by_side", SideBySide)
