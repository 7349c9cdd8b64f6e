"""minGRU: a gated recurrence whose gates read only the current token.

For a token's input h: z = sigmoid(Wz h + bz), u = Wx h + bx, candidate = u + 1/2 where u >= 0 and
sigmoid(u) below, state S_t = (1 - z) S_(t-1) + z candidate element by element, output
Wo (S_t * silu(Wg h)).  The state has `width` lanes, starts at zero, is float32 and lives in the
request's state slot.  The three input projections are one stacked product (a fourth may ride
along, see `take_side`); gates, candidate, recurrence and the product with silu are one kernel
(`csrc/recurrence.cu`), 32-bit whatever the products' precision.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.store import TensorSpec
from .base import CacheNeed, StateNeed, register_part
from .linear import Linear


class SideProjection:
    """Mixers and feed-forwards whose first step is a product of their input may carry one more
    projection of the same input in that product (`take_side(weight, bias)`, CPU tensors as
    stored): its result of the last `forward` is `side_pre` [T, rows of weight], float32, still
    lacking `side_bias`.  The arrangement of a layer uses it for a gate on the sublayer's output.
    The stacked product is computed WITHOUT its biases: `stack_bias` (float32, one a column, or
    None) is added by the kernels that consume the columns, which spares a pass over the product."""

    side_rows = 0
    side_pre = None
    side_bias = None
    stack_bias = None

    def _stack(self, runtime, weights, biases, side):
        """One Linear over `weights` stacked row-wise (+ the side projection); `biases` are
        per-weight float tensors or None (zeros)."""
        self.side_rows = 0
        if side is not None:
            weights, biases = weights + [side[0]], biases + [side[1]]
            self.side_rows = side[0].shape[0]
        self.own_rows = sum(w.shape[0] for w in weights) - self.side_rows
        self.stack_bias = self.side_bias = None
        if any(b is not None for b in biases):
            bias = torch.cat([torch.zeros(w.shape[0], dtype=torch.float32, device=w.device) if b is None
                              else b.to(torch.float32) for w, b in zip(weights, biases)])
            self.stack_bias = runtime.vector(bias)
            if self.side_rows and biases[-1] is not None:
                self.side_bias = self.stack_bias[self.own_rows:]
        return Linear(runtime.matrix(torch.cat(weights, dim=0)))

    def _keep_side(self, product):
        self.side_pre = product[:, self.own_rows:] if self.side_rows else None


class MinGRU(SideProjection):
    graph_safe = True    # launches depend on device-side metadata alone

    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        hidden, width = p["hidden_size"], p["width"]
        return [TensorSpec(x + ".z", (width, hidden)), TensorSpec(x + ".z.b", (width,)),
                TensorSpec(x + ".x", (width, hidden)), TensorSpec(x + ".x.b", (width,)),
                TensorSpec(x + ".g", (width, hidden)), TensorSpec(x + ".o", (hidden, width))]

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.hidden, self.width = int(p["hidden_size"]), int(p["width"])
        self._own = ([store.get(x + ".z"), store.get(x + ".x"), store.get(x + ".g")],
                     [store.get(x + ".z.b"), store.get(x + ".x.b"), None])
        self.inputs = self._stack(runtime, list(self._own[0]), list(self._own[1]), None)
        self.out = Linear(runtime.matrix(store.get(x + ".o")))

    def take_side(self, weight, bias):
        self.inputs = self._stack(self.runtime, list(self._own[0]), list(self._own[1]), (weight, bias))

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.width,)))

    def shape_key(self, q_lens):
        return "scan1" if max(q_lens) == 1 else "scan"

    def streamed_weights(self):
        return [self.inputs.weight, self.out.weight]

    def forward(self, h, ctx, cache):
        w = self.width
        product = self.inputs.forward(h, out_dtype=torch.float32)
        y = self.runtime.empty(ctx.n_tokens, w)
        ops.min_gru_scan(product, 0, w, 2 * w, w, cache.state, ctx.q_start, ctx.state_slot,
                         max(ctx.max_q_len, 1), y, bias=self.stack_bias)
        self._keep_side(product)
        return self.out.forward(y, partials_ok=True)


register_part("mixer", "min_gru", MinGRU)
