"""Two mixers side by side: both read the same input, and the layer's mixer output is
left_scale * left(h) + right_scale * right(h).  Either side is any registered mixer; together they
may need keys and values (one of them) and per-request state (one of them), which the cache manager
serves through the one binding of the call.  Where both sides offer their input products as a stack
(`input_stack` / `forward_projected`), the two stacks are ONE product of the common input.  The two
outputs are not added here: they are handed on as scaled terms, and whoever adds the mixer's output
to the stream (or norms it first) sums them in float32 on the way."""
from __future__ import annotations

import torch

from ..config.spec import ConfigError
from .base import CacheNeed, ScaledTerms, build_part, part_class, register_part
from .linear import Linear
from .recurrent import stacked_rows


class ParallelMixers:
    @staticmethod
    def tensors(spec):
        out = []
        for side in ("left", "right"):
            sub = spec.params[side]
            out += part_class("mixer", sub.kind).tensors(sub)
        return out

    def __init__(self, spec, store, runtime):
        p = spec.params
        self.runtime = runtime
        self.left = build_part("mixer", p["left"], store, runtime)
        self.right = build_part("mixer", p["right"], store, runtime)
        self.left_scale, self.right_scale = float(p["left_scale"]), float(p["right_scale"])
        self.graph_safe = all(getattr(m, "graph_safe", False) for m in (self.left, self.right))
        self.inputs, self.right_at = None, 0
        if all(hasattr(m, "input_stack") and hasattr(m, "forward_projected") for m in (self.left, self.right)):
            (w_left, b_left), (w_right, b_right) = self.left.input_stack(), self.right.input_stack()
            if b_left is None and b_right is None:
                self.right_at = -(-w_left.shape[0] // 8) * 8      # the right side's columns start on 32 bytes
                self.inputs = Linear(runtime.matrix(stacked_rows([stacked_rows([w_left]), w_right])))

    def cache_need(self):
        needs = [self.left.cache_need(), self.right.cache_need()]
        kv = [n.kv for n in needs if n.kv is not None]
        state = [n.state for n in needs if n.state is not None]
        if len(kv) > 1 or len(state) > 1:
            raise ConfigError("of two mixers side by side, one may keep keys and values and one a state")
        return CacheNeed(kv=kv[0] if kv else None, state=state[0] if state else None)

    def batch_annotations(self):
        found = []
        for m in (self.left, self.right):
            found += list(getattr(m, "batch_annotations", lambda: [])())
        return found

    def shape_key(self, q_lens):
        return tuple(m.shape_key(q_lens) for m in (self.left, self.right) if hasattr(m, "shape_key"))

    def streamed_weights(self):
        out = [] if self.inputs is None else [self.inputs.weight]
        for m in (self.left, self.right):
            out += [w for w in getattr(m, "streamed_weights", lambda: [])() if w is not None]
        return out

    def forward(self, h, ctx, cache):
        if self.inputs is not None:
            proj = self.inputs.forward(h, out_dtype=torch.float32)
            left = self.left.forward_projected(proj, 0, ctx, cache)
            right = self.right.forward_projected(proj, self.right_at, ctx, cache)
        else:
            left, right = self.left.forward(h, ctx, cache), self.right.forward(h, ctx, cache)
        for y in (left, right):
            if isinstance(y, ScaledTerms):
                raise ConfigError("mixers side by side do not nest")
        return ScaledTerms([(left, self.left_scale), (right, self.right_scale)])


register_part("mixer", "parallel_mixers", ParallelMixers)
