"""Attention whose keys and values are expanded from a small latent per token, so that the
latent is all the cache keeps.

Per token, from the mixer's input h:
  query latent   cq = rms_norm(Wdq h) * g_q;   queries q = Wuq cq, head by head
                 [dim lanes without position | rot_dim lanes that carry the position]
  kv latent      c = rms_norm((Wdkv h)[:kv_rank]) * g_c;   the last rot_dim rows of Wdkv h are one
                 positional key part shared by all heads (not normed)
  per head       key = [Wuk_h c | rotated shared part], value = Wuv_h c,
                 score = q . key * scale, softmax (with a window and / or a sink), output Wo on the
                 concatenated heads.
The cache row of a token is [c | rotated shared part | zeros up to a multiple of 16 lanes].

How it is computed.  Nothing lies between Wuq and the score but the rotation of the positional
lanes, and nothing between the weighted sum of values and Wo, so the expansions are folded into
the projections once, at load time, in float64:
  score_h = (Wuk_h^T Wuq_h[:dim]) cq . c + rot(q_h[dim:]) . rot(shared)
  output  = sum_h (Wo[:, h] Wuv_h) (sum_j p_hj c_j)
The attention is then attention of `heads` query heads over ONE cached head of kv_rank + rot_dim
lanes whose values are the leading kv_rank lanes of the same rows: the framework's paged kernels
take it with the cache pool passed as keys and as values (the value lanes behind kv_rank meet
zero columns of the folded output projection).  Per token this costs heads * kv_rank * (q_rank +
hidden) multiply-adds for the two folded products, against heads * (dim * (q_rank + kv_rank) +
vdim * (kv_rank + hidden)) unfolded: less or about as much while the latent is not much wider than
a head.
"""
from __future__ import annotations

import torch

from ..config.spec import ConfigError
from ..kernels import ops
from ..weights.store import TensorSpec
from .attention import PagedAttention
from .base import CacheNeed, KVNeed, build_part, register_part
from .linear import Linear
from .recurrent import SideProjection

ROW_MULTIPLE = 16       # cache rows are padded to whole 16 lanes (the tensor-core kernels' step)


class LatentAttention(PagedAttention, SideProjection):
    @staticmethod
    def tensors(spec):
        p, x = spec.params, spec.prefix
        hidden, heads = p["hidden_size"], p["heads"]
        rot = p.get("rot_dim", 0)
        out = [TensorSpec(x + ".dq", (p["q_rank"], hidden)),
               TensorSpec(x + ".dq.norm", (p["q_rank"],), "one_plus_normal"),
               TensorSpec(x + ".uq", (heads * (p["dim"] + rot), p["q_rank"])),
               TensorSpec(x + ".dkv", (p["kv_rank"] + rot, hidden)),
               TensorSpec(x + ".dkv.norm", (p["kv_rank"],), "one_plus_normal"),
               TensorSpec(x + ".uk", (heads * p["dim"], p["kv_rank"])),
               TensorSpec(x + ".uv", (heads * p["vdim"], p["kv_rank"]))]
        if p.get("sink"):
            out.append(TensorSpec(x + ".sink", (heads,), "normal", 1.0))
        out.append(TensorSpec(x + ".o", (hidden, heads * p["vdim"])))
        return out

    def __init__(self, spec, store, runtime):
        p, x = spec.params, spec.prefix
        self.runtime = runtime
        self.hidden, self.heads = int(p["hidden_size"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.rot_dim = int(p.get("rot_dim", 0))
        self.eps = float(p["eps"])
        self.scale = float(p["scale"])
        self.window = p.get("window")          # None: every earlier key; n: the n keys before the query too
        if self.window is not None and int(self.window) < 0:
            raise ConfigError("a window reaches back a number of keys that is not negative")
        self.position = None
        self.rot_dims = 0
        if self.rot_dim:
            if p.get("position") is None:
                raise ConfigError("latent attention with positional lanes needs a position encoding")
            self.position = build_part("position", p["position"], store, runtime)
            self.rot_dims = self.position.dims
            if self.rot_dims > self.rot_dim:
                raise ConfigError(f"{self.rot_dims} rotated lanes do not fit {self.rot_dim} positional lanes")
        # what the paged kernels see: `heads` query heads over one cached head of `row` lanes
        self.nh, self.nkv = self.heads, 1
        self.row = -(-(self.kv_rank + self.rot_dim) // ROW_MULTIPLE) * ROW_MULTIPLE
        self.d = self.row
        self.sink = runtime.vector(store.get(x + ".sink")) if p.get("sink") else None
        self.q_gain = runtime.vector(store.get(x + ".dq.norm"))
        self.c_gain = runtime.vector(store.get(x + ".dkv.norm"))
        self._own = [store.get(x + ".dq"), store.get(x + ".dkv")]
        self.inputs = self._stack(runtime, list(self._own), [None, None], None)
        q_folded, o_folded = self._fold(store.get(x + ".uq"), store.get(x + ".uk"), store.get(x + ".uv"),
                                        store.get(x + ".o"))
        self.q_proj = Linear(runtime.matrix(q_folded))
        self.out = Linear(runtime.matrix(o_folded))

    def _fold(self, uq, uk, uv, o):
        """(queries straight into the latent's lanes [heads * row, q_rank], output projection
        straight from the weighted latents [hidden, heads * row]), float64 products rounded once."""
        H, dim, vdim, rank, rot, row = self.heads, self.dim, self.vdim, self.kv_rank, self.rot_dim, self.row
        f64 = torch.float64
        uq = uq.to(f64).view(H, dim + rot, self.q_rank)
        uk = uk.to(f64).view(H, dim, rank)
        uv = uv.to(f64).view(H, vdim, rank)
        o = o.to(f64).view(self.hidden, H, vdim)
        q_folded = torch.zeros((H, row, self.q_rank), dtype=f64, device=uq.device)
        q_folded[:, :rank] = torch.matmul(uk.transpose(1, 2), uq[:, :dim])
        q_folded[:, rank:rank + rot] = uq[:, dim:]
        o_folded = torch.zeros((self.hidden, H, row), dtype=f64, device=uq.device)
        o_folded[:, :, :rank] = torch.einsum("ohv,hvr->ohr", o, uv)
        return (q_folded.view(H * row, self.q_rank).to(torch.float32),
                o_folded.view(self.hidden, H * row).to(torch.float32))

    def take_side(self, weight, bias):
        self.inputs = self._stack(self.runtime, list(self._own), [None, None], (weight, bias))

    def cache_need(self):
        return CacheNeed(kv=KVNeed(1, self.row, self.window, planes=1))

    def streamed_weights(self):
        return [self.inputs.weight, self.q_proj.weight, self.out.weight]

    def forward(self, h, ctx, cache):
        group = ctx.groups[cache.group]
        product = self.inputs.forward(h, out_dtype=torch.float32)
        cq = self.runtime.empty(ctx.n_tokens, self.q_rank)
        freq = self.position.inv_freq if self.position is not None else None
        ops.latent_prepare(product, 0, self.q_rank, self.q_rank, self.kv_rank, self.rot_dim, self.rot_dims,
                           self.q_gain, self.c_gain, self.eps, freq, ctx.pos, ctx.row_req,
                           group.slots if cache.writes else None, cq, cache.k_pool)
        q = self.q_proj.forward(cq)
        if self.rot_dims:
            ops.rotate_interleaved(q, self.heads, self.kv_rank, self.rot_dims, freq, ctx.pos, ctx.row_req)
        mixed = self.runtime.empty(ctx.n_tokens, self.heads * self.row)
        self.attend(q, mixed, ctx, group, cache)
        self._keep_side(product)
        return self.out.forward(mixed, partials_ok=True)


register_part("mixer", "latent_attention", LatentAttention)
