"""A plain, slow restatement of the Pufuzen decoder on the CPU, one function per mechanism,
token by token where a mechanism is a recurrence.  It reads config.json and the weight file
itself and shares nothing with the engine: it is what the engine is compared with.

Everything is computed in float64 unless `dtype` says otherwise, so that it stands between
the engine's two precisions as the exact answer.
"""
import json
import math
import os

import torch


def load_folder(folder, dtype=torch.float64):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    weights = {k: (v.to(dtype) if v.is_floating_point() else v)
               for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, weights


# ---- mechanisms ---------------------------------------------------------------------------
def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis (gain may be None)."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if gain is None else y * gain


def linear(x, w, b=None):
    y = x @ w.t()
    return y if b is None else y + b


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def min_gru(h, w, prefix, state=None):
    """Gated recurrence whose gates see only the current token.  h [T, hidden]; returns the
    mixer's output [T, hidden] and the state after the last token [width]."""
    z = sigmoid(linear(h, w[prefix + "z"], w[prefix + "z.b"]))
    u = linear(h, w[prefix + "x"], w[prefix + "x.b"])
    candidate = torch.where(u >= 0, u + 0.5, sigmoid(u))
    g = linear(h, w[prefix + "g"])
    s = torch.zeros(z.shape[1], dtype=h.dtype) if state is None else state.clone()
    rows = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * candidate[t]
        rows.append(s * (g[t] * sigmoid(g[t])))
    return linear(torch.stack(rows), w[prefix + "o"]), s


def rotate_interleaved(x, positions, base, dims):
    """Rotary encoding on the first `dims` lanes of the last axis, lane 2i paired with lane
    2i + 1, angle = position * base^(-2i / dims); the other lanes pass.  x [T, ..., n]."""
    out = x.clone()
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]            # [T, half]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def latent_attention(h, w, prefix, m, eps, first_position=0, rot=None, window=None, sink=False):
    """Attention whose keys and values are expanded from a small latent per token.  h holds a
    whole sequence from `first_position` on ([T, hidden]).  m: the mixer's sizes.  rot =
    (base, dims) rotates the last `rot_dim` lanes of every query head and the one shared key
    part; window = n lets a position see itself and the n - 1 before it; sink adds exp(sink_h)
    to the softmax's denominator."""
    T = h.shape[0]
    H, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    rdim = m.get("rot_dim", 0) if rot is not None else 0
    positions = torch.arange(first_position, first_position + T)
    cq = rms_norm(linear(h, w[prefix + "dq"]), w[prefix + "dq.norm"], eps)
    q = linear(cq, w[prefix + "uq"]).view(T, H, dim + rdim)
    down = linear(h, w[prefix + "dkv"])
    c = rms_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    k = linear(c, w[prefix + "uk"]).view(T, H, dim)
    v = linear(c, w[prefix + "uv"]).view(T, H, vdim)
    if rdim:
        base, dims = rot
        q = torch.cat([q[..., :dim], rotate_interleaved(q[..., dim:], positions, base, dims)], dim=-1)
        shared = rotate_interleaved(down[:, rank:rank + rdim], positions, base, dims)
        k = torch.cat([k, shared[:, None, :].expand(T, H, rdim)], dim=-1)
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for head in range(H):
            scores = (k[lo:i + 1, head] @ q[i, head]) * m["scale"]
            top = scores.max()
            if sink:
                top = torch.maximum(top, w[prefix + "sink"][head])
            e = torch.exp(scores - top)
            total = e.sum()
            if sink:
                total = total + torch.exp(w[prefix + "sink"][head] - top)
            out[i, head] = (e / total) @ v[lo:i + 1, head]
    return linear(out.reshape(T, H * vdim), w[prefix + "o"])


def poly_norm_mlp(h, w, prefix, eps):
    """down(a N(z) + b N(z^2) + c N(z^3) + e), z = up(h); N divides a token's vector by its
    root mean square."""
    z = linear(h, w[prefix + "up"], w[prefix + "up.b"])
    a, b, c, e = [w[prefix + "act"][i] for i in range(4)]
    act = a * rms_norm(z, None, eps) + b * rms_norm(z * z, None, eps) + c * rms_norm(z * z * z, None, eps) + e
    return linear(act, w[prefix + "down"], w[prefix + "down.b"])


def residual_gate(h, w, name):
    return sigmoid(linear(h, w[name], w[name + ".b"]))


# ---- the model ----------------------------------------------------------------------------
def mixer(layer, h, w, prefix, eps):
    kind, m = layer["type"], layer["mixer"]
    if kind == "mingru":
        return min_gru(h, w, prefix)[0]
    if kind == "latent_attention":
        return latent_attention(h, w, prefix, m, eps, window=m["mask"]["size"])
    if kind == "latent_attention_2":
        return latent_attention(h, w, prefix, m, eps, rot=(m["rot"]["base"], m["rot"]["dims"]), sink=True)
    raise ValueError(f"unknown layer type {kind}")


def forward(cfg, w, ids, keep_layers=False):
    """Logits [T, vocab] of one whole sequence; with `keep_layers` also the residual stream
    after every layer [layers, T, width]."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(ids, dtype=torch.long)]
    kept = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        x = x + mixer(layer, h, w, p + "mix.", eps) * residual_gate(h, w, p + "rg1")
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError("only dense feed-forwards exist in this design")
            h = rms_norm(x, w[p + "norm2"], eps)
            x = x + poly_norm_mlp(h, w, p + "mlp.", eps) * residual_gate(h, w, p + "rg2")
        kept.append(x)
    logits = linear(rms_norm(x, w["final.norm"], eps), w["head"]) * cfg["logit_scale"]
    return (logits, torch.stack(kept)) if keep_layers else logits


def greedy_generate(cfg, w, prompt, n):
    ids, out = list(prompt), []
    for _ in range(n):
        nxt = int(torch.argmax(forward(cfg, w, ids)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out
