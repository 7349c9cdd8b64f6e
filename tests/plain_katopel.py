"""A plain, slow restatement of the Katopel decoder on the CPU, one function per mechanism,
token by token where a mechanism is a recurrence.  It reads config.json and the weight file
itself and shares nothing with the engine: it is what the engine is compared with.

Everything is computed in float64 unless `dtype` says otherwise, so that it stands between the
engine's two precisions as the exact answer.
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
def linear(x, w, b=None):
    y = x @ w.t()
    return y if b is None else y + b


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def layer_norm(x, gain, bias, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * gain + bias over the last axis."""
    mean = x.mean(dim=-1, keepdim=True)
    dev = x - mean
    return dev / torch.sqrt((dev * dev).mean(dim=-1, keepdim=True) + eps) * gain + bias


def short_convolution(x, taps, history=None):
    """Causal convolution over time, channel by channel.  x [T, C], taps [C, n] with the last
    column weighing the current token; `history` [n - 1, C] are the inputs before x (zeros at the
    start of a sequence).  Returns the outputs [T, C] and the last n - 1 inputs."""
    n = taps.shape[1]
    past = torch.zeros(n - 1, x.shape[1], dtype=x.dtype) if history is None else history
    full = torch.cat([past, x], dim=0)
    out = torch.zeros_like(x)
    for j in range(n):
        out = out + full[j:j + x.shape[0]] * taps[:, j]
    return out, full[full.shape[0] - (n - 1):]


def unit_vectors(x):
    """Every vector of the last axis divided by sqrt(sum of squares + 1e-6)."""
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta_rule(q, k, v, beta, decay, state=None):
    """One head.  q, k [T, dim], v [T, vdim], beta, decay [T].  Per token: S <- decay S;
    u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Returns o [T, vdim] and the last S."""
    S = torch.zeros(q.shape[1], v.shape[1], dtype=q.dtype) if state is None else state.clone()
    rows = []
    for t in range(q.shape[0]):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        rows.append(S.t() @ q[t])
    return torch.stack(rows), S


def delta_mixer(h, w, prefix, m, eps):
    """The gated-delta-rule mixer over a whole sequence from its start.  h [T, width]."""
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q, _ = short_convolution(linear(h, w[prefix + "q"]), w[prefix + "q.conv"])
    k, _ = short_convolution(linear(h, w[prefix + "k"]), w[prefix + "k.conv"])
    v, _ = short_convolution(linear(h, w[prefix + "v"]), w[prefix + "v.conv"])
    q = unit_vectors(silu(q).view(T, groups, dim)) * dim ** -0.5
    k = unit_vectors(silu(k).view(T, groups, dim))
    v = silu(v).view(T, heads, vdim)
    beta = sigmoid(linear(h, w[prefix + "b"]))
    decay = torch.exp(-torch.exp(w[prefix + "A_log"]) * softplus(linear(h, w[prefix + "a"]) + w[prefix + "dt_bias"]))
    gate = silu(linear(h, w[prefix + "g"])).view(T, heads, vdim)
    outs = []
    for head in range(heads):
        g = head // (heads // groups)
        o, _ = gated_delta_rule(q[:, g], k[:, g], v[:, head], beta[:, head], decay[:, head])
        o = o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps) * w[prefix + "norm"]
        outs.append(o * gate[:, head])
    return linear(torch.cat(outs, dim=1), w[prefix + "o"])


def rotate_interleaved(x, positions, base, dims):
    """Rotary encoding on the first `dims` lanes of the last axis, lane 2i paired with lane
    2i + 1, angle = position * base^(-2i / dims); the other lanes pass.  x [T, heads, n]."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(x.dtype) * base ** (-2.0 * i / dims)
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def chunked_attention(h, w, prefix, m):
    """Softmax attention in which position i sees j <= i of its own chunk only (chunks of
    mask.size positions counted from 0).  Grouped heads, biases, rotary lanes on q and k."""
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    positions = torch.arange(T)
    q = linear(h, w[prefix + "q"], w[prefix + "q.b"]).view(T, heads, dim)
    k = linear(h, w[prefix + "k"], w[prefix + "k.b"]).view(T, groups, dim)
    v = linear(h, w[prefix + "v"], w[prefix + "v.b"]).view(T, groups, vdim)
    if m.get("rot") is not None:
        q = rotate_interleaved(q, positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))
        k = rotate_interleaved(k, positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    seen = positions[None, :] <= positions[:, None]
    if m.get("mask") is not None:
        size = int(m["mask"]["size"])
        seen = seen & ((positions[None, :] // size) == (positions[:, None] // size))
    outs = []
    for head in range(heads):
        g = head // (heads // groups)
        score = (q[:, head] @ k[:, g].t()) * float(m["scale"])
        score = score.masked_fill(~seen, -math.inf)
        outs.append(torch.softmax(score, dim=-1) @ v[:, g])
    return linear(torch.cat(outs, dim=1), w[prefix + "o"])


def parallel_mixer(h, w, prefix, m, eps):
    left = chunked_attention(h, w, prefix + "left.", m["left"])
    right = delta_mixer(h, w, prefix + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def gated_feed_forward(h, w, prefix):
    return linear(silu(linear(h, w[prefix + "gate"])) * linear(h, w[prefix + "up"]), w[prefix + "down"])


def routed_feed_forward(h, w, prefix, mlp):
    """Every token goes to the `top` experts with the largest router logits, weighed by the
    softmax over those logits alone; a shared expert, where there is one, serves every token and
    is scaled by the sigmoid of one more projection."""
    top = int(mlp["router"]["top"])
    logits = linear(h, w[prefix + "router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(logits[t], top).indices
        share = torch.softmax(logits[t][chosen], dim=-1)
        for e, s in zip(chosen.tolist(), share):
            out[t] = out[t] + s * gated_feed_forward(h[t:t + 1], w, f"{prefix}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + sigmoid(linear(h, w[prefix + "shared.sg"])) * gated_feed_forward(h, w, prefix + "shared.")
    return out


# ---- the model ----------------------------------------------------------------------------
def run_order(cfg):
    """[(layer, pass number or None)]: the layers before the loop, the looped layers `times`
    times, the rest; the pass number stands at a pass's first layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop["stop"]) <= int(loop["start"]):
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def forward(cfg, w, ids, keep=None):
    """Logits [T, vocab] of a whole sequence from its start.  `keep` (a list) receives the
    residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    dtype = w["embed"].dtype
    x0 = w["embed"][torch.tensor(list(ids), dtype=torch.long)] * float(cfg["embedding"]["scale"])
    x = x0.clone()
    for index, turn in run_order(cfg):
        layer, p = cfg["layers"][index], f"l{index}."
        if turn is not None:
            if turn > 0:
                x = x + x0
            x = x + w["loop.step"][turn]
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "delta":
            y = delta_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + layer_norm(y, w[p + "norm1b"], w[p + "norm1b.b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            y = gated_feed_forward(h, w, p + "mlp.") if mlp["kind"] == "dense" else \
                routed_feed_forward(h, w, p + "mlp.", mlp)
            x = x + layer_norm(y, w[p + "norm2b"], w[p + "norm2b.b"], eps)
        if keep is not None:
            keep.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return linear(x, w["embed"]).to(dtype)


def greedy_generate(cfg, w, prompt, n_new):
    ids, out = list(prompt), []
    for _ in range(n_new):
        out.append(int(torch.argmax(forward(cfg, w, ids)[-1])))
        ids.append(out[-1])
    return out
