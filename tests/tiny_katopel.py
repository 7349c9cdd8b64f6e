"""Small Katopel configurations for the tests.  They differ from one another in every size, in the
order and kinds of the layers, in which layers have a feed-forward and of which kind, in chunk
sizes, loops and constants."""
import torch

import plain_katopel as plain
from tokenizer_b200 import write_random_model
from tokenizer_b200.config import KatopelConfig


def delta(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp}


def parallel(left, right, left_scale, right_scale, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right["mixer"], "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, scale, size=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def config(layers, vocab, width, eps, scale, loop=None):
    raw = {"architecture": "Katopel", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": scale}, "layers": layers}
    if loop is not None:
        raw["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return KatopelConfig.from_dict(raw)


# name -> (configuration, seed, page size)
def tiny_a():
    """Two mixers side by side first (one shared key/value head, chunks of 24 on pages of 8, half of a head
    rotated), routed experts with a shared one, a layer without a feed-forward; layers 1 and 2 run
    three times."""
    return config([parallel(attention(4, 1, 32, 16, 0.2, size=24, rot=(10000.0, 16)), delta(2, 1, 16, 24, 3), 0.7, 1.3, dense(136)),
                   delta(3, 3, 24, 40, 2, moe(6, 2, 40, shared=56)),
                   delta(4, 2, 8, 8, 4)], vocab=301, width=96, eps=1e-5, scale=2.0, loop=(1, 3, 3)), 3, 8


def tiny_b():
    """Sizes the tensor-core kernels take (cache rows of 64 and 128 lanes), chunks of 100 that do not
    fit the pages, matrices of 96 rows, a whole head rotated, a layer of plain causal attention without chunks, one expert
    a token and no shared one; no loop."""
    return config([parallel(attention(4, 2, 64, 64, 0.125, size=100, rot=(500.0, 64)), delta(2, 2, 96, 128, 4), 1.0, 0.5, moe(4, 1, 64)),
                   parallel(attention(2, 2, 128, 96, 0.09, rot=(1000000.0, 32)), delta(8, 2, 32, 32, 4), 0.4, 2.0, dense(256))],
                  vocab=1000, width=128, eps=1e-6, scale=1.0), 4, 16


def tiny_c():
    """Sizes that no vector load fits (a width of 50, a vocabulary of 77, heads of 10 and 6 lanes), a
    convolution of one tap (no kept inputs) and one of five, chunks of one position (a token sees
    itself alone), no rotation, every expert chosen, a loop of a single pass, pages of 32."""
    return config([delta(1, 1, 10, 6, 5, dense(30)),
                   parallel(attention(3, 3, 10, 20, 0.3, size=1), delta(2, 1, 6, 10, 1), 1.5, 0.25, moe(3, 3, 14, shared=10))],
                  vocab=77, width=50, eps=3e-6, scale=0.5, loop=(0, 2, 1)), 5, 32


def tiny_d():
    """Two layers of mixers side by side inside a loop that starts behind the first layer and ends before
    the last: chunks of 7 (shorter than a page) and of 50 in two cache groups of unlike rows, a head
    wider in its keys than in its values and rotated whole, one without a feed-forward, a delta rule
    of one head."""
    return config([delta(2, 1, 12, 20, 3, moe(5, 2, 16, shared=24)),
                   parallel(attention(2, 2, 48, 16, 0.2, size=7, rot=(100.0, 48)), delta(4, 4, 16, 16, 2), 0.9, 0.8, dense(72)),
                   parallel(attention(6, 3, 16, 32, 0.3, size=50, rot=(10000.0, 8)), delta(1, 1, 20, 12, 4), 1.2, 0.3),
                   delta(2, 2, 32, 64, 4, dense(40))], vocab=120, width=64, eps=2e-6, scale=1.5, loop=(1, 3, 2)), 6, 16


TINY = {"a": tiny_a, "b": tiny_b, "c": tiny_c, "d": tiny_d}
# sharper attention, so that a key seen or missed moves the logits in bfloat16 too, and an embedding that
# makes logits of a size against which a tolerance means something
SHARPEN = {r"left\.q$": 6.0, r"^embed$": 5.0, r"\.router$": 5.0}


def settle_routing(folder, cfg):
    """Make every token's CHOICE of experts safe from rounding, so that bfloat16 runs can be compared
    (where two router logits nearly tie, rounding anywhere upstream decides, and the outputs differ by an
    expert): lane 0 of the feed-forward's input is pinned near 6 (gain 1/4, bias 6 of the norm in front),
    and the router rows of the `top` favoured experts weigh it by 2, which lifts their logits about 12
    above the others'.  Inside the chosen set the logits, and with them the shares, still vary from token
    to token.  Which experts a token chooses varies in the runs without this (float32)."""
    import os
    from tokenizer_b200.weights.safetensors_io import read_safetensors, write_safetensors
    path = os.path.join(folder, "model.safetensors")
    tensors = dict(read_safetensors(path))
    for index, layer in enumerate(cfg.layers):
        mlp = layer.get("mlp")
        if not mlp or mlp["kind"] != "moe":
            continue
        experts, top = mlp["router"]["experts"], mlp["router"]["top"]
        favoured = [(3 * index + 2 * k + 1) % experts for k in range(experts)]
        favoured = list(dict.fromkeys(favoured + list(range(experts))))[:top]
        gain, bias, router = (tensors[f"l{index}.norm2"].clone(), tensors[f"l{index}.norm2.b"].clone(),
                              tensors[f"l{index}.mlp.router"].clone())
        gain[0], bias[0] = 0.25, 6.0
        router[:, 0] = 0.0
        router[favoured, 0] = 2.0
        tensors[f"l{index}.norm2"], tensors[f"l{index}.norm2.b"], tensors[f"l{index}.mlp.router"] = gain, bias, router
    write_safetensors(path, tensors)


def make_folder(tmp_path_factory, name, scale=SHARPEN, settled=True):
    cfg, seed, page = TINY[name]()
    folder = str(tmp_path_factory.mktemp(f"katopel_{name}"))
    write_random_model(folder, cfg, seed, scale=scale)
    if settled:
        settle_routing(folder, cfg)
    return folder, cfg, page


def reference_logits(folder, requests):
    """{request: array [len, vocab]} from the plain implementation (float64, kept as float32)."""
    cfg, weights = plain.load_folder(folder)
    return {name: plain.forward(cfg, weights, ids).to(torch.float32).numpy() for name, ids in requests.items()}
