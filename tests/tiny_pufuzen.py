"""Small Pufuzen configurations for the tests.  They differ from one another in every size,
in the order of the layers, in which layers have a feed-forward, in windows and constants."""
import torch

import plain_pufuzen as plain
from tokenizer_b200 import write_random_model
from tokenizer_b200.config import PufuzenConfig


def gru(width, ff=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def windowed(heads, dim, vdim, q_rank, kv_rank, size, scale, ff=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": scale, "mask": {"size": size}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def rotary(heads, dim, rot_dim, vdim, q_rank, kv_rank, base, scale, ff=None):
    return {"type": "latent_attention_2",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
                      "kv_rank": kv_rank, "scale": scale, "rot": {"base": base, "dims": rot_dim}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, vocab, width, eps, logit_scale):
    return PufuzenConfig.from_dict({"architecture": "Pufuzen", "vocab": vocab, "width": width,
                                    "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers})


# name -> (configuration, seed, page size)
def tiny_p():
    """A recurrence first; cache rows of 48 and 32 lanes; a window of 7; a feed-forward on a
    recurrent layer and none on an attention layer."""
    return config([gru(72, ff=136), windowed(3, 32, 24, 40, 48, 7, 0.2), rotary(5, 16, 8, 40, 56, 24, 10000.0, 0.3, ff=80),
                   gru(40)], vocab=301, width=96, eps=1e-6, logit_scale=0.5), 3, 8


def tiny_q():
    """Attention first; a cache row of 128 lanes with a sink (the widest tiles' kernel), 16 heads
    over a window of 33 (a cache row of 64 lanes)."""
    return config([rotary(2, 64, 16, 16, 32, 112, 500.0, 0.11, ff=192), windowed(16, 8, 8, 24, 64, 33, 0.35, ff=64),
                   gru(64, ff=72)], vocab=1000, width=64, eps=1e-5, logit_scale=3.0), 4, 16


def tiny_r():
    """Sizes the fast kernels do not take: 17 heads, a cache row of 144 lanes, a window of one key,
    odd widths."""
    return config([windowed(17, 8, 4, 16, 24, 1, 0.5), gru(50), rotary(3, 24, 10, 12, 20, 130, 77.0, 0.2, ff=40),
                   windowed(2, 16, 20, 12, 40, 100, 0.25)], vocab=130, width=40, eps=3e-6, logit_scale=1.0), 5, 32


def tiny_s():
    """Sizes that no vector load fits (a width of 50, a vocabulary of 77, latents of 10 and 18 lanes, one
    head), a window longer than any request, a window of two keys, pages of 64."""
    return config([rotary(1, 10, 6, 6, 10, 18, 1000.0, 0.3), gru(33, ff=30), windowed(1, 6, 10, 14, 18, 500, 0.4, ff=26),
                   windowed(3, 10, 6, 10, 12, 2, 0.3)], vocab=77, width=50, eps=1e-5, logit_scale=2.0), 6, 64


def tiny_t():
    """Recurrent layers alone: a model that keeps no keys at all."""
    return config([gru(48, ff=64), gru(96), gru(32, ff=40)], vocab=200, width=32, eps=1e-6, logit_scale=1.5), 7, 16


TINY = {"p": tiny_p, "q": tiny_q, "r": tiny_r, "s": tiny_s, "t": tiny_t}
# sharper attention and larger sinks, so that a key seen or missed moves the logits in bfloat16 too
SHARPEN = {r"mix\.uq$": 6.0, r"mix\.sink$": 2.0, r"^embed$|^head$": 5.0}


def make_folder(tmp_path_factory, name, scale=SHARPEN):
    cfg, seed, page = TINY[name]()
    folder = str(tmp_path_factory.mktemp(f"pufuzen_{name}"))
    write_random_model(folder, cfg, seed, scale=scale)
    return folder, cfg, page


def reference_logits(folder, requests):
    """{request: array [len, vocab]} from the plain implementation (float64, kept as float32)."""
    cfg, weights = plain.load_folder(folder)
    return {name: plain.forward(cfg, weights, ids).to(torch.float32).numpy() for name, ids in requests.items()}
