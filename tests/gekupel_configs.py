"""Small Gekupel configurations for the tests: sizes that differ from one another in every field; values that a
particular model may happen to make equal (key and value sizes, heads and key/value heads, rotated and unrotated sizes,
the two latents' ranks) or 1 (the experts a token uses, the key/value heads) are chosen apart."""
import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(ff, experts, top):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}


def attention(heads, kv_heads, dim, vdim, chunk, scale, mlp=None, weights_of=None):
    out = {"mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": chunk}, "scale": scale, "vdim": vdim},
           "mlp": mlp, "type": "attention"}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, scale, base, scaling=None, mlp=None, weights_of=None):
    """``scaling`` (factor, original, fast, slow) makes the layer one of the second kind (scaled rotation and a sink)."""
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    out = {"mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "mask": {"size": window}, "q_rank": q_rank, "rot": rot,
                     "rot_dim": rot_dim, "scale": scale, "vdim": vdim},
           "mlp": mlp, "type": "latent_attention_2" if scaling is not None else "latent_attention"}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


# A: every kind of layer, a shared layer, a layer without feed-forward; windows and chunks shorter than the prompts
GEK_A = {
    "architecture": "Gekupel", "embedding": {"scale": 6.0}, "norm": {"eps": 1e-5}, "vocab": 190, "width": 96,
    "layers": [
        latent(3, 24, 8, 40, 56, 48, 21, 0.2, 10000.0, scaling=(4.0, 64, 16.0, 2.0), mlp=dense(136)),
        attention(6, 2, 24, 40, 19, 0.3, mlp=moe(40, 5, 2)),
        latent(2, 16, 24, 8, 40, 72, 9, 0.15, 300.0, mlp=moe(72, 3, 1)),
        attention(6, 2, 24, 40, 19, 0.3, mlp=moe(40, 5, 2), weights_of=1),
        latent(5, 8, 16, 16, 24, 40, 50, 0.25, 50000.0, scaling=(1.5, 32, 8.0, 1.0)),
    ],
}

# B: as many key/value heads as heads, one key/value head for eight heads (four heads to a warp of the attention
# kernel), a value size below a warp, three experts to a token out of four, a window longer than every prompt of the tests
GEK_B = {
    "architecture": "Gekupel", "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "vocab": 260, "width": 128,
    "layers": [
        attention(4, 4, 16, 24, 64, 0.25, mlp=moe(56, 4, 3)),
        latent(9, 32, 4, 24, 64, 136, 400, 0.17, 1000.0, mlp=dense(200)),
        attention(8, 1, 40, 12, 7, 0.2, mlp=dense(72)),
        latent(2, 12, 32, 48, 16, 24, 33, 0.3, 200.0, scaling=(8.0, 16, 4.0, 0.5), mlp=moe(24, 9, 4), weights_of=None),
        attention(5, 5, 10, 7, 30, 0.4),
    ],
}


# C: sizes that fit no tile: a width and ranks that are no multiples of 8, three heads, rotated parts of 12 and 6, value
# sizes of 28 and 10, seven experts of 44 of which a token uses three, a window of 5 and blocks of 3 (shorter than a page),
# a window of one token, and a layer that runs the weights of a later layer
GEK_C = {
    "architecture": "Gekupel", "embedding": {"scale": 2.5}, "norm": {"eps": 1e-4}, "vocab": 131, "width": 100,
    "layers": [
        attention(3, 3, 20, 28, 3, 0.35, mlp=moe(44, 7, 3), weights_of=2),
        latent(3, 20, 12, 28, 36, 52, 5, 0.22, 77.0, scaling=(3.0, 8, 2.0, 0.25), mlp=moe(44, 7, 3)),
        attention(3, 3, 20, 28, 3, 0.35, mlp=moe(44, 7, 3)),
        latent(6, 10, 6, 10, 30, 34, 1, 0.5, 1000.0, mlp=dense(60)),
        latent(3, 20, 12, 28, 36, 52, 5, 0.22, 77.0, scaling=(3.0, 8, 2.0, 0.25), mlp=moe(44, 7, 3), weights_of=1),
    ],
}


def make_model_dir(config, seed, out_dir, dtype="bfloat16", std=0.12):
    from geneinfer_b200.weights import write_random_model
    return write_random_model(config, seed, out_dir, dtype, std=std)
