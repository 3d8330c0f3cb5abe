"""Small Nipadra configurations for the tests: sizes that differ from one another in every field, with
values that a particular model may happen to make equal (key and value sizes, heads and key/value heads,
rotary and head size) or 1 (groups, norm groups) chosen apart."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def lightning(heads, dim, vdim, decay, ff=None, act=None):
    mlp = None if ff is None else {"ff": ff, "kind": "dense"}
    if mlp is not None and act:
        mlp["act"] = act
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def parallel(left, right, left_scale, right_scale, ff=None, act=None):
    mlp = None if ff is None else {"ff": ff, "kind": "dense"}
    if mlp is not None and act:
        mlp["act"] = act
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def attention(heads, kv_heads, dim, window, rot_dims, base, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window},
            "rot": {"base": base, "dims": rot_dims}, "scale": scale}


def state_space(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


# P: a parallel layer first, partial rotation, as many key/value heads as heads, two groups, two norm groups, four taps
NIP_P = {
    "architecture": "Nipadra", "width": 96, "vocab": 211, "norm": {"eps": 1e-5}, "postln_alpha": 1.5,
    "layers": [
        parallel(attention(4, 4, 32, 20, 16, 10000.0, 0.3), state_space(4, 24, 16, 2, 4, 2), 0.7, 1.25, ff=136),
        lightning(3, 16, 32, [1.0, 0.9, 0.5], ff=72, act="silu"),
        parallel(attention(6, 2, 16, 7, 16, 500.0, 0.5), state_space(2, 40, 48, 1, 2, 1), 1.0, 0.4),
        lightning(2, 48, 24, [0.97, 0.0]),
    ],
}

# Q: head size 64 (the size the tensor-core attention kernels serve), a window longer than most test prompts and
# one shorter than a page, tanh-GELU in one feed-forward, one tap (no convolution state)
NIP_Q = {
    "architecture": "Nipadra", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
    "layers": [
        lightning(4, 32, 16, [0.6, 0.85, 0.99, 0.999]),
        parallel(attention(4, 2, 64, 150, 32, 500000.0, 0.125), state_space(8, 16, 32, 4, 3, 4), 0.6, 0.5, ff=200),
        parallel(attention(2, 1, 64, 9, 64, 100.0, 0.2), state_space(3, 32, 8, 3, 1, 3), 0.5, 0.5, ff=64, act="gelu_tanh"),
    ],
}

# L: linear attention only (a model that keeps no pages at all); A: the parallel pair only, each layer its own window
NIP_L = {
    "architecture": "Nipadra", "width": 64, "vocab": 150, "norm": {"eps": 1e-6}, "postln_alpha": 1.0,
    "layers": [lightning(2, 32, 32, [0.9, 0.99], ff=96), lightning(4, 16, 16, [0.5, 0.8, 0.95, 1.0])],
}
NIP_A = {
    "architecture": "Nipadra", "width": 80, "vocab": 170, "norm": {"eps": 1e-5}, "postln_alpha": 3.0,
    "layers": [
        parallel(attention(5, 5, 16, 33, 8, 1000.0, 0.25), state_space(5, 16, 16, 5, 2, 5), 1.0, 1.0),
        parallel(attention(2, 1, 48, 5, 48, 20.0, 0.15), state_space(1, 80, 64, 1, 5, 1), 0.3, 0.9, ff=100),
    ],
}

SHARP = {"std": 0.12}


def make_model_dir(config, seed, out_dir, dtype="bfloat16", std=0.12):
    from geneinfer_b200.weights import write_random_model
    return write_random_model(config, seed, out_dir, dtype, std=std)
