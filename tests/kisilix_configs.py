"""Small Kisilix configurations for the tests.  They differ from one another in every size and constant:
width, vocabulary, eps, the constant on the stream's side of the sums, the order of the layers, which
layers have a feed-forward and of which kind, head counts and grouping (one key head for several heads,
several state-space groups), key, value and state sizes (equal, smaller, larger, no multiples of 32),
taps (1 to 5), norm parts, windows and pooled blocks (a window that is no multiple of the block, a block
larger than the window, larger than a cache page, a block of one position), rotated part of the head
(none, part, all), scales, expert counts, choices and groups (none, some kept, all kept)."""


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def ssm(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def att(heads, kv_heads, dim, vdim, scale, rot_dims, base, size, pool):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"dims": rot_dims, "base": base}, "mask": {"size": size, "pool": pool}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, count, keep, ff, shared_ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}},
            "expert": {"ff": ff}, "shared": {"ff": shared_ff}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# attention first; two heads on a key head everywhere; a window that is no multiple of its block
K_A = {
    "architecture": "Kisilix", "vocab": 200, "width": 64, "max_positions": 512, "norm": {"eps": 1e-5}, "postln_alpha": 1.5,
    "layers": [
        layer("attention", att(4, 2, 32, 16, 0.2, 16, 10000.0, 20, 6), dense(96, 1.5)),
        layer("channel_delta", delta(4, 2, 16, 24, 4), moe(8, 2, 4, 2, 32, 48)),
        layer("mamba2", ssm(4, 16, 24, 2, 2, 3), None),
        layer("attention", att(2, 1, 16, 48, 0.3, 16, 1000.0, 33, 5), moe(6, 3, 1, 1, 24, 16)),
    ],
}

# heads of 64 and 128, a block larger than a cache page, a block of one position, one choice of many
K_B = {
    "architecture": "Kisilix", "vocab": 150, "width": 72, "max_positions": 640, "norm": {"eps": 1e-6}, "postln_alpha": 1.0,
    "layers": [
        layer("mamba2", ssm(3, 64, 64, 1, 3, 2), dense(48, 7.0)),
        layer("attention", att(3, 3, 64, 64, 0.125, 64, 200000.0, 70, 72), moe(12, 1, 3, 1, 16, 40)),
        layer("channel_delta", delta(3, 3, 64, 32, 2), None),
        layer("attention", att(4, 1, 128, 128, 0.09, 32, 1e6, 9, 1), moe(4, 4, 2, 2, 40, 8)),
    ],
}

# sizes that are no multiple of 32 (some of 8 only), no rotation of queries and keys in one layer, one tap,
# a window of one position
K_C = {
    "architecture": "Kisilix", "vocab": 97, "width": 40, "max_positions": 400, "norm": {"eps": 1e-4}, "postln_alpha": 0.75,
    "layers": [
        layer("channel_delta", delta(3, 1, 24, 40, 1), dense(56, 0.5)),
        layer("attention", att(5, 5, 24, 40, 0.25, 0, 10000.0, 1, 4), None),
        layer("mamba2", ssm(5, 8, 40, 5, 1, 5), moe(9, 2, 3, 2, 16, 24)),
        layer("attention", att(2, 2, 96, 32, 0.1, 48, 20000.0, 64, 64), dense(40, 3.0)),
        layer("mamba2", ssm(2, 48, 16, 1, 4, 4), moe(5, 5, 1, 1, 8, 32)),
    ],
}

# larger states (key heads of 128 and a state of 256 rows), a window of a page, blocks of a page
K_D = {
    "architecture": "Kisilix", "vocab": 320, "width": 96, "max_positions": 700, "norm": {"eps": 1e-5}, "postln_alpha": 3.0,
    "layers": [
        layer("channel_delta", delta(2, 2, 128, 64, 5), moe(16, 4, 4, 1, 24, 56)),
        layer("mamba2", ssm(4, 32, 256, 2, 1, 4), dense(80, 2.5)),
        layer("attention", att(6, 2, 64, 32, 0.15, 64, 50000.0, 128, 64), moe(10, 3, 5, 3, 16, 16)),
    ],
}

ALL = {"A": K_A, "B": K_B, "C": K_C, "D": K_D}
