"""Small Tevilix configurations for the tests.  They differ from one another in every size and constant: width,
vocabulary, eps, embedding scale, the order of the layers and the looped range (none, one layer, several, all),
which layers have a feed-forward and of which kind, head counts and grouping (one key head for all heads, a key
head per head), key and value sizes (equal, smaller, larger, no multiples of 8), the rotated part of a head
(none, part, all), the positions' scaling (also 1), windows (one position, a few, more than a cache page, none),
the side-by-side weights (also 1), recurrent widths, the gates' cap, expert counts, choices and groups (none,
some kept, all kept, groups of one expert)."""


def att(heads, kv_heads, dim, vdim, scale, rot_dims, base, factor, size):
    a = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims is not None:
        a["rot"] = {"dims": rot_dims, "base": base}
        if factor is not None:
            a["rot"]["scaling"] = {"factor": factor}
    if size:
        a["mask"] = {"size": size}
    return a


def par(left, left_scale, width, right_scale):
    return {"left": left, "left_scale": left_scale, "right": {"width": width}, "right_scale": right_scale}


def mls(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, count, keep, scale, ff):
    r = {"experts": experts, "top": top, "scale": scale}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "router": r, "expert": {"ff": ff}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# the matrix memory first; two layers looped twice; three heads on a key head; a window shorter than a page
T_A = {
    "architecture": "Tevilix", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [
        layer("mlstm", mls(4, 16, 24, 8.0), dense(96)),
        layer("parallel", par(att(6, 2, 32, 16, 0.2, 16, 10000.0, 4.0, 20), 0.7, 48, 1.3), moe(8, 2, 4, 2, 1.5, 32)),
        layer("mlstm", mls(2, 64, 32, 15.0), None),
        layer("parallel", par(att(2, 1, 16, 48, 0.3, 16, 1000.0, None, 33), 1.0, 80, 1.0), moe(6, 3, None, None, 1.0, 24)),
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}

# heads of 64 and 128, a window longer than a page, every layer looped, one choice of many, groups of one expert
T_B = {
    "architecture": "Tevilix", "vocab": 150, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 6.0},
    "layers": [
        layer("parallel", par(att(3, 3, 64, 64, 0.125, 64, 200000.0, 1.0, 70), 1.2, 40, 0.5), moe(12, 1, 3, 1, 2.0, 16)),
        layer("mlstm", mls(3, 32, 64, 10.0), moe(4, 2, 4, 3, 0.5, 40)),
        layer("parallel", par(att(4, 1, 128, 128, 0.09, 32, 1e6, 8.0, 9), 0.9, 72, 0.9), dense(48)),
    ],
    "loop": {"start": 0, "stop": 3, "times": 2},
}

# sizes that are no multiple of 8, no rotation in one layer, a window of one position, no loop, no window in one layer
T_C = {
    "architecture": "Tevilix", "vocab": 97, "width": 40, "norm": {"eps": 1e-4},
    "layers": [
        layer("parallel", par(att(5, 5, 12, 20, 0.25, None, None, None, 1), 1.0, 25, 2.0), dense(56)),
        layer("mlstm", mls(5, 10, 6, 9.0), None),
        layer("parallel", par(att(2, 2, 24, 10, 0.4, 0, 10000.0, 2.0, 0), 0.6, 33, 1.1), moe(9, 2, 3, 2, 3.0, 14)),
        layer("mlstm", mls(1, 40, 40, 5.0), moe(5, 5, 1, 1, 1.0, 8)),
        layer("parallel", par(att(3, 1, 40, 24, 0.1, 40, 20000.0, 1.5, 64), 1.5, 16, 0.3), dense(24)),
    ],
}

# larger states, one layer run three times, eight heads, a window of two pages
T_D = {
    "architecture": "Tevilix", "vocab": 320, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 9.5},
    "layers": [
        layer("parallel", par(att(8, 4, 64, 32, 0.15, 32, 50000.0, 3.0, 128), 0.85, 200, 1.15), moe(16, 4, 4, 1, 1.75, 24)),
        layer("mlstm", mls(3, 128, 64, 11.0), dense(80)),
        layer("mlstm", mls(6, 32, 16, 20.0), moe(10, 3, 5, 3, 1.0, 16)),
    ],
    "loop": {"start": 1, "stop": 2, "times": 3},
}

# no size that is a multiple of 8 (not the width, no head size, no feed-forward width, not the vocabulary)
T_E = {
    "architecture": "Tevilix", "vocab": 101, "width": 42, "norm": {"eps": 1e-5}, "embedding": {"scale": 5.0},
    "layers": [
        layer("mlstm", mls(3, 14, 9, 7.0), moe(6, 2, 2, 1, 1.25, 10)),
        layer("parallel", par(att(3, 1, 10, 6, 0.35, 6, 5000.0, 1.25, 17), 0.9, 27, 1.2), dense(30)),
    ],
    "loop": {"start": 1, "stop": 2, "times": 2},
}

ALL = {"A": T_A, "B": T_B, "C": T_C, "D": T_D, "E": T_E}


def random_config(rng) -> dict:
    """A configuration drawn at random: layer count and order, which layers have which feed-forward, every size (also
    off the 8-number grid), windows around the page and tile borders or none, the rotated part, the looped range."""
    def pick(xs):
        return xs[int(rng.integers(0, len(xs)))]

    def attention():
        kv = pick([1, 1, 2, 2, 3, 4])
        a = att(kv * pick([1, 2, 3, 4]), kv, pick([8, 16, 24, 32, 48, 64, 96, 128, 20, 36]), pick([8, 16, 32, 40, 64, 128, 12]),
                float(rng.uniform(0.05, 0.4)), None, None, None, 0)
        if rng.random() < 0.85:
            a["rot"] = {"dims": pick([a["dim"], a["dim"] // 2, a["dim"] // 4]) // 2 * 2, "base": pick([100.0, 10000.0, 5e5])}
            if rng.random() < 0.7:
                a["rot"]["scaling"] = {"factor": pick([1.0, 2.0, 4.0, 1.5])}
        if rng.random() < 0.85:
            a["mask"] = {"size": pick([1, 2, 7, 31, 32, 33, 64, 65, 100, 128, 200])}
        return a

    def feed_forward():
        r = rng.random()
        if r < 0.2:
            return None
        if r < 0.5:
            return dense(pick([24, 64, 100, 256]))
        count, per = pick([1, 2, 3, 4]), pick([1, 2, 3, 4, 8])
        keep = int(rng.integers(1, count + 1))
        top = int(rng.integers(1, min(keep * per, 6) + 1))
        return moe(count * per, top, count if rng.random() < 0.8 or keep < count else None, keep, pick([1.0, 2.0, 0.5]),
                   pick([8, 24, 40, 96]))

    layers = []
    for _ in range(int(rng.integers(1, 5))):
        if rng.random() < 0.5:
            layers.append(layer("parallel", par(attention(), pick([1.0, 0.7, 1.3]), pick([16, 40, 100, 300, 33]),
                                                pick([1.0, 1.2, 0.6])), feed_forward()))
        else:
            layers.append(layer("mlstm", mls(pick([1, 2, 3, 6]), pick([8, 16, 32, 64, 128, 20]), pick([8, 16, 64, 33, 128]),
                                             pick([5.0, 10.0, 15.0, 30.0])), feed_forward()))
    cfg = {"architecture": "Tevilix", "vocab": pick([64, 101, 500]), "width": pick([32, 40, 48, 64, 72, 96, 128, 192, 50, 84]),
           "norm": {"eps": pick([1e-5, 1e-6])}, "embedding": {"scale": pick([1.0, 4.0, 9.0])}, "layers": layers}
    if rng.random() < 0.6:
        a = int(rng.integers(0, len(layers)))
        cfg["loop"] = {"start": a, "stop": int(rng.integers(a, len(layers) + 1)), "times": int(rng.integers(1, 4))}
    return cfg
