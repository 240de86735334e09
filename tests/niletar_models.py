"""Small Niletar configurations and random weights for the tests, written from scratch here (checkpoint names and
config.json keys as a user's folder has them).  The configurations differ from one another in everything a configuration
can say: order of the layers, layers that take an earlier layer's weights, widths, heads and groups (one, some, as many
as heads), key and value sizes (equal, values wider, values narrower, no multiples of 8), rotated sizes (none, a
part, all of the head), frequency scaling or none, taps of the convolutions, state sizes (odd ones, more than a
thread's registers hold in the smallest kernel), parts of the norm (one, some), ranks, the residual's multiplier, the
two mixers' weights, layers without a feed-forward."""
import json
import os

import torch


def dense(ff):
    return {"kind": "dense", "ff": ff}


def mamba2(heads, vdim, state, groups, norm_groups, conv, mlp, weights_of=None):
    out = {"type": "mamba2", "mlp": mlp,
           "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def left(heads, kv_heads, dim, vdim, rot_dims, base, scale, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot, "scale": scale, "vdim": vdim}


def right(heads, kv_heads, dim, vdim, conv):
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}


def parallel(l, r, left_scale, right_scale, mlp, weights_of=None):
    out = {"type": "parallel", "mlp": mlp, "mixer": {"left": l, "left_scale": left_scale, "right": r, "right_scale": right_scale}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def config(vocab, width, alpha, layers, eps=1e-5):
    return {"architecture": "Niletar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
            "layers": layers}


_SCALING = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}
_P_SSM = mamba2(3, 8, 5, 1, 3, 3, dense(40))
_P_PAR = parallel(left(4, 1, 24, 8, 6, 50.0, 0.2, _SCALING), right(4, 2, 12, 20, 2), 0.7, 1.3, dense(40))
_S_PAR = parallel(left(8, 2, 128, 64, 64, 1000.0, 0.09), right(2, 1, 96, 40, 4), 1.0, 0.25, dense(72))

CONFIGS = {
    # the scan first; one group and a norm in three parts; values narrower than keys; a fourth of the head rotated, with
    # scaled frequencies whose three ranges all occur; the third and fourth layer run with the weights of the second
    # and the first and states of their own
    "p": config(97, 48, 2.5, [_P_SSM, _P_PAR, dict(_P_PAR, weights_of=1), dict(_P_SSM, weights_of=0)], eps=1e-4),
    # values wider than keys, the whole head rotated, as many key heads as query heads on both sides, five taps, a norm
    # in one part, as many groups as heads, an odd state size, a layer without a feed-forward, a multiplier of 1
    "q": config(130, 64, 1.0, [parallel(left(2, 2, 16, 40, 16, 300.0, 0.3), right(3, 3, 8, 8, 5), 1.0, 1.0, None),
                               mamba2(4, 16, 33, 4, 1, 5, dense(36)),
                               parallel(left(2, 2, 16, 40, 16, 300.0, 0.3), right(3, 3, 8, 8, 5), 1.0, 1.0, dense(36))]),
    # no size a multiple of 8; nothing rotated in one layer, two values in the other; one tap (no convolution at all)
    # beside two
    "r": config(75, 36, 4.0, [parallel(left(3, 1, 10, 6, 0, 20.0, 0.5), right(2, 1, 6, 5, 1), 0.4, 0.9, dense(22)),
                              mamba2(5, 6, 7, 1, 5, 2, None),
                              parallel(left(6, 3, 6, 10, 2, 20.0, 0.5), right(6, 2, 5, 3, 2), 0.4, 0.9, dense(22))],
                eps=1e-6),
    # heads of 128 keys and 64 values (the tensor-core attention kernels in bfloat16), a delta rule with 96 key channels
    # and 40 values (two runs of value columns), a state of 128 rows
    "s": config(101, 64, 1.5, [_S_PAR, mamba2(2, 48, 128, 2, 2, 4, dense(72)), dict(_S_PAR, weights_of=0)]),
}
RANKS = {"p": (5, 3), "q": (8, 16), "r": (3, 7), "s": (16, 8)}  # of the decay's and the gate's low-rank pairs


def tensors(cfg, ranks, seed, std=0.08, sink_std=1.0):
    """Matrices ~ N(0, std) with the projections of queries, keys and gates four times wider (a tiny model with
    N(0, 0.02) has near-uniform attention rows in which a dropped key hardly shows), sinks ~ N(0, sink_std), norm
    weights around zero, taps around 1 / taps, all rounded to bfloat16 as a checkpoint stores them."""
    g = torch.Generator().manual_seed(seed)
    out = {}

    def mat(name, *shape, s=std):
        out[name] = (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    def around(name, n, centre, spread):
        out[name] = (centre + spread * (2 * torch.rand(n, generator=g) - 1)).to(torch.bfloat16)

    d = cfg["width"]
    mat("embed", cfg["vocab"], d, s=1.0)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        around(p + "norm1", d, 0.0, 0.4)
        if layer["type"] == "mamba2":
            h, v, n, gr, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = h * v, h * v + 2 * gr * n
            mat(p + "mix.in", inner + ch + h, d, s=4 * std)
            mat(p + "mix.conv", ch, taps, s=0.6)
            mat(p + "mix.conv.b", ch, s=0.3)
            around(p + "mix.dt_bias", h, 0.0, 1.0), around(p + "mix.A_log", h, -0.5, 1.0), around(p + "mix.D", h, 1.0, 0.5)
            around(p + "mix.norm", inner, 1.0, 0.4)
            mat(p + "mix.o", d, inner)
        else:
            l, r = m["left"], m["right"]
            h, kv, k, v = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            q = p + "mix.left."
            mat(q + "q", h * k, d, s=4 * std), mat(q + "q.b", h * k, s=0.5)
            mat(q + "k", kv * k, d, s=4 * std), mat(q + "k.b", kv * k, s=0.5)
            mat(q + "v", kv * v, d, s=4 * std), mat(q + "v.b", kv * v, s=0.5)
            mat(q + "sink", h, s=sink_std), mat(q + "g", h * v, d, s=4 * std), mat(q + "o", d, h * v)
            h, kv, k, v, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            ra, rg = ranks
            q = p + "mix.right."
            for n, rows in (("q", kv * k), ("k", kv * k), ("v", h * v)):
                mat(q + n, rows, d, s=4 * std)
                mat(q + n + ".conv", rows, taps, s=0.6)
            mat(q + "b", h, d, s=4 * std)
            around(q + "A_log", h, -1.0, 1.0), around(q + "norm", v, 1.0, 0.4)
            mat(q + "a1", ra, d, s=4 * std), mat(q + "a2", h * k, ra, s=0.5), mat(q + "dt_bias", h * k, s=1.0)
            mat(q + "g1", rg, d, s=4 * std), mat(q + "g2", h * v, rg, s=0.5)
            mat(q + "o", d, h * v)
        if layer["mlp"] is not None:
            f = layer["mlp"]["ff"]
            around(p + "norm2", d, 0.0, 0.4)
            mat(p + "mlp.gate", f, d, s=4 * std), mat(p + "mlp.up", f, d, s=4 * std), mat(p + "mlp.down", d, f)
    around("final.norm", d, 0.0, 0.4)
    mat("head", cfg["vocab"], d)
    return out


def write_folder(path, cfg, weights):
    from fms_b200.weights.safetensors_io import write_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.contiguous() for k, v in weights.items()}, {})
    return path


def prompt(cfg, length, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, cfg["vocab"], (length,), generator=g).tolist()
