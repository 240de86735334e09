"""Small Goletar configurations and random weights for the tests, written from scratch here (checkpoint names and
config.json keys as a user's folder has them).  The sizes differ from one another in everything a configuration can
say: order of the layers, widths, heads, head sizes, rotated sizes (also fewer rotated values than the rotated part
holds), latent sizes, experts, experts per token (1, 2, 3), limits, multipliers of the pair hash, layers without a
feed-forward."""
import json
import os

import torch


def mingru(width, mlp):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, base, mlp, rot_dims=None, scale=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
                      "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}}


def experts(n, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": n, "top": top}}


def config(vocab, width, layers, eps=1e-5, buckets=61, mul_prev=7, mul_cur=13):
    return {"architecture": "Goletar", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": layers}


CONFIGS = {
    # attention first, two experts a token, a layer without a feed-forward, fewer rotated values than the part holds
    "p": config(97, 48, [latent(3, 16, 8, 12, 24, 5000.0, experts(5, 2, 20, 1.0), rot_dims=4),
                         mingru(40, None),
                         latent(3, 16, 8, 12, 24, 5000.0, experts(5, 2, 20, 1.0), rot_dims=4),
                         mingru(40, experts(5, 2, 20, 1.0))], eps=1e-4, buckets=31, mul_prev=3, mul_cur=5),
    # two recurrent layers in a row, one and three experts a token, hash products beyond 32 bits, a layer with one
    # head whose rotated part is larger than its unrotated one, values wider than keys
    "q": config(130, 64, [mingru(64, experts(3, 1, 36, 0.5)), mingru(72, experts(7, 3, 12, 2.5)),
                          latent(1, 8, 24, 40, 32, 100.0, experts(7, 3, 12, 2.5)),
                          latent(5, 24, 4, 8, 16, 100.0, None)], eps=1e-6, buckets=257, mul_prev=40_000_003,
                mul_cur=1_000_033),
    # a latent of 64 values and a row of 96: a prompt's rows of this one take the tensor-core attention kernel in
    # bfloat16 (five heads: a block holds four tokens of eight head places, three of them empty), and its experts'
    # products the library's grouped product
    "s": config(101, 64, [latent(5, 16, 32, 24, 64, 1000.0, experts(6, 2, 24, 1.0)), mingru(48, experts(6, 2, 24, 1.0)),
                          latent(5, 16, 32, 24, 64, 1000.0, None)], eps=1e-5, buckets=53, mul_prev=11, mul_cur=3),
    # sizes that are no multiples of 8 or 32, nine heads (more than one block of the attention kernel takes)
    "r": config(75, 36, [latent(9, 6, 2, 5, 10, 20.0, experts(4, 4, 9, 1.5)), mingru(35, experts(4, 4, 9, 1.5))],
                eps=1e-5, buckets=11, mul_prev=1, mul_cur=1),
}


def tensors(cfg, seed, std=0.08, router_std=0.6, sink_std=1.0):
    """Matrices ~ N(0, std) (a tiny model with N(0, 0.02) has near-uniform attention rows in which a dropped key
    hardly shows), router rows wider so that the experts' scores are well apart, sinks ~ N(0, sink_std), norm
    numbers 0.5 + U(0, 1), all rounded to bfloat16 as a checkpoint stores them."""
    g = torch.Generator().manual_seed(seed)
    out = {}

    def mat(name, *shape, s=std):
        out[name] = (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    def number(name):
        out[name] = (0.5 + torch.rand((), generator=g)).to(torch.bfloat16)

    d = cfg["width"]
    mat("embed", cfg["vocab"], d, s=1.0)
    mat("bigram", cfg["embedding"]["bigram"]["buckets"] + 1, d, s=1.0)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        number(p + "norm1"), number(p + "norm1b")
        if layer["type"] == "mingru":
            w = m["width"]
            for n in ("z", "x", "g"):
                mat(p + "mix." + n, w, d, s=4 * std)
            mat(p + "mix.z.b", w, s=1.0), mat(p + "mix.x.b", w, s=1.0)
            mat(p + "mix.o", d, w)
        else:
            h, dim, rot, v, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            mat(p + "mix.q", h * (dim + rot), d, s=4 * std)
            mat(p + "mix.dkv", r + rot, d, s=4 * std)
            out[p + "mix.dkv.norm"] = (0.5 + torch.rand(r, generator=g)).to(torch.bfloat16)
            mat(p + "mix.uk", h * dim, r, s=4 * std), mat(p + "mix.uv", h * v, r)
            mat(p + "mix.sink", h, s=sink_std), mat(p + "mix.g", h, d, s=4 * std), mat(p + "mix.o", d, h * v)
        if layer["mlp"] is not None:
            mlp = layer["mlp"]
            number(p + "norm2"), number(p + "norm2b")
            mat(p + "mlp.router", mlp["router"]["experts"], d, s=router_std)
            for j in range(mlp["router"]["experts"]):
                mat(p + f"mlp.e{j}.gate", mlp["expert"]["ff"], d, s=4 * std)
                mat(p + f"mlp.e{j}.up", mlp["expert"]["ff"], d, s=4 * std)
                mat(p + f"mlp.e{j}.down", d, mlp["expert"]["ff"])
    number("final.norm")
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
