"""A plain, slow restatement of the Goletar design: whole sequences, no cache, no batching, one function per
mechanism, float64 by default.  It reads a configuration (the config.json dictionary) and the checkpoint's tensors by
their checkpoint names and shares no code with the library.

    embedding        e_t = embed[tok_t] + bigram[(tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets]; bigram[buckets] for t = 0
    scalar norm      n(x) = g * x / sqrt(mean(x^2) + eps), g one number
    layer            x += n1b(mixer(n1(x)));  x += n2b(experts(n2(x))) where the layer has a feed-forward
    mingru           z = sigmoid(Wz h + bz); u = Wx h + bx; c = u + 1/2 (u >= 0) | sigmoid(u) (u < 0)
                     S_t = (1 - z) S_(t-1) + z c; y = Wo (S_t * silu(Wg h))
    latent attention q = Wq h (per head [dim | rot]); [c' | kr] = Wdkv h; c = rmsnorm(c') * w; k_h = [Wuk,h c | kr];
                     v_h = Wuv,h c; rotation of the rot parts (adjacent pairs, first rot.dims values, angle = p * base^(-2i/dims));
                     s = q.k * scale, causal; p = exp(s) / (sum exp(s) + exp(sink_h)); o_h = sigmoid(Wg h)_h * sum p v; y = Wo o
    experts          s = sigmoid(Wr h); the top-k s; y = sum_e expert_e(s_e * h);
                     expert(v) = Wdown (g * sigmoid(1.702 g) * (u + 1)), g = min(Wgate v, limit), u = clamp(Wup v, +-limit)
    output           logits = head n_final(x)
"""
import math

import torch


def scalar_norm(x, g, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def pair_hash_embedding(tokens, embed, bigram, buckets, mul_prev, mul_cur):
    rows = [buckets if t == 0 else (tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets for t in range(len(tokens))]
    return embed[torch.tensor(tokens)] + bigram[torch.tensor(rows)]


def mingru(h, wz, bz, wx, bx, wg, wo, state=None):
    z = torch.sigmoid(h @ wz.T + bz)
    u = h @ wx.T + bx
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    s = torch.zeros(wz.shape[0], dtype=h.dtype) if state is None else state
    out = []
    for t in range(h.shape[0]):
        s = (1 - z[t]) * s + z[t] * cand[t]
        out.append(s)
    g = h @ wg.T
    return (torch.stack(out) * (g * torch.sigmoid(g))) @ wo.T


def rotate_pairs(v, positions, dims, base):
    """v [n, ..., width]: the first ``dims`` values of the last axis are rotated pair by pair, the rest pass."""
    half = dims // 2
    if half == 0:
        return v
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    ang = positions.to(v.dtype)[:, None] * f[None]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cs, sn = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * cs - b * sn
    out[..., 1:dims:2] = b * cs + a * sn
    return out


def latent_attention(h, m, eps, wq, wdkv, wnorm, wuk, wuv, sink, wg, wo, first_position=0):
    n = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    dims, base = m["rot"]["dims"], m["rot"]["base"]
    pos = torch.arange(first_position, first_position + n)
    q = (h @ wq.T).view(n, heads, dim + rot)
    dkv = h @ wdkv.T
    c = dkv[:, :rank]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * wnorm
    kr = rotate_pairs(dkv[:, rank:], pos, dims, base)
    qr = rotate_pairs(q[:, :, dim:], pos, dims, base)
    ku = (c @ wuk.T).view(n, heads, dim)
    v = (c @ wuv.T).view(n, heads, vdim)
    s = (torch.einsum("ihd,jhd->hij", q[:, :, :dim], ku) + torch.einsum("ihr,jr->hij", qr, kr)) * m["scale"]
    s = s.masked_fill(~torch.tril(torch.ones(n, n, dtype=torch.bool)), -math.inf)
    top = torch.maximum(s.max(-1).values, sink[:, None])
    e = torch.exp(s - top[..., None])
    p = e / (e.sum(-1) + torch.exp(sink[:, None] - top))[..., None]
    o = torch.einsum("hij,jhv->ihv", p, v) * torch.sigmoid(h @ wg.T)[:, :, None]
    return o.reshape(n, heads * vdim) @ wo.T, p


def routed_experts(h, router, gates, ups, downs, top, limit):
    logit = h @ router.T
    scores = torch.sigmoid(logit)
    out = torch.zeros_like(h)
    chosen = []
    for t in range(h.shape[0]):
        order = sorted(range(scores.shape[1]), key=lambda e: (-scores[t, e].item(), e))[:top]
        chosen.append(order)
        for e in order:
            v = scores[t, e] * h[t]
            g = torch.clamp(gates[e] @ v, max=limit)
            u = torch.clamp(ups[e] @ v, -limit, limit)
            out[t] += downs[e] @ (g * torch.sigmoid(1.702 * g) * (u + 1))
    return out, chosen


def routing_margin(h, router, top):
    """Per token: how far the last chosen expert's router logit lies above the best one left out, relative to the
    largest logit of the token (infinite where every expert is chosen).  A test that compares a 16-bit run with this
    restatement looks only at tokens whose margin is wider than 16-bit rounding."""
    logit = (h @ router.T).sort(-1, descending=True).values
    if top >= logit.shape[1]:
        return torch.full((h.shape[0],), math.inf, dtype=h.dtype)
    return (logit[:, top - 1] - logit[:, top]) / logit.abs().max(-1).values.clamp_min(1.0)


class PlainGoletar:
    def __init__(self, config: dict, tensors: dict, dtype=torch.float64):
        self.cfg = config
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.eps = config["norm"]["eps"]

    def logits(self, tokens, layers_out=None):
        cfg, w, eps = self.cfg, self.w, self.eps
        pairs = cfg["embedding"]["bigram"]
        x = pair_hash_embedding(list(tokens), w["embed"], w["bigram"], pairs["buckets"], pairs["mul_prev"], pairs["mul_cur"])
        self.margin = torch.full((len(tokens),), math.inf, dtype=x.dtype)  # of the last call: see routing_margin
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            h = scalar_norm(x, w[p + "norm1"], eps)
            if layer["type"] == "mingru":
                a = mingru(h, w[p + "mix.z"], w[p + "mix.z.b"], w[p + "mix.x"], w[p + "mix.x.b"], w[p + "mix.g"], w[p + "mix.o"])
            else:
                a, _ = latent_attention(h, layer["mixer"], eps, w[p + "mix.q"], w[p + "mix.dkv"], w[p + "mix.dkv.norm"],
                                        w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.sink"], w[p + "mix.g"], w[p + "mix.o"])
            x = x + scalar_norm(a, w[p + "norm1b"], eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                h = scalar_norm(x, w[p + "norm2"], eps)
                n_e = mlp["router"]["experts"]
                self.margin = torch.minimum(self.margin, routing_margin(h, w[p + "mlp.router"], mlp["router"]["top"]))
                y, _ = routed_experts(h, w[p + "mlp.router"], [w[p + f"mlp.e{j}.gate"] for j in range(n_e)],
                                      [w[p + f"mlp.e{j}.up"] for j in range(n_e)],
                                      [w[p + f"mlp.e{j}.down"] for j in range(n_e)], mlp["router"]["top"],
                                      mlp["expert"]["limit"])
                x = x + scalar_norm(y, w[p + "norm2b"], eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        return scalar_norm(x, w["final.norm"], eps) @ w["head"].T
