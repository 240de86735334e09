"""A plain, slow restatement of the Niletar design: whole sequences, no cache, no batching, one function per
mechanism, float64 by default.  It reads a configuration (the config.json dictionary) and the checkpoint's tensors by
their checkpoint names and shares no code with the library.

    norm             n(x) = x / sqrt(mean(x^2) + eps) * (1 + w)
    layer            x = n1(alpha x + mixer(x));  x = n2(alpha x + mlp(x)) where the layer has a feed-forward
    mamba2           [z | x | B | C | dt] = Win h; (x, B, C) = silu(conv(x, B, C) + b); dt = softplus(dt + dt_bias)
                     S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T;  y_t = S_t^T C_t + D x_t
                     out = Wo (groupnorm(y * silu(z)) * w)
    parallel         left_scale * attention(h) + right_scale * delta_rule(h)
    attention        q, k, v = Wq h + bq, Wk h + bk, Wv h + bv; pairs (2i, 2i+1) of the first rot.dims values rotated by
                     p * f_i, f_i rescaled for long wavelengths; q, k divided by their root mean square; s = q.k * scale,
                     causal; p = exp(s) / (sum exp(s) + exp(sink_h)); out = Wo (sum p v * sigmoid(Wg h))
    delta rule       q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h)); q, k unit vectors, q / sqrt(dim)
                     beta = sigmoid(Wb h); g = exp(-exp(A_log_h) softplus(Wa2 Wa1 h + dt_bias))   (per head and key channel)
                     S = g S; u = beta (v - S^T k); S = S + k u^T; o = S^T q
                     out = Wo (o / rms(o) * w * sigmoid(Wg2 Wg1 h))
    dense            Wdown (silu(Wgate h) * Wup h)
    output           logits = head n_final(x)
"""
import math

import torch


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def offset_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1 + w)


def causal_conv(x, taps_w, bias=None, before=None):
    """x [n, channels]; taps_w [channels, taps], its last column multiplies the current row; rows before the start
    are zeros (or ``before`` [taps - 1, channels])."""
    n, c = x.shape
    taps = taps_w.shape[1]
    pad = torch.zeros(taps - 1, c, dtype=x.dtype) if before is None else before
    xp = torch.cat([pad, x], 0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + xp[j:j + n] * taps_w[:, j][None]
    return out if bias is None else out + bias[None]


def rotary_frequencies(dims, base, scaling=None):
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for v in f:
            wavelength = 2 * math.pi / v
            if wavelength < orig / high:
                out.append(v)
            elif wavelength > orig / low:
                out.append(v / factor)
            else:
                s = (orig / wavelength - low) / (high - low)
                out.append((1 - s) * v / factor + s * v)
        f = out
    return f


def rotate_pairs(v, positions, dims, freqs):
    """v [n, heads, width]: the first ``dims`` values of every head, pair (2i, 2i + 1) by the angle p * f_i."""
    if dims == 0:
        return v
    ang = positions.to(v.dtype)[:, None] * torch.tensor(freqs, dtype=v.dtype)[None]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * cs - b * sn
    out[..., 1:dims:2] = b * cs + a * sn
    return out


def sink_attention(h, m, eps, t, p, first_position=0):
    """t: the checkpoint's tensors, p: the prefix of this mixer's names ('l0.mix.left.')."""
    n = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ t[p + "q"].T + t[p + "q.b"]).view(n, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).view(n, G, d)
    v = (h @ t[p + "v"].T + t[p + "v.b"]).view(n, G, dv)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    pos = torch.arange(first_position, first_position + n)
    if dims:
        f = rotary_frequencies(dims, float(rot["base"]), rot.get("scaling"))
        q, k = rotate_pairs(q, pos, dims, f), rotate_pairs(k, pos, dims, f)
    q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps)
    k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps)
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    sink = t[p + "sink"]
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * float(m["scale"])
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, sink[head])
        e = torch.exp(s - top)
        w = e / (e.sum(-1, keepdim=True) + torch.exp(sink[head] - top))
        out[:, head] = w @ v[:, kv]
    gate = torch.sigmoid(h @ t[p + "g"].T)
    return (out.reshape(n, H * dv) * gate) @ t[p + "o"].T


def gated_delta_rule(h, m, eps, t, p):
    n = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_conv(h @ t[p + "q"].T, t[p + "q.conv"])).view(n, G, d)
    k = silu(causal_conv(h @ t[p + "k"].T, t[p + "k.conv"])).view(n, G, d)
    v = silu(causal_conv(h @ t[p + "v"].T, t[p + "v.conv"])).view(n, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ t[p + "b"].T)  # [n, H]
    a = (h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "dt_bias"]
    decay = torch.exp(-torch.exp(t[p + "A_log"])[None, :, None] * softplus(a).view(n, H, d))
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for i in range(n):
            S = decay[i, head][:, None] * S
            u = beta[i, head] * (v[i, head] - S.T @ k[i, kv])
            S = S + torch.outer(k[i, kv], u)
            out[i, head] = S.T @ q[i, kv]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * t[p + "norm"]
    gate = torch.sigmoid((h @ t[p + "g1"].T) @ t[p + "g2"].T)
    return (out.reshape(n, H * dv) * gate) @ t[p + "o"].T


def parallel_mixer(h, m, eps, t, p, first_position=0):
    left = sink_attention(h, m["left"], eps, t, p + "left.", first_position)
    right = gated_delta_rule(h, m["right"], eps, t, p + "right.")
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def mamba2(h, m, eps, t, p):
    n = h.shape[0]
    H, dv, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * dv
    proj = h @ t[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, t[p + "conv"], t[p + "conv.b"]))
    x = xbc[:, :inner].view(n, H, dv)
    B = xbc[:, inner:inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = softplus(dt + t[p + "dt_bias"])  # [n, H]
    A = torch.exp(t[p + "A_log"])
    y = torch.zeros(n, H, dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(N, dv, dtype=h.dtype)
        for i in range(n):
            S = torch.exp(-A[head] * dt[i, head]) * S + dt[i, head] * torch.outer(B[i, g], x[i, head])
            y[i, head] = S.T @ C[i, g] + t[p + "D"][head] * x[i, head]
    y = y.reshape(n, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = y.view(n, parts, inner // parts)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    return (y.reshape(n, inner) * t[p + "norm"]) @ t[p + "o"].T


def dense(h, t, p):
    return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def logits(cfg, tensors, tokens, dtype=torch.float64, first_position=0, layers_out=None):
    """Logits [len(tokens), vocab] of one whole sequence.  ``layers_out``: a list that receives the stream after every
    layer."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    x = t["embed"][torch.tensor(list(tokens))]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        if layer["type"] == "mamba2":
            a = mamba2(x, layer["mixer"], eps, t, p + "mix.")
        elif layer["type"] == "parallel":
            a = parallel_mixer(x, layer["mixer"], eps, t, p + "mix.", first_position)
        else:
            raise ValueError(layer["type"])
        x = offset_norm(alpha * x + a, t[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = offset_norm(alpha * x + dense(x, t, p + "mlp."), t[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x)
    return offset_norm(x, t["final.norm"], eps) @ t["head"].T
