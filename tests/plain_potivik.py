"""A plain, slow implementation of the Potivik design, one function per
mechanism, on whole sequences with torch tensors on the CPU (float64 unless
told otherwise).  It shares no code with the engine: the GPU tests compare the
engine with these functions.

Notation: T tokens, d model width, H heads.  ``W`` maps tensor names (without
the layer prefix) to tensors, linear weights stored [out, in].
"""
from __future__ import annotations

import math

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rotate_pairs(v, positions, base, dims):
    """v [T, ..., D]: the first ``dims`` entries of the last axis are rotated,
    entry 2i with entry 2i+1, by positions[t] * base^(-2i/dims)."""
    out = v.clone()
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]            # [T, half]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_attention(h, m, W, eps):
    """h [T, d]; m: the mixer's sizes and constants.  Every position sees itself and the
    window - 1 positions before it."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, rdims, scale = m["rot"]["base"], m["rot"].get("dims", dr), m["scale"]
    window = (m.get("mask") or {}).get("size") or T              # no mask: every earlier position
    pos = torch.arange(T)
    q = (h @ W["q"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_pairs(q[..., dn:], pos, base, rdims)
    dkv = h @ W["dkv"].T
    c = rms_norm(dkv[:, :r], W["dkv.norm"], eps)
    k_rot = rotate_pairs(dkv[:, r:], pos, base, rdims)                 # [T, dr], one for all heads
    k_plain = (c @ W["uk"].T).reshape(T, H, dn)
    v = (c @ W["uv"].T).reshape(T, H, dv)
    gate = torch.sigmoid(h @ W["g"].T)                                 # [T, H]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        lo = max(0, t - window + 1)
        s = (torch.einsum("hd,jhd->hj", q_plain[t], k_plain[lo:t + 1])
             + torch.einsum("hd,jd->hj", q_rot[t], k_rot[lo:t + 1])) * scale
        p = torch.softmax(s, dim=-1)
        out[t] = torch.einsum("hj,jhd->hd", p, v[lo:t + 1])
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ W["o"].T


def causal_conv(x, taps, bias):
    """x [T, C]; taps [C, K] whose last column multiplies the current token; zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], 0)
    out = torch.zeros_like(x)
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    return out + bias


def mamba2(h, m, W, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ W["in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W["conv"], W["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W["dt_bias"])                                   # [T, H]
    decay = torch.exp(-torch.exp(W["A_log"]) * dt)                     # [T, H]
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    per = H // G
    for t in range(T):
        for hh in range(H):
            g = hh // per
            S[hh] = decay[t, hh] * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + W["D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms_norm(y.reshape(T, ng, inner // ng), None, eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


def clamped_glu(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def dense_ff(h, f, W):
    return clamped_glu(h, W["gate"], W["up"], W["down"], f["limit"])


def moe_ff(h, f, W):
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(h @ W["router"].T)                               # [T, E]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            xin = (s[t, e] * h[t])[None, :]
            out[t] = out[t] + clamped_glu(xin, W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], f["expert"]["limit"])[0]
    if f.get("shared"):
        sh = clamped_glu(h, W["shared.gate"], W["shared.up"], W["shared.down"], f["shared"]["limit"])
        out = out + torch.sigmoid(h @ W["shared.sg"].T) * sh
    return out


def token_side(x, tokens, table, lo, hi, W, eps):
    e = table[tokens][:, lo:hi]
    g = gelu_tanh(x @ W["gate"].T) * e
    y = g @ W["proj"].T
    return x + rms_norm(y, W["norm"], eps)


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def forward(cfg, W, tokens, dtype=torch.float64, collect_layers=False):
    """Logits [T, vocab] of a whole sequence (and, on request, the residual stream after every layer)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = W["embed"][tokens]
    side = cfg.get("token_side")
    after = []
    for i, layer in enumerate(cfg["layers"]):
        L = sub(W, f"l{i}.")
        h = layer_norm(x, L["norm1"], eps)
        mix = {"latent_attention": latent_attention, "mamba2": mamba2}[layer["type"]]
        x = x + layer_norm(mix(h, layer["mixer"], sub(L, "mix."), eps), L["norm1b"], eps)
        if layer.get("mlp"):
            h = layer_norm(x, L["norm2"], eps)
            ff = {"dense": dense_ff, "moe": moe_ff}[layer["mlp"]["kind"]]
            x = x + layer_norm(ff(h, layer["mlp"], sub(L, "mlp.")), L["norm2b"], eps)
        if side:
            d = side["dim"]
            x = token_side(x, tokens, W["side.embed"], i * d, (i + 1) * d, sub(L, "side."), eps)
        after.append(x)
    z = layer_norm(x, W["final.norm"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        z = cap * torch.tanh(z / cap)
    return (z, torch.stack(after)) if collect_layers else z
