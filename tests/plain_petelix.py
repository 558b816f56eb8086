"""A plain, slow implementation of the Petelix design in float64, one function
per mechanism, written from the design's equations.  It shares no code with the
engine: the tests compare the two.

A model is (config dict, {tensor name: tensor}).  Sequences are handled one at
a time and whole: position t sees what the design lets it see of positions 0..t.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def rotate_pairs(x, positions, base, dims):
    """x [T, heads, dim]: entries (2i, 2i+1), i < dims/2, of every head are turned by the
    angle position * base^(-2i/dims); the other entries stay."""
    if dims == 0:
        return x
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    ang = positions.to(F64)[:, None] * torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def keys_and_values(h, w, m, eps, positions):
    """What an attention layer with projections of its own puts into its cache:
    keys after the norm over the whole projection and the rotation, and values."""
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    k = rms_norm(h @ w["k"].T, w["k.norm"], eps).reshape(-1, G, dim)
    rot = m.get("rot") or {}
    k = rotate_pairs(k, positions, rot.get("base", 1.0), int(rot.get("dims", 0)))
    v = (h @ w["v"].T).reshape(-1, G, vdim)
    return k, v


def sink_softmax_attention(q, k, v, scale, softcap, window):
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim] of one sequence.  Position i sees j with
    0 <= i - j < window (all j <= i without one).  The scores pass cap * tanh(s / cap) when
    there is a cap; the weights are exp(s_j) / (1 + sum exp(s_j))."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd, :] @ k[:, g, :].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        seen = (j <= i) if not window else ((j <= i) & (i - j < window))
        e = torch.where(seen, torch.exp(s), torch.zeros_like(s))
        p = e / (1.0 + e.sum(-1, keepdim=True))
        out[:, hd, :] = p @ v[:, g, :]
    return out


def attention_mixer(h, w, m, eps, positions, kv):
    """The whole mixer for one sequence.  ``kv``: (keys, values) of the layer whose cache
    this layer reads, or None for a layer with projections of its own.  Returns
    (output [T, width], (keys, values))."""
    H, dim = m["heads"], m["dim"]
    q = rms_norm(h @ w["q"].T, w["q.norm"], eps).reshape(-1, H, dim)
    rot = m.get("rot") or {}
    q = rotate_pairs(q, positions, rot.get("base", 1.0), int(rot.get("dims", 0)))
    if kv is None:
        kv = keys_and_values(h, w, m, eps, positions)
    mask = m.get("mask") or {}
    o = sink_softmax_attention(q, kv[0], kv[1], m["scale"], m.get("softcap") or 0.0, mask.get("size"))
    o = o.reshape(o.shape[0], -1) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T, kv


def route(h, w, r):
    """Which experts each token uses and with which weights: (choice [T, top], weight [T, top]).
    Softmax scores over all router outputs; the choice is made on score + correction inside
    the groups that are kept; the weight is the score itself."""
    z = h @ w["router"].T
    s = torch.softmax(z, -1)
    c = s + w["correction"] if "correction" in w else s.clone()
    n = c.shape[1]
    groups = r.get("groups") or {}
    count, keep = int(groups.get("count", 1)), int(groups.get("keep", groups.get("count", 1)))
    if count > 1 and keep < count:
        best = c.reshape(-1, count, n // count).max(-1).values
        kept = torch.topk(best, keep, dim=-1).indices
        allowed = torch.zeros(c.shape[0], count, dtype=torch.bool)
        allowed.scatter_(1, kept, True)
        allowed = allowed[:, :, None].expand(-1, -1, n // count).reshape(-1, n)
        c = torch.where(allowed, c, torch.full_like(c, -math.inf))
    choice = torch.topk(c, int(r["top"]), dim=-1).indices
    return choice, torch.gather(s, 1, choice)


def expert(h, w, e):
    g = h @ w[f"e{e}.gate"].T
    return ((g * torch.sigmoid(g)) * (h @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T


def routed_experts(h, w, f):
    """Weighted sum of the chosen experts' outputs; the last ``identity`` router outputs
    stand for experts that return their input."""
    r = f["router"]
    E = int(r["experts"])
    choice, weight = route(h, w, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(choice[t].tolist(), weight[t]):
            out[t] += p * (expert(h[t:t + 1], w, e)[0] if e < E else h[t])
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, want=None, layers_out=None):
    """Logits [len(want) or T, vocab] of one sequence; ``layers_out`` (a list) receives the
    stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tokens))
    x = tensors["embed"].to(F64)[ids] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    caches = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, tensors[p + "norm1"].to(F64), eps)
        src = m.get("kv_from")
        y, kv = attention_mixer(h, sub(tensors, p + "mix."), m, eps, pos, None if src is None else caches[src])
        caches[i] = kv
        x = x + y
        if layer.get("mlp") is not None:
            h = rms_norm(x, tensors[p + "norm2"].to(F64), eps)
            x = x + routed_experts(h, sub(tensors, p + "mlp."), layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, tensors["final.norm"].to(F64), eps)
    if want is not None:
        x = x[torch.as_tensor(want, dtype=torch.long)]
    return x @ tensors["head"].to(F64).T
