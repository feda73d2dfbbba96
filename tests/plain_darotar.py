"""Darotar, slowly and plainly: whole sequences in float64, one function per mechanism. Shares no code with the
package; the tests compare the engine with it.

A model is ``(config dict, {tensor name: tensor})``. ``logits(cfg, w, ids)`` returns ``[len(ids), vocab]``;
``forward(cfg, w, ids)`` also returns the residual stream after every layer.
"""
import math

import torch

F = torch.float64

# With a storage type set (``with stored_as(torch.bfloat16):``) every tensor that an engine would keep in that type between
# two operations (what the sublayers read, projections, cached rows, activations) is rounded to it and taken on in
# float64. The difference to the unrounded result is what rounding alone does to this model's logits: the tests judge
# an engine's bfloat16 results by a multiple of it.
_STORED = None


class stored_as:
    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global _STORED
        self.before, _STORED = _STORED, self.dtype

    def __exit__(self, *exc):
        global _STORED
        _STORED = self.before


def kept(x):
    return x if _STORED is None else x.to(_STORED).to(F)


def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    return rms_unit(x, eps) * w


def frequencies(rot):
    """One frequency per rotated pair; a linear scaling divides all of them."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    sc = rot.get("scaling")
    return f / float(sc["factor"]) if sc else f


def rotate_interleaved(x, rot, first=0):
    """x [T, heads, d]: the first rot.dims elements of every head turned by position; element 2i with 2i + 1."""
    dims = int(rot["dims"])
    a = (first + torch.arange(x.shape[0], dtype=F))[:, None] * frequencies(rot)[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def rotate_half(x, rot, first=0):
    """x [T, heads, d]: the first rot.dims elements of every head turned by position; element i with i + dims/2."""
    dims = int(rot["dims"])
    half = dims // 2
    a = (first + torch.arange(x.shape[0], dtype=F))[:, None] * frequencies(rot)[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def visible(t_len, window=None):
    """[T, T] bool: j <= i, and with a window also i - j < window."""
    i = torch.arange(t_len)[:, None]
    j = torch.arange(t_len)[None, :]
    m = j <= i
    if window:
        m = m & (i - j < window)
    return m


def softmax_rows(s, mask, sink=None):
    """Softmax over the visible keys of every row; with ``sink`` the denominator has exp(sink) once more."""
    s = s.masked_fill(~mask, -math.inf)
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, torch.full_like(top, float(sink)))
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(float(sink) - top)
    return e / den


def attention_mixer(m, w, p, h, eps):
    """Windowed softmax attention whose values are the projected keys themselves."""
    t_len = h.shape[0]
    heads, groups, dim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w[p + ".q"].t()).view(t_len, heads, dim)
    k = (h @ w[p + ".k"].t()).view(t_len, groups, dim)
    v = kept(k)
    q, k = rotate_interleaved(q, m["rot"]), rotate_interleaved(k, m["rot"])
    q, k = kept(rms_unit(q, eps)), kept(rms_unit(k, eps))
    mask = visible(t_len, m["mask"]["size"] if m.get("mask") else None)
    rep = heads // groups
    out = torch.zeros(t_len, heads, dim, dtype=F)
    for n in range(heads):
        s = (q[:, n] @ k[:, n // rep].t()) * float(m["scale"])
        out[:, n] = softmax_rows(s, mask) @ v[:, n // rep]
    return kept(out).reshape(t_len, -1) @ w[p + ".o"].t()


def latent_rows(m, w, p, h, eps):
    """What a latent layer caches per position: the normed latent and the shared rotated key part."""
    rank = int(m["kv_rank"])
    z = h @ w[p + ".dkv"].t()
    c = norm(z[:, :rank], w[p + ".dkv.norm"], eps)
    kr = rotate_half(z[:, None, rank:], m["rot"])[:, 0]
    return kept(c), kept(kr)


def latent_mixer(m, w, p, h, eps, rows):
    """Attention through a latent with a sink in the softmax and a gate on the output. ``rows`` = (latent, rotated key
    part) of this layer or of the layer it borrows them from."""
    t_len = h.shape[0]
    heads, dim, rdim, vdim = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    c, kr = rows
    cq = kept(norm(h @ w[p + ".dq"].t(), w[p + ".dq.norm"], eps))
    q = (cq @ w[p + ".uq"].t()).view(t_len, heads, dim + rdim)
    q_plain, q_rot = kept(q[..., :dim]), kept(rotate_half(q[..., dim:], m["rot"]))
    k_plain = (c @ w[p + ".uk"].t()).view(t_len, heads, dim)
    v = (c @ w[p + ".uv"].t()).view(t_len, heads, vdim)
    mask = visible(t_len, m["mask"]["size"] if m.get("mask") else None)
    out = torch.zeros(t_len, heads, vdim, dtype=F)
    for n in range(heads):
        s = (q_plain[:, n] @ k_plain[:, n].t() + q_rot[:, n] @ kr.t()) * float(m["scale"])
        out[:, n] = softmax_rows(s, mask, sink=w[p + ".sink"][n]) @ v[:, n]
    gate = torch.sigmoid(h @ w[p + ".g"].t())
    return kept(out.reshape(t_len, -1) * gate) @ w[p + ".o"].t()


def routed_experts(mlp, w, p, h):
    """Every token goes to the ``top`` experts with the largest sigmoid scores; the score multiplies the expert's input."""
    n_exp, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    s = torch.sigmoid(h @ w[p + ".router"].t())
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(s[t], top).indices.tolist()
        for e in chosen:
            x = s[t, e] * h[t]
            g = x @ w[f"{p}.e{e}.gate"].t()
            u = x @ w[f"{p}.e{e}.up"].t()
            out[t] += kept(g * torch.sigmoid(g) * u) @ w[f"{p}.e{e}.down"].t()
    assert n_exp >= top
    return out


def forward(cfg, w, ids):
    w = {k: v.to(F) for k, v in w.items() if v.is_floating_point()}
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)]
    streams = []
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix"
        h = kept(x)         # the sublayers read the stream itself (an engine: in its storage type)
        if layer["type"] == "attention":
            y = attention_mixer(m, w, p, h, eps)
        else:
            src = m.get("kv_from")
            if src is None:
                cached[i] = latent_rows(m, w, p, h, eps)
                src = i
            y = latent_mixer(m, w, p, h, eps, cached[src])
        x = x + mult * norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + mult * norm(routed_experts(layer["mlp"], w, f"l{i}.mlp", kept(x)), w[f"l{i}.norm2"], eps)
        streams.append(x)
    return kept(norm(x, w["final.norm"], eps)) @ w["head"].t(), streams


def logits(cfg, w, ids):
    return forward(cfg, w, ids)[0]
