"""Dusilorn, slowly and plainly: whole sequences in float64, one function per mechanism. Shares no code with the
package; the tests compare the engine with it.

A model is ``(config dict, {tensor name: tensor})``. ``logits(cfg, w, ids)`` returns ``[len(ids), vocab]``;
``forward(cfg, w, ids)`` also returns the residual stream after every layer.

With a storage type set (``with stored_as(torch.bfloat16):``) every tensor that an engine keeps in that type between two
operations is rounded to it; the distance to the unrounded result is what rounding alone does to the model's logits.
"""
import math

import torch

F = torch.float64
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


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The layer norm of the design: the gain is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def rotate_half_pairs(x, rot, first=0):
    """x [T, heads, d]: element i of the first rot.dims elements of a head is paired with element i + dims/2."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = (first + torch.arange(x.shape[0], dtype=F))[:, None] * f[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def mask_window(t_len, size):
    i, j = torch.arange(t_len)[:, None], torch.arange(t_len)[None, :]
    return (j <= i) & (i - j < size)


def mask_chunk(t_len, size):
    i, j = torch.arange(t_len)[:, None], torch.arange(t_len)[None, :]
    return (j <= i) & (i // size == j // size)


def capped(s, cap):
    return cap * torch.tanh(s / cap) if cap else s


def softmax_visible(s, mask, sink=None):
    """Softmax of every row over its visible keys; a sink adds exp(sink) to the denominator, once, with no value."""
    s = s.masked_fill(~mask, -math.inf)
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.clamp(top, min=float(sink))
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + math.exp(float(sink)) * torch.exp(-top)
    return e / den


def mixed_values(m, w, p, v, shared):
    """v of a layer with v_mix: the first such layer leaves its own values for the later ones, which blend theirs with them."""
    if not m.get("v_mix"):
        return v
    if "v_first" not in shared:
        shared["v_first"] = v
        return v
    lam = w[p + ".vmix"]
    return (1.0 - lam) * v + lam * shared["v_first"]


def heads_attend(q, k, v, m, mask, sinks=None):
    t_len, heads = q.shape[0], q.shape[1]
    rep = heads // k.shape[1]
    out = torch.zeros(t_len, heads, v.shape[-1], dtype=F)
    for n in range(heads):
        s = capped((q[:, n] @ k[:, n // rep].t()) * float(m["scale"]), float(m.get("softcap") or 0.0))
        out[:, n] = softmax_visible(s, mask, None if sinks is None else sinks[n]) @ v[:, n // rep]
    return out


def chunked_sink_attention(m, w, p, h, eps, shared):
    """Mixer 'attention': q and k normed over the whole projection, no positions, chunked mask, a sink per head."""
    t_len = h.shape[0]
    heads, groups, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = unit_rms(h @ w[p + ".q"].t(), eps) * w[p + ".q.norm"]
    k = unit_rms(h @ w[p + ".k"].t(), eps) * w[p + ".k.norm"]
    v = mixed_values(m, w, p, h @ w[p + ".v"].t(), shared)
    q, k, v = kept(q).view(t_len, heads, dim), kept(k).view(t_len, groups, dim), kept(v).view(t_len, groups, vdim)
    out = heads_attend(q, k, v, m, mask_chunk(t_len, int(m["mask"]["size"])), w[p + ".sink"])
    return kept(out).reshape(t_len, -1) @ w[p + ".o"].t()


def rotary_window_attention(m, w, p, h, eps, shared):
    """Mixer 'attention_2': rotated q and k, sliding window, ordinary softmax."""
    t_len = h.shape[0]
    heads, groups, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rotate_half_pairs((h @ w[p + ".q"].t()).view(t_len, heads, dim), m["rot"])
    k = rotate_half_pairs((h @ w[p + ".k"].t()).view(t_len, groups, dim), m["rot"])
    v = mixed_values(m, w, p, h @ w[p + ".v"].t(), shared)
    q, k, v = kept(q), kept(k), kept(v).view(t_len, groups, vdim)
    out = heads_attend(q, k, v, m, mask_window(t_len, int(m["mask"]["size"])))
    return kept(out).reshape(t_len, -1) @ w[p + ".o"].t()


def dense_ff(w, p, h):
    g, u = h @ w[p + ".gate"].t(), h @ w[p + ".up"].t()
    return kept(g * torch.sigmoid(g) * u) @ w[p + ".down"].t()


def small_expert(w, p, h):
    """W_down relu(W_up h)^2."""
    return kept(torch.relu(h @ w[p + ".up"].t()) ** 2) @ w[p + ".down"].t()


def route(mlp, w, p, h):
    """Per token: the chosen router outputs (the first of equal ones) and their weights."""
    top = int(mlp["router"]["top"])
    s = torch.softmax(h @ w[p + ".router"].t(), dim=-1)
    choice = s + w[p + ".correction"]
    chosen, weights = [], []
    for t in range(h.shape[0]):
        order = sorted(range(s.shape[1]), key=lambda e: (-float(choice[t, e]), e))[:top]
        sel = s[t, order]
        chosen.append(order)
        weights.append(sel / (sel.sum() + 1e-20))
    return chosen, weights


def mixture(mlp, w, p, h):
    n_exp = int(mlp["router"]["experts"])
    chosen, weights = route(mlp, w, p, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            out[t] += wt * (small_expert(w, f"{p}.e{e}", h[t:t + 1])[0] if e < n_exp else h[t])   # the last outputs: identity
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[p + ".shared.sg"].t()) * small_expert(w, p + ".shared", h)
    return out


def forward(cfg, w, ids):
    w = {k: v.to(F) for k, v in w.items() if v.is_floating_point()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    streams, shared = [], {}
    for i, layer in enumerate(cfg["layers"]):
        mixer = chunked_sink_attention if layer["type"] == "attention" else rotary_window_attention
        y = mixer(layer["mixer"], w, f"l{i}.mix", kept(norm_one_plus(x, w[f"l{i}.norm1"], eps)), eps, shared)
        x = x + norm_one_plus(y, w[f"l{i}.norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = kept(norm_one_plus(x, w[f"l{i}.norm2"], eps))
            y = dense_ff(w, f"l{i}.mlp", h) if mlp["kind"] == "dense" else mixture(mlp, w, f"l{i}.mlp", h)
            x = x + norm_one_plus(y, w[f"l{i}.norm2b"], eps)
        streams.append(x)
    out = kept(norm_one_plus(x, w["final.norm"], eps)) @ w["head"].t() * float(cfg["logit_scale"])
    return out, streams


def logits(cfg, w, ids):
    return forward(cfg, w, ids)[0]
