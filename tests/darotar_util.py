"""Small Darotar configurations and weights for the tests: sizes that differ from layer to layer, include 1 and values
that are no powers of two, and weights large enough that every mechanism moves the logits."""
import json
import os

import torch


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attention(heads, kv_heads, dim, rot_dims, base, factor=None, window=None, scale=None, mlp=None):
    rot = {"dims": rot_dims, "base": base}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "rot": rot, "scale": scale if scale is not None else 3.0 / dim}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, base, scale=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "rot": {"dims": rot_dim, "base": base}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


# A rotation of part of a head; a window of 5 (no multiple of a page); one kv head; a layer without a feed-forward; a
# latent layer read by a later one with other head counts and widths; every expert used by every token in one layer.
CFG_A = {"architecture": "Darotar", "vocab": 131, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.7, "layers": [
    attention(4, 2, 12, 8, 500.0, factor=2.0, window=5, mlp=moe(5, 2, 24)),
    latent(3, 8, 4, 6, 10, 12, 10000.0, mlp=None),
    latent(2, 6, 4, 10, 7, 12, 10000.0, kv_from=1, mlp=moe(3, 3, 16)),
    attention(3, 1, 16, 16, 100.0, factor=1.5, window=300, mlp=moe(6, 1, 20)),
    latent(1, 4, 2, 4, 5, 6, 50.0, mlp=moe(4, 2, 8)),
]}
# Sizes that the tensor-core kernels take (heads of 16 and 32, latents of 32 + 8), a residual factor of 1, a window of 17, an
# attention layer without a window, a latent layer first, read by the last layer.
CFG_B = {"architecture": "Darotar", "vocab": 77, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 1.0, "layers": [
    latent(4, 16, 8, 16, 24, 32, 1e6, mlp=moe(4, 1, 32)),
    attention(6, 3, 32, 32, 30000.0, factor=8.0, window=17, mlp=moe(7, 2, 40)),
    attention(2, 2, 16, 4, 1000.0, mlp=None),
    latent(2, 8, 8, 24, 16, 32, 1e6, kv_from=0, mlp=moe(2, 1, 64)),
]}
# Larger: pages of 16 and prompts of a few hundred tokens cross many pages and several windows; key tiles of 64.
CFG_C = {"architecture": "Darotar", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.6, "layers": [
    attention(8, 2, 64, 64, 10000.0, factor=4.0, window=70, mlp=moe(8, 2, 48)),
    latent(4, 32, 16, 24, 40, 48, 1e5, mlp=moe(8, 2, 48)),
    latent(8, 16, 16, 16, 32, 48, 1e5, kv_from=1, mlp=None),
    attention(4, 4, 32, 16, 10000.0, factor=1.0, window=129, mlp=moe(3, 1, 96)),
]}


def make_weights(plan, seed):
    """bfloat16 tensors for every tensor of ``plan``: matrices N(0, 1.2^2 / fan_in), so activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for ts in plan.tensor_specs():
        x = torch.randn(ts.shape, generator=g, dtype=torch.float32)
        if ts.init == "matrix":
            x = x * (1.2 / ts.shape[-1] ** 0.5)
        elif ts.init == "embedding":
            x = x * (1.0 if ts.name == "embed" else 1.2 / ts.shape[-1] ** 0.5)
        elif ts.init == "gain":
            x = 1.0 + 0.1 * x
        elif ts.init == "bias":
            x = 0.1 * x
        elif ts.init == "unit":
            x = 0.7 * x
        else:
            raise ValueError(ts.init)
        out[ts.name] = x.to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, weights=None):
    """A model folder of ``cfg``. ``weights``: a function that changes the random tensors in place before they are written."""
    from nanoinfer_b200.registry import config_from_json_dict, plan_for
    from nanoinfer_b200.weights.safetensors_io import save_safetensors
    plan = plan_for(config_from_json_dict(cfg))
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = make_weights(plan, seed)
    if weights is not None:
        weights(tensors)
    save_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder


def pin_routing(cfg, classes=8):
    """A change of the random tensors after which the routing is the same in every precision: the first ``classes``
    channels of the stream hold a one-hot class of the token (token id modulo ``classes``), no branch ever adds to them
    (the gains of every norm are zero there), and the routers read nothing else. Every router logit is then one product
    of two numbers that bfloat16 holds, equal in 16, 32 and 64 bits, and an expert's logits lie a sixteenth apart, so a
    comparison of bfloat16 logits with the plain implementation cannot rest on a close call or a tie between two experts (in 32-bit the tests keep the random routers).
    The experts still read the whole stream, each token scaled by its score."""
    def change(t):
        emb = t["embed"]
        emb[:, :classes] = 0
        emb[torch.arange(emb.shape[0]), torch.arange(emb.shape[0]) % classes] = 2.0
        for i, layer in enumerate(cfg["layers"]):
            t[f"l{i}.norm1"][:classes] = 0
            if layer.get("mlp") is not None:
                t[f"l{i}.norm2"][:classes] = 0
                r = t[f"l{i}.mlp.router"]
                r[:, classes:] = 0
                # per class the experts in a random order, a sixteenth apart: numbers that bfloat16 holds, no two equal
                g = torch.Generator().manual_seed(100 + i)
                for c in range(classes):
                    order = torch.randperm(r.shape[0], generator=g).float()
                    r[:, c] = ((order - (r.shape[0] - 1) / 2) / 16).to(r.dtype)
    return change


def read_model(folder):
    from nanoinfer_b200.weights.safetensors_io import SafetensorsFile
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    sf = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return cfg, {n: sf.tensor(n) for n in sf.names()}


def plain_logits(folder, ids, stored_as=None):
    """Float64 logits [len(ids), vocab] of the plain implementation; with ``stored_as`` every tensor that an engine keeps
    between two operations is rounded to that type on the way."""
    import plain_darotar as plain
    cfg, w = read_model(folder)
    if stored_as is None:
        return plain.logits(cfg, w, list(ids))
    with plain.stored_as(stored_as):
        return plain.logits(cfg, w, list(ids))


def assert_within_rounding(got, ref, rounded, what="", factor=3.0):
    """``got`` (an engine in bfloat16) against ``ref`` (the plain implementation in float64), judged by what rounding alone
    does to this model: ``rounded`` is the plain implementation with its stored tensors rounded to bfloat16. Root mean
    square and largest error may be ``factor`` times those of ``rounded``; an error that a wrong key, window or state
    makes is of the order of the logits themselves."""
    got, ref, rounded = got.detach().double().cpu(), ref.double(), rounded.double()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert not torch.isnan(got).any() and not torch.isinf(got).any(), f"{what}: NaN or inf in the result"
    err, noise = (got - ref).abs(), (rounded - ref).abs()
    e_rms, n_rms = err.pow(2).mean().sqrt().item(), noise.pow(2).mean().sqrt().item()
    assert n_rms < 0.05 * ref.pow(2).mean().sqrt().item(), f"{what}: rounding alone moves this model's logits too far to judge by"
    assert e_rms <= factor * n_rms, f"{what}: rms err {e_rms:.3e} > {factor} x {n_rms:.3e}"
    assert err.max().item() <= factor * noise.max().item(), f"{what}: max err {err.max().item():.3e} > {factor} x {noise.max().item():.3e}"


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def random_config(rng):
    """A configuration with random layer order, sizes (odd ones, ones, sizes no kernel's fast path takes) and constants."""
    width = rng.choice([40, 64, 72, 100, 128, 192, 258])
    layers, owners = [], []
    for i in range(rng.randint(2, 7)):
        mlp = rng.choice([None, "moe", "moe", "moe"])
        if mlp is not None:
            experts = rng.choice([1, 2, 3, 5, 8, 33])
            mlp = moe(experts, rng.choice([t for t in (1, 2, 3, 4) if t <= experts]), rng.choice([8, 24, 40, 64, 130]))
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([4, 8, 12, 16, 24, 40, 64, 96, 136])
            rot = rng.choice([d for d in (2, 4, 8, 16, 32, dim) if d <= dim])
            layers.append(attention(kv * rng.choice([1, 2, 4]), kv, dim, rot, rng.choice([100.0, 10000.0, 1e6]),
                                    factor=rng.choice([None, 1.0, 2.0, 4.0, 32.0]), window=rng.choice([None, 1, 2, 5, 16, 17, 31, 32, 33, 64, 100]),
                                    scale=rng.choice([None, 0.2]), mlp=mlp))
            continue
        src = rng.choice(owners) if owners and rng.random() < 0.4 else None
        if src is None:
            rank, rdim, base = rng.choice([4, 8, 24, 32, 50, 64, 120]), rng.choice([2, 4, 8, 16, 30]), rng.choice([100.0, 10000.0, 1e6])
            owners.append(i)
        else:
            o = layers[src]["mixer"]
            rank, rdim, base = o["kv_rank"], o["rot_dim"], o["rot"]["base"]
        layers.append(latent(rng.choice([1, 2, 3, 5, 8]), rng.choice([4, 8, 12, 16, 32, 40]), rdim, rng.choice([3, 8, 16, 24, 64]),
                             rng.choice([5, 16, 24, 64]), rank, base, scale=rng.choice([None, 0.15]), kv_from=src, mlp=mlp))
    return {"architecture": "Darotar", "vocab": rng.choice([50, 131, 257, 1000]), "width": width,
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-4])}, "residual_mult": rng.choice([0.25, 0.5, 1.0, 1.5]), "layers": layers}


def larger_config(rng):
    """A configuration at sizes of a small real model: widths of 128 to 384, heads of 32 to 128, 4 to 16 experts."""
    width = rng.choice([128, 192, 256, 320, 384])
    layers, owners = [], []
    for i in range(rng.randint(3, 8)):
        e = rng.choice([4, 8, 10, 16])
        mlp = rng.choice([None, 1, 1, 1]) and moe(e, rng.choice([1, 2, 3]), rng.choice([32, 64, 128]))
        if rng.random() < 0.45:
            kv = rng.choice([1, 2, 4]); dim = rng.choice([32, 64, 96, 128])
            layers.append(attention(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim, dim // 2, 16]), rng.choice([1e4, 2e4, 1e6]),
                                    factor=rng.choice([None, 2.0, 4.0, 8.0]), window=rng.choice([16, 48, 64, 96, 100, 128]), scale=rng.choice([None, 0.15]), mlp=mlp))
            continue
        src = rng.choice(owners) if owners and rng.random() < 0.45 else None
        if src is None:
            rank, rdim, base = rng.choice([32, 64, 96, 128]), rng.choice([8, 16, 32, 64]), rng.choice([1e4, 1e6])
            owners.append(i)
        else:
            o = layers[src]["mixer"]; rank, rdim, base = o["kv_rank"], o["rot_dim"], o["rot"]["base"]
        layers.append(latent(rng.choice([2, 4, 8, 16]), rng.choice([16, 32, 64]), rdim, rng.choice([16, 32, 64]), rng.choice([48, 72, 128]), rank, base,
                             scale=rng.choice([None, 0.14]), kv_from=src, mlp=mlp))
    return {"architecture": "Darotar", "vocab": rng.choice([500, 1000]), "width": width, "norm": {"eps": 1e-6},
            "residual_mult": rng.choice([0.5, 0.7, 1.0]), "layers": layers}


def mixed_schedule(rng, lens):
    """Steps of [(request, count)]: at most four live, each request first in portions, its last tokens one by one."""
    pending, live, at, steps = list(range(len(lens))), [], {}, []
    while pending or live:
        while pending and len(live) < 4 and (not live or rng.random() < 0.6):
            r = pending.pop(0); live.append(r); at[r] = 0
        step = []
        for r in list(live):
            if rng.random() < 0.15 and len(live) > 1:
                continue        # left out of this step
            left = lens[r] - at[r]
            c = 1 if left <= 20 else min(left - 20, rng.choice([2, 3, 7, 16, 33, 64, 100]))
            step.append((r, c)); at[r] += c
            if at[r] == lens[r]:
                live.remove(r)
        if step:
            steps.append(step)
    return steps


