"""Small Dusilorn configurations and weights for the tests: sizes that differ from layer to layer, include 1 and values that
are no powers of two, and weights large enough that every mechanism moves the logits."""
import json
import os

import torch

from darotar_util import assert_within_rounding, mixed_schedule, tokens  # noqa: F401  (helpers that know no design)


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def chunked(heads, kv_heads, dim, vdim, size, cap=25.0, v_mix=True, scale=None, mlp=None):
    """A layer of type ``attention``: whole-projection q/k norm, chunked mask, sink."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size}, "softcap": cap, "v_mix": v_mix,
         "scale": scale if scale is not None else 1.5 / dim ** 0.5}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def windowed(heads, kv_heads, dim, vdim, size, rot_dims, base, cap=25.0, v_mix=True, scale=None, mlp=None):
    """A layer of type ``attention_2``: rotated q and k, sliding window."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size}, "softcap": cap, "v_mix": v_mix,
         "rot": {"dims": rot_dims, "base": base}, "scale": scale if scale is not None else dim ** -0.5}
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def model(vocab, width, layers, eps=1e-5, emb=3.0, logit=0.5):
    return {"architecture": "Dusilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb},
            "logit_scale": logit, "layers": layers}


# The first layer does not blend (v_mix starts at the second); a layer without v_mix between two that have it; one kv head;
# a window of 5 and a chunk of 3 (no multiples of a page); every kind of feed-forward incl. none; all router outputs chosen in
# one layer; identity outputs; a shared expert wider and one narrower than the experts.
CFG_A = model(131, 64, [
    windowed(4, 2, 12, 6, 5, 8, 500.0, v_mix=False, mlp=dense(40)),
    chunked(3, 1, 8, 10, 3, cap=5.0, mlp=moe(5, 2, 24, identity=2, shared=40)),
    windowed(2, 2, 16, 4, 300, 16, 100.0, cap=0.0, v_mix=False, mlp=None),
    chunked(5, 5, 4, 2, 7, mlp=moe(3, 3, 16)),
    windowed(2, 1, 6, 10, 9, 2, 1e4, mlp=moe(4, 1, 8, identity=1, shared=8)),
], eps=1e-6, emb=2.0, logit=1.5)
# Sizes that the tensor-core kernels take (heads of 16..64, widths in multiples of 8), a chunk of 17 and a window of 33.
CFG_B = model(77, 96, [
    chunked(4, 2, 32, 24, 17, mlp=moe(7, 2, 40, identity=1, shared=24)),
    windowed(6, 3, 32, 16, 33, 16, 30000.0, mlp=dense(64)),
    windowed(2, 2, 16, 24, 8, 16, 1000.0, cap=30.0, mlp=moe(4, 1, 32)),
    chunked(8, 1, 16, 48, 64, mlp=moe(2, 2, 64, identity=3)),
], emb=4.0, logit=2.5)
# Larger: pages of 16 and prompts of a few hundred tokens cross many pages, chunks and windows; key tiles of 64.
CFG_C = model(300, 128, [
    windowed(8, 2, 64, 32, 70, 32, 1e6, mlp=dense(192)),
    chunked(8, 2, 48, 32, 48, mlp=moe(8, 2, 48, identity=2, shared=96)),
    windowed(4, 4, 96, 16, 129, 48, 1e4, mlp=moe(6, 3, 32, shared=32)),
    chunked(4, 1, 128, 64, 100, mlp=None),
], emb=6.0, logit=1.0)


# Heads of 64 and 128 with values as wide as keys: in bfloat16 prompt portions take the attention kernel with scores in tensor
# memory (cap, chunk, window and sink in its softmax warps), decoded tokens the mma.sync kernel with split keys.
CFG_D = model(200, 128, [
    windowed(4, 2, 64, 64, 70, 32, 1e6, mlp=dense(96)),
    chunked(4, 2, 64, 64, 48, mlp=moe(6, 2, 32, identity=1, shared=64)),
    windowed(2, 1, 128, 128, 129, 64, 1e4, cap=50.0, mlp=moe(4, 1, 64)),
    chunked(8, 1, 128, 128, 100, mlp=None),
], emb=5.0, logit=1.0)


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
        elif ts.init == "bias":             # gains stored around zero, corrections of a router
            x = (0.02 if ts.name.endswith(".correction") else 0.1) * x
        elif ts.init == "unit":             # sinks
            x = 0.7 * x
        elif ts.init == "mix01":            # blend factors
            x = torch.rand(ts.shape, generator=g)
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
    """A change of the random tensors after which rounding cannot change the routing: the first ``classes`` channels of the
    stream hold a one-hot class of the token (token id modulo ``classes``), no branch ever adds to them (the gains of the
    norms on the branches' outputs are zero there, i.e. stored as -1), and the routers read nothing else. A router logit
    is then one product whose second factor is a multiple of a quarter, an expert's logits lie far apart, and the
    corrections (multiples of 0.03 in a random order) decide among scores that rounding moves by far less."""
    def change(t):
        emb = t["embed"]
        emb[:, :classes] = 0
        emb[torch.arange(emb.shape[0]), torch.arange(emb.shape[0]) % classes] = 2.0
        for i, layer in enumerate(cfg["layers"]):
            t[f"l{i}.norm1b"][:classes] = -1.0
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            t[f"l{i}.norm2b"][:classes] = -1.0
            if mlp["kind"] != "moe":
                continue
            t[f"l{i}.norm2"][:classes] = 0.0        # the class channels reach the router with the gain 1
            r = t[f"l{i}.mlp.router"]
            r[:, classes:] = 0
            g = torch.Generator().manual_seed(100 + i)
            for c in range(classes):
                order = torch.randperm(r.shape[0], generator=g).float()
                r[:, c] = ((order - (r.shape[0] - 1) / 2) / 4).to(r.dtype)
            t[f"l{i}.mlp.correction"].copy_((torch.randperm(r.shape[0], generator=g).float() * 0.03).to(r.dtype))
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
    import plain_dusilorn as plain
    cfg, w = read_model(folder)
    if stored_as is None:
        return plain.logits(cfg, w, list(ids))
    with plain.stored_as(stored_as):
        return plain.logits(cfg, w, list(ids))


def random_config(rng, small=True):
    """A configuration with random layer order, sizes and constants. ``small``: odd sizes, ones, sizes no kernel's fast path
    takes; else sizes of a small real model (widths of 128 to 384, heads of 32 to 128, 4 to 16 experts)."""
    width = rng.choice([40, 64, 72, 100, 136] if small else [128, 192, 256, 320, 384])
    kv = rng.choice([1, 2, 3] if small else [1, 2, 4])
    vdim = rng.choice([3, 4, 8, 10, 24] if small else [16, 32, 48, 64, 128])
    layers = []
    for _ in range(rng.randint(2, 6)):
        kind = rng.choice([None, "dense", "moe", "moe", "moe"])
        if kind == "dense":
            mlp = dense(rng.choice([8, 24, 50] if small else [64, 128, 256]))
        elif kind == "moe":
            experts = rng.choice([1, 2, 3, 5, 8, 33] if small else [4, 8, 10, 16])
            identity = rng.choice([0, 0, 1, 2, 3])
            mlp = moe(experts, rng.choice([t for t in (1, 2, 3, 4) if t <= experts + identity]), rng.choice([8, 24, 40, 66] if small else [32, 64, 128]),
                      identity=identity, shared=rng.choice([None, 8, 24, 40] if small else [None, 64, 128]))
        else:
            mlp = None
        v_mix = rng.random() < 0.75
        # layers that blend share one shape of values; the others choose their own
        g, vd = (kv, vdim) if v_mix else (rng.choice([1, 2]), rng.choice([4, 8, 16] if small else [16, 32]))
        heads = g * rng.choice([1, 2, 4])
        dim = rng.choice([4, 8, 12, 16, 24, 40, 64, 136] if small else [32, 64, 96, 128])
        cap = rng.choice([0.0, 5.0, 25.0, 50.0])
        size = rng.choice([1, 2, 5, 16, 17, 31, 32, 33, 64, 100] if small else [16, 48, 64, 96, 100, 130])
        if rng.random() < 0.5:
            layers.append(chunked(heads, g, dim, vd, size, cap=cap, v_mix=v_mix, scale=rng.choice([None, 0.2]), mlp=mlp))
        else:
            rot = rng.choice([d for d in (2, 4, 8, 16, 32, dim) if d <= dim and d % 2 == 0])
            layers.append(windowed(heads, g, dim, vd, size, rot, rng.choice([100.0, 1e4, 1e6]), cap=cap, v_mix=v_mix,
                                   scale=rng.choice([None, 0.2]), mlp=mlp))
    return model(rng.choice([50, 131, 257, 1000]), width, layers, eps=rng.choice([1e-6, 1e-5, 1e-4]), emb=rng.choice([1.0, 2.0, 7.0]),
                 logit=rng.choice([0.5, 1.0, 3.0]))
