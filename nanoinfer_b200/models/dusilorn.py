"""``Dusilorn``: a decoder whose layers are listed one by one in config.json. Every sublayer stands between two norms
(gains stored around zero): ``x += norm1b(mixer(norm1(x)))``, then ``x += norm2b(ff(norm2(x)))``. The embedding is multiplied
by ``embedding.scale``, the logits by ``logit_scale``; the head is a matrix of its own. Mixers, both softmax attention with
grouped key/value heads, keys and values of different widths, soft-capped scores and values that may be blended with those
of the first layer that says ``v_mix``:

* ``attention``: q and k normed over the whole projection (plain gains of the projections' sizes), no rotation, a chunked
  mask (a position sees the earlier positions of its own block of ``mask.size``, counted from the sequence's start) and a
  learned sink per head in the softmax's denominator;
* ``attention_2``: rotation of the first ``rot.dims`` elements of every q and k head (element i paired with i + dims/2),
  a sliding window of ``mask.size`` positions, ordinary softmax.

The feed-forward is absent, dense (SwiGLU) or a mixture of experts ``W_down relu(W_up h)^2``: softmax scores over all router
outputs, a stored correction added for the choice only, the chosen scores renormalized, the weight on the expert's output;
the last ``router.identity`` router outputs stand for the input itself; an optional shared expert of the same form runs for
every token, times ``sigmoid(W_sg h)``.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_scale``, ``layers``: a list of
``{"type", "mixer": {heads kv_heads dim vdim scale softcap v_mix mask.size rot.{dims, base}}, "mlp": null | {"kind": "dense",
"ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "identity", "top"}, "shared": {"ff"}}}``.

Tensor names: ``embed``, ``head``, ``final.norm``, per layer i ``l<i>.norm1 norm1b norm2 norm2b``, ``l<i>.mix.{q k v o}``,
``l<i>.mix.{q.norm k.norm sink}`` (``attention``), ``l<i>.mix.vmix``, ``l<i>.mlp.{gate up down}`` (dense) or
``l<i>.mlp.{router correction}``, ``l<i>.mlp.e<j>.{up down}``, ``l<i>.mlp.shared.{up down sg}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig
from ..parts.embedding import LinearHead, TokenEmbedding
from ..parts.feedforward import RoutedExperts, SwiGLU
from ..parts.flex_attention import FlexAttention
from ..parts.norm import RMSNorm
from ..parts.spec import LayerSpec, ModelPlan, ScheduleEntry
from ..registry import register_architecture

_MIXERS = ("attention", "attention_2")
# Positions are turned into angles in 32-bit floats, which hold every integer up to 2^24.
_MAX_POSITIONS = 1 << 24


def _int(d: Mapping[str, Any], key: str, where: str, least: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"config.json: {where}.{key} must be an integer of at least {least}, got {v!r}")
    return v


def _num(d: Mapping[str, Any], key: str, where: str, positive: bool = True) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"config.json: {where}.{key} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


def _obj(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} must be an object")
    return v


def _mask(m: Mapping[str, Any], where: str) -> int:
    """``mask.size`` of a mixer, 0 without a mask (every earlier position is seen)."""
    return 0 if m.get("mask") is None else _int(_obj(m, "mask", where), "size", where + ".mask")


@dataclass(frozen=True)
class DusilornConfig(ModelConfig):
    layers: Tuple[dict, ...] = ()
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_scale: float = 1.0

    @classmethod
    def from_json_dict(cls, d: Mapping[str, Any]) -> "DusilornConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        eps = _num(_obj(d, "norm", "config"), "eps", "norm")
        emb_scale = 1.0 if d.get("embedding") is None else _num(_obj(d, "embedding", "config"), "scale", "embedding", positive=False)
        logit_scale = 1.0 if d.get("logit_scale") is None else _num(d, "logit_scale", "config", positive=False)
        shared_values: Optional[int] = None
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type must be one of {_MIXERS}")
            m = _obj(layer, "mixer", where)
            where += ".mixer"
            heads, kv, dim = _int(m, "heads", where), _int(m, "kv_heads", where), _int(m, "dim", where)
            if heads % kv:
                raise ConfigError(f"config.json: {where}.heads must be a multiple of kv_heads")
            vdim = _int(m, "vdim", where) if "vdim" in m else dim
            _num(m, "scale", where)
            if m.get("softcap") is not None and _num(m, "softcap", where, positive=False) < 0:      # 0: the scores are not capped
                raise ConfigError(f"config.json: {where}.softcap must not be negative")
            _mask(m, where)
            if layer["type"] == "attention_2":
                rot = _obj(m, "rot", where)
                dims = _int(rot, "dims", where + ".rot")
                if dims % 2 or dims > dim:
                    raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim")
                _num(rot, "base", where + ".rot")
            if m.get("v_mix"):
                if shared_values is not None and shared_values != kv * vdim:
                    raise ConfigError(f"config.json: {where}: layers that blend their values need kv_heads * vdim = {shared_values}")
                shared_values = kv * vdim
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            where = f"layers[{i}].mlp"
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"config.json: {where} must be null or of kind 'dense' or 'moe'")
            if mlp["kind"] == "dense":
                _int(mlp, "ff", where)
                continue
            _int(_obj(mlp, "expert", where), "ff", where + ".expert")
            router = _obj(mlp, "router", where)
            experts = _int(router, "experts", where + ".router")
            identity = _int(router, "identity", where + ".router", least=0) if router.get("identity") is not None else 0
            if not (1 <= _int(router, "top", where + ".router") <= experts + identity):
                raise ConfigError(f"config.json: {where}.router.top must be at most experts + identity")
            if mlp.get("shared") is not None:
                _int(_obj(mlp, "shared", where), "ff", where + ".shared")
        eos = d.get("eos_token_id")
        return cls(architecture=str(d.get("architecture") or "Dusilorn"), model_type="dusilorn",
                   vocab_size=_int(d, "vocab", "config"), hidden_size=_int(d, "width", "config"),
                   num_hidden_layers=len(layers), max_position_embeddings=_MAX_POSITIONS, tie_word_embeddings=False,
                   eos_token_id=int(eos) if isinstance(eos, int) and not isinstance(eos, bool) else -1,
                   layers=tuple(layers), norm_eps=eps, embedding_scale=emb_scale, logit_scale=logit_scale)

    def to_json_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
             "layers": [dict(layer) for layer in self.layers]}
        if self.eos_token_id >= 0:
            d["eos_token_id"] = self.eos_token_id
        return d


def _feed_forward(prefix: str, hidden: int, mlp: Mapping[str, Any]):
    if mlp["kind"] == "dense":
        return SwiGLU.spec(prefix, hidden, int(mlp["ff"]), names=("gate", "up", "down"))
    router = mlp["router"]
    shared = mlp.get("shared")
    return RoutedExperts.spec(prefix, hidden, int(mlp["expert"]["ff"]), int(router["experts"]), int(router["top"]),
                              score="softmax", correction=True, renormalize=True, weight_on="output", gated=False,
                              identity=int(router.get("identity") or 0), shared=0 if shared is None else int(shared["ff"]))


def dusilorn_plan(cfg: DusilornConfig) -> ModelPlan:
    h, eps = cfg.hidden_size, cfg.norm_eps
    layers: List[LayerSpec] = []
    ignored: List[str] = []
    first_mix: Optional[int] = next((i for i, layer in enumerate(cfg.layers) if layer["mixer"].get("v_mix")), None)
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer["mixer"]
        size = _mask(m, f"layers[{i}].mixer")
        v_mix = None if not m.get("v_mix") else ("first" if i == first_mix else "blend")
        if v_mix != "blend":
            ignored.append(f"{p}.mix.vmix")       # a checkpoint may hold the number for layers that never use it
        common = dict(softcap=float(m.get("softcap") or 0.0), v_mix=v_mix)
        dims = (h, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])), float(m["scale"]), eps)
        if layer["type"] == "attention":
            mixer = FlexAttention.spec(f"{p}.mix", *dims, qk_norm="whole", chunk=size, sink=True, **common)
        else:
            rot = m["rot"]
            mixer = FlexAttention.spec(f"{p}.mix", *dims, rot=(int(rot["dims"]), float(rot["base"])), window=size, **common)
        parts = {"mixer_norm": RMSNorm.spec(h, eps, f"{p}.norm1", gain_offset=1.0), "mixer": mixer,
                 "mixer_out_norm": RMSNorm.spec(h, eps, f"{p}.norm1b", gain_offset=1.0)}
        if layer.get("mlp") is not None:
            parts["ffn_norm"] = RMSNorm.spec(h, eps, f"{p}.norm2", gain_offset=1.0)
            parts["ffn"] = _feed_forward(f"{p}.mlp", h, layer["mlp"])
            parts["ffn_out_norm"] = RMSNorm.spec(h, eps, f"{p}.norm2b", gain_offset=1.0)
        else:
            ignored += [f"{p}.norm2", f"{p}.norm2b"]        # no feed-forward: no use for its norms, should a checkpoint hold them
        layers.append(LayerSpec("sandwich_norm", parts))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=TokenEmbedding.spec("embed", cfg.vocab_size, h, cfg.embedding_scale), positions={}, layers=layers,
        schedule=[ScheduleEntry(i) for i in range(len(layers))],
        # the factor on the logits rides on the last norm's gain: head(s * n) = s * head(n)
        final_norm=RMSNorm.spec(h, eps, "final.norm", gain_offset=1.0, gain_scale=cfg.logit_scale),
        lm_head=LinearHead.spec("head", cfg.vocab_size, h), eos_token_id=cfg.eos_token_id, ignored_tensors=tuple(ignored))


register_architecture("Dusilorn", DusilornConfig, dusilorn_plan)
