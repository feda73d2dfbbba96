"""``Darotar``: a decoder whose layers are listed one by one in config.json. A layer adds the RMS norm of a sublayer's
OUTPUT to the stream, times ``residual_mult``: ``x += m * norm1(mixer(x))``, then ``x += m * norm2(ff(x))``; the sublayers
read the stream itself. Mixers:

* ``attention``: softmax attention with grouped key/value heads whose values are the projected keys (no value matrix),
  rotation of interleaved pairs with linearly scaled positions, a unit RMS norm of every q and k head after the
  rotation, and a sliding window;
* ``latent_attention``: attention through a latent (queries through a latent of their own), half-split rotated pairs,
  a learned sink in the softmax's denominator, a sigmoid gate on the concatenated heads, causal. With ``kv_from`` the
  layer reads the cached rows of an earlier latent layer and has no ``dkv`` tensors.

The feed-forward is a mixture of small gated experts (sigmoid router, the ``top`` largest scores, the score multiplies
the expert's input) or absent. The head is a matrix of its own.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``layers``: a list of ``{"type",
"mixer": {...}, "mlp": {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}} | null}``. Mixer keys:
``attention``: ``heads kv_heads dim vdim scale rot.{dims, base, scaling.factor}`` and optionally ``mask.size``;
``latent_attention``: ``heads dim rot_dim vdim q_rank kv_rank scale rot.{dims, base}``, optionally ``mask.size`` and
``kv_from``.

Tensor names: ``embed``, ``head``, ``final.norm``, per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.<name>``,
``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{gate, up, down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Tuple

from ..config.model_config import ConfigError, ModelConfig
from ..parts.embedding import LinearHead, TokenEmbedding
from ..parts.feedforward import RoutedExperts
from ..parts.flex_attention import FlexAttention
from ..parts.latent_attention import LatentAttention
from ..parts.norm import RMSNorm
from ..parts.position import FrequencyRotary
from ..parts.spec import LayerSpec, ModelPlan, ScheduleEntry
from ..registry import register_architecture

_MIXERS = ("attention", "latent_attention")
# Positions are turned into angles in 32-bit floats, which hold every integer up to 2^24.
_MAX_POSITIONS = 1 << 24


def _int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
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


def _window(m: Mapping[str, Any], where: str) -> int:
    """``mask.size`` of a mixer, 0 without a mask (every earlier position is seen)."""
    if m.get("mask") is None:
        return 0
    return _int(_obj(m, "mask", where), "size", where + ".mask")


def _check_rot(m: Mapping[str, Any], where: str, width: int, exact: bool) -> None:
    rot = _obj(m, "rot", where)
    dims = _int(rot, "dims", where + ".rot")
    if dims % 2 or dims > width or (exact and dims != width):
        raise ConfigError(f"config.json: {where}.rot.dims must be even and {'equal to rot_dim' if exact else 'at most dim'}")
    _num(rot, "base", where + ".rot")
    if rot.get("scaling") is not None:
        _num(_obj(rot, "scaling", where + ".rot"), "factor", where + ".rot.scaling")


@dataclass(frozen=True)
class DarotarConfig(ModelConfig):
    layers: Tuple[dict, ...] = ()
    norm_eps: float = 1e-6
    residual_mult: float = 1.0

    @classmethod
    def from_json_dict(cls, d: Mapping[str, Any]) -> "DarotarConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        eps = _num(_obj(d, "norm", "config"), "eps", "norm")
        mult = _num(d, "residual_mult", "config", positive=False) if "residual_mult" in d else 1.0
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type must be one of {_MIXERS}")
            m = _obj(layer, "mixer", where)
            where += ".mixer"
            _num(m, "scale", where)
            _window(m, where)
            if layer["type"] == "attention":
                heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
                if heads % kv:
                    raise ConfigError(f"config.json: {where}.heads must be a multiple of kv_heads")
                dim = _int(m, "dim", where)
                if int(m.get("vdim", dim)) != dim:
                    raise ConfigError(f"config.json: {where}.vdim must equal dim: the values are the projected keys")
                _check_rot(m, where, dim, exact=False)
            else:
                for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
                    _int(m, k, where)
                _check_rot(m, where, m["rot_dim"], exact=True)
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < i):
                        raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer")
                    o = layers[src]
                    if o.get("type") != "latent_attention" or o["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}.kv_from names a layer that caches no latent of its own")
                    if any(o["mixer"].get(k) != m.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                        raise ConfigError(f"config.json: {where} and layer {src} must agree in kv_rank, rot_dim and rot")
            mlp = layer.get("mlp")
            if mlp is not None:
                where = f"layers[{i}].mlp"
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    raise ConfigError(f"config.json: {where} must be null or of kind 'moe'")
                _int(_obj(mlp, "expert", where), "ff", where + ".expert")
                router = _obj(mlp, "router", where)
                if _int(router, "top", where + ".router") > _int(router, "experts", where + ".router"):
                    raise ConfigError(f"config.json: {where}.router.top must be at most experts")
        eos = d.get("eos_token_id")
        return cls(architecture=str(d.get("architecture") or "Darotar"), model_type="darotar",
                   vocab_size=_int(d, "vocab", "config"), hidden_size=_int(d, "width", "config"),
                   num_hidden_layers=len(layers), max_position_embeddings=_MAX_POSITIONS, tie_word_embeddings=False,
                   eos_token_id=int(eos) if isinstance(eos, int) and not isinstance(eos, bool) else -1,
                   layers=tuple(layers), norm_eps=eps, residual_mult=mult)

    def to_json_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
             "layers": [dict(layer) for layer in self.layers]}
        if self.eos_token_id >= 0:
            d["eos_token_id"] = self.eos_token_id
        return d


def _rotary_name(rot: Mapping[str, Any]) -> str:
    sc = rot.get("scaling") or {}
    return "rot:" + ",".join(str(x) for x in (rot["dims"], rot["base"], sc.get("factor")))


def darotar_plan(cfg: DarotarConfig) -> ModelPlan:
    h, eps = cfg.hidden_size, cfg.norm_eps
    positions: Dict[str, Any] = {}
    # A latent that later layers read stays cached as long as the widest window among its readers (0: all of it).
    keep: Dict[int, int] = {}
    for i, layer in enumerate(cfg.layers):
        if layer["type"] == "latent_attention":
            m = layer["mixer"]
            owner = i if m.get("kv_from") is None else int(m["kv_from"])
            w = _window(m, f"layers[{i}].mixer")
            keep[owner] = 0 if (w == 0 or keep.get(owner, -1) == 0) else max(keep.get(owner, 0), w)
    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer["mixer"]
        window = _window(m, f"layers[{i}].mixer")
        reads = None
        if layer["type"] == "attention":
            rot = m["rot"]
            factor = float((rot.get("scaling") or {}).get("factor", 1.0))
            mixer = FlexAttention.spec(f"{p}.mix", h, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["dim"]),
                                       float(m["scale"]), eps, rot=(int(rot["dims"]), float(rot["base"])), window=window,
                                       rot_layout="interleaved", rot_factor=factor, unit_norm_after_rot=True,
                                       values_from_keys=True)
        else:
            rot = m["rot"]
            name = _rotary_name(rot)
            positions.setdefault(name, FrequencyRotary.spec(int(rot["dims"]), float(rot["base"]), rot.get("scaling"), layout="half"))
            reads = m.get("kv_from")
            owner = i if reads is None else int(reads)
            mixer = LatentAttention.spec(f"{p}.mix", h, int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]),
                                         int(m["q_rank"]), int(m["kv_rank"]), float(m["scale"]), window, keep[owner], eps, name,
                                         owns_kv=reads is None, sink=True, out_gate=True)
        parts = {"mixer": mixer, "mixer_norm": RMSNorm.spec(h, eps, f"{p}.norm1")}
        mlp = layer.get("mlp")
        if mlp is not None:
            parts["ffn"] = RoutedExperts.spec(f"{p}.mlp", h, int(mlp["expert"]["ff"]), int(mlp["router"]["experts"]),
                                              int(mlp["router"]["top"]))
            parts["ffn_norm"] = RMSNorm.spec(h, eps, f"{p}.norm2")
        layers.append(LayerSpec("output_norm", parts, {"mult": cfg.residual_mult}))
        schedule.append(ScheduleEntry(i, reads_cache_of=None if reads is None else int(reads)))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=TokenEmbedding.spec("embed", cfg.vocab_size, h), positions=positions, layers=layers, schedule=schedule,
        final_norm=RMSNorm.spec(h, eps, "final.norm"), lm_head=LinearHead.spec("head", cfg.vocab_size, h),
        eos_token_id=cfg.eos_token_id,
        # a layer without a feed-forward has no use for a second norm, should a checkpoint hold one
        ignored_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if layer.get("mlp") is None))


register_architecture("Darotar", DarotarConfig, darotar_plan)
