"""``Vafozen``: a decoder whose layers are listed one by one in config.json. Every layer is a parallel block with ONE
norm (gain stored around zero) whose output both the mixer and the SwiGLU feed-forward read. Mixers:

* ``parallel``: softmax attention (per-head norm of q and k, a bias by distance, a chunked mask) beside gated linear
  attention;
* ``parallel_2``: softmax attention (short convolutions on q, k and v, rotation, soft-capped scores, a sigmoid gate on the
  output) beside a time mix with token shift;
* ``mamba2``: a state-space mixer with scalar decays per head.

The two halves of a pair are summed with the factors ``left_scale`` and ``right_scale``. The embedding is multiplied by
``embedding.scale``; the head is a matrix of its own.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``layers``: a list of
``{"type", "mixer": {...}, "mlp": {"kind": "dense", "ff"} | null}``. Keys of a softmax half (``mixer.left``): ``heads kv_heads dim
scale``, optionally ``vdim`` (default ``dim``) and, where the type has them, ``conv``, ``rot.{dims, base}``, ``softcap``, ``mask.size``. Keys of a right half:
``heads dim`` and optionally ``vdim`` (default ``dim``), for ``parallel`` also ``tau``; the inner width of its decay map is
the row count of its ``a1`` / ``w1`` tensor (or ``decay_rank``, which the random-weights mode writes). ``mamba2``: ``heads vdim
state groups norm_groups conv``.

Tensor names: ``embed``, ``head``, ``final.norm``, per layer i ``l<i>.norm1``, ``l<i>.mix.[left.|right.]<name>``,
``l<i>.mlp.{gate, up, down}``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, List, Mapping, Tuple

from ..config.model_config import ConfigError, ModelConfig
from ..parts.embedding import LinearHead, TokenEmbedding
from ..parts.feedforward import SwiGLU
from ..parts.flex_attention import FlexAttention
from ..parts.linear_state import GatedLinearAttention, Mamba2Mixer, ShiftedTimeMix
from ..parts.norm import RMSNorm
from ..parts.side_by_side import SideBySide
from ..parts.spec import LayerSpec, ModelPlan, ScheduleEntry
from ..registry import register_architecture

_TYPES = ("parallel", "parallel_2", "mamba2")
# Positions are turned into angles in 32-bit floats, which hold every integer up to 2^24.
_MAX_POSITIONS = 1 << 24
# The bias by distance of a ``parallel`` layer's softmax half: head h of H has the slope 2^(-8 (h + 1) / H).
_SLOPE_SPAN = 8.0
# Which tensor's row count gives the inner width of a right half's decay map.
_RANK_TENSOR = {"parallel": "a1", "parallel_2": "w1"}


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


def _check_softmax_half(m: Mapping[str, Any], where: str) -> None:
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}.heads must be a multiple of kv_heads")
    dim = _int(m, "dim", where)
    if "vdim" in m:
        _int(m, "vdim", where)
    _num(m, "scale", where)
    if "conv" in m:
        _int(m, "conv", where)
    if "rot" in m:
        rot = _obj(m, "rot", where)
        dims = _int(rot, "dims", where + ".rot")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim")
        _num(rot, "base", where + ".rot")
    if "softcap" in m:
        _num(m, "softcap", where)
    if "mask" in m:
        _int(_obj(m, "mask", where), "size", where + ".mask")


@dataclass(frozen=True)
class VafozenConfig(ModelConfig):
    layers: Tuple[dict, ...] = ()
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0

    @classmethod
    def from_json_dict(cls, d: Mapping[str, Any]) -> "VafozenConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        eps = _num(_obj(d, "norm", "config"), "eps", "norm")
        emb = d.get("embedding")
        scale = 1.0 if emb is None else _num(_obj(d, "embedding", "config"), "scale", "embedding")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in _TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {_TYPES}")
            m = _obj(layer, "mixer", where)
            where += ".mixer"
            if layer["type"] == "mamba2":
                for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv"):
                    _int(m, k, where)
                if m["heads"] % m["groups"] or (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    raise ConfigError(f"config.json: {where}: heads must be a multiple of groups, heads * vdim of norm_groups")
            else:
                _check_softmax_half(_obj(m, "left", where), where + ".left")
                r = _obj(m, "right", where)
                _int(r, "heads", where + ".right")
                _int(r, "dim", where + ".right")
                if "vdim" in r:
                    _int(r, "vdim", where + ".right")
                if "decay_rank" in r:
                    _int(r, "decay_rank", where + ".right")
                if layer["type"] == "parallel":
                    _num(r, "tau", where + ".right")
                _num(m, "left_scale", where, positive=False)
                _num(m, "right_scale", where, positive=False)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: layers[{i}].mlp must be null or of kind 'dense'")
                _int(mlp, "ff", f"layers[{i}].mlp")
        eos = d.get("eos_token_id")
        return cls(architecture=str(d.get("architecture") or "Vafozen"), model_type="vafozen",
                   vocab_size=_int(d, "vocab", "config"), hidden_size=_int(d, "width", "config"),
                   num_hidden_layers=len(layers), max_position_embeddings=_MAX_POSITIONS, tie_word_embeddings=False,
                   eos_token_id=int(eos) if isinstance(eos, int) and not isinstance(eos, bool) else -1,
                   layers=tuple(layers), norm_eps=eps, embedding_scale=scale)

    def with_tensor_shapes(self, shapes: Mapping[str, Any]) -> "VafozenConfig":
        """The inner width of a right half's decay map is the number of rows of its first decay matrix; config.json
        need not state it."""
        layers = []
        for i, layer in enumerate(self.layers):
            name = f"l{i}.mix.right.{_RANK_TENSOR.get(layer['type'], '')}"
            if layer["type"] in _RANK_TENSOR and "decay_rank" not in layer["mixer"]["right"] and name in shapes:
                right = dict(layer["mixer"]["right"], decay_rank=int(tuple(shapes[name])[0]))
                layer = dict(layer, mixer=dict(layer["mixer"], right=right))
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    def to_json_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
             "layers": [dict(layer) for layer in self.layers]}
        if self.eos_token_id >= 0:
            d["eos_token_id"] = self.eos_token_id
        return d


def _softmax_half(prefix: str, hidden: int, m: Mapping[str, Any], kind: str, eps: float, out_scale: float):
    rot = m.get("rot")
    in_pair_1 = kind == "parallel"
    return FlexAttention.spec(
        prefix, hidden, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])), float(m["scale"]), eps,
        bias=True, out_bias=True, conv=int(m.get("conv", 0)), qk_norm=in_pair_1,
        rot=None if rot is None else (int(rot["dims"]), float(rot["base"])), softcap=float(m.get("softcap", 0.0)),
        slope_span=_SLOPE_SPAN if in_pair_1 else 0.0, chunk=int(m["mask"]["size"]) if "mask" in m else 0,
        out_gate=not in_pair_1, out_scale=out_scale)


def vafozen_plan(cfg: VafozenConfig) -> ModelPlan:
    h, eps = cfg.hidden_size, cfg.norm_eps
    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    for i, layer in enumerate(cfg.layers):
        p, m, kind = f"l{i}", layer["mixer"], layer["type"]
        if kind == "mamba2":
            mixer = Mamba2Mixer.spec(f"{p}.mix", h, int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]),
                                     int(m["norm_groups"]), int(m["conv"]), eps)
        else:
            r = m["right"]
            if "decay_rank" not in r:
                raise ConfigError(f"layers[{i}].mixer.right: the decay map's inner width is given neither by 'decay_rank' nor "
                                  f"by the shape of '{p}.mix.right.{_RANK_TENSOR[kind]}'")
            left = _softmax_half(f"{p}.mix.left", h, m["left"], kind, eps, float(m["left_scale"]))
            heads, dim, vdim = int(r["heads"]), int(r["dim"]), int(r.get("vdim", r["dim"]))
            if kind == "parallel":
                right = GatedLinearAttention.spec(f"{p}.mix.right", h, heads, dim, vdim, int(r["decay_rank"]), float(r["tau"]), eps,
                                                  float(m["right_scale"]))
            else:
                right = ShiftedTimeMix.spec(f"{p}.mix.right", h, heads, dim, vdim, int(r["decay_rank"]), eps, float(m["right_scale"]))
            mixer = SideBySide.spec(left, right)
        parts = {"mixer_norm": RMSNorm.spec(h, eps, f"{p}.norm1", gain_offset=1.0), "mixer": mixer}
        if layer.get("mlp") is not None:
            parts["ffn"] = SwiGLU.spec(f"{p}.mlp", h, int(layer["mlp"]["ff"]), names=("gate", "up", "down"))
        layers.append(LayerSpec("parallel", parts))
        schedule.append(ScheduleEntry(i))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=TokenEmbedding.spec("embed", cfg.vocab_size, h, cfg.embedding_scale), positions={}, layers=layers,
        schedule=schedule, final_norm=RMSNorm.spec(h, eps, "final.norm", gain_offset=1.0),
        lm_head=LinearHead.spec("head", cfg.vocab_size, h), eos_token_id=cfg.eos_token_id)


register_architecture("Vafozen", VafozenConfig, vafozen_plan)
