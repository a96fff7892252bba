"""``Nezalorn``: a decoder whose layers are listed one by one in config.json, each with one of three mixers
(attention through a latent with a sliding window, the generalized delta rule, a gated linear recurrence), a
PolyNorm feed-forward (or none) beside the mixer in a parallel block, and a learned weighted average over the
results of all layers so far as what the next layer reads. Logits go through the embedding table.

config.json: ``architecture`` (the name), ``vocab``, ``width``, ``norm.eps``, ``layers``: a list of
``{"type", "mixer": {...}, "mlp": {"kind": "dense", "ff"} | null}``. Mixer keys: ``latent_attention``: ``heads dim
rot_dim vdim q_rank kv_rank scale mask.size rot.{dims, base, scaling.{factor, original, fast, slow}}`` and optionally
``kv_from`` (the layer whose cached rows it reads; it has then no ``dkv`` tensors); ``general_delta``: ``heads dim``
and optionally ``decay_rank`` (the decay map's inner width; without it the shape of ``w1`` gives it); ``rglru``: ``width conv blocks``.

Tensor names: ``embed``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.dwa``,
``l<i>.mix.<name>``, ``l<i>.mlp.{up, up.b, down, down.b, act}``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig
from ..parts.delta_rule import GeneralizedDeltaRule
from ..parts.depth import DepthAverage
from ..parts.embedding import LinearHead, TokenEmbedding
from ..parts.feedforward import PolyNormFeedForward
from ..parts.latent_attention import LatentAttention
from ..parts.norm import RMSNorm
from ..parts.position import FrequencyRotary
from ..parts.rglru import GatedLinearRecurrence
from ..parts.spec import LayerSpec, ModelPlan, ScheduleEntry
from ..registry import register_architecture

_MIXERS = ("latent_attention", "general_delta", "rglru")
# Positions are turned into angles in 32-bit floats, which hold every integer up to 2^24.
_MAX_POSITIONS = 1 << 24


def _int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _num(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class NezalornConfig(ModelConfig):
    layers: Tuple[dict, ...] = ()
    norm_eps: float = 1e-5

    @classmethod
    def from_json_dict(cls, d: Mapping[str, Any]) -> "NezalornConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type must be one of {_MIXERS}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            kind = layer["type"]
            if kind == "latent_attention":
                for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
                    _int(m, k, where + ".mixer")
                _num(m, "scale", where + ".mixer")
                if not isinstance(m.get("mask"), dict):
                    raise ConfigError(f"config.json: {where}.mixer.mask must be an object with 'size'")
                _int(m["mask"], "size", where + ".mixer.mask")
                rot = m.get("rot")
                if not isinstance(rot, dict):
                    raise ConfigError(f"config.json: {where}.mixer.rot must be an object")
                if _int(rot, "dims", where + ".mixer.rot") != m["rot_dim"] or m["rot_dim"] % 2:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims must equal rot_dim and be even")
                _num(rot, "base", where + ".mixer.rot")
                sc = rot.get("scaling")
                if sc is not None:
                    if not isinstance(sc, dict):
                        raise ConfigError(f"config.json: {where}.mixer.rot.scaling must be an object or null")
                    for k in ("factor", "original", "fast", "slow"):
                        if _num(sc, k, where + ".mixer.rot.scaling") <= 0:
                            raise ConfigError(f"config.json: {where}.mixer.rot.scaling.{k} must be > 0")
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < i):
                        raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier layer")
                    o = layers[src]
                    if o.get("type") != "latent_attention" or o["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}.mixer.kv_from names a layer that caches no latent of its own")
                    if any(o["mixer"].get(k) != m.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                        raise ConfigError(f"config.json: {where} and layer {src} must agree in kv_rank, rot_dim and rot")
            elif kind == "general_delta":
                _int(m, "heads", where + ".mixer")
                _int(m, "dim", where + ".mixer")
                if "decay_rank" in m:
                    _int(m, "decay_rank", where + ".mixer")
            else:
                w, b = _int(m, "width", where + ".mixer"), _int(m, "blocks", where + ".mixer")
                _int(m, "conv", where + ".mixer")
                if w % b:
                    raise ConfigError(f"config.json: {where}.mixer.width must be a multiple of blocks")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp must be null or of kind 'dense'")
                _int(mlp, "ff", where + ".mlp")
            checked.append(layer)
        eps = _num(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be > 0")
        eos = d.get("eos_token_id")
        return cls(architecture=str(d.get("architecture") or "Nezalorn"), model_type="nezalorn",
                   vocab_size=_int(d, "vocab", "config"), hidden_size=_int(d, "width", "config"),
                   num_hidden_layers=len(checked), max_position_embeddings=_MAX_POSITIONS,
                   tie_word_embeddings=True, eos_token_id=int(eos) if isinstance(eos, int) and not isinstance(eos, bool) else -1,
                   layers=tuple(checked), norm_eps=eps)

    def with_tensor_shapes(self, shapes: Mapping[str, Any]) -> "NezalornConfig":
        """The inner width of a delta-rule layer's decay map is the number of rows of its ``w1`` tensor; config.json
        need not state it (``mixer.decay_rank``, which the random-weights mode writes)."""
        layers = []
        for i, layer in enumerate(self.layers):
            name = f"l{i}.mix.w1"
            if layer["type"] == "general_delta" and "decay_rank" not in layer["mixer"] and name in shapes:
                layer = dict(layer, mixer=dict(layer["mixer"], decay_rank=int(tuple(shapes[name])[0])))
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    def to_json_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "layers": [dict(layer) for layer in self.layers]}
        if self.eos_token_id >= 0:
            d["eos_token_id"] = self.eos_token_id
        return d


def _rotary_name(rot: Mapping[str, Any]) -> str:
    sc = rot.get("scaling") or {}
    return "rot:" + ",".join(str(x) for x in (rot["dims"], rot["base"], sc.get("factor"), sc.get("original"),
                                               sc.get("fast"), sc.get("slow")))


def nezalorn_plan(cfg: NezalornConfig) -> ModelPlan:
    h, eps, n_layers = cfg.hidden_size, cfg.norm_eps, len(cfg.layers)
    positions: Dict[str, Any] = {}
    # A latent that later layers read must stay cached as long as the widest window among its readers.
    keep: Dict[int, int] = {}
    for i, layer in enumerate(cfg.layers):
        if layer["type"] == "latent_attention":
            owner = layer["mixer"].get("kv_from", i)
            if owner is None:
                owner = i
            keep[owner] = max(keep.get(owner, 0), int(layer["mixer"]["mask"]["size"]))
    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer["mixer"]
        reads = None
        if layer["type"] == "latent_attention":
            name = _rotary_name(m["rot"])
            positions.setdefault(name, FrequencyRotary.spec(int(m["rot"]["dims"]), float(m["rot"]["base"]), m["rot"].get("scaling")))
            reads = m.get("kv_from")
            owner = i if reads is None else int(reads)
            mixer = LatentAttention.spec(f"{p}.mix", h, int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]),
                                         int(m["q_rank"]), int(m["kv_rank"]), float(m["scale"]), int(m["mask"]["size"]),
                                         keep[owner], eps, name, owns_kv=reads is None)
        elif layer["type"] == "general_delta":
            if "decay_rank" not in m:
                raise ConfigError(f"layers[{i}].mixer: the decay map's inner width is given neither by 'decay_rank' nor by "
                                  f"the shape of '{p}.mix.w1'")
            mixer = GeneralizedDeltaRule.spec(f"{p}.mix", h, int(m["heads"]), int(m["dim"]), int(m["decay_rank"]), eps)
        else:
            mixer = GatedLinearRecurrence.spec(f"{p}.mix", h, int(m["width"]), int(m["conv"]), int(m["blocks"]))
        parts = {"mixer_norm": RMSNorm.spec(h, eps, f"{p}.norm1"), "mixer": mixer}
        if layer.get("mlp") is not None:
            parts["ffn_norm"] = RMSNorm.spec(h, eps, f"{p}.norm2")
            parts["ffn"] = PolyNormFeedForward.spec(f"{p}.mlp", h, int(layer["mlp"]["ff"]), eps)
        parts["depth"] = DepthAverage.spec(f"{p}.dwa", i + 2, n_layers + 1)
        layers.append(LayerSpec("parallel", parts))
        schedule.append(ScheduleEntry(i, reads_cache_of=None if reads is None else int(reads)))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=TokenEmbedding.spec("embed", cfg.vocab_size, h), positions=positions, layers=layers, schedule=schedule,
        final_norm=RMSNorm.spec(h, eps, "final.norm"), lm_head=LinearHead.spec("embed", cfg.vocab_size, h),
        eos_token_id=cfg.eos_token_id)


register_architecture("Nezalorn", NezalornConfig, nezalorn_plan)
