"""Typed configuration of the Gebadra design and its model as data.

config.json keys: ``architecture`` ("Gebadra"), ``width``, ``vocab``, ``norm.eps``, ``streams``
(residual streams; absent: the plain residual sum) and ``layers``, a list of entries with
``type`` ("lightning" or "parallel"), ``mixer`` (the mixer's sizes and constants), ``mlp``
(``{"kind": "dense", "ff": n}`` or null) and optionally ``weights_of: j`` (the layer runs layer
j's tensors with a cache and state of its own).

Tensors: ``embed``, ``head``, ``final.norm`` (+ ``.b``); per layer ``l<i>.norm1``, ``l<i>.norm2``
(+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``l<i>.hc{1,2}.{in,out,mix}``.

lightning: q, k, v through silu, decayed linear attention, one RMS norm over all heads with a
gain, a sigmoid gate.  parallel: the mean of two branches, each under an RMS norm with a gain:
``left`` = softmax attention over a window plus pooled blocks (query/key norm over the whole
projection, rotary on neighbouring pairs with linear scaling, head-mixed probabilities),
``right`` = retention (keys scaled by dim^-1/2, a unit RMS norm per head, a silu gate).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .specs import BlockSpec, ConfigError, ModelSpec, PartSpec, RunStep

_LAYER_TYPES = ("lightning", "parallel")


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"{where} lacks {key!r}")
    return d[key]


def _positive(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


@dataclass
class GebadraConfig:
    width: int
    vocab: int
    eps: float
    streams: Optional[int]
    layers: List[dict]
    raw: Dict[str, Any]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GebadraConfig":
        cfg = cls(width=_positive(_need(d, "width", "config.json"), "width"),
                  vocab=_positive(_need(d, "vocab", "config.json"), "vocab"),
                  eps=float(_need(_need(d, "norm", "config.json"), "eps", "norm")),
                  streams=d.get("streams"), layers=list(_need(d, "layers", "config.json")), raw=dict(d))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps!r}")
        if self.streams is not None:
            _positive(self.streams, "streams")
            if self.streams > 8:
                raise ConfigError(f"at most 8 residual streams are supported, got {self.streams}")
        if not self.layers:
            raise ConfigError("layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in _LAYER_TYPES:
                raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {', '.join(_LAYER_TYPES)}")
            m = _need(layer, "mixer", where)
            if kind == "lightning":
                self._check_linear(m, where + ".mixer")
            else:
                left, right = _need(m, "left", where + ".mixer"), _need(m, "right", where + ".mixer")
                self._check_linear(right, where + ".mixer.right")
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive(_need(left, key, where + ".mixer.left"), f"{where}.mixer.left.{key}")
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"{where}.mixer.left: heads must be a multiple of kv_heads")
                if left["dim"] % 2:
                    raise ConfigError(f"{where}.mixer.left: dim must be even")
                mask = _need(left, "mask", where + ".mixer.left")
                _positive(_need(mask, "size", where + ".mixer.left.mask"), "mask.size")
                if mask.get("pool") is not None:
                    _positive(mask["pool"], "mask.pool")
                _need(left, "scale", where + ".mixer.left")
                rot = left.get("rot")
                if rot is not None:
                    dims = _positive(_need(rot, "dims", where + ".mixer.left.rot"), "rot.dims")
                    if dims % 2 or dims > left["dim"]:
                        raise ConfigError(f"{where}.mixer.left.rot.dims must be even and at most dim")
                    if not float(_need(rot, "base", where + ".mixer.left.rot")) > 0:
                        raise ConfigError("rot.base must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not supported (only 'dense')")
                _positive(_need(mlp, "ff", where + ".mlp"), f"{where}.mlp.ff")
            if layer.get("weights_of") is not None:
                j = self.owner_of(i)
                if self.layers[j]["type"] != kind:
                    raise ConfigError(f"{where}.weights_of names a layer of another type")

    def owner_of(self, i: int) -> int:
        """The layer whose tensors layer i runs: itself, or the layer its ``weights_of`` names (followed
        through layers that name another in turn)."""
        seen = {i}
        while self.layers[i].get("weights_of") is not None:
            j = self.layers[i]["weights_of"]
            if not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < len(self.layers) or j in seen:
                raise ConfigError(f"layers[{i}].weights_of must name another layer that has tensors of its own")
            seen.add(j)
            i = j
        return i

    @staticmethod
    def _check_linear(m: dict, where: str) -> None:
        for key in ("heads", "dim", "vdim"):
            _positive(_need(m, key, where), f"{where}.{key}")
        decay = _need(m, "decay", where)
        if not isinstance(decay, (list, tuple)) or len(decay) != m["heads"]:
            raise ConfigError(f"{where}.decay must list one decay per head")

    # ------------------------------------------------------------------ the model as data
    def _linear(self, m: dict, lightning: bool) -> PartSpec:
        names = dict(q="q", k="k", v="v", g="g", o="o", norm="norm")
        common = dict(hidden_size=self.width, num_heads=int(m["heads"]), key_dim=int(m["dim"]),
                      value_dim=int(m["vdim"]), decay=tuple(float(x) for x in m["decay"]), eps=self.eps,
                      tensor_names=names, weight_suffix="")
        if lightning:
            return PartSpec("linear_attention", dict(common, activation="silu", key_scale=1.0, out_norm="joint",
                                                     norm_gain=True, gate="sigmoid"))
        return PartSpec("linear_attention", dict(common, activation="none", key_scale=float(m["dim"]) ** -0.5,
                                                 out_norm="head", norm_gain=False, gate="silu"))

    def _softmax(self, m: dict) -> PartSpec:
        rot = m.get("rot")
        rotary = None
        if rot is not None:
            scaling = rot.get("scaling") or {}
            rotary = dict(base=float(rot["base"]), dims=int(rot["dims"]), factor=float(scaling.get("factor", 1.0)))
        mask = m["mask"]
        return PartSpec("pooled_window_attention", dict(
            hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
            key_dim=int(m["dim"]), value_dim=int(m["vdim"]), scale=float(m["scale"]), window=int(mask["size"]),
            pool=int(mask["pool"]) if mask.get("pool") else None, eps=self.eps, rotary=rotary, qk_norm=True,
            talking_heads=True,
            tensor_names=dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", talk="talk"),
            weight_suffix=""))

    def _mixer(self, layer: dict) -> PartSpec:
        m = layer["mixer"]
        if layer["type"] == "lightning":
            return self._linear(m, True)
        return PartSpec("parallel", dict(hidden_size=self.width, eps=self.eps, gain_name="out",
                                         branches=(("left", self._softmax(m["left"])),
                                                   ("right", self._linear(m["right"], False)))))

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("layernorm", dict(size=self.width, eps=self.eps, weight_name="", bias_name=".b"))
        blocks, block_of = [], {}
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is not None:
                continue
            mlp = layer.get("mlp")
            ffn = None
            if mlp is not None:
                ffn = PartSpec("swiglu", dict(hidden_size=self.width, intermediate_size=int(mlp["ff"]),
                                              tensor_names=dict(gate="gate", up="up", down="down"), weight_suffix=""))
            block_of[i] = len(blocks)
            blocks.append(BlockSpec(
                kind="streams", mixer=self._mixer(layer), feed_forward=ffn, norm_mixer=norm,
                norm_feed_forward=norm if ffn is not None else None, prefix=f"l{i}.",
                names=dict(mixer="mix.", feed_forward="mlp.", norm_mixer="norm1", norm_feed_forward="norm2",
                           streams_mixer="hc1.", streams_feed_forward="hc2."),
                args=dict(streams=self.streams)))
        run = tuple(RunStep(block=block_of[self.owner_of(i)], cache_layer=i) for i in range(len(self.layers)))
        return ModelSpec(
            architecture="Gebadra", hidden_size=self.width, vocab_size=self.vocab, blocks=tuple(blocks),
            run_order=run, final_norm=norm, embedding_name="embed", final_norm_name="final.norm",
            lm_head_name="head", max_position=1 << 30, eos_token_ids=(),
            residual_streams=self.streams or 1)
