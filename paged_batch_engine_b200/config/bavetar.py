"""Typed configuration of the Bavetar design and its model as data.

config.json keys: ``architecture`` ("Bavetar"), ``width``, ``vocab``, ``norm.eps``,
``logit_scale``, ``logit_softcap`` and ``layers``, a list of entries with ``type``
("mamba2" or "latent_attention"), ``mixer`` (the mixer's sizes and constants) and ``mlp``
(``{"kind": "dense", "ff": n}``, ``{"kind": "moe", "expert": {"ff": n}, "router": {"experts",
"top", "scale", "groups": {"count", "keep"}}}`` or null).

Tensors: ``embed`` (also the output head), ``final.norm``; per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*`` and ``l<i>.mlp.*``.

A layer adds two branches computed from norms of the same residual: x + mixer(norm1(x)) +
mlp(norm2(x)).  mamba2: a selective state-space recurrence behind a short causal convolution,
gated, with a grouped RMS norm.  latent_attention: softmax attention over a compressed latent per
token with a rotated key part shared by the heads, a sink in the softmax and a sigmoid gate per
head.  The dense feed-forward squares a relu; the routed one picks gated silu experts from the
best groups.  The logits are scaled and soft-capped.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .specs import BlockSpec, ConfigError, ModelSpec, PartSpec, RunStep

_LAYER_TYPES = ("mamba2", "latent_attention")
_MLP_KINDS = ("dense", "moe")


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"{where} lacks {key!r}")
    return d[key]


def _positive(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


@dataclass
class BavetarConfig:
    width: int
    vocab: int
    eps: float
    logit_scale: float
    logit_softcap: Optional[float]
    layers: List[dict]
    raw: Dict[str, Any]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "BavetarConfig":
        cap = d.get("logit_softcap")
        cfg = cls(width=_positive(_need(d, "width", "config.json"), "width"),
                  vocab=_positive(_need(d, "vocab", "config.json"), "vocab"),
                  eps=float(_need(_need(d, "norm", "config.json"), "eps", "norm")),
                  logit_scale=float(d.get("logit_scale", 1.0)),
                  logit_softcap=float(cap) if cap else None,
                  layers=list(_need(d, "layers", "config.json")), raw=dict(d))
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps!r}")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        if not self.layers:
            raise ConfigError("layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in _LAYER_TYPES:
                raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {', '.join(_LAYER_TYPES)}")
            m = _need(layer, "mixer", where)
            mw = where + ".mixer"
            if kind == "mamba2":
                for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    _positive(_need(m, key, mw), f"{mw}.{key}")
                if m["heads"] % m["groups"]:
                    raise ConfigError(f"{mw}: heads must be a multiple of groups")
                if (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    raise ConfigError(f"{mw}: heads * vdim must be a multiple of norm_groups")
                if m["conv"] > 16:
                    raise ConfigError(f"{mw}: at most 16 convolution taps are supported")
            else:
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
                    _positive(_need(m, key, mw), f"{mw}.{key}")
                if m["rot_dim"] % 2:
                    raise ConfigError(f"{mw}.rot_dim must be even")
                _need(m, "scale", mw)
                rot = _need(m, "rot", mw)
                dims = _positive(_need(rot, "dims", mw + ".rot"), "rot.dims")
                if dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"{mw}.rot.dims must be even and at most rot_dim")
                if not float(_need(rot, "base", mw + ".rot")) > 0:
                    raise ConfigError("rot.base must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                mk = mlp.get("kind", "dense")
                if mk not in _MLP_KINDS:
                    raise ConfigError(f"{where}.mlp.kind {mk!r} is not supported; known: {', '.join(_MLP_KINDS)}")
                if mk == "dense":
                    _positive(_need(mlp, "ff", where + ".mlp"), f"{where}.mlp.ff")
                else:
                    _positive(_need(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert"), "expert.ff")
                    r = _need(mlp, "router", where + ".mlp")
                    E = _positive(_need(r, "experts", where + ".mlp.router"), "router.experts")
                    top = _positive(_need(r, "top", where + ".mlp.router"), "router.top")
                    g = r.get("groups") or {}
                    count = _positive(g.get("count", 1), "router.groups.count")
                    keep = _positive(g.get("keep", count), "router.groups.keep")
                    if E % count or keep > count or top > keep * (E // count):
                        raise ConfigError(f"{where}.mlp.router: experts divide into equal groups, keep <= count, "
                                          "and the kept groups hold at least `top` experts")

    # ------------------------------------------------------------------ the model as data
    def _mixer(self, layer: dict) -> PartSpec:
        m = layer["mixer"]
        if layer["type"] == "mamba2":
            return PartSpec("selective_state_space", dict(
                hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["vdim"]), state_dim=int(m["state"]),
                groups=int(m["groups"]), conv_taps=int(m["conv"]), norm_groups=int(m["norm_groups"]), eps=self.eps))
        rot = m["rot"]
        return PartSpec("latent_attention", dict(
            hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
            value_dim=int(m["vdim"]), kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), scale=float(m["scale"]),
            eps=self.eps, rotary=dict(base=float(rot["base"]), dims=int(rot["dims"])), sink=True, out_gate=True))

    def _mlp(self, mlp: Optional[dict]) -> Optional[PartSpec]:
        if mlp is None:
            return None
        if mlp.get("kind", "dense") == "dense":
            return PartSpec("activation_mlp", dict(hidden_size=self.width, intermediate_size=int(mlp["ff"]),
                                                   activation="relu2", tensor_names=dict(up="up", down="down"),
                                                   weight_suffix=""))
        r = mlp["router"]
        g = r.get("groups") or {}
        count = int(g.get("count", 1))
        return PartSpec("routed_experts", dict(
            hidden_size=self.width, intermediate_size=int(mlp["expert"]["ff"]), num_experts=int(r["experts"]),
            top=int(r["top"]), groups=count, keep=int(g.get("keep", count)), scale=float(r.get("scale", 1.0))))

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", dict(size=self.width, eps=self.eps, weight_name=""))
        blocks = []
        for i, layer in enumerate(self.layers):
            ffn = self._mlp(layer.get("mlp"))
            blocks.append(BlockSpec(
                kind="parallel", mixer=self._mixer(layer), feed_forward=ffn, norm_mixer=norm,
                norm_feed_forward=norm if ffn is not None else None, prefix=f"l{i}.",
                names=dict(mixer="mix.", feed_forward="mlp.", norm_mixer="norm1", norm_feed_forward="norm2")))
        run = tuple(RunStep(block=i, cache_layer=i) for i in range(len(self.layers)))
        return ModelSpec(
            architecture="Bavetar", hidden_size=self.width, vocab_size=self.vocab, blocks=tuple(blocks),
            run_order=run, final_norm=norm, embedding_name="embed", final_norm_name="final.norm",
            lm_head_name=None, max_position=1 << 30, eos_token_ids=(),
            logit_scale=self.logit_scale, logit_softcap=self.logit_softcap)
