"""Navulorn: typed configuration from config.json and the model it describes.

A decoder whose layers are listed one by one in config.json (`layers`: each entry names its mixer
`type`, the mixer's sizes and its feed-forward, or none).  The norms stand behind the residual sums and
their results are the stream: x <- norm1(alpha x + mixer(x)), x <- norm2(alpha x + ff(x)), with one
`postln_alpha` for the model; the sublayers read the stream itself.  The embedding is multiplied by
`embedding.scale` and joined by a row of a second table chosen by the pair (previous token, token); the
logits come from an untied head behind the final norm and are capped by a tanh (`logit_softcap`).

Mixers: ``attention`` (grouped heads with value heads of their own size; an RMS norm over the WHOLE query
projection and the whole key projection with a weight per column, then the rotation of the first rot.dims
entries of every head in the (i, i + dims/2) layout, optionally with the long-context frequency rule
`rot.scaling` = {factor, low, high, original}; a sliding window `mask.size`; one sigmoid gate per head),
``latent_attention`` (keys and values through a shared normed latent of `kv_rank` entries and one rotated
key part of `rot_dim` entries for all heads, rotated in the (2i, 2i + 1) layout; queries projected directly;
sliding window) and ``mlstm`` (the matrix memory with exponential gates capped at `gate_cap`, per-head unit
norm with a weight, sigmoid output gate).  Feed-forwards: ``dense`` (gated unit with the tanh form of gelu)
and ``moe`` (routed SiLU experts: the `top` largest router logits, bias included, win and their weights
are the softmax over those logits alone).

config.json keys: architecture, vocab, width, embedding.{scale, bigram.{buckets, mul_prev, mul_cur}},
layers[].{type, mixer, mlp}, norm.eps, postln_alpha, logit_softcap.
Tensors: embed, bigram, final.norm, head and l<i>.{norm1, norm2, mix.*, mlp.*}.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .base import ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, optional, require


def _section(d, key, where):
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: required section '{key}' is missing")
    return v


def _positive(d, keys, where):
    for k in keys:
        if require(d, k, int, where) <= 0:
            raise ConfigError(f"{where}: '{k}' must be positive")


def _check_rot(rot, dim, where):
    if require(rot, "dims", int, where) <= 0 or rot["dims"] % 2:
        raise ConfigError(f"{where}: 'dims' must be positive and even")
    if rot["dims"] > dim:
        raise ConfigError(f"{where}: 'dims' {rot['dims']} exceeds the rotated size {dim}")
    if not require(rot, "base", float, where) > 1.0:
        raise ConfigError(f"{where}: 'base' must be larger than 1")
    sc = rot.get("scaling")
    if sc is not None:
        if not isinstance(sc, Mapping):
            raise ConfigError(f"{where}.scaling must be an object or null")
        sw = where + ".scaling"
        factor, low, high, orig = (require(sc, k, float, sw) for k in ("factor", "low", "high", "original"))
        if not (factor > 0 and orig > 0 and high > low > 0):
            raise ConfigError(f"{sw}: needs factor > 0, original > 0 and high > low > 0")


def _window(mx, where) -> int:
    mask = mx.get("mask")
    if mask is None:
        return 0
    if not isinstance(mask, Mapping):
        raise ConfigError(f"{where}.mask must be an object or null")
    if require(mask, "size", int, where + ".mask") <= 0:
        raise ConfigError(f"{where}.mask: 'size' must be positive")
    return mask["size"]


def _check_mlp(mlp, where):
    kind = require(mlp, "kind", str, where)
    if kind == "dense":
        if require(mlp, "ff", int, where) <= 0:
            raise ConfigError(f"{where}: 'ff' must be positive")
    elif kind == "moe":
        ex = _section(mlp, "expert", where)
        if require(ex, "ff", int, where + ".expert") <= 0:
            raise ConfigError(f"{where}.expert: 'ff' must be positive")
        r = _section(mlp, "router", where)
        _positive(r, ("experts", "top"), where + ".router")
        if r["top"] > r["experts"]:
            raise ConfigError(f"{where}.router: 'top' {r['top']} exceeds the {r['experts']} experts")
    else:
        raise ConfigError(f"{where}: kind {kind!r} is not supported (dense, moe)")


@dataclass(frozen=True)
class NavulornConfig(ModelConfig):
    vocab: int
    width: int
    layers: tuple                  # of plain dicts as config.json gives them (validated)
    norm_eps: float
    alpha: float = 1.0             # postln_alpha
    embed_scale: float = 1.0
    bigram: Optional[tuple] = None   # (buckets, mul_prev, mul_cur) or None
    logit_softcap: float = 0.0
    architecture: str = "Navulorn"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "NavulornConfig":
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: required key 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"config.json: layers[{i}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"{where} must be an object")
            typ = require(layer, "type", str, where)
            mx = _section(layer, "mixer", where)
            mw = where + ".mixer"
            _positive(mx, ("heads", "dim", "vdim"), mw)
            if typ == "attention":
                if require(mx, "kv_heads", int, mw) <= 0 or mx["heads"] % mx["kv_heads"]:
                    raise ConfigError(f"{mw}: heads {mx['heads']} is not a multiple of kv_heads {mx.get('kv_heads')}")
                require(mx, "scale", float, mw)
                _check_rot(_section(mx, "rot", mw), mx["dim"], mw + ".rot")
                _window(mx, mw)
            elif typ == "latent_attention":
                _positive(mx, ("rot_dim", "kv_rank"), mw)
                require(mx, "scale", float, mw)
                rot = _section(mx, "rot", mw)
                _check_rot(rot, mx["rot_dim"], mw + ".rot")
                if rot["dims"] != mx["rot_dim"]:
                    raise ConfigError(f"{mw}.rot: 'dims' {rot['dims']} must equal rot_dim {mx['rot_dim']}")
                _window(mx, mw)
            elif typ == "mlstm":
                if require(mx, "gate_cap", float, mw) <= 0:
                    raise ConfigError(f"{mw}: 'gate_cap' must be positive")
            else:
                raise ConfigError(f"{where}: mixer type {typ!r} is not supported (attention, latent_attention, mlstm)")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{where}.mlp must be an object or null")
                _check_mlp(mlp, where + ".mlp")
            checked.append(copy.deepcopy(dict(layer)))
        norm = _section(d, "norm", "config.json")
        emb = d.get("embedding") or {}
        if not isinstance(emb, Mapping):
            raise ConfigError("config.json: 'embedding' must be an object")
        bigram = emb.get("bigram")
        if bigram is not None:
            if not isinstance(bigram, Mapping):
                raise ConfigError("config.json: embedding.bigram must be an object or null")
            bw = "config.json: embedding.bigram"
            bigram = (require(bigram, "buckets", int, bw), require(bigram, "mul_prev", int, bw),
                      require(bigram, "mul_cur", int, bw))
            if bigram[0] <= 0 or bigram[1] < 0 or bigram[2] < 0:
                raise ConfigError(f"{bw}: 'buckets' must be positive and the multipliers not negative")
        cfg = cls(vocab=require(d, "vocab", int), width=require(d, "width", int), layers=tuple(checked),
                  norm_eps=require(norm, "eps", float, "config.json: norm"),
                  alpha=optional(d, "postln_alpha", float, 1.0),
                  embed_scale=optional(emb, "scale", float, 1.0, "config.json: embedding"), bigram=bigram,
                  logit_softcap=optional(d, "logit_softcap", float, 0.0))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not cfg.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if cfg.logit_softcap < 0:
            raise ConfigError("config.json: 'logit_softcap' must not be negative")
        return cfg

    def to_dict(self) -> dict:
        emb = {"scale": self.embed_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "embedding": emb,
             "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps}, "postln_alpha": self.alpha}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d

    # ------------------------------------------------------------------ the model as data
    def _mixer(self, i: int, layer) -> PartSpec:
        p, mx, d = f"l{i}.mix.", layer["mixer"], self.width
        if layer["type"] == "attention":
            return PartSpec("gated_attention", {
                "hidden_size": d, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"], "head_dim": mx["dim"],
                "v_head_dim": mx["vdim"], "scale": float(mx["scale"]), "qk_norm": "row", "eps": self.norm_eps,
                "window": _window(mx, "mixer"), "gate": "sigmoid", "gate_per_head": True}, p)
        if layer["type"] == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": d, "num_heads": mx["heads"], "head_dim": mx["dim"], "rot_dim": mx["rot_dim"],
                "v_head_dim": mx["vdim"], "kv_rank": mx["kv_rank"], "q_rank": 0, "eps": self.norm_eps,
                "scale": float(mx["scale"]), "window": _window(mx, "mixer")}, p)
        return PartSpec("mlstm", {
            "hidden_size": d, "num_heads": mx["heads"], "head_dim": mx["dim"], "v_head_dim": mx["vdim"],
            "gate_cap": float(mx["gate_cap"]), "q_scale": float(mx["dim"]) ** -0.5, "eps": self.norm_eps,
            "gate": "sigmoid"}, p)

    @staticmethod
    def _position(layer) -> Optional[PartSpec]:
        if layer["type"] == "mlstm":
            return None
        rot = layer["mixer"]["rot"]
        sc = rot.get("scaling")
        return PartSpec("rotary_scaled", {
            "dims": rot["dims"], "base": float(rot["base"]),
            "scaling": None if sc is None else {k: float(sc[k]) for k in ("factor", "low", "high", "original")},
            "layout": "half" if layer["type"] == "attention" else "pairs"})

    def _ffn(self, i: int, mlp):
        if mlp is None:
            return None
        d, p = self.width, f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return PartSpec("clamped_glu", {"hidden_size": d, "intermediate_size": mlp["ff"], "limit": 0.0,
                                            "shift": 0.0, "activation": "gelu_tanh"}, p)
        r = mlp["router"]
        return PartSpec("routed_experts", {
            "hidden_size": d, "intermediate_size": mlp["expert"]["ff"], "num_experts": r["experts"], "top_k": r["top"],
            "score": "softmax", "correction": False, "normalize": True, "weight_eps": 0.0, "route_scale": 1.0,
            "router_bias": True}, p)

    def model_spec(self) -> ModelSpec:
        d = self.width
        norm = lambda name: PartSpec("rms_norm", {"size": d, "eps": self.norm_eps, "tensor": name})
        layers = []
        for i, layer in enumerate(self.layers):
            ffn = self._ffn(i, layer.get("mlp"))
            norms = {"mixer": norm(f"l{i}.norm1")}
            if ffn is not None:
                norms["ffn"] = norm(f"l{i}.norm2")
            layers.append(LayerSpec(block="sum_norm", mixer=self._mixer(i, layer), ffn=ffn, norms=norms,
                                    position=self._position(layer), block_params={"alpha": self.alpha}))
        emb = {"vocab_size": self.vocab, "hidden_size": d, "tensor": "embed", "scale": self.embed_scale}
        if self.bigram is not None:
            emb["pair"] = {"tensor": "bigram", "buckets": self.bigram[0], "mul_prev": self.bigram[1],
                           "mul_cur": self.bigram[2]}
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=d, embedding=PartSpec("embedding", emb),
            layers=tuple(layers), run_order=tuple(RunEntry(i) for i in range(len(layers))),
            final_norm=norm("final.norm"),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": d, "tensor": "head",
                                         "softcap": self.logit_softcap}),
            max_position=0)
