"""Divuzen: typed configuration from config.json and the model it describes.

A decoder whose layers are listed one by one in config.json (`layers`: each entry names its mixer
`type`, the mixer's sizes and its feed-forward, or none).  Every sublayer stands between two norms:
x <- x + norm1b(mixer(norm1(x))), x <- x + norm2b(ff(norm2(x))); all norms are RMS norms whose
weight is stored around zero and applied as (1 + w).  The LM head is the embedding table and the
logits are multiplied by `logit_scale`.

Mixers: ``attention`` (grouped heads with value heads of their own size; RMS norm per head with a
weight on queries and keys, then a rotation of the first rot.dims entries in neighbouring pairs
(2i, 2i + 1); causal; a learned sink per head in the softmax's denominator; with `kv_from: j` the
layer has no keys and values of its own and reads those of layer j) and ``retention`` (linear
attention with a fixed decay per head and a state per request; rotation in the (i, i + dims/2)
layout; keys scaled by dim^-1/2; each head's output divided by its root mean square, gated by
silu(W_g h)).  Feed-forwards: ``dense`` (a gated unit with clamped branches, g = min(gate, limit),
u = clamp(up, +-limit), y = g sigmoid(1.702 g) (u + 1)) and ``moe`` (routed SwiGLU experts chosen by
sigmoid scores plus a correction inside the best groups of experts, and a gated shared expert).

config.json keys: architecture, vocab, width, layers[].{type, mixer, mlp}, norm.eps, logit_scale.
Tensors: embed, final.norm and l<i>.{norm1, norm1b, norm2, norm2b, mix.*, mlp.*}.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, optional, require

GLU_ALPHA = 1.702          # the design fixes these: the dense unit's sigmoid slope and its shift of the up branch,
GLU_SHIFT = 1.0
GROUP_BEST = 2             # how many of a group's choice scores make the group's score,
WEIGHT_EPS = 1e-20         # and what is added to the sum of the chosen scores before the division


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
        raise ConfigError(f"{where}: 'dims' {rot['dims']} exceeds the head size {dim}")
    if not require(rot, "base", float, where) > 1.0:
        raise ConfigError(f"{where}: 'base' must be larger than 1")


def _check_expert(sec, where):
    if not isinstance(sec, Mapping) or require(sec, "ff", int, where) <= 0:
        raise ConfigError(f"{where}: 'ff' must be positive")


def _check_mlp(mlp, where):
    kind = require(mlp, "kind", str, where)
    if kind == "dense":
        if require(mlp, "ff", int, where) <= 0:
            raise ConfigError(f"{where}: 'ff' must be positive")
        if not require(mlp, "limit", float, where) > 0:
            raise ConfigError(f"{where}: 'limit' must be positive")
    elif kind == "moe":
        _check_expert(_section(mlp, "expert", where), where + ".expert")
        r = _section(mlp, "router", where)
        rw = where + ".router"
        _positive(r, ("experts", "top"), rw)
        require(r, "scale", float, rw)
        groups = r.get("groups")
        count = keep = 1
        if groups is not None:
            if not isinstance(groups, Mapping):
                raise ConfigError(f"{rw}.groups must be an object or null")
            _positive(groups, ("count", "keep"), rw + ".groups")
            count, keep = groups["count"], groups["keep"]
        if r["experts"] % count or keep > count:
            raise ConfigError(f"{rw}: {r['experts']} experts do not form {count} equal groups of which {keep} are kept")
        if r["top"] > keep * (r["experts"] // count):
            raise ConfigError(f"{rw}: 'top' {r['top']} exceeds the experts of the kept groups")
        if mlp.get("shared") is not None:
            _check_expert(mlp["shared"], where + ".shared")
    else:
        raise ConfigError(f"{where}: kind {kind!r} is not supported (dense, moe)")


@dataclass(frozen=True)
class DivuzenConfig(ModelConfig):
    vocab: int
    width: int
    layers: tuple                  # of plain dicts as config.json gives them (validated)
    norm_eps: float
    logit_scale: float = 1.0
    architecture: str = "Divuzen"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DivuzenConfig":
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
            _check_rot(_section(mx, "rot", mw), mx["dim"], mw + ".rot")
            if typ == "attention":
                if require(mx, "kv_heads", int, mw) <= 0 or mx["heads"] % mx["kv_heads"]:
                    raise ConfigError(f"{mw}: heads {mx['heads']} is not a multiple of kv_heads {mx.get('kv_heads')}")
                require(mx, "scale", float, mw)
                src = mx.get("kv_from")
                if src is not None:
                    src = require(mx, "kv_from", int, mw)
                    if not 0 <= src < i:
                        raise ConfigError(f"{mw}: 'kv_from' {src} must name an earlier layer")
                    other = checked[src]
                    om = other["mixer"]
                    if other["type"] != "attention" or om.get("kv_from") is not None:
                        raise ConfigError(f"{mw}: 'kv_from' {src} must name an attention layer with keys and values of its own")
                    if any(om[k] != mx[k] for k in ("kv_heads", "dim", "vdim")) or dict(om["rot"]) != dict(mx["rot"]):
                        raise ConfigError(f"{mw}: layer {src}, whose keys and values this layer reads, has other "
                                          f"key/value heads, head sizes or rotation")
            elif typ == "retention":
                decay = mx.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != mx["heads"]:
                    raise ConfigError(f"{mw}: 'decay' must list one number per head")
                for x in decay:
                    if isinstance(x, bool) or not isinstance(x, (int, float)) or not 0.0 <= float(x) <= 1.0:
                        raise ConfigError(f"{mw}: 'decay' entries must be numbers in [0, 1]")
            else:
                raise ConfigError(f"{where}: mixer type {typ!r} is not supported (attention, retention)")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{where}.mlp must be an object or null")
                _check_mlp(mlp, where + ".mlp")
            checked.append(copy.deepcopy(dict(layer)))
        norm = _section(d, "norm", "config.json")
        cfg = cls(vocab=require(d, "vocab", int), width=require(d, "width", int), layers=tuple(checked),
                  norm_eps=require(norm, "eps", float, "config.json: norm"),
                  logit_scale=optional(d, "logit_scale", float, 1.0))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not cfg.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
                "logit_scale": self.logit_scale}

    # ------------------------------------------------------------------ the model as data
    def _mixer(self, i: int, layer) -> PartSpec:
        p, mx, d = f"l{i}.mix.", layer["mixer"], self.width
        if layer["type"] == "attention":
            return PartSpec("attention", {
                "hidden_size": d, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"], "head_dim": mx["dim"],
                "v_head_dim": mx["vdim"], "scale": float(mx["scale"]), "qk_norm": True, "qk_norm_eps": self.norm_eps,
                "sink": True, "own_kv": mx.get("kv_from") is None, "names": "short"}, p)
        return PartSpec("retention", {
            "hidden_size": d, "num_heads": mx["heads"], "head_dim": mx["dim"], "v_head_dim": mx["vdim"],
            "decay": tuple(float(x) for x in mx["decay"]), "key_scale": float(mx["dim"]) ** -0.5, "eps": self.norm_eps,
            "gate": "silu"}, p)

    @staticmethod
    def _position(layer) -> PartSpec:
        rot = layer["mixer"]["rot"]
        return PartSpec("rotary_scaled", {"dims": rot["dims"], "base": float(rot["base"]), "scaling": None,
                                          "layout": "pairs" if layer["type"] == "attention" else "half"})

    def _ffn(self, i: int, mlp):
        if mlp is None:
            return None
        d, p = self.width, f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return PartSpec("clamped_glu", {"hidden_size": d, "intermediate_size": mlp["ff"], "limit": float(mlp["limit"]),
                                            "alpha": GLU_ALPHA, "shift": GLU_SHIFT}, p)
        r = mlp["router"]
        groups = r.get("groups") or {"count": 1, "keep": 1}
        shared = mlp.get("shared")
        return PartSpec("routed_experts", {
            "hidden_size": d, "intermediate_size": mlp["expert"]["ff"], "num_experts": r["experts"], "top_k": r["top"],
            "n_groups": groups["count"], "keep_groups": groups["keep"], "group_best": GROUP_BEST,
            "score": "sigmoid", "correction": True, "normalize": True, "weight_eps": WEIGHT_EPS,
            "route_scale": float(r["scale"]), "shared_size": shared["ff"] if shared else 0,
            "shared_gate": bool(shared)}, p)

    def model_spec(self) -> ModelSpec:
        d = self.width
        norm = lambda name: PartSpec("rms_norm", {"size": d, "eps": self.norm_eps, "tensor": name, "one_plus": True})
        layers, run = [], []
        for i, layer in enumerate(self.layers):
            ffn = self._ffn(i, layer.get("mlp"))
            norms = {"mixer": norm(f"l{i}.norm1"), "mixer_out": norm(f"l{i}.norm1b")}
            if ffn is not None:
                norms["ffn"] = norm(f"l{i}.norm2")
                norms["ffn_out"] = norm(f"l{i}.norm2b")
            layers.append(LayerSpec(block="sandwich_norm", mixer=self._mixer(i, layer), ffn=ffn, norms=norms,
                                    position=self._position(layer)))
            run.append(RunEntry(i, cache_of=layer["mixer"].get("kv_from") if layer["type"] == "attention" else None))
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=d,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": d, "tensor": "embed"}),
            layers=tuple(layers), run_order=tuple(run), final_norm=norm("final.norm"),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": d, "tied_to": "embed",
                                         "tensor": "head", "scale": self.logit_scale}),
            max_position=0)
