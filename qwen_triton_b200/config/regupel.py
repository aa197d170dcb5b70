"""Typed configuration of the Regupel design, read from config.json.

The file names its design under ``architecture`` and gives ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``residual_mult``, ``logit_scale`` and a list ``layers``.  An entry has ``type`` (its mixer: ``attention`` or ``parallel``), the
mixer's sizes and constants under ``mixer`` and its feed-forward under ``mlp`` (null for none).  An entry with ``weights_of``: j
has no tensors of its own: it runs layer j's (mixer, feed-forward and norms) with a cache and state of its own, and the rest
of the entry equals layer j's.  Layers need not be alike.

``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot.dims`` / ``rot.base`` / ``rot.scaling`` (``factor``, ``low``,
``high``, ``original``; absent: plain rotation; no ``rot``: none), ``mask.size`` (absent: every earlier token is seen).
``parallel``: two mixers under ``left`` and ``right`` and the constants ``left_scale`` and ``right_scale``; ``left`` has ``heads``,
``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` and ``mask.keep_first``; ``right`` has ``heads``, ``dim``, ``vdim`` and ``decay``
(one number per head).  ``mlp``: ``kind`` "moe" with ``expert.ff``, ``router.experts``, ``router.top`` and ``shared.ff`` (absent: no
shared expert).

What the design fixes, and ``model_spec`` therefore states as parameters of the parts: no norm in front of a sublayer and a
layer norm with weight and bias on what it returns, x += m LN(sublayer(x)) (``residual_mult`` rides on the norm's weight and
bias); in ``attention`` a rotate-half rotation of the first ``rot.dims`` elements with frequencies stretched by wavelength,
q and k divided by their root mean square per head without a weight, a softmax whose denominator holds one stored number per
head, and a sigmoid gate of one number per head; in ``parallel`` a left attention whose q and k are RMS-normed over the
whole projection with weights, without rotation, under a window that keeps the first tokens, beside a linear attention with
a constant decay per head on SiLU'd q, k and v whose heads are RMS-normed together and gated; experts with the SiLU gate
chosen by a sigmoid router, their scores (not renormalised) multiplying the experts' inputs, plus a shared expert; the head
is the embedding table (without the embedding's scale) times ``logit_scale``; tensor names ``embed``, ``final.norm`` (+ ``.b``)
and ``l<i>.{norm1,norm2}`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.{router,e<k>.*,shared.*}`` without a ``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .qwen3 import ConfigError
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MAX_POSITIONS = 1 << 20          # the design names no longest sequence; the rotation table is made for the cache's length


@dataclass(frozen=True)
class RegupelAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None = None          # mask.size
    keep_first: int = 0                # mask.keep_first (the left mixer of a parallel layer)
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_scaling: tuple | None = None   # (factor, low, high, original)


@dataclass(frozen=True)
class RegupelLinear:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]


@dataclass(frozen=True)
class RegupelExperts:
    ff: int
    experts: int
    top: int
    shared_ff: int | None


@dataclass(frozen=True)
class RegupelLayer:
    type: str                                  # "attention" or "parallel"
    attention: RegupelAttention                # the mixer, or the left one of a parallel layer
    linear: RegupelLinear | None = None        # the right mixer of a parallel layer
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: RegupelExperts | None = None
    weights_of: int | None = None


def _need(mapping: Mapping[str, Any], key: str, where: str):
    if not isinstance(mapping, Mapping) or mapping.get(key) is None:
        raise ConfigError(f"config.json lacks {where}.{key}" if where else f"config.json lacks the key {key!r}")
    return mapping[key]


def _attention(mixer: Mapping[str, Any], at: str) -> RegupelAttention:
    heads, dim = int(_need(mixer, "heads", at)), int(_need(mixer, "dim", at))
    mask = mixer.get("mask") or {}
    rot = mixer.get("rot") or {}
    scaling = rot.get("scaling")
    if scaling is not None:
        scaling = tuple(float(_need(scaling, key, f"{at}.rot.scaling")) for key in ("factor", "low", "high", "original"))
    return RegupelAttention(heads=heads, kv_heads=int(mixer.get("kv_heads") or heads), dim=dim, vdim=int(mixer.get("vdim") or dim),
                            scale=float(_need(mixer, "scale", at)), window=int(mask["size"]) if mask.get("size") is not None else None,
                            keep_first=int(mask.get("keep_first") or 0), rot_dims=int(rot.get("dims") or 0),
                            rot_base=float(rot.get("base", 10000.0)), rot_scaling=scaling)


def _experts(mlp, at: str) -> RegupelExperts | None:
    if mlp is None:
        return None
    if _need(mlp, "kind", at) != "moe":
        raise ConfigError(f"{at}: the Regupel design has no feed-forward {mlp['kind']!r}")
    router = _need(mlp, "router", at)
    shared = mlp.get("shared")
    return RegupelExperts(ff=int(_need(_need(mlp, "expert", at), "ff", f"{at}.expert")), experts=int(_need(router, "experts", f"{at}.router")),
                          top=int(_need(router, "top", f"{at}.router")), shared_ff=int(_need(shared, "ff", f"{at}.shared")) if shared is not None else None)


@dataclass(frozen=True)
class RegupelConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    logit_scale: float
    layers: tuple[RegupelLayer, ...]
    architecture: str = "Regupel"
    raw: Mapping[str, Any] = field(default_factory=dict, repr=False, compare=False)

    family = "regupel"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_hf_config(cls, raw: Mapping[str, Any]) -> "RegupelConfig":
        if not isinstance(raw, Mapping):
            raise TypeError(f"unsupported config type: {type(raw)!r}")
        entries = _need(raw, "layers", "")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for index, entry in enumerate(entries):
            where = f"layers[{index}]"
            kind = _need(entry, "type", where)
            mixer = _need(entry, "mixer", where)
            common = dict(type=kind, mlp=_experts(entry.get("mlp"), f"{where}.mlp"),
                          weights_of=int(entry["weights_of"]) if entry.get("weights_of") is not None else None)
            if kind == "attention":
                layers.append(RegupelLayer(attention=_attention(mixer, f"{where}.mixer"), **common))
            elif kind == "parallel":
                right = _need(mixer, "right", f"{where}.mixer")
                at = f"{where}.mixer.right"
                heads, dim = int(_need(right, "heads", at)), int(_need(right, "dim", at))
                linear = RegupelLinear(heads=heads, dim=dim, vdim=int(right.get("vdim") or dim), decay=tuple(float(d) for d in _need(right, "decay", at)))
                layers.append(RegupelLayer(attention=_attention(_need(mixer, "left", f"{where}.mixer"), f"{where}.mixer.left"), linear=linear,
                                           left_scale=float(mixer.get("left_scale", 1.0)), right_scale=float(mixer.get("right_scale", 1.0)), **common))
            else:
                raise ConfigError(f"{where}: the Regupel design has no mixer {kind!r}")
        config = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                     norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm")),
                     embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)), residual_mult=float(raw.get("residual_mult", 1.0)),
                     logit_scale=float(raw.get("logit_scale", 1.0)), layers=tuple(layers), architecture=str(raw.get("architecture", "Regupel")),
                     raw=dict(raw))
        config.validate()
        return config

    def validate(self) -> None:
        problems: list[str] = []
        if self.vocab <= 0 or self.width <= 0:
            problems.append("vocab and width must be positive")
        if self.norm_eps <= 0.0:
            problems.append("norm.eps must be positive")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            a = layer.attention
            if min(a.heads, a.kv_heads, a.dim, a.vdim) <= 0:
                problems.append(f"{where}: heads, kv_heads, dim and vdim must be positive")
                continue
            if a.heads % a.kv_heads:
                problems.append(f"{where}: heads={a.heads} is not a multiple of kv_heads={a.kv_heads}")
            if a.window is not None and a.window <= 0:
                problems.append(f"{where}: mask.size={a.window} must be positive")
            if a.keep_first < 0 or (a.keep_first and layer.type == "attention"):
                problems.append(f"{where}: mask.keep_first={a.keep_first} (the left mixer of a parallel layer keeps first tokens)")
            if a.rot_dims % 2 or not 0 <= a.rot_dims <= a.dim or (a.rot_dims and layer.type == "parallel"):
                problems.append(f"{where}: rot.dims={a.rot_dims} must be even and at most dim={a.dim}; a parallel layer's left mixer has no rotation")
            if layer.type == "parallel":
                r = layer.linear
                if min(r.heads, r.dim, r.vdim) <= 0 or len(r.decay) != r.heads:
                    problems.append(f"{where}.mixer.right: heads, dim and vdim must be positive, with one decay per head ({len(r.decay)} for {r.heads})")
                elif not all(0.0 <= d <= 1.0 for d in r.decay):
                    problems.append(f"{where}.mixer.right: decays must lie in [0, 1]")
            m = layer.mlp
            if m is not None and (min(m.ff, m.experts, m.top) <= 0 or m.top > m.experts or (m.shared_ff is not None and m.shared_ff <= 0)):
                problems.append(f"{where}.mlp: ff={m.ff}, {m.top} of {m.experts} experts, shared ff={m.shared_ff}")
            if layer.weights_of is not None:
                # a layer may name one that itself runs another's tensors: the owner is where that chain ends
                owner = self.layers[layer.weights_of] if 0 <= layer.weights_of < index else None
                if owner is None:
                    problems.append(f"{where}: weights_of={layer.weights_of} must name an earlier layer")
                elif (owner.type, owner.attention, owner.linear, owner.left_scale, owner.right_scale, owner.mlp) != \
                        (layer.type, layer.attention, layer.linear, layer.left_scale, layer.right_scale, layer.mlp):
                    problems.append(f"{where}: its entry differs from that of layer {layer.weights_of}, whose tensors it uses")
        if problems:
            raise ConfigError("invalid Regupel configuration: " + "; ".join(problems))

    # ------------------------------------------------------------------ export
    @staticmethod
    def _attention_dict(a: RegupelAttention, left: bool) -> dict[str, Any]:
        out: dict[str, Any] = {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "scale": a.scale, "vdim": a.vdim}
        if a.window is not None:
            out["mask"] = {"keep_first": a.keep_first, "size": a.window} if left else {"size": a.window}
        if a.rot_dims:
            rot: dict[str, Any] = {"base": a.rot_base, "dims": a.rot_dims}
            if a.rot_scaling is not None:
                rot["scaling"] = dict(zip(("factor", "low", "high", "original"), a.rot_scaling))
            out["rot"] = rot
        return out

    def to_hf_dict(self) -> dict[str, Any]:
        """The config.json that parses back into this configuration."""
        layers = []
        for layer in self.layers:
            if layer.type == "attention":
                mixer = self._attention_dict(layer.attention, left=False)
            else:
                r = layer.linear
                mixer = {"left": self._attention_dict(layer.attention, left=True), "left_scale": layer.left_scale,
                         "right": {"decay": list(r.decay), "dim": r.dim, "heads": r.heads, "vdim": r.vdim}, "right_scale": layer.right_scale}
            mlp = None
            if layer.mlp is not None:
                mlp = {"expert": {"ff": layer.mlp.ff}, "kind": "moe", "router": {"experts": layer.mlp.experts, "top": layer.mlp.top}}
                if layer.mlp.shared_ff is not None:
                    mlp["shared"] = {"ff": layer.mlp.shared_ff}
            entry: dict[str, Any] = {"mixer": mixer, "mlp": mlp, "type": layer.type}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            layers.append(entry)
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale}, "layers": layers,
                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab,
                "width": self.width}

    # ------------------------------------------------------------------ parts
    def _attention_part(self, a: RegupelAttention, left: bool, init_std: float) -> PartSpec:
        if a.rot_dims == 0:
            position = PartSpec("none")
        else:
            params: dict[str, Any] = {"theta": a.rot_base, "rotary_dim": a.rot_dims, "head_dim": a.dim}
            if a.rot_scaling is not None:
                params.update(zip(("factor", "low", "high", "original"), a.rot_scaling))
            position = PartSpec("rope_wavelength", params)
        common = {"hidden_size": self.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
                  "scale": a.scale, "window": a.window, "qk_norm_eps": self.norm_eps, "position": position, "float_out": True,
                  "float_proj": True, "init_std": init_std, "q": "q", "k": "k", "v": "v", "o": "o", "weight_suffix": ""}
        if left:
            return PartSpec("attention", {**common, "keep_first": a.keep_first, "qk_norm": "whole", "q_norm": "q.norm", "k_norm": "k.norm",
                                          "norm_suffix": ""})
        return PartSpec("attention", {**common, "qk_norm": "unit", "sink": "learned", "sink_name": "sink", "head_gate": True, "g": "g"})

    def model_spec(self) -> ModelSpec:
        init_std = 0.06
        no_norm = PartSpec("none", {"size": self.width})
        # the constant on every sublayer's addition rides on the weight and bias of the norm that the addition passes
        post_norm = PartSpec("layernorm", {"size": self.width, "eps": self.norm_eps, "suffix": "", "bias_suffix": ".b", "scale": self.residual_mult})
        block = PartSpec("sandwich", {"mixer": "mix", "feed_forward": "mlp", "mixer_norm": "unused1", "mixer_post_norm": "norm1",
                                      "feed_forward_norm": "unused2", "feed_forward_post_norm": "norm2"})
        layers, schedule, at = [], [], {}
        for index, layer in enumerate(self.layers):
            if layer.weights_of is not None:
                at[index] = at[layer.weights_of]          # the owner's, also where the named layer runs another's itself
                schedule.append(LayerCall(layer=at[index]))
                continue
            if layer.type == "attention":
                mixer = self._attention_part(layer.attention, False, init_std)
            else:
                r = layer.linear
                right = PartSpec("linear_attention", {"hidden_size": self.width, "num_heads": r.heads, "head_dim": r.dim, "v_head_dim": r.vdim,
                                                      "decay": tuple(r.decay), "eps": self.norm_eps, "activation": "silu", "gate": True,
                                                      "float_out": True, "init_std": init_std, "weight_suffix": ""})
                mixer = PartSpec("side_by_side", {"hidden_size": self.width, "left": self._attention_part(layer.attention, True, init_std),
                                                  "right": right, "left_scale": layer.left_scale, "right_scale": layer.right_scale})
            feed_forward = None
            if layer.mlp is not None:
                m = layer.mlp
                feed_forward = PartSpec("routed_experts", {
                    "hidden_size": self.width, "expert_size": m.ff, "experts": m.experts, "top": m.top, "activation": "silu", "normalize": False,
                    "weight_on": "input", "shared": {"intermediate_size": m.shared_ff} if m.shared_ff is not None else None, "shared_gated": False,
                    "router": "router", "expert": "e{}", "gate": "gate", "up": "up", "down": "down", "shared_name": "shared", "weight_suffix": "",
                    "init_std": init_std, "router_init_std": 0.3})
            at[index] = len(layers)
            layers.append(LayerSpec(prefix=f"l{index}", block=block, mixer=mixer, feed_forward=feed_forward, norm=no_norm,
                                    extra={"post_norm": post_norm}))
            schedule.append(LayerCall(layer=at[index]))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            embedding=PartSpec("token_embedding", {"name": "embed", "scale": self.embedding_scale, "init_std": 0.5}),
            layers=tuple(layers), schedule=tuple(schedule),
            # the logits' constant factor rides on the final norm's weight and bias: the head's product is linear in its input
            final_norm=PartSpec("layernorm", {"size": self.width, "eps": self.norm_eps, "suffix": "", "bias_suffix": ".b", "name": "final.norm",
                                              "scale": self.logit_scale}),
            head=PartSpec("linear_head", {"name": "head", "tied_to": "embed", "init_std": 0.25}),
            max_positions=MAX_POSITIONS, eos_token_ids=(),
        )
        spec.validate()
        return spec
