"""Typed configuration of the Bisodra design, read from config.json.

The file names its design under ``architecture`` and gives ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``logit_scale`` and a list ``layers``.  An entry has ``type`` (its mixer: ``attention`` or ``latent_attention``), the mixer's
sizes and constants under ``mixer`` and its feed-forward under ``mlp`` (null for none).  Layers need not be alike.

``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim`` (the values are the keys, so it equals ``dim``), ``scale``, ``conv``
(taps of the short convolution on q and k), ``mask.size`` (absent: every earlier token is seen) and ``mask.keep_first``.
``latent_attention``: ``heads``, ``dim`` (unrotated) and ``rot_dim`` (rotated) query/key sizes per head, ``vdim``, ``q_rank``,
``kv_rank``, ``scale``, ``rot.dims`` / ``rot.base`` / ``rot.scaling`` (``factor``, ``original``, ``fast``, ``slow``; absent: plain
rotation) and ``kv_from`` (the layer whose cached latent and rotated key part this one reads instead of making its own).
``mlp``: ``kind`` "dense" with ``ff``.

What the design fixes, and ``model_spec`` therefore states as parameters of the parts: a layer norm with a weight and no
bias before and after each sublayer (x += norm_b(sublayer(norm_a(x)))); in ``attention`` biased q, k and o projections, a
linear distance bias with slopes 2^(-8 (h + 1) / H), a softmax with a sink term of score 0 and a sigmoid gate on the
heads' outputs; in ``latent_attention`` RMS norms on both latents, a rotate-half rotation of the shared key part and of
the rotated query part, causal softmax and the same kind of gate; a feed-forward of two matrices with the exact GELU; the
head is the embedding table (without the embedding's scale) times ``logit_scale``; tensor names ``embed``, ``final.norm``
and ``l<i>.{norm1,norm1b,norm2,norm2b,mix.*,mlp.*}`` without a ``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .qwen3 import ConfigError
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MAX_POSITIONS = 1 << 20          # the design names no longest sequence; the rotation table is made for the cache's length


@dataclass(frozen=True)
class BisodraLayer:
    type: str                       # "attention" or "latent_attention"
    heads: int
    dim: int
    vdim: int
    scale: float
    ff: int | None                  # width of the feed-forward's middle; None: no feed-forward
    # attention
    kv_heads: int = 0
    conv: int = 1
    window: int | None = None       # mask.size
    keep_first: int = 0
    # latent_attention
    rot_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    rot_dims: int = 0               # how many of the rot_dim elements turn
    rot_base: float = 10000.0
    rot_scaling: tuple | None = None   # (factor, original, fast, slow)
    kv_from: int | None = None


def _need(mapping: Mapping[str, Any], key: str, where: str):
    if not isinstance(mapping, Mapping) or mapping.get(key) is None:
        raise ConfigError(f"config.json lacks {where}.{key}" if where else f"config.json lacks the key {key!r}")
    return mapping[key]


@dataclass(frozen=True)
class BisodraConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple[BisodraLayer, ...]
    architecture: str = "Bisodra"
    raw: Mapping[str, Any] = field(default_factory=dict, repr=False, compare=False)

    family = "bisodra"

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
    def from_hf_config(cls, raw: Mapping[str, Any]) -> "BisodraConfig":
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
            at = f"{where}.mixer"
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if _need(mlp, "kind", f"{where}.mlp") != "dense":
                    raise ConfigError(f"{where}.mlp: the Bisodra design has no feed-forward {mlp['kind']!r}")
                ff = int(_need(mlp, "ff", f"{where}.mlp"))
            heads, dim = int(_need(mixer, "heads", at)), int(_need(mixer, "dim", at))
            common = dict(type=kind, heads=heads, dim=dim, vdim=int(mixer.get("vdim") or dim), scale=float(_need(mixer, "scale", at)), ff=ff)
            if kind == "attention":
                mask = mixer.get("mask") or {}
                layers.append(BisodraLayer(**common, kv_heads=int(mixer.get("kv_heads") or heads), conv=int(mixer.get("conv") or 1),
                                           window=int(mask["size"]) if mask.get("size") is not None else None,
                                           keep_first=int(mask.get("keep_first") or 0)))
            elif kind == "latent_attention":
                rot = mixer.get("rot") or {}
                rot_dim = int(mixer.get("rot_dim") or 0)
                scaling = rot.get("scaling")
                if scaling is not None:
                    scaling = tuple(float(_need(scaling, key, f"{at}.rot.scaling")) for key in ("factor", "original", "fast", "slow"))
                layers.append(BisodraLayer(**common, rot_dim=rot_dim, q_rank=int(_need(mixer, "q_rank", at)), kv_rank=int(_need(mixer, "kv_rank", at)),
                                           rot_dims=int(rot["dims"]) if rot.get("dims") is not None else rot_dim,
                                           rot_base=float(rot.get("base", 10000.0)), rot_scaling=scaling,
                                           kv_from=int(mixer["kv_from"]) if mixer.get("kv_from") is not None else None))
            else:
                raise ConfigError(f"{where}: the Bisodra design has no mixer {kind!r}")
        config = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                     norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm")),
                     embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)), logit_scale=float(raw.get("logit_scale", 1.0)),
                     layers=tuple(layers), architecture=str(raw.get("architecture", "Bisodra")), raw=dict(raw))
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
            if min(layer.heads, layer.dim, layer.vdim) <= 0:
                problems.append(f"{where}: heads, dim and vdim must be positive")
                continue
            if layer.ff is not None and layer.ff <= 0:
                problems.append(f"{where}.mlp: ff={layer.ff}")
            if layer.type == "attention":
                if layer.kv_heads <= 0 or layer.heads % layer.kv_heads:
                    problems.append(f"{where}: heads={layer.heads} is not a multiple of kv_heads={layer.kv_heads}")
                if layer.vdim != layer.dim:
                    problems.append(f"{where}: the values are the keys, so vdim={layer.vdim} must equal dim={layer.dim}")
                if not 1 <= layer.conv <= 16:
                    problems.append(f"{where}: conv={layer.conv} taps (1..16)")
                if layer.window is not None and layer.window <= 0:
                    problems.append(f"{where}: mask.size={layer.window} must be positive")
                if layer.keep_first < 0:
                    problems.append(f"{where}: mask.keep_first={layer.keep_first}")
            else:
                if min(layer.q_rank, layer.kv_rank) <= 0 or layer.rot_dim < 0:
                    problems.append(f"{where}: q_rank, kv_rank must be positive and rot_dim not negative")
                if layer.rot_dims % 2 or not 0 <= layer.rot_dims <= layer.rot_dim:
                    problems.append(f"{where}: rot.dims={layer.rot_dims} must be even and at most rot_dim={layer.rot_dim}")
                if layer.kv_from is not None:
                    source = self.layers[layer.kv_from] if 0 <= layer.kv_from < index else None
                    if source is None or source.type != "latent_attention" or source.kv_from is not None:
                        problems.append(f"{where}: kv_from={layer.kv_from} must name an earlier latent_attention layer with a latent of its own")
                    elif (source.kv_rank, source.rot_dim, source.rot_dims, source.rot_base, source.rot_scaling) != \
                            (layer.kv_rank, layer.rot_dim, layer.rot_dims, layer.rot_base, layer.rot_scaling):
                        problems.append(f"{where}: kv_rank, rot_dim or rotation differ from those of layer {layer.kv_from}, whose cache it reads")
        if problems:
            raise ConfigError("invalid Bisodra configuration: " + "; ".join(problems))

    # ------------------------------------------------------------------ export
    def to_hf_dict(self) -> dict[str, Any]:
        """The config.json that parses back into this configuration."""
        layers = []
        for layer in self.layers:
            mixer: dict[str, Any] = {"dim": layer.dim, "heads": layer.heads, "scale": layer.scale, "vdim": layer.vdim}
            if layer.type == "attention":
                mixer.update(conv=layer.conv, kv_heads=layer.kv_heads)
                if layer.window is not None:
                    mixer["mask"] = {"keep_first": layer.keep_first, "size": layer.window}
            else:
                mixer.update(kv_rank=layer.kv_rank, q_rank=layer.q_rank, rot_dim=layer.rot_dim)
                rot: dict[str, Any] = {"base": layer.rot_base, "dims": layer.rot_dims}
                if layer.rot_scaling is not None:
                    rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), layer.rot_scaling))
                mixer["rot"] = rot
                if layer.kv_from is not None:
                    mixer["kv_from"] = layer.kv_from
            layers.append({"mixer": mixer, "mlp": {"ff": layer.ff, "kind": "dense"} if layer.ff is not None else None, "type": layer.type})
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale}, "layers": layers,
                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def model_spec(self) -> ModelSpec:
        norm_params = {"size": self.width, "eps": self.norm_eps, "suffix": ""}
        norm = PartSpec("layernorm", norm_params)
        block = PartSpec("sandwich", {"mixer": "mix", "feed_forward": "mlp", "mixer_norm": "norm1", "mixer_post_norm": "norm1b",
                                      "feed_forward_norm": "norm2", "feed_forward_post_norm": "norm2b"})
        init_std = 0.06
        layers, schedule = [], []
        for index, layer in enumerate(self.layers):
            if layer.type == "attention":
                mixer = PartSpec("conv_attention", {
                    "hidden_size": self.width, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads, "head_dim": layer.dim,
                    "scale": layer.scale, "conv": layer.conv, "window": layer.window, "keep_first": layer.keep_first, "sink": True,
                    "gate": True, "bias": True, "slope_bits": 8.0, "float_out": True, "init_std": init_std,
                    "q": "q", "k": "k", "g": "g", "o": "o", "weight_suffix": "", "bias_suffix": ".b", "conv_suffix": ".conv"})
            else:
                if layer.rot_dims == 0:
                    position = PartSpec("none")
                elif layer.rot_scaling is not None:
                    factor, original, fast, slow = layer.rot_scaling
                    position = PartSpec("rope_yarn", {"theta": layer.rot_base, "rotary_dim": layer.rot_dims, "head_dim": layer.rot_dim,
                                                      "factor": factor, "original": original, "fast": fast, "slow": slow})
                else:
                    position = PartSpec("rope", {"theta": layer.rot_base, "rotary_dim": layer.rot_dims, "head_dim": layer.rot_dim,
                                                 "angles": "float64"})
                mixer = PartSpec("latent_attention", {
                    "hidden_size": self.width, "num_heads": layer.heads, "head_dim": layer.dim, "rot_dim": layer.rot_dim,
                    "v_head_dim": layer.vdim, "q_rank": layer.q_rank, "kv_rank": layer.kv_rank, "scale": layer.scale, "eps": self.norm_eps,
                    "position": position, "own_kv": layer.kv_from is None, "gate": True, "float_out": True, "init_std": init_std,
                    "dq": "dq", "uq": "uq", "dkv": "dkv", "uk": "uk", "uv": "uv", "g": "g", "o": "o", "weight_suffix": "", "norm_suffix": ".norm"})
            feed_forward = None
            if layer.ff is not None:
                feed_forward = PartSpec("plain_mlp", {"hidden_size": self.width, "intermediate_size": layer.ff, "activation": "gelu",
                                                      "up": "up", "down": "down", "weight_suffix": "", "float_out": True, "init_std": init_std})
            layers.append(LayerSpec(prefix=f"l{index}", block=block, mixer=mixer, feed_forward=feed_forward, norm=norm))
            schedule.append(LayerCall(layer=index, cache_of=layer.kv_from))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            embedding=PartSpec("token_embedding", {"name": "embed", "scale": self.embedding_scale, "init_std": 0.5}),
            layers=tuple(layers), schedule=tuple(schedule),
            # the logits' constant factor rides on the final norm's weight: the head's product is linear in its input
            final_norm=PartSpec("layernorm", {**norm_params, "name": "final.norm", "scale": self.logit_scale}),
            head=PartSpec("linear_head", {"name": "head", "tied_to": "embed", "init_std": 0.25}),
            max_positions=MAX_POSITIONS, eos_token_ids=(),
        )
        spec.validate()
        return spec
