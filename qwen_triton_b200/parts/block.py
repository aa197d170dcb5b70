"""Arrangements of norm, mixer and feed-forward around the residual stream.

``pre_norm``: h += mixer(norm(h)); h += feed_forward(norm(h)) (qwen_triton/models/core.py:126-152).
Each addition is left pending on the stream and folded in by the next norm kernel.  A layer whose
``feed_forward`` is None has the first half only; a weight stored for the norm of the missing half is read past.
"""
from __future__ import annotations

from dataclasses import replace

from ..config.spec import LayerSpec
from ..weights.tensors import TensorSpec
from .base import DeferredProduct, ResidualStream, Runtime, part_class, register_block


@register_block("pre_norm")
class PreNormBlock:
    def __init__(self, layer: LayerSpec, runtime: Runtime) -> None:
        names = self._names(layer)
        norms = self._norm_specs(layer)
        self.mixer_norm = part_class("norm", norms[0])(norms[0].params, names["mixer_norm"], runtime)
        self.mixer = part_class("mixer", layer.mixer)(layer.mixer.params, names["mixer"], runtime)
        self.feed_forward_norm = self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = part_class("norm", norms[1])(norms[1].params, names["feed_forward_norm"], runtime)
            self.feed_forward = part_class("feed_forward", layer.feed_forward)(layer.feed_forward.params,
                                                                               names["feed_forward"], runtime)

    @staticmethod
    def _names(layer: LayerSpec) -> dict[str, str]:
        p = layer.block.params
        return {key: f"{layer.prefix}.{p.get(key, key)}" for key in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")}

    @staticmethod
    def _norm_specs(layer: LayerSpec):
        """The norm in front of the mixer and the one in front of the feed-forward: ``layer.norm`` for both unless
        ``layer.extra`` names another kind for one of them."""
        return layer.extra.get("mixer_norm", layer.norm), layer.extra.get("feed_forward_norm", layer.norm)

    @classmethod
    def expected_tensors(cls, layer: LayerSpec) -> dict[str, TensorSpec]:
        names = cls._names(layer)
        out: dict[str, TensorSpec] = {}
        norms = cls._norm_specs(layer)
        out.update(part_class("norm", norms[0]).expected_tensors(norms[0].params, names["mixer_norm"]))
        second = part_class("norm", norms[1]).expected_tensors(norms[1].params, names["feed_forward_norm"])
        out.update(part_class("mixer", layer.mixer).expected_tensors(layer.mixer.params, names["mixer"]))
        if layer.feed_forward is None:
            out.update({name: replace(spec, optional=True) for name, spec in second.items()})
            return out
        out.update(second)
        out.update(part_class("feed_forward", layer.feed_forward).expected_tensors(layer.feed_forward.params,
                                                                                   names["feed_forward"]))
        return out

    def cache_requests(self):
        """What this block keeps per sequence: its mixer's request.  (A block with several such parts returns a
        list, and its ``forward`` then gets a tuple of cache views in the same order.)"""
        return self.mixer.cache_request()

    def parts(self) -> tuple:
        """The parts this block runs in a step."""
        return tuple(part for part in (self.mixer_norm, self.feed_forward_norm, self.mixer, self.feed_forward) if part is not None)

    @property
    def graph_safe(self) -> bool:
        """True if a one-token step through this block only launches kernels (every part says so of itself)."""
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def load(self, source) -> None:
        for part in self.parts():
            part.load(source)

    @staticmethod
    def _normed(norm, stream: ResidualStream, consumer):
        """The consumer's input: ``ScaledRows`` where the norm offers them and the consumer takes them."""
        if getattr(norm, "offers_scaled_rows", False) and getattr(consumer, "takes_scaled_rows", False):
            return norm.apply(stream, lazy=True)
        return norm.apply(stream)

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self._normed(self.mixer_norm, stream, self.mixer)
        stream.add(self.mixer.forward(x, ctx, cache))
        if self.feed_forward is None:
            return
        x = self._normed(self.feed_forward_norm, stream, self.feed_forward)
        stream.add(self.feed_forward.forward(x, ctx))


@register_block("sandwich")
class SandwichBlock(PreNormBlock):
    """A norm before and after each sublayer: h += post1(mixer(norm1(h))); h += post2(feed_forward(norm2(h))).

    What a sublayer returns is left pending on the stream together with the norm it is to pass (``stream.add(...,
    post=)``); the next norm in front of a sublayer (or the model's final norm) folds both, so it must be one that says
    ``folds_post_norm``.  The tensors of the two further norms are named by the block parameters ``mixer_post_norm`` and
    ``feed_forward_post_norm``."""

    def __init__(self, layer: LayerSpec, runtime: Runtime) -> None:
        super().__init__(layer, runtime)
        names = self._post_names(layer)
        norm = layer.extra.get("post_norm", layer.norm)
        self.mixer_post_norm = part_class("norm", norm)(norm.params, names[0], runtime)
        self.feed_forward_post_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_post_norm = part_class("norm", norm)(norm.params, names[1], runtime)
        for part in (self.mixer_norm, self.feed_forward_norm):
            if part is not None and not getattr(part, "folds_post_norm", False):
                raise ValueError(f"{layer.prefix}: a sandwich block needs norms that fold an addition's own norm")

    @staticmethod
    def _post_names(layer: LayerSpec) -> tuple[str, str]:
        p = layer.block.params
        return (f"{layer.prefix}.{p.get('mixer_post_norm', 'mixer_post_norm')}",
                f"{layer.prefix}.{p.get('feed_forward_post_norm', 'feed_forward_post_norm')}")

    @classmethod
    def expected_tensors(cls, layer: LayerSpec) -> dict[str, TensorSpec]:
        out = super().expected_tensors(layer)
        names = cls._post_names(layer)
        norm = layer.extra.get("post_norm", layer.norm)
        out.update(part_class("norm", norm).expected_tensors(norm.params, names[0]))
        second = part_class("norm", norm).expected_tensors(norm.params, names[1])
        if layer.feed_forward is None:
            second = {name: replace(spec, optional=True) for name, spec in second.items()}
        out.update(second)
        return out

    def parts(self) -> tuple:
        return super().parts() + tuple(part for part in (self.mixer_post_norm, self.feed_forward_post_norm) if part is not None)

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self.mixer_norm.apply(stream)
        result = self.mixer.forward(x, ctx, cache)
        stream.add(result.run() if isinstance(result, DeferredProduct) else result, post=self.mixer_post_norm)
        if self.feed_forward is None:
            return
        x = self.feed_forward_norm.apply(stream)
        result = self.feed_forward.forward(x, ctx)
        stream.add(result.run() if isinstance(result, DeferredProduct) else result, post=self.feed_forward_post_norm)


@register_block("parallel")
class ParallelBlock(PreNormBlock):
    """One norm, read by the mixer and by the feed-forward alike: h = norm(x); x += mixer(h) + feed_forward(h).

    Both results are left pending on the stream, side by side; the next norm (one that ``folds_several``) adds them
    in one pass.  The norm's tensors are named by the block parameter ``mixer_norm``; there is no second norm."""

    def __init__(self, layer: LayerSpec, runtime: Runtime) -> None:
        names = self._names(layer)
        norm = self._norm_specs(layer)[0]
        self.mixer_norm = part_class("norm", norm)(norm.params, names["mixer_norm"], runtime)
        if not getattr(self.mixer_norm, "folds_several", False) and layer.feed_forward is not None:
            raise ValueError(f"{layer.prefix}: a parallel block needs a norm that folds several pending additions")
        self.mixer = part_class("mixer", layer.mixer)(layer.mixer.params, names["mixer"], runtime)
        self.feed_forward_norm = None
        self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward = part_class("feed_forward", layer.feed_forward)(layer.feed_forward.params, names["feed_forward"], runtime)

    @classmethod
    def expected_tensors(cls, layer: LayerSpec) -> dict[str, TensorSpec]:
        names = cls._names(layer)
        norm = cls._norm_specs(layer)[0]
        out: dict[str, TensorSpec] = {}
        out.update(part_class("norm", norm).expected_tensors(norm.params, names["mixer_norm"]))
        out.update(part_class("mixer", layer.mixer).expected_tensors(layer.mixer.params, names["mixer"]))
        if layer.feed_forward is not None:
            out.update(part_class("feed_forward", layer.feed_forward).expected_tensors(layer.feed_forward.params, names["feed_forward"]))
        return out

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self.mixer_norm.apply(stream)
        for part, args in ((self.mixer, (x, ctx, cache)), (self.feed_forward, (x, ctx))):
            if part is None:
                continue
            result = part.forward(*args)
            if isinstance(result, DeferredProduct):
                # few tokens: the part's last product adds itself to the float stream in its epilogue (nothing else
                # reads the stream until the next norm; the other part reads the normed rows)
                if result.linear.fusable(stream.residual.shape[0]):
                    result.linear.into_residual(result.x, stream.residual)
                    continue
                result = result.run()
            stream.add_beside(result)
