"""RMSNorm fused with the residual addition that precedes it.

y = x * rsqrt(mean(x^2) + eps) * w in float with one rounding at the end, as in the reference
(qwen_triton/kernels/rmsnorm.py:35-42; module qwen_triton/modules/norms.py:9-21).

Parameters beyond ``size`` and ``eps``: ``groups`` (default 1) splits a row into that many equal consecutive parts,
each divided by its own root mean square, the weight spanning the whole row; ``suffix`` (default ".weight") is what
the weight's tensor name adds to the norm's name.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.kernels import ScaledRows
from ..weights.tensors import TensorSpec
from .base import ResidualStream, Runtime, register_norm, to_device


@register_norm("rmsnorm")
class RMSNorm:
    graph_safe = True

    def __init__(self, params, name: str, runtime: Runtime) -> None:
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.groups = int(params.get("groups", 1))
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"{name}: {self.groups} groups do not divide a width of {self.size}")
        # apply(..., lazy=True) may hand on ScaledRows: one factor per row, so only where the row is one group
        self.offers_scaled_rows = self.groups == 1
        self.tensor = name + str(params.get("suffix", ".weight"))
        self.name = name
        self.runtime = runtime
        self.weight: torch.Tensor | None = None
        runtime.workspace.declare("normed", runtime.max_step_tokens * self.size, runtime.dtype)
        runtime.workspace.declare("normed.sq", -(-self.size // 128) * kernels.FUSED_MAX_ROWS, torch.float32)

    @classmethod
    def expected_tensors(cls, params, name: str) -> dict[str, TensorSpec]:
        return {name + str(params.get("suffix", ".weight")): TensorSpec((int(params["size"]),), role="vector", init_std=0.1, init_mean=1.0)}

    def load(self, source) -> None:
        self.weight = to_device(source(self.tensor), torch.float32, self.runtime.device)

    def apply(self, stream: ResidualStream, rows: torch.Tensor | None = None, lazy: bool = False):
        """Fold the pending delta into the stream and return the normed rows.

        With ``rows`` (int32 row numbers) only those rows are produced and the stream stays as it is.

        Where the pending delta is a product that has not been launched and takes the fused form (few tokens,
        bfloat16), it is launched here with the residual addition in its epilogue.  With ``lazy`` (the consumer is
        a product that takes ``ScaledRows``) the same launch also prepares this norm: it writes the stream times
        the norm's weight and the rows' sums of squares, and the rows' factor is applied by the consumer's
        epilogue; no norm kernel runs.
        """
        ws = self.runtime.workspace
        if stream.more:
            raise RuntimeError(f"{self.name}: this norm folds one pending addition; the stream holds {1 + len(stream.more)}")
        if stream.post is not None:
            raise RuntimeError(f"{self.name}: the pending addition is to pass a norm of its own first, which this norm does not fold")
        deferred = stream.take_deferred()
        if deferred is not None:
            count = stream.residual.shape[0]
            if not deferred.linear.fusable(count):
                stream.pending = deferred.run()
            elif rows is None and lazy and self.offers_scaled_rows:
                xw = ws.view("normed", count, self.size)
                sq = ws.view("normed.sq", -(-self.size // 128), count)
                return deferred.linear.into_residual(deferred.x, stream.residual, self.weight, self.eps, xw, sq)
            else:
                deferred.linear.into_residual(deferred.x, stream.residual)
        count = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = ws.view("normed", count, self.size)
        kernels.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out, rows, self.groups)
        if rows is None:
            stream.pending = None
        return out


@register_norm("dynamic_tanh")
class DynamicTanh:
    """A norm that takes no statistics: y = tanh(alpha * x) * w + b with one number ``alpha`` and vectors w, b.

    Parameters: ``size``; the tensor-name pieces ``suffix`` (weight, default ".weight"), ``bias_suffix`` (".bias") and
    ``alpha_suffix`` (".alpha").  It folds every pending addition of the stream (``folds_several``: a block whose mixer
    and feed-forward read the same rows leaves two), which must be float sums."""

    graph_safe = True
    folds_several = True
    offers_scaled_rows = False

    def __init__(self, params, name: str, runtime: Runtime) -> None:
        self.size = int(params["size"])
        self.name = name
        self.runtime = runtime
        self.tensors = self._tensor_names(params, name)
        self.weight = self.bias = None
        self.alpha = 1.0
        runtime.workspace.declare("normed", runtime.max_step_tokens * self.size, runtime.dtype)

    @staticmethod
    def _tensor_names(params, name: str) -> tuple[str, str, str]:
        return (name + str(params.get("suffix", ".weight")), name + str(params.get("bias_suffix", ".bias")),
                name + str(params.get("alpha_suffix", ".alpha")))

    @classmethod
    def expected_tensors(cls, params, name: str) -> dict[str, TensorSpec]:
        weight, bias, alpha = cls._tensor_names(params, name)
        size = int(params["size"])
        return {weight: TensorSpec((size,), role="vector", init_std=0.1, init_mean=1.0),
                bias: TensorSpec((size,), role="vector", init_std=0.05, init_mean=0.0),
                alpha: TensorSpec((), role="vector", init_std=0.05, init_mean=0.6)}

    def load(self, source) -> None:
        weight, bias, alpha = self.tensors
        self.weight = to_device(source(weight), torch.float32, self.runtime.device)
        self.bias = to_device(source(bias), torch.float32, self.runtime.device)
        self.alpha = float(source(alpha).float().reshape(-1)[0])          # read once, when the model is loaded

    def apply(self, stream: ResidualStream, rows: torch.Tensor | None = None, lazy: bool = False):
        if stream.post is not None:
            raise RuntimeError(f"{self.name}: the pending addition is to pass a norm of its own first, which this norm does not fold")
        deltas = stream.take_all() if rows is None else ([stream.pending] if stream.pending is not None else []) + stream.more
        count = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.workspace.view("normed", count, self.size)
        while len(deltas) > 2:             # the kernel adds two; a third is folded by a pass of its own
            kernels.add_dyt(stream.residual, deltas[:2], self.weight, self.bias, self.alpha, self.runtime.workspace.view(
                "normed", stream.residual.shape[0], self.size))
            if rows is not None:
                raise RuntimeError(f"{self.name}: more than two pending additions while only listed rows are wanted")
            deltas = deltas[2:]
        kernels.add_dyt(stream.residual, deltas, self.weight, self.bias, self.alpha, out, rows)
        return out


@register_norm("layernorm")
class LayerNorm:
    """y = (x - mean) / sqrt(var + eps) * w (+ b) over the row, the variance being the mean of the squared deviations.
    Parameters: ``size``, ``eps``, ``suffix`` (what the weight's tensor name adds to the norm's name, default ".weight"),
    ``bias_suffix`` (the same for a bias; absent: the norm has none) and ``scale`` (default 1): a constant that multiplies
    weight and bias when they are loaded, for a model whose logits are the head's product times a constant (the product
    is linear, so the factor may ride on its input) or whose sublayers are added to the stream times a constant.

    ``folds_post_norm``: where the stream's pending addition is to pass a norm of its own first (``stream.post``, another
    norm of this kind: a layer that norms what a sublayer returns before adding it), the same launch norms the addition,
    adds it and norms the new stream."""

    graph_safe = True
    offers_scaled_rows = False
    folds_post_norm = True

    def __init__(self, params, name: str, runtime: Runtime) -> None:
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.scale = float(params.get("scale", 1.0))
        self.tensor = name + str(params.get("suffix", ".weight"))
        self.bias_tensor = name + str(params["bias_suffix"]) if params.get("bias_suffix") is not None else None
        self.name = name
        self.runtime = runtime
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None
        runtime.workspace.declare("normed", runtime.max_step_tokens * self.size, runtime.dtype)

    @classmethod
    def expected_tensors(cls, params, name: str) -> dict[str, TensorSpec]:
        out = {name + str(params.get("suffix", ".weight")): TensorSpec((int(params["size"]),), role="vector", init_std=0.1, init_mean=1.0)}
        if params.get("bias_suffix") is not None:
            out[name + str(params["bias_suffix"])] = TensorSpec((int(params["size"]),), role="vector", init_std=0.1, init_mean=0.0)
        return out

    def load(self, source) -> None:
        self.weight = to_device(source(self.tensor), torch.float32, self.runtime.device)
        if self.bias_tensor is not None:
            self.bias = to_device(source(self.bias_tensor), torch.float32, self.runtime.device)
        if self.scale != 1.0:
            self.weight = self.weight * self.scale
            self.bias = self.bias * self.scale if self.bias is not None else None

    def apply(self, stream: ResidualStream, rows: torch.Tensor | None = None, lazy: bool = False):
        if stream.more:
            raise RuntimeError(f"{self.name}: this norm folds one pending addition; the stream holds {1 + len(stream.more)}")
        post = stream.post
        if post is not None and not isinstance(post, LayerNorm):
            raise RuntimeError(f"{self.name}: the pending addition's own norm is not a layer norm")
        if post is not None and post.eps != self.eps:
            raise RuntimeError(f"{self.name}: the pending addition's own norm has eps={post.eps}, this one {self.eps}")
        count = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.workspace.view("normed", count, self.size)
        kernels.add_layernorm(stream.residual, stream.pending, post.weight if post is not None else None, self.weight, self.eps, out, rows,
                              post_bias=post.bias if post is not None else None, bias=self.bias)
        if rows is None:
            stream.pending = None
            stream.post = None
        return out


@register_norm("none")
class NoNorm:
    """No norm: a sublayer that reads the stream itself.  ``apply`` folds the pending addition into the stream (after the
    addition's own layer norm where it has one, ``stream.post``: ``folds_post_norm``) and returns the stream's rows in the
    activation type.  Parameter: ``size``.  It has no tensors."""

    graph_safe = True
    offers_scaled_rows = False
    folds_post_norm = True

    def __init__(self, params, name: str, runtime: Runtime) -> None:
        self.size = int(params["size"])
        self.name = name
        self.runtime = runtime
        runtime.workspace.declare("normed", runtime.max_step_tokens * self.size, runtime.dtype)

    @classmethod
    def expected_tensors(cls, params, name: str) -> dict[str, TensorSpec]:
        return {}

    def load(self, source) -> None:
        pass

    def apply(self, stream: ResidualStream, rows: torch.Tensor | None = None, lazy: bool = False):
        if stream.more:
            raise RuntimeError(f"{self.name}: one pending addition is folded here; the stream holds {1 + len(stream.more)}")
        post = stream.post
        if post is not None and not isinstance(post, LayerNorm):
            raise RuntimeError(f"{self.name}: the pending addition's own norm is not a layer norm")
        count = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.workspace.view("normed", count, self.size)
        kernels.add_layernorm(stream.residual, stream.pending, post.weight if post is not None else None, None,
                              post.eps if post is not None else 1e-6, out, rows, post_bias=post.bias if post is not None else None)
        if rows is None:
            stream.pending = None
            stream.post = None
        return out
