"""A recurrent mixer: the gated delta rule with one decay per head and key channel.

Per head a float state S [dim, vdim] is carried from token to token of a sequence:

    S <- diag(g_t) S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t

where o_t is read after token t has been written.  Around it:

* q = W_q h and k = W_k h ([kv_heads, dim]; head h reads kv head h // (heads / kv_heads)), v = W_v h ([heads, vdim]);
  each passes a short causal convolution per channel (``conv`` taps, the last one the current token's, zeros before
  the sequence's start) and SiLU; q and k are then made unit vectors per head, x / sqrt(sum x^2 + 1e-6), q also
  times dim^-1/2;
* beta = sigmoid(W_b h), one per head;
* g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 h) + dt_bias)), [heads, dim]: a projection through few columns (the
  kernels pass its logarithm on);
* every head's o is divided by its root mean square over vdim (``eps`` inside the root), times a weight [vdim] shared
  by the heads, times sigmoid(W_g2 (W_g1 h)) ([heads, vdim]); then W_o.

Per sequence the mixer keeps two things, both float, both in the cache's per-slot state (zero for a new sequence):
the states S [heads, dim, vdim] and the last ``conv`` - 1 inputs of the convolutions.  The six projections of h run as
one product with float sums; everything between it and the output projection is float (``csrc/delta_rule.cu``).

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``v_head_dim``, ``conv``, ``eps``,
``decay_rank`` and ``gate_rank`` (columns of the two narrow projections; read from the tensors' shapes by the
configuration), ``float_out``, ``init_std``, and the tensor names (``q``, ``k``, ``v``, ``beta``, ``decay_in``,
``decay_out``, ``decay_bias``, ``decay_rate``, ``gate_in``, ``gate_out``, ``norm``, ``o``, ``conv_suffix``,
``weight_suffix``).
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..weights.tensors import TensorSpec
from .base import DeferredProduct, Runtime, StateRequest, register_mixer, to_device
from .linear import Linear

_UNIT_EPS = 1e-6      # inside the root of the unit norms of q and k
_FEW_TOKENS = 4       # steps in which no sequence brings more tokens run the recurrence token by token


@register_mixer("gated_delta_rule")
class GatedDeltaRule:
    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.params = dict(params)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.kv_heads = int(params.get("num_kv_heads") or self.heads)
        self.dim = int(params["head_dim"])
        self.vdim = int(params.get("v_head_dim") or self.dim)
        self.taps = int(params.get("conv", 1))
        self.eps = float(params.get("eps", 1e-6))
        self.decay_rank = int(params["decay_rank"])
        self.gate_rank = int(params["gate_rank"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{prefix}: {self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"{prefix}: a convolution of {self.taps} taps (1..16)")
        if self.dim > 512:
            raise ValueError(f"{prefix}: {self.dim} key channels per head are beyond what the recurrence kernel holds (512)")
        self.channels = 2 * self.kv_heads * self.dim + self.heads * self.vdim
        # columns of the first product: q | k | v | beta | decay_in | gate_in, padded to a multiple of 8
        self.at_decay = self.channels + self.heads
        self.at_gate = self.at_decay + self.decay_rank
        used = self.at_gate + self.gate_rank
        self.proj_rows = -(-used // 8) * 8
        self.proj = Linear("delta.proj", self.proj_rows, self.hidden, runtime, float_out=True)
        float_out = bool(params.get("float_out", False))
        self.o = Linear("delta.o" + (".float" if float_out else ""), self.hidden, self.heads * self.vdim, runtime, float_out=float_out, role="attn_out")
        ws = runtime.workspace
        tokens = runtime.max_step_tokens
        for name, width in (("delta.q", self.kv_heads * self.dim), ("delta.k", self.kv_heads * self.dim), ("delta.v", self.heads * self.vdim),
                            ("delta.beta", self.heads), ("delta.decay", self.heads * self.dim), ("delta.gate", self.heads * self.vdim),
                            ("delta.read", self.heads * self.vdim)):
            ws.declare(name, tokens * width, torch.float32)
        ws.declare("delta.normed", tokens * self.heads * self.vdim, runtime.dtype)
        ws.declare("delta.chunks", tokens * self.heads * (4 * self.dim + 2 * kernels.DELTA_CHUNK + 4), torch.float32)
        self.conv = self.decay_out = self.decay_bias = self.decay_rate = self.gate_out = self.norm = None

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _names(params, prefix: str) -> dict[str, str]:
        w = str(params.get("weight_suffix", ".weight"))
        conv = str(params.get("conv_suffix", ".conv"))
        defaults = {"q": "q", "k": "k", "v": "v", "beta": "beta", "decay_in": "decay_in", "decay_out": "decay_out", "gate_in": "gate_in",
                    "gate_out": "gate_out", "o": "o"}
        n = {key: f"{prefix}.{params.get(key, default)}{w}" for key, default in defaults.items()}
        for key in ("q", "k", "v"):
            n[key + "_conv"] = f"{prefix}.{params.get(key, key)}{conv}"
        for key, default in (("decay_bias", "decay_bias"), ("decay_rate", "decay_rate"), ("norm", "norm")):
            n[key] = f"{prefix}.{params.get(key, default)}"
        return n

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, heads, dim = int(params["hidden_size"]), int(params["num_heads"]), int(params["head_dim"])
        kv_heads, vdim, taps = int(params.get("num_kv_heads") or heads), int(params.get("v_head_dim") or dim), int(params.get("conv", 1))
        ra, rg = int(params["decay_rank"]), int(params["gate_rank"])
        n = cls._names(params, prefix)
        std = float(params.get("init_std", 0.02))
        narrow = float(params.get("narrow_init_std", 0.2))
        out = {n["q"]: TensorSpec((kv_heads * dim, hidden), init_std=std), n["k"]: TensorSpec((kv_heads * dim, hidden), init_std=std),
               n["v"]: TensorSpec((heads * vdim, hidden), init_std=std), n["beta"]: TensorSpec((heads, hidden), init_std=std),
               n["decay_in"]: TensorSpec((ra, hidden), init_std=std), n["decay_out"]: TensorSpec((heads * dim, ra), init_std=narrow),
               n["gate_in"]: TensorSpec((rg, hidden), init_std=std), n["gate_out"]: TensorSpec((heads * vdim, rg), init_std=narrow),
               n["o"]: TensorSpec((hidden, heads * vdim), init_std=std),
               n["decay_bias"]: TensorSpec((heads * dim,), role="vector", init_std=0.5, init_mean=-3.0),
               n["decay_rate"]: TensorSpec((heads,), role="vector", init_std=0.3, init_mean=0.0),
               n["norm"]: TensorSpec((vdim,), role="vector", init_std=0.1, init_mean=1.0)}
        # a convolution of one tap is a factor per channel; a model may leave such tensors out (all ones)
        for key, channels in (("q_conv", kv_heads * dim), ("k_conv", kv_heads * dim), ("v_conv", heads * vdim)):
            out[n[key]] = TensorSpec((channels, taps), role="vector", init_std=0.3, init_mean=0.3, optional=taps == 1)
        return out

    def load(self, source) -> None:
        n = self._names(self.params, self.prefix)
        dtype, device = self.runtime.dtype, self.runtime.device
        rows = [source(n[key]).to(dtype) for key in ("q", "k", "v", "beta", "decay_in", "gate_in")]
        used = sum(r.shape[0] for r in rows)
        if self.proj_rows > used:
            rows.append(torch.zeros(self.proj_rows - used, self.hidden, dtype=dtype, device=rows[0].device))
        self.proj.set_weight(torch.cat(rows, dim=0))
        self.o.set_weight(source(n["o"]))
        pieces = []
        for key, channels in (("q", self.kv_heads * self.dim), ("k", self.kv_heads * self.dim), ("v", self.heads * self.vdim)):
            stored = source(n[key + "_conv"])
            pieces.append(stored.float().cpu() if stored is not None else torch.ones(channels, self.taps))
        conv = torch.cat(pieces, dim=0)
        self.conv = to_device(conv, torch.float32, device)
        # the narrow projections' second matrices: float, transposed to [rank, N] so that neighbouring threads read neighbouring outputs
        self.decay_out = to_device(source(n["decay_out"]).float().t(), torch.float32, device)
        self.gate_out = to_device(source(n["gate_out"]).float().t(), torch.float32, device)
        self.decay_bias = to_device(source(n["decay_bias"]), torch.float32, device)
        self.decay_rate = to_device(source(n["decay_rate"]), torch.float32, device)
        self.norm = to_device(source(n["norm"]), torch.float32, device)

    # ------------------------------------------------------------------ what it keeps per sequence
    def cache_request(self):
        return [StateRequest((self.heads, self.dim, self.vdim), torch.float32),
                StateRequest((max(self.taps - 1, 1), self.channels), torch.float32)]

    # ------------------------------------------------------------------ run
    def forward(self, x, ctx, cache):
        states, kept = cache
        if not states.writable:
            raise ValueError(f"{self.prefix}: a recurrent mixer cannot read another layer's state")
        tokens = x.shape[0]
        ws = self.runtime.workspace
        proj = self.proj(x)
        q = ws.view("delta.q", tokens, self.kv_heads, self.dim)
        k = ws.view("delta.k", tokens, self.kv_heads, self.dim)
        v = ws.view("delta.v", tokens, self.heads, self.vdim)
        beta = ws.view("delta.beta", tokens, self.heads)
        decay = ws.view("delta.decay", tokens, self.heads, self.dim)
        gate = ws.view("delta.gate", tokens, self.heads, self.vdim)
        read = ws.view("delta.read", tokens, self.heads, self.vdim)
        kept_rows = kept.state if self.taps > 1 else kept.state[:, :0]
        kernels.delta_prepare(proj, self.conv, kept_rows, ctx, q, k, v, beta, self.heads, self.kv_heads, self.dim, self.vdim, _UNIT_EPS)
        kernels.lowrank(proj, self.at_decay, self.decay_out, decay.view(tokens, self.heads * self.dim), self.decay_bias, self.decay_rate, self.dim)
        kernels.lowrank(proj, self.at_gate, self.gate_out, gate.view(tokens, self.heads * self.vdim))
        if ctx.max_q_len > _FEW_TOKENS and self.dim <= kernels.DELTA_CHUNKED_MAX_DIM:
            kernels.delta_scan_chunked(q, k, v, beta, decay, states.state, read,
                                       ws.view("delta.chunks", tokens * self.heads * (4 * self.dim + 2 * kernels.DELTA_CHUNK + 4)), ctx)
        else:
            kernels.delta_scan(q, k, v, beta, decay, states.state, read, ctx)
        normed = ws.view("delta.normed", tokens, self.heads, self.vdim)
        kernels.gated_head_norm(read, gate, self.norm, self.eps, normed)
        normed = normed.view(tokens, self.heads * self.vdim)
        # few tokens: the product is left to the block, which launches it with the residual addition in its epilogue
        return DeferredProduct(self.o, normed) if self.o.fusable(tokens) else self.o(normed)


@register_mixer("linear_attention")
class LinearAttention:
    """Linear attention with a constant decay per head ("lightning attention"):

        S <- decay_h S + k_t v_t^T;   o_t = S^T q_t

    with q = act(W_q h), k = act(W_k h) ([heads, dim]) and v = act(W_v h) ([heads, vdim]), act = SiLU (``activation``: "silu"
    or "none"), no other scale.  The heads' outputs of a token are RMS-normed together (one mean over all heads x vdim
    elements, ``eps`` inside the root) with a weight of that size, multiplied by sigmoid(W_g h) (``gate``) and projected by
    W_o.  Per sequence the mixer keeps the states, float, zero for a new sequence, in the cache's per-slot state rows
    (stored transposed, [heads, vdim, dim]).  The four projections of h run as one product with float sums; SiLU, the
    recurrence, the norm and the gate are float (``csrc/linear_attention.cu``).

    Parameters: ``hidden_size``, ``num_heads``, ``head_dim``, ``v_head_dim``, ``decay`` (one number per head), ``eps``,
    ``activation``, ``gate``, ``float_out``, ``init_std``, and the tensor-name pieces ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``,
    ``weight_suffix``."""

    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix, self.runtime, self.params = prefix, runtime, dict(params)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.dim = int(params["head_dim"])
        self.vdim = int(params.get("v_head_dim") or self.dim)
        self.eps = float(params.get("eps", 1e-6))
        self.gated = bool(params.get("gate", True))
        activation = params.get("activation", "silu")
        if activation not in ("silu", "none"):
            raise ValueError(f"{prefix}: activation {activation!r} on q, k and v (silu or none)")
        self.act = activation == "silu"
        decay = [float(d) for d in params["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"{prefix}: {len(decay)} decays for {self.heads} heads")
        if self.dim > kernels.LINEAR_ATTENTION_MAX_DIM:
            raise ValueError(f"{prefix}: {self.dim} key channels per head are beyond what the recurrence kernel holds "
                             f"({kernels.LINEAR_ATTENTION_MAX_DIM})")
        self.decay_values = decay
        self.decay = None
        self.at_k = self.heads * self.dim
        self.at_v = 2 * self.heads * self.dim
        self.at_gate = self.at_v + self.heads * self.vdim
        used = self.at_gate + (self.heads * self.vdim if self.gated else 0)
        self.proj_rows = -(-used // 8) * 8
        self.proj = Linear("linattn.proj", self.proj_rows, self.hidden, runtime, float_out=True)
        float_out = bool(params.get("float_out", False))
        self.o = Linear("linattn.o" + (".float" if float_out else ""), self.hidden, self.heads * self.vdim, runtime, float_out=float_out, role="attn_out")
        ws = runtime.workspace
        ws.declare("linattn.read", runtime.max_step_tokens * self.heads * self.vdim, torch.float32)
        ws.declare("linattn.qkv", runtime.max_step_tokens * self.at_gate, torch.float32)
        ws.declare("linattn.normed", runtime.max_step_tokens * self.heads * self.vdim, runtime.dtype)
        self.norm = None

    @staticmethod
    def _names(params, prefix: str) -> dict[str, str]:
        w = str(params.get("weight_suffix", ".weight"))
        n = {key: f"{prefix}.{params.get(key, key)}{w}" for key in ("q", "k", "v", "g", "o")}
        n["norm"] = f"{prefix}.{params.get('norm', 'norm')}"
        return n

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, heads, dim = int(params["hidden_size"]), int(params["num_heads"]), int(params["head_dim"])
        vdim = int(params.get("v_head_dim") or dim)
        n = cls._names(params, prefix)
        std = float(params.get("init_std", 0.02))
        out = {n["q"]: TensorSpec((heads * dim, hidden), init_std=std), n["k"]: TensorSpec((heads * dim, hidden), init_std=std),
               n["v"]: TensorSpec((heads * vdim, hidden), init_std=std), n["o"]: TensorSpec((hidden, heads * vdim), init_std=std),
               n["norm"]: TensorSpec((heads * vdim,), role="vector", init_std=0.1, init_mean=1.0)}
        if params.get("gate", True):
            out[n["g"]] = TensorSpec((heads * vdim, hidden), init_std=std)
        return out

    def load(self, source) -> None:
        n = self._names(self.params, self.prefix)
        dtype, device = self.runtime.dtype, self.runtime.device
        rows = [source(n[key]).to(dtype) for key in (("q", "k", "v", "g") if self.gated else ("q", "k", "v"))]
        used = sum(r.shape[0] for r in rows)
        if self.proj_rows > used:
            rows.append(torch.zeros(self.proj_rows - used, self.hidden, dtype=dtype, device=rows[0].device))
        self.proj.set_weight(torch.cat(rows, dim=0))
        self.o.set_weight(source(n["o"]))
        self.norm = to_device(source(n["norm"]), torch.float32, device)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)

    def cache_request(self):
        return StateRequest((self.heads, self.vdim, self.dim), torch.float32)

    def forward(self, x, ctx, cache):
        if not cache.writable:
            raise ValueError(f"{self.prefix}: a recurrent mixer cannot read another layer's state")
        tokens = x.shape[0]
        ws = self.runtime.workspace
        proj = self.proj(x)
        read = ws.view("linattn.read", tokens, self.heads, self.vdim)
        # q, k and v are summed and activated once, not by every block of the recurrence that reads them
        ready = kernels.linear_attention_prepare(proj, self.at_gate, ws.view("linattn.qkv", tokens, self.at_gate), self.act)
        kernels.linear_attention_scan(ready, 0, self.at_k, self.at_v, self.decay, cache.state, read, ctx, self.dim, False)
        normed = ws.view("linattn.normed", tokens, self.heads * self.vdim)
        kernels.linear_attention_gate_norm(read.view(tokens, self.heads * self.vdim), proj if self.gated else None, self.at_gate, self.norm,
                                           self.eps, 1.0, normed)
        return self.o(normed)
