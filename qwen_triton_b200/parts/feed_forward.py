"""Dense gated feed-forward: down(act(gate(x)) * up(x)) (qwen_triton/modules/mlp.py:10-22, where act is SiLU;
here it is a parameter: any of ``kernels.ACTIVATIONS``, or ``kernels.CAPPED_GATE`` with ``limit``:
g' = min(g, limit), u' = clamp(u, -limit, limit), y = g' sigmoid(1.702 g') (u' + 1), computed by the gate kernel
in the same places as the other activations: the products' epilogues, or the gate kernel).  ``weight_suffix`` is what the tensor names add to the projections' names (default
".weight"); ``float_out`` makes the down projection hand on float sums.

gate and up run as one product over the fused weight [gate; up].  In bfloat16 its rows alternate 16 of gate and
16 of up, so that the GEMM for many tokens can apply the SiLU gate in its epilogue (one warp then holds both halves
of 16 features) and write the activation directly; few tokens take the split-K product and the separate kernel,
which reads the same layout.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.kernels import GemmOut
from ..weights.tensors import TensorSpec
from .base import DeferredProduct, Runtime, register_feed_forward, to_device
from .linear import Linear


@register_feed_forward("gated_mlp")
class GatedMLP:
    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params.get("activation", "silu")
        self.capped = self.activation == kernels.CAPPED_GATE
        self.limit = float(params.get("limit", 0.0))
        if self.activation not in kernels.ACTIVATIONS and not self.capped:
            raise ValueError(f"{prefix}: gate activation {self.activation!r} is not one of {sorted(kernels.ACTIVATIONS) + [kernels.CAPPED_GATE]}")
        if self.capped and self.limit <= 0.0:
            raise ValueError(f"{prefix}: the capped gate needs a positive limit")
        self.names = self._names(params)
        # the gate in a product's epilogue: its rows then alternate 16 of gate and 16 of up
        fused = runtime.dtype == torch.bfloat16 and self.inter % kernels.SWIGLU_GROUP == 0 and self.hidden % 8 == 0
        self.group = kernels.SWIGLU_GROUP if fused else 0
        float_out = bool(params.get("float_out", False))
        key = str(params.get("buffers", "mlp"))           # several such parts in one layer keep their buffers apart
        self.gate_up = Linear(f"{key}.gate_up", 2 * self.inter, self.hidden, runtime, role="gate" if fused else "")
        self.down = Linear(f"{key}.down" + (".float" if float_out else ""), self.hidden, self.inter, runtime,
                           role="mlp_out", float_out=float_out)
        self.act_buffer = f"{key}.act"
        runtime.workspace.declare(self.act_buffer, runtime.max_step_tokens * self.inter, runtime.dtype)
        # few tokens: the gate in the epilogue of the gate/up product, which then also applies the factor of the norm
        # in front of it (``ScaledRows``)
        self.takes_scaled_rows = bool(self.group) and self.gate_up.fused_capable

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, inter = int(params["hidden_size"]), int(params["intermediate_size"])
        n = cls._names(params)
        std = float(params.get("init_std", 0.02))
        return {f"{prefix}.{n['gate']}": TensorSpec((inter, hidden), init_std=std),
                f"{prefix}.{n['up']}": TensorSpec((inter, hidden), init_std=std),
                f"{prefix}.{n['down']}": TensorSpec((hidden, inter), init_std=std)}

    @staticmethod
    def _names(params) -> dict[str, str]:
        suffix = str(params.get("weight_suffix", ".weight"))
        return {k: params.get(k, f"{k}_proj") + suffix for k in ("gate", "up", "down")}

    def load(self, source) -> None:
        n, p = self.names, self.prefix
        gate, up = source(f"{p}.{n['gate']}"), source(f"{p}.{n['up']}")
        self.gate_up.set_weight(kernels.interleave_gate_up(gate.to(self.runtime.dtype), up.to(self.runtime.dtype), self.group))
        self.down.set_weight(source(f"{p}.{n['down']}"))

    def forward(self, x, ctx):
        tokens = x.shape[0]
        act = self.runtime.workspace.view(self.act_buffer, tokens, self.inter)
        if self.takes_scaled_rows and self.gate_up.fusable(tokens):
            self.gate_up.into_swiglu(x, act, self.activation, self.limit)
        elif self.group and kernels.gemm_uses_pairs(x, self.gate_up.weight):
            kernels.gemm_tc_pair(x, self.gate_up.weight, GemmOut(act.view(1, tokens, self.inter)), swiglu=True, activation=self.activation,
                                 limit=self.limit)
        elif self.group and kernels.gemm_tc_supported(x, self.gate_up.weight) and self.gate_up.plan_splits(tokens) == 1:
            # a weight whose tiles fill the machine unsplit: the gate in the plain product's epilogue
            kernels.gemm_tc(x, self.gate_up.weight, GemmOut(act.view(1, tokens, self.inter)), swiglu=True, activation=self.activation,
                            limit=self.limit)
        else:
            kernels.swiglu(self.gate_up(x), act, self.group, self.activation, self.limit)
        # few tokens: the down projection is left to the norm behind it, which launches it with the residual addition
        # (and its own preparation) in the product's epilogue
        return DeferredProduct(self.down, act) if self.down.fusable(tokens) else self.down(act)


@register_feed_forward("plain_mlp")
class PlainMLP:
    """A feed-forward of two matrices with an activation between them and no gate: down(act(up(x))).

    Parameters: ``hidden_size``, ``intermediate_size``, ``activation`` (one of ``kernels.ACTIVATIONS``, default the exact
    GELU), the tensor-name pieces ``up``, ``down``, ``weight_suffix`` (default ".weight"), ``float_out`` (the down
    projection hands on float sums) and ``buffers``.  The activation is taken on the up product's sums in float."""

    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params.get("activation", "gelu")
        if self.activation not in kernels.ACTIVATIONS:
            raise ValueError(f"{prefix}: activation {self.activation!r} is not one of {sorted(kernels.ACTIVATIONS)}")
        self.names = self._names(params)
        float_out = bool(params.get("float_out", False))
        key = str(params.get("buffers", "mlp"))
        self.up = Linear(f"{key}.up.plain", self.inter, self.hidden, runtime)
        self.down = Linear(f"{key}.down" + (".float" if float_out else ""), self.hidden, self.inter, runtime, float_out=float_out)
        self.act_buffer = f"{key}.act"
        runtime.workspace.declare(self.act_buffer, runtime.max_step_tokens * self.inter, runtime.dtype)

    @staticmethod
    def _names(params) -> dict[str, str]:
        suffix = str(params.get("weight_suffix", ".weight"))
        return {k: params.get(k, f"{k}_proj") + suffix for k in ("up", "down")}

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, inter = int(params["hidden_size"]), int(params["intermediate_size"])
        n = cls._names(params)
        std = float(params.get("init_std", 0.02))
        return {f"{prefix}.{n['up']}": TensorSpec((inter, hidden), init_std=std),
                f"{prefix}.{n['down']}": TensorSpec((hidden, inter), init_std=std)}

    def load(self, source) -> None:
        n, p = self.names, self.prefix
        self.up.set_weight(source(f"{p}.{n['up']}"))
        self.down.set_weight(source(f"{p}.{n['down']}"))

    def forward(self, x, ctx):
        tokens = x.shape[0]
        act = self.runtime.workspace.view(self.act_buffer, tokens, self.inter)
        kernels.activation(self.up(x), act, self.activation)
        return self.down(act)


# Most (token, expert) pairs that run as matrix-vector passes, each streaming its expert's rows once: up to two pairs
# per expert, and never more than 64.  Beyond, pairs that share an expert would each read its weights again (from L2 at
# best), so the pairs are ordered by expert and the products run in tiles on the tensor cores, every expert read once
# (8 experts of 1,024 x 4,096 at 64 pairs: 0.77 ms a four-layer step per pair, against the dense model's 0.32).
_PAIRS_BY_PAIR = 64


@register_feed_forward("table_experts")
class TableExperts:
    """A set of small two-matrix feed-forward layers ("experts"), down_e(act(up_e(x))) without biases, of which every
    token runs the ``top`` that an integer table [vocab, top] names for its token id; their outputs are summed with
    the weight ``pair_weight`` each (default 1 / top, the mean).  There is no learned router: the choice depends on
    the token id alone, so it is read on the device from the step's token ids and a step launches the same kernels
    whatever the tokens are.

    Parameters: ``hidden_size``, ``expert_size`` (width of an expert's middle), ``experts``, ``top``, ``vocab_size``,
    ``activation`` (one of ``kernels.ACTIVATIONS``), and the tensor-name pieces ``table``, ``expert`` (a format of the
    expert's number), ``up``, ``down``, ``weight_suffix``.
    """

    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["expert_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.vocab = int(params["vocab_size"])
        self.activation = params.get("activation", "gelu")
        if self.activation not in kernels.ACTIVATIONS:
            raise ValueError(f"{prefix}: activation {self.activation!r} is not one of {sorted(kernels.ACTIVATIONS)}")
        if not 0 < self.top <= self.experts:
            raise ValueError(f"{prefix}: {self.top} experts per token out of {self.experts}")
        self.pair_weight = float(params.get("pair_weight", 1.0 / self.top))
        self.params = dict(params)
        self.up = self.down = self.table = None
        ws = runtime.workspace
        ws.declare("experts.out", runtime.max_step_tokens * self.hidden, torch.float32)
        # many tokens in bfloat16: the pairs ordered by expert in tiles of rows, both products on the tensor cores
        self.tiled = runtime.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0
        pairs = runtime.max_step_tokens * self.top
        rows = pairs
        if self.tiled:
            tiles = kernels.expert_tiles(pairs, self.experts)
            rows = tiles * kernels.EXPERT_TILE_ROWS
            ws.declare("experts.ordered", rows * self.hidden, runtime.dtype)
            ws.declare("experts.y", rows * self.hidden, runtime.dtype)
            ws.declare("experts.route", pairs + rows + tiles, torch.int32)
        ws.declare("experts.mid", rows * self.inter, runtime.dtype)

    @staticmethod
    def _tensor_names(params, prefix: str) -> tuple[str, list[tuple[str, str]]]:
        suffix = str(params.get("weight_suffix", ".weight"))
        expert = str(params.get("expert", "experts.{}"))
        up, down = params.get("up", "up"), params.get("down", "down")
        pairs = [(f"{prefix}.{expert.format(e)}.{up}{suffix}", f"{prefix}.{expert.format(e)}.{down}{suffix}")
                 for e in range(int(params["experts"]))]
        return f"{prefix}.{params.get('table', 'table')}", pairs

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, inter = int(params["hidden_size"]), int(params["expert_size"])
        table, pairs = cls._tensor_names(params, prefix)
        out = {table: TensorSpec((int(params["vocab_size"]), int(params["top"])), role="table", table_high=int(params["experts"]))}
        for up, down in pairs:
            out[up] = TensorSpec((inter, hidden), init_std=0.05)
            out[down] = TensorSpec((hidden, inter), init_std=0.05)
        return out

    def load(self, source) -> None:
        table, pairs = self._tensor_names(self.params, self.prefix)
        dtype, device = self.runtime.dtype, self.runtime.device
        self.up = torch.stack([source(up).to(device=device, dtype=dtype) for up, _ in pairs]).contiguous()
        self.down = torch.stack([source(down).to(device=device, dtype=dtype) for _, down in pairs]).contiguous()
        table = source(table)
        if int(table.min()) < 0 or int(table.max()) >= self.experts:
            raise ValueError(f"{self.prefix}: the table names experts outside 0..{self.experts - 1}")
        self.table = to_device(table, torch.int32, device)

    def forward(self, x, ctx) -> GemmOut:
        tokens = x.shape[0]
        ws = self.runtime.workspace
        out = ws.view("experts.out", tokens, self.hidden)
        pairs = tokens * self.top
        if self.tiled and pairs > min(_PAIRS_BY_PAIR, 2 * self.experts):
            tiles = kernels.expert_tiles(pairs, self.experts)
            rows = tiles * kernels.EXPERT_TILE_ROWS
            kernels.experts_tiled(x, ctx.token_ids, self.table, self.up, self.down, ws.view("experts.ordered", rows, self.hidden),
                                  ws.view("experts.mid", rows, self.inter), ws.view("experts.y", rows, self.hidden),
                                  ws.view("experts.route", pairs + rows + tiles), out, self.activation, self.pair_weight)
        else:
            mid = ws.view("experts.mid", pairs, self.inter)
            kernels.experts_by_pair(x, ctx.token_ids, self.table, self.up, self.down, mid, out, self.activation, self.pair_weight)
        return GemmOut(out.view(1, tokens, self.hidden))


@register_feed_forward("routed_experts")
class RoutedExperts:
    """Experts chosen by a learned router: logits z = W_router h in float, scores sigmoid(z), the ``top`` largest
    chosen, their weights the scores over their sum (+ 1e-20) times ``route_scale``; the output is the weighted sum of
    the chosen experts' outputs.  An expert is gated, down(gate(gate_proj h, up_proj h)), with the activation
    ``activation`` (``kernels.CAPPED_GATE`` with ``limit``, or one of ``kernels.ACTIVATIONS``) and no biases.  With
    ``shared`` (a dict: ``intermediate_size``, ``limit``) a further expert of the same form runs for every token and is
    added, times sigmoid(w_gate . h), one number per token; its gate is one more row of the router's product.

    ``normalize`` = False: the weights are the chosen scores themselves (times ``route_scale``), not divided by their sum.
    ``weight_on`` = "input": a pair's weight multiplies what its expert reads, not what it returns: the output is the sum of
    expert_e(w_e h), which for a gated expert is another function of w_e.  ``shared_gated`` = False: the shared expert is
    added as it is, without a gate (and without the router's extra row).

    The routing is computed on the device by a kernel behind the router's product, so a step launches the same
    kernels whatever the tokens are.  Few (token, expert) pairs run as matrix-vector passes per pair, many are
    ordered by expert and run in tiles on the tensor cores (``experts.cu``, ``experts_tc.cu``), as for experts chosen
    by a table.

    Parameters: ``hidden_size``, ``expert_size``, ``experts``, ``top``, ``route_scale``, ``activation``, ``limit``,
    ``shared``, and the tensor-name pieces ``router``, ``expert`` (a format of the expert's number), ``gate``, ``up``,
    ``down``, ``shared_name``, ``shared_gate``, ``weight_suffix``.
    """

    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.params = dict(params)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["expert_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.route_scale = float(params.get("route_scale", 1.0))
        self.activation = params.get("activation", "silu")
        self.limit = float(params.get("limit", 0.0))
        if self.activation not in kernels.ACTIVATIONS and self.activation != kernels.CAPPED_GATE:
            raise ValueError(f"{prefix}: gate activation {self.activation!r} is not one of {sorted(kernels.ACTIVATIONS) + [kernels.CAPPED_GATE]}")
        if not 0 < self.top <= self.experts:
            raise ValueError(f"{prefix}: {self.top} experts per token out of {self.experts}")
        self.normalize = bool(params.get("normalize", True))
        self.weight_on = str(params.get("weight_on", "output"))
        if self.weight_on not in ("output", "input"):
            raise ValueError(f"{prefix}: weight_on={self.weight_on!r} is neither 'output' nor 'input'")
        self.shared_gated = bool(params.get("shared_gated", True))
        shared = params.get("shared")
        self.shared = None
        if shared is not None:
            self.shared = GatedMLP({"hidden_size": self.hidden, "intermediate_size": int(shared["intermediate_size"]),
                                    "activation": self.activation, "limit": float(shared.get("limit", self.limit)),
                                    "gate": params.get("gate", "gate"), "up": params.get("up", "up"), "down": params.get("down", "down"),
                                    "weight_suffix": params.get("weight_suffix", ".weight"), "float_out": True, "buffers": "experts.shared",
                                    "init_std": float(params.get("init_std", 0.02))},
                                   f"{prefix}.{params.get('shared_name', 'shared')}", runtime)
        self.router = Linear("experts.router", self.experts + (1 if self.shared and self.shared_gated else 0), self.hidden, runtime, float_out=True)
        self.up = self.down = None
        ws = runtime.workspace
        tokens = runtime.max_step_tokens
        ws.declare("experts.out", tokens * self.hidden, torch.float32)
        ws.declare("experts.chosen", tokens * self.top, torch.int32)
        ws.declare("experts.weights", tokens * self.top, torch.float32)
        ws.declare("experts.shared_gate", tokens, torch.float32)
        self.tiled = runtime.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0
        pairs = tokens * self.top
        rows = pairs
        if self.tiled:
            tiles = kernels.expert_tiles(pairs, self.experts)
            rows = tiles * kernels.EXPERT_TILE_ROWS
            ws.declare("experts.ordered", rows * self.hidden, runtime.dtype)
            ws.declare("experts.y", rows * self.hidden, runtime.dtype)
            ws.declare("experts.route", pairs + rows + tiles, torch.int32)
            ws.declare("experts.wide", rows * 2 * self.inter, runtime.dtype)
        ws.declare("experts.mid", rows * self.inter, runtime.dtype)

    @staticmethod
    def _tensor_names(params, prefix: str):
        suffix = str(params.get("weight_suffix", ".weight"))
        expert = str(params.get("expert", "experts.{}"))
        names = [tuple(f"{prefix}.{expert.format(e)}.{params.get(k, k)}{suffix}" for k in ("gate", "up", "down"))
                 for e in range(int(params["experts"]))]
        shared_gate = f"{prefix}.{params.get('shared_name', 'shared')}.{params.get('shared_gate', 'gate_weight')}"
        return f"{prefix}.{params.get('router', 'router')}{suffix}", names, shared_gate

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, inter, experts = int(params["hidden_size"]), int(params["expert_size"]), int(params["experts"])
        router, names, shared_gate = cls._tensor_names(params, prefix)
        std = float(params.get("init_std", 0.02))
        out = {router: TensorSpec((experts, hidden), init_std=float(params.get("router_init_std", 0.1)))}
        for gate, up, down in names:
            out[gate] = TensorSpec((inter, hidden), init_std=std)
            out[up] = TensorSpec((inter, hidden), init_std=std)
            out[down] = TensorSpec((hidden, inter), init_std=std)
        shared = params.get("shared")
        if shared is not None:
            sub = {"hidden_size": hidden, "intermediate_size": int(shared["intermediate_size"]), "gate": params.get("gate", "gate"),
                   "up": params.get("up", "up"), "down": params.get("down", "down"), "weight_suffix": params.get("weight_suffix", ".weight"),
                   "init_std": std}
            out.update(GatedMLP.expected_tensors(sub, f"{prefix}.{params.get('shared_name', 'shared')}"))
            if params.get("shared_gated", True):
                out[shared_gate] = TensorSpec((1, hidden), init_std=float(params.get("router_init_std", 0.1)))
        return out

    def load(self, source) -> None:
        router, names, shared_gate = self._tensor_names(self.params, self.prefix)
        dtype, device = self.runtime.dtype, self.runtime.device
        self.up = torch.stack([torch.cat((source(gate).to(dtype), source(up).to(dtype)), dim=0).to(device) for gate, up, _ in names]).contiguous()
        self.down = torch.stack([source(down).to(device=device, dtype=dtype) for _, _, down in names]).contiguous()
        rows = [source(router).to(dtype)]
        if self.shared is not None:
            self.shared.load(source)
            if self.shared_gated:
                rows.append(source(shared_gate).to(dtype).reshape(1, self.hidden))
        self.router.set_weight(torch.cat(rows, dim=0))

    def forward(self, x, ctx) -> GemmOut:
        tokens = x.shape[0]
        ws = self.runtime.workspace
        out = ws.view("experts.out", tokens, self.hidden)
        chosen = ws.view("experts.chosen", tokens, self.top)
        weights = ws.view("experts.weights", tokens, self.top)
        gate = ws.view("experts.shared_gate", tokens) if self.shared is not None and self.shared_gated else None
        kernels.route_top(self.router(x), chosen, weights, gate, self.experts, self.route_scale, self.normalize)
        on_input = self.weight_on == "input"
        out_weights, in_weights = (None, weights) if on_input else (weights, None)
        base = None
        if self.shared is not None:
            base = self.shared.forward(x, ctx)
            base = base.run() if hasattr(base, "run") else base
        pairs = tokens * self.top
        if self.tiled and pairs > min(_PAIRS_BY_PAIR, 2 * self.experts):
            tiles = kernels.expert_tiles(pairs, self.experts)
            rows = tiles * kernels.EXPERT_TILE_ROWS
            kernels.experts_tiled(x, None, chosen, self.up, self.down, ws.view("experts.ordered", rows, self.hidden),
                                  ws.view("experts.mid", rows, self.inter), ws.view("experts.y", rows, self.hidden),
                                  ws.view("experts.route", pairs + rows + tiles), out, self.activation, pair_weight=1.0, pair_weights=out_weights,
                                  gated=True, limit=self.limit, wide=ws.view("experts.wide", rows, 2 * self.inter), base=base, row_scale=gate,
                                  in_weights=in_weights)
        else:
            kernels.experts_by_pair(x, None, chosen, self.up, self.down, ws.view("experts.mid", pairs, self.inter), out, self.activation,
                                    pair_weight=1.0, pair_weights=out_weights, gated=True, limit=self.limit, base=base, row_scale=gate,
                                    in_weights=in_weights)
        return GemmOut(out.view(1, tokens, self.hidden))
