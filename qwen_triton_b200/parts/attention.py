"""Softmax attention over the paged cache with grouped kv heads, optional per-head q/k RMSNorm,
a position encoding part and an optional window.

Order as in the reference (qwen_triton/modules/attention.py:53-73,125-128): project, norm q and k
per head over head_dim *before* rotation, rotate, write k/v to the cache, attend, project out.
The three projections run as one product over the row-concatenated weight [q; k; v].

Further parameters, each off unless given, for designs that treat scores or values differently:

* ``v_head_dim``: head size of the values where it is not the keys' (the output projection then reads
  ``num_heads * v_head_dim`` columns);
* ``o_bias``: whether the output projection has a bias (default: what ``bias`` says for all four);
* ``v_norm`` with ``v_norm_eps``: every value head is divided by its root mean square before it is cached;
* ``v_blend`` = "source" | "blend" with ``v_blend_key``: a "source" layer keeps its (treated) values of the step's
  tokens in a float buffer named by the key; a "blend" layer replaces its own by (1 - w) v + w v_source, w being
  the float tensor named by ``names["v_blend_weight"]``; what is blended is what is cached;
* ``distance_penalty`` = "log": the score of key j for the query at position i loses r1_h ln(1 + r2_h (i - j)),
  with one r1 and r2 per query head (tensors ``names["r1"]``, ``names["r2"]``);
* ``weight_suffix`` / ``bias_suffix``: what a projection's tensor names add to the projection's name
  (default ".weight" / ".bias"); ``norm_suffix``: the same for the q/k norm weights (default ".weight");
* ``chunk``: a query at position i sees key j <= i only if i // chunk == j // chunk (positions from the sequence's
  start).  The cache keeps every key, so that another layer may read them under a mask of its own;
* ``maps`` = 2 with ``diff``: differential attention.  q and k hold two score maps per head, stored head by head
  as [map 1, map 2]; each map is a softmax attention of its own over the head's one set of values (size
  ``v_head_dim``), and the head's output is o = a1 - lambda a2, divided by its root mean square (``head_norm_eps``
  inside the root, no weight), times (1 - diff), with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff from four
  vectors of the layer (tensors ``names["lq1"]`` ...).  The projections' rows are reordered map-major when loaded,
  so that map m of head h is query head m * H + h and reads key head m * G + g; the value cache has G heads;
* ``float_out``: the output projection hands on float sums (for a float residual addition);
* ``qk_norm`` = "unit": q and k heads are divided by their root mean square (``qk_norm_eps``) without a weight; a
  rotation leaves a head's sum of squares as it is, so this is also the norm of a design that divides after rotating;
  ``qk_norm`` = "whole": q and k are RMS-normed over all their heads at once, with weights of the projections' sizes;
* ``keep_first`` (with ``window``): the first positions of a sequence stay visible to every later query, at their true
  positions; the cache then keeps every key (no ring) and the kernels mask;
* ``sink`` = "learned": the softmax's denominator also holds exp(s_h), one stored number per query head
  (tensor ``names["sink"]``) that is not scaled and has no value; ``sink`` = True: the same with s_h = 0;
* ``head_gate``: every head's output is multiplied by sigmoid(w_h . x), one number per head; the rows W_g [heads, hidden]
  (tensor ``names["g"]``) ride at the end of the q/k/v projection, whose sums are then float (``float_proj`` asks for
  float sums by itself).

Values that are treated (``v_norm``, ``v_blend``, a head size of their own) go with no rotation and no q/k norm:
bias, treatment and the cache write are then one kernel behind the projection (``kernels.qkv_treat_write``).
"""
from __future__ import annotations

import math

import torch

from ..ops import kernels
from ..ops.kernels import GemmOut
from ..weights.tensors import TensorSpec
from .base import DeferredProduct, KVRequest, Runtime, part_class, register_mixer, to_device
from .linear import Linear

_DECODE_BLOCKS_PER_SM = 3           # blocks of the generic one-token kernel that are resident at once
_MAX_SPLIT_PAIRS = 640              # (sequence, split) pairs the scratch holds
_MIN_KEYS_PER_SPLIT = 128


@register_mixer("attention")
class Attention:
    graph_safe = True      # forward() only launches kernels: a decode step with this mixer can be captured in a CUDA graph

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.hidden = int(params["hidden_size"])
        self.maps = int(params.get("maps", 1))
        if self.maps not in (1, 2):
            raise ValueError(f"{prefix}: {self.maps} score maps per head (1, or 2 for differential attention)")
        self.heads_out = int(params["num_heads"])                  # heads as the output projection sees them
        self.v_heads = int(params["num_kv_heads"])                 # value heads
        self.nq = self.maps * self.heads_out                       # heads as the attention kernels see them: one per map
        self.nkv = self.maps * self.v_heads
        self.d = int(params["head_dim"])
        self.chunk = int(params["chunk"]) if params.get("chunk") else None
        self.diff = float(params.get("diff", 0.0))
        self.head_norm_eps = float(params.get("head_norm_eps", 1e-6))
        self.lam = 0.0
        self.scale = float(params.get("scale", self.d ** -0.5))
        self.window = params.get("window")
        self.own_kv = bool(params.get("own_kv", True))
        self.norm_mode = {False: None, None: None, True: "head", "head": "head", "unit": "unit", "whole": "whole"}.get(params.get("qk_norm", False), "?")
        if self.norm_mode == "?":
            raise ValueError(f"{prefix}: qk_norm={params.get('qk_norm')!r} is none of False, True, 'unit', 'whole'")
        self.qk_norm = self.norm_mode in ("head", "whole")          # norms that have weights
        self.keep_first = int(params.get("keep_first") or 0) if params.get("window") else 0
        self.sink = params.get("sink", False)
        if self.sink not in (False, True, "learned"):
            raise ValueError(f"{prefix}: sink={self.sink!r} is none of False, True, 'learned'")
        self.head_gate = bool(params.get("head_gate", False))
        self.float_proj = bool(params.get("float_proj", False)) or self.head_gate
        self.sinks = None
        self.bias = bool(params.get("bias", False))        # q, k, v and o projections with a bias (attention.py:38-41)
        self.o_bias = bool(params.get("o_bias", self.bias))
        self.eps = float(params.get("qk_norm_eps", 1e-6))
        self.names = self._names(params)
        self.dv = int(params.get("v_head_dim") or self.d)
        self.v_norm_eps = float(params.get("v_norm_eps", 1e-6)) if params.get("v_norm", False) else None
        self.v_blend = params.get("v_blend")
        if self.v_blend not in (None, "source", "blend"):
            raise ValueError(f"{prefix}: v_blend={self.v_blend!r} is neither 'source' nor 'blend'")
        self.penalised = self._penalised(params, prefix)
        self.r1 = self.r2 = self.blend_weight = self.qkv_bias = None
        if self.nq % self.nkv:
            raise ValueError(f"{prefix}: {self.nq} query heads are not a multiple of {self.nkv} kv heads")
        if max(self.d, self.dv) > 256:
            raise ValueError(f"{prefix}: head_dim={max(self.d, self.dv)} is beyond what the attention kernels take (256)")
        position_spec = params["position"]
        self.position = part_class("position", position_spec)(position_spec.params, runtime)
        self.interleaved = bool(getattr(self.position, "interleaved", False))      # which elements of a head form a rotation pair
        self.cos_sin: torch.Tensor | None = None
        self.q_weight = self.k_weight = None
        # values that are treated before they are cached: bias, treatment and cache write are one kernel of their own
        self.treated = self.v_norm_eps is not None or self.v_blend is not None or self.dv != self.d
        # values of their own shape that are otherwise untouched go with q/k norm and rotation (one kernel writes all)
        self.own_values = self.treated and self.v_norm_eps is None and self.v_blend is None and not self.bias
        if self.maps > 1 or self.norm_mode in ("unit", "whole") or self.float_proj:
            self.own_values = True            # the general kernel behind the projection
        if self.own_values:
            self.treated = False
        if self.treated and (self.qk_norm or not self.own_kv or position_spec.kind != "none"):
            raise ValueError(f"{prefix}: treated values (v_norm, v_blend) go with no rotation, no q/k norm and keys of the layer's own")
        if self.maps > 1 and (self.bias or self.window or self.penalised or self.sink or self.head_gate or self.norm_mode in ("unit", "whole")):
            raise ValueError(f"{prefix}: differential attention goes with no bias, window, distance penalty, sink, gate or norm of another kind")
        if (self.keep_first or self.sink or self.head_gate or self.norm_mode in ("unit", "whole")) and (self.treated or self.bias or not self.own_kv or self.chunk):
            raise ValueError(f"{prefix}: kept first keys, a sink, a gate per head and the unit and whole-row norms go with untreated values, "
                             "no bias, no chunks and keys of the layer's own")
        self.gate_cols = -(-self.heads_out // 8) * 8 if self.head_gate else 0       # the gate's rows, padded so that rows of sums stay aligned
        # the mma.sync attention kernels take values as wide as the keys (and compute the distance penalty, given a
        # positive scale); everything else goes to the generic kernels
        self.mma_scores = self.dv == self.d and (not self.penalised or self.scale > 0)
        proj_rows = self.nq * self.d + ((self.nkv * self.d + self.v_heads * self.dv) if self.own_kv else 0) + self.gate_cols
        self.at_gate = proj_rows - self.gate_cols
        if self.own_values:
            self.qkv = Linear("attn.qkv.own_values" + (".float" if self.float_proj else ""), proj_rows, self.hidden, runtime, float_out=self.float_proj)
        elif self.treated:
            self.qkv = Linear("attn.qkv.sums", proj_rows, self.hidden, runtime, float_out=True)      # float sums: the bias is added behind it
        else:
            self.qkv = Linear("attn.qkv" + (".biased" if self.bias else ""), proj_rows, self.hidden, runtime, role="qkv", bias=self.bias)
        self.float_out = bool(params.get("float_out", False))
        self.o = Linear("attn.o" + (".biased" if self.o_bias else "") + (".float" if self.float_out else ""), self.hidden,
                        self.heads_out * self.dv, runtime, role="attn_out", bias=self.o_bias, float_out=self.float_out)
        ws = runtime.workspace
        ws.declare("attn.q", runtime.max_step_tokens * self.nq * self.d, runtime.dtype)
        ws.declare("attn.ctx", runtime.max_step_tokens * self.nq * self.dv, runtime.dtype)
        if self.maps > 1:
            ws.declare("attn.heads", runtime.max_step_tokens * self.heads_out * self.dv, runtime.dtype)
        ws.declare("attn.part_acc", _MAX_SPLIT_PAIRS * self.nq * self.dv, torch.float32)
        ws.declare("attn.part_ml", _MAX_SPLIT_PAIRS * self.nq * 2, torch.float32)
        if self.norm_mode == "whole":
            ws.declare("attn.row_inv", runtime.max_step_tokens * 2, torch.float32)
        self.side_name = "attn.values." + str(params.get("v_blend_key", "first"))
        if self.v_blend is not None:
            ws.declare(self.side_name, runtime.max_step_tokens * self.nkv * self.dv, torch.float32)
        # few tokens: the projection takes rows whose norm factor is still to be applied (``ScaledRows``)
        self.takes_scaled_rows = self.qkv.fused_capable and not self.own_values

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _names(params) -> dict[str, str]:
        n = {k: params.get(k, k) for k in ("q", "k", "v", "o", "q_norm", "k_norm", "r1", "r2", "v_blend_weight", "lq1", "lk1", "lq2", "lk2", "sink", "g")}
        n["w"], n["b"] = str(params.get("weight_suffix", ".weight")), str(params.get("bias_suffix", ".bias"))
        n["nw"] = str(params.get("norm_suffix", ".weight"))
        n["sink"] = str(params.get("sink_name", "sink"))          # ``sink`` itself says whether there is one
        return n

    @staticmethod
    def _penalised(params, prefix: str) -> bool:
        kind = params.get("distance_penalty")
        if kind not in (None, "log"):
            raise ValueError(f"{prefix}: distance_penalty={kind!r}; the attention kernels compute 'log'")
        return kind is not None

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, nq, nkv, d = (int(params[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        dv = int(params.get("v_head_dim") or d)
        maps = int(params.get("maps", 1))
        n = cls._names(params)
        own_kv = bool(params.get("own_kv", True))
        std = float(params.get("init_std", 0.02))
        out = {f"{prefix}.{n['q']}{n['w']}": TensorSpec((maps * nq * d, hidden), init_std=std),
               f"{prefix}.{n['o']}{n['w']}": TensorSpec((hidden, nq * dv), init_std=std)}
        if own_kv:
            out[f"{prefix}.{n['k']}{n['w']}"] = TensorSpec((maps * nkv * d, hidden), init_std=std)
            out[f"{prefix}.{n['v']}{n['w']}"] = TensorSpec((nkv * dv, hidden), init_std=std)
        if maps > 1:
            for name in ("lq1", "lk1", "lq2", "lk2"):
                out[f"{prefix}.{n[name]}"] = TensorSpec((d,), role="vector", init_std=0.1, init_mean=0.0)
        if params.get("bias", False):
            # the reference starts a bias at zero (models/core.py:269-270); random ones so that a bias that is skipped shows
            for name in (("q",) + (("o",) if params.get("o_bias", True) else ()) + (("k", "v") if own_kv else ())):
                rows = out[f"{prefix}.{n[name]}{n['w']}"].shape[0]
                out[f"{prefix}.{n[name]}{n['b']}"] = TensorSpec((rows,), role="vector", init_std=0.1, init_mean=0.0)
        if cls._penalised(params, prefix):
            # r2 stays positive, so that 1 + r2 * distance does; the draw's tails end six deviations from the mean
            out[f"{prefix}.{n['r1']}"] = TensorSpec((nq,), role="vector", init_std=0.3, init_mean=1.0)
            out[f"{prefix}.{n['r2']}"] = TensorSpec((nq,), role="vector", init_std=0.04, init_mean=0.3)
        if params.get("v_blend") is not None or params.get("v_blend_weight_stored", False):
            # a source layer stores the weight too and never reads it; a layer outside the scheme may store it
            out[f"{prefix}.{n['v_blend_weight']}"] = TensorSpec((), role="vector", init_std=0.08, init_mean=0.4,
                                                                optional=params.get("v_blend") != "blend")
        if params.get("qk_norm", False) in (True, "head", "whole"):
            whole = params.get("qk_norm") == "whole"
            out[f"{prefix}.{n['q_norm']}{n['nw']}"] = TensorSpec((nq * d if whole else d,), role="vector", init_std=0.1, init_mean=1.0)
            if own_kv:
                out[f"{prefix}.{n['k_norm']}{n['nw']}"] = TensorSpec((nkv * d if whole else d,), role="vector", init_std=0.1, init_mean=1.0)
        if params.get("sink", False) == "learned":
            out[f"{prefix}.{n['sink']}"] = TensorSpec((nq,), role="vector", init_std=1.0, init_mean=0.0)
        if params.get("head_gate", False):
            out[f"{prefix}.{n['g']}{n['w']}"] = TensorSpec((nq, hidden), init_std=std)
        return out

    def load(self, source) -> None:
        n, p = self.names, self.prefix
        def map_major(weight: torch.Tensor, heads: int) -> torch.Tensor:
            """Rows stored [head][map][d] as [map][head][d]: a map is then a head of its own for the kernels."""
            if self.maps == 1:
                return weight
            return weight.view(heads, self.maps, self.d, weight.shape[1]).transpose(0, 1).reshape(weight.shape)

        rows = [map_major(source(f"{p}.{n['q']}{n['w']}"), self.heads_out)]
        if self.own_kv:
            rows += [map_major(source(f"{p}.{n['k']}{n['w']}"), self.v_heads), source(f"{p}.{n['v']}{n['w']}")]
        if self.maps > 1:
            # one number for the layer, made once on the host (the same bits wherever the tensors were drawn)
            vec = {name: source(f"{p}.{n[name]}").double().cpu() for name in ("lq1", "lk1", "lq2", "lk2")}
            self.lam = float(torch.exp((vec["lq1"] * vec["lk1"]).sum()) - torch.exp((vec["lq2"] * vec["lk2"]).sum())) + self.diff
        if self.head_gate:
            gate = source(f"{p}.{n['g']}{n['w']}")
            rows += [gate, torch.zeros(self.gate_cols - gate.shape[0], self.hidden, dtype=gate.dtype, device=gate.device)]
        if self.sink == "learned":
            self.sinks = to_device(source(f"{p}.{n['sink']}"), torch.float32, self.runtime.device)
        self.qkv.set_weight(torch.cat([r.to(self.runtime.dtype) for r in rows], dim=0))
        self.o.set_weight(source(f"{p}.{n['o']}{n['w']}"))
        if self.bias:
            names = ("q", "k", "v") if self.own_kv else ("q",)
            bias = torch.cat([source(f"{p}.{n[name]}{n['b']}").float() for name in names], dim=0)
            if self.treated:
                self.qkv_bias = to_device(bias, torch.float32, self.runtime.device)
            else:
                self.qkv.set_bias(bias)
            if self.o_bias:
                self.o.set_bias(source(f"{p}.{n['o']}{n['b']}"))
        if self.penalised:
            self.r1 = to_device(source(f"{p}.{n['r1']}"), torch.float32, self.runtime.device)
            self.r2 = to_device(source(f"{p}.{n['r2']}"), torch.float32, self.runtime.device)
        if self.v_blend == "blend":
            self.blend_weight = to_device(source(f"{p}.{n['v_blend_weight']}"), torch.float32, self.runtime.device).reshape(1)
        if self.qk_norm:
            self.q_weight = to_device(source(f"{p}.{n['q_norm']}{n['nw']}"), torch.float32, self.runtime.device)
            if self.own_kv:
                self.k_weight = to_device(source(f"{p}.{n['k_norm']}{n['nw']}"), torch.float32, self.runtime.device)
        tables = self.runtime.options.setdefault("position_tables", {})
        key = self.position.key() + (self.runtime.max_positions,)
        if key not in tables:
            tables[key] = self.position.table(self.runtime.max_positions)
        self.cos_sin = tables[key]

    # ------------------------------------------------------------------ cache
    def cache_request(self) -> KVRequest | None:
        return KVRequest(self.nkv, self.d, None if self.keep_first else self.window, self.dv if self.dv != self.d else None,
                         self.v_heads if self.v_heads != self.nkv else None)

    # ------------------------------------------------------------------ run
    def _splits(self, ctx, cache) -> tuple[int, int]:
        """How a one-token step cuts the keys of each sequence: (blocks per sequence and kv head, warps per block).

        The tensor-core kernel gives every warp a key range of its own.  Measured on the B200: with a moderate
        number of (sequence, kv head) pairs, about one block of four warps per SM and as few partial results as that
        allows; with very few pairs, blocks of six warps and a count weighed against the cost of merging them (below);
        with blocks for two per SM, three warps each and no cut at all.  Every range keeps at least
        two tiles of 32 keys.  The generic kernel (other element types and head sizes) takes one range per
        block: the count whose blocks fill whole waves of three blocks per SM nearly as well as the best one.
        """
        span = ctx.max_context if not self.window else min(ctx.max_context, self.window + self.keep_first)
        if self.chunk:
            span = min(span, self.chunk)
        group = self.nq // self.nkv
        most = max(1, min(_MAX_SPLIT_PAIRS // ctx.n_seqs, 32))
        if self.mma_scores and self.runtime.dtype == torch.bfloat16 and self.d % 16 == 0 and self.d <= 128 and cache.page_tokens == 64:
            pairs = ctx.n_seqs * self.nkv * math.ceil(group / 16)
            tiles = math.ceil(span / 32)
            sms = self.runtime.sm_count
            splits = max(1, min(sms // pairs, most))
            # blocks of four warps are one to an SM, of three two: three where that makes one wave of what would be two
            # with a nearly empty second one (160-192 blocks: 2-5 % shorter steps at batch 20-24 of the 8B shape), and
            # where there are blocks for three waves and more (batch 56-64: 6 %)
            warps = 3 if pairs * splits >= 3 * sms or sms < pairs * splits <= 2 * sms else 4
            if splits >= 4:
                # Few pairs (batch 1 to 4 with eight kv heads): blocks of six warps, and as many of them per pair as
                # pays: a block draws about 80 GB/s of keys and values, a merge through a cluster of up to four blocks
                # costs about 1.5 us, of six 3 us, and more blocks than a cluster holds (scratch memory and the combine
                # kernel) 13 us.  Clusters of five and seven, and more than eight clusters of eight, are left out: they
                # pack the SMs of a GPC badly beside the next product's clusters (batch 2, cache 8,192: 3.80 ms a step
                # with eight blocks per pair, 3.57 with five, 3.51 with six).  Timed in the model, 8B shape, batch 1: cache 2,048: 3.09 ms a step
                # with four blocks against 3.15 with eight; 8,192: 3.32 against 3.54 with four; 32,768: 3.99 with
                # eighteen against 4.23 with eight and 5.26 with four.
                warps = kernels.DECODE_WARPS_MAX
                pair_bytes = 4.0 * span * self.d                      # keys and values of one pair, bfloat16
                best = None
                for count in range(1, splits + 1):
                    if count > 1 and count * warps * 2 > tiles:
                        break
                    if count in (5, 7) or (count == 8 and pairs > 8):        # eight clusters of eight still find a GPC each
                        continue
                    merge = 0.0 if count == 1 else 1.5e-6 if count <= 4 else 3e-6 if count <= 8 else 13e-6
                    cost = merge + pair_bytes / (count * 80e9)
                    if best is None or cost < best[0]:
                        best = (cost, count)
                splits = best[1]
            while splits > 1 and splits * warps * 2 > tiles:
                splits -= 1
            while warps > 1 and splits * warps * 2 > tiles:
                warps -= 1
            return splits, warps
        heads_per_block = 8 if group > 4 else max(1, group)
        blocks = ctx.n_seqs * self.nkv * math.ceil(group / heads_per_block)
        most = max(1, min(span // _MIN_KEYS_PER_SPLIT, most))
        fills = []
        resident = _DECODE_BLOCKS_PER_SM * self.runtime.sm_count
        for splits in range(1, most + 1):
            total = blocks * splits
            fills.append(total / (math.ceil(total / resident) * resident))
        enough = max(fills) - 0.13
        return next(splits for splits, fill in enumerate(fills, start=1) if fill >= enough), 1

    def forward(self, x, ctx, cache):
        tokens = x.shape[0]
        ws = self.runtime.workspace
        q = ws.view("attn.q", tokens, self.nq, self.d)
        out = ws.view("attn.ctx", tokens, self.nq, self.dv)
        table = ctx.block_table(cache.group)
        write = cache.writable and self.own_kv
        rotary_dim = 0 if self.cos_sin is None else self.cos_sin.shape[1]
        penalty = (self.r1, self.r2) if self.penalised else None
        if self.treated:
            side = ws.view(self.side_name, tokens, self.nkv, self.dv) if self.v_blend is not None else None
            kernels.qkv_treat_write(self.qkv(x), self.qkv_bias, q, cache.k if write else None, cache.v if write else None,
                                    ctx.token_seq, ctx.token_pos, table if write else None, self.nq, self.nkv, self.d, self.dv,
                                    cache.page_tokens, cache.ring_tokens, v_norm_eps=self.v_norm_eps,
                                    blend_from=side if self.v_blend == "blend" else None, blend_weight=self.blend_weight,
                                    keep_to=side if self.v_blend == "source" else None, write_kv=write)
        elif not self.own_values and self.qkv.fusable(tokens) and kernels.fused_qkv_supported(self.d, rotary_dim):
            # few tokens: per-head norm, rotation and the cache write in the projection's epilogue
            self.qkv.into_qkv(x, q, cache.k if write else None, cache.v if write else None, ctx.token_seq, ctx.token_pos,
                              table if write else None, self.q_weight, self.k_weight, self.eps, self.cos_sin, self.nq, self.nkv,
                              self.d, cache.page_tokens, cache.ring_tokens, write_kv=write, interleaved=self.interleaved)
        else:
            proj = self.qkv(x)
            kernels.qk_norm_rope_write(
                proj, q, cache.k if write else None, cache.v if write else None, ctx.token_seq, ctx.token_pos,
                table if write else None, self.q_weight, self.k_weight, self.eps, self.cos_sin, self.nq, self.nkv, self.d,
                cache.page_tokens, cache.ring_tokens, write_kv=write, kv_in_proj=self.own_kv, interleaved=self.interleaved,
                v_heads=self.v_heads if self.own_values else None, v_head_dim=self.dv if self.own_values else None,
                unit_norm=self.norm_mode == "unit", row_inv=ws.view("attn.row_inv", tokens, 2) if self.norm_mode == "whole" else None,
                extra_cols=self.gate_cols)
        if ctx.is_decode:
            n_splits, warps = self._splits(ctx, cache)
            kernels.attention_decode(q, cache.k, cache.v, out, table, ctx.seq_len, self.nkv, cache.page_tokens,
                                     cache.ring_tokens, self.window, self.scale, n_splits,
                                     ws.view("attn.part_acc", _MAX_SPLIT_PAIRS * self.nq * self.dv),
                                     ws.view("attn.part_ml", _MAX_SPLIT_PAIRS * self.nq * 2), warps=warps, penalty=penalty,
                                     chunk=self.chunk, keep_first=self.keep_first, sink=bool(self.sink), sinks=self.sinks)
        else:
            kernels.attention_prefill(q, cache.k, cache.v, out, table, ctx.seq_start, ctx.seq_past, ctx.max_q_len,
                                      self.nkv, cache.page_tokens, cache.ring_tokens, self.window, self.scale, penalty=penalty,
                                      chunk=self.chunk, keep_first=self.keep_first, sink=bool(self.sink), sinks=self.sinks)
        if self.head_gate:
            kernels.gate_mul(out.view(tokens, self.nq * self.dv), proj, self.at_gate, group=self.dv)
        if self.maps > 1:
            heads = ws.view("attn.heads", tokens, self.heads_out, self.dv)
            kernels.map_difference(out, heads, self.lam, self.head_norm_eps, 1.0 - self.diff)
            out = heads
        out = out.view(tokens, self.heads_out * self.dv)
        return DeferredProduct(self.o, out) if self.o.fusable(tokens) else self.o(out)
