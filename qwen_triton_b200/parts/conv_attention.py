"""Softmax attention whose queries and keys pass a short causal convolution over time and whose values are the keys.

Per token, from the mixer's input h: q = conv(W_q h + b_q), k = conv(W_k h + b_k) (a convolution of ``conv`` taps on every
channel, zeros before the sequence's start; the last ``conv`` - 1 projected rows of a sequence are part of its state), no
W_v: the value of a key is the key as it leaves the convolution, so one pool holds both.  Grouped heads (query head h reads
key head h // (H / G)), no rotation.  The score of key j for the query at position i is q . k * ``scale`` minus a linear
distance bias slope_h (i - j) with slope_h = 2^(-``slope_bits`` (h + 1) / H) (``slope_bits`` 8 by default).  A query sees
the last ``window`` positions (absent: all) and, with ``keep_first``, the first ``keep_first`` positions of the sequence
besides, at their true distances.  With ``sink`` the softmax has one more term of score 0 that carries no value.  The
concatenated heads are multiplied by sigmoid(W_g h) (``gate``), then projected by W_o (+ b_o).

q, k and the gate run as one product over the row-concatenated weight [q; k; g] whose float sums (bias added) the
convolution kernel reads: convolution sums, scores, softmax, distance bias and the gate are float.

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``, ``conv``, ``window``, ``keep_first``,
``sink``, ``gate`` (bool), ``bias`` (q, k and o), ``slope_bits``, ``float_out``, and the tensor-name pieces ``q``, ``k``, ``g``,
``o``, ``weight_suffix``, ``bias_suffix``, ``conv_suffix``.

A windowed layer with kept first keys holds every key of its sequences in the cache and masks in the kernels (tiles
between the kept keys and the window are skipped, not read).
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..weights.tensors import TensorSpec
from .attention import _MAX_SPLIT_PAIRS, _MIN_KEYS_PER_SPLIT
from .base import KVRequest, Runtime, StateRequest, register_mixer, to_device
from .linear import Linear


@register_mixer("conv_attention")
class ConvAttention:
    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix, self.runtime, self.params = prefix, runtime, params
        self.hidden = int(params["hidden_size"])
        self.nq, self.nkv, self.d = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        if self.nq % self.nkv:
            raise ValueError(f"{prefix}: {self.nq} query heads are not a multiple of {self.nkv} kv heads")
        if self.d > 512:
            raise ValueError(f"{prefix}: head_dim={self.d} is beyond what the attention kernels take for values (512)")
        self.scale = float(params.get("scale", self.d ** -0.5))
        self.taps = int(params.get("conv", 1))
        if not 1 <= self.taps <= 16:
            raise ValueError(f"{prefix}: a convolution of {self.taps} taps (1..16)")
        self.window = int(params["window"]) if params.get("window") else None
        self.keep_first = int(params.get("keep_first") or 0) if self.window else 0
        self.sink = bool(params.get("sink", False))
        self.gated = bool(params.get("gate", True))
        self.bias = bool(params.get("bias", True))
        self.slope_bits = float(params.get("slope_bits", 8.0))
        self.channels = (self.nq + self.nkv) * self.d
        self.at_gate = self.channels
        used = self.channels + (self.nq * self.d if self.gated else 0)
        self.proj_rows = -(-used // 8) * 8
        self.proj = Linear("conv_attn.proj", self.proj_rows, self.hidden, runtime, float_out=True, bias=self.bias)
        float_out = bool(params.get("float_out", False))
        self.o = Linear("conv_attn.o" + (".biased" if self.bias else "") + (".float" if float_out else ""), self.hidden, self.nq * self.d,
                        runtime, bias=self.bias, float_out=float_out)
        ws = runtime.workspace
        ws.declare("attn.q", runtime.max_step_tokens * self.nq * self.d, runtime.dtype)
        ws.declare("attn.ctx", runtime.max_step_tokens * self.nq * self.d, runtime.dtype)
        ws.declare("attn.part_acc", _MAX_SPLIT_PAIRS * self.nq * self.d, torch.float32)
        ws.declare("attn.part_ml", _MAX_SPLIT_PAIRS * self.nq * 2, torch.float32)
        self.conv = self.slopes = None

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _names(params, prefix: str) -> dict[str, str]:
        w, b = str(params.get("weight_suffix", ".weight")), str(params.get("bias_suffix", ".bias"))
        conv = str(params.get("conv_suffix", ".conv"))
        n = {}
        for key in ("q", "k", "g", "o"):
            stem = f"{prefix}.{params.get(key, key)}"
            n[key], n[key + "_bias"], n[key + "_conv"] = stem + w, stem + b, stem + conv
        return n

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, nq, nkv, d = (int(params[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        taps = int(params.get("conv", 1))
        n = cls._names(params, prefix)
        std = float(params.get("init_std", 0.02))
        out = {n["q"]: TensorSpec((nq * d, hidden), init_std=std), n["k"]: TensorSpec((nkv * d, hidden), init_std=std),
               n["o"]: TensorSpec((hidden, nq * d), init_std=std)}
        if params.get("gate", True):
            out[n["g"]] = TensorSpec((nq * d, hidden), init_std=std)
        if params.get("bias", True):
            out[n["q_bias"]] = TensorSpec((nq * d,), role="vector", init_std=0.1)
            out[n["k_bias"]] = TensorSpec((nkv * d,), role="vector", init_std=0.1)
            out[n["o_bias"]] = TensorSpec((hidden,), role="vector", init_std=0.1)
        out[n["q_conv"]] = TensorSpec((nq * d, taps), role="vector", init_std=0.3, init_mean=0.3)
        out[n["k_conv"]] = TensorSpec((nkv * d, taps), role="vector", init_std=0.3, init_mean=0.3)
        return out

    def load(self, source) -> None:
        n = self._names(self.params, self.prefix)
        dtype, device = self.runtime.dtype, self.runtime.device
        rows = [source(n["q"]).to(dtype), source(n["k"]).to(dtype)]
        if self.gated:
            rows.append(source(n["g"]).to(dtype))
        used = sum(r.shape[0] for r in rows)
        if self.proj_rows > used:
            rows.append(torch.zeros(self.proj_rows - used, self.hidden, dtype=dtype, device=rows[0].device))
        self.proj.set_weight(torch.cat(rows, dim=0))
        self.o.set_weight(source(n["o"]))
        if self.bias:
            bias = torch.zeros(self.proj_rows, dtype=torch.float32)
            bias[:self.channels] = torch.cat([source(n["q_bias"]).float().cpu(), source(n["k_bias"]).float().cpu()], dim=0)
            self.proj.set_bias(bias)
            self.o.set_bias(source(n["o_bias"]))
        self.conv = to_device(torch.cat([source(n["q_conv"]).float().cpu(), source(n["k_conv"]).float().cpu()], dim=0), torch.float32, device)
        slopes = [2.0 ** (-self.slope_bits * (h + 1) / self.nq) for h in range(self.nq)]
        self.slopes = torch.tensor(slopes, dtype=torch.float32, device=device)

    # ------------------------------------------------------------------ what it keeps per sequence
    def cache_request(self):
        """The keys (which are the values too) and the convolutions' last inputs.  With kept first keys every key stays
        in the cache; a plain window keeps a ring of them."""
        window = self.window if self.window and not self.keep_first else None
        return [KVRequest(self.nkv, self.d, window, shared_values=True),
                StateRequest((max(self.taps - 1, 1), self.channels), torch.float32)]

    # ------------------------------------------------------------------ run
    def _splits(self, ctx) -> int:
        """Key ranges per (sequence, kv head group) of a one-token step: enough blocks to fill the SMs, each range at
        least ``_MIN_KEYS_PER_SPLIT`` keys."""
        span = ctx.max_context if not self.window else min(ctx.max_context, self.window + self.keep_first)
        group = self.nq // self.nkv
        blocks = ctx.n_seqs * self.nkv * -(-group // (8 if group > 4 else max(1, group)))
        most = max(1, min(span // _MIN_KEYS_PER_SPLIT, _MAX_SPLIT_PAIRS // ctx.n_seqs, 32))
        return max(1, min(most, (2 * self.runtime.sm_count) // max(blocks, 1)))

    def forward(self, x, ctx, cache):
        keys, kept = cache
        if not keys.writable:
            raise ValueError(f"{self.prefix}: this mixer's keys are made by its own convolution; it reads no other layer's cache")
        tokens = x.shape[0]
        ws = self.runtime.workspace
        proj = self.proj(x)
        q = ws.view("attn.q", tokens, self.nq, self.d)
        out = ws.view("attn.ctx", tokens, self.nq, self.d)
        table = ctx.block_table(keys.group)
        kernels.conv_qk_write(proj, self.conv, kept.state, ctx, q, keys.k, table, self.nq, self.nkv, self.d, keys.page_tokens,
                              keys.ring_tokens)
        penalty = (self.slopes, None)
        if ctx.is_decode:
            kernels.attention_decode(q, keys.k, keys.k, out, table, ctx.seq_len, self.nkv, keys.page_tokens, keys.ring_tokens, self.window,
                                     self.scale, self._splits(ctx), ws.view("attn.part_acc", _MAX_SPLIT_PAIRS * self.nq * self.d),
                                     ws.view("attn.part_ml", _MAX_SPLIT_PAIRS * self.nq * 2), penalty=penalty, keep_first=self.keep_first,
                                     sink=self.sink)
        else:
            kernels.attention_prefill(q, keys.k, keys.k, out, table, ctx.seq_start, ctx.seq_past, ctx.max_q_len, self.nkv,
                                      keys.page_tokens, keys.ring_tokens, self.window, self.scale, penalty=penalty,
                                      keep_first=self.keep_first, sink=self.sink)
        out = out.view(tokens, self.nq * self.d)
        if self.gated:
            kernels.gate_mul(out, proj, self.at_gate)
        return self.o(out)
