"""Softmax attention through a latent: per token the cache holds one normed latent vector and one rotated key part that
all heads share, and every head expands its keys and values from the latent with matrices of its own.

From the mixer's input h: the query latent c_q = rms(W_dq h) w_q and q = W_uq c_q, laid out head by head as
[``head_dim`` plain | ``rot_dim`` rotated]; W_dkv h = [``kv_rank`` | ``rot_dim``] rows, of which the first, RMS-normed with a
weight, are the latent c and the last, rotated by the position encoding, the key part k_r shared by the heads.  Head h has
k_h = W_uk_h c and v_h = W_uv_h c; its score is (q_plain_h . k_h + q_rot_h . k_r) * ``scale``, causal, plain softmax; the
concatenated heads are multiplied by sigmoid(W_g h) and projected by W_o.  Only c and k_r are cached.

What runs: since q_plain_h . (W_uk_h c) = (W_uk_h^T q_plain_h) . c, every head's query becomes
[W_uk_h^T q_plain_h | q_rot_h] (a product per head, ``kernels.head_product``) and the attention kernels run all heads
against the one cached row [c | k_r] per token, with the row's first ``kv_rank`` elements as values; the head's output is
W_uv_h (sum_j p_j c_j), a second product per head, in whose epilogue the gate is applied.  Keys and values are never
expanded per token, in prompts or in one-token steps.

A layer with ``own_kv`` false has no W_dkv: it reads the cache rows of the schedule position named by ``LayerCall.cache_of``
(which must have the same ``kv_rank``, ``rot_dim`` and rotation) under its own W_uk, W_uv, queries and everything else.

Norms, rotation (float cos/sin table), scores, softmax and the gate are float; the query latent, the queries, the cache
rows and the heads' outputs are rounded to the activation type between the products.

Parameters: ``hidden_size``, ``num_heads``, ``head_dim``, ``rot_dim``, ``v_head_dim``, ``q_rank``, ``kv_rank``, ``scale``, ``eps``,
``position`` (a position part over ``rot_dim``), ``own_kv``, ``gate``, ``float_out``, and the tensor-name pieces ``dq``, ``uq``,
``dkv``, ``uk``, ``uv``, ``g``, ``o``, ``weight_suffix``, ``norm_suffix``.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..weights.tensors import TensorSpec
from .attention import _MAX_SPLIT_PAIRS, _MIN_KEYS_PER_SPLIT
from .base import KVRequest, Runtime, part_class, register_mixer, to_device
from .linear import Linear


@register_mixer("latent_attention")
class LatentAttention:
    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix, self.runtime, self.params = prefix, runtime, params
        self.hidden = int(params["hidden_size"])
        self.heads, self.d, self.rot, self.dv = (int(params[k]) for k in ("num_heads", "head_dim", "rot_dim", "v_head_dim"))
        self.q_rank, self.rank = int(params["q_rank"]), int(params["kv_rank"])
        self.row = self.rank + self.rot                        # one cached row, and one head's query as the kernels see it
        if self.row > 640 or self.rank > 512:
            raise ValueError(f"{prefix}: a latent of {self.rank} + {self.rot} elements is beyond what the attention kernels take (512 + 128)")
        self.scale = float(params["scale"])
        self.eps = float(params.get("eps", 1e-6))
        self.own_kv = bool(params.get("own_kv", True))
        self.gated = bool(params.get("gate", True))
        position_spec = params["position"]
        self.position = part_class("position", position_spec)(position_spec.params, runtime)
        if getattr(self.position, "interleaved", False):
            raise ValueError(f"{prefix}: the latent attention kernels rotate element i with element i + dims / 2")
        self.cos_sin = None
        self.at_kv = self.q_rank
        self.at_gate = self.q_rank + (self.row if self.own_kv else 0)
        used = self.at_gate + (self.heads * self.dv if self.gated else 0)
        self.proj_rows = -(-used // 8) * 8
        self.proj = Linear("latent.proj" + ("" if self.own_kv else ".reader"), self.proj_rows, self.hidden, runtime, float_out=True)
        self.uq = Linear("latent.uq", self.heads * (self.d + self.rot), self.q_rank, runtime)
        float_out = bool(params.get("float_out", False))
        self.o = Linear("latent.o" + (".float" if float_out else ""), self.hidden, self.heads * self.dv, runtime, float_out=float_out)
        ws = runtime.workspace
        tokens = runtime.max_step_tokens
        ws.declare("latent.cq", tokens * self.q_rank, runtime.dtype)
        ws.declare("latent.q", tokens * self.heads * self.row, runtime.dtype)
        ws.declare("latent.ctx", tokens * self.heads * self.rank, runtime.dtype)
        ws.declare("latent.heads", tokens * self.heads * self.dv, runtime.dtype)
        ws.declare("attn.part_acc", _MAX_SPLIT_PAIRS * self.heads * self.rank, torch.float32)
        ws.declare("attn.part_ml", _MAX_SPLIT_PAIRS * self.heads * 2, torch.float32)
        self.q_norm = self.kv_norm = self.uk_t = self.uv = None

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _names(params, prefix: str) -> dict[str, str]:
        w, nw = str(params.get("weight_suffix", ".weight")), str(params.get("norm_suffix", ".norm"))
        n = {key: f"{prefix}.{params.get(key, key)}{w}" for key in ("dq", "uq", "dkv", "uk", "uv", "g", "o")}
        n["dq_norm"], n["dkv_norm"] = f"{prefix}.{params.get('dq', 'dq')}{nw}", f"{prefix}.{params.get('dkv', 'dkv')}{nw}"
        return n

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, heads, d, rot, dv = (int(params[k]) for k in ("hidden_size", "num_heads", "head_dim", "rot_dim", "v_head_dim"))
        q_rank, rank = int(params["q_rank"]), int(params["kv_rank"])
        n = cls._names(params, prefix)
        std = float(params.get("init_std", 0.02))
        out = {n["dq"]: TensorSpec((q_rank, hidden), init_std=std), n["dq_norm"]: TensorSpec((q_rank,), role="vector", init_std=0.1, init_mean=1.0),
               n["uq"]: TensorSpec((heads * (d + rot), q_rank), init_std=std), n["uk"]: TensorSpec((heads * d, rank), init_std=std),
               n["uv"]: TensorSpec((heads * dv, rank), init_std=std), n["o"]: TensorSpec((hidden, heads * dv), init_std=std)}
        if params.get("gate", True):
            out[n["g"]] = TensorSpec((heads * dv, hidden), init_std=std)
        if params.get("own_kv", True):
            out[n["dkv"]] = TensorSpec((rank + rot, hidden), init_std=std)
            out[n["dkv_norm"]] = TensorSpec((rank,), role="vector", init_std=0.1, init_mean=1.0)
        return out

    def load(self, source) -> None:
        n = self._names(self.params, self.prefix)
        dtype, device = self.runtime.dtype, self.runtime.device
        rows = [source(n["dq"]).to(dtype)]
        if self.own_kv:
            rows.append(source(n["dkv"]).to(dtype))
        if self.gated:
            rows.append(source(n["g"]).to(dtype))
        used = sum(r.shape[0] for r in rows)
        if self.proj_rows > used:
            rows.append(torch.zeros(self.proj_rows - used, self.hidden, dtype=dtype, device=rows[0].device))
        self.proj.set_weight(torch.cat(rows, dim=0))
        self.uq.set_weight(source(n["uq"]))
        self.o.set_weight(source(n["o"]))
        self.q_norm = to_device(source(n["dq_norm"]), torch.float32, device)
        if self.own_kv:
            self.kv_norm = to_device(source(n["dkv_norm"]), torch.float32, device)
        # W_uk per head, transposed: [heads, kv_rank, head_dim], the matrix of the product that carries a head's plain
        # query part into the latent's space; W_uv is stored as that product's matrix already: [heads, v_head_dim, kv_rank]
        self.uk_t = to_device(source(n["uk"]).view(self.heads, self.d, self.rank).transpose(1, 2), dtype, device)
        self.uv = to_device(source(n["uv"]).view(self.heads, self.dv, self.rank), dtype, device)
        tables = self.runtime.options.setdefault("position_tables", {})
        key = self.position.key() + (self.runtime.max_positions,)
        if key not in tables:
            tables[key] = self.position.table(self.runtime.max_positions)
        self.cos_sin = tables[key]

    # ------------------------------------------------------------------ what it keeps per sequence
    def cache_request(self):
        return KVRequest(1, self.row, None, shared_values=True)

    def _splits(self, ctx, page_tokens: int) -> int:
        """Partial results per (sequence, head) of a one-token step.  The tensor-core kernel runs one block per SM, each
        with up to 64 heads of a sequence and a range of its pages; with at most 16 (32) heads a block cuts the keys of
        every page into 4 (2) parts, each a partial result of its own.  The generic kernel runs four heads a block,
        several blocks per SM."""
        if kernels.attention_latent_shape(self.runtime.dtype, self.row, self.rank, page_tokens) and self.scale > 0:
            parts = 4 if self.heads <= 16 else 2 if self.heads <= 32 else 1
            if parts * ctx.n_seqs > _MAX_SPLIT_PAIRS:
                parts = 1
            blocks = ctx.n_seqs * -(-self.heads // 64)
            most = max(1, min(ctx.max_context // _MIN_KEYS_PER_SPLIT, _MAX_SPLIT_PAIRS // (ctx.n_seqs * parts), 32))
            return parts * max(1, min(most, self.runtime.sm_count // max(blocks, 1)))
        blocks = ctx.n_seqs * -(-self.heads // 4)
        most = max(1, min(ctx.max_context // _MIN_KEYS_PER_SPLIT, _MAX_SPLIT_PAIRS // ctx.n_seqs, 32))
        return max(1, min(most, (2 * self.runtime.sm_count) // max(blocks, 1)))

    # ------------------------------------------------------------------ run
    def forward(self, x, ctx, cache):
        tokens = x.shape[0]
        ws = self.runtime.workspace
        write = cache.writable and self.own_kv
        if cache.k is None or cache.k.shape[-1] != self.row:
            raise ValueError(f"{self.prefix}: the cache rows it reads are not {self.rank} + {self.rot} elements long")
        table = ctx.block_table(cache.group)
        proj = self.proj(x)
        cq = ws.view("latent.cq", tokens, self.q_rank)
        kernels.latent_prepare(proj, self.q_norm, self.kv_norm, self.eps, self.cos_sin, cq, cache.k if write else None, ctx.token_seq,
                               ctx.token_pos, table if write else None, self.rank, self.rot, cache.page_tokens, cache.ring_tokens, write_kv=write)
        q_full = self.uq(cq)                                                    # [*, T, heads * (d + rot)]
        q = ws.view("latent.q", tokens, self.heads, self.row)
        kernels.head_product(q_full, self.uk_t, q, x_row=self.heads * (self.d + self.rot), x_head=self.d + self.rot)
        kernels.latent_query_rot(q_full, self.cos_sin, ctx.token_pos, q, self.heads, self.d, self.rot, self.rank)
        out = ws.view("latent.ctx", tokens, self.heads, self.rank)
        if ctx.is_decode:
            kernels.attention_decode(q, cache.k, cache.k, out, table, ctx.seq_len, 1, cache.page_tokens, cache.ring_tokens, None, self.scale,
                                     self._splits(ctx, cache.page_tokens), ws.view("attn.part_acc", _MAX_SPLIT_PAIRS * self.heads * self.rank),
                                     ws.view("attn.part_ml", _MAX_SPLIT_PAIRS * self.heads * 2), v_dim=self.rank)
        else:
            kernels.attention_prefill(q, cache.k, cache.k, out, table, ctx.seq_start, ctx.seq_past, ctx.max_q_len, 1, cache.page_tokens,
                                      cache.ring_tokens, None, self.scale, v_dim=self.rank)
        heads = ws.view("latent.heads", tokens, self.heads, self.dv)
        kernels.head_product(out, self.uv, heads, x_row=self.heads * self.rank, x_head=self.rank,
                             gate=proj if self.gated else None, gate_offset=self.at_gate)
        return self.o(heads.view(tokens, self.heads * self.dv))
