"""Python entry to the CUDA kernels: argument checks, then a ctypes call on the current stream.

Every function works on CUDA tensors only and raises if given anything else;
there is no host implementation behind them.  ``GemmOut`` is how a matrix
product hands its result to the next kernel: either the finished matrix or
split-K partial sums that the consumer adds up in float.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from . import _build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_c_int, _c_ll, _c_float, _c_ptr = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p

_SIGNATURES = {
    "elementwise": {
        "qt_embedding": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr],
        "qt_add_bias": [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
        "qt_add_rmsnorm": [_c_ptr, _c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_float, _c_ptr, _c_int, _c_ptr, _c_int,
                           _c_int, _c_int, _c_ptr],
        "qt_qkv_treat_write": [_c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                               _c_int, _c_int, _c_float, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                               _c_int, _c_int, _c_ptr],
        "qt_qk_norm_rope_write": [_c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                  _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                  _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_ptr],
        "qt_swiglu": [_c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr],
        "qt_add_dyt": [_c_ptr, _c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_ptr, _c_int,
                       _c_int, _c_ptr],
        "qt_map_difference": [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_float, _c_ptr],
    },
    "delta_rule": {
        "qt_delta_prepare": [_c_ptr, _c_int, _c_ll, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                             _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr],
        "qt_lowrank": [_c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr],
        "qt_delta_scan": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
        "qt_gated_head_norm": [_c_ptr, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr],
        "qt_delta_scan_chunked": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                  _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    },
    "linear_attention": {
        "qt_linear_attention_scan": [_c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int,
                                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
        "qt_linear_attention_prepare": [_c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr],
        "qt_linear_attention_gate_norm": [_c_ptr, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_ptr, _c_float, _c_float, _c_ptr, _c_int, _c_int,
                                          _c_int, _c_ptr],
    },
    "attention": {
        "qt_attention_prefill": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int,
                                 _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr, _c_int, _c_int,
                                 _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
        "qt_attention_decode": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int,
                                _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int,
                                _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    },
    "layernorm": {
        "qt_add_layernorm": [_c_ptr, _c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_ptr],
        "qt_weighted_sum": [_c_ptr, _c_int, _c_int, _c_ll, _c_float, _c_ptr, _c_int, _c_int, _c_ll, _c_float, _c_ptr, _c_ll, _c_ptr],
        "qt_activation": [_c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    },
    "short_conv": {
        "qt_conv_qk_write": [_c_ptr, _c_int, _c_ll, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
                             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
        "qt_gate_mul": [_c_ptr, _c_int, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    },
    "latent": {
        "qt_latent_prepare": [_c_ptr, _c_int, _c_ll, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr,
                              _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
        "qt_latent_query_rot": [_c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                _c_int, _c_ptr],
        "qt_head_product": [_c_ptr, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ll, _c_ll, _c_int,
                            _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    },
    "attention_latent": {
        # q, cache, out, block_table, max_blocks, seq_start, seq_past, seq_len, n_seqs, max_q_len, heads, row, rank, page_tokens, scale,
        # n_splits, part_acc, part_ml, stream
        "qt_attention_latent": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                _c_float, _c_int, _c_ptr, _c_ptr, _c_ptr],
    },
    "experts": {
        "qt_experts_by_pair": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                               _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_int, _c_float, _c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_ptr],
        "qt_route_top": [_c_ptr, _c_int, _c_ll, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr],
        "qt_experts_route": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                             _c_int, _c_ptr, _c_ptr],
        "qt_experts_combine": [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr],
    },
    "experts_tc": {
        "qt_expert_gemm": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    },
    "attention_mma": {
        "qt_attention_decode_mma": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                    _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr, _c_ptr],
        "qt_attention_decode_ws": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                   _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                   _c_int, _c_int, _c_ptr, _c_ptr],
        "qt_attention_prefill_mma": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    },
    "attention_tc": {
        "qt_attention_prefill_tc": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
                                    _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr],
    },
    "gemm_simt": {
        "qt_gemm_simt": [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    },
    "gemm_tc": {
        "qt_gemm_tc": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr],
        "qt_gemm_tc_pair": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ll, _c_int, _c_ptr,
                            _c_ptr, _c_int, _c_ptr, _c_ptr],
        "qt_gemm_tc_pair_slots": [],
    },
    "gemm_fused": {
        "qt_gemm_fused": [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_ptr, _c_int, _c_int, _c_float,
                          _c_ptr, _c_int, _c_int, _c_float,
                          _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                          _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_float,
                          _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    },
    "sampling": {
        "qt_argmax": [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
        "qt_sample": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
        "qt_sample_keyed": [_c_ptr, _c_float, _c_ll, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_float, _c_ptr],
        "qt_feed_tokens": [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr],
    },
}
_BOUND: dict[str, ctypes._CFuncPtr] = {}


class KernelError(RuntimeError):
    pass


def _fn(library: str, name: str):
    fn = _BOUND.get(name)
    if fn is None:
        lib = _build.load_library(library)
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[library][name]
        fn.restype = _c_int
        _BOUND[name] = fn
    return fn


_LAUNCHES = 0


def launch_count() -> int:
    """Kernel launches made through this module since the process started."""
    return _LAUNCHES


def count_launches(n: int) -> None:
    """Account for kernels launched outside this module's calls (a replayed CUDA graph of them)."""
    global _LAUNCHES
    _LAUNCHES += n


def _call(library: str, name: str, *args, launches: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += launches
    code = _fn(library, name)(*args)
    if code != 0:
        raise KernelError(f"{name} failed ({code}): {_build.last_error(library)}")


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch, so by torch's two direct calls where it has them:
    building a Stream object costs as much host time as the rest of a launch."""
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return _RAW_STREAM(_RAW_DEVICE())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def _need(tensor: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no host path)")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if shape is not None and tuple(tensor.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(tensor.shape)}")


def _code(tensor: torch.Tensor, name: str) -> int:
    if tensor.dtype not in _CODES:
        raise KernelError(f"{name}: element type {tensor.dtype} is neither float32 nor bfloat16")
    return _CODES[tensor.dtype]


@dataclass
class GemmOut:
    """Result of a matrix product: ``tensor`` is [splits, M, N]; the value is the sum over splits.

    Rows and columns are dense (stride N, 1); the stride between splits may be larger than M * N
    when the tensor is a view of a larger buffer.
    """

    tensor: torch.Tensor

    def __post_init__(self) -> None:
        t = self.tensor
        if t.dim() != 3 or t.stride(2) != 1 or t.stride(1) != t.shape[2]:
            raise KernelError(f"GemmOut needs a [splits, M, N] tensor with dense rows, got {tuple(t.shape)} / {t.stride()}")

    @property
    def n_splits(self) -> int:
        return self.tensor.shape[0]

    @property
    def split_stride(self) -> int:
        return self.tensor.stride(0) if self.tensor.shape[0] > 1 else 0

    @property
    def rows(self) -> int:
        return self.tensor.shape[1]

    @property
    def cols(self) -> int:
        return self.tensor.shape[2]

    def value(self) -> torch.Tensor:
        """The finished matrix in float (for tests and host-side use)."""
        return self.tensor.float().sum(dim=0)


# ----------------------------------------------------------------------------- elementwise
def embedding(residual: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0) -> None:
    """residual[t] = table[ids[t]] * scale in float.  ids: int32 [T]."""
    tokens, hidden = residual.shape
    _need(residual, "residual", torch.float32)
    _need(table, "table")
    _need(ids, "ids", torch.int32, (tokens,))
    if table.shape[1] != hidden:
        raise KernelError(f"embedding: table width {table.shape[1]} != stream width {hidden}")
    _call("elementwise", "qt_embedding", _ptr(residual), _ptr(table), _ptr(ids), tokens, hidden, table.shape[0],
          _code(table, "table"), float(scale), _stream())


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    """out [T, N] float32 += bias [N] float32, in place: the bias of a projection on its float sums."""
    _need(out, "out", torch.float32)
    _need(bias, "bias", torch.float32, (out.shape[-1],))
    if out.dim() != 2:
        raise KernelError(f"add_bias: out must be [rows, cols], got {tuple(out.shape)}")
    _call("elementwise", "qt_add_bias", _ptr(out), _ptr(bias), out.shape[0], out.shape[1], _stream())


def add_rmsnorm(residual: torch.Tensor, delta: GemmOut | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None, groups: int = 1) -> None:
    """stream += delta; out = rmsnorm(stream) * weight.  With ``groups`` > 1 a row is that many equal consecutive
    parts, each divided by its own root mean square; the weight spans the whole row.

    Without ``rows`` every row of ``residual`` [T, H] is updated in place and normed into ``out`` [T, H].
    With ``rows`` (int32 [K]) only those rows are normed into ``out`` [K, H] and the stream is left as it is.
    """
    hidden = residual.shape[1]
    if groups < 1 or hidden % groups:
        raise KernelError(f"add_rmsnorm: {groups} groups do not divide a width of {hidden}")
    _need(residual, "residual", torch.float32)
    _need(weight, "weight", torch.float32, (hidden,))
    n_rows = residual.shape[0] if rows is None else rows.shape[0]
    _need(out, "out", shape=(n_rows, hidden))
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if delta is not None:
        if not delta.tensor.is_cuda or (delta.rows, delta.cols) != tuple(residual.shape):
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.tensor.shape)} does not match the stream {tuple(residual.shape)}")
    _call("elementwise", "qt_add_rmsnorm", _ptr(residual), _ptr(delta.tensor) if delta else None,
          _code(delta.tensor, "delta") if delta else F32, delta.n_splits if delta else 1,
          delta.split_stride if delta else 0, _ptr(weight), float(eps), _ptr(out), _code(out, "out"), _ptr(rows),
          n_rows, hidden, int(groups), _stream())


def qkv_treat_write(qkv: GemmOut, bias: torch.Tensor | None, q_out: torch.Tensor, k_cache: torch.Tensor | None,
                    v_cache: torch.Tensor | None, token_seq: torch.Tensor, token_pos: torch.Tensor,
                    block_table: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                    page_tokens: int, ring_tokens: int, v_norm_eps: float | None = None,
                    blend_from: torch.Tensor | None = None, blend_weight: torch.Tensor | None = None,
                    keep_to: torch.Tensor | None = None, write_kv: bool = True) -> None:
    """What follows the fused projection of a mixer without rotation: the bias, then q to ``q_out`` and k, v into the
    cache.  Values (head size ``v_head_dim``) are first divided by their root mean square per head (``v_norm_eps``
    given), then blended, v = (1 - w) v + w * ``blend_from`` [T, nkv, dv] with w = ``blend_weight`` (a float on the
    device), then copied to ``keep_to`` [T, nkv, dv] (float), each where given.  All in float.

    qkv [*, T, nq d + nkv d + nkv dv]; q_out [T, nq, d]; k cache [pages, nkv, page_tokens, d], v cache [..., dv]."""
    tokens = qkv.rows
    width = (num_heads + num_kv_heads) * head_dim + num_kv_heads * v_head_dim
    if qkv.cols != width:
        raise KernelError(f"qkv_treat_write: projection width {qkv.cols} != nq d + nkv d + nkv dv = {width}")
    _need(q_out, "q_out", shape=(tokens, num_heads, head_dim))
    _need(token_seq, "token_seq", torch.int32, (tokens,))
    _need(token_pos, "token_pos", torch.int32, (tokens,))
    if bias is not None:
        _need(bias, "bias", torch.float32, (width,))
    max_blocks = 0
    if write_kv:
        _need(block_table, "block_table", torch.int32)
        max_blocks = block_table.shape[1]
        for name, cache, size in (("k_cache", k_cache, head_dim), ("v_cache", v_cache, v_head_dim)):
            _need(cache, name, q_out.dtype)
            if tuple(cache.shape[1:]) != (num_kv_heads, page_tokens, size):
                raise KernelError(f"{name}: shape {tuple(cache.shape)} is not [pages, {num_kv_heads}, {page_tokens}, {size}]")
    for name, side in (("blend_from", blend_from), ("keep_to", keep_to)):
        if side is not None:
            _need(side, name, torch.float32, (tokens, num_kv_heads, v_head_dim))
    if blend_from is not None:
        _need(blend_weight, "blend_weight", torch.float32)
    _call("elementwise", "qt_qkv_treat_write", _ptr(qkv.tensor), _code(qkv.tensor, "qkv"), qkv.n_splits, qkv.split_stride,
          _ptr(bias), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _code(q_out, "q_out"), _ptr(token_seq), _ptr(token_pos),
          _ptr(block_table), max_blocks, 0 if v_norm_eps is None else 1, float(v_norm_eps or 0.0), _ptr(blend_from),
          _ptr(blend_weight), _ptr(keep_to), tokens, num_heads, num_kv_heads, head_dim, v_head_dim, page_tokens, ring_tokens,
          1 if write_kv else 0, _stream())


def qk_norm_rope_write(qkv: GemmOut, q_out: torch.Tensor, k_cache: torch.Tensor | None, v_cache: torch.Tensor | None,
                       token_seq: torch.Tensor, token_pos: torch.Tensor, block_table: torch.Tensor | None,
                       q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                       cos_sin: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int,
                       page_tokens: int, ring_tokens: int, write_kv: bool = True, kv_in_proj: bool = True,
                       interleaved: bool = False, v_heads: int | None = None, v_head_dim: int | None = None, unit_norm: bool = False,
                       row_inv: torch.Tensor | None = None, extra_cols: int = 0) -> None:
    """Per-head q/k RMSNorm, rotation and the cache write, from the fused projection output.

    ``unit_norm``: q and k heads are divided by their root mean square without a weight (no q_weight / k_weight).
    ``row_inv`` (float scratch [T, 2]): q and k are normed over all their heads at once, with weights [nq d] and [nkv d].
    ``extra_cols``: further columns of the projection behind q, k and v, which are left alone.

    qkv [*, T, (nq + 2 nkv) d]; q_out [T, nq, d]; caches [pages, nkv, page_tokens, d]; cos_sin float [P, rd]
    (cos | sin of the rd/2 pair angles); pairs are (i, i + rd/2), or (2i, 2i + 1) with ``interleaved``.
    With ``v_heads`` / ``v_head_dim`` the values have a head count and size of their own: qkv is then
    [*, T, (nq + nkv) d + nv dv] and the value cache [pages, nv, page_tokens, dv].
    """
    tokens = qkv.rows
    nv, dv = int(v_heads or num_kv_heads), int(v_head_dim or head_dim)
    width = num_heads * head_dim + ((num_kv_heads * head_dim + nv * dv) if kv_in_proj else 0) + int(extra_cols)
    whole = row_inv is not None
    if whole:
        _need(row_inv, "row_inv", torch.float32, (tokens, 2))
    if qkv.cols != width:
        raise KernelError(f"qk_norm_rope_write: projection width {qkv.cols} != nq d + nkv d + nv dv = {width}")
    _need(q_out, "q_out", shape=(tokens, num_heads, head_dim))
    _need(token_seq, "token_seq", torch.int32, (tokens,))
    _need(token_pos, "token_pos", torch.int32, (tokens,))
    for name, w, heads in (("q_weight", q_weight, num_heads), ("k_weight", k_weight, num_kv_heads)):
        if w is not None:
            _need(w, name, torch.float32, (heads * head_dim if whole else head_dim,))
    rotary_dim, max_pos = 0, 0
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        max_pos, rotary_dim = cos_sin.shape
    max_blocks = 0
    if write_kv:
        _need(block_table, "block_table", torch.int32)
        max_blocks = block_table.shape[1]
        for name, cache, heads, size in (("k_cache", k_cache, num_kv_heads, head_dim), ("v_cache", v_cache, nv, dv)):
            _need(cache, name, q_out.dtype)
            if tuple(cache.shape[1:]) != (heads, page_tokens, size):
                raise KernelError(f"{name}: shape {tuple(cache.shape)} is not [pages, {heads}, {page_tokens}, {size}]")
    _call("elementwise", "qt_qk_norm_rope_write", _ptr(qkv.tensor), _code(qkv.tensor, "qkv"), qkv.n_splits,
          qkv.split_stride, _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _code(q_out, "q_out"), _ptr(token_seq),
          _ptr(token_pos), _ptr(block_table), max_blocks, _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos_sin),
          rotary_dim, max_pos, tokens, num_heads, num_kv_heads, head_dim, page_tokens, ring_tokens,
          1 if write_kv else 0, 1 if kv_in_proj else 0, 1 if interleaved else 0, nv, dv, 1 if unit_norm else 0, 1 if whole else 0,
          _ptr(row_inv), int(extra_cols), _stream())


def add_dyt(residual: torch.Tensor, deltas, weight: torch.Tensor, bias: torch.Tensor, alpha: float, out: torch.Tensor,
            rows: torch.Tensor | None = None) -> None:
    """stream += the deltas (up to two ``GemmOut`` of float sums); out = tanh(alpha * stream) * weight + bias.

    Without ``rows`` every row of ``residual`` [T, H] is updated in place and normed into ``out`` [T, H]; with ``rows``
    (int32 [K]) only those rows are normed into ``out`` [K, H] and the stream is left as it is."""
    hidden = residual.shape[1]
    _need(residual, "residual", torch.float32)
    _need(weight, "weight", torch.float32, (hidden,))
    _need(bias, "bias", torch.float32, (hidden,))
    n_rows = residual.shape[0] if rows is None else rows.shape[0]
    _need(out, "out", shape=(n_rows, hidden))
    if rows is not None:
        _need(rows, "rows", torch.int32)
    deltas = [d for d in deltas if d is not None]
    if len(deltas) > 2:
        raise KernelError(f"add_dyt: {len(deltas)} pending additions (at most two)")
    args = []
    for delta in deltas + [None] * (2 - len(deltas)):
        if delta is None:
            args += [None, 1, 0]
            continue
        if not delta.tensor.is_cuda or delta.tensor.dtype != torch.float32 or (delta.rows, delta.cols) != tuple(residual.shape):
            raise KernelError(f"add_dyt: a delta of {tuple(delta.tensor.shape)} {delta.tensor.dtype} for a float stream {tuple(residual.shape)}")
        args += [_ptr(delta.tensor), delta.n_splits, delta.split_stride]
    _call("elementwise", "qt_add_dyt", _ptr(residual), *args, _ptr(weight), _ptr(bias), float(alpha), _ptr(out), _code(out, "out"),
          _ptr(rows), n_rows, hidden, _stream())


def map_difference(ctx: torch.Tensor, out: torch.Tensor, lam: float, eps: float, post: float) -> None:
    """Two attention maps into one head: ctx [T, 2 * H, dv] holds the maps' results map-major; out [T, H, dv] =
    unit_rms(ctx[:, h] - lam * ctx[:, H + h]) * post, the root mean square over dv with ``eps`` inside the root."""
    tokens, heads, dv = out.shape
    _need(out, "out")
    _need(ctx, "ctx", out.dtype, (tokens, 2 * heads, dv))
    _call("elementwise", "qt_map_difference", _ptr(ctx), _ptr(out), _code(out, "out"), tokens, heads, dv, float(lam), float(eps),
          float(post), _stream())


def add_layernorm(residual: torch.Tensor, delta: GemmOut | None, post_weight: torch.Tensor | None, weight: torch.Tensor | None, eps: float,
                  out: torch.Tensor, rows: torch.Tensor | None = None, post_bias: torch.Tensor | None = None,
                  bias: torch.Tensor | None = None) -> None:
    """Layer norm around the float stream: d = delta, normed with ``post_weight`` (and ``post_bias``) first where that is given;
    stream += d; out = (stream - mean) / sqrt(var + eps) * weight (+ ``bias``), the variance being the mean squared deviation.
    Without ``weight`` the new stream itself is written to ``out`` (in its element type).

    Without ``rows`` every row of ``residual`` [T, H] is updated in place and normed into ``out`` [T, H]; with ``rows``
    (int32 [K]) only those rows are normed into ``out`` [K, H] and the stream is left as it is."""
    hidden = residual.shape[1]
    _need(residual, "residual", torch.float32)
    for name, vector in (("weight", weight), ("post_weight", post_weight), ("bias", bias), ("post_bias", post_bias)):
        if vector is not None:
            _need(vector, name, torch.float32, (hidden,))
    n_rows = residual.shape[0] if rows is None else rows.shape[0]
    _need(out, "out", shape=(n_rows, hidden))
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if delta is not None and (not delta.tensor.is_cuda or (delta.rows, delta.cols) != tuple(residual.shape)):
        raise KernelError(f"add_layernorm: delta {tuple(delta.tensor.shape)} does not match the stream {tuple(residual.shape)}")
    _call("layernorm", "qt_add_layernorm", _ptr(residual), _ptr(delta.tensor) if delta else None,
          _code(delta.tensor, "delta") if delta else F32, delta.n_splits if delta else 1, delta.split_stride if delta else 0,
          _ptr(post_weight), _ptr(post_bias), _ptr(weight), _ptr(bias), float(eps), _ptr(out), _code(out, "out"), _ptr(rows), n_rows, hidden,
          _stream())


def weighted_sum(a: GemmOut, wa: float, b: GemmOut, wb: float, out: torch.Tensor) -> GemmOut:
    """out [T, N] (float) = wa * a + wb * b, the two products' split sums added in their order."""
    if (a.rows, a.cols) != (b.rows, b.cols):
        raise KernelError(f"weighted_sum: {tuple(a.tensor.shape)} and {tuple(b.tensor.shape)}")
    _need(a.tensor, "a")
    _need(b.tensor, "b")
    _need(out, "out", torch.float32, (a.rows, a.cols))
    _call("layernorm", "qt_weighted_sum", _ptr(a.tensor), _code(a.tensor, "a"), a.n_splits, a.split_stride, float(wa), _ptr(b.tensor),
          _code(b.tensor, "b"), b.n_splits, b.split_stride, float(wb), _ptr(out), a.rows * a.cols, _stream())
    return GemmOut(out.view(1, a.rows, a.cols))


def activation(x: GemmOut, out: torch.Tensor, name: str = "gelu") -> None:
    """out [T, N] = act(x) elementwise in float, x a product's sums; ``name`` is one of ``ACTIVATIONS``."""
    _need(out, "out", shape=(x.rows, x.cols))
    _call("layernorm", "qt_activation", _ptr(x.tensor), _code(x.tensor, "x"), x.n_splits, x.split_stride, _ptr(out), _code(out, "out"),
          x.rows, x.cols, activation_code(name), _stream())


def conv_qk_write(proj: GemmOut, taps: torch.Tensor, kept: torch.Tensor, ctx, q_out: torch.Tensor, k_cache: torch.Tensor | None,
                  block_table: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int, page_tokens: int,
                  ring_tokens: int, write_kv: bool = True) -> None:
    """A short causal convolution over time on every channel of the queries and keys that lead the columns of ``proj``
    (float sums [*, T, >= (nq + nkv) d]), in float: ``taps`` [channels, n] with the last column the current token's; the
    inputs before a step's first token come from ``kept`` [slots + 1, n - 1, channels], zeros at a sequence's start,
    which is then brought up to date.  Queries go to ``q_out`` [T, nq, d], keys into the paged cache."""
    tokens = proj.rows
    channels = (num_heads + num_kv_heads) * head_dim
    n_taps = taps.shape[1]
    _need(proj.tensor, "proj", torch.float32)
    _need(taps, "taps", torch.float32, (channels, n_taps))
    _need(kept, "kept", torch.float32)
    if tuple(kept.shape[1:]) != (max(n_taps - 1, 1), channels):
        raise KernelError(f"conv_qk_write: kept inputs {tuple(kept.shape)} are not [slots, {max(n_taps - 1, 1)}, {channels}]")
    _need(q_out, "q_out", shape=(tokens, num_heads, head_dim))
    max_blocks = 0
    if write_kv:
        _need(block_table, "block_table", torch.int32)
        max_blocks = block_table.shape[1]
        _need(k_cache, "k_cache", q_out.dtype)
        if tuple(k_cache.shape[1:]) != (num_kv_heads, page_tokens, head_dim):
            raise KernelError(f"k_cache: shape {tuple(k_cache.shape)} is not [pages, {num_kv_heads}, {page_tokens}, {head_dim}]")
    _call("short_conv", "qt_conv_qk_write", _ptr(proj.tensor), proj.n_splits, proj.split_stride, proj.cols, _ptr(taps), _ptr(kept),
          _ptr(ctx.token_seq), _ptr(ctx.token_pos), _ptr(ctx.seq_start), _ptr(ctx.slots), _ptr(q_out), _ptr(k_cache), _code(q_out, "q_out"),
          _ptr(block_table), max_blocks, tokens, ctx.n_seqs, num_heads, num_kv_heads, head_dim, n_taps, page_tokens, ring_tokens,
          1 if write_kv else 0, _stream(), launches=2 if n_taps > 1 else 1)


def gate_mul(x: torch.Tensor, gate: GemmOut, offset: int, group: int = 1) -> None:
    """x [T, N] *= sigmoid(columns ``offset`` .. ``offset + N`` of ``gate``), in float, in place.  With ``group`` > 1 every
    ``group`` consecutive columns of x share one gate column (one number per head): columns ``offset`` .. ``offset + N / group``."""
    _need(x, "x")
    _need(gate.tensor, "gate", torch.float32)
    if x.dim() != 2 or gate.rows != x.shape[0]:
        raise KernelError(f"gate_mul: x {tuple(x.shape)} and a gate of {gate.rows} rows")
    _call("short_conv", "qt_gate_mul", _ptr(x), _code(x, "x"), _ptr(gate.tensor), gate.n_splits, gate.split_stride, gate.cols, int(offset),
          x.shape[0], x.shape[1], int(group), _stream())


def latent_prepare(proj: GemmOut, q_norm: torch.Tensor, kv_norm: torch.Tensor | None, eps: float, cos_sin: torch.Tensor | None,
                   cq_out: torch.Tensor, cache: torch.Tensor | None, token_seq: torch.Tensor, token_pos: torch.Tensor,
                   block_table: torch.Tensor | None, rank: int, rot: int, page_tokens: int, ring_tokens: int, write_kv: bool = True) -> None:
    """From the float sums ``proj`` [*, T, >= q_rank (+ rank + rot)] of a latent-attention mixer's first projection: the
    query latent's RMS norm (``q_norm`` [q_rank]) into ``cq_out`` [T, q_rank] and, with ``write_kv``, the cache row of every
    token: the key/value latent's RMS norm (``kv_norm`` [rank]) followed by the shared key part of ``rot`` elements, of
    which the first ``cos_sin.shape[1]`` are rotated by the token's position.  ``cache`` is [pages, 1, page_tokens, rank + rot]."""
    tokens = proj.rows
    q_rank = q_norm.shape[0]
    _need(proj.tensor, "proj", torch.float32)
    _need(q_norm, "q_norm", torch.float32)
    _need(cq_out, "cq_out", shape=(tokens, q_rank))
    _need(token_seq, "token_seq", torch.int32, (tokens,))
    _need(token_pos, "token_pos", torch.int32, (tokens,))
    rotary_dim, max_pos, max_blocks = 0, 0, 0
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        max_pos, rotary_dim = cos_sin.shape
    if write_kv:
        _need(kv_norm, "kv_norm", torch.float32, (rank,))
        _need(block_table, "block_table", torch.int32)
        max_blocks = block_table.shape[1]
        _need(cache, "cache", cq_out.dtype)
        if tuple(cache.shape[1:]) != (1, page_tokens, rank + rot):
            raise KernelError(f"cache: shape {tuple(cache.shape)} is not [pages, 1, {page_tokens}, {rank + rot}]")
    _call("latent", "qt_latent_prepare", _ptr(proj.tensor), proj.n_splits, proj.split_stride, proj.cols, _ptr(q_norm), _ptr(kv_norm),
          float(eps), _ptr(cos_sin), rotary_dim, max_pos, _ptr(cq_out), _ptr(cache), _code(cq_out, "cq_out"), _ptr(token_seq),
          _ptr(token_pos), _ptr(block_table), max_blocks, tokens, q_rank, int(rank), int(rot), page_tokens, ring_tokens,
          1 if write_kv else 0, _stream())


def latent_query_rot(q: GemmOut, cos_sin: torch.Tensor | None, token_pos: torch.Tensor, out: torch.Tensor, heads: int, dim: int, rot: int,
                     out_offset: int) -> None:
    """The last ``rot`` elements of every head of ``q`` [*, T, heads (dim + rot)], the first ``cos_sin.shape[1]`` of them
    rotated by the token's position, into ``out`` [T, heads, row] at ``out_offset`` of every head's row."""
    tokens = q.rows
    if q.cols != heads * (dim + rot) or out.dim() != 3 or tuple(out.shape[:2]) != (tokens, heads):
        raise KernelError(f"latent_query_rot: q {tuple(q.tensor.shape)}, out {tuple(out.shape)} for {heads} heads of {dim} + {rot}")
    _need(out, "out")
    _need(token_pos, "token_pos", torch.int32, (tokens,))
    rotary_dim = 0
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        rotary_dim = cos_sin.shape[1]
    _call("latent", "qt_latent_query_rot", _ptr(q.tensor), _code(q.tensor, "q"), q.n_splits, q.split_stride, _ptr(cos_sin), rotary_dim,
          _ptr(token_pos), _ptr(out), _code(out, "out"), tokens, heads, dim, rot, out.shape[2], int(out_offset), _stream())


def head_product(x, weight: torch.Tensor, out: torch.Tensor, *, x_row: int, x_head: int, x_offset: int = 0, out_offset: int = 0,
                 gate: GemmOut | None = None, gate_offset: int = 0) -> None:
    """A product per head: out[t, h, out_offset + n] = sum_k x[t, h, k] weight[h, n, k], every head with a matrix of its own,
    summed in float.  ``x`` is a tensor or a ``GemmOut`` (partial sums are added first) whose element (t, h, k) lies at
    t * x_row + h * x_head + x_offset + k; ``out`` is [T, heads, row].  With ``gate`` (float sums [*, T, cols]) the result
    is multiplied by sigmoid(gate[t, gate_offset + h * N + n])."""
    heads, n, k = weight.shape
    _need(weight, "weight")
    _need(out, "out")
    tokens = out.shape[0]
    if out.dim() != 3 or out.shape[1] != heads or out_offset + n > out.shape[2]:
        raise KernelError(f"head_product: out {tuple(out.shape)} for {heads} heads of {n} at {out_offset}")
    if isinstance(x, GemmOut):
        x_tensor, splits, stride = x.tensor, x.n_splits, x.split_stride
    else:
        _need(x, "x")
        x_tensor, splits, stride = x, 1, 0
    if gate is not None:
        _need(gate.tensor, "gate", torch.float32)
    _call("latent", "qt_head_product", _ptr(x_tensor), _code(x_tensor, "x"), splits, stride, int(x_row), int(x_head), int(x_offset),
          _ptr(weight), _code(weight, "weight"), _ptr(out), _code(out, "out"), out.shape[1] * out.shape[2], out.shape[2], int(out_offset),
          _ptr(gate.tensor) if gate is not None else None, gate.n_splits if gate is not None else 1,
          gate.split_stride if gate is not None else 0, gate.cols if gate is not None else 0, int(gate_offset), tokens, heads, n, k, _stream())


# ----------------------------------------------------------------------------- the gated delta rule
def delta_prepare(proj: GemmOut, taps: torch.Tensor, kept: torch.Tensor, ctx, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                  beta: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, unit_eps: float) -> None:
    """What stands between the first projection of a delta-rule mixer and its recurrence, in float: the short causal
    convolution per channel over q | k | v (``taps`` [channels, n_taps], last column the current token's; the inputs
    before a step's first token come from ``kept`` [slots + 1, n_taps - 1, channels], which is then brought up to
    date), SiLU, q and k to unit length per head (``unit_eps`` inside the root; q also times dim^-1/2), and
    beta = sigmoid of the ``heads`` columns behind q | k | v.  ``ctx`` is the step (sequence and position of every
    token, the sequences' first rows, lengths before the step and slots)."""
    tokens = proj.rows
    channels = 2 * kv_heads * dim + heads * vdim
    n_taps = taps.shape[1]
    _need(proj.tensor, "proj", torch.float32)
    _need(taps, "taps", torch.float32, (channels, n_taps))
    _need(kept, "kept", torch.float32)
    if tuple(kept.shape[1:]) != (n_taps - 1, channels):
        raise KernelError(f"delta_prepare: kept inputs {tuple(kept.shape)} are not [slots, {n_taps - 1}, {channels}]")
    _need(q, "q", torch.float32, (tokens, kv_heads, dim))
    _need(k, "k", torch.float32, (tokens, kv_heads, dim))
    _need(v, "v", torch.float32, (tokens, heads, vdim))
    _need(beta, "beta", torch.float32, (tokens, heads))
    _call("delta_rule", "qt_delta_prepare", _ptr(proj.tensor), proj.n_splits, proj.split_stride, proj.cols, _ptr(taps), _ptr(kept),
          _ptr(ctx.token_seq), _ptr(ctx.token_pos), _ptr(ctx.seq_start), _ptr(ctx.seq_past), _ptr(ctx.slots), _ptr(q), _ptr(k), _ptr(v),
          _ptr(beta), tokens, ctx.n_seqs, heads, kv_heads, dim, vdim, n_taps, float(unit_eps), _stream(), launches=2 if n_taps > 1 else 1)


def lowrank(proj: GemmOut, offset: int, weight: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
            rate_log: torch.Tensor | None = None, per_rate: int = 0) -> None:
    """out [T, N] (float) = f(weight^T x + bias) for x = columns ``offset`` .. ``offset + rank`` of ``proj`` and
    ``weight`` [rank, N] (float, the second matrix of a projection through a few columns, transposed).  With
    ``rate_log`` [N / per_rate] f is the logarithm of a decay, -exp(rate_log[n / per_rate]) * softplus(.); else the sigmoid."""
    rank, n_out = weight.shape
    _need(proj.tensor, "proj", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(out, "out", torch.float32, (proj.rows, n_out))
    if bias is not None:
        _need(bias, "bias", torch.float32, (n_out,))
    if rate_log is not None:
        _need(rate_log, "rate_log", torch.float32, (n_out // max(per_rate, 1),))
    _call("delta_rule", "qt_lowrank", _ptr(proj.tensor), proj.n_splits, proj.split_stride, proj.cols, int(offset), rank, _ptr(weight),
          _ptr(bias), _ptr(rate_log), int(per_rate), _ptr(out), proj.rows, n_out, 0 if rate_log is not None else 1, _stream())


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
               out: torch.Tensor, ctx) -> None:
    """The gated delta rule over the tokens of every sequence of the step, from and into ``state``
    [slots + 1, heads, dim, vdim] (float): S <- diag(exp(decay_t)) S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T;
    out_t = S^T q_t.  q, k [T, kv_heads, dim]; v, out [T, heads, vdim]; beta [T, heads]; decay [T, heads, dim], the decays'
    logarithms.  Token by token: the form for steps of few tokens per sequence."""
    tokens, heads, vdim = v.shape
    kv_heads, dim = q.shape[1], q.shape[2]
    for name, tensor, shape in (("q", q, (tokens, kv_heads, dim)), ("k", k, (tokens, kv_heads, dim)), ("v", v, (tokens, heads, vdim)),
                                ("beta", beta, (tokens, heads)), ("decay", decay, (tokens, heads, dim)), ("out", out, (tokens, heads, vdim))):
        _need(tensor, name, torch.float32, shape)
    _need(state, "state", torch.float32)
    if tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"delta_scan: state {tuple(state.shape)} is not [slots, {heads}, {dim}, {vdim}]")
    _call("delta_rule", "qt_delta_scan", _ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(decay), _ptr(state), _ptr(out), _ptr(ctx.seq_start),
          _ptr(ctx.slots), ctx.n_seqs, heads, kv_heads, dim, vdim, _stream())


DELTA_CHUNK = 16               # tokens per chunk of the chunked recurrence
DELTA_CHUNKED_MAX_DIM = 256    # key channels per head it takes


def delta_scan_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                       out: torch.Tensor, scratch: torch.Tensor, ctx) -> None:
    """The same recurrence as ``delta_scan`` in chunks of 16 tokens: what does not depend on the state (keys and queries
    scaled by the running decays, the chunk's two triangular matrices) is made for all chunks at once, and the walk over
    a sequence's chunks has no chain from token to token.  Float throughout; results differ from the token-by-token
    form by rounding.  ``scratch``: float, at least T * heads * (4 * dim + 36) elements."""
    tokens, heads, vdim = v.shape
    kv_heads, dim = q.shape[1], q.shape[2]
    for name, tensor, shape in (("q", q, (tokens, kv_heads, dim)), ("k", k, (tokens, kv_heads, dim)), ("v", v, (tokens, heads, vdim)),
                                ("beta", beta, (tokens, heads)), ("decay", decay, (tokens, heads, dim)), ("out", out, (tokens, heads, vdim))):
        _need(tensor, name, torch.float32, shape)
    _need(state, "state", torch.float32)
    if tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"delta_scan_chunked: state {tuple(state.shape)} is not [slots, {heads}, {dim}, {vdim}]")
    _need(scratch, "scratch", torch.float32)
    rows = tokens * heads * dim
    if scratch.numel() < 4 * rows + tokens * heads * (2 * DELTA_CHUNK + 4):
        raise KernelError("delta_scan_chunked: the scratch buffer is too small")
    parts = [scratch[i * rows:(i + 1) * rows] for i in range(4)] + [scratch[4 * rows:]]
    _call("delta_rule", "qt_delta_scan_chunked", _ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(decay), _ptr(state), _ptr(out),
          *[_ptr(part) for part in parts], _ptr(ctx.seq_start), _ptr(ctx.slots), ctx.n_seqs, int(ctx.max_q_len), heads, kv_heads, dim, vdim,
          _stream(), launches=2)


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out [T, heads, vdim] = o / sqrt(mean(o^2) + eps) * weight [vdim] * gate, per head; o and gate float."""
    tokens, heads, vdim = o.shape
    _need(o, "o", torch.float32)
    if gate is not None:
        _need(gate, "gate", torch.float32, (tokens, heads, vdim))
    _need(weight, "weight", torch.float32, (vdim,))
    _need(out, "out", shape=(tokens, heads, vdim))
    _call("delta_rule", "qt_gated_head_norm", _ptr(o), _ptr(gate), _ptr(weight), float(eps), _ptr(out), _code(out, "out"), tokens, heads,
          vdim, _stream())


LINEAR_ATTENTION_MAX_DIM = 256     # key channels per head that the decayed linear attention's kernel holds


def linear_attention_scan(proj: GemmOut, at_q: int, at_k: int, at_v: int, decay: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
                          ctx, dim: int, act: bool = True) -> None:
    """Linear attention with a constant decay per head over the step's packed sequences: per head S <- decay_h S + k_t v_t^T,
    o_t = S^T q_t, float throughout.  q, k ([heads, dim]) and v ([heads, vdim]) are the columns of ``proj`` (float sums
    [*, T, cols]) from ``at_q``, ``at_k``, ``at_v`` on, and pass SiLU first where ``act``.  ``state`` [slots, heads, vdim, dim]
    (the state transposed) is read and written at the rows ``ctx.slots`` names; ``out`` [T, heads, vdim]."""
    tokens, heads, vdim = out.shape
    _need(proj.tensor, "proj", torch.float32)
    _need(out, "out", torch.float32)
    _need(decay, "decay", torch.float32, (heads,))
    _need(state, "state", torch.float32)
    if proj.rows != tokens or tuple(state.shape[1:]) != (heads, vdim, dim):
        raise KernelError(f"linear_attention_scan: state {tuple(state.shape)} is not [slots, {heads}, {vdim}, {dim}], or {proj.rows} rows for {tokens} tokens")
    _call("linear_attention", "qt_linear_attention_scan", _ptr(proj.tensor), proj.n_splits, proj.split_stride, proj.cols, int(at_q), int(at_k),
          int(at_v), _ptr(decay), _ptr(state), _ptr(out), _ptr(ctx.seq_start), _ptr(ctx.slots), ctx.n_seqs, heads, int(dim), vdim,
          1 if act else 0, int(ctx.max_q_len), _stream())


def linear_attention_prepare(proj: GemmOut, cols: int, out: torch.Tensor, act: bool = True) -> GemmOut:
    """out [T, cols] (float) = SiLU (with ``act``) of the first ``cols`` columns of ``proj`` (float sums [*, T, all]): q, k
    and v of a step summed and activated once, ahead of the recurrence."""
    _need(proj.tensor, "proj", torch.float32)
    _need(out, "out", torch.float32, (proj.rows, int(cols)))
    _call("linear_attention", "qt_linear_attention_prepare", _ptr(proj.tensor), proj.n_splits, proj.split_stride, proj.cols, int(cols), _ptr(out),
          proj.rows, 1 if act else 0, _stream())
    return GemmOut(out.view(1, proj.rows, int(cols)))


def linear_attention_gate_norm(o: torch.Tensor, proj: GemmOut | None, at_gate: int, weight: torch.Tensor, eps: float, scale: float,
                               out: torch.Tensor) -> None:
    """out [T, N] = o / sqrt(mean(o^2) + eps) * weight * sigmoid(columns ``at_gate`` .. of ``proj``) * scale, the mean over the
    token's whole row (all heads at once); o float, rounded once to ``out``'s type."""
    tokens, width = o.shape
    _need(o, "o", torch.float32)
    _need(weight, "weight", torch.float32, (width,))
    _need(out, "out", shape=(tokens, width))
    if proj is not None:
        _need(proj.tensor, "proj", torch.float32)
    _call("linear_attention", "qt_linear_attention_gate_norm", _ptr(o), _ptr(proj.tensor) if proj is not None else None,
          proj.n_splits if proj is not None else 1, proj.split_stride if proj is not None else 0, proj.cols if proj is not None else 0,
          int(at_gate), _ptr(weight), float(eps), float(scale), _ptr(out), _code(out, "out"), tokens, width, _stream())


SWIGLU_GROUP = 16      # rows of gate and of up that alternate in a weight laid out for the GEMM's gated epilogue
# gate activations of a gated feed-forward, act(gate) * up: names a configuration may use -> the kernels' codes
ACTIVATIONS = {"silu": 0, "swish": 0, "gelu_pytorch_tanh": 1, "gelu_tanh": 1, "gelu": 2, "relu": 3}
# a gate that also treats the up value and has a parameter ``limit``: g' = min(g, limit), u' = clamp(u, -limit, limit),
# y = g' sigmoid(1.702 g') (u' + 1).  Taken, with ``limit``, by ``swiglu``, the experts' kernels and the products' gated epilogues.
CAPPED_GATE = "capped_sigmoid"
_CAPPED_CODE = 4


def activation_code(name: str, capped_ok: bool = False) -> int:
    if capped_ok and name == CAPPED_GATE:
        return _CAPPED_CODE
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"unknown gate activation {name!r}; the kernels compute {sorted(ACTIVATIONS)}") from None



def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int) -> torch.Tensor:
    """[gate; up] with the rows alternating ``group`` of gate and ``group`` of up (``group`` 0: gate, then up)."""
    if group == 0:
        return torch.cat((gate, up), dim=0)
    inter, hidden = gate.shape
    if inter % group:
        raise KernelError(f"rows in groups of {group} do not divide {inter}")
    return torch.stack((gate.view(inter // group, group, hidden), up.view(inter // group, group, hidden)), dim=1).reshape(2 * inter, hidden)


def swiglu(gate_up: GemmOut, out: torch.Tensor, group: int = 0, activation: str = "silu", limit: float = 0.0) -> None:
    """out[t, i] = act(gate[t, i]) * up[t, i] where gate_up[t] holds gate then up (``group`` 0) or alternates
    ``group`` elements of gate and ``group`` of up; ``activation`` is one of ``ACTIVATIONS``."""
    tokens, inter = out.shape
    _need(out, "out")
    if (gate_up.rows, gate_up.cols) != (tokens, 2 * inter):
        raise KernelError(f"swiglu: input {tuple(gate_up.tensor.shape)} does not match output {tuple(out.shape)}")
    _call("elementwise", "qt_swiglu", _ptr(gate_up.tensor), _code(gate_up.tensor, "gate_up"), gate_up.n_splits,
          gate_up.split_stride, _ptr(out), _code(out, "out"), tokens, inter, int(group), activation_code(activation, True), float(limit),
          _stream())


# ----------------------------------------------------------------------------- attention
def _check_attention(q, k_cache, v_cache, out, block_table, num_kv_heads, page_tokens, penalty=None, v_dim=None):
    _need(q, "q")
    tokens, num_heads, head_dim = q.shape
    _need(k_cache, "k_cache", q.dtype)
    _need(v_cache, "v_cache", q.dtype)
    if v_dim is not None and not 0 < v_dim <= v_cache.shape[-1]:
        raise KernelError(f"values of {v_dim} elements in cache rows of {v_cache.shape[-1]}")
    v_dim = v_dim or v_cache.shape[-1]              # values may have a head size of their own, or be the head of longer rows
    _need(out, "out", q.dtype, (tokens, num_heads, v_dim))
    if tuple(k_cache.shape[1:]) != (num_kv_heads, page_tokens, head_dim):
        raise KernelError(f"cache shape {tuple(k_cache.shape)} is not [pages, {num_kv_heads}, {page_tokens}, {head_dim}]")
    if (v_cache.shape[0], v_cache.shape[2]) != (k_cache.shape[0], k_cache.shape[2]) or num_kv_heads % v_cache.shape[1]:
        raise KernelError(f"value cache {tuple(v_cache.shape)} does not go with key cache {tuple(k_cache.shape)}")
    _need(block_table, "block_table", torch.int32)
    if penalty is not None:
        for name, factor in zip(("r1", "r2"), penalty):
            if factor is not None or name == "r1":
                _need(factor, f"distance penalty {name}", torch.float32, (num_heads,))
    return tokens, num_heads, head_dim


def _extended_choice(q, k_cache, v_cache, page_tokens: int, ring_tokens: int, scale: float, penalty, keep_first: int, sink: bool, v_dim,
                     chunk, impl: str | None, mma: str) -> str | None:
    """The kernel for a call that asks for a linear distance penalty (``penalty`` = (slopes, None)), kept first keys, a
    softmax sink, or values that are the head of the cached key rows; None for a call that asks for none of these.  The
    mma.sync kernels (``mma`` names the caller's) compute the first three for values as wide as the keys; the generic
    kernels compute all four."""
    if not ((penalty is not None and penalty[1] is None) or keep_first > 0 or sink or v_dim is not None):
        return None
    fits = (v_dim is None and v_cache.shape[-1] == q.shape[2] and attention_mma_supported(q, page_tokens) and scale > 0
            and not (keep_first > 0 and (ring_tokens or chunk)))
    if impl in (None, mma) and fits:
        return mma
    if impl in (None, "generic"):
        return "generic"
    raise KernelError(f"attention kernel {impl!r} does not take this call (linear penalty, kept first keys, sink or values inside the key rows)")


def _plain_attention(q: torch.Tensor, v_cache: torch.Tensor, penalty) -> bool:
    """Whether every tensor-core attention kernel may take this call: values as wide as keys, no distance penalty."""
    return penalty is None and v_cache.shape[-1] == q.shape[2]


def _special_mask(k_cache: torch.Tensor, v_cache: torch.Tensor, chunk) -> bool:
    """A mask in chunks, or fewer value heads than key heads: every kernel computes these but the block-tile decode
    kernel ("mma" for one-token steps)."""
    return bool(chunk) or v_cache.shape[1] != k_cache.shape[1]


def _penalised_choice(q: torch.Tensor, v_cache: torch.Tensor, page_tokens: int, scale: float, impl: str | None, mma: str) -> str:
    """The kernel for a call that is not plain: the tensor-core kernels compute the distance penalty (values as wide
    as keys, a positive scale; ``mma`` names the mma.sync kernel of the caller, and a prefill of head size 64 or 128
    takes the tcgen05 kernel first); the generic kernels take the rest."""
    fits = v_cache.shape[-1] == q.shape[2] and attention_mma_supported(q, page_tokens) and scale > 0
    if fits and mma == "mma" and impl in (None, "tc") and attention_tc_supported(q, page_tokens):
        return "tc"
    if impl in (None, mma):
        if fits:
            return mma
        if impl is None:
            return "generic"
    if impl != "generic":
        raise KernelError(f"attention kernel {impl!r} does not take this call (a distance penalty, or values of another head size)")
    return "generic"


def attention_mma_supported(q: torch.Tensor, page_tokens: int) -> bool:
    """The tensor-core attention kernels take bfloat16, head sizes in steps of 16 up to 128, pages of 64 tokens."""
    return q.dtype == torch.bfloat16 and q.shape[2] % 16 == 0 and q.shape[2] <= 128 and page_tokens == 64


def attention_tc_supported(q: torch.Tensor, page_tokens: int) -> bool:
    """The tcgen05 prefill attention takes bfloat16, head size 64 or 128, pages of 64 tokens."""
    return q.dtype == torch.bfloat16 and q.shape[2] in (64, 128) and page_tokens == 64


def _pick_attention(q: torch.Tensor, page_tokens: int, impl: str | None, prefill: bool = False) -> str:
    if impl is None:
        if prefill and attention_tc_supported(q, page_tokens):
            return "tc"
        return "mma" if attention_mma_supported(q, page_tokens) else "generic"
    if impl == "tc" and not (prefill and attention_tc_supported(q, page_tokens)):
        raise KernelError(f"the tcgen05 attention kernel does not take {q.dtype}, head_dim={q.shape[2]}, pages of {page_tokens}")
    if impl == "mma" and not attention_mma_supported(q, page_tokens):
        raise KernelError(f"the tensor-core attention kernels do not take {q.dtype}, head_dim={q.shape[2]}, pages of {page_tokens}")
    if impl not in ("tc", "mma", "generic"):
        raise KernelError(f"unknown attention implementation {impl!r}")
    return impl


def attention_latent_supported(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, num_kv_heads: int, page_tokens: int,
                               ring_tokens: int, window, scale: float, penalty, chunk, keep_first: int, sink: bool, v_dim) -> bool:
    """The tensor-core kernel for cached latent rows takes bfloat16, one key head whose rows are the values' source
    too, rows and value sizes that are multiples of 8 (values up to 512, a row within shared memory), a positive
    scale, pages of 64 tokens and a plain causal softmax."""
    return (v_dim is not None and v_cache is k_cache and num_kv_heads == 1 and not ring_tokens and not window and penalty is None
            and not chunk and not keep_first and not sink and scale > 0 and attention_latent_shape(q.dtype, q.shape[2], v_dim, page_tokens))


def attention_latent_shape(dtype: torch.dtype, row: int, rank: int, page_tokens: int) -> bool:
    """The element type and sizes that the tensor-core kernel for cached latent rows takes (QT_B200_LATENT_MMA=0: none)."""
    return (dtype == torch.bfloat16 and page_tokens == 64 and row % 8 == 0 and rank % 8 == 0 and 8 <= rank <= min(row, 512)
            and 3 * 64 * (-(-row // 16) * 16 + 8) * 2 <= 227 * 1024 and not os.environ.get("QT_B200_LATENT_MMA", "1").startswith("0"))


def _attention_latent(q, cache, out, block_table, seq_start, seq_past, seq_len, n_seqs, max_q_len, page_tokens, scale, v_dim, n_splits,
                      part_acc, part_ml) -> None:
    _call("attention_latent", "qt_attention_latent", _ptr(q), _ptr(cache), _ptr(out), _ptr(block_table), block_table.shape[1],
          _ptr(seq_start) if seq_start is not None else None, _ptr(seq_past) if seq_past is not None else None,
          _ptr(seq_len) if seq_len is not None else None, n_seqs, int(max_q_len), q.shape[1], q.shape[2], int(v_dim), page_tokens, float(scale),
          int(n_splits), _ptr(part_acc) if n_splits > 1 else None, _ptr(part_ml) if n_splits > 1 else None, _stream())


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                      block_table: torch.Tensor, seq_start: torch.Tensor, seq_past: torch.Tensor, max_q_len: int,
                      num_kv_heads: int, page_tokens: int, ring_tokens: int, window: int | None, scale: float,
                      impl: str | None = None, penalty: tuple[torch.Tensor, torch.Tensor] | None = None,
                      chunk: int | None = None, keep_first: int = 0, sink: bool = False, v_dim: int | None = None,
                      sinks: torch.Tensor | None = None) -> None:
    """Causal attention of packed sequences over the cache (which already holds this step's keys).
    ``chunk``: a query at position i sees key j only if i // chunk == j // chunk as well.  A value cache with fewer
    heads than the key cache serves key head g with value head g % (value heads).
    ``impl`` forces a kernel ("tc": tcgen05, "mma": mma.sync, "generic"); by default the shape decides.
    ``penalty`` = (r1, r2), float [heads] each: the score of key j for the query at position i loses
    r1_h * ln(1 + r2_h * (i - j)); ``penalty`` = (slopes, None): it loses slope_h * (i - j).
    ``keep_first``: a windowed query also sees the keys at positions below it.  ``sink``: the softmax has one more term
    of score 0 without a value, or, with ``sinks`` (float [heads]), of the head's own score, taken as it is (not scaled).  ``v_dim``: the values are the first ``v_dim`` elements of the rows of ``v_cache`` (which
    may be the key cache itself)."""
    _, num_heads, head_dim = _check_attention(q, k_cache, v_cache, out, block_table, num_kv_heads, page_tokens, penalty, v_dim)
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, (num_heads,))
        sink = True
    if impl in (None, "latent") and attention_latent_supported(q, k_cache, v_cache, num_kv_heads, page_tokens, ring_tokens, window, scale, penalty,
                                                               chunk, keep_first, sink, v_dim):
        n_seqs = seq_past.shape[0]
        _need(seq_start, "seq_start", torch.int32, (n_seqs + 1,))
        _need(seq_past, "seq_past", torch.int32)
        if block_table.shape[0] < n_seqs:
            raise KernelError("attention_prefill: block table has fewer rows than sequences")
        _attention_latent(q, k_cache, out, block_table, seq_start, seq_past, None, n_seqs, max_q_len, page_tokens, scale, v_dim, 1, None, None)
        return
    if impl == "latent":
        raise KernelError("the tensor-core kernel for cached latent rows does not take this call")
    extended = _extended_choice(q, k_cache, v_cache, page_tokens, ring_tokens, scale, penalty, keep_first, sink, v_dim, chunk, impl, "mma")
    if extended is not None:
        impl = extended
    elif not _plain_attention(q, v_cache, penalty):
        impl = _penalised_choice(q, v_cache, page_tokens, scale, impl, "mma")
    n_seqs = seq_past.shape[0]
    _need(seq_start, "seq_start", torch.int32, (n_seqs + 1,))
    _need(seq_past, "seq_past", torch.int32)
    if block_table.shape[0] < n_seqs:
        raise KernelError("attention_prefill: block table has fewer rows than sequences")
    choice = _pick_attention(q, page_tokens, impl, prefill=True)
    if choice == "tc":
        _call("attention_tc", "qt_attention_prefill_tc", _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), q.shape[0],
              k_cache.shape[0], _ptr(block_table), block_table.shape[1], _ptr(seq_start), _ptr(seq_past), n_seqs,
              int(max_q_len), num_heads, num_kv_heads, head_dim, page_tokens, ring_tokens, int(window or 0), float(scale),
              _ptr(penalty[0]) if penalty else None, _ptr(penalty[1]) if penalty else None, int(chunk or 0), v_cache.shape[1],
              _ptr(_status_word(q.device)), _stream())
        return
    if choice == "mma":
        _call("attention_mma", "qt_attention_prefill_mma", _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out),
              _ptr(block_table), block_table.shape[1], _ptr(seq_start), _ptr(seq_past), n_seqs, int(max_q_len), num_heads,
              num_kv_heads, head_dim, page_tokens, ring_tokens, int(window or 0), float(scale),
              _ptr(penalty[0]) if penalty else None, _ptr(penalty[1]) if penalty else None, int(chunk or 0), v_cache.shape[1],
              int(keep_first), 1 if sink else 0, _ptr(sinks), _stream())
        return
    _call("attention", "qt_attention_prefill", _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _code(q, "q"),
          _ptr(block_table), block_table.shape[1], _ptr(seq_start), _ptr(seq_past), n_seqs, int(max_q_len), num_heads,
          num_kv_heads, head_dim, page_tokens, ring_tokens, int(window or 0), float(scale), int(v_dim or v_cache.shape[-1]),
          _ptr(penalty[0]) if penalty else None, _ptr(penalty[1]) if penalty else None, int(chunk or 0), v_cache.shape[1],
          int(keep_first), 1 if sink else 0, v_cache.shape[-1], _ptr(sinks), _stream())


def _ws_merges_in_cluster(n_splits: int, warps: int, group: int, head_dim: int) -> bool:
    """Whether qt_attention_decode_ws merges its blocks in one launch (the rule of attention_mma.cu)."""
    if os.environ.get("QT_B200_DECODE_CLUSTER", "1").startswith("0") or not 2 <= n_splits <= 8:
        return False
    rows = min(group, 16)
    rings = 16 * (head_dim + 8) * 2 + warps * 4 * 32 * (head_dim + 8) * 2
    return rings + n_splits * (rows * head_dim + 2 * rows) * 4 <= 227 * 1024


DECODE_WARPS_MAX = 6     # warps per block of the one-range-per-warp decode kernel


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     block_table: torch.Tensor, seq_len: torch.Tensor, num_kv_heads: int, page_tokens: int,
                     ring_tokens: int, window: int | None, scale: float, n_splits: int,
                     part_acc: torch.Tensor | None, part_ml: torch.Tensor | None, impl: str | None = None,
                     warps: int = 1, penalty: tuple[torch.Tensor, torch.Tensor] | None = None, chunk: int | None = None,
                     keep_first: int = 0, sink: bool = False, v_dim: int | None = None, sinks: torch.Tensor | None = None) -> None:
    """One query token per sequence; ``seq_len`` counts the keys it sees (its own included).

    With ``n_splits`` > 1 the keys of each sequence are cut into that many ranges whose partial
    results pass through ``part_acc`` (float, >= B nq splits d) and ``part_ml`` (float, >= B nq splits 2).
    The tensor-core kernels are "ws" (every warp of a block walks a range of its own: n_splits * warps
    ranges, n_splits partial results; the default where it applies) and "mma" (the four warps of a block
    share each tile); "generic" takes every element type and head size.
    """
    n_seqs, num_heads, head_dim = _check_attention(q, k_cache, v_cache, out, block_table, num_kv_heads, page_tokens, penalty, v_dim)
    _need(seq_len, "seq_len", torch.int32, (n_seqs,))
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, (num_heads,))
        sink = True
    if impl in (None, "latent") and attention_latent_supported(q, k_cache, v_cache, num_kv_heads, page_tokens, ring_tokens, window, scale, penalty,
                                                               chunk, keep_first, sink, v_dim):
        if n_splits > 1:
            _need(part_acc, "part_acc", torch.float32)
            _need(part_ml, "part_ml", torch.float32)
            if part_acc.numel() < n_seqs * num_heads * n_splits * v_dim or part_ml.numel() < n_seqs * num_heads * n_splits * 2:
                raise KernelError("attention_decode: scratch is too small for this batch and split count")
        _attention_latent(q, k_cache, out, block_table, None, None, seq_len, n_seqs, 1, page_tokens, scale, v_dim, n_splits, part_acc, part_ml)
        return
    if impl == "latent":
        raise KernelError("the tensor-core kernel for cached latent rows does not take this call")
    if impl == "mma" and _special_mask(k_cache, v_cache, chunk):
        raise KernelError("the block-tile decode kernel takes no mask in chunks and no value heads shared by several key heads")
    extended = _extended_choice(q, k_cache, v_cache, page_tokens, ring_tokens, scale, penalty, keep_first, sink, v_dim, chunk, impl, "ws")
    if extended is not None:
        impl = extended
    elif not _plain_attention(q, v_cache, penalty):
        impl = _penalised_choice(q, v_cache, page_tokens, scale, impl, "ws")
    if n_splits > 1:
        _need(part_acc, "part_acc", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_acc.numel() < n_seqs * num_heads * n_splits * (v_dim or v_cache.shape[-1]) or part_ml.numel() < n_seqs * num_heads * n_splits * 2:
            raise KernelError("attention_decode: scratch is too small for this batch and split count")
    if impl == "ws" and not attention_mma_supported(q, page_tokens):
        raise KernelError(f"the tensor-core attention kernels do not take {q.dtype}, head_dim={q.shape[2]}, pages of {page_tokens}")
    picked = "ws" if impl == "ws" else _pick_attention(q, page_tokens, impl)
    if picked == "mma" and impl is None:
        picked = "ws"
    common = (_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.shape[1], _ptr(seq_len),
              n_seqs, num_heads, num_kv_heads, head_dim, page_tokens, ring_tokens, int(window or 0), float(scale), int(n_splits))
    launches = 2 if n_splits > 1 else 1
    if picked == "ws" and _ws_merges_in_cluster(n_splits, warps, num_heads // num_kv_heads, head_dim):
        launches = 1
    if picked == "ws":
        _call("attention_mma", "qt_attention_decode_ws", *common, int(warps), _ptr(part_acc), _ptr(part_ml),
              _ptr(penalty[0]) if penalty else None, _ptr(penalty[1]) if penalty else None, int(chunk or 0), v_cache.shape[1],
              int(keep_first), 1 if sink else 0, _ptr(sinks), _stream(), launches=launches)
    elif picked == "mma":
        _call("attention_mma", "qt_attention_decode_mma", *common, _ptr(part_acc), _ptr(part_ml), _stream(), launches=launches)
    else:
        _call("attention", "qt_attention_decode", *common[:4], _code(q, "q"), *common[4:], _ptr(part_acc), _ptr(part_ml),
              int(v_dim or v_cache.shape[-1]), _ptr(penalty[0]) if penalty else None, _ptr(penalty[1]) if penalty else None,
              int(chunk or 0), v_cache.shape[1], int(keep_first), 1 if sink else 0, v_cache.shape[-1], _ptr(sinks), _stream(), launches=launches)


# ----------------------------------------------------------------------------- experts chosen by a table
def route_top(logits: GemmOut, chosen: torch.Tensor, weights: torch.Tensor, gate: torch.Tensor | None, experts: int, scale: float,
              normalize: bool = True) -> None:
    """A learned router's choice from float logits [*, T, cols]: scores = sigmoid(logits[:, :experts]); ``chosen``
    [T, top] (int32) the ``top`` largest, ``weights`` [T, top] their scores over their sum (+ 1e-20) times ``scale``;
    ``gate`` [T] = sigmoid(logits[:, experts]) where given (a shared expert's gate, one number per token).  Without
    ``normalize`` the weights are the chosen scores themselves times ``scale``."""
    tokens, top = chosen.shape
    _need(logits.tensor, "logits", torch.float32)
    _need(chosen, "chosen", torch.int32, (logits.rows, top))
    _need(weights, "weights", torch.float32, (tokens, top))
    if gate is not None:
        _need(gate, "gate", torch.float32, (tokens,))
    _call("experts", "qt_route_top", _ptr(logits.tensor), logits.n_splits, logits.split_stride, logits.cols, _ptr(chosen), _ptr(weights),
          _ptr(gate), tokens, int(experts), top, float(scale), 1 if normalize else 0, _stream())


def _expert_extras(tokens: int, top: int, width: int, pair_weights, base: GemmOut | None, row_scale):
    """Checked optional operands of the expert kernels: per-pair weights, a further term and its per-token factor."""
    if pair_weights is not None:
        _need(pair_weights, "pair_weights", torch.float32, (tokens, top))
    if base is not None:
        _need(base.tensor, "base", torch.float32)
        if (base.rows, base.cols) != (tokens, width):
            raise KernelError(f"experts: a further term of {tuple(base.tensor.shape)} for an output of [{tokens}, {width}]")
    if row_scale is not None:
        _need(row_scale, "row_scale", torch.float32, (tokens,))
    return (_ptr(pair_weights), _ptr(base.tensor) if base is not None else None, base.n_splits if base is not None else 1,
            base.split_stride if base is not None else 0, _ptr(row_scale))


def experts_by_pair(x: torch.Tensor, token_ids: torch.Tensor | None, table: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
                    mid: torch.Tensor, out: torch.Tensor, activation: str, pair_weight: float = 1.0,
                    pair_weights: torch.Tensor | None = None, gated: bool = False, limit: float = 0.0,
                    base: GemmOut | None = None, row_scale: torch.Tensor | None = None, in_weights: torch.Tensor | None = None) -> None:
    """out [T, width] (float) = pair_weight * sum over the ``top`` experts e that ``table[token_ids[t]]`` names of
    down[e] act(up[e] x[t]): one matrix-vector pass per (token, expert) pair, the form for few tokens.
    up [E, ff, width], down [E, width, ff], mid [T * top, ff] (scratch for the activations), all of x's element type.

    Without ``token_ids`` row t of ``table`` [T, top] names token t's experts (a router's choice).  ``pair_weights``
    [T, top] weighs every pair by itself.  ``gated``: up is [E, 2 ff, width], ff gate rows then ff up rows, and
    mid = act(gate) * up, or the capped gate with ``limit``.  ``base`` (float sums [*, T, width]) times
    ``row_scale`` [T] (1 without it) is added to the result.  ``in_weights`` [T, top]: a pair's expert reads its token's row
    times the pair's weight (the weight on the input instead of the output)."""
    tokens, width = x.shape
    experts, ff = up.shape[0], up.shape[1] // (2 if gated else 1)
    top = table.shape[1]
    _need(x, "x")
    if in_weights is not None:
        _need(in_weights, "in_weights", torch.float32, (tokens, top))
    if token_ids is not None:
        _need(token_ids, "token_ids", torch.int32, (tokens,))
    _need(table, "table", torch.int32)
    _need(up, "up", x.dtype, (experts, (2 if gated else 1) * ff, width))
    _need(down, "down", x.dtype, (experts, width, ff))
    _need(mid, "mid", x.dtype, (tokens * top, ff))
    _need(out, "out", torch.float32, (tokens, width))
    weights_ptr, base_ptr, base_splits, base_stride, scale_ptr = _expert_extras(tokens, top, width, pair_weights, base, row_scale)
    _call("experts", "qt_experts_by_pair", _ptr(x), _ptr(token_ids), _ptr(table), _ptr(up), _ptr(down), _ptr(mid), _ptr(out),
          _code(x, "x"), tokens, table.shape[0], top, experts, width, ff, activation_code(activation, gated), float(pair_weight),
          weights_ptr, 1 if gated else 0, float(limit), base_ptr, base_splits, base_stride, scale_ptr, _ptr(in_weights), _stream(), launches=2)


EXPERT_TILE_ROWS = 128      # rows of one tile of the tiled expert products (the MMA's M)


def expert_tiles(pairs: int, experts: int) -> int:
    """Tiles that hold ``pairs`` rows ordered by expert, however they fall: every expert's run ends in a tile of its own."""
    return pairs // EXPERT_TILE_ROWS + experts


def experts_tiled_supported(x: torch.Tensor, up: torch.Tensor) -> bool:
    """The tiled expert products take bfloat16 with widths that are multiples of 8 (16-byte rows)."""
    return x.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and up.shape[1] % 8 == 0 and up.shape[2] % 8 == 0


def experts_tiled(x: torch.Tensor, token_ids: torch.Tensor | None, table: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
                  ordered: torch.Tensor, mid: torch.Tensor, y: torch.Tensor, route: torch.Tensor, out: torch.Tensor,
                  activation: str, pair_weight: float = 1.0, pair_weights: torch.Tensor | None = None, gated: bool = False,
                  limit: float = 0.0, wide: torch.Tensor | None = None, base: GemmOut | None = None,
                  row_scale: torch.Tensor | None = None, in_weights: torch.Tensor | None = None) -> None:
    """The same result as ``experts_by_pair`` for many tokens: the (token, expert) pairs are ordered by expert on the
    device, each expert's run padded to whole tiles of 128 rows, and both products run tile by tile on the tensor
    cores.  Scratch: ``ordered`` [rows, width], ``mid`` [rows, ff], ``y`` [rows, width] (bfloat16) with
    rows = expert_tiles(T * top, E) * 128, and ``route`` (int32, T * top + rows + rows / 128 words); gated experts
    also ``wide`` [rows, 2 ff] (their first product, before the gate kernel)."""
    tokens, width = x.shape
    experts, ff = up.shape[0], up.shape[1] // (2 if gated else 1)
    top = table.shape[1]
    tiles = expert_tiles(tokens * top, experts)
    rows = tiles * EXPERT_TILE_ROWS
    _need(x, "x", torch.bfloat16)
    if token_ids is not None:
        _need(token_ids, "token_ids", torch.int32, (tokens,))
    _need(table, "table", torch.int32)
    _need(up, "up", torch.bfloat16, (experts, (2 if gated else 1) * ff, width))
    _need(down, "down", torch.bfloat16, (experts, width, ff))
    _need(ordered, "ordered", torch.bfloat16, (rows, width))
    _need(mid, "mid", torch.bfloat16, (rows, ff))
    _need(y, "y", torch.bfloat16, (rows, width))
    _need(route, "route", torch.int32, (tokens * top + rows + tiles,))
    _need(out, "out", torch.float32, (tokens, width))
    if in_weights is not None:
        _need(in_weights, "in_weights", torch.float32, (tokens, top))
    weights_ptr, base_ptr, base_splits, base_stride, scale_ptr = _expert_extras(tokens, top, width, pair_weights, base, row_scale)
    pair_row, row_token, tile_expert = route[:tokens * top], route[tokens * top:tokens * top + rows], route[tokens * top + rows:]
    status = _status_word(x.device)
    _call("experts", "qt_experts_route", _ptr(x), _ptr(token_ids), _ptr(table), _ptr(ordered), _ptr(pair_row), _ptr(row_token),
          _ptr(tile_expert), tokens, table.shape[0], top, experts, width, EXPERT_TILE_ROWS, tiles, _ptr(in_weights), _stream(), launches=2)
    if gated:
        _need(wide, "wide", torch.bfloat16, (rows, 2 * ff))
        _call("experts_tc", "qt_expert_gemm", _ptr(ordered), _ptr(up), _ptr(wide), BF16, _ptr(tile_expert), tiles, experts, 2 * ff, width,
              -1, _ptr(status), _stream())
        swiglu(GemmOut(wide.view(1, rows, 2 * ff)), mid, 0, activation, limit)
    else:
        _call("experts_tc", "qt_expert_gemm", _ptr(ordered), _ptr(up), _ptr(mid), BF16, _ptr(tile_expert), tiles, experts, ff, width,
              activation_code(activation), _ptr(status), _stream())
    _call("experts_tc", "qt_expert_gemm", _ptr(mid), _ptr(down), _ptr(y), BF16, _ptr(tile_expert), tiles, experts, width, ff,
          -1, _ptr(status), _stream())
    _call("experts", "qt_experts_combine", _ptr(y), BF16, _ptr(pair_row), _ptr(out), tokens, top, width, float(pair_weight),
          weights_ptr, base_ptr, base_splits, base_stride, scale_ptr, _stream())


# ----------------------------------------------------------------------------- matrix product
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: GemmOut) -> None:
    """out = a [M, K] @ w [N, K]^T on the FMA pipe (float accumulation, any sizes)."""
    _need(a, "a")
    _need(w, "w", a.dtype)
    if a.shape[1] != w.shape[1] or out.n_splits != 1 or (out.rows, out.cols) != (a.shape[0], w.shape[0]):
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.tensor.shape)} do not fit")
    _call("gemm_simt", "qt_gemm_simt", _ptr(a), _ptr(w), _code(a, "a"), _ptr(out.tensor), _code(out.tensor, "out"),
          a.shape[0], w.shape[0], a.shape[1], _stream())


# ----------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32)
    _need(out, "out", torch.int32, (logits.shape[0],))
    _call("sampling", "qt_argmax", _ptr(logits), _ptr(out), logits.shape[0], logits.shape[1], _stream())


def feed_tokens(ids: torch.Tensor, chosen: torch.Tensor, vocab: int) -> None:
    """ids[i] (a row number of ``chosen``, or negative) becomes the token chosen for that row (0 if negative)."""
    _need(ids, "ids", torch.int32)
    _need(chosen, "chosen", torch.int32)
    _call("sampling", "qt_feed_tokens", _ptr(ids), _ptr(chosen), ids.numel(), chosen.numel(), int(vocab), _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
    rows = logits.shape[0]
    _need(logits, "logits", torch.float32)
    _need(temperature, "temperature", torch.float32, (rows,))
    _need(uniform, "uniform", torch.float32, (rows,))
    _need(out, "out", torch.int32, (rows,))
    _call("sampling", "qt_sample", _ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(out), rows, logits.shape[1],
          _stream())


def sample_keyed(logits: torch.Tensor, temperature: float, seed: int, keys: torch.Tensor, out: torch.Tensor,
                 top_k: int = 0, top_p: float = 1.0) -> None:
    """Temperature sampling with the uniform number of each row made on the device from (seed, request, step);
    ``keys`` int32 [rows, 2] holds each row's request and step number.  ``top_k`` > 0 keeps the k largest logits (and
    what ties with the k-th), ``top_p`` < 1 of those the most likely tokens whose renormalised probabilities first sum
    to it (and what ties with the last)."""
    rows = logits.shape[0]
    if not 0.0 < top_p <= 1.0 or top_k < 0:
        raise KernelError(f"sample: top_k={top_k} must not be negative and top_p={top_p} must lie in (0, 1]")
    _need(logits, "logits", torch.float32)
    _need(keys, "keys", torch.int32, (rows, 2))
    _need(out, "out", torch.int32, (rows,))
    seed &= (1 << 64) - 1
    _call("sampling", "qt_sample_keyed", _ptr(logits), float(temperature), seed - (1 << 64) if seed >> 63 else seed, _ptr(keys),
          _ptr(out), rows, logits.shape[1], int(top_k), float(top_p), _stream())


_STATUS: dict[int, torch.Tensor] = {}
_TC_TILES = (16, 32, 64, 128, 256)
_SM_COUNTS: dict[int, int] = {}


def sm_count(device: torch.device | str | None = None) -> int:
    """Streaming multiprocessors of ``device`` (asked once per device)."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _SM_COUNTS:
        _SM_COUNTS[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _SM_COUNTS[index]

TC_MAX_BLOCK_TOKENS = 128      # tokens per block that ``gemm`` gives the one-block kernel (256 measured slower at every split count)


def _status_word(device: torch.device) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _STATUS:
        _STATUS[index] = torch.zeros(4, dtype=torch.int32, device=device)
    return _STATUS[index]


def status_word(device: torch.device | str = "cuda") -> torch.Tensor:
    """The device words the tensor-core kernels report into (word 0: the code of a wait that ran out, else 0)."""
    return _status_word(torch.device(device))


def check_status(device: torch.device | str = "cuda") -> None:
    """Raise if a bounded wait inside a tensor-core kernel ran out since the last check (synchronises)."""
    word = _status_word(torch.device(device))
    code = int(word[0].item())
    if code != 0:
        word.zero_()
        tail = _PAIR_TAIL.get(word.device.index)
        if tail is not None:
            tail[1].zero_()                    # flags of the pair kernel's last wave that the failed launch left up
        role = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue", 4: "the MMA issuer (for a free accumulator)",
                5: "a kernel whose shared memory was less aligned than its launch allowed for",
                6: "a pair that finishes a tile (for another pair's sums)"}.get(code, f"role {code}")
        raise KernelError(f"gemm_tc: a wait of {role} ran out; the result of that launch is invalid")


def tc_token_tile(rows: int) -> int:
    for tile in _TC_TILES:
        if rows <= tile:
            return min(tile, TC_MAX_BLOCK_TOKENS)
    return TC_MAX_BLOCK_TOKENS


def tc_normalise_splits(k: int, wanted: int) -> int:
    """The largest split count <= ``wanted`` that leaves no split without a 64-wide K block."""
    blocks = -(-k // 64)
    wanted = max(1, min(wanted, blocks))
    per = -(-blocks // wanted)
    return -(-blocks // per)


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: GemmOut, token_tile: int | None = None, stages: int = 0,
            swiglu: bool = False, activation: str = "silu", limit: float = 0.0) -> None:
    """out = a [M, K] @ w [N, K]^T on the tcgen05 tensor cores; bfloat16 inputs, K a multiple of 8.

    ``out`` is [1, M, N] bfloat16 or float, or [splits, M, N] float for split-K partial sums.  With ``swiglu`` the
    rows of ``w`` alternate SWIGLU_GROUP of a gate and of an up projection and ``out`` [1, M, N / 2] (bfloat16)
    receives act(gate) * up from the epilogue.
    """
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    rows, k = a.shape
    cols = w.shape[0] // 2 if swiglu else w.shape[0]
    if k != w.shape[1] or (out.rows, out.cols) != (rows, cols) or (swiglu and (out.n_splits != 1 or w.shape[0] % (2 * SWIGLU_GROUP)
                                                                                   or out.tensor.dtype != torch.bfloat16)):
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.tensor.shape)} do not fit")
    if rows == 0:
        return
    if not out.tensor.is_cuda or out.tensor.dtype not in _CODES:
        raise KernelError("gemm_tc: the output must be a bfloat16 or float32 CUDA tensor")
    tile = token_tile or tc_token_tile(rows)
    _call("gemm_tc", "qt_gemm_tc", _ptr(a), _ptr(w), _ptr(out.tensor), _code(out.tensor, "out"), rows, w.shape[0], k, tile,
          out.n_splits, out.split_stride, int(stages), 1 if swiglu else 0, activation_code(activation, True) if swiglu else 0,
          float(limit), _ptr(_status_word(a.device)), _stream())


_PAIR_TAIL: dict[int, tuple[torch.Tensor, torch.Tensor, int]] = {}


def _pair_tail(device: torch.device) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Scratch of the pair kernel's last wave (one accumulator tile per resident pair, and the flags that guard the
    slots), made once per device: (slots, flags, pairs)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _PAIR_TAIL:
        pairs = max(1, sm_count(device) // 2)  # one resident pair per TPC at most
        floats = _fn("gemm_tc", "qt_gemm_tc_pair_slots")()
        _PAIR_TAIL[index] = (torch.empty(pairs * floats, dtype=torch.float32, device=device),
                             torch.zeros(pairs * 8, dtype=torch.int32, device=device), pairs)
    return _PAIR_TAIL[index]


def pair_tail_mode() -> int:
    """``QT_B200_PAIR_TAIL``: 0 or unset = every tile of the pair kernel by one pair; -1 = the last wave by K ranges
    where the kernel's model of the time saved says it pays; 1 = wherever the tiles do not divide by the pairs.
    Off by default: launched alone at full clocks the cut saves up to a quarter of a product with a long K and a
    half-empty last wave, but a whole prefill runs at the power limit, where idle pairs in a last wave leave their
    power to the others, and measured the same or slower with it."""
    return int(os.environ.get("QT_B200_PAIR_TAIL", "0"))


def gemm_tc_pair(a: torch.Tensor, w: torch.Tensor, out: GemmOut, swiglu: bool = False, activation: str = "silu",
                 tail: int | None = None, limit: float = 0.0) -> None:
    """The same product by pairs of blocks on the two SMs of a TPC (tcgen05 cta_group::2): 256 weight rows x
    256 tokens per tile, each block staging half of both operands; one persistent pair per TPC with two
    accumulators in tensor memory.  Meant for many tokens; ``out`` may be [splits, M, N] float partial sums, which
    pays for a few hundred tokens whose tiles alone do not fill the TPCs.

    With ``swiglu`` the rows of ``w`` alternate SWIGLU_GROUP of a gate and of an up projection
    (``interleave_gate_up``) and ``out`` [1, M, N / 2] receives act(gate) * up from the epilogue."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    rows, k = a.shape
    cols = w.shape[0] // 2 if swiglu else w.shape[0]
    if k != w.shape[1] or (out.rows, out.cols) != (rows, cols) or (swiglu and (out.n_splits != 1 or w.shape[0] % (2 * SWIGLU_GROUP))):
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.tensor.shape)} do not fit")
    if rows == 0:
        return
    if not out.tensor.is_cuda or out.tensor.dtype not in _CODES:
        raise KernelError("gemm_tc_pair: the output must be a bfloat16 or float32 CUDA tensor")
    tail = pair_tail_mode() if tail is None else int(tail)
    slots, flags, pairs = _pair_tail(a.device) if tail != 0 and out.n_splits == 1 else (None, None, 0)
    _call("gemm_tc", "qt_gemm_tc_pair", _ptr(a), _ptr(w), _ptr(out.tensor), _code(out.tensor, "out"), rows, w.shape[0], k,
          1 if swiglu else 0, activation_code(activation, True) if swiglu else 0, float(limit), out.n_splits, out.split_stride,
          tail, _ptr(slots) if slots is not None else None, _ptr(flags) if flags is not None else None, pairs,
          _ptr(_status_word(a.device)), _stream())


def gemm_uses_pairs(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm`` gives this product to the pair kernel (a static choice by element type and shape)."""
    if not gemm_tc_supported(a, w):
        return False
    # more than 256 tokens; or more than one block's 128 with a weight whose tiles fill the machine unsplit (the fused
    # gate/up projection, the head), which single blocks would read once per token tile
    return a.shape[0] > _TC_TILES[-1] or (a.shape[0] > TC_MAX_BLOCK_TOKENS and w.shape[0] >= 128 * sm_count(a.device))


def gemm(a: torch.Tensor, w: torch.Tensor, out: GemmOut) -> None:
    """out = a @ w^T with the kernel that fits the element type and shape (a static choice):
    tensor cores for bfloat16 with 16-byte aligned rows, the FMA kernel for float32 and the rest."""
    if gemm_tc_supported(a, w):
        if gemm_uses_pairs(a, w):
            gemm_tc_pair(a, w, out)         # more tokens than one block's tile: pairs of blocks, a third less operand traffic
        else:
            gemm_tc(a, w, out)
    elif out.n_splits == 1:
        gemm_simt(a, w, out)
    else:
        raise KernelError("gemm: split-K output is only produced by the tensor-core kernel")


# ----------------------------------------------------------------------------- products of a decode step, fused
FUSED_MAX_ROWS = 128        # most tokens the fused product takes (one token tile per block)
FUSED_MAX_SPLITS = 8        # blocks of a cluster that share a weight tile
_EPI_STORE, _EPI_RESIDUAL, _EPI_SWIGLU, _EPI_QKV = 0, 1, 2, 3


def fused_enabled(role: str) -> bool:
    """``QT_B200_FUSED`` in the environment: "0" turns the fused products off, a comma-separated list keeps only the
    named ones ("qkv", "gate", "attn_out", "mlp_out"); unset or "1": all of them."""
    setting = os.environ.get("QT_B200_FUSED", "1")
    if setting in ("1", ""):
        return True
    return setting != "0" and role in setting.split(",")


@dataclass
class ScaledRows:
    """Rows handed from an RMSNorm to the product behind it with the norm half done: ``tensor`` [M, K] holds
    bf16(r * g) for the stream rows r and the norm's weight g, and the rows' factor rsqrt(mean(r^2) + eps) is
    still to be applied, by the product's epilogue (the product is linear in its input).  ``sq`` [tiles, M]
    holds the sums of squares of r over ``tiles`` column ranges; mean(r^2) = sum over tiles / ``width``."""

    tensor: torch.Tensor
    sq: torch.Tensor
    width: int
    eps: float

    @property
    def shape(self):
        return self.tensor.shape


def fused_supported(w: torch.Tensor) -> bool:
    """The fused products take bfloat16 weights [N, K] with K a multiple of 8, 16-byte aligned."""
    return w.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous()


def fused_qkv_supported(head_dim: int, rotary_dim: int) -> bool:
    """The fused q/k-norm + rotation + cache write needs whole heads inside a 128-row weight tile and rotation
    pairs that four-element pieces can exchange."""
    return head_dim >= 16 and 128 % head_dim == 0 and rotary_dim % 8 == 0 and rotary_dim <= head_dim


def _fused(x, w: torch.Tensor, splits: int, epilogue: int, *, out=None, residual=None, norm_w=None, xw=None, sq_out=None,
           q_out=None, k_cache=None, v_cache=None, token_seq=None, token_pos=None, block_table=None, q_w=None, k_w=None,
           qk_eps=0.0, cos_sin=None, nq=0, nkv=0, d=0, page_tokens=0, ring_tokens=0, write_kv=False, stages: int = 0,
           act: int = 0, interleaved: bool = False, limit: float = 0.0) -> None:
    scaled = x if isinstance(x, ScaledRows) else None
    a = scaled.tensor if scaled is not None else x
    _need(a, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    rows, k = a.shape
    if k != w.shape[1]:
        raise KernelError(f"gemm_fused: x {tuple(a.shape)} and w {tuple(w.shape)} do not fit")
    if not 0 < rows <= FUSED_MAX_ROWS:
        raise KernelError(f"gemm_fused: {rows} tokens (1..{FUSED_MAX_ROWS})")
    if scaled is not None:
        _need(scaled.sq, "sq", torch.float32)
        if scaled.sq.dim() != 2 or scaled.sq.shape[1] != rows:
            raise KernelError(f"gemm_fused: sums of squares {tuple(scaled.sq.shape)} for {rows} rows")
    rotary_dim, max_pos = (0, 0) if cos_sin is None else (cos_sin.shape[1], cos_sin.shape[0])
    _call("gemm_fused", "qt_gemm_fused", _ptr(a), _ptr(w), rows, w.shape[0], k, tc_token_tile(rows), int(splits), int(stages), epilogue,
          _ptr(scaled.sq) if scaled is not None else None, scaled.sq.shape[0] if scaled is not None else 0,
          scaled.width if scaled is not None else 0, float(scaled.eps) if scaled is not None else 0.0,
          _ptr(out), _CODES.get(out.dtype, -1) if out is not None else 0, int(act), float(limit),
          _ptr(residual), _ptr(norm_w), _ptr(xw), _ptr(sq_out),
          _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(token_seq), _ptr(token_pos), _ptr(block_table),
          block_table.shape[1] if block_table is not None else 0, _ptr(q_w), _ptr(k_w), float(qk_eps),
          _ptr(cos_sin), rotary_dim, max_pos, nq, nkv, d, page_tokens, ring_tokens, 1 if write_kv else 0,
          1 if interleaved else 0, _ptr(_status_word(a.device)), _stream())


def gemm_fused_store(x, w: torch.Tensor, out: torch.Tensor, splits: int = 1, stages: int = 0) -> None:
    """out [M, N] (float or bfloat16) = x w^T, times the rows' deferred norm factor if ``x`` is ``ScaledRows``."""
    _need(out, "out", shape=(x.shape[0], w.shape[0]))
    _fused(x, w, splits, _EPI_STORE, out=out, stages=stages)


def gemm_fused_residual(x, w: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor | None = None,
                        eps: float = 0.0, xw: torch.Tensor | None = None, sq: torch.Tensor | None = None, splits: int = 1,
                        stages: int = 0) -> "ScaledRows | None":
    """residual [M, N] (float, in place) += x w^T.  With ``norm_weight`` [N] the RMSNorm that follows is prepared in
    the same launch: ``xw`` [M, N] = bf16(residual * norm_weight) and ``sq`` [ceil(N / 128), M] = the rows' sums of
    squares per 128 columns; returns them as ``ScaledRows`` for the product behind the norm."""
    rows, n = x.shape[0], w.shape[0]
    _need(residual, "residual", torch.float32, (rows, n))
    if norm_weight is None:
        _fused(x, w, splits, _EPI_RESIDUAL, residual=residual, stages=stages)
        return None
    _need(norm_weight, "norm_weight", torch.float32, (n,))
    _need(xw, "xw", torch.bfloat16, (rows, n))
    _need(sq, "sq", torch.float32, (-(-n // 128), rows))
    _fused(x, w, splits, _EPI_RESIDUAL, residual=residual, norm_w=norm_weight, xw=xw, sq_out=sq, stages=stages)
    return ScaledRows(xw, sq, n, float(eps))


def gemm_fused_swiglu(x, w: torch.Tensor, out: torch.Tensor, splits: int = 1, stages: int = 0, activation: str = "silu",
                      limit: float = 0.0) -> None:
    """out [M, N / 2] (bfloat16) = act(gate) * up for a weight whose rows alternate SWIGLU_GROUP of gate and of up."""
    if w.shape[0] % (2 * SWIGLU_GROUP):
        raise KernelError(f"gemm_fused_swiglu: {w.shape[0]} rows are not gate and up rows in groups of {SWIGLU_GROUP}")
    _need(out, "out", torch.bfloat16, (x.shape[0], w.shape[0] // 2))
    _fused(x, w, splits, _EPI_SWIGLU, out=out, stages=stages, act=activation_code(activation, True), limit=limit)


def gemm_fused_qkv(x, w: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None, v_cache: torch.Tensor | None,
                   token_seq: torch.Tensor, token_pos: torch.Tensor, block_table: torch.Tensor | None,
                   q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float, cos_sin: torch.Tensor | None,
                   num_heads: int, num_kv_heads: int, head_dim: int, page_tokens: int, ring_tokens: int,
                   write_kv: bool = True, splits: int = 1, stages: int = 0, interleaved: bool = False) -> None:
    """The fused projection [q; k; v] (or q alone) with per-head q/k RMSNorm, rotation and the cache write done in
    its epilogue: what ``gemm`` followed by ``qk_norm_rope_write`` does, in one launch."""
    rows = x.shape[0]
    rotary_dim = 0 if cos_sin is None else cos_sin.shape[1]
    if not fused_qkv_supported(head_dim, rotary_dim):
        raise KernelError(f"gemm_fused_qkv: head_dim={head_dim} with rotary_dim={rotary_dim} is not taken")
    _need(q_out, "q_out", torch.bfloat16, (rows, num_heads, head_dim))
    _need(token_seq, "token_seq", torch.int32, (rows,))
    _need(token_pos, "token_pos", torch.int32, (rows,))
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _need(weight, name, torch.float32, (head_dim,))
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
    if write_kv:
        _need(block_table, "block_table", torch.int32)
        for name, cache in (("k_cache", k_cache), ("v_cache", v_cache)):
            _need(cache, name, torch.bfloat16)
            if tuple(cache.shape[1:]) != (num_kv_heads, page_tokens, head_dim):
                raise KernelError(f"{name}: shape {tuple(cache.shape)} is not [pages, {num_kv_heads}, {page_tokens}, {head_dim}]")
    _fused(x, w, splits, _EPI_QKV, q_out=q_out, k_cache=k_cache if write_kv else None, v_cache=v_cache if write_kv else None,
           token_seq=token_seq, token_pos=token_pos, block_table=block_table if write_kv else None, q_w=q_weight, k_w=k_weight,
           qk_eps=eps, cos_sin=cos_sin, nq=num_heads, nkv=num_kv_heads, d=head_dim, page_tokens=page_tokens,
           ring_tokens=ring_tokens, write_kv=write_kv, stages=stages, interleaved=interleaved)
