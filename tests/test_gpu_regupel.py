"""The Regupel design on the GPU against the plain implementation (tests/plain_regupel.py): every mechanism alone at the
kernels, with inputs made so that a fault shows (a key just outside a window, the first key that is no longer kept, a
sink that takes the weight no key earns, a far key among hundreds, a write to the state that must survive hundreds of
tokens), then whole models through the engine: whole prompts, token by token, portions down to two tokens, unequal
batches, slots, state rows and pages used again, long decoding, greedy generation through the entry point, the command
line and the trace replay."""
import functools
import json
import math
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest
import torch

import plain_regupel as plain
from qwen_triton_b200 import Engine, QwenB200ForCausalLM, StepEntry, config_from_dict, load_preset, write_random_model
from qwen_triton_b200.ops import kernels
from qwen_triton_b200.ops.kernels import GemmOut
from qwen_triton_b200.weights import Checkpoint, write_safetensors
from test_gpu_vunepel import STORE, _Step, close, paged

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent
DTYPES = ("fp32", "bf16")
PAGE = 64
_KEEP = []

# a third configuration beside the two presets: a width off 8 (no tensor-core products), an attention layer first whose
# values are wider than its keys, one key head per query head and one key head for all, a rotation of two elements and
# one of the whole head without stretching, a window of one position, more kept first keys than the window is long, no
# kept keys, no mask, decays of 0 and of 1, a state of 136 key channels, one expert, as many chosen as there are, no
# shared expert, a layer without a feed-forward, a parallel layer run twice, constants of 1
ODD = {
    "architecture": "Regupel", "vocab": 61, "width": 36, "norm": {"eps": 1e-3}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
    "residual_mult": 1.0,
    "layers": [
        {"type": "attention", "mlp": {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 1, "top": 1}},
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 12, "vdim": 20, "scale": 0.3, "mask": {"size": 1}, "rot": {"base": 100.0, "dims": 2}}},
        {"type": "parallel", "mlp": {"kind": "moe", "expert": {"ff": 9}, "router": {"experts": 3, "top": 3}, "shared": {"ff": 7}},
         "mixer": {"left": {"heads": 5, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.5, "mask": {"size": 5, "keep_first": 9}}, "left_scale": 1.0,
                   "right": {"heads": 2, "dim": 136, "vdim": 6, "decay": [0.0, 1.0]}, "right_scale": 1.0}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 20, "vdim": 10, "scale": 0.2, "rot": {"base": 10000.0, "dims": 20}}},
        {"type": "parallel", "mlp": {"kind": "moe", "expert": {"ff": 9}, "router": {"experts": 3, "top": 3}, "shared": {"ff": 7}},
         "mixer": {"left": {"heads": 5, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.5, "mask": {"size": 5, "keep_first": 9}}, "left_scale": 1.0,
                   "right": {"heads": 2, "dim": 136, "vdim": 6, "decay": [0.0, 1.0]}, "right_scale": 1.0}, "weights_of": 1},
        {"type": "parallel", "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 7, "top": 2}},
         "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "mask": {"size": 70, "keep_first": 0}}, "left_scale": 0.3,
                   "right": {"heads": 1, "dim": 10, "vdim": 33, "decay": [0.9]}, "right_scale": 2.0}},
    ],
}
MODELS = ("regupel-tiny-a", "regupel-tiny-b", "odd")
CASES = [(name, dtype) for name in MODELS for dtype in DTYPES]


def config_of(name):
    return config_from_dict(ODD) if name == "odd" else load_preset(name)


@functools.lru_cache(maxsize=None)
def model(name: str, dtype: str, peaky: bool = False):
    """(folder, raw config, float weights for the plain implementation).  ``peaky``: the left mixers' q and k norm weights
    are three times as large, so that few keys, far ones among them, carry each of their softmaxes (the attention layers'
    queries and keys have unit root mean square whatever the weights are; their sharpness is the configuration's scale)."""
    config = config_of(name)
    holder = tempfile.TemporaryDirectory(prefix=f"qt_{name}_{dtype}_")
    _KEEP.append(holder)
    folder = write_random_model(holder.name, config, seed=13 + len(name), dtype=STORE[dtype])
    if peaky:
        checkpoint = Checkpoint(folder)
        tensors = {n: checkpoint.read(n) for n in checkpoint.names()}
        for n in list(tensors):
            if n.endswith((".q.norm", ".k.norm")):
                tensors[n] = (tensors[n].float() * 3.0).to(tensors[n].dtype)
        write_safetensors(Path(folder) / "model.safetensors", tensors)
    checkpoint = Checkpoint(folder)
    weights = {n: checkpoint.read(n).float() for n in checkpoint.names()}
    return folder, config.to_hf_dict(), weights


@functools.lru_cache(maxsize=None)
def oracle_and_margins(name: str, dtype: str, peaky: bool, tokens: tuple):
    _, raw, weights = model(name, dtype, peaky)
    margins = []
    logits = plain.forward(raw, weights, list(tokens), margins=margins).float()
    return logits, (torch.stack(margins).min(dim=0).values if margins else torch.full((len(tokens),), math.inf, dtype=torch.float64))


def oracle(name: str, dtype: str, peaky: bool, tokens: tuple) -> torch.Tensor:
    return oracle_and_margins(name, dtype, peaky, tokens)[0]


CLOSE_CALL = 0.15      # a router's gap, over the scale of its logits, below which bfloat16 may choose otherwise


def close_rows(actual, name, dtype, peaky, tokens, rows, what):
    """The engine's logits for the positions ``rows`` (a slice) of a request against the plain implementation's.  float32:
    every element.  bfloat16: per position relative to the logits' scale (the bar of ``close``), and no test rests on a
    close call: a position at which some router's choice is nearly a tie in the plain implementation may fall the other
    way in bfloat16 (another expert, whose output the norm behind it brings to the same size), so such positions are
    only asked to be finite."""
    want, margins = oracle_and_margins(name, dtype, peaky, tuple(tokens))
    want, margins = want[rows], margins[rows]
    if dtype != "bf16":
        return close(actual, want, dtype, what, model_rows=True)
    actual = actual.float().cpu()
    assert actual.shape == want.shape and bool(torch.isfinite(actual).all()), what
    clear = margins >= CLOSE_CALL
    if bool(clear.any()):
        close(actual[clear], want[clear], dtype, what, model_rows=True)


def tokens_of(name: str, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(277 + seed)
    return torch.randint(0, config_of(name).vocab_size, (length,), generator=generator).tolist()


def engine_of(name, dtype, peaky=False, **kwargs) -> Engine:
    kwargs.setdefault("max_tokens", 2048)
    return Engine.from_pretrained(model(name, dtype, peaky)[0], dtype=dtype, **kwargs)


def as_int(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ============================================================================= mechanisms alone
@pytest.mark.parametrize("width, rows", [(96, 5), (130, 33), (7, 1), (1024, 3), (5000, 2)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_with_bias_on_a_sublayer_output(width, rows, out_dtype):
    """stream += LN(d) w + b, the stream itself handed on (no norm in front of the next sublayer); then the model's last
    norm with weight and bias on listed rows; split sums in both places."""
    torch.manual_seed(width)
    x = torch.randn(rows, width)
    parts = torch.randn(3, rows, width)
    w, b, wf, bf = (torch.randn(width) * s + m for s, m in ((0.2, 1.0), (0.3, 0.0), (0.2, 1.0), (0.3, 0.0)))
    want_stream = x.double() + plain.layer_norm(parts.double().sum(0), w.double(), b.double(), 1e-5)
    stream = x.to(DEV)
    out = torch.empty(rows, width, dtype=out_dtype, device=DEV)
    kernels.add_layernorm(stream, GemmOut(parts.to(DEV)), w.to(DEV), None, 1e-5, out, post_bias=b.to(DEV))
    torch.testing.assert_close(stream.cpu().double(), want_stream, atol=2e-5, rtol=1e-5)
    tol = dict(atol=2e-5, rtol=1e-5) if out_dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(out.float().cpu().double(), want_stream, **tol)
    # the last norm: a pending addition with its own norm, listed rows, the stream left as it is
    listed = as_int([rows - 1, 0])
    before = stream.clone()
    more = torch.randn(1, rows, width)
    want = plain.layer_norm(want_stream + plain.layer_norm(more[0].double(), w.double(), b.double(), 1e-5), wf.double(), bf.double(), 1e-5)
    out = torch.empty(2, width, dtype=out_dtype, device=DEV)
    kernels.add_layernorm(stream, GemmOut(more.to(DEV)), w.to(DEV), wf.to(DEV), 1e-5, out, listed, post_bias=b.to(DEV), bias=bf.to(DEV))
    assert torch.equal(stream, before)
    tol = dict(atol=1e-4, rtol=1e-4) if out_dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(out.float().cpu().double(), want[[rows - 1, 0]], **tol)


def test_weighted_sum_of_two_products():
    torch.manual_seed(1)
    a, b = torch.randn(3, 7, 50), torch.randn(1, 7, 50).to(torch.bfloat16)
    out = torch.empty(7, 50, device=DEV)
    got = kernels.weighted_sum(GemmOut(a.to(DEV)), 0.7, GemmOut(b.to(DEV)), 1.3, out)
    torch.testing.assert_close(got.value().cpu(), 0.7 * a.sum(0) + 1.3 * b[0].float(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("scaling", [None, {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 1024}, {"factor": 3.0, "low": 2.0, "high": 5.0, "original": 40}])
@pytest.mark.parametrize("dims, base", [(48, 300000.0), (2, 100.0), (64, 10000.0)])
def test_stretched_frequencies_of_the_rotation_table(scaling, dims, base):
    """The table's angles against the plain frequencies; with the second set of constants pairs fall into all three
    bands (kept, divided, blended)."""
    from qwen_triton_b200.parts.base import Runtime, Workspace
    from qwen_triton_b200.parts.position import WavelengthRotaryTable
    runtime = Runtime(device=torch.device(DEV), dtype=torch.float32, max_step_tokens=8, max_positions=64, workspace=Workspace(torch.device(DEV)))
    params = {"theta": base, "rotary_dim": dims, "head_dim": dims, **(scaling or {})}
    table = WavelengthRotaryTable(params, runtime).table(3000).cpu().double()
    freqs = plain.stretched_frequencies(dims, base, scaling)
    angle = torch.arange(3000, dtype=torch.float64)[:, None] * freqs[None, :]
    torch.testing.assert_close(table, torch.cat((angle.cos(), angle.sin()), dim=-1), atol=1e-7, rtol=0)
    if scaling is not None and scaling["original"] == 40 and dims == 64:
        plain_f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        ratio = freqs / plain_f
        assert bool((ratio == 1.0).any()) and bool(((ratio - 1 / 3.0).abs() < 1e-12).any()) and bool(((ratio > 0.34) & (ratio < 0.99)).any())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode, nq, nkv, d, dv, rot", [("unit", 4, 2, 16, 8, 8), ("unit", 3, 3, 20, 36, 20), ("unit", 2, 1, 128, 64, 32), ("whole", 4, 2, 16, 16, 0),
                                                      ("whole", 5, 1, 24, 8, 0), ("whole", 2, 2, 64, 64, 0), ("unit", 1, 1, 12, 12, 2)])
def test_rotation_norms_and_the_cache_write(dtype, mode, nq, nkv, d, dv, rot):
    """Queries out and keys and values into a scrambled paged cache, from split sums with further columns behind them: the
    rotation of a part of a head followed by the division by the head's root mean square, and the norm over the whole
    projection with weights, at positions far into a sequence."""
    torch.manual_seed(nq * d + dv)
    store = STORE[dtype]
    tokens, extra, eps = 9, 8, 1e-5
    cols = nq * d + nkv * d + nkv * dv + extra
    parts = torch.randn(2, tokens, cols)
    positions = torch.tensor([0, 1, 63, 64, 65, 127, 128, 300, 301])
    rows = parts.double().sum(0)
    q = rows[:, :nq * d].view(tokens, nq, d)
    k = rows[:, nq * d:(nq + nkv) * d].view(tokens, nkv, d)
    v = rows[:, (nq + nkv) * d:(nq + nkv) * d + nkv * dv].view(tokens, nkv, dv)
    cos_sin = qw = kw = row_inv = None
    if mode == "unit":
        freqs = plain.stretched_frequencies(rot, 10000.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64})
        want_q = plain.rms_divide(plain.rotate(q, positions, freqs, rot), eps)
        want_k = plain.rms_divide(plain.rotate(k, positions, freqs, rot), eps)
        angle = torch.arange(400, dtype=torch.float64)[:, None] * freqs[None, :]
        cos_sin = torch.cat((angle.cos(), angle.sin()), dim=-1).float().to(DEV)
    else:
        qw, kw = torch.randn(nq * d) * 0.2 + 1.0, torch.randn(nkv * d) * 0.2 + 1.0
        want_q = (plain.rms_divide(q.reshape(tokens, -1), eps) * qw.double()).view(tokens, nq, d)
        want_k = (plain.rms_divide(k.reshape(tokens, -1), eps) * kw.double()).view(tokens, nkv, d)
        qw, kw = qw.to(DEV), kw.to(DEV)
        row_inv = torch.empty(tokens, 2, device=DEV)
    order = [5, 2, 0, 4, 1, 3]
    k_cache = torch.full((6, nkv, PAGE, d), 77.0, dtype=store, device=DEV)
    v_cache = torch.full((6, nkv, PAGE, dv), 77.0, dtype=store, device=DEV)
    q_out = torch.empty(tokens, nq, d, dtype=store, device=DEV)
    kernels.qk_norm_rope_write(GemmOut(parts.to(DEV)), q_out, k_cache, v_cache, as_int([0] * tokens), as_int(positions.tolist()), as_int([order]), qw, kw,
                               eps, cos_sin, nq, nkv, d, PAGE, 0, v_heads=nkv, v_head_dim=dv, unit_norm=mode == "unit", row_inv=row_inv, extra_cols=extra)
    close(q_out, want_q, dtype, "queries")
    for i, pos in enumerate(positions.tolist()):
        close(k_cache[order[pos // PAGE], :, pos % PAGE], want_k[i], dtype, f"key at {pos}")
        close(v_cache[order[pos // PAGE], :, pos % PAGE], v[i], dtype, f"value at {pos}")
    assert float((k_cache.float() == 77.0).float().mean()) > 0.9          # nothing else was written


def sink_attention_all_ways(q, k, v, size, keep_first, sinks, scale, dtype, prompt, what, order=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] (rounded to the type already): the first ``prompt`` positions as one prompt,
    a later portion of it from the cache, and the remaining positions one at a time with several counts of key ranges,
    through every kernel that takes the call, against the plain heads."""
    total, nq, d = q.shape
    nkv, dv = k.shape[1], v.shape[2]
    store = STORE[dtype]
    want = plain.masked_softmax_attention(q.double(), k.double(), v.double(), scale, size, keep_first, sinks.double() if sinks is not None else None)
    order = order or list(range(-(-total // PAGE)))[::-1]
    k_pool, v_pool = paged(k, PAGE, order, store), paged(v, PAGE, order, store)
    table = as_int([order + [0]])
    options = dict(keep_first=keep_first, sinks=sinks.to(DEV) if sinks is not None else None)
    tensor_cores = dtype == "bf16" and d == dv and d % 16 == 0 and d <= 128
    for impl in (["generic", "mma"] if tensor_cores else ["generic"]):
        out = torch.full((prompt, nq, dv), float("nan"), dtype=store, device=DEV)
        kernels.attention_prefill(q[:prompt].to(DEV, store), k_pool, v_pool, out, table, as_int([0, prompt]), as_int([0]), prompt, nkv, PAGE, 0,
                                  size, scale, impl=impl, **options)
        close(out, want[:prompt], dtype, f"{what}: prompt, {impl}")
        begin = prompt * 2 // 3
        out = torch.full((prompt - begin, nq, dv), float("nan"), dtype=store, device=DEV)
        kernels.attention_prefill(q[begin:prompt].to(DEV, store), k_pool, v_pool, out, table, as_int([0, prompt - begin]), as_int([begin]),
                                  prompt - begin, nkv, PAGE, 0, size, scale, impl=impl, **options)
        close(out, want[begin:prompt], dtype, f"{what}: portion from {begin}, {impl}")
    for impl in (["generic", "ws"] if tensor_cores else ["generic"]):
        for t in range(prompt, total):
            for splits, warps in ((1, 1), (3, 2), (8, 4)):
                out = torch.full((1, nq, dv), float("nan"), dtype=store, device=DEV)
                kernels.attention_decode(q[t:t + 1].to(DEV, store), k_pool, v_pool, out, table, as_int([t + 1]), nkv, PAGE, 0, size, scale, splits,
                                         torch.empty(8 * nq * dv, device=DEV), torch.empty(16 * nq, device=DEV), impl=impl,
                                         warps=warps if impl == "ws" else 1, **options)
                close(out, want[t:t + 1], dtype, f"{what}: token {t}, {impl}, {splits} ranges")
    kernels.check_status(DEV)
    return want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, dv, size, keep_first, sink", [(4, 2, 48, 48, 37, 5, False), (8, 4, 128, 64, 150, 0, True), (3, 3, 20, 36, 1, 2, True),
                                                                   (2, 2, 64, 64, 100, 0, True), (5, 5, 32, 32, None, 0, True), (2, 1, 128, 128, 5, 70, False),
                                                                   (6, 1, 16, 16, 64, 64, True), (1, 1, 24, 8, 70, 129, False), (16, 1, 64, 64, 65, 1, True)])
def test_windows_kept_first_keys_and_learned_sinks(dtype, nq, nkv, d, dv, size, keep_first, sink):
    """Random queries, keys and values, 300 positions: the window's first page lies several pages behind the kept keys'
    last, and both edges fall inside pages, at their borders and across them; one stored sink per head, of either sign."""
    torch.manual_seed(nq * d + dv)
    store = STORE[dtype]
    total = 300
    q = (torch.randn(total, nq, d) * 1.5).to(store).float()
    k, v = torch.randn(total, nkv, d).to(store).float(), torch.randn(total, nkv, dv).to(store).float()
    sinks = torch.randn(nq) * 2.0 if sink else None
    sink_attention_all_ways(q, k, v, size, keep_first, sinks, 1.0 / math.sqrt(d), dtype, 290, f"{nq} heads of {d}/{dv}, window {size}, kept {keep_first}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, dv, size, keep_first", [(32, 32, 37, 6), (64, 64, 64, 64), (128, 64, 100, 1), (16, 16, 1, 63), (48, 48, 129, 65), (64, 64, 80, 0)])
def test_keys_just_inside_and_just_outside_the_window_and_the_kept_keys(dtype, d, dv, size, keep_first):
    """For every query from position 200 on, the key just outside its window and the first key that is no longer kept
    would score 60, the key just inside the window and the last kept key score 30, everything else about 0: the output is
    a mixture of the visible marked keys' values alone (element 1 of it is 1; a seen hidden key would pull it towards 2)."""
    torch.manual_seed(d)
    store = STORE[dtype]
    total, nq, nkv = 270, 2, 1
    k = torch.randn(total, nkv, d) * 0.02
    k[:, :, 1] = 0.0
    v = torch.randn(total, nkv, dv) * 0.02
    v[:, :, 1] = 0.0
    if keep_first:
        k[keep_first - 1, :, 1], v[keep_first - 1, :, 1] = 1.0, 1.0
        k[keep_first, :, 1], v[keep_first, :, 1] = 2.0, 2.0
    q = torch.zeros(total, nq, d)
    q[:, :, 1] = 30.0
    for t in range(200, total, 3):
        kt, vt = k.clone(), v.clone()
        kt[t - size, :, 1], vt[t - size, :, 1] = 2.0, 2.0
        if size > 1:
            kt[t - size + 1, :, 1], vt[t - size + 1, :, 1] = 1.0, 1.0
        kt, vt, qt = kt.to(store).float(), vt.to(store).float(), q.to(store).float()
        order = [4, 1, 3, 0, 2]
        k_pool, v_pool = paged(kt[:t + 1], PAGE, order, store), paged(vt[:t + 1], PAGE, order, store)
        table = as_int([order + [0]])
        want = plain.masked_softmax_attention(qt[:t + 1].double(), kt[:t + 1].double(), vt[:t + 1].double(), 1.0, size, keep_first, None)
        if size > 1 or keep_first:
            assert float((want[t, :, 1] - 1.0).abs().max()) < 1e-3           # what the plain heads say is what this test means
        tensor_cores = dtype == "bf16" and d == dv
        for impl in (["generic", "ws"] if tensor_cores else ["generic"]):
            out = torch.full((1, nq, dv), float("nan"), dtype=store, device=DEV)
            kernels.attention_decode(qt[t:t + 1].to(DEV, store), k_pool, v_pool, out, table, as_int([t + 1]), nkv, PAGE, 0, size, 1.0, 2,
                                     torch.empty(4 * nq * dv, device=DEV), torch.empty(8 * nq, device=DEV), impl=impl, keep_first=keep_first)
            close(out, want[t:t + 1], dtype, f"token {t}, {impl}")
        begin = t - 39                                      # the same query as the last row of a portion of 40
        for impl in (["generic", "mma"] if tensor_cores else ["generic"]):
            out = torch.full((40, nq, dv), float("nan"), dtype=store, device=DEV)
            kernels.attention_prefill(qt[begin:t + 1].to(DEV, store), k_pool, v_pool, out, table, as_int([0, 40]), as_int([begin]), 40, nkv,
                                      PAGE, 0, size, 1.0, impl=impl, keep_first=keep_first)
            close(out, want[begin:t + 1], dtype, f"portion ending at {t}, {impl}")
    kernels.check_status(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, dv", [(24, 40), (64, 64)])
def test_the_sink_takes_the_weight_that_no_key_earns(dtype, d, dv):
    """Scores of -40 and below with a sink of 0: the output vanishes, where without the sink term the softmax would still
    spread a whole unit.  Equal scores of 0 with a sink of ln 3: n keys share n / (n + 3).  A sink of -30: it does not
    matter.  The sink is taken as it is: a score scale of 0.5 changes the keys' scores and not the sink's."""
    torch.manual_seed(d)
    store = STORE[dtype]
    total, nq, nkv = 150, 3, 1
    k = torch.zeros(total, nkv, d)
    k[:, :, 0] = 1.0
    v = torch.randn(total, nkv, dv) * 0.05
    v[:, :, 0] = 1.0
    q = torch.zeros(total, nq, d)
    q[0:50, :, 0] = -80.0
    q, k, v = q.to(store).float(), k.to(store).float(), v.to(store).float()
    sinks = torch.tensor([0.0, math.log(3.0), -30.0])
    want = sink_attention_all_ways(q, k, v, None, 0, sinks, 0.5, dtype, 140, "sink")
    assert float(want[:50, 0].abs().max()) < 1e-12
    count = torch.arange(51, 151, dtype=torch.float64)
    torch.testing.assert_close(want[50:, 1, 0], count / (count + 3.0), atol=1e-9, rtol=1e-9)
    torch.testing.assert_close(want[50:, 2, 0], torch.ones(100, dtype=torch.float64), atol=1e-9, rtol=1e-9)


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_among_hundreds(dtype):
    """Key 3 of 700 scores far above the rest; the output is its value, also against a sink of 5."""
    torch.manual_seed(3)
    store = STORE[dtype]
    total, nq, nkv, d, dv = 700, 4, 2, 64, 64
    k, v = torch.randn(total, nkv, d) * 0.1, torch.randn(total, nkv, dv) * 0.1
    k[3] = 0.0
    k[3, :, 0] = 8.0
    v[3, :, 0] = 8.0
    q = torch.randn(total, nq, d) * 0.1
    q[650:, :, 0] = 40.0
    q, k, v = q.to(store).float(), k.to(store).float(), v.to(store).float()
    want = sink_attention_all_ways(q, k, v, None, 0, torch.full((nq,), 5.0), 1.0, dtype, 690, "far key", order=list(range(11)))
    assert float((want[650:, :, 0] - 8.0).abs().max()) < 1e-3


def test_a_gate_of_one_number_per_head():
    torch.manual_seed(5)
    tokens, heads, dv, offset = 6, 5, 12, 16
    x = torch.randn(tokens, heads * dv)
    gate = torch.randn(2, tokens, offset + 8)
    for store in (torch.float32, torch.bfloat16):
        got = x.to(DEV, store)
        kernels.gate_mul(got, GemmOut(gate.to(DEV)), offset, group=dv)
        want = x.to(store).float().view(tokens, heads, dv) * torch.sigmoid(gate.sum(0)[:, offset:offset + heads])[:, :, None]
        torch.testing.assert_close(got.float().cpu(), want.view(tokens, -1), atol=1e-6 if store == torch.float32 else 2e-2, rtol=1e-2)


@pytest.mark.parametrize("heads, dim, vdim", [(2, 16, 32), (3, 12, 20), (1, 72, 136), (2, 130, 40), (6, 64, 32), (1, 256, 8), (2, 128, 128)])
def test_linear_attention_with_a_decay_per_head_in_portions(heads, dim, vdim):
    """Two sequences in slots out of order, run in unequal portions (one token, two, 16, 17, 50): the state that a portion
    leaves is what the next one starts from; split sums; SiLU on the way in; decays of 0 and of 1 among them.  Then the
    norm over all heads with the gate."""
    torch.manual_seed(heads * dim + vdim)
    lengths = {0: 86, 1: 53}
    cols = 2 * heads * dim + 2 * heads * vdim + 8
    at_k, at_v, at_gate = heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim
    decay = torch.tensor(([0.0, 1.0, 0.9, 0.5, 0.97, 0.999] * 2)[:heads])
    rows = {s: torch.randn(2, n, cols) * 0.7 for s, n in lengths.items()}
    want = {}
    for s, n in lengths.items():
        r = rows[s].double().sum(0)
        q, k = plain.silu(r[:, :at_k]).view(n, heads, dim), plain.silu(r[:, at_k:at_v]).view(n, heads, dim)
        v = plain.silu(r[:, at_v:at_gate]).view(n, heads, vdim)
        want[s] = plain.decayed_linear_attention(q, k, v, decay.double())
    states = torch.full((5, heads, vdim, dim), 55.0, device=DEV)
    slot = {0: 3, 1: 1}
    states[3].zero_()
    states[1].zero_()
    got = {s: [] for s in lengths}
    done = {0: 0, 1: 0}
    for portion in ((1, 2), (2, 1), (16, 17), (17, 16), (50, 17)):
        live = [s for s in (1, 0) if done[s] < lengths[s]]
        counts = [min(portion[s], lengths[s] - done[s]) for s in live]
        proj = torch.cat([rows[s][:, done[s]:done[s] + c] for s, c in zip(live, counts)], dim=1).to(DEV)
        out = torch.full((sum(counts), heads, vdim), float("nan"), device=DEV)
        step = _Step(counts, [done[s] for s in live], [slot[s] for s in live])
        kernels.linear_attention_scan(GemmOut(proj), 0, at_k, at_v, decay.to(DEV), states, out, step, dim, True)
        at = 0
        for s, c in zip(live, counts):
            got[s].append(out[at:at + c].cpu())
            at += c
            done[s] += c
    for s in lengths:
        torch.testing.assert_close(torch.cat(got[s]).double(), want[s], atol=2e-4, rtol=2e-4)
    assert float((states[0] - 55.0).abs().max()) == 0.0 and float((states[4] - 55.0).abs().max()) == 0.0
    # norm over all heads, gate, into both element types
    o = want[0].float().reshape(lengths[0], heads * vdim)
    weight = torch.randn(heads * vdim) * 0.2 + 1.0
    gate = rows[0].sum(0)[:, at_gate:at_gate + heads * vdim]
    wanted = plain.rms_divide(o.double(), 1e-5) * weight.double() * torch.sigmoid(gate.double())
    for store in (torch.float32, torch.bfloat16):
        out = torch.empty(lengths[0], heads * vdim, dtype=store, device=DEV)
        kernels.linear_attention_gate_norm(o.to(DEV), GemmOut(rows[0].to(DEV)), at_gate, weight.to(DEV), 1e-5, 1.0, out)
        torch.testing.assert_close(out.float().cpu().double(), wanted, atol=1e-4 if store == torch.float32 else 3e-2, rtol=1e-2)


def test_a_write_to_the_state_survives_hundreds_of_tokens():
    """With a decay of 1 the first token's key and value are read back by a query 600 tokens later; with a decay of 0.99
    they arrive times 0.99^599; with a decay of 0 only the query's own token answers."""
    heads, dim, vdim, tokens = 3, 16, 8, 601
    cols = 2 * heads * dim + heads * vdim
    rows = torch.zeros(1, tokens, cols)
    rows[0, 0, heads * dim:2 * heads * dim] = 1.0                        # k_0 = ones
    rows[0, 0, 2 * heads * dim:] = torch.arange(1, heads * vdim + 1).float()          # v_0
    rows[0, -1, :heads * dim] = 1.0 / dim                                # q_600 = ones / dim
    rows[0, -1, heads * dim:2 * heads * dim] = 1.0
    rows[0, -1, 2 * heads * dim:] = 100.0
    states = torch.zeros(2, heads, vdim, dim, device=DEV)
    out = torch.empty(tokens, heads, vdim, device=DEV)
    decay = torch.tensor([1.0, 0.99, 0.0])
    done = 0
    for count in (300, 1, 1, 299):
        kernels.linear_attention_scan(GemmOut(rows[:, done:done + count].to(DEV)), 0, heads * dim, 2 * heads * dim, decay.to(DEV), states, out[done:done + count],
                                      _Step([count], [done], [1]), dim, False)
        done += count
    first = torch.arange(1, heads * vdim + 1).float().view(heads, vdim)
    want = first * (decay ** 600)[:, None] + 100.0
    torch.testing.assert_close(out[-1].cpu(), want, atol=1e-3, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, width, ff, experts, top, shared", [(5, 64, 24, 6, 2, 40), (70, 96, 16, 5, 3, None), (300, 64, 32, 4, 1, 16), (3, 36, 9, 3, 3, 7),
                                                                    (40, 72, 20, 1, 1, None)])
def test_experts_weighted_at_their_input(dtype, tokens, width, ff, experts, top, shared):
    """The routed feed-forward part alone (router, choice, scores as they are, the score on the expert's input, the shared
    expert added without a gate) against the plain one, for few pairs (a pass per pair) and many (tiles of rows)."""
    from qwen_triton_b200.parts.base import Runtime, Workspace
    from qwen_triton_b200.parts.feed_forward import RoutedExperts
    torch.manual_seed(tokens + width)
    store = STORE[dtype]
    device = torch.device(DEV)
    runtime = Runtime(device=device, dtype=store, max_step_tokens=512, max_positions=64, workspace=Workspace(device))
    params = {"hidden_size": width, "expert_size": ff, "experts": experts, "top": top, "activation": "silu", "normalize": False, "weight_on": "input",
              "shared": {"intermediate_size": shared} if shared else None, "shared_gated": False, "router": "router", "expert": "e{}", "gate": "gate",
              "up": "up", "down": "down", "shared_name": "shared", "weight_suffix": ""}
    part = RoutedExperts(params, "l0.mlp", runtime)
    tensors = {}
    for name, spec in RoutedExperts.expected_tensors(params, "l0.mlp").items():
        std = 1.0 if name.endswith("router") else 0.3
        tensors[name] = (torch.randn(*spec.shape) * std).to(store)
    part.load(lambda name: tensors[name])
    runtime.workspace.allocate()
    x = torch.randn(tokens, width).to(store)
    got = part.forward(x.to(DEV), None).value()
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.routed_feed_forward(x.double(), {n: t.double() for n, t in tensors.items()}, "l0.mlp", mlp)
    if dtype == "fp32":
        torch.testing.assert_close(got.cpu().double(), want, atol=2e-4, rtol=2e-4)
    else:
        off = (got.cpu().double() - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
        assert float(off.mean()) < 0.02 and int((off > 0.08).sum()) <= max(1, tokens // 50), f"mean {float(off.mean()):.4f}, worst {float(off.max()):.4f}"
    kernels.check_status(DEV)


# ============================================================================= whole models through the engine
def run_whole(engine, tokens):
    slot = engine.new_sequence()
    try:
        return engine.step([StepEntry(slot, list(tokens), list(range(len(tokens))))])
    finally:
        engine.release(slot)


@pytest.mark.parametrize("name, dtype", CASES)
def test_each_request_alone_and_whole(name, dtype):
    engine = engine_of(name, dtype, peaky=True)
    for length, seed in ((1, 0), (7, 1), (150, 2)):
        tokens = tokens_of(name, length, seed)
        close_rows(run_whole(engine, tokens), name, dtype, True, tokens, slice(None), f"{name} {length} tokens")
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", CASES)
def test_prompt_then_token_by_token_across_window_and_page_edges(name, dtype):
    """A prompt of 20 tokens, then 130 tokens one by one: every window and kept range of the model passes over decoded
    tokens, and positions 63, 64, 65, 127, 128 are decoded."""
    engine = engine_of(name, dtype, peaky=True)
    tokens = tokens_of(name, 150, 3)
    slot = engine.new_sequence()
    rows = [engine.step([StepEntry(slot, tokens[:20], [19])])]
    rows += [engine.step([StepEntry(slot, [t], [0])]) for t in tokens[20:]]
    engine.release(slot)
    close_rows(torch.cat(rows), name, dtype, True, tokens, slice(19, None), name)
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", CASES)
def test_token_by_token_from_the_first_token(name, dtype):
    engine = engine_of(name, dtype)
    tokens = tokens_of(name, 24, 4)
    slot = engine.new_sequence()
    rows = [engine.step([StepEntry(slot, [t], [0])]) for t in tokens]
    engine.release(slot)
    close_rows(torch.cat(rows), name, dtype, False, tokens, slice(None), name)


@pytest.mark.parametrize("name, dtype", CASES)
@pytest.mark.parametrize("portion", [2, 3, 17, 64, 100])
def test_portions_of_a_prompt(name, dtype, portion):
    engine = engine_of(name, dtype, peaky=True)
    tokens = tokens_of(name, 140, 5)
    slot = engine.new_sequence()
    rows = []
    for begin in range(0, len(tokens), portion):
        piece = tokens[begin:begin + portion]
        rows.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]))
    engine.release(slot)
    close_rows(torch.cat(rows), name, dtype, True, tokens, slice(None), f"{name} in portions of {portion}")
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", CASES)
def test_passes_smaller_than_a_prompt_and_a_prompt_of_more_than_256_tokens(name, dtype):
    """max_step_tokens = 96 cuts the prompt into passes; 300 tokens take the products' many-row forms and, for the
    windowed layers, several chunks of the ring."""
    tokens = tokens_of(name, 300, 6)
    for limit in (96, 4096):
        engine = engine_of(name, dtype, peaky=True, max_step_tokens=limit)
        close_rows(run_whole(engine, tokens), name, dtype, True, tokens, slice(None), f"{name}, passes of {limit}")
        engine.check_kernels()


@pytest.mark.parametrize("name, dtype", CASES)
def test_unequal_batches_with_slots_states_and_pages_used_again(name, dtype):
    """Three unequal requests start together and are decoded together; one ends early; a fourth takes the slot, state rows
    and pages that were given back, and must find a state of zero there."""
    engine = engine_of(name, dtype, peaky=True, max_tokens=640)
    lengths, more = (70, 1, 129), (6, 3, 9)
    requests = [tokens_of(name, n + m, 10 + i) for i, (n, m) in enumerate(zip(lengths, more))]
    slots = [engine.new_sequence() for _ in requests]
    got = [[] for _ in requests]
    out = engine.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, requests, lengths)])
    for i in range(3):
        got[i].append(out[i:i + 1])
    live = [0, 1, 2]
    for t in range(max(more)):
        for i in list(live):
            if t >= more[i]:
                engine.release(slots[i])
                live.remove(i)
        out = engine.step([StepEntry(slots[i], [requests[i][lengths[i] + t]], [0]) for i in live])
        for row, i in enumerate(live):
            got[i].append(out[row:row + 1])
    late = tokens_of(name, 90, 20)
    slot = engine.new_sequence()
    assert slot in slots[:2]
    rows = engine.step([StepEntry(slot, late, list(range(90))), StepEntry(slots[2], [requests[2][-1]], [])])
    close_rows(rows, name, dtype, True, late, slice(None), f"{name}: a request in a slot used again")
    for i, (n, req) in enumerate(zip(lengths, requests)):
        close_rows(torch.cat(got[i]), name, dtype, True, req, slice(n - 1, n + more[i]), f"{name} batch row {i}")
    engine.release(slot)
    engine.release(slots[2])
    engine.cache.book.check()
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", [("regupel-tiny-a", "fp32"), ("regupel-tiny-a", "bf16"), ("regupel-tiny-b", "bf16"), ("odd", "fp32")])
def test_many_short_requests_at_once(name, dtype):
    engine = engine_of(name, dtype, peaky=True, max_tokens=4096)
    requests = [tokens_of(name, 2 + (5 * i) % 23, 30 + i) for i in range(21)]
    slots = [engine.new_sequence() for _ in requests]
    out = engine.step([StepEntry(s, r[:-1], list(range(len(r) - 1))) for s, r in zip(slots, requests)])
    last = engine.step([StepEntry(s, r[-1:], [0]) for s, r in zip(slots, requests)])
    at = 0
    for i, req in enumerate(requests):
        rows = torch.cat([out[at:at + len(req) - 1], last[i:i + 1]])
        at += len(req) - 1
        close_rows(rows, name, dtype, True, req, slice(None), f"{name} request {i} of 21")
    for slot in slots:
        engine.release(slot)
    engine.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_of_several_rows(dtype):
    """Five rows decoded for 150 steps from short prompts: every window of the model passes over decoded tokens several
    times over, the kept first keys are decoded ones for the rows whose prompt is shorter than what is kept, and the
    states carry 150 updates."""
    name = "regupel-tiny-a"
    engine = engine_of(name, dtype, peaky=True)
    requests = [tokens_of(name, 1 + 2 * i + 150, 40 + i) for i in range(5)]
    slots = [engine.new_sequence() for _ in requests]
    engine.step([StepEntry(slot, req[:1 + 2 * i], []) for i, (slot, req) in enumerate(zip(slots, requests))])
    last = None
    for step in range(150):
        last = engine.step([StepEntry(slot, [req[1 + 2 * i + step]], [0]) for i, (slot, req) in enumerate(zip(slots, requests))]).cpu()
    for i, req in enumerate(requests):
        close_rows(last[i:i + 1], name, dtype, True, req, slice(len(req) - 1, None), f"row {i} after 150 steps")
    engine.check_kernels()


@pytest.mark.parametrize("name", MODELS)
def test_greedy_generation_through_the_entry_point(name):
    folder, _, _ = model(name, "fp32")
    lm = QwenB200ForCausalLM.from_pretrained_hf(folder, dtype="fp32", max_tokens=1024)
    prompts = [tokens_of(name, n, 60 + n) for n in (5, 1, 40)]
    results = lm.generate(prompts, max_new_tokens=12, ignore_eos=True)
    for prompt, result in zip(prompts, results):
        assert len(result.tokens) == 12
        sequence = list(prompt)
        for token in result.tokens:
            logits = oracle(name, "fp32", False, tuple(sequence))[-1]
            best = logits.topk(2).values
            if float(best[0] - best[1]) > 1e-3:          # a clear choice: the library must have made it
                assert int(logits.argmax()) == token, f"{name}: after {len(sequence)} tokens"
            sequence.append(token)
    lm16 = QwenB200ForCausalLM.from_pretrained_hf(model(name, "bf16")[0], dtype="bf16", max_tokens=1024)
    for result in lm16.generate(prompts, max_new_tokens=12, ignore_eos=True, temperature=0.7, seed=3):
        assert len(result.tokens) == 12 and all(0 <= t < config_of(name).vocab_size for t in result.tokens)


def test_random_weights_on_the_device_equal_the_written_folder():
    name = "regupel-tiny-b"
    folder, _, _ = model(name, "bf16")
    tokens = tokens_of(name, 50, 70)
    written = run_whole(Engine.from_pretrained(folder, dtype="bf16", max_tokens=512), tokens)
    drawn = run_whole(Engine.from_config(config_of(name), seed=13 + len(name), dtype="bf16", max_tokens=512), tokens)
    assert torch.equal(written, drawn)


def test_command_line_with_a_preset_and_random_weights():
    result = subprocess.run([sys.executable, "-m", "qwen_triton_b200.scripts.smoke", "--preset", "regupel-tiny-a", "--random-weights",
                             "--random-prompts", "9,2", "--max-new-tokens", "5", "--dtype", "bf16"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]


@pytest.mark.parametrize("dtype, name", [("float32", "fp32"), ("bfloat16", "bf16")])
def test_trace_replay_of_a_folder(tmp_path, dtype, name):
    """bin/trace_run as a child process: two requests start together, decode together, one ends earlier; a third comes
    alone afterwards and finds their slots and state rows."""
    model_name = "regupel-tiny-a"
    folder, _, _ = model(model_name, name)
    a, b, c = tokens_of(model_name, 90, 90), tokens_of(model_name, 31, 91), tokens_of(model_name, 70, 92)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:80], "want": [0, 63, 64, 79]}, {"id": "b", "tokens": b[:30], "want": [29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[80]], "want": [0]}, {"id": "b", "tokens": [b[30]], "want": [0]}], "end": ["b"]}]
    for i in range(81, 90):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [a[i]], "want": [0] if i % 2 else []}], "end": ["a"] if i == 89 else []})
    steps.append({"step": len(steps), "entries": [{"id": "c", "tokens": c, "want": [69]}], "end": ["c"]})
    out = tmp_path / "out"
    result = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "160"],
                            input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert result.returncode == 0, result.stderr[-2000:]
    assert [line for line in result.stdout.splitlines() if line.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    want = {key: oracle_and_margins(model_name, name, False, tuple(req)) for key, req in (("a", a), ("b", b), ("c", c))}
    at = {"a": 0, "b": 0, "c": 0}
    import numpy as np
    for record in steps:
        rows = []
        for entry in record["entries"]:
            rows += [(want[entry["id"]][0][at[entry["id"]] + w], want[entry["id"]][1][at[entry["id"]] + w]) for w in entry["want"]]
            at[entry["id"]] += len(entry["tokens"])
        path = out / f"{record['step']}.f32"
        if not rows:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(len(rows), -1).copy())
        clear = torch.tensor([name != "bf16" or float(margin) >= CLOSE_CALL for _, margin in rows])
        assert bool(torch.isfinite(got).all())
        if bool(clear.any()):
            close(got[clear], torch.stack([row for row, _ in rows])[clear], name, f"step {record['step']}", model_rows=True)
