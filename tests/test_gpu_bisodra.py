"""The Bisodra design on the GPU against the plain implementation (tests/plain_bisodra.py): every mechanism alone at the
kernels, with inputs made so that a fault shows (a key just outside a window, the first key that is no longer kept, a
row whose whole weight goes to the sink, a far key among hundreds), then whole models through the engine: whole prompts,
token by token, portions down to two tokens, unequal batches, slots and pages used again, long decoding, greedy
generation through the entry point, the command line and the trace replay."""
import functools
import json
import math
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest
import torch

import plain_bisodra as plain
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

# a third configuration beside the two presets: an attention layer first and last; one key head per query head and one
# key head for all; convolutions of one and of seven taps; more kept first keys than the window is long; a window of one
# position; no mask at all; two readers of one layer's latent, one directly behind it; latents and ranks that differ from
# one another; a plain rotation of a part of the rotated elements; layers without a feed-forward; scales of 1
ODD = {
    "architecture": "Bisodra", "vocab": 61, "width": 40, "norm": {"eps": 1e-4}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
    "layers": [
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 16, "scale": 0.3, "conv": 1, "mask": {"size": 5, "keep_first": 9}}},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 24},
         "mixer": {"heads": 2, "dim": 12, "rot_dim": 6, "vdim": 20, "q_rank": 9, "kv_rank": 40, "scale": 0.35, "rot": {"base": 100.0, "dims": 2}}},
        {"type": "latent_attention", "mlp": None,
         "mixer": {"heads": 5, "dim": 8, "rot_dim": 6, "vdim": 4, "q_rank": 33, "kv_rank": 40, "scale": 0.5, "kv_from": 1,
                   "rot": {"base": 100.0, "dims": 2}}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 72},
         "mixer": {"heads": 5, "kv_heads": 1, "dim": 24, "vdim": 24, "scale": 0.2, "conv": 7}},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 8},
         "mixer": {"heads": 1, "dim": 4, "rot_dim": 6, "vdim": 70, "q_rank": 4, "kv_rank": 40, "scale": 0.6, "kv_from": 1,
                   "rot": {"base": 100.0, "dims": 2}}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 16},
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.25, "conv": 2, "mask": {"size": 1, "keep_first": 0}}},
    ],
}
MODELS = ("bisodra-tiny-a", "bisodra-tiny-b", "odd")
CASES = [(name, dtype) for name in MODELS for dtype in DTYPES]


def config_of(name):
    return config_from_dict(ODD) if name == "odd" else load_preset(name)


@functools.lru_cache(maxsize=None)
def model(name: str, dtype: str, peaky: bool = False):
    """(folder, raw config, float weights for the plain implementation).  ``peaky``: the query and key matrices are two
    and a half times as large, so that few keys, far ones among them, carry each softmax."""
    config = config_of(name)
    holder = tempfile.TemporaryDirectory(prefix=f"qt_{name}_{dtype}_")
    _KEEP.append(holder)
    folder = write_random_model(holder.name, config, seed=11 + len(name), dtype=STORE[dtype])
    if peaky:
        checkpoint = Checkpoint(folder)
        tensors = {n: checkpoint.read(n) for n in checkpoint.names()}
        for n in list(tensors):
            if n.endswith((".mix.q", ".mix.k", ".mix.uq", ".mix.uk")):
                tensors[n] = (tensors[n].float() * 2.5).to(tensors[n].dtype)
        write_safetensors(Path(folder) / "model.safetensors", tensors)
    checkpoint = Checkpoint(folder)
    weights = {n: checkpoint.read(n).float() for n in checkpoint.names()}
    return folder, config.to_hf_dict(), weights


@functools.lru_cache(maxsize=None)
def oracle(name: str, dtype: str, peaky: bool, tokens: tuple) -> torch.Tensor:
    _, raw, weights = model(name, dtype, peaky)
    return plain.forward(raw, weights, list(tokens), torch.float64).float()


def tokens_of(name: str, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(177 + seed)
    return torch.randint(0, config_of(name).vocab_size, (length,), generator=generator).tolist()


def engine_of(name, dtype, peaky=False, **kwargs) -> Engine:
    kwargs.setdefault("max_tokens", 2048)
    return Engine.from_pretrained(model(name, dtype, peaky)[0], dtype=dtype, **kwargs)


def as_int(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("width, rows", [(96, 5), (130, 33), (7, 1), (1024, 3), (5000, 2), (2052, 4)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_before_and_after_a_sublayer(width, rows, out_dtype):
    """stream += norm_b(delta), then norm_a(stream): both with the mean taken off, a weight and no bias.  Rows with a
    large mean and a small spread tell a layer norm from an RMS norm and a variance around the mean from a mean square."""
    torch.manual_seed(width)
    eps = 1e-5
    stream = torch.randn(rows, width) * 0.3 + 7.0
    delta = torch.randn(2, rows, width) + 3.0
    post, weight = torch.rand(width) + 0.5, torch.rand(width) + 0.5
    want_stream = stream.double() + plain.layer_norm(delta.double().sum(0), post.double(), eps)
    want = plain.layer_norm(want_stream, weight.double(), eps)
    residual = stream.to(DEV)
    out = torch.empty(rows, width, dtype=out_dtype, device=DEV)
    kernels.add_layernorm(residual, GemmOut(delta.to(DEV)), post.to(DEV), weight.to(DEV), eps, out)
    torch.testing.assert_close(residual.cpu(), want_stream.float(), atol=1e-4, rtol=1e-5)
    tol = dict(atol=2e-4, rtol=2e-4) if out_dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out.float().cpu(), want.float(), **tol)
    # no delta: the stream stays; chosen rows only
    picked = as_int(sorted({0, rows - 1}))
    some = torch.empty(picked.shape[0], width, dtype=out_dtype, device=DEV)
    before = residual.clone()
    kernels.add_layernorm(residual, None, None, weight.to(DEV), eps, some, rows=picked)
    assert torch.equal(before, residual)
    torch.testing.assert_close(some.float().cpu(), want[picked.cpu().long()].float(), **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, taps", [(4, 2, 16, 4), (3, 3, 12, 1), (2, 1, 40, 7), (5, 1, 8, 2), (1, 1, 64, 16)])
def test_short_convolution_of_queries_and_keys_in_portions(dtype, nq, nkv, d, taps):
    """Two sequences whose tokens arrive in unequal portions (of one and two tokens among them, shorter than the taps
    reach back), their last inputs kept in slots that are not in order; queries against the plain convolution of the
    whole sequences, keys read back from the pages."""
    torch.manual_seed(d + taps)
    store = STORE[dtype]
    lengths = (70, 23)
    channels = (nq + nkv) * d
    extra = 24                                            # columns behind the channels (a gate's) stay untouched
    inputs = [torch.randn(n, channels + extra, dtype=torch.float64) for n in lengths]
    weights = torch.randn(channels, taps) * 0.5
    want = [plain.short_conv(u[:, :channels], weights.double()) for u in inputs]
    slots, orders = [3, 1], ([4, 0], [2])
    kept = torch.zeros(5, max(taps - 1, 1), channels, device=DEV)
    pool = torch.full((6, nkv, PAGE, d), 50.0, dtype=store, device=DEV)
    table = as_int([orders[0], orders[1] + [5]])
    got, done = [[], []], [0, 0]
    for portion in ((33, 1), (1, 2), (2, 20), (34, 0)):
        live = [s for s in (0, 1) if portion[s]]
        step = _Step([portion[s] for s in live], [done[s] for s in live], [slots[s] for s in live])
        rows = torch.cat([inputs[s][done[s]:done[s] + portion[s]] for s in live], dim=0)
        proj = GemmOut(torch.stack((rows * 0.25, rows * 0.75)).float().to(DEV).contiguous())
        q = torch.empty(rows.shape[0], nq, d, dtype=store, device=DEV)
        kernels.conv_qk_write(proj, weights.to(DEV), kept, step, q, pool, table[live].contiguous(), nq, nkv, d, PAGE, 0)
        at = 0
        for s in live:
            got[s].append(q[at:at + portion[s]].float().cpu())
            at += portion[s]
            done[s] += portion[s]
    kernels.check_status(DEV)
    assert float(kept[[0, 2, 4]].abs().max()) == 0.0
    for s in (0, 1):
        close(torch.cat(got[s]).reshape(lengths[s], -1), want[s][:, :nq * d], dtype, f"queries of sequence {s}")
        keys = torch.stack([pool[orders[s][t // PAGE], :, t % PAGE] for t in range(lengths[s])]).float().cpu()
        close(keys.reshape(lengths[s], -1), want[s][:, nq * d:], dtype, f"keys of sequence {s}")
        if taps > 1:                                      # what is kept: the raw inputs of the last taps - 1 positions
            torch.testing.assert_close(kept[slots[s]].cpu(), inputs[s][-(taps - 1):, :channels].float(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sigmoid_gate_and_the_exact_gelu(dtype):
    torch.manual_seed(5)
    store = STORE[dtype]
    x = torch.randn(37, 48).to(store)
    gate = torch.randn(2, 37, 80) * 2.0
    got = x.to(DEV)
    kernels.gate_mul(got, GemmOut(gate.to(DEV)), 24)
    close(got, x.double() * torch.sigmoid(gate.double().sum(0)[:, 24:72]), dtype, "gate")
    z = torch.linspace(-6.0, 6.0, 37 * 80).view(1, 37, 80)
    out = torch.empty(37, 80, dtype=store, device=DEV)
    kernels.activation(GemmOut(z.to(DEV).contiguous()), out, "gelu")
    want = plain.gelu_erf(z[0].double())
    close(out, want, dtype, "gelu")
    if dtype == "fp32":                                   # the erf form, not its tanh approximation (they differ by 5e-4 near |z| = 2)
        tanh_form = torch.nn.functional.gelu(z[0].double(), approximate="tanh")
        assert float((tanh_form - want).abs().max()) > 3e-4 > float((out.cpu().double() - want).abs().max())


def attention_impls(dtype, d, decode):
    """The generic kernels take every type and size; in bfloat16, heads in steps of 16 up to 128 also run on mma.sync
    tiles (the engine's choice there)."""
    if dtype != "bf16" or d % 16 or d > 128:
        return ["generic"]
    return ["generic", "ws" if decode else "mma"]


def biased_attention_all_ways(q, k, size, keep_first, scale, dtype, prompt, what, order=None):
    """q [T, H, d], k [T, G, d] (rounded to the type already): the first ``prompt`` positions as one prompt, a later
    portion of it from the cache, and the remaining positions one at a time with several counts of key ranges, through
    every kernel that takes the call, against the plain heads."""
    total, nq, d = q.shape
    nkv = k.shape[1]
    store = STORE[dtype]
    want = plain.biased_heads(q.double(), k.double(), torch.arange(total), scale, size, keep_first)
    order = order or list(range(-(-total // PAGE)))[::-1]
    pool = paged(k, PAGE, order, store)
    table = as_int([order + [0]])
    slope = plain.slopes(nq, torch.float32).to(DEV)
    options = dict(penalty=(slope, None), keep_first=keep_first, sink=True)
    for impl in attention_impls(dtype, d, decode=False):
        out = torch.full((prompt, nq, d), float("nan"), dtype=store, device=DEV)
        kernels.attention_prefill(q[:prompt].to(DEV, store), pool, pool, out, table, as_int([0, prompt]), as_int([0]), prompt, nkv, PAGE, 0,
                                  size, scale, impl=impl, **options)
        close(out, want[:prompt], dtype, f"{what}: prompt, {impl}")
        begin = prompt * 2 // 3
        out = torch.full((prompt - begin, nq, d), float("nan"), dtype=store, device=DEV)
        kernels.attention_prefill(q[begin:prompt].to(DEV, store), pool, pool, out, table, as_int([0, prompt - begin]), as_int([begin]),
                                  prompt - begin, nkv, PAGE, 0, size, scale, impl=impl, **options)
        close(out, want[begin:prompt], dtype, f"{what}: portion from {begin}, {impl}")
    for impl in attention_impls(dtype, d, decode=True):
        for t in range(prompt, total):
            for splits, warps in ((1, 1), (3, 2), (8, 4)):
                out = torch.full((1, nq, d), float("nan"), dtype=store, device=DEV)
                kernels.attention_decode(q[t:t + 1].to(DEV, store), pool, pool, out, table, as_int([t + 1]), nkv, PAGE, 0, size, scale, splits,
                                         torch.empty(8 * nq * d, device=DEV), torch.empty(16 * nq, device=DEV), impl=impl,
                                         warps=warps if impl == "ws" else 1, **options)
                close(out, want[t:t + 1], dtype, f"{what}: token {t}, {impl}, {splits} ranges")
    kernels.check_status(DEV)
    return want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, size, keep_first", [(4, 2, 48, 37, 5), (6, 1, 16, 64, 64), (3, 3, 20, 1, 2), (2, 2, 64, 100, 0), (5, 5, 32, None, 0),
                                                         (2, 1, 128, 5, 70), (8, 2, 80, 130, 3), (1, 1, 24, 70, 129), (16, 1, 64, 65, 1)])
def test_linear_bias_kept_first_keys_and_sink(dtype, nq, nkv, d, size, keep_first):
    """Random queries and keys, 300 positions: the window's first page lies several pages behind the kept keys' last,
    and the window's edge and the kept keys' edge fall inside pages, at their borders and across them."""
    torch.manual_seed(nq * d)
    store = STORE[dtype]
    total = 300
    q = (torch.randn(total, nq, d) * 1.5).to(store).float()
    k = torch.randn(total, nkv, d).to(store).float()
    biased_attention_all_ways(q, k, size, keep_first, 1.0 / math.sqrt(d), dtype, 290, f"{nq} heads of {d}, window {size}, kept {keep_first}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, size, keep_first", [(32, 37, 6), (64, 64, 64), (128, 100, 1), (16, 1, 63), (48, 129, 65)])
def test_keys_just_inside_and_just_outside_the_window_and_the_kept_keys(dtype, d, size, keep_first):
    """For every query from position 200 on, the key just outside its window and the first key that is no longer kept
    would score 60, the key just inside the window and the last kept key score 30, everything else about 0: the output
    is a mixture of the two visible keys alone (dimension 1 of it is 1; a seen hidden key would make it 2)."""
    torch.manual_seed(d)
    store = STORE[dtype]
    total, nq, nkv = 270, 2, 1
    k = torch.randn(total, nkv, d) * 0.02
    k[:, :, 1] = 0.0
    k[keep_first - 1, :, 1] = 1.0
    k[keep_first, :, 1] = 2.0
    q = torch.zeros(total, nq, d)
    q[:, :, 1] = 30.0
    # the window's edge wanders with the query: mark, for the query at t, the keys t - size (outside) and t - size + 1
    # (inside) through a dimension of their own, so that other queries do not see these marks as scores
    want_rows = []
    for t in range(200, total):
        kt = k.clone()
        kt[t - size, :, 1] = 2.0
        if size > 1:
            kt[t - size + 1, :, 1] = 1.0
        kt = kt.to(store).float()
        qt = q.to(store).float()
        pool = paged(kt[:t + 1], PAGE, [4, 1, 3, 0, 2], store)
        table = as_int([[4, 1, 3, 0, 2, 0]])
        slope = plain.slopes(nq, torch.float32).to(DEV)
        want = plain.biased_heads(qt[t:t + 1].double(), kt[:t + 1].double(), torch.tensor([t]), 1.0, size, keep_first)
        if size > 1:
            assert float((want[..., 1] - 1.0).abs().max()) < 1e-3           # what the plain heads say is what this test means
        for impl in attention_impls(dtype, d, decode=True):
            out = torch.full((1, nq, d), float("nan"), dtype=store, device=DEV)
            kernels.attention_decode(qt[t:t + 1].to(DEV, store), pool, pool, out, table, as_int([t + 1]), nkv, PAGE, 0, size, 1.0, 2,
                                     torch.empty(4 * nq * d, device=DEV), torch.empty(8 * nq, device=DEV), impl=impl,
                                     penalty=(slope, None), keep_first=keep_first, sink=True)
            close(out, want, dtype, f"token {t}, {impl}")
        if t % 16 == 0:                                    # the same query as the last row of a portion of 40
            begin = t - 39
            rows = plain.biased_heads(qt[begin:t + 1].double(), kt[:t + 1].double(), torch.arange(begin, t + 1), 1.0, size, keep_first)
            for impl in attention_impls(dtype, d, decode=False):
                out = torch.full((40, nq, d), float("nan"), dtype=store, device=DEV)
                kernels.attention_prefill(qt[begin:t + 1].to(DEV, store), pool, pool, out, table, as_int([0, 40]), as_int([begin]), 40, nkv,
                                          PAGE, 0, size, 1.0, impl=impl, penalty=(slope, None), keep_first=keep_first, sink=True)
                close(out, rows, dtype, f"portion ending at {t}, {impl}")
        want_rows.append(want)
    kernels.check_status(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [24, 64])
def test_the_sink_takes_the_weight_that_no_key_earns(dtype, d):
    """Scores of -40 and below: without the sink term the softmax would still spread a whole unit over the keys; with it
    the output vanishes.  Scores around 0: every key and the sink weigh about the same.  Scores of +40: the sink does
    not matter."""
    torch.manual_seed(d)
    store = STORE[dtype]
    total, nq, nkv = 150, 2, 2
    k = torch.randn(total, nkv, d) * 0.05
    k[:, :, 0] = 1.0
    q = torch.zeros(total, nq, d)
    q[0:50, :, 0], q[100:, :, 0] = -40.0, 40.0
    q, k = q.to(store).float(), k.to(store).float()
    want = biased_attention_all_ways(q, k, None, 0, 1.0, dtype, 140, "sink")
    assert float(want[:50].abs().max()) < 1e-12 and float((want[120:, :, 0] - 1.0).abs().max()) < 1e-6
    count = torch.arange(51, 100, dtype=torch.float64)              # with equal scores of 0: n keys and the sink share the unit
    slope = plain.slopes(nq, torch.float64)
    for h in range(nq):
        weights = torch.stack([torch.exp(-slope[h] * torch.arange(int(n), dtype=torch.float64)).sum() for n in count])
        torch.testing.assert_close(want[50:99, h, 0], weights / (1.0 + weights), atol=1e-9, rtol=1e-9)


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_among_hundreds(dtype):
    """Key 3 of 700 scores far above the rest even after its distance is taken off; the output is that key."""
    torch.manual_seed(3)
    store = STORE[dtype]
    total, nq, nkv, d = 700, 4, 2, 64
    k = torch.randn(total, nkv, d) * 0.1
    k[3] = 0.0
    k[3, :, 0] = 8.0
    q = torch.randn(total, nq, d) * 0.1
    q[650:, :, 0] = 40.0
    q, k = q.to(store).float(), k.to(store).float()
    want = biased_attention_all_ways(q, k, None, 0, 1.0, dtype, 690, "far key", order=list(range(11)))
    assert float((want[650:, :, 0] - 8.0).abs().max()) < 1e-3


def rotation_table(rot, positions: int) -> torch.Tensor:
    """float32 [positions, dims]: cos | sin of every pair's angle, times the magnitude, as the kernels read them."""
    f, magnitude = plain.yarn_frequencies(rot)
    angles = torch.arange(positions, dtype=torch.float64)[:, None] * f[None, :]
    return (torch.cat((angles.cos(), angles.sin()), dim=-1) * magnitude).float().to(DEV)


ROTATIONS = [{"dims": 8, "base": 10000.0}, {"dims": 2, "base": 100.0},
             {"dims": 16, "base": 1000000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 1.0}},
             {"dims": 4, "base": 50.0, "scaling": {"factor": 40.0, "original": 16, "fast": 4.0, "slow": 2.0}}]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_rank, rank, rot_dim, heads, dim, rot", [(24, 40, 8, 3, 12, ROTATIONS[0]), (9, 132, 6, 1, 20, ROTATIONS[1]),
                                                                   (128, 64, 16, 6, 32, ROTATIONS[2]), (4, 8, 4, 5, 4, ROTATIONS[3]),
                                                                   (100, 260, 24, 2, 40, ROTATIONS[2])])
def test_latent_rows_and_rotated_parts(dtype, q_rank, rank, rot_dim, heads, dim, rot):
    """The first projection's sums -> the normed query latent, and per token one cache row [normed latent | shared key
    part, its first rot.dims elements turned by the position]; the rotated part of every head's query likewise.  Two
    sequences at positions far apart, pages out of order."""
    torch.manual_seed(rank + rot_dim)
    store = STORE[dtype]
    eps = 1e-5
    lengths, past = (21, 70), (50, 0)
    step = _Step(list(lengths), list(past), [0, 1])
    tokens = sum(lengths)
    cols = -(-(q_rank + rank + rot_dim + 5) // 8) * 8
    sums = torch.randn(tokens, cols, dtype=torch.float64) * 3.0
    q_w, kv_w = torch.rand(q_rank) + 0.5, torch.rand(rank) + 0.5
    table = rotation_table(rot, 200)
    pool = torch.full((5, 1, PAGE, rank + rot_dim), 50.0, dtype=store, device=DEV)
    pages = as_int([[3, 1], [0, 4]])
    cq = torch.empty(tokens, q_rank, dtype=store, device=DEV)
    proj = GemmOut(torch.stack((sums * 0.5, sums * 0.5)).float().to(DEV).contiguous())
    kernels.latent_prepare(proj, q_w.to(DEV), kv_w.to(DEV), eps, table, cq, pool, step.token_seq, step.token_pos, pages, rank, rot_dim, PAGE, 0)
    positions = step.token_pos.cpu().long()
    close(cq, plain.rms_norm(sums[:, :q_rank], q_w.double(), eps), dtype, "query latent")
    want_c = plain.rms_norm(sums[:, q_rank:q_rank + rank], kv_w.double(), eps)
    want_shared = plain.rotate_half(sums[:, q_rank + rank:q_rank + rank + rot_dim], positions, rot)
    at = 0
    for s, n in enumerate(lengths):
        rows = torch.stack([pool[int(pages[s, (past[s] + t) // PAGE]), 0, (past[s] + t) % PAGE] for t in range(n)]).float().cpu()
        close(rows[:, :rank], want_c[at:at + n], dtype, f"latent of sequence {s}")
        close(rows[:, rank:], want_shared[at:at + n], dtype, f"shared key part of sequence {s}")
        at += n
    # a reader of another layer's rows writes none
    before = pool.clone()
    kernels.latent_prepare(proj, q_w.to(DEV), None, eps, table, cq, None, step.token_seq, step.token_pos, None, rank, rot_dim, PAGE, 0, write_kv=False)
    assert torch.equal(before, pool)
    # the queries' rotated parts, behind ``rank`` elements of every head's row
    q_full = torch.randn(tokens, heads * (dim + rot_dim), dtype=torch.float64).to(store)
    out = torch.full((tokens, heads, rank + rot_dim), 7.0, dtype=store, device=DEV)
    kernels.latent_query_rot(GemmOut(q_full.to(DEV)[None]), table, step.token_pos, out, heads, dim, rot_dim, rank)
    turned = plain.rotate_half(q_full.double().view(tokens, heads, dim + rot_dim)[..., dim:], positions, rot)
    close(out[..., rank:], turned, dtype, "rotated query parts")
    assert float((out[..., :rank].float() - 7.0).abs().max()) == 0.0
    kernels.check_status(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, heads, n, k, gated", [(5, 3, 40, 12, False), (70, 1, 36, 132, True), (300, 6, 80, 128, True), (1, 5, 4, 8, True),
                                                       (33, 2, 260, 40, False), (17, 8, 128, 512, True)])
def test_a_product_per_head(dtype, tokens, heads, n, k, gated):
    """out[t, h] = W_h x[t, h] with a matrix per head, read at an offset of every head's part of x and written at an offset
    of every head's row, and with the sigmoid gate in its epilogue."""
    torch.manual_seed(n + k)
    store = STORE[dtype]
    x_head, x_offset, out_row, out_offset = k + 8, 8, n + 16, 16
    x = (torch.randn(tokens, heads, x_head) * 0.5).to(store)
    weight = (torch.randn(heads, n, k) * 0.3).to(store)
    gate = torch.randn(2, tokens, 24 + heads * n) if gated else None
    want = torch.einsum("thk,hnk->thn", x[..., x_offset:].double(), weight.double())
    if gated:
        want = want * torch.sigmoid(gate.double().sum(0)[:, 24:].view(tokens, heads, n))
    out = torch.full((tokens, heads, out_row), 7.0, dtype=store, device=DEV)
    kernels.head_product(x.to(DEV), weight.to(DEV), out, x_row=heads * x_head, x_head=x_head, x_offset=x_offset, out_offset=out_offset,
                         gate=GemmOut(gate.to(DEV)) if gated else None, gate_offset=24)
    scale = float(want.abs().max())
    close(out[..., out_offset:].float() / scale, want / scale, dtype, "product per head")
    assert float((out[..., :out_offset].float() - 7.0).abs().max()) == 0.0
    # x as a product's partial sums
    halves = GemmOut(torch.stack((x.float() * 0.25, x.float() * 0.75)).view(2, tokens, heads * x_head).to(DEV).contiguous())
    kernels.head_product(halves, weight.to(DEV), out, x_row=heads * x_head, x_head=x_head, x_offset=x_offset, out_offset=out_offset,
                         gate=GemmOut(gate.to(DEV)) if gated else None, gate_offset=24)
    close(out[..., out_offset:].float() / scale, want / scale, dtype, "product per head of partial sums")
    kernels.check_status(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, rank, rot_dim", [(3, 40, 8), (1, 132, 6), (6, 128, 16), (5, 8, 4), (2, 260, 24), (16, 512, 64),
                                                   (7, 56, 8), (4, 64, 24), (40, 96, 16), (70, 32, 16), (3, 264, 8)])
def test_attention_over_latent_rows(dtype, heads, rank, rot_dim):
    """Every head's query [rank | rot_dim] against the one cached row per token, whose first ``rank`` elements are the
    values: a prompt, a later portion and single tokens.  One far row carries the softmax of the last queries.  In
    bfloat16 the sizes that are multiples of 8 run on the tensor cores (rows padded to 16, head counts that do not divide a
    tile of 64 rows, more heads than a tile has rows, a value size that the two warps of a row group share unevenly), the
    others and float in the generic kernels."""
    torch.manual_seed(rank)
    store = STORE[dtype]
    total, prompt = 200, 190
    row = rank + rot_dim
    c = torch.randn(total, rank).to(store).float()
    shared = torch.randn(total, rot_dim).to(store).float()
    c[7], shared[7] = (c[7] * 4.0).to(store).float(), (shared[7] * 4.0).to(store).float()
    q = (torch.randn(total, heads, row) * 0.7).to(store).float()
    q[150:] = (q[150:] + 0.5 * torch.cat((c[7], shared[7]))[None, None, :]).to(store).float()
    scale = 1.0 / math.sqrt(row)
    eye = torch.eye(rank, dtype=torch.float64).repeat(heads, 1)
    want = plain.latent_heads(q[..., :rank].double(), q[..., rank:].double(), c.double(), shared.double(), eye, eye, torch.arange(total), scale)
    assert float((want[150:] - c[7].double()).abs().max()) < 1e-3
    order = [2, 0, 3, 1]
    pool = paged(torch.cat((c, shared), dim=1)[:, None, :], PAGE, order, store)
    table = as_int([order + [0]])
    out = torch.full((prompt, heads, rank), float("nan"), dtype=store, device=DEV)
    kernels.attention_prefill(q[:prompt].to(DEV, store), pool, pool, out, table, as_int([0, prompt]), as_int([0]), prompt, 1, PAGE, 0, None, scale,
                              v_dim=rank)
    close(out, want[:prompt], dtype, "prompt")
    out = torch.full((prompt - 120, heads, rank), float("nan"), dtype=store, device=DEV)
    kernels.attention_prefill(q[120:prompt].to(DEV, store), pool, pool, out, table, as_int([0, prompt - 120]), as_int([120]), prompt - 120, 1, PAGE,
                              0, None, scale, v_dim=rank)
    close(out, want[120:prompt], dtype, "portion")
    # single tokens late and early in the sequence (fewer keys than a page, than a part of a page, one more than a page),
    # with partial results that a block delivers one, two or four at a time
    for t in list(range(prompt, total)) + [0, 4, 16, 39, 63, 64]:
        for splits in (1, 3) if prompt < t < total - 1 else (1, 2, 3, 4, 8):
            out = torch.full((1, heads, rank), float("nan"), dtype=store, device=DEV)
            kernels.attention_decode(q[t:t + 1].to(DEV, store), pool, pool, out, table, as_int([t + 1]), 1, PAGE, 0, None, scale, splits,
                                     torch.full((8 * heads * rank,), float("nan"), device=DEV), torch.full((16 * heads,), float("nan"), device=DEV),
                                     v_dim=rank)
            close(out, want[t:t + 1], dtype, f"token {t}, {splits} partial results")
    kernels.check_status(DEV)


# ----------------------------------------------------------------------------- models and their oracle
def run_whole(engine, tokens):
    slot = engine.new_sequence()
    try:
        return engine.step([StepEntry(slot, list(tokens), list(range(len(tokens))))]).cpu()
    finally:
        engine.release(slot)


@pytest.mark.parametrize("name, dtype", CASES)
def test_each_request_alone_and_whole(name, dtype):
    engine = engine_of(name, dtype, peaky=True)
    for length, seed in ((1, 0), (2, 1), (7, 2), (150, 3)):
        tokens = tokens_of(name, length, seed)
        close(run_whole(engine, tokens), oracle(name, dtype, True, tuple(tokens)), dtype, f"{name} {length} tokens", model_rows=True)
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", CASES)
def test_prompt_then_token_by_token_across_window_and_page_edges(name, dtype):
    """A prompt that ends just before a page's edge, then 85 tokens one by one: they cross the page edges at 64 and 128,
    the windows of the models (1, 5, 33, 64, 70) pass over decoded tokens, and the first keys that a window keeps (2, 5,
    9, 64) leave the window while they stay seen; in captured steps from the second on."""
    engine = engine_of(name, dtype, peaky=True)
    tokens = tokens_of(name, 145, 4)
    want = oracle(name, dtype, True, tuple(tokens))
    slot = engine.new_sequence()
    got = [engine.step([StepEntry(slot, tokens[:60], list(range(60)))]).cpu()]
    for t in range(60, len(tokens)):
        got.append(engine.step([StepEntry(slot, [tokens[t]], [0])]).cpu())
    engine.release(slot)
    close(torch.cat(got), want, dtype, f"{name} token by token", model_rows=True)
    assert engine.graph_replays > 0
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", CASES)
def test_token_by_token_from_the_first_token(name, dtype):
    """No prompt at all: the convolutions start from zeros, the sink is the only other term of the first softmax."""
    engine = engine_of(name, dtype, peaky=True)
    tokens = tokens_of(name, 40, 14)
    slot = engine.new_sequence()
    got = [engine.step([StepEntry(slot, [t], [0])]).cpu() for t in tokens]
    engine.release(slot)
    close(torch.cat(got), oracle(name, dtype, True, tuple(tokens)), dtype, f"{name} from the first token", model_rows=True)


@pytest.mark.parametrize("name, dtype", CASES)
@pytest.mark.parametrize("portion", [2, 3, 17, 64, 100])
def test_portions_of_a_prompt(name, dtype, portion):
    engine = engine_of(name, dtype, peaky=True)
    tokens = tokens_of(name, 141, 5)
    want = oracle(name, dtype, True, tuple(tokens))
    slot = engine.new_sequence()
    got = []
    for begin in range(0, len(tokens), portion):
        piece = tokens[begin:begin + portion]
        got.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]).cpu())
    engine.release(slot)
    close(torch.cat(got), want, dtype, f"{name} in portions of {portion}", model_rows=True)


@pytest.mark.parametrize("name, dtype", CASES)
def test_passes_smaller_than_a_prompt(name, dtype):
    """A step whose tokens do not fit one pass is cut inside the engine; the convolutions' kept inputs go from pass to
    pass."""
    engine = engine_of(name, dtype, peaky=True, max_step_tokens=48)
    tokens = tokens_of(name, 130, 6)
    close(run_whole(engine, tokens), oracle(name, dtype, True, tuple(tokens)), dtype, f"{name} in passes of 48", model_rows=True)


@pytest.mark.parametrize("name, dtype", CASES)
def test_a_prompt_of_more_than_256_tokens(name, dtype):
    """Beyond 256 rows the products run by block pairs; every window is far shorter than the prompt, so most key tiles
    between the kept keys and the window are skipped.  Then four one-token steps."""
    engine = engine_of(name, dtype, peaky=True)
    tokens = tokens_of(name, 304, 8)
    want = oracle(name, dtype, True, tuple(tokens))
    slot = engine.new_sequence()
    got = [engine.step([StepEntry(slot, tokens[:300], list(range(300)))]).cpu()]
    for t in range(300, 304):
        got.append(engine.step([StepEntry(slot, [tokens[t]], [0])]).cpu())
    engine.release(slot)
    close(torch.cat(got), want, dtype, f"{name} 300 tokens and four more", model_rows=True)
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", CASES)
def test_unequal_batches_with_slots_and_pages_used_again(name, dtype):
    """Three turns on one engine.  Each: unequal prompts in one batch (one of a single token), then decoded together
    while the shorter requests end earlier; the slots, kept convolution inputs and pages of a turn are used again by
    the next, whose requests must not see what the earlier ones left there."""
    engine = engine_of(name, dtype, peaky=True, max_tokens=640)
    for turn in range(3):
        lengths = [(1, 5), (70, 9), (33, 2), (129, 12)][turn % 2:][:3]
        requests = [tokens_of(name, prompt + decoded, 10 * turn + i) for i, (prompt, decoded) in enumerate(lengths)]
        slots = [engine.new_sequence() for _ in requests]
        got = [[] for _ in requests]
        logits = engine.step([StepEntry(slot, req[:prompt], list(range(prompt))) for slot, req, (prompt, _) in zip(slots, requests, lengths)]).cpu()
        at = 0
        for i, (prompt, _) in enumerate(lengths):
            got[i].append(logits[at:at + prompt])
            at += prompt
        for step in range(max(d for _, d in lengths)):
            live = [i for i, (_, d) in enumerate(lengths) if step < d]
            logits = engine.step([StepEntry(slots[i], [requests[i][lengths[i][0] + step]], [0]) for i in live]).cpu()
            for row, i in enumerate(live):
                got[i].append(logits[row:row + 1])
            for i, (_, d) in enumerate(lengths):
                if step == d - 1:
                    engine.release(slots[i])
        for i, req in enumerate(requests):
            close(torch.cat(got[i]), oracle(name, dtype, True, tuple(req)), dtype, f"{name} turn {turn} request {i}", model_rows=True)
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", [("bisodra-tiny-a", "fp32"), ("bisodra-tiny-a", "bf16"), ("bisodra-tiny-b", "bf16"), ("odd", "fp32")])
def test_many_short_requests_at_once(name, dtype):
    """Twenty-one requests of 1 to 41 tokens start together and are decoded together for six steps: more rows than the
    cluster-fused products take, a captured step padded to 32 rows, and every request against its own run."""
    engine = engine_of(name, dtype, peaky=True)
    requests = [tokens_of(name, 1 + 2 * i + 6, 100 + i) for i in range(21)]
    slots = [engine.new_sequence() for _ in requests]
    logits = engine.step([StepEntry(slot, req[:-6], list(range(len(req) - 6))) for slot, req in zip(slots, requests)]).cpu()
    got, at = [], 0
    for req in requests:
        got.append([logits[at:at + len(req) - 6]])
        at += len(req) - 6
    for step in range(6):
        logits = engine.step([StepEntry(slot, [req[len(req) - 6 + step]], [0]) for slot, req in zip(slots, requests)]).cpu()
        for i in range(len(requests)):
            got[i].append(logits[i:i + 1])
    for slot in slots:
        engine.release(slot)
    for i, req in enumerate(requests):
        close(torch.cat(got[i]), oracle(name, dtype, True, tuple(req)), dtype, f"{name} request {i} of 21", model_rows=True)
    engine.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_of_several_rows(dtype):
    """Five rows decoded for 150 steps from short prompts: every window of the model passes over decoded tokens several
    times over, and the kept first keys are decoded ones for the rows whose prompt is shorter than what is kept."""
    name = "bisodra-tiny-a"
    engine = engine_of(name, dtype, peaky=True)
    requests = [tokens_of(name, 3 + 2 * i + 150, 40 + i) for i in range(5)]
    slots = [engine.new_sequence() for _ in requests]
    engine.step([StepEntry(slot, req[:3 + 2 * i], []) for i, (slot, req) in enumerate(zip(slots, requests))])
    last = None
    for step in range(150):
        last = engine.step([StepEntry(slot, [req[3 + 2 * i + step]], [0]) for i, (slot, req) in enumerate(zip(slots, requests))]).cpu()
    for i, req in enumerate(requests):
        close(last[i:i + 1], oracle(name, dtype, True, tuple(req))[-1:], dtype, f"row {i} after 150 steps", model_rows=True)
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
    # the same in bfloat16 with temperature runs and stays within the vocabulary
    lm16 = QwenB200ForCausalLM.from_pretrained_hf(model(name, "bf16")[0], dtype="bf16", max_tokens=1024)
    for result in lm16.generate(prompts, max_new_tokens=12, ignore_eos=True, temperature=0.7, seed=3):
        assert len(result.tokens) == 12 and all(0 <= t < config_of(name).vocab_size for t in result.tokens)


def test_random_weights_on_the_device_equal_the_written_folder():
    name = "bisodra-tiny-b"
    folder, _, _ = model(name, "bf16")
    tokens = tokens_of(name, 50, 70)
    written = run_whole(Engine.from_pretrained(folder, dtype="bf16", max_tokens=512), tokens)
    drawn = run_whole(Engine.from_config(config_of(name), seed=11 + len(name), dtype="bf16", max_tokens=512), tokens)
    assert torch.equal(written, drawn)


def test_command_line_with_a_preset_and_random_weights():
    result = subprocess.run([sys.executable, "-m", "qwen_triton_b200.scripts.smoke", "--preset", "bisodra-tiny-a", "--random-weights",
                             "--random-prompts", "9,2", "--max-new-tokens", "5", "--dtype", "bf16"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]


@pytest.mark.parametrize("dtype, name", [("float32", "fp32"), ("bfloat16", "bf16")])
def test_trace_replay_of_a_folder(tmp_path, dtype, name):
    """bin/trace_run as a child process: two requests start together, decode together, one ends earlier; a third
    comes alone afterwards and finds their slots."""
    model_name = "bisodra-tiny-a"
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
    want = {"a": oracle(model_name, name, False, tuple(a)), "b": oracle(model_name, name, False, tuple(b)), "c": oracle(model_name, name, False, tuple(c))}
    at = {"a": 0, "b": 0, "c": 0}
    import numpy as np
    for record in steps:
        rows = []
        for entry in record["entries"]:
            rows += [want[entry["id"]][at[entry["id"]] + w] for w in entry["want"]]
            at[entry["id"]] += len(entry["tokens"])
        path = out / f"{record['step']}.f32"
        if not rows:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(len(rows), -1).copy())
        close(got, torch.stack(rows), name, f"step {record['step']}", model_rows=True)
