"""Decode and prefill throughput of the Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl b200|reference] [--temperature T]
    python bench.py --workload 0.6b-unequal | 32b-long | lederax-layers | vunepel-layers | bisodra-layers | regupel-layers

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 from a 2,048-token cache,
timed on the device over the decode steps (step function plus greedy sampling kernel, tokens given
ahead); ``e2e`` is the same through the Python entry point with host token ids in and out at every
step; ``prefill`` is one 2,048-token prompt; ``roofline`` is the decode step's bytes (every weight
once plus the live cache) over its time against the measured HBM copy bandwidth; ``points`` holds
batch 1 and 64 with their fractions.  Weights are random, token ids are uniform random with a fixed seed.

A timed region runs at least K steps and at least ``--min-seconds`` (2 by default): a region of a few
dozen steps is shorter than the clock sampler's period and than the drift of the clocks under the power
cap.  ``steps`` is the number of steps actually timed, ``config.steps_requested`` is K.

``--workload`` runs one of the secondary workloads instead: ``0.6b-unequal`` (Qwen3-0.6B shape, 16 prompts with
lengths uniform in 64..2,048, 128 new tokens each, through ``generate``), ``32b-long`` (Qwen3-32B shape, batch
64 decoded from 2,048 to 4,096 positions, with the roofline fraction in windows of 64 steps near 2,048, 3,072 and 4,096),
``lederax-layers`` (four layers of the Lederax design at three sets of sizes that resemble a real model's, beside a Qwen3
dense model of the same width, heads, window and as many weights read per token: prefill of one prompt and one-token steps
at batch 8 and 64, each with its share of the measured peaks), ``vunepel-layers`` (the same for four layers of the
Vunepel design: differential attention with a dense feed-forward, two gated-delta-rule layers with routed experts, an
attention layer that reads the first one's keys and values; ``--size``, ``--arm`` and ``--phase`` run one of its
measurements alone, for a profiler), ``bisodra-layers`` (the same for four layers of the Bisodra design: attention through
a latent, attention with a short convolution on q and k under a window with kept first keys, a latent layer that reads the
first one's cache rows, a second convolution layer; the same three options), ``regupel-layers`` (four layers of the Regupel
design: two parallel layers, windowed attention with kept first keys beside a linear attention with a decay per head, and two
attention layers with a sink and a gate per head, each with routed experts and a shared expert, beside the Vunepel layers
of equal size; the same three options).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--preset", default="qwen3-8b")
    parser.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (0: all)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--prompt-len", type=int, default=2048)
    parser.add_argument("--no-points", action="store_true")
    parser.add_argument("--no-prefill", action="store_true")
    parser.add_argument("--min-seconds", type=float, default=2.0, help="a timed region lasts at least this long")
    parser.add_argument("--temperature", type=float, default=0.0, help="sampling temperature of the end-to-end run (0: greedy)")
    parser.add_argument("--workload", default=None, choices=["0.6b-unequal", "32b-long", "lederax-layers", "vunepel-layers", "bisodra-layers", "regupel-layers"])
    parser.add_argument("--size", default=None, help="vunepel-layers, bisodra-layers: only the size whose name starts with this")
    parser.add_argument("--arm", default=None, choices=["vunepel", "bisodra", "regupel", "dense"], help="vunepel-layers, bisodra-layers, regupel-layers: only this model")
    parser.add_argument("--phase", default=None, choices=["prefill", "decode8", "decode64"], help="vunepel-layers, bisodra-layers: only this measurement")
    return parser.parse_args()


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            flat = {}
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                value = data.get(key)
                if isinstance(value, dict):
                    value = value.get("value")
                if value:
                    flat[key] = float(value)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return flat, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.device_index = device_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.device_index), "-lms", "50"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 5]
        os.unlink(self.file.name)
        clocks, max_clock, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in rows:
            try:
                clocks.append(int(row[0]))
                max_clock = max(max_clock, int(row[1]))
            except ValueError:
                continue
            for name, cell in zip(names, row[2:6]):
                if cell.strip().lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None, "sm_max_mhz": max_clock or None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def random_prompts(batch: int, length: int, vocab: int, seed: int) -> list[list[int]]:
    import torch
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=generator).tolist()


# ----------------------------------------------------------------------------- this library
def model_numbers(config, layers: int) -> dict:
    h, d, nq, nkv, inter, vocab = (config.hidden_size, config.head_dim, config.num_attention_heads,
                                   config.num_key_value_heads, config.intermediate_size, config.vocab_size)
    per_layer = h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * inter
    return {"linear_params": per_layer * layers, "head_params": vocab * h,
            "kv_bytes_per_token": 2 * layers * nkv * d * 2,
            "attn_flops_per_pair": 4 * nq * d * layers}


def steps_for(ms_per_step: float, requested: int, min_seconds: float, most: int) -> int:
    """Steps of a timed region: at least the requested number and at least ``min_seconds`` of them, within ``most``."""
    return max(1, min(most, max(requested, int(min_seconds * 1e3 / max(ms_per_step, 1e-3)) + 1)))


def time_decode(model, prompts, steps: int, warmup: int, vocab: int, min_seconds: float, most_steps: int):
    """Device-timed decode: the batch's cache is filled by a real prefill, then ``warmup`` untimed steps of one
    given token per sequence, each followed by the greedy sampling kernel, then the timed region."""
    import torch
    from qwen_triton_b200 import StepEntry
    from qwen_triton_b200.ops import kernels

    engine = model.engine
    slots = [engine.new_sequence() for _ in prompts]
    for start in range(0, len(prompts), 2):      # fill the cache two prompts at a time
        part = range(start, min(start + 2, len(prompts)))
        engine.step([StepEntry(slots[i], prompts[i], []) for i in part])
    generator = torch.Generator().manual_seed(7)
    out = torch.empty(len(prompts), dtype=torch.int32, device=engine.device)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one(tokens):
        logits = engine.step([StepEntry(slot, [tok], [0]) for slot, tok in zip(slots, tokens)])
        kernels.argmax(logits, out)

    probe = 4                                    # untimed steps after the warm-up, only to size the timed region
    feed = torch.randint(0, vocab, (warmup + probe, len(prompts)), generator=generator).tolist()
    for tokens in feed[:warmup]:
        one(tokens)
    torch.cuda.synchronize()
    begin.record()
    for tokens in feed[warmup:]:
        one(tokens)
    end.record()
    torch.cuda.synchronize()
    steps = steps_for(begin.elapsed_time(end) / probe, steps, min_seconds, most_steps)
    warmup += probe
    feed = torch.randint(0, vocab, (steps, len(prompts)), generator=generator).tolist()
    launches = kernels.launch_count()
    with ClockSampler() as clocks:
        begin.record()
        for tokens in feed:
            one(tokens)
        end.record()
        torch.cuda.synchronize()
    launches = kernels.launch_count() - launches
    ms = begin.elapsed_time(end) / steps
    context = len(prompts[0]) + warmup + steps // 2          # mean cache length during the timed steps
    for slot in slots:
        engine.release(slot)
    return ms, launches, clocks.summary(), context, steps


def time_e2e(model, prompts, steps: int, warmup: int, min_seconds: float, most_steps: int, temperature: float = 0.0):
    """Through the entry point: host token ids in, sampled token ids back on the host, every step."""
    import torch
    run = model.start_batch(prompts, max_new_tokens=warmup + most_steps + 8, temperature=temperature, seed=5, ignore_eos=True)
    run.start()
    for _ in range(warmup):
        run.advance()
    torch.cuda.synchronize()
    wall = time.perf_counter()
    for _ in range(4):                           # untimed, only to size the timed region
        run.advance()
    torch.cuda.synchronize()
    steps = steps_for((time.perf_counter() - wall) * 1e3 / 4, steps, min_seconds, most_steps)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall = time.perf_counter()
    begin.record()
    for _ in range(steps):
        run.advance()
    end.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - wall) * 1e3 / steps
    ms = max(begin.elapsed_time(end) / steps, wall)
    h2d = model.engine.last_meta_bytes + (8 * len(prompts) if temperature > 0 else 0)     # sampling keys: request and step per row
    run.close()
    return ms, h2d, 4 * len(prompts), steps


VUNEPEL_SIZES = (
    # name, width, attention heads (two score maps each), kv heads, map and value size, chunk, delta heads, delta kv heads, delta key size,
    # delta value size, narrow columns, experts, top, expert width, shared width, dense width
    ("w2048-h8x2x128-chunk1024-delta16x128-e16x1024-top2", 2048, 8, 2, 128, 1024, 16, 4, 128, 128, 64, 16, 2, 1024, 1024, 6144),
    ("w4096-h16x2x128-chunk4096-delta32x128-e16x2048-top2", 4096, 16, 4, 128, 4096, 32, 8, 128, 128, 128, 16, 2, 2048, 2048, 12288),
    ("w1024-h8x2x64-chunk512-delta8x64-e8x2048-top1", 1024, 8, 8, 64, 512, 8, 8, 64, 128, 32, 8, 1, 2048, 1024, 3072),
)


def run_vunepel_layers(args) -> dict:
    """Prefill and one-token steps of four Vunepel layers at sizes that resemble a real model's (an attention layer
    with a dense feed-forward, two delta-rule layers with routed experts and a shared expert, an attention layer that
    reads the first one's keys and values, with routed experts), and of the Qwen3 dense layers that come closest: same
    width and vocabulary, one head per score map with the same head size, a window as long as the chunk, and a gated
    feed-forward that reads as many weights per token as the four layers' feed-forwards do on average."""
    import torch

    from qwen_triton_b200 import QwenB200ForCausalLM, config_from_dict

    peak, peak_source = peaks()
    vocab, prompt_len = 32768, args.prompt_len
    out = []
    for size in VUNEPEL_SIZES:
        name, width, heads, kv_heads, dim, chunk, d_heads, d_kv, d_dim, d_vdim, rank, experts, top, ff, shared, dense_ff = size
        if args.size and not name.startswith(args.size):
            continue
        moe = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 2.0}, "expert": {"ff": ff, "limit": 7.0},
               "shared": {"ff": shared, "limit": 7.0}}
        attention = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "diff": 0.3,
                     "rot": {"dims": dim // 2, "base": 500000.0}, "mask": {"size": chunk}}
        delta = {"heads": d_heads, "kv_heads": d_kv, "dim": d_dim, "vdim": d_vdim, "conv": 4, "ranks": {"decay": rank, "gate": rank}}
        vunepel = {"architecture": "Vunepel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
                   "layers": [{"type": "attention", "mixer": attention, "mlp": {"kind": "dense", "ff": dense_ff, "limit": 7.0}},
                              {"type": "channel_delta", "mixer": delta, "mlp": moe},
                              {"type": "channel_delta", "mixer": delta, "mlp": moe},
                              {"type": "attention", "mixer": {**attention, "kv_from": 0}, "mlp": moe}]}
        layers = 4
        # weights a token multiplies with, per layer kind (the experts: the chosen ones and the shared one)
        attn_own = width * (2 * heads + 2 * kv_heads) * dim + width * kv_heads * dim + heads * dim * width
        attn_reader = width * 2 * heads * dim + heads * dim * width
        delta_w = width * (2 * d_kv * d_dim + d_heads * d_vdim + d_heads + 2 * rank) + rank * d_heads * (d_dim + d_vdim) + d_heads * d_vdim * width
        moe_token = 3 * width * (ff * top + shared) + width * (experts + 1)
        mixers = attn_own + attn_reader + 2 * delta_w
        token_weights = mixers + 3 * width * dense_ff + 3 * moe_token
        inter = max(64, round((3 * width * dense_ff + 3 * moe_token) / 4 / (3 * width) / 64) * 64)
        dense = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": vocab, "hidden_size": width,
                 "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": 2 * heads,
                 "num_key_value_heads": 2 * kv_heads, "head_dim": dim, "max_position_embeddings": 32768,
                 "use_sliding_window": True, "sliding_window": chunk, "max_window_layers": 0}
        dense_token = layers * (width * (2 * heads + 4 * kv_heads) * dim + 2 * heads * dim * width + 3 * width * inter)
        entry = {"size": name, "layers": layers, "dense_intermediate": inter}
        # keys a query sees on average: within its chunk (vunepel) or its window (dense)
        seen = lambda context, span: min(context, span) / 2 if context <= span else span / 2

        def moe_read(rows):
            return 3 * width * (ff * min(experts, rows * top) + shared) + width * (experts + 1)

        arms = (("vunepel", vunepel, token_weights, lambda rows: mixers + 3 * width * dense_ff + 3 * moe_read(rows),
                 4 * 2 * 2 * heads * dim, 2 * (2 * 2 * kv_heads * dim + kv_heads * dim * 2), 2 * d_heads * d_dim * d_vdim * 4 * 2),
                ("dense", dense, dense_token, lambda rows: dense_token, 4 * layers * 2 * heads * dim, layers * 2 * 2 * kv_heads * dim * 2, 0))
        for label, raw, per_token, read_of, attn_flops_per_key, kv_bytes_per_key, state_bytes in arms:
            if args.arm and label != args.arm:
                continue
            model = QwenB200ForCausalLM.from_config(config_from_dict(raw), seed=1, dtype="bf16",
                                                    max_tokens=64 * (prompt_len + 512), max_seq_len=prompt_len + 512,
                                                    max_step_tokens=max(4096, prompt_len), chunk_tokens=prompt_len)
            result = {}
            if args.phase in (None, "prefill"):
                ms = time_prefill(model, prompt_len, vocab, repeats=args.steps if args.phase else 5, warmup=args.warmup if args.phase else 3)
                keys = seen(prompt_len, chunk) if label == "vunepel" else min(chunk, prompt_len / 2)
                flops = 2 * prompt_len * (per_token + vocab * width / prompt_len) + attn_flops_per_key * prompt_len * keys
                result["prefill"] = {"tokens": prompt_len, "ms": round(ms, 3), "tokens_per_s": round(prompt_len * 1e3 / ms),
                                     "tensor_fraction": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)}
            for batch in (8, 64):
                if args.phase not in (None, f"decode{batch}"):
                    continue
                prompts = random_prompts(batch, prompt_len, vocab, 300 + batch)
                ms, launches, clocks, context, steps = time_decode(model, prompts, args.steps, args.warmup, vocab,
                                                                   args.min_seconds / 4, 256)
                keys = (context % chunk) if label == "vunepel" else min(chunk, context)
                read = 2 * (read_of(batch) + vocab * width) + batch * (keys * kv_bytes_per_key + state_bytes)
                result[f"decode_batch{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch * 1e3 / ms),
                                                   "launches_per_step": round(launches / steps, 1), "steps": steps,
                                                   "hbm_fraction": round(read / (ms * 1e-3) / (peak["hbm_gbs"] * 1e9), 4),
                                                   "clocks": clocks}
            entry[label] = result
            print(f"[bench] {name} {label}: " + json.dumps({k: {a: b for a, b in v.items() if a != 'clocks'} for k, v in result.items()}),
                  file=sys.stderr, flush=True)
            del model
            torch.cuda.empty_cache()
        out.append(entry)
    return {"workload": args.workload, "impl": "b200", "dtype": "bf16", "data": "synthetic", "n_gpus": 1,
            "config": {"prompt_len": prompt_len, "layers": 4, "vocab": vocab, "peaks": peak_source,
                       "l2": "weights, caches and states of a step exceed L2 at every size but the smallest"},
            "sizes": out}


BISODRA_SIZES = (
    # name, width, latent heads, plain and rotated query/key size, value size, query latent, key/value latent,
    # convolution-attention heads, kv heads, head size, window, kept first keys, feed-forward width
    ("w2048-latent16x128+64-r512-conv16x128-win1024-ff8192", 2048, 16, 128, 64, 128, 768, 512, 16, 4, 128, 1024, 64, 8192),
    ("w4096-latent32x128+64-r512-conv32x128-win4096-ff16384", 4096, 32, 128, 64, 128, 1536, 512, 32, 8, 128, 4096, 128, 16384),
    ("w1024-latent8x64+32-r256-conv8x64-win512-ff4096", 1024, 8, 64, 32, 64, 384, 256, 8, 8, 64, 512, 16, 4096),
)


def run_bisodra_layers(args) -> dict:
    """Prefill and one-token steps of four Bisodra layers at sizes that resemble a real model's (attention through a
    latent; attention with a short convolution on q and k, a window with kept first keys, a distance bias and a sink; a
    latent layer that reads the first one's cache rows; a second convolution layer; each with a feed-forward of two
    matrices), and of the Qwen3 dense layers that come closest: same width and vocabulary, the convolution layers' heads,
    kv heads and head size, full attention in the first two layers and the same window in the last two, and a gated
    feed-forward that reads as many weights per token."""
    import torch

    from qwen_triton_b200 import QwenB200ForCausalLM, config_from_dict

    peak, peak_source = peaks()
    vocab, prompt_len = 32768, args.prompt_len
    out = []
    for size in BISODRA_SIZES:
        name, width, l_heads, l_dim, l_rot, l_vdim, q_rank, kv_rank, heads, kv_heads, dim, window, keep, ff = size
        if args.size and not name.startswith(args.size):
            continue
        rot = {"base": 1000000.0, "dims": l_rot, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
        latent = {"heads": l_heads, "dim": l_dim, "rot_dim": l_rot, "vdim": l_vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                  "scale": (l_dim + l_rot) ** -0.5, "rot": rot}
        conv = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "conv": 4,
                "mask": {"size": window, "keep_first": keep}}
        mlp = {"kind": "dense", "ff": ff}
        bisodra = {"architecture": "Bisodra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
                   "logit_scale": 1.0,
                   "layers": [{"type": "latent_attention", "mixer": latent, "mlp": mlp}, {"type": "attention", "mixer": conv, "mlp": mlp},
                              {"type": "latent_attention", "mixer": {**latent, "kv_from": 0}, "mlp": mlp},
                              {"type": "attention", "mixer": conv, "mlp": mlp}]}
        layers = 4
        row = kv_rank + l_rot
        # weights a token multiplies with, per layer kind (the per-head matrices of a latent layer once each)
        latent_reader = width * (q_rank + l_heads * l_vdim) + q_rank * l_heads * (l_dim + l_rot) + l_heads * kv_rank * (l_dim + l_vdim) \
            + l_heads * l_vdim * width
        latent_own = latent_reader + width * row
        conv_w = width * (2 * heads + kv_heads) * dim + heads * dim * width
        token_weights = latent_own + latent_reader + 2 * conv_w + layers * 2 * width * ff
        inter = max(64, round(2 * ff / 3 / 64) * 64)
        dense = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": vocab, "hidden_size": width,
                 "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": heads,
                 "num_key_value_heads": kv_heads, "head_dim": dim, "max_position_embeddings": 32768,
                 "use_sliding_window": True, "sliding_window": window, "max_window_layers": 2}
        dense_token = layers * (width * (heads + 2 * kv_heads) * dim + heads * dim * width + 3 * width * inter)
        entry = {"size": name, "layers": layers, "dense_intermediate": inter}

        def mean_keys(length, span, kept):
            """Keys a query of a prompt sees on average: all earlier ones, or the window's and the kept first ones."""
            if span is None:
                return (length + 1) / 2
            return sum(min(i + 1, span) + max(0, min(kept, i + 1 - span)) for i in range(length)) / length

        def live_keys(context, span, kept):
            return context if span is None else min(context, span + max(0, min(kept, context - span)))

        # per key and query token: attention FLOPs (scores and values), and bytes of cache a one-token step reads per key
        arms = (("bisodra", bisodra, token_weights,
                 ((2 * l_heads * (row + kv_rank), None, 0, 2 * row), (4 * heads * dim, window, keep, 2 * kv_heads * dim)) * 2),
                ("dense", dense, dense_token,
                 ((4 * heads * dim, None, 0, 4 * kv_heads * dim),) * 2 + ((4 * heads * dim, window, 0, 4 * kv_heads * dim),) * 2))
        for label, raw, per_token, attention in arms:
            if args.arm and label != args.arm:
                continue
            model = QwenB200ForCausalLM.from_config(config_from_dict(raw), seed=1, dtype="bf16",
                                                    max_tokens=64 * (prompt_len + 512), max_seq_len=prompt_len + 512,
                                                    max_step_tokens=max(4096, prompt_len), chunk_tokens=prompt_len)
            result = {}
            if args.phase in (None, "prefill"):
                ms = time_prefill(model, prompt_len, vocab, repeats=args.steps if args.phase else 5, warmup=args.warmup if args.phase else 3)
                flops = 2 * prompt_len * (per_token + vocab * width / prompt_len) \
                    + sum(f * prompt_len * mean_keys(prompt_len, span, kept) for f, span, kept, _ in attention)
                result["prefill"] = {"tokens": prompt_len, "ms": round(ms, 3), "tokens_per_s": round(prompt_len * 1e3 / ms),
                                     "tensor_fraction": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)}
            for batch in (8, 64):
                if args.phase not in (None, f"decode{batch}"):
                    continue
                prompts = random_prompts(batch, prompt_len, vocab, 300 + batch)
                ms, launches, clocks, context, steps = time_decode(model, prompts, args.steps, args.warmup, vocab,
                                                                   args.min_seconds / 4, 256)
                read = 2 * (per_token + vocab * width) + batch * sum(b * live_keys(context, span, kept) for _, span, kept, b in attention)
                result[f"decode_batch{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch * 1e3 / ms),
                                                   "launches_per_step": round(launches / steps, 1), "steps": steps,
                                                   "hbm_fraction": round(read / (ms * 1e-3) / (peak["hbm_gbs"] * 1e9), 4),
                                                   "clocks": clocks}
            entry[label] = result
            print(f"[bench] {name} {label}: " + json.dumps({k: {a: b for a, b in v.items() if a != 'clocks'} for k, v in result.items()}),
                  file=sys.stderr, flush=True)
            del model
            torch.cuda.empty_cache()
        out.append(entry)
    return {"workload": args.workload, "impl": "b200", "dtype": "bf16", "data": "synthetic", "n_gpus": 1,
            "config": {"prompt_len": prompt_len, "layers": 4, "vocab": vocab, "peaks": peak_source,
                       "l2": "weights and caches of a step exceed L2 at every size but the smallest"},
            "sizes": out}


REGUPEL_SIZES = (
    # name, width, attention heads, kv heads, head size (keys and values), window, kept first keys, rotated elements,
    # linear-attention heads, key size, value size, experts, top, expert width, shared width
    ("w2048-h16x128-win1024-lin16x128-e16x1024-top2", 2048, 16, 4, 128, 1024, 64, 64, 16, 128, 128, 16, 2, 1024, 1024),
    ("w4096-h32x128-win4096-lin32x128-e16x2048-top2", 4096, 32, 8, 128, 4096, 128, 64, 32, 128, 128, 16, 2, 2048, 2048),
    ("w1024-h8x64-win512-lin8x64-e8x2048-top1", 1024, 8, 8, 64, 512, 16, 32, 8, 64, 128, 8, 1, 2048, 1024),
)


def run_regupel_layers(args) -> dict:
    """Prefill and one-token steps of four Regupel layers at sizes that resemble a real model's (a parallel layer: windowed
    attention with kept first keys beside a linear attention with a decay per head; an attention layer with a stretched
    rotation, a sink and a gate per head; a second parallel layer; a second attention layer; each with routed experts
    and a shared expert), and of the Vunepel layers that come closest (the library's other design with a recurrent mixer
    beside attention and routed experts with a shared expert): same width and vocabulary, a delta-rule layer with the same
    heads and state size where the parallel layer stands, an attention layer with as many score maps of the same size
    under a chunk as long as the window, the same experts."""
    import torch

    from qwen_triton_b200 import QwenB200ForCausalLM, config_from_dict

    peak, peak_source = peaks()
    vocab, prompt_len = 32768, args.prompt_len
    out = []
    for size in REGUPEL_SIZES:
        name, width, heads, kv_heads, dim, window, keep, rot, r_heads, r_dim, r_vdim, experts, top, ff, shared = size
        if args.size and not name.startswith(args.size):
            continue
        moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}, "shared": {"ff": shared}}
        attention = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": window},
                     "rot": {"base": 1000000.0, "dims": rot, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 8192}}}
        left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": window, "keep_first": keep}}
        right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": [1.0 - 2.0 ** (-1 - 7 * h / max(r_heads - 1, 1)) for h in range(r_heads)]}
        parallel = {"left": left, "right": right, "left_scale": 0.7, "right_scale": 1.2}
        regupel = {"architecture": "Regupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
                   "logit_scale": 1.0, "residual_mult": 0.4,
                   "layers": [{"type": "parallel", "mixer": parallel, "mlp": moe}, {"type": "attention", "mixer": attention, "mlp": moe},
                              {"type": "parallel", "mixer": parallel, "mlp": moe}, {"type": "attention", "mixer": attention, "mlp": moe}]}
        v_moe = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 2.0}, "expert": {"ff": ff, "limit": 7.0},
                 "shared": {"ff": shared, "limit": 7.0}}
        v_heads, v_kv = max(1, heads // 2), max(1, kv_heads // 2)
        v_attention = {"heads": v_heads, "kv_heads": v_kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "diff": 0.3,
                       "rot": {"dims": rot, "base": 500000.0}, "mask": {"size": window}}
        delta = {"heads": r_heads, "kv_heads": r_heads, "dim": r_dim, "vdim": r_vdim, "conv": 4, "ranks": {"decay": 64, "gate": 64}}
        vunepel = {"architecture": "Vunepel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
                   "layers": [{"type": "channel_delta", "mixer": delta, "mlp": v_moe}, {"type": "attention", "mixer": v_attention, "mlp": v_moe},
                              {"type": "channel_delta", "mixer": delta, "mlp": v_moe}, {"type": "attention", "mixer": v_attention, "mlp": v_moe}]}
        layers = 4
        # weights a token multiplies with, per layer kind (the experts: the chosen ones and the shared one)
        attn_w = width * ((heads + 2 * kv_heads) * dim + heads) + heads * dim * width
        left_w = width * (heads + 2 * kv_heads) * dim + heads * dim * width
        right_w = width * r_heads * (2 * r_dim + 2 * r_vdim) + r_heads * r_vdim * width
        moe_token = 3 * width * (ff * top + shared) + width * experts
        mixers = 2 * attn_w + 2 * (left_w + right_w)
        token_weights = mixers + layers * moe_token
        v_attn_w = width * (2 * v_heads + 2 * v_kv) * dim + width * v_kv * dim + v_heads * dim * width
        v_delta_w = width * (2 * r_heads * r_dim + r_heads * r_vdim + r_heads + 128) + 64 * r_heads * (r_dim + r_vdim) + r_heads * r_vdim * width
        v_mixers = 2 * v_attn_w + 2 * v_delta_w
        v_token = v_mixers + layers * (moe_token + width)
        entry = {"size": name, "layers": layers}

        def moe_read(rows):
            return 3 * width * (ff * min(experts, rows * top) + shared) + width * experts

        def mean_keys(length, span, kept):
            return sum(min(i + 1, span) + max(0, min(kept, i + 1 - span)) for i in range(length)) / length

        def live_keys(context, span, kept):
            return min(context, span + max(0, min(kept, context - span)))

        # per arm: model, weights per token, weights a step of `rows` tokens reads, attention as (FLOPs per query and key, window,
        # kept keys, cache bytes per key) per layer that has one, bytes of state read and written per sequence and step
        arms = (("regupel", regupel, token_weights, lambda rows: mixers + layers * moe_read(rows),
                 ((4 * heads * dim, window, keep, 4 * kv_heads * dim), (4 * heads * dim, window, 0, 4 * kv_heads * dim)) * 2,
                 2 * r_heads * r_dim * r_vdim * 4 * 2),
                ("vunepel", vunepel, v_token, lambda rows: v_mixers + layers * (moe_read(rows) + width),
                 ((4 * 2 * v_heads * dim, window, 0, 2 * (2 * v_kv * dim + v_kv * dim)),) * 2, 2 * r_heads * r_dim * r_vdim * 4 * 2))
        for label, raw, per_token, read_of, attention_layers, state_bytes in arms:
            if args.arm and label != args.arm:
                continue
            model = QwenB200ForCausalLM.from_config(config_from_dict(raw), seed=1, dtype="bf16",
                                                    max_tokens=64 * (prompt_len + 512), max_seq_len=prompt_len + 512,
                                                    max_step_tokens=max(4096, prompt_len), chunk_tokens=prompt_len)
            result = {}
            if args.phase in (None, "prefill"):
                ms = time_prefill(model, prompt_len, vocab, repeats=args.steps if args.phase else 5, warmup=args.warmup if args.phase else 3)
                if label == "regupel":
                    pairs = sum(f * prompt_len * mean_keys(prompt_len, span, kept) for f, span, kept, _ in attention_layers)
                else:                      # a chunk's queries see the chunk's earlier keys
                    pairs = sum(f * prompt_len * (min(prompt_len, span) / 2) for f, span, _, _ in attention_layers)
                flops = 2 * prompt_len * (per_token + vocab * width / prompt_len) + pairs
                result["prefill"] = {"tokens": prompt_len, "ms": round(ms, 3), "tokens_per_s": round(prompt_len * 1e3 / ms),
                                     "tensor_fraction": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)}
            for batch in (8, 64):
                if args.phase not in (None, f"decode{batch}"):
                    continue
                prompts = random_prompts(batch, prompt_len, vocab, 300 + batch)
                ms, launches, clocks, context, steps = time_decode(model, prompts, args.steps, args.warmup, vocab,
                                                                   args.min_seconds / 4, 256)
                if label == "regupel":
                    keys = sum(b * live_keys(context, span, kept) for _, span, kept, b in attention_layers)
                else:
                    keys = sum(b * (context % span) for _, span, _, b in attention_layers)
                read = 2 * (read_of(batch) + vocab * width) + batch * (keys + state_bytes)
                result[f"decode_batch{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch * 1e3 / ms),
                                                   "launches_per_step": round(launches / steps, 1), "steps": steps,
                                                   "hbm_fraction": round(read / (ms * 1e-3) / (peak["hbm_gbs"] * 1e9), 4),
                                                   "clocks": clocks}
            entry[label] = result
            print(f"[bench] {name} {label}: " + json.dumps({k: {a: b for a, b in v.items() if a != 'clocks'} for k, v in result.items()}),
                  file=sys.stderr, flush=True)
            del model
            torch.cuda.empty_cache()
        out.append(entry)
    return {"workload": args.workload, "impl": "b200", "dtype": "bf16", "data": "synthetic", "n_gpus": 1,
            "config": {"prompt_len": prompt_len, "layers": 4, "vocab": vocab, "peaks": peak_source,
                       "l2": "weights, caches and states of a step exceed L2 at every size but the smallest"},
            "sizes": out}


def time_prefill(model, tokens: int, vocab: int, repeats: int = 5, warmup: int = 3):
    import torch
    from qwen_triton_b200 import StepEntry
    engine = model.engine
    prompt = random_prompts(1, tokens, vocab, 11)[0]
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for it in range(warmup + repeats):
        slot = engine.new_sequence()
        torch.cuda.synchronize()
        begin.record()
        engine.step([StepEntry(slot, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.release(slot)
        if it >= warmup:
            times.append(begin.elapsed_time(end))
    return statistics.median(times)


def config_keys(preset: dict, args, layers: int) -> dict:
    """The flat description of the model and workload that both arms print."""
    return {
        "model": f"{args.preset} shape, random weights", "layers": layers, "layers_of_model": preset["num_hidden_layers"],
        "hidden": preset["hidden_size"], "heads": preset["num_attention_heads"], "kv_heads": preset["num_key_value_heads"],
        "head_dim": preset["head_dim"], "intermediate": preset["intermediate_size"], "vocab": preset["vocab_size"],
        "global_batch": args.batch, "prompt_len": args.prompt_len, "parallelism": "single_gpu",
        "steps_requested": args.steps, "min_seconds": args.min_seconds,
        "l2": "inputs larger than L2: every step streams all weights",
    }


def preset_json(name: str) -> dict:
    return json.loads((ROOT / "qwen_triton_b200" / "config" / "presets" / f"{name}.json").read_text())


MOST_STEPS = 1024        # a timed region never runs more steps than this (sizes the cache)


def run_b200(args) -> dict:
    import dataclasses

    from qwen_triton_b200 import QwenB200ForCausalLM, load_preset

    full = load_preset(args.preset)
    layers = args.layers or full.num_hidden_layers
    config = full if layers == full.num_hidden_layers else dataclasses.replace(
        full, num_hidden_layers=layers, layer_types=full.layer_types[:layers])
    peak, peak_source = peaks()
    numbers = model_numbers(config, layers)
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    most_steps = max(args.steps, MOST_STEPS)
    max_context = -(-(args.prompt_len + args.warmup + most_steps + 16) // 64) * 64
    max_tokens = max(batches) * max_context + 4096
    model = QwenB200ForCausalLM.from_config(config, seed=0, dtype="bf16", max_tokens=max_tokens,
                                            max_seq_len=max_context, max_step_tokens=4096)
    vocab = config.vocab_size
    weight_bytes = 2 * (numbers["linear_params"] + numbers["head_params"])      # the embedding is read row-wise only

    from qwen_triton_b200.ops import kernels

    def progress(text: str) -> None:
        kernels.check_status(model.engine.device)        # raises if a bounded wait inside a kernel ran out
        print(f"[bench] {text}", file=sys.stderr, flush=True)

    def fraction(batch: int, result: dict) -> float:
        step_bytes = weight_bytes + batch * result["context"] * numbers["kv_bytes_per_token"]
        return step_bytes / (result["ms"] * 1e-3) / 1e9 / peak["hbm_gbs"]

    progress(f"model built: {layers} layers")
    results = {}
    for batch in batches:
        prompts = random_prompts(batch, args.prompt_len, vocab, 100 + batch)
        seconds = args.min_seconds if batch == args.batch else args.min_seconds / 2
        ms, launches, clocks, context, steps = time_decode(model, prompts, args.steps, args.warmup, vocab, seconds, most_steps)
        progress(f"decode at batch {batch}: {ms:.3f} ms per step over {steps} steps")
        results[batch] = {"ms": ms, "tok_s": batch * 1e3 / ms, "launches": launches, "clocks": clocks,
                          "context": context, "steps": steps}
    main = results[args.batch]
    step_bytes = weight_bytes + args.batch * main["context"] * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (main["ms"] * 1e-3) / 1e9

    prompts = random_prompts(args.batch, args.prompt_len, vocab, 100 + args.batch)
    e2e_ms, h2d, d2h, e2e_steps = time_e2e(model, prompts, args.steps, args.warmup, args.min_seconds, most_steps, args.temperature)
    progress(f"end to end at batch {args.batch}: {e2e_ms:.3f} ms per step over {e2e_steps} steps")

    points = {}
    for batch, result in results.items():
        if batch != args.batch:
            points[f"decode_b{batch}"] = round(result["tok_s"], 2)
            points[f"decode_b{batch}_frac"] = round(fraction(batch, result), 4)
    line = {
        "metric": "decode_tokens_per_s", "value": round(main["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": main["steps"], "warmup": args.warmup, "ms_per_step": round(main["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "b200",
        "config": {**config_keys(preset_json(args.preset), args, layers), "seq_len": args.prompt_len + args.warmup + main["steps"],
                   "context_mean": main["context"], "peaks": peak_source},
        "clocks": main["clocks"],
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps, "temperature": args.temperature},
        "gpu_launches": main["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "bytes_per_step": step_bytes},
        "points": points,
    }
    if not args.no_prefill:
        tokens = args.prompt_len
        ms = time_prefill(model, tokens, vocab)
        progress(f"prefill of {tokens} tokens: {ms:.3f} ms")
        flops = 2 * tokens * numbers["linear_params"] + 2 * numbers["head_params"] \
            + numbers["attn_flops_per_pair"] * tokens * (tokens + 1) // 2
        line["prefill"] = {"value": round(tokens * 1e3 / ms, 1), "tokens": tokens, "ms": round(ms, 3),
                           "frac": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4), "flops": flops}
    return line


# ----------------------------------------------------------------------------- the Lederax design beside the dense model
LEDERAX_SIZES = (
    # name, width, heads, kv heads, head size, window, experts, top, expert width
    ("w2048-h16-win1024-e32x1024-top2", 2048, 16, 4, 128, 1024, 32, 2, 1024),
    ("w4096-h32-win4096-e16x2048-top2", 4096, 32, 8, 128, 4096, 16, 2, 2048),
    ("w1024-h16-d64-win512-e8x4096-top1", 1024, 16, 16, 64, 512, 8, 1, 4096),
)


def run_lederax_layers(args) -> dict:
    """Prefill and one-token steps of a few Lederax layers at sizes that resemble a real model's, and of the Qwen3
    dense layers that come closest: same width, heads, head size, window and vocabulary, and a gated feed-forward
    that reads as many weights per token as the chosen experts do (3 h i = 2 h ff top)."""
    import torch

    from qwen_triton_b200 import QwenB200ForCausalLM, config_from_dict

    peak, peak_source = peaks()
    layers, vocab, prompt_len = args.layers or 4, 32768, args.prompt_len
    out = []
    for name, width, heads, kv_heads, dim, window, experts, top, ff in LEDERAX_SIZES:
        inter = max(64, round(2 * ff * top / 3 / 64) * 64)
        lederax = {"architecture": "Lederax", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
                   "norm": {"eps": 1e-6, "groups": 4},
                   "layers": [{"type": "attention",
                               "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                                         "mask": {"size": window}, "v_mix": True},
                               "mlp": {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}}] * layers}
        dense = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": vocab, "hidden_size": width,
                 "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": heads,
                 "num_key_value_heads": kv_heads, "head_dim": dim, "max_position_embeddings": 32768,
                 "use_sliding_window": True, "sliding_window": window, "max_window_layers": 0}
        attention = width * (heads + 2 * kv_heads) * dim + heads * dim * width
        entry = {"size": name, "layers": layers, "dense_intermediate": inter}
        for label, raw, mlp_read, mlp_flops in (("lederax", lederax, lambda rows: 2 * width * ff * min(experts, rows * top), 2 * width * ff * top),
                                                ("dense", dense, lambda rows: 3 * width * inter, 3 * width * inter)):
            model = QwenB200ForCausalLM.from_config(config_from_dict(raw), seed=1, dtype="bf16",
                                                    max_tokens=64 * (prompt_len + 512), max_seq_len=prompt_len + 512,
                                                    max_step_tokens=max(4096, prompt_len), chunk_tokens=prompt_len)
            result = {}
            ms = time_prefill(model, prompt_len, vocab)
            flops = 2 * prompt_len * (layers * (attention + mlp_flops) + vocab * width / prompt_len) \
                + 4 * layers * heads * dim * prompt_len * min(window, prompt_len / 2)
            result["prefill"] = {"tokens": prompt_len, "ms": round(ms, 3), "tokens_per_s": round(prompt_len * 1e3 / ms),
                                 "tensor_fraction": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)}
            for batch in (8, 64):
                prompts = random_prompts(batch, prompt_len, vocab, 300 + batch)
                ms, launches, clocks, context, steps = time_decode(model, prompts, args.steps, args.warmup, vocab,
                                                                   args.min_seconds / 4, 256)
                read = 2 * (layers * (attention + mlp_read(batch)) + vocab * width) \
                    + batch * min(window, context) * layers * 2 * kv_heads * dim * 2
                result[f"decode_batch{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch * 1e3 / ms),
                                                   "launches_per_step": round(launches / steps, 1), "steps": steps,
                                                   "hbm_fraction": round(read / (ms * 1e-3) / (peak["hbm_gbs"] * 1e9), 4),
                                                   "clocks": clocks}
            entry[label] = result
            print(f"[bench] {name} {label}: " + json.dumps({k: {a: b for a, b in v.items() if a != 'clocks'} for k, v in result.items()}),
                  file=sys.stderr, flush=True)
            del model
            torch.cuda.empty_cache()
        out.append(entry)
    return {"workload": args.workload, "impl": "b200", "dtype": "bf16", "data": "synthetic", "n_gpus": 1,
            "config": {"prompt_len": prompt_len, "layers": layers, "vocab": vocab, "peaks": peak_source,
                       "l2": "weights and caches of a step exceed L2 at every size but the smallest"},
            "sizes": out}


# ----------------------------------------------------------------------------- secondary workloads
def run_workload(args) -> dict:
    """BASELINE's secondary workloads as they are stated."""
    if args.workload == "lederax-layers":
        return run_lederax_layers(args)
    if args.workload == "vunepel-layers":
        return run_vunepel_layers(args)
    if args.workload == "bisodra-layers":
        return run_bisodra_layers(args)
    if args.workload == "regupel-layers":
        return run_regupel_layers(args)
    import torch

    from qwen_triton_b200 import QwenB200ForCausalLM, StepEntry, load_preset
    from qwen_triton_b200.ops import kernels

    peak, peak_source = peaks()
    if args.workload == "0.6b-unequal":
        config = load_preset("qwen3-0.6b")
        numbers = model_numbers(config, config.num_hidden_layers)
        generator = torch.Generator().manual_seed(16)
        lengths = torch.randint(64, 2049, (16,), generator=generator).tolist()
        prompts = [torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for n in lengths]
        new_tokens = 128
        model = QwenB200ForCausalLM.from_config(config, seed=0, dtype="bf16", max_tokens=16 * 2304 + 4096, max_seq_len=2304)
        times = []
        for _ in range(4):                                   # the first run warms up (launches, then captured steps)
            torch.cuda.synchronize()
            with ClockSampler() as clocks:
                start = time.perf_counter()
                results = model.generate(prompts, max_new_tokens=new_tokens, ignore_eos=True)
                torch.cuda.synchronize()
                times.append(time.perf_counter() - start)
        assert all(len(r.tokens) == new_tokens for r in results)
        seconds = statistics.median(times[1:])
        # decode alone, device-timed, from the same unequal caches
        engine = model.engine
        slots = [engine.new_sequence() for _ in prompts]
        for i in range(0, 16, 4):
            engine.step([StepEntry(slots[j], prompts[j], []) for j in range(i, i + 4)])
        out = torch.empty(16, dtype=torch.int32, device=engine.device)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        feed = torch.randint(0, config.vocab_size, (8 + new_tokens, 16), generator=generator).tolist()
        for row in feed[:8]:
            kernels.argmax(engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, row)]), out)
        begin.record()
        for row in feed[8:]:
            kernels.argmax(engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, row)]), out)
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / new_tokens
        weight_bytes = 2 * (numbers["linear_params"] + numbers["head_params"])
        step_bytes = weight_bytes + (sum(lengths) + 16 * (8 + new_tokens // 2)) * numbers["kv_bytes_per_token"]
        return {"workload": args.workload, "impl": "b200", "dtype": "bf16", "data": "synthetic",
                "config": {"model": "qwen3-0.6b shape, random weights", "layers": config.num_hidden_layers, "requests": 16,
                           "prompt_tokens": sum(lengths), "prompt_min": min(lengths), "prompt_max": max(lengths),
                           "new_tokens": new_tokens, "peaks": peak_source},
                "generate": {"seconds": round(seconds, 4), "new_tokens_per_s": round(16 * new_tokens / seconds, 1),
                             "all_tokens_per_s": round((sum(lengths) + 16 * new_tokens) / seconds, 1)},
                "decode": {"ms_per_step": round(ms, 4), "tokens_per_s": round(16e3 / ms, 1),
                           "frac": round(step_bytes / (ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4), "bytes_per_step": step_bytes},
                "clocks": clocks.summary()}

    config = load_preset("qwen3-32b")
    numbers = model_numbers(config, config.num_hidden_layers)
    batch, first, last = 64, 2048, 4096
    model = QwenB200ForCausalLM.from_config(config, seed=0, dtype="bf16", max_tokens=batch * last + 4096, max_seq_len=last,
                                            max_step_tokens=4096)
    engine = model.engine
    print("[bench] model built", file=sys.stderr, flush=True)
    prompts = random_prompts(batch, first, config.vocab_size, 164)
    slots = [engine.new_sequence() for _ in prompts]
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for i in range(0, batch, 2):
        engine.step([StepEntry(slots[j], prompts[j], []) for j in range(i, i + 2)])
    end.record()
    torch.cuda.synchronize()
    prefill_ms = begin.elapsed_time(end)
    kernels.check_status(engine.device)
    print(f"[bench] prompts: {prefill_ms:.0f} ms", file=sys.stderr, flush=True)
    out = torch.zeros(batch, dtype=torch.int32, device=engine.device)
    weight_bytes = 2 * (numbers["linear_params"] + numbers["head_params"])
    marks, window = {}, 64
    # windows of 64 steps, clear of the first steps (launched, then captured) and of the context buckets' edges
    # (a new bucket's first two steps are launched and captured as well)
    centres = (first + 96, (first + last) // 2 - 64, last - 64)
    starts = {c - window // 2: c for c in centres}
    stops = {c + window // 2: c for c in centres}
    events = {c: [torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)] for c in centres}
    total_begin, total_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rows = list(range(batch))
    with ClockSampler() as clocks:
        total_begin.record()
        for position in range(first, last):                  # the token fed at this step sits at `position`
            if position in starts:
                events[starts[position]][0].record()
            plan = engine.plan_decode(slots)
            if position == first:                            # the first tokens come from the host, the others stay on the device
                logits = engine.run_planned(plan, [p[-1] for p in prompts])
            else:
                logits = engine.run_planned(plan, rows, chosen=out)
            kernels.argmax(logits, out)
            if position + 1 in stops:
                events[stops[position + 1]][1].record()
        total_end.record()
        torch.cuda.synchronize()
    kernels.check_status(engine.device)
    total_ms = total_begin.elapsed_time(total_end)
    for centre, pair in events.items():
        ms = pair[0].elapsed_time(pair[1]) / window
        step_bytes = weight_bytes + batch * centre * numbers["kv_bytes_per_token"]
        marks[f"ctx_{centre}"] = {"ms_per_step": round(ms, 3), "tokens_per_s": round(batch * 1e3 / ms, 1),
                                  "frac": round(step_bytes / (ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4)}
    return {"workload": args.workload, "impl": "b200", "dtype": "bf16", "data": "synthetic",
            "config": {"model": "qwen3-32b shape, random weights", "layers": config.num_hidden_layers, "global_batch": batch,
                       "from": first, "to": last, "peaks": peak_source},
            "prefill": {"tokens": batch * first, "ms": round(prefill_ms, 1), "tokens_per_s": round(batch * first * 1e3 / prefill_ms, 1)},
            "decode": {"steps": last - first, "seconds": round(total_ms / 1e3, 3),
                       "tokens_per_s": round(batch * (last - first) * 1e3 / total_ms, 1), **marks},
            "clocks": clocks.summary()}


# ----------------------------------------------------------------------------- the reference
def run_reference(args) -> dict:
    """The unmodified reference installed under baseline/_ref, through its own public API: build the model
    from the same configuration with random weights, prefill the batch with ``use_cache=True``, then time
    one-token forwards with ``logits_to_keep=1`` followed by argmax, as its ``greedy_generate`` does
    (qwen_triton/models/core.py:392-409).  ``value`` is timed on the device with the tokens given ahead; ``e2e``
    is that loop as the reference's generation runs it: token ids from the host to the device, forward, argmax,
    ids back to the host, every step, by the wall clock."""
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "qwen_triton").exists():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --target baseline/_ref of the reference)"}
    try:
        os.environ.setdefault("HF_HUB_OFFLINE", "1")
        sys.path.insert(0, str(ref_root))
        import torch
        from qwen_triton.configs import QwenTritonConfig
        from qwen_triton.models import QwenTritonForCausalLM

        preset = preset_json(args.preset)
        full_layers = preset["num_hidden_layers"]
        layers = args.layers or full_layers
        most_steps = max(args.steps, 256)
        preset["num_hidden_layers"] = layers
        preset["max_position_embeddings"] = -(-(args.prompt_len + 2 * (args.warmup + most_steps) + 8) // 64) * 64
        torch.manual_seed(0)
        with torch.device("cuda"):
            model = QwenTritonForCausalLM.from_config(QwenTritonConfig.from_hf_config(preset))
        model = model.to(torch.bfloat16).eval()
        vocab = preset["vocab_size"]
        ids = torch.tensor(random_prompts(args.batch, args.prompt_len, vocab, 100 + args.batch), device="cuda")
        generator = torch.Generator().manual_seed(7)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.no_grad():
            out = model(input_ids=ids, use_cache=True, logits_to_keep=1)
            cache = out.past_key_values

            def one(tokens):
                nonlocal cache
                step = model(input_ids=tokens, past_key_values=cache, use_cache=True, logits_to_keep=1)
                cache = step.past_key_values
                return step.logits[:, -1].argmax(dim=-1)

            feed = torch.randint(0, vocab, (args.warmup, args.batch, 1), generator=generator).cuda()
            torch.cuda.synchronize()
            begin.record()
            for t in range(args.warmup):
                one(feed[t])
            end.record()
            torch.cuda.synchronize()
            steps = steps_for(begin.elapsed_time(end) / max(1, args.warmup), args.steps, args.min_seconds, most_steps)
            feed = torch.randint(0, vocab, (steps, args.batch, 1), generator=generator).cuda()
            with ClockSampler() as clocks:
                begin.record()
                for t in range(steps):
                    one(feed[t])
                end.record()
                torch.cuda.synchronize()
            ms = begin.elapsed_time(end) / steps

            # end to end: the last tokens go from the host to the device, the chosen ones come back, every step
            e2e_steps = steps_for(ms, args.steps, args.min_seconds, most_steps)
            host = torch.randint(0, vocab, (args.batch, 1), generator=generator).pin_memory()
            back = torch.empty(args.batch, dtype=torch.long).pin_memory()
            torch.cuda.synchronize()
            wall = time.perf_counter()
            for _ in range(e2e_steps):
                chosen = one(host.to("cuda", non_blocking=True))
                back.copy_(chosen, non_blocking=True)
                torch.cuda.synchronize()
                host.copy_(back[:, None])
            e2e_ms = (time.perf_counter() - wall) * 1e3 / e2e_steps
        return {
            "metric": "decode_tokens_per_s", "value": round(args.batch * 1e3 / ms, 2), "unit": "tokens/s", "n_gpus": 1,
            "steps": steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {**config_keys(preset_json(args.preset), args, layers), "seq_len": args.prompt_len + args.warmup + steps,
                       "context_mean": args.prompt_len + args.warmup + steps // 2},
            "clocks": clocks.summary(),
            "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": 8 * args.batch, "d2h_bytes_per_step": 8 * args.batch, "steps": e2e_steps},
        }
    except Exception as exc:  # the reference could not run here: say why in one line
        return {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:200] if str(exc) else ''}"}


def main() -> int:
    args = parse_args()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    if args.workload:
        if args.impl == "reference":
            line = {"impl": "reference", "workload": args.workload,
                    "unavailable": "the secondary workloads are measured for this library only (the reference has no generation benchmark)"}
        else:
            line = run_workload(args)
    else:
        line = run_reference(args) if args.impl == "reference" else run_b200(args)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
