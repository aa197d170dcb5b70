"""Bisodra models drawn at random from what config.json allows (widths, head counts and sizes off 8 and off 16 among
them, the order and number of layers, windows down to one position with and without kept first keys, convolutions of one
to eight taps, latents of many sizes with part of the rotated elements turning, stretched and plain rotations, readers of
another layer's latent, layers without a feed-forward), each run whole, token by token, in portions and as an unequal
batch in both types against the plain implementation."""
import random
import tempfile
from pathlib import Path

import pytest
import torch

import plain_bisodra as plain
from qwen_triton_b200 import Engine, StepEntry, config_from_dict, write_random_model
from qwen_triton_b200.weights import Checkpoint, write_safetensors
from test_gpu_vunepel import STORE, close

pytestmark = pytest.mark.gpu


def draw(seed: int) -> dict:
    rng = random.Random(7000 + seed)
    width = rng.choice([36, 40, 64, 72, 96, 100, 128, 200])
    layers, owners = [], []
    for index in range(rng.randint(1, 6)):
        mlp = None if rng.random() < 0.2 else {"kind": "dense", "ff": rng.choice([8, 20, 48, 100, 136, 256])}
        if rng.random() < 0.5:
            kv_heads = rng.choice([1, 2, 3])
            dim = rng.choice([4, 8, 12, 16, 20, 32, 40, 64, 72, 128])
            mixer = {"heads": kv_heads * rng.choice([1, 2, 4, 5]), "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                     "conv": rng.choice([1, 2, 3, 4, 4, 5, 8]), "scale": round(rng.uniform(0.05, 0.5), 3)}
            if rng.random() < 0.8:
                mixer["mask"] = {"size": rng.choice([1, 2, 7, 33, 64, 65, 100, 190]), "keep_first": rng.choice([0, 0, 1, 3, 20, 64, 70])}
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
            continue
        if owners and rng.random() < 0.4:                   # reads the latent of an earlier layer under its own matrices
            source = rng.choice(owners)
            first = layers[source]["mixer"]
            mixer = {"kv_rank": first["kv_rank"], "rot_dim": first["rot_dim"], "rot": first["rot"], "kv_from": source}
        else:
            rot_dim = rng.choice([2, 4, 8, 16, 24, 64])
            rot = {"dims": rng.choice([d for d in (2, 4, 8, rot_dim) if d <= rot_dim]), "base": rng.choice([100.0, 10000.0, 1000000.0])}
            if rng.random() < 0.6:
                rot["scaling"] = {"factor": rng.choice([2.0, 4.0, 40.0]), "original": rng.choice([32, 100, 1024]),
                                  "fast": rng.choice([32.0, 8.0]), "slow": rng.choice([1.0, 2.0])}
            mixer = {"kv_rank": rng.choice([4, 8, 24, 40, 64, 96, 136, 260]), "rot_dim": rot_dim, "rot": rot}
            owners.append(index)
        mixer.update(heads=rng.choice([1, 2, 3, 5, 8]), dim=rng.choice([4, 8, 16, 24, 40, 64]), vdim=rng.choice([4, 8, 20, 48, 64, 100]),
                     q_rank=rng.choice([4, 8, 24, 64, 100]), scale=round(rng.uniform(0.05, 0.5), 3))
        layers.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Bisodra", "vocab": rng.randint(30, 300), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])},
            "embedding": {"scale": rng.choice([1.0, 3.0, 11.5])}, "logit_scale": rng.choice([1.0, 2.0, 0.7]), "layers": layers}


@pytest.mark.parametrize("dtype", ("fp32", "bf16"))
@pytest.mark.parametrize("seed", range(12))
def test_a_model_drawn_at_random(seed, dtype):
    raw = draw(seed)
    config = config_from_dict(raw)
    with tempfile.TemporaryDirectory() as holder:
        folder = write_random_model(holder, config, seed=seed, dtype=STORE[dtype])
        checkpoint = Checkpoint(folder)
        tensors = {n: checkpoint.read(n) for n in checkpoint.names()}
        for n in list(tensors):                    # sharper attention than the draw gives
            if n.endswith((".mix.q", ".mix.k", ".mix.uq", ".mix.uk")):
                tensors[n] = (tensors[n].float() * 2.5).to(tensors[n].dtype)
        write_safetensors(Path(folder) / "model.safetensors", tensors)
        weights = {n: t.float() for n, t in tensors.items()}
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=2048, max_step_tokens=random.Random(seed).choice([96, 512, 4096]))
    generator = torch.Generator().manual_seed(seed)
    lengths = (200, 1, 70)
    requests = [torch.randint(0, config.vocab_size, (n + 8,), generator=generator).tolist() for n in lengths]
    wants = [plain.forward(raw, weights, r, torch.float64).float() for r in requests]
    what = f"seed {seed}: {raw}"
    # whole, then the same request with its last 40 tokens one by one, then in portions of 19
    slot = engine.new_sequence()
    close(engine.step([StepEntry(slot, requests[0], list(range(len(requests[0]))))]), wants[0], dtype, "whole, " + what, model_rows=True)
    engine.release(slot)
    slot = engine.new_sequence()
    head = len(requests[0]) - 40
    rows = [engine.step([StepEntry(slot, requests[0][:head], [head - 1])])]
    rows += [engine.step([StepEntry(slot, [t], [0])]) for t in requests[0][head:]]
    engine.release(slot)
    close(torch.cat(rows), wants[0][head - 1:], dtype, "token by token, " + what, model_rows=True)
    slot = engine.new_sequence()
    rows = []
    for begin in range(0, len(requests[0]), 19):
        piece = requests[0][begin:begin + 19]
        rows.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]))
    engine.release(slot)
    close(torch.cat(rows), wants[0], dtype, "in portions, " + what, model_rows=True)
    # an unequal batch, then eight tokens each
    slots = [engine.new_sequence() for _ in requests]
    rows = [[] for _ in requests]
    out = engine.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, requests, lengths)])
    for i in range(len(requests)):
        rows[i].append(out[i:i + 1])
    for t in range(8):
        out = engine.step([StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, requests, lengths)])
        for i in range(len(requests)):
            rows[i].append(out[i:i + 1])
    for i, n in enumerate(lengths):
        close(torch.cat(rows[i]), wants[i][n - 1:], dtype, f"batch row {i}, " + what, model_rows=True)
    for s in slots:
        engine.release(s)
    engine.cache.book.check()
    engine.check_kernels()
