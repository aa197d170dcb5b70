"""Regupel models drawn at random from what config.json allows (widths, head counts and sizes off 8 and off 16 among them,
values narrower and wider than keys, the order and number of layers, windows down to one position with and without kept
first keys, rotations of a part or the whole of a head with and without stretching, states of 4 to 200 key channels, decays
from 0 to 1, 1 to 9 experts with 1 to all of them chosen, with and without a shared expert, layers without a feed-forward,
layers that run another layer's tensors), each run whole, token by token, in portions and as an unequal batch in both
types against the plain implementation."""
import random
import tempfile
from pathlib import Path

import pytest
import torch

import plain_regupel as plain
from qwen_triton_b200 import Engine, StepEntry, config_from_dict, write_random_model
from qwen_triton_b200.weights import Checkpoint, write_safetensors
from test_gpu_vunepel import STORE, close as close_all

CLOSE_CALL = 0.15      # a router's gap, over the scale of its logits, below which bfloat16 may choose otherwise

pytestmark = pytest.mark.gpu


def draw_attention(rng, left: bool) -> dict:
    kv_heads = rng.choice([1, 2, 3])
    dim = rng.choice([4, 8, 12, 16, 20, 32, 40, 64, 72, 128])
    mixer = {"heads": kv_heads * rng.choice([1, 2, 4, 5]), "kv_heads": kv_heads, "dim": dim, "vdim": rng.choice([4, 8, 20, dim, dim, 48, 100]),
             "scale": round(rng.uniform(0.05, 0.5), 3)}
    if rng.random() < 0.8:
        mixer["mask"] = {"size": rng.choice([1, 2, 7, 33, 64, 65, 100, 190])}
        if left:
            mixer["mask"]["keep_first"] = rng.choice([0, 0, 1, 3, 20, 64, 70])
    if not left and rng.random() < 0.85:
        dims = rng.choice([d for d in (2, 4, 8, 16, dim) if d <= dim and d % 2 == 0])
        mixer["rot"] = {"dims": dims, "base": rng.choice([100.0, 10000.0, 300000.0])}
        if rng.random() < 0.6:
            low = rng.choice([1.0, 2.0])
            mixer["rot"]["scaling"] = {"factor": rng.choice([2.0, 6.0, 40.0]), "low": low, "high": low + rng.choice([1.0, 3.0]),
                                       "original": rng.choice([16, 100, 1024])}
    return mixer


def draw(seed: int) -> dict:
    rng = random.Random(9000 + seed)
    width = rng.choice([36, 40, 64, 72, 96, 100, 128, 200])
    layers, owners = [], []
    for index in range(rng.randint(1, 6)):
        if owners and rng.random() < 0.25:
            layers.append({**layers[rng.choice(owners)], "weights_of": None})
            layers[-1]["weights_of"] = next(i for i in owners if layers[i]["mixer"] is layers[-1]["mixer"])
            continue
        mlp = None
        if rng.random() > 0.2:
            experts = rng.choice([1, 2, 4, 7, 9])
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([8, 9, 20, 48, 100])}, "router": {"experts": experts, "top": rng.randint(1, min(experts, 3))}}
            if rng.random() < 0.6:
                mlp["shared"] = {"ff": rng.choice([7, 16, 40, 136])}
        if rng.random() < 0.5:
            layers.append({"type": "attention", "mixer": draw_attention(rng, False), "mlp": mlp})
        else:
            heads = rng.choice([1, 2, 3, 6])
            right = {"heads": heads, "dim": rng.choice([4, 10, 16, 64, 72, 128, 200]), "vdim": rng.choice([4, 8, 20, 32, 33, 64]),
                     "decay": [rng.choice([0.0, 1.0, 0.5, round(rng.uniform(0.8, 0.999), 4)]) for _ in range(heads)]}
            layers.append({"type": "parallel", "mlp": mlp,
                           "mixer": {"left": draw_attention(rng, True), "right": right, "left_scale": rng.choice([1.0, 0.7, 0.35]),
                                     "right_scale": rng.choice([1.0, 1.2, 2.0])}})
        owners.append(index)
    return {"architecture": "Regupel", "vocab": rng.randint(30, 300), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])},
            "embedding": {"scale": rng.choice([1.0, 2.5, 11.5])}, "logit_scale": rng.choice([1.0, 1.5, 0.7]),
            "residual_mult": rng.choice([1.0, 0.25, 0.5]), "layers": layers}


@pytest.mark.parametrize("dtype", ("fp32", "bf16"))
@pytest.mark.parametrize("seed", range(12))
def test_a_model_drawn_at_random(seed, dtype):
    raw = draw(seed)
    config = config_from_dict(raw)
    raw = config.to_hf_dict()
    with tempfile.TemporaryDirectory() as holder:
        folder = write_random_model(holder, config, seed=seed, dtype=STORE[dtype])
        checkpoint = Checkpoint(folder)
        tensors = {n: checkpoint.read(n) for n in checkpoint.names()}
        for n in list(tensors):                    # sharper attention than the draw gives
            if n.endswith((".q.norm", ".k.norm")):
                tensors[n] = (tensors[n].float() * 2.5).to(tensors[n].dtype)
        write_safetensors(Path(folder) / "model.safetensors", tensors)
        weights = {n: t.float() for n, t in tensors.items()}
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=2048, max_step_tokens=random.Random(seed).choice([96, 512, 4096]))
    generator = torch.Generator().manual_seed(seed)
    lengths = (200, 1, 70)
    requests = [torch.randint(0, config.vocab_size, (n + 8,), generator=generator).tolist() for n in lengths]
    wants, clear = [], []
    for r in requests:
        margins = []
        wants.append(plain.forward(raw, weights, r, margins=margins).float())
        clear.append(torch.stack(margins).min(dim=0).values >= CLOSE_CALL if margins and dtype == "bf16" else torch.ones(len(r), dtype=torch.bool))
    what = f"seed {seed}: {raw}"

    def close(actual, request, rows, text):
        """Positions at which a router's choice is nearly a tie in the plain implementation may fall the other way in
        bfloat16; they are only asked to be finite (float32 holds every position)."""
        actual = actual.float().cpu()
        assert bool(torch.isfinite(actual).all()), text
        keep = clear[request][rows]
        if bool(keep.any()):
            close_all(actual[keep], wants[request][rows][keep], dtype, text, model_rows=True)

    # whole, then the same request with its last 40 tokens one by one, then in portions of 19
    slot = engine.new_sequence()
    close(engine.step([StepEntry(slot, requests[0], list(range(len(requests[0]))))]), 0, slice(None), "whole, " + what)
    engine.release(slot)
    slot = engine.new_sequence()
    head = len(requests[0]) - 40
    rows = [engine.step([StepEntry(slot, requests[0][:head], [head - 1])])]
    rows += [engine.step([StepEntry(slot, [t], [0])]) for t in requests[0][head:]]
    engine.release(slot)
    close(torch.cat(rows), 0, slice(head - 1, None), "token by token, " + what)
    slot = engine.new_sequence()
    rows = []
    for begin in range(0, len(requests[0]), 19):
        piece = requests[0][begin:begin + 19]
        rows.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]))
    engine.release(slot)
    close(torch.cat(rows), 0, slice(None), "in portions, " + what)
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
        close(torch.cat(rows[i]), i, slice(n - 1, None), f"batch row {i}, " + what)
    for s in slots:
        engine.release(s)
    engine.cache.book.check()
    engine.check_kernels()
