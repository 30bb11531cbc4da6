"""Small Givirax configurations that differ from one another in every size and option, and a writer of their folders.

          width vocab layers (heads/kv/dim, window/keep, feed-forward)                                    passes
    gv_a    48    97   3/1/16 9/2 dense 40 | 3/1/16 9/2 routed 5 top 2 ff 24 | 3/1/16 9/2 none             layers 1..2 three times
    gv_b    80   131   4/4/24 33/0 routed 3 top 1 ff 16 | 2/1/40 20/5 dense 72 | 4/2/24 7/7 routed 2 top 2   none
    gv_c    96   150   6/2/64 70/3 dense 128 | 6/2/64 70/3 routed 4 top 4 ff 32                            layer 0 twice
    gv_d    50    61   5/5/10 1000/1 routed 6 top 3 ff 12 | 1/1/50 3/1 none                                 layers 0..1 once
Widths 50 and rows of 10 elements fit no vector width; gv_b's layers have three different cache shapes; gv_c has the head
size that tensor-core kernels take; in gv_d a window is wider than any sequence used and another is 3; scales, eps and the
embedding's factor all differ (one factor is 1)."""
import json
import os

import torch


def _attn(heads, kv, dim, size, keep, scale):
    return {"dim": dim, "heads": heads, "kv_heads": kv, "vdim": dim, "scale": scale, "mask": {"size": size, "keep_first": keep}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


GV_A = {"architecture": "Givirax", "vocab": 97, "width": 48, "max_positions": 160, "embedding": {"scale": 2.5},
        "norm": {"eps": 1e-5}, "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [_layer(_attn(3, 1, 16, 9, 2, 0.3), _dense(40)), _layer(_attn(3, 1, 16, 9, 2, 0.3), _moe(5, 2, 24)),
                   _layer(_attn(3, 1, 16, 9, 2, 0.3), None)]}
GV_B = {"architecture": "Givirax", "vocab": 131, "width": 80, "max_positions": 200, "embedding": {"scale": 1.0},
        "norm": {"eps": 1e-6},
        "layers": [_layer(_attn(4, 4, 24, 33, 0, 0.2), _moe(3, 1, 16)), _layer(_attn(2, 1, 40, 20, 5, 0.15), _dense(72)),
                   _layer(_attn(4, 2, 24, 7, 7, 0.25), _moe(2, 2, 16))]}
GV_C = {"architecture": "Givirax", "vocab": 150, "width": 96, "max_positions": 400, "embedding": {"scale": 9.0},
        "norm": {"eps": 1e-5}, "loop": {"start": 0, "stop": 1, "times": 2},
        "layers": [_layer(_attn(6, 2, 64, 70, 3, 0.125), _dense(128)), _layer(_attn(6, 2, 64, 70, 3, 0.125), _moe(4, 4, 32))]}
GV_D = {"architecture": "Givirax", "vocab": 61, "width": 50, "max_positions": 120, "embedding": {"scale": 0.7},
        "norm": {"eps": 1e-4}, "loop": {"start": 0, "stop": 2, "times": 1},
        "layers": [_layer(_attn(5, 5, 10, 1000, 1, 0.4), _moe(6, 3, 12)), _layer(_attn(1, 1, 50, 3, 1, 0.2), None)]}

# name -> (config, seed, page size)
SETUPS = {"gv_a": (GV_A, 11, 16), "gv_b": (GV_B, 12, 32), "gv_c": (GV_C, 13, 16), "gv_d": (GV_D, 14, 64)}


def write_model(path, cfg, seed, sharpen=4.0):
    """Random weights through the package's random-weights writer (tensor names and shapes come from the architecture),
    then made sharp: query weights are scaled up so that attention concentrates on few keys (a key read from a wrong
    page, a window one token off or a lost first token then moves the logits by far more than rounding), router rows
    are scaled so that experts are chosen with clear margins, and the per-pass vectors are made large."""
    from cppvllm_b200.weights.random_init import random_tensors
    from cppvllm_b200.weights.safetensors_io import save_safetensors
    os.makedirs(path, exist_ok=True)
    tensors = random_tensors(cfg, seed, std=0.08, norm_spread=0.3)
    for k in list(tensors):
        t = tensors[k].float()
        if k.endswith(".mix.q"):
            t = t * sharpen
        elif k.endswith(".router"):
            t = t * 3.0
        elif k.endswith(".router.b") or k == "loop.step":
            t = t * 5.0
        elif k in ("embed", "pos"):
            t = t * 4.0
        tensors[k] = t.to(torch.bfloat16)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(path, "model.safetensors"), tensors)
    return path


def write_all(base):
    return {name: write_model(os.path.join(base, name), cfg, seed) for name, (cfg, seed, _) in SETUPS.items()}


def page_size(name):
    return SETUPS[name][2]


def config(name):
    return SETUPS[name][0]


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
