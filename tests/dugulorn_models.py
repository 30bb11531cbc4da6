"""Small Dugulorn configurations that differ from one another in every size and option, and a writer of their folders.

    dg_a  width 48, vocab 97:  latent 3 heads 16+8/12, ranks 24/16, stretched rotation, ff 40 | lightning 2 x 10 x 7 |
                               latent reading layer 0's cache, ff 56 | delta 4 heads over 2, 12 x 20, 3 taps, ff 40
    dg_b  width 64, vocab 131: delta 2 heads over 1, 64 x 40, 4 taps | latent 4 heads 32+16/32, ranks 48/48, only 8 of the 16
                               positional elements turn, no stretching, ff 96 | lightning 2 x 64 x 64, ff 72 | latent reading layer 1
    dg_c  width 96, vocab 150: latent 20 heads 8+32/8, ranks 16/32, ff 64 | delta 3 heads, 40 x 33, 1 tap | lightning 2 x 130 x 5,
                               decays 1 and 0.5 | delta 2 heads over 2, 16 x 64, 2 taps
    dg_d  width 50, vocab 61:  lightning 1 x 33 x 50 alone
Widths 50 and odd head sizes fit no vector width; dg_b's latent entries (48 + 16 = 64, value 48) and dg_c's (32 + 32, value 32)
take the tensor-core attention kernel in bf16, dg_c with 20 heads in two groups when it decodes; dg_a's entries (16 + 8) take
the general kernel; ranks of the delta mixers' low-rank projections, eps, scales and decays all differ (one decay is 1)."""
import json
import os

import torch


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


_ROT_A = _rot(8, 100.0, (3.0, 40, 8.0, 1.0))
_ROT_B = _rot(8, 10000.0)
_ROT_C = _rot(32, 5000.0, (8.0, 64, 16.0, 2.0))

DG_A = {"architecture": "Dugulorn", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "layers": [
    _layer("latent_attention", _latent(3, 16, 8, 12, 24, 16, 0.3, _ROT_A), 40),
    _layer("lightning", {"heads": 2, "dim": 10, "vdim": 7, "decay": [0.9, 0.995]}),
    _layer("latent_attention", _latent(3, 16, 8, 12, 24, 16, 0.3, _ROT_A, kv_from=0), 56),
    _layer("channel_delta", {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "conv": 3, "a_rank": 6, "g_rank": 10}, 40)]}
DG_B = {"architecture": "Dugulorn", "vocab": 131, "width": 64, "norm": {"eps": 1e-6}, "layers": [
    _layer("channel_delta", {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 40, "conv": 4, "a_rank": 8, "g_rank": 8}),
    _layer("latent_attention", _latent(4, 32, 16, 32, 48, 48, 0.2, _ROT_B), 96),
    _layer("lightning", {"heads": 2, "dim": 64, "vdim": 64, "decay": [0.97, 0.8]}, 72),
    _layer("latent_attention", _latent(4, 32, 16, 32, 48, 48, 0.2, _ROT_B, kv_from=1))]}
DG_C = {"architecture": "Dugulorn", "vocab": 150, "width": 96, "norm": {"eps": 1e-4}, "layers": [
    _layer("latent_attention", _latent(20, 8, 32, 8, 16, 32, 0.25, _ROT_C), 64),
    _layer("channel_delta", {"heads": 3, "kv_heads": 3, "dim": 40, "vdim": 33, "conv": 1, "a_rank": 5, "g_rank": 3}),
    _layer("lightning", {"heads": 2, "dim": 130, "vdim": 5, "decay": [1.0, 0.5]}),
    _layer("channel_delta", {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 64, "conv": 2, "a_rank": 16, "g_rank": 4})]}
DG_D = {"architecture": "Dugulorn", "vocab": 61, "width": 50, "norm": {"eps": 1e-5}, "layers": [
    _layer("lightning", {"heads": 1, "dim": 33, "vdim": 50, "decay": [0.99]})]}

# name -> (config, seed, page size)
SETUPS = {"dg_a": (DG_A, 21, 16), "dg_b": (DG_B, 22, 32), "dg_c": (DG_C, 23, 16), "dg_d": (DG_D, 24, 64)}


def write_model(path, cfg, seed, sharpen=4.0):
    """Random weights through the package's random-weights writer (tensor names and shapes come from the architecture),
    then made telling: query up-projections are scaled up so that attention concentrates on few keys (a key read from a
    wrong page or a lost first token then moves the logits by far more than rounding); the delta mixers' decay rates are
    pushed down so that their matrices remember hundreds of tokens (a state that is lost or zeroed at a cut shows); biases,
    convolution taps and norm weights are made large enough to matter."""
    from cppvllm_b200.weights.random_init import random_tensors
    from cppvllm_b200.weights.safetensors_io import save_safetensors
    os.makedirs(path, exist_ok=True)
    tensors = random_tensors(cfg, seed, std=0.08, norm_spread=0.3)
    for k in list(tensors):
        t = tensors[k].float()
        if k.endswith(".mix.uq"):
            t = t * sharpen
        elif k.endswith(".A_log"):
            t = t * 5.0 - 3.0
        elif k.endswith(".conv") or k.endswith(".b") and ".mlp." in k or k.endswith("dt_bias"):
            t = t * 6.0
        elif k.endswith("norm1") or k.endswith("norm2") or k in ("embed.norm", "final.norm"):
            t = t * 3.0
        elif k.endswith(".mix.a2") or k.endswith(".mix.g2") or k.endswith(".mix.b") or k.endswith(".mix.g"):
            t = t * 4.0
        tensors[k] = t.to(torch.bfloat16)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(path, "model.safetensors"), tensors)
    return path


def random_config(seed):
    """A configuration drawn at random: 2 to 6 layers of any kind in any order, with or without feed-forwards, latent layers
    that read an earlier one's cache now and then, sizes that are odd, prime, 1 or large, every option on or off."""
    import random
    rng = random.Random(seed)
    width, layers, writers = rng.choice([32, 40, 64, 72, 96, 128, 50]), [], []
    for i in range(rng.randrange(2, 7)):
        kind = rng.choice(["latent_attention", "lightning", "channel_delta"])
        ff = rng.choice([None, rng.randrange(8, 200)])
        if kind == "latent_attention":
            if writers and rng.random() < 0.4:
                j = rng.choice(writers)
                m = dict(layers[j]["mixer"], kv_from=j, heads=rng.choice([1, 2, 3, 5, 8, 17]), dim=rng.choice([4, 8, 16, 24, 32]),
                         vdim=rng.choice([4, 8, 12, 32, 40]), q_rank=rng.randrange(4, 64), scale=rng.uniform(0.05, 0.4))
            else:
                rot_dim = rng.choice([2, 4, 8, 16, 32, 6])
                scaling = (rng.choice([2.0, 4.0, 1.0, 16.0]), rng.choice([16, 64, 1000]), rng.choice([32.0, 8.0, 4.0]), rng.choice([1.0, 2.0, 0.5]))
                rot = _rot(rng.choice(range(2, rot_dim + 1, 2)), rng.choice([100.0, 10000.0, 37.5]), scaling if rng.random() < 0.6 else None)
                m = _latent(rng.choice([1, 2, 3, 4, 8, 20]), rng.choice([4, 8, 16, 32, 64, 10]), rot_dim, rng.choice([4, 8, 16, 32, 64, 9]),
                            rng.randrange(4, 96), rng.choice([8, 16, 32, 48, 64, 96, 20, 7]), rng.uniform(0.05, 0.4), rot)
                writers.append(i)
        elif kind == "lightning":
            H = rng.choice([1, 2, 3, 6])
            m = {"heads": H, "dim": rng.choice([4, 16, 33, 64, 100, 200]), "vdim": rng.choice([3, 16, 32, 40, 70]),
                 "decay": [rng.choice([1.0, 0.999, 0.9, 0.6, rng.uniform(0.3, 1.0)]) for _ in range(H)]}
        else:
            G = rng.choice([1, 2, 3])
            m = {"heads": G * rng.choice([1, 2, 3]), "kv_heads": G, "dim": rng.choice([4, 16, 32, 48, 64, 130]), "vdim": rng.choice([4, 16, 32, 64, 33]),
                 "conv": rng.choice([1, 2, 3, 4, 5]), "a_rank": rng.randrange(2, 30), "g_rank": rng.randrange(2, 30)}
        layers.append(_layer(kind, m, ff))
    return {"architecture": "Dugulorn", "vocab": rng.randrange(40, 300), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6, 1e-3])},
            "layers": layers}


def write_all(base):
    return {name: write_model(os.path.join(base, name), cfg, seed) for name, (cfg, seed, _) in SETUPS.items()}


def page_size(name):
    return SETUPS[name][2]


def config(name):
    return SETUPS[name][0]


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
