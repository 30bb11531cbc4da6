"""Plain, slow implementation of the Givirax decoder: whole sequences, no cache, no batching, one function per
mechanism, float64 on the CPU.  It shares no code with the package under test: its own config.json reading, its own
safetensors reading and its own arithmetic, written from the design's equations:

    x_0      = E[token] * s + P[position]
    layer    : n = x / sqrt(mean(x^2) + eps) * w;   x <- x + (mix(n) + ff(n))          (one norm, both sublayers read it)
    mix      : q = Wq n, k = Wk n, v = k;  head h reads kv head floor(h / (H / G));  a_ij = c * q_i . k_j over the j with
               j <= i and (i - j < window or j < keep_first);  softmax over those;  y = Wo concat_h(sum_j a_ij k_j)
    ff dense : Wd gelu_tanh(Wu n)
    ff routed: z = Wr n + b;  C = top-k of z;  w_e = exp(z_e) / sum_{c in C} exp(z_c);
               y = sum_k weight_k * Wd_e (silu(Wg_e n) * (Wu_e n))
    passes   : layers start..stop-1 run `times` times; before pass t: x <- x + x_0 (t > 0), then x <- x + step[t]
    logits   = H (x / sqrt(mean(x^2) + eps) * w_final)
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F = torch.float64


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_weights(model_dir: str) -> dict:
    """Own reader of the container: 8 bytes of header length, a JSON header, raw little-endian data."""
    out = {}
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        raw = data[meta["data_offsets"][0]:meta["data_offsets"][1]]
        if meta["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
        else:
            raise ValueError(f"{name}: element type {meta['dtype']}")
        out[name] = t.reshape(meta["shape"]).to(F)
    return out


def embed(w: dict, cfg: dict, tokens) -> torch.Tensor:
    tok = torch.tensor(list(tokens), dtype=torch.long)
    scale = (cfg.get("embedding") or {}).get("scale", 1.0)
    return w["embed"][tok] * scale + w["pos"][: len(tokens)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def visible(n: int, window: int, keep_first: int) -> torch.Tensor:
    """[n, n] mask: row i sees column j."""
    out = torch.zeros(n, n, dtype=torch.bool)
    for i in range(n):
        for j in range(i + 1):
            out[i, j] = (window <= 0) or (i - j < window) or (j < keep_first)
    return out


def attention(n: torch.Tensor, wq, wk, wo, heads: int, kv_heads: int, dim: int, scale: float, window: int, keep_first: int):
    T = n.shape[0]
    q = (n @ wq.T).view(T, heads, dim)
    k = (n @ wk.T).view(T, kv_heads, dim)
    mask = visible(T, window, keep_first)
    outs = []
    for h in range(heads):
        g = h // (heads // kv_heads)
        rows = []
        for i in range(T):
            js = [j for j in range(T) if mask[i, j]]
            s = torch.stack([(q[i, h] * k[j, g]).sum() * scale for j in js])
            p = torch.exp(s - s.max())
            p = p / p.sum()
            rows.append(sum(p[a] * k[j, g] for a, j in enumerate(js)))
        outs.append(torch.stack(rows))
    return torch.cat(outs, dim=-1) @ wo.T


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_ff(n, w_up, w_down):
    return gelu_tanh(n @ w_up.T) @ w_down.T


def route(n, w_router, b_router, top: int):
    """Per token: (chosen experts, their weights)."""
    z = n @ w_router.T + b_router
    chosen, weights = [], []
    for t in range(n.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-float(z[t, e]), e))[:top]
        zt = torch.stack([z[t, e] for e in order])
        p = torch.exp(zt - zt.max())
        chosen.append(order)
        weights.append(p / p.sum())
    return chosen, weights


def routed_ff(n, w: dict, prefix: str, experts: int, top: int):
    chosen, weights = route(n, w[prefix + "router"], w[prefix + "router.b"], top)
    out = torch.zeros_like(n)
    for t in range(n.shape[0]):
        for e, p in zip(chosen[t], weights[t]):
            g = w[f"{prefix}e{e}.gate"] @ n[t]
            u = w[f"{prefix}e{e}.up"] @ n[t]
            out[t] += p * (w[f"{prefix}e{e}.down"] @ (g * torch.sigmoid(g) * u))
    return out


def layer(x, w: dict, cfg: dict, i: int):
    L = cfg["layers"][i]
    m = L["mixer"]
    mask = m.get("mask") or {}
    n = rms_norm(x, w[f"l{i}.norm1"], cfg["norm"]["eps"])
    y = attention(n, w[f"l{i}.mix.q"], w[f"l{i}.mix.k"], w[f"l{i}.mix.o"], m["heads"], m.get("kv_heads", m["heads"]), m["dim"],
                  m["scale"], mask.get("size", 0), mask.get("keep_first", 0))
    f = L.get("mlp")
    if f is not None and f["kind"] == "dense":
        y = y + dense_ff(n, w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"])
    elif f is not None:
        y = y + routed_ff(n, w, f"l{i}.mlp.", f["router"]["experts"], f["router"]["top"])
    return x + y


def hidden_states(model_dir: str, tokens, w=None, cfg=None):
    """The residual stream after every layer run, as a list, and the final one."""
    cfg = cfg or read_config(model_dir)
    w = w or read_weights(model_dir)
    x = embed(w, cfg, tokens)
    x0 = x.clone()
    runs = []
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    for i in range(loop["start"]):
        x = layer(x, w, cfg, i)
        runs.append(x)
    if loop["stop"] > loop["start"]:
        for t in range(loop["times"]):
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
            for i in range(loop["start"], loop["stop"]):
                x = layer(x, w, cfg, i)
                runs.append(x)
    for i in range(loop["stop"], len(cfg["layers"])):
        x = layer(x, w, cfg, i)
        runs.append(x)
    return runs, x


def forward(model_dir: str, tokens, w=None, cfg=None) -> torch.Tensor:
    """Logits [len(tokens), vocab] in float64."""
    cfg = cfg or read_config(model_dir)
    w = w or read_weights(model_dir)
    _, x = hidden_states(model_dir, tokens, w, cfg)
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def greedy_generate(model_dir: str, prompt, n: int):
    cfg, w = read_config(model_dir), read_weights(model_dir)
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(model_dir, seq, w, cfg)[-1].argmax()))
    return seq[len(prompt):]
