"""Plain, slow implementation of the Dugulorn decoder: whole sequences, no cache, no batching, one function per
mechanism, float64 on the CPU.  It shares no code with the package under test: its own config.json reading, its own
safetensors reading and its own arithmetic.  In this file's notation (rms_e(x) = sqrt(mean(x^2) + e), n(x; w) =
x / rms_e(x) * w, sg = logistic function):

    x_0       = n(E[token]; 1 + w_embed)
    layer     : x <- x + n(mix(x); 1 + w_1);  with a feed-forward also  x <- x + n(ff(x); 1 + w_2)   (norms behind the sublayers)
    ff        : Wd relu(Wu x + bu)^2 + bd
    latent    : cq = n(Wdq x; w_dq);  q = Wuq cq, per head [nope | rope];  [c_raw | kr_raw] = Wdkv x;  c = n(c_raw; w_dkv);
                kr = R_p(kr_raw), one for all heads;  k_h = Wuk_h c, v_h = Wuv_h c;
                s_ij = scale (q_nope_i . k_j + R_i(q_rope_i) . kr_j), j <= i;  softmax;  y = Wo concat_h(sg(Wg x)_h * sum_j a_ij v_j).
                A layer with kv_from = j reads layer j's (c, kr).
    rotation  : pairs (2i, 2i+1) of the first `dims` elements turn by p * f_i; the frequencies are blended between f_i and
                f_i / factor by a ramp over the pair index, and cos and sin are multiplied by 0.1 ln(factor) + 1
    lightning : q = silu(Wq x), k = silu(Wk x), v = silu(Wv x);  S <- d_h S + k v^T;  o = S^T q;
                y = Wo (n(concat_h o; w) * sg(Wg x))
    delta     : q, k, v = silu(conv(W. x)) (causal, per channel);  q, k <- unit vectors per head (q also / sqrt(dim));
                b = sg(Wb x);  g = exp(-exp(A_h) softplus(Wa2 Wa1 x + dt));  S <- diag(g) S;  u = b (v - S^T k);
                S <- S + k u^T;  o = S^T q;  y = Wo concat_h(n(o_h; w) * sg(Wg2 Wg1 x)_h)
    logits    = E n(x; 1 + w_final)

`rnd` (default: the identity) is applied where an engine with 16-bit activations rounds: operands and results of matrix
products; with it the file predicts the size of that engine's rounding error.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F = torch.float64


def identity(x):
    return x


def to_bf16(x):
    return x.to(torch.float32).to(torch.bfloat16).to(F)


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
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: element type {meta['dtype']}")
        t = t.reshape(meta["shape"])
        out[name] = t.to(F) if t.dtype.is_floating_point else t
    return out


# ---- norms -------------------------------------------------------------------------------------------------------

def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


def norm_around_zero(x, w, eps):
    """The weight is stored as its distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def logistic(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * logistic(x)


# ---- rotation ----------------------------------------------------------------------------------------------------

def rotation_frequencies(rot: dict):
    """Per pair frequency and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F), 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, ..., n]: the first rot.dims elements of the last axis turn, pairs (2i, 2i+1); the others pass."""
    freq, mag = rotation_frequencies(rot)
    dims = int(rot["dims"])
    ang = positions.to(F)[:, None] * freq[None, :]                       # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = (torch.cos(ang) * mag).reshape(shape), (torch.sin(ang) * mag).reshape(shape)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---- mixers ------------------------------------------------------------------------------------------------------

def latent_keys(x, w, p, m, eps, positions, rnd=identity):
    """What a latent-attention layer leaves for its own and for later layers' use: (c [T, rank], kr [T, rot_dim])."""
    R = int(m["kv_rank"])
    kv = rnd(rnd(x) @ w[p + "dkv"].T)
    c = rnd(norm_plain(kv[:, :R], w[p + "dkv.norm"], eps))
    kr = rnd(rotate(kv[:, R:], positions, m["rot"]))
    return c, kr


def causal_attention(q_nope, q_rope, k, kr, v, scale):
    """q_nope, k [T, H, dn]; q_rope [T, H, dr]; kr [T, dr] (one for all heads); v [T, H, dv].  Token i sees every j <= i;
    ordinary softmax.  Returns [T, H, dv]."""
    T, H = q_nope.shape[0], q_nope.shape[1]
    visible = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for h in range(H):
        s = (q_nope[:, h] @ k[:, h].T + q_rope[:, h] @ kr.T) * scale
        s = s.masked_fill(~visible, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, h]
    return out


def latent_attention(x, w, p, m, eps, positions, keys, rnd=identity):
    T = x.shape[0]
    H, dn, dr, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    c, kr = keys
    xr = rnd(x)
    cq = rnd(norm_plain(rnd(xr @ w[p + "dq"].T), w[p + "dq.norm"], eps))
    q = rnd(cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_nope, q_rope = q[..., :dn], rotate(q[..., dn:], positions, m["rot"])
    k = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    gate = logistic(rnd(xr @ w[p + "g"].T))                               # [T, H]
    out = causal_attention(q_nope, q_rope, k, kr, v, float(m["scale"])) * gate[:, :, None]
    return rnd(rnd(out.reshape(T, H * dv)) @ w[p + "o"].T)


def lightning_rule(q, k, v, decays):
    """q, k [T, H, dk], v [T, H, dv]: per head S <- d S + k v^T, o = S^T q, from S = 0.  Returns o [T, H, dv]."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    o = torch.zeros(T, H, dv, dtype=F)
    for h in range(H):
        S = torch.zeros(dk, dv, dtype=F)
        for t in range(T):
            S = float(decays[h]) * S + torch.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ q[t, h]
    return o


def lightning(x, w, p, m, eps, rnd=identity):
    T = x.shape[0]
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    xr = rnd(x)
    q = silu(rnd(xr @ w[p + "q"].T)).reshape(T, H, dk)
    k = silu(rnd(xr @ w[p + "k"].T)).reshape(T, H, dk)
    v = silu(rnd(xr @ w[p + "v"].T)).reshape(T, H, dv)
    o = lightning_rule(q, k, v, m["decay"])
    y = norm_plain(o.reshape(T, H * dv), w[p + "norm"], eps) * logistic(rnd(xr @ w[p + "g"].T))
    return rnd(rnd(y) @ w[p + "o"].T)


def causal_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K]; the last column multiplies the current token, zeros stand before the start."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=F), u], dim=0)
    out = torch.zeros(T, C, dtype=F)
    for j in range(K):
        out += padded[j:j + T] * taps[:, j][None, :]
    return out


def unit_vectors(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def softplus(a):
    return torch.where(a > 30, a, torch.log1p(torch.exp(torch.clamp(a, max=30.0))))


def delta_rule(q, k, v, g, beta):
    """q, k [T, G, dk], v [T, H, dv], g [T, H, dk], beta [T, H]: per head (reading q/k head h // (H / G)), from S = 0:
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.  Returns o [T, H, dv]."""
    T, G, dk = q.shape
    H, dv = v.shape[1], v.shape[2]
    o = torch.zeros(T, H, dv, dtype=F)
    for h in range(H):
        kv = h // (H // G)
        S = torch.zeros(dk, dv, dtype=F)
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            o[t, h] = S.T @ q[t, kv]
    return o


def channel_delta(x, w, p, m, eps, rnd=identity):
    T = x.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    xr = rnd(x)
    q = silu(causal_conv(rnd(xr @ w[p + "q"].T), w[p + "q.conv"])).reshape(T, G, dk)
    k = silu(causal_conv(rnd(xr @ w[p + "k"].T), w[p + "k.conv"])).reshape(T, G, dk)
    v = silu(causal_conv(rnd(xr @ w[p + "v"].T), w[p + "v.conv"])).reshape(T, H, dv)
    q = unit_vectors(q) * dk ** -0.5
    k = unit_vectors(k)
    beta = logistic(xr @ w[p + "b"].T)                                    # [T, H]
    a = rnd(rnd(xr @ w[p + "a1"].T)) @ w[p + "a2"].T + w[p + "dt_bias"]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, dk))      # [T, H, dk]
    o = delta_rule(q, k, v, g, beta)
    gate = logistic(rnd(rnd(rnd(xr @ w[p + "g1"].T)) @ w[p + "g2"].T)).reshape(T, H, dv)
    y = norm_plain(o, w[p + "norm"], eps) * gate
    return rnd(rnd(y.reshape(T, H * dv)) @ w[p + "o"].T)


def feed_forward(x, w, p, rnd=identity):
    a = torch.relu(rnd(rnd(x) @ w[p + "up"].T) + w[p + "up.b"]) ** 2
    return rnd(rnd(a) @ w[p + "down"].T) + w[p + "down.b"]


# ---- the model -----------------------------------------------------------------------------------------------------

def forward(model_dir: str, tokens, rounding: str = "none", return_layers: bool = False, weights=None, config=None):
    """Logits [T, vocab] of one sequence (float64); with return_layers also the stream after every layer [L, T, width]."""
    cfg = config if config is not None else read_config(model_dir)
    w = weights if weights is not None else read_weights(model_dir)
    rnd = to_bf16 if rounding == "bfloat16" else identity
    eps = float(cfg["norm"]["eps"])
    tok = torch.tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = norm_around_zero(w["embed"][tok], w["embed.norm"], eps)
    kept, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.mix.", layer["mixer"], layer["type"]
        if kind == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_keys(x, w, p, m, eps, positions, rnd)
                src = i
            y = latent_attention(x, w, p, m, eps, positions, kept[int(src)], rnd)
        elif kind == "lightning":
            y = lightning(x, w, p, m, eps, rnd)
        elif kind == "channel_delta":
            y = channel_delta(x, w, p, m, eps, rnd)
        else:
            raise ValueError(f"layer {i}: mixer '{kind}'")
        x = x + norm_around_zero(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"layer {i}: feed-forward '{layer['mlp']['kind']}'")
            x = x + norm_around_zero(feed_forward(x, w, f"l{i}.mlp.", rnd), w[f"l{i}.norm2"], eps)
        streams.append(x.clone())
    logits = rnd(norm_around_zero(x, w["final.norm"], eps)) @ w["embed"].T
    return (logits, torch.stack(streams)) if return_layers else logits


def greedy_generate(model_dir: str, prompt, n: int):
    cfg, w = read_config(model_dir), read_weights(model_dir)
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(forward(model_dir, toks, weights=w, config=cfg)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
