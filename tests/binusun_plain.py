"""Plain, slow restatement of the Binusun decoder in float64 numpy: one function per mechanism, whole sequences at once,
no cache, no batching.  It shares no code with the product path and is what the GPU engine is compared with.

Notation: T tokens, D width, H query heads, G key/value heads, d per-head query/key size, dv value size."""
from __future__ import annotations

import math

import numpy as np


def scalar_rms_norm(x, gain, eps):
    """y = x / sqrt(mean(x^2) + eps) * gain, one gain for every coordinate."""
    x = np.asarray(x, np.float64)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * float(gain)


def unit_rms(x, eps):
    x = np.asarray(x, np.float64)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims); with `scaling` the long wavelengths are slowed down by `factor`, short ones kept, and the band
    between original/high and original/low is blended linearly in original/wavelength."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], np.float64)
    if scaling:
        fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = f.copy()
        for i, fi in enumerate(f):
            wl = 2.0 * math.pi / fi
            if wl < orig / hi:
                out[i] = fi
            elif wl > orig / lo:
                out[i] = fi / fac
            else:
                s = (orig / wl - lo) / (hi - lo)
                out[i] = (1.0 - s) * fi / fac + s * fi
        f = out
    return f


def rotate_interleaved(x, pos, freqs):
    """x [T, heads, d]; coordinates (2i, 2i+1) of the first 2*len(freqs) are rotated by pos * f_i, the rest pass."""
    x = np.array(x, np.float64)
    n = len(freqs)
    ang = np.asarray(pos, np.float64)[:, None] * freqs[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., 0:2 * n:2].copy(), x[..., 1:2 * n:2].copy()
    x[..., 0:2 * n:2] = a * c - b * s
    x[..., 1:2 * n:2] = b * c + a * s
    return x


def windowed_attention(h, W, mc, eps, pos0=0):
    """Grouped-query softmax attention over the last `mask.size` positions (the current one included), rotary q/k that are
    then brought to unit RMS per head, and a sigmoid gate per head on the output."""
    T = h.shape[0]
    H, G, d = mc["heads"], mc["kv_heads"], mc["dim"]
    dv = mc["vdim"]
    q = (h @ W["q"].T).reshape(T, H, d)
    k = (h @ W["k"].T).reshape(T, G, d)
    v = (h @ W["v"].T).reshape(T, G, dv)
    rot = mc.get("rot")
    pos = np.arange(pos0, pos0 + T)
    if rot:
        fr = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_interleaved(q, pos, fr), rotate_interleaved(k, pos, fr)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    gate = 1.0 / (1.0 + np.exp(-(h @ W["g"].T)))          # [T, H]
    win = mc["mask"]["size"]
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        sc = (q[:, hd] @ k[:, g].T) * mc["scale"]
        i, j = np.arange(T)[:, None], np.arange(T)[None, :]
        vis = (i - j >= 0) & (i - j < win)
        sc = np.where(vis, sc, -np.inf)
        sc = sc - sc.max(-1, keepdims=True)
        p = np.exp(sc)
        p /= p.sum(-1, keepdims=True)
        out[:, hd] = (p @ v[:, g]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * dv) @ W["o"].T


def wkv_mixer(h, W, mc, eps):
    """Token-shifted linear recurrence: per head a [d, d] state S; o_t = (S + diag(u) k_t v_t^T)^T r_t,
    then S <- diag(w_t) S + k_t v_t^T with a data-dependent decay w_t in (0, 1)."""
    T, D = h.shape
    H, d = mc["heads"], mc["dim"]
    prev = np.vstack([np.zeros((1, D)), h[:-1]])
    mix = {s: h + (prev - h) * W["mu." + s][None, :] for s in "rkvgw"}
    r = (mix["r"] @ W["r"].T).reshape(T, H, d)
    k = (mix["k"] @ W["k"].T).reshape(T, H, d)
    v = (mix["v"] @ W["v"].T).reshape(T, H, d)
    gz = mix["g"] @ W["g"].T
    gate = gz / (1.0 + np.exp(-gz))
    dec = np.exp(-np.exp(np.tanh(mix["w"] @ W["w1"].T) @ W["w2"].T + W["w0"][None, :])).reshape(T, H, d)
    u = W["u"].reshape(H, d)
    S = np.zeros((H, d, d))
    o = np.zeros((T, H, d))
    for t in range(T):
        for hd in range(H):
            kv = np.outer(k[t, hd], v[t, hd])
            o[t, hd] = (S[hd] + u[hd][:, None] * kv).T @ r[t, hd]
            S[hd] = dec[t, hd][:, None] * S[hd] + kv
    o = unit_rms(o, eps).reshape(T, H * d) * W["norm"][None, :] * gate
    return o @ W["o"].T


def dense_ff(h, W, act="relu"):
    z = h @ W["gate"].T
    a = np.maximum(z, 0.0) if act == "relu" else z
    return (a * (h @ W["up"].T)) @ W["down"].T


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer_runs(cfg):
    """The order in which layers run: a block [start, stop) repeated `times` times; each entry is (layer, first of a pass)."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(lp["start"])]
    for _ in range(lp["times"]):
        runs += [(i, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    runs += [(i, False) for i in range(lp["stop"], n)]
    return runs


def forward(cfg, weights, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (weights: name -> float array)."""
    W = {k: np.asarray(v, np.float64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][np.asarray(tokens)]
    x = x0.copy()
    trace = []
    for li, first in layer_runs(cfg):
        L = cfg["layers"][li]
        p = "l%d." % li
        if first:
            x = np.concatenate([x, x0], -1) @ W["loop.in"].T
        h = scalar_rms_norm(x, W[p + "norm1"], eps)
        mw = sub(W, p + "mix.")
        m = windowed_attention(h, mw, L["mixer"], eps) if L["type"] == "attention" else wkv_mixer(h, mw, L["mixer"], eps)
        x = x + scalar_rms_norm(m, W[p + "norm1b"], eps)
        if L.get("mlp"):
            h = scalar_rms_norm(x, W[p + "norm2"], eps)
            x = x + scalar_rms_norm(dense_ff(h, sub(W, p + "mlp.")), W[p + "norm2b"], eps)
        trace.append(x.copy())
    logits = (scalar_rms_norm(x, W["final.norm"], eps) @ W["head"].T) * cfg["logit_scale"]
    return (logits, np.stack(trace)) if return_layers else logits
