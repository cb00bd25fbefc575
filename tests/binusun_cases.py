"""Small Binusun configurations with random weights for the tests, and helpers that run them through the engine.

Weights are rounded to bfloat16-representable values, so the bf16 and the fp32 engine and the plain implementation all see
exactly the same numbers."""
from __future__ import annotations

import math

import numpy as np


def attn_layer(heads=4, kv_heads=2, dim=32, vdim=32, window=16, rot_dims=16, base=10000.0, scaling=None, scale=None, ff=0):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
          "rot": {"base": base, "dims": rot_dims}, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if scaling:
        mx["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": mx, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def wkv_layer(heads=2, dim=16, ff=0, rank=4):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": {"kind": "dense", "ff": ff} if ff else None, "_rank": rank}


def make_config(layers, vocab=97, width=48, loop=None, eps=1e-5, logit_scale=0.5):
    cfg = {"architecture": "Binusun", "layers": layers, "logit_scale": logit_scale, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def to_bf16_values(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def random_weights(cfg, seed=0, decay_bias=-1.0, gain=1.0):
    """Weights of a size that keeps activations O(1); decay_bias shifts the recurrence's decay offset (very negative: a decay
    close to 1, i.e. a long memory)."""
    rng = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(o, i, amp=1.0):
        return to_bf16_values(rng.standard_normal((o, i)).astype(np.float32) * (amp / math.sqrt(i)))

    def scalar(lo=0.5, hi=1.5):
        return to_bf16_values(np.float32(rng.uniform(lo, hi) * gain)).reshape(())

    W["embed"] = to_bf16_values(rng.standard_normal((V, D)).astype(np.float32))
    if cfg.get("loop"):
        W["loop.in"] = mat(D, 2 * D, 1.4)
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        mx = L["mixer"]
        W[p + "norm1"], W[p + "norm1b"] = scalar(), scalar()
        if L["type"] == "attention":
            H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(H * d, D), mat(G * d, D), mat(G * dv, D)
            W[p + "mix.g"], W[p + "mix.o"] = mat(H, D, 2.0), mat(D, H * dv)
        else:
            H, d, R = mx["heads"], mx["dim"], L.get("_rank", 4)
            C = H * d
            for s in "rkvgw":
                W[p + "mix.mu." + s] = to_bf16_values(rng.uniform(0, 1, D).astype(np.float32))
            for s in "rkvg":
                W[p + "mix." + s] = mat(C, D)
            W[p + "mix.w1"], W[p + "mix.w2"] = mat(R, D), mat(C, R)
            W[p + "mix.w0"] = to_bf16_values((rng.uniform(-1, 1, C) + decay_bias).astype(np.float32))
            W[p + "mix.u"] = to_bf16_values(rng.uniform(-1, 1, (H, d)).astype(np.float32))
            W[p + "mix.norm"] = to_bf16_values(rng.uniform(0.5, 1.5, C).astype(np.float32))
            W[p + "mix.o"] = mat(D, C)
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            W[p + "norm2"], W[p + "norm2b"] = scalar(), scalar()
            W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"] = mat(F, D), mat(F, D), mat(D, F)
    W["final.norm"] = scalar()
    W["head"] = mat(V, D)
    return W


def public_config(cfg):
    """The configuration as a checkpoint folder carries it (test-only keys removed)."""
    out = dict(cfg)
    out["layers"] = [{k: v for k, v in L.items() if not k.startswith("_")} for L in cfg["layers"]]
    return out


def build_engine(cfg, W, dtype="float32", max_tokens=1024, max_seqs=4):
    from turboinfer_b200 import models
    return models.REGISTRY["Binusun"](public_config(cfg), W, dtype, max_tokens, max_seqs)


def rel_err(got, want):
    """RMS over the vocabulary of the difference (means taken off), relative to the RMS of the expected logits; max over rows."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float((np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean(-1) + 1e-30)).max())


def run_schedule(m, requests, schedule):
    """requests: name -> tokens; schedule: list of steps, a step a list of (name, count).  Every token's logits are collected.
    A request's pages and slot are given back right after its last token.  Returns name -> [len, vocab]."""
    at = {k: 0 for k in requests}
    seq, out = {}, {k: [] for k in requests}
    for step in schedule:
        entries, names = [], []
        for name, count in step:
            if name not in seq:
                seq[name] = m.open()
            entries.append((seq[name], requests[name][at[name]:at[name] + count]))
            names.append(name)
        lg = m.step(entries, [list(range(len(e[1]))) for e in entries])
        off = 0
        for name, e in zip(names, entries):
            out[name].append(lg[off:off + len(e[1])])
            off += len(e[1])
            at[name] += len(e[1])
            if at[name] == len(requests[name]):
                m.close(seq.pop(name))
    return {k: np.concatenate(v) for k, v in out.items() if v}
