"""Small Tudasun configurations with random weights for the tests, and helpers that run them through the engine.

Weights are rounded to bfloat16-representable values, so the bf16 and the fp32 engine and the plain implementation all see
exactly the same numbers."""
from __future__ import annotations

import math

import numpy as np

from binusun_cases import rel_err, run_schedule, to_bf16_values  # noqa: F401  (re-exported for the tests)


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=4, identity=2, top=2, count=3, keep=2, ff=16, shared=24):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if count:
        m["router"]["groups"] = {"count": count, "keep": keep}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def gla_layer(heads=2, dim=16, vdim=24, tau=8.0, mlp=None, rank=4):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp, "_rank": rank}


def hgrn2_layer(heads=3, dim=8, vdim=16, mlp=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def latent_layer(heads=2, dim=12, rot_dim=8, vdim=20, kv_rank=24, base=10000.0, scale=None, kv_from=None, mlp=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": {"base": base, "dims": rot_dim},
          "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def make_config(layers, vocab=131, width=48, eps=1e-5, softcap=12.0, side=6):
    cfg = {"architecture": "Tudasun", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if softcap:
        cfg["logit_softcap"] = softcap
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def random_weights(cfg, seed=0, decay_bias=1.0, lower_hi=0.9, sink=None, router_amp=3.0, decisive=False):
    """decisive: the router's corrections are two apart, so the choice of experts does not depend on the token (the weights still
    do) and a rounding difference in front of the router cannot flip it -- for comparisons in bf16 mode; decay_bias: offset of the gla decay's pre-activation (large: decays close to 1, a long memory); lower_hi: upper end of
    the hgrn2 lower bounds; sink: a fixed value for every head's sink (default: random)."""
    rng = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(o, i, amp=1.0):
        return to_bf16_values(rng.standard_normal((o, i)).astype(np.float32) * (amp / math.sqrt(i)))

    def vec(n, lo, hi):
        return to_bf16_values(rng.uniform(lo, hi, n).astype(np.float32))

    def around_zero(n):
        return to_bf16_values((rng.standard_normal(n) * 0.2).astype(np.float32))

    W["embed"] = to_bf16_values(rng.standard_normal((V, D)).astype(np.float32))
    ds = cfg["token_side"]["dim"] if cfg.get("token_side") else 0
    if ds:
        W["side.embed"] = to_bf16_values(rng.standard_normal((V, ds * len(cfg["layers"]))).astype(np.float32))
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        mx = L["mixer"]
        H = mx["heads"]
        W[p + "norm1"], W[p + "norm1b"] = around_zero(D), around_zero(D)
        W[p + "rg1"], W[p + "rg1.b"] = mat(D, D), around_zero(D)
        if L["type"] == "gla":
            C, Cv, R = H * mx["dim"], H * mx["vdim"], L.get("_rank", 4)
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"], W[p + "mix.g"] = mat(C, D, 2.0), mat(C, D), mat(Cv, D), mat(Cv, D)
            W[p + "mix.a1"], W[p + "mix.a2"] = mat(R, D), mat(C, R, 2.0)
            W[p + "mix.a2.b"] = to_bf16_values((rng.uniform(-1, 1, C) + decay_bias).astype(np.float32))
            W[p + "mix.norm"], W[p + "mix.o"] = vec(mx["vdim"], 0.5, 1.5), mat(D, Cv)
        elif L["type"] == "hgrn2":
            C, Cv = H * mx["dim"], H * mx["vdim"]
            W[p + "mix.q"], W[p + "mix.f"], W[p + "mix.v"] = mat(C, D, 2.0), mat(C, D, 2.0), mat(Cv, D)
            W[p + "mix.f.b"], W[p + "mix.lower"] = around_zero(C), vec(C, 0.0, lower_hi)
            W[p + "mix.norm"], W[p + "mix.o"] = vec(mx["vdim"], 0.5, 1.5), mat(D, Cv)
        else:
            d, dr, dv, r = mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
            W[p + "mix.q"] = mat(H * (d + dr), D, 2.0)
            if mx.get("kv_from") is None:
                W[p + "mix.dkv"], W[p + "mix.dkv.norm"] = mat(r + dr, D, 2.0), vec(r, 0.5, 1.5)
            W[p + "mix.uk"], W[p + "mix.uv"] = mat(H * d, r, 2.0), mat(H * dv, r)
            W[p + "mix.sink"] = to_bf16_values(np.full(H, sink, np.float32)) if sink is not None else to_bf16_values(rng.standard_normal(H).astype(np.float32))
            W[p + "mix.o"] = mat(D, H * dv)
        mlp = L.get("mlp")
        if mlp:
            W[p + "norm2"], W[p + "norm2b"] = around_zero(D), around_zero(D)
            W[p + "rg2"], W[p + "rg2.b"] = mat(D, D), around_zero(D)
            if mlp["kind"] == "dense":
                W[p + "mlp.up"], W[p + "mlp.down"] = mat(mlp["ff"], D), mat(D, mlp["ff"])
                W[p + "mlp.act"] = vec(4, -1.0, 1.0)
            else:
                r, F = mlp["router"], mlp["expert"]["ff"]
                n = r["experts"] + r.get("identity", 0)
                for e in range(r["experts"]):
                    q = p + "mlp.e%d." % e
                    W[q + "gate"], W[q + "up"], W[q + "down"] = mat(F, D, 1.5), mat(F, D, 1.5), mat(D, F, 1.5)
                W[p + "mlp.router"] = mat(n, D, router_amp)
                W[p + "mlp.correction"] = to_bf16_values(rng.permutation(n).astype(np.float32) * 2.0) if decisive else vec(n, -0.15, 0.15)
                if mlp.get("shared"):
                    Fs = mlp["shared"]["ff"]
                    W[p + "mlp.shared.gate"], W[p + "mlp.shared.up"], W[p + "mlp.shared.down"] = mat(Fs, D), mat(Fs, D), mat(D, Fs)
                    W[p + "mlp.shared.sg"] = mat(1, D, 2.0)
        if ds:
            W[p + "side.gate"], W[p + "side.proj"], W[p + "side.norm"] = mat(ds, D, 2.0), mat(D, ds), vec(D, 0.2, 0.6)
    W["final.norm"] = around_zero(D)
    W["head"] = mat(V, D, 3.0)
    return W


def public_config(cfg):
    """The configuration as a checkpoint folder carries it (test-only keys removed)."""
    out = dict(cfg)
    out["layers"] = [{k: v for k, v in L.items() if not k.startswith("_")} for L in cfg["layers"]]
    return out


def build_engine(cfg, W, dtype="float32", max_tokens=1024, max_seqs=4):
    from turboinfer_b200 import models
    return models.REGISTRY["Tudasun"](public_config(cfg), W, dtype, max_tokens, max_seqs)


def row_errs(got, want):
    """Per row: RMS over the vocabulary of the difference (means taken off) relative to the RMS of the expected logits."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean(-1) + 1e-30)
