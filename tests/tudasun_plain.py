"""Plain, slow implementation of the Tudasun decoder design (numpy, float64): the oracle of tests/test_gpu_tudasun.py.

One function per mechanism, written from the design's equations; nothing here is shared with the engine.  A model is a
configuration dictionary (the keys of config.json) and a dictionary name -> float array.  Sequences are processed one token
at a time through explicit caches, so the same code answers "what are the logits at position p" whatever the engine's
batching was.

  norm            y = x / sqrt(mean(x^2) + eps) * (1 + w)             (vector gain stored around zero)
  plain norm      y = x / sqrt(mean(x^2) + eps) * w
  gated residual  sublayer(h) * sigmoid(R h + b), then the norm behind the sublayer, then the residual sum
  gla             S <- diag(a) S + k v^T, o = S^T q, a = sigmoid(A2 A1 h + b)^(1/tau), q scaled by dim^-1/2, per-head plain
                  norm over the value size, times silu(G h), output projection
  hgrn2           S <- diag(f) S + (1 - f) v^T, o = S^T q, f = l + (1 - l) sigmoid(F h + b), q = silu(Q h)
  latent          keys and values are linear images of a cached low-rank vector c (plain-normed) plus one rotated key part
                  shared by the heads; softmax over all earlier positions with one extra, value-less term exp(sink_h)
  dense ff        D act(U h), act = a N(z) + b N(z^2) + c N(z^3) + e, N = division by the root mean square over the ff size
  expert ff       router softmax over real + identity experts, choice by score + correction inside the best groups,
                  weights renormalised over the chosen ones; a shared expert scaled by a sigmoid of one more projection
  side input      per layer: gelu_tanh(Gs x) * side_embedding[token, layer slice], projected, plain-normed, added
  output          norm, head, cap * tanh(logits / cap)
"""
from __future__ import annotations

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def rms_div(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    return rms_div(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_div(x, eps) * w


def rotate_pairs(v, pos, dims, base):
    """Coordinates (2i, 2i+1), i < dims/2, of the last axis are turned by the angle pos * base^(-2i/dims)."""
    out = np.array(v, dtype=np.float64, copy=True)
    i = np.arange(dims // 2)
    ang = pos * base ** (-2.0 * i / dims)
    c, s = np.cos(ang), np.sin(ang)
    a, b = out[..., 0:dims:2].copy(), out[..., 1:dims:2].copy()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def polynorm(z, coef, eps):
    a, b, c, e = [float(t) for t in coef]
    return a * rms_div(z, eps) + b * rms_div(z * z, eps) + c * rms_div(z * z * z, eps) + e


def gla_decay(h, W, p, tau):
    z = W[p + "a2"] @ (W[p + "a1"] @ h) + W[p + "a2.b"]
    return sigmoid(z) ** (1.0 / tau)


def recurrence_step(S, decay, write, v, read):
    """S [heads, dk, dv] <- decay[..., None] * S + write[..., None] * v[:, None, :]; returns (S, o [heads, dv]) with o = S^T read."""
    S = decay[:, :, None] * S + write[:, :, None] * v[:, None, :]
    return S, np.einsum("hkv,hk->hv", S, read)


def head_norm(o, w, eps):
    return rms_div(o, eps) * w[None, :]


def route(h, W, p, mlp, eps_sum=1e-20):
    """-> list of (expert index, weight) for one token; indices >= experts are identity experts."""
    r = mlp["router"]
    n_real, n_id, top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
    z = W[p + "router"] @ h
    z = z - z.max()
    s = np.exp(z) / np.exp(z).sum()
    choice = s + W[p + "correction"]
    n = n_real + n_id
    g = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(g["count"]), int(g["keep"])
    size = n // count
    gscore = np.array([choice[i * size:(i + 1) * size].max() for i in range(count)])
    allowed = np.zeros(n, bool)
    for gi in np.argsort(-gscore, kind="stable")[:keep]:
        allowed[gi * size:(gi + 1) * size] = True
    masked = np.where(allowed, choice, -np.inf)
    picked = np.argsort(-masked, kind="stable")[:top]
    tot = s[picked].sum() + eps_sum
    return [(int(i), float(s[i] / tot)) for i in picked]


def glu_expert(h, W, p):
    return W[p + "down"] @ (silu(W[p + "gate"] @ h) * (W[p + "up"] @ h))


def expert_ff(h, W, p, mlp):
    n_real = int(mlp["router"]["experts"])
    y = np.zeros_like(h)
    for i, w in route(h, W, p, mlp):
        y = y + w * (glu_expert(h, W, p + "e%d." % i) if i < n_real else h)
    if mlp.get("shared"):
        y = y + sigmoid(float((W[p + "shared.sg"] @ h)[0])) * glu_expert(h, W, p + "shared.")
    return y


def dense_ff(h, W, p, eps):
    return W[p + "down"] @ polynorm(W[p + "up"] @ h, W[p + "act"], eps)


class PlainTudasun:
    """Token-by-token evaluation with explicit state: `state = new_state()`, `logits, layers = token(state, tok)`."""

    def __init__(self, cfg: dict, weights: dict):
        self.cfg = cfg
        self.W = {k: np.asarray(v, np.float64) for k, v in weights.items() if not np.issubdtype(np.asarray(v).dtype, np.integer)}
        self.eps = float(cfg["norm"]["eps"])
        self.side = int(cfg["token_side"]["dim"]) if cfg.get("token_side") else 0

    def new_state(self):
        st = {"pos": 0, "layers": []}
        for L in self.cfg["layers"]:
            mx = L["mixer"]
            if L["type"] in ("gla", "hgrn2"):
                st["layers"].append({"S": np.zeros((mx["heads"], mx["dim"], mx["vdim"]))})
            else:
                st["layers"].append({"c": [], "kr": []})
        return st

    def mixer(self, i, L, h, st, pos):
        W, p, mx, eps = self.W, "l%d.mix." % i, L["mixer"], self.eps
        H = int(mx["heads"])
        if L["type"] == "gla":
            d, dv = int(mx["dim"]), int(mx["vdim"])
            q = (W[p + "q"] @ h).reshape(H, d) * d ** -0.5
            k = (W[p + "k"] @ h).reshape(H, d)
            v = (W[p + "v"] @ h).reshape(H, dv)
            a = gla_decay(h, W, p, float(mx["tau"])).reshape(H, d)
            st["S"], o = recurrence_step(st["S"], a, k, v, q)
            o = head_norm(o, W[p + "norm"], eps).reshape(-1) * silu(W[p + "g"] @ h)
            return W[p + "o"] @ o
        if L["type"] == "hgrn2":
            d, dv = int(mx["dim"]), int(mx["vdim"])
            q = silu(W[p + "q"] @ h).reshape(H, d)
            v = (W[p + "v"] @ h).reshape(H, dv)
            low = W[p + "lower"]
            f = (low + (1.0 - low) * sigmoid(W[p + "f"] @ h + W[p + "f.b"])).reshape(H, d)
            st["S"], o = recurrence_step(st["S"], f, 1.0 - f, v, q)
            return W[p + "o"] @ head_norm(o, W[p + "norm"], eps).reshape(-1)
        if L["type"] == "latent_attention":
            d, dr, dv, rank = int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"]), int(mx["kv_rank"])
            rot = mx["rot"]
            q = (W[p + "q"] @ h).reshape(H, d + dr)
            q_plain, q_rot = q[:, :d], rotate_pairs(q[:, d:], pos, int(rot["dims"]), float(rot["base"]))
            src = mx.get("kv_from")
            if src is None:
                t = W[p + "dkv"] @ h
                st["c"].append(norm_plain(t[:rank], W[p + "dkv.norm"], eps))
                st["kr"].append(rotate_pairs(t[rank:], pos, int(rot["dims"]), float(rot["base"])))
                cache = st
            else:
                cache = self._state["layers"][int(src)]
            c, kr = np.stack(cache["c"]), np.stack(cache["kr"])          # [n, rank], [n, dr]
            k_plain = (c @ W[p + "uk"].T).reshape(-1, H, d)
            val = (c @ W[p + "uv"].T).reshape(-1, H, dv)
            sc = (np.einsum("hd,nhd->hn", q_plain, k_plain) + q_rot @ kr.T) * float(mx["scale"])
            sink = W[p + "sink"]
            m = np.maximum(sc.max(axis=1), sink)
            e = np.exp(sc - m[:, None])
            wgt = e / (e.sum(axis=1) + np.exp(sink - m))[:, None]
            return W[p + "o"] @ np.einsum("hn,nhv->hv", wgt, val).reshape(-1)
        raise ValueError(L["type"])

    def token(self, st, tok):
        W, eps, cfg = self.W, self.eps, self.cfg
        self._state = st
        pos = st["pos"]
        x = W["embed"][tok].copy()
        after = []
        for i, L in enumerate(cfg["layers"]):
            p = "l%d." % i
            h = norm_one_plus(x, W[p + "norm1"], eps)
            r = self.mixer(i, L, h, st["layers"][i], pos) * sigmoid(W[p + "rg1"] @ h + W[p + "rg1.b"])
            x = x + norm_one_plus(r, W[p + "norm1b"], eps)
            if L.get("mlp"):
                h = norm_one_plus(x, W[p + "norm2"], eps)
                y = dense_ff(h, W, p + "mlp.", eps) if L["mlp"]["kind"] == "dense" else expert_ff(h, W, p + "mlp.", L["mlp"])
                y = y * sigmoid(W[p + "rg2"] @ h + W[p + "rg2.b"])
                x = x + norm_one_plus(y, W[p + "norm2b"], eps)
            if self.side:
                e = W["side.embed"][tok][i * self.side:(i + 1) * self.side]
                y = W[p + "side.proj"] @ (gelu_tanh(W[p + "side.gate"] @ x) * e)
                x = x + norm_plain(y, W[p + "side.norm"], eps)
            after.append(x.copy())
        st["pos"] = pos + 1
        z = W["head"] @ norm_one_plus(x, W["final.norm"], eps)
        cap = cfg.get("logit_softcap")
        if cap:
            z = float(cap) * np.tanh(z / float(cap))
        return z, np.stack(after)

    def run(self, tokens):
        """-> (logits [n, vocab], residual stream after every layer [layers, n, width])"""
        st = self.new_state()
        outs = [self.token(st, int(t)) for t in tokens]
        return np.stack([o[0] for o in outs]), np.stack([o[1] for o in outs], axis=1)
