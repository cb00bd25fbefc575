"""CPU-side checks around the Tudasun model: the plain implementation's own invariants (each mechanism against a second, direct
formula) and the configuration reader.  No GPU, no engine library."""
import math

import numpy as np

import tudasun_plain as plain
from tudasun_cases import dense, gla_layer, hgrn2_layer, latent_layer, make_config, moe, public_config, random_weights, rel_err


def toks(n, vocab, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def test_prefix_property():
    # causal: the logits of a prefix do not change when tokens are appended
    cfg = make_config([gla_layer(mlp=moe()), latent_layer(mlp=dense(16)), hgrn2_layer(), latent_layer(kv_from=1)])
    W = random_weights(cfg, seed=1)
    t = toks(30, cfg["vocab"])
    m = plain.PlainTudasun(cfg, W)
    assert rel_err(m.run(t)[0][:17], m.run(t[:17])[0]) < 1e-12


def test_recurrence_is_the_unrolled_sum():
    # o_t = sum_{s <= t} (q_t * prod_{s < r <= t} a_r) . w_s  v_s
    rng = np.random.default_rng(2)
    H, dk, dv, n = 2, 5, 3, 9
    a, w, q = rng.uniform(0.3, 1, (n, H, dk)), rng.standard_normal((n, H, dk)), rng.standard_normal((n, H, dk))
    v = rng.standard_normal((n, H, dv))
    S = np.zeros((H, dk, dv))
    for t in range(n):
        S, o = plain.recurrence_step(S, a[t], w[t], v[t], q[t])
        want = np.zeros((H, dv))
        for s in range(t + 1):
            want += np.einsum("hk,hv->hv", q[t] * np.prod(a[s + 1:t + 1], axis=0) * w[s], v[s])
        assert np.allclose(o, want)


def test_gla_decay_is_a_root_of_a_sigmoid():
    cfg = make_config([gla_layer(tau=4.0)])
    W = {k: np.asarray(v, np.float64) for k, v in random_weights(cfg, seed=3).items()}
    h = np.random.default_rng(3).standard_normal(cfg["width"])
    a = plain.gla_decay(h, W, "l0.mix.", 4.0)
    z = W["l0.mix.a2"] @ (W["l0.mix.a1"] @ h) + W["l0.mix.a2.b"]
    assert np.allclose(a ** 4.0, 1 / (1 + np.exp(-z))) and (a > 0).all() and (a < 1).all()


def test_rotation_pairs_neighbours():
    x = np.arange(8, dtype=np.float64) + 1
    y = plain.rotate_pairs(x, 3, 4, 100.0)
    assert np.array_equal(y[4:], x[4:])
    a = 3 * 100.0 ** (-2.0 / 4)
    assert np.allclose(y[2:4], [x[2] * math.cos(a) - x[3] * math.sin(a), x[3] * math.cos(a) + x[2] * math.sin(a)])
    assert np.array_equal(plain.rotate_pairs(x, 0, 8, 100.0), x)


def test_polynorm_terms():
    z = np.array([1.0, -2.0, 3.0, 0.5])
    y = plain.polynorm(z, [2.0, 0.0, 0.0, 0.25], 0.0)
    assert np.allclose(y, 2 * z / np.sqrt((z ** 2).mean()) + 0.25)
    y = plain.polynorm(z, [0.0, 1.0, -1.0, 0.0], 0.0)
    assert np.allclose(y, z ** 2 / np.sqrt((z ** 4).mean()) - z ** 3 / np.sqrt((z ** 6).mean()))


def test_router_groups_identity_and_weights():
    mlp = moe(experts=4, identity=2, top=2, count=3, keep=1)
    D = 6
    W = {"router": np.zeros((6, D)), "correction": np.zeros(6)}
    h = np.ones(D)
    W["router"][:, 0] = [0.0, 3.0, 2.9, 0.1, 1.0, 2.0]            # groups {0,1} {2,3} {4,5}: the best single score is in group 0
    picks = plain.route(h, W, "", mlp)
    assert [i for i, _ in picks] == [1, 0] and abs(sum(w for _, w in picks) - 1) < 1e-12
    W["correction"][:] = [0, 0, 0, 0, 0, 1.0]                      # the correction moves the choice to group 2 ...
    picks = plain.route(h, W, "", mlp)
    assert [i for i, _ in picks] == [5, 4]
    s = np.exp(W["router"][:, 0]) / np.exp(W["router"][:, 0]).sum()
    assert np.allclose([w for _, w in picks], s[[5, 4]] / s[[5, 4]].sum())   # ... but not the weights
    W["correction"][:] = -5.0                                      # negative choice scores: a group outside the kept ones still loses
    W["correction"][2] = -4.0
    assert [i for i, _ in plain.route(h, W, "", mlp)] == [2, 3]


def test_sink_only_enlarges_the_denominator():
    cfg = make_config([latent_layer(heads=1)], side=0)
    W = random_weights(cfg, seed=5)
    t = toks(6, cfg["vocab"])
    lo, hi = dict(W), dict(W)
    lo["l0.mix.sink"], hi["l0.mix.sink"] = np.array([-40.0]), np.array([40.0])
    a = plain.PlainTudasun(cfg, lo).run(t)[1]
    b = plain.PlainTudasun(cfg, hi).run(t)[1]
    x = np.asarray(W["embed"], np.float64)[t]
    assert np.abs(a[0] - x).max() > 0.1          # without a sink the mixer adds its (normed) output ...
    assert np.abs(b[0] - x).max() < 1e-6         # ... with a huge one the weights vanish and nothing is added (the norm behind maps 0 to 0)


def test_config_reader_and_registry():
    from turboinfer_b200 import models, seq
    cfg = public_config(make_config([gla_layer(heads=3, dim=8, vdim=12, tau=5.0, mlp=dense(44), rank=7),
                                     latent_layer(heads=5, dim=10, rot_dim=4, vdim=6, kv_rank=18, base=77.0, scale=0.3, mlp=moe(experts=6, identity=3, top=4, count=3, keep=2, ff=20, shared=28)),
                                     hgrn2_layer(heads=2, dim=16, vdim=8), latent_layer(heads=2, dim=10, rot_dim=4, vdim=6, kv_rank=18, base=77.0, kv_from=1,
                                                                                       mlp=moe(experts=2, identity=0, top=1, count=0, shared=0))],
                                    vocab=55, width=40, eps=1e-4, softcap=9.0, side=3))
    assert "Tudasun" in models.REGISTRY
    shapes = {"l0.mix.a1": (7, 40), "l0.rg1": (40, 40), "l1.rg1": (40, 40), "l2.rg1": (40, 40), "l3.rg1": (40, 40)}
    d, (g, a, h, b) = models.tudasun_descs(cfg, seq.F32, 300, 3, shapes)
    assert (d.vocab, d.width, d.n_layers, d.loop_times, d.max_tokens, d.max_seqs, d.side_dim, d.norm_kind) == (55, 40, 4, 0, 300, 3, 3, seq.NORM_ONE_PLUS)
    assert abs(d.norm_eps - 1e-4) < 1e-10 and d.logit_softcap == 9.0 and d.mode == seq.F32
    assert (g.mixer, g.heads, g.dim, g.vdim, g.decay_rank, g.decay_tau, g.ff_kind, g.ff, g.res_gate) == (seq.MIXER_GLA, 3, 8, 12, 7, 5.0, seq.FF_POLYNORM, 44, 1)
    assert (a.mixer, a.heads, a.dim, a.rot_dims, a.vdim, a.kv_rank, a.kv_from, a.sink) == (seq.MIXER_LATENT, 5, 10, 4, 6, 18, -1, 1)
    assert abs(a.scale - 0.3) < 1e-7 and a.rot_base == 77.0
    assert (a.ff_kind, a.ff, a.experts, a.identity, a.top, a.groups, a.groups_keep, a.shared_ff) == (seq.FF_EXPERTS, 20, 6, 3, 4, 3, 2, 28)
    assert (h.mixer, h.heads, h.dim, h.vdim, h.ff) == (seq.MIXER_HGRN2, 2, 16, 8, 0)
    assert (b.kv_from, b.experts, b.identity, b.top, b.groups, b.groups_keep, b.shared_ff) == (1, 2, 0, 1, 1, 1, 0)
    cfg["token_side"], cfg["logit_softcap"] = None, None
    d, _ = models.tudasun_descs(cfg, seq.BF16, 64, 1, shapes)
    assert d.side_dim == 0 and d.logit_softcap == 0.0
