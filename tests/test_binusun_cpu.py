"""CPU-side checks around the Binusun model: the plain implementation's own invariants, the configuration reader, the
safetensors reader / writer, and the layer-run order of a looped block.  No GPU, no engine library."""
import json
import math
import os

import numpy as np

import binusun_plain as plain
from binusun_cases import attn_layer, make_config, public_config, random_weights, rel_err, wkv_layer


def test_plain_prefix_property():
    # causal: the logits of a prefix do not change when tokens are appended
    cfg = make_config([wkv_layer(), attn_layer(window=6, ff=32)], loop=(0, 2, 2))
    W = random_weights(cfg, seed=1)
    toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg["vocab"], 30)]
    a, b = plain.forward(cfg, W, toks), plain.forward(cfg, W, toks[:17])
    assert rel_err(a[:17], b) < 1e-12


def test_plain_window_hides_old_tokens():
    cfg = make_config([attn_layer(window=4)])
    W = random_weights(cfg, seed=2)
    toks = list(range(20))
    other = [50] + toks[1:]
    a, b = plain.forward(cfg, W, toks), plain.forward(cfg, W, other)
    assert rel_err(a[4:], b[4:]) < 1e-12 and rel_err(a[3:4], b[3:4]) > 1e-6


def test_layer_runs_order():
    cfg = make_config([wkv_layer(), attn_layer(), attn_layer(), wkv_layer()], loop=(1, 3, 3))
    assert plain.layer_runs(cfg) == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    cfg = make_config([wkv_layer(), attn_layer()])
    assert plain.layer_runs(cfg) == [(0, False), (1, False)]


def test_rotation_is_interleaved_and_partial():
    x = np.arange(2 * 1 * 8, dtype=np.float64).reshape(2, 1, 8) + 1
    f = plain.rotary_frequencies(4, 100.0)
    y = plain.rotate_interleaved(x, [0, 3], f)
    assert np.array_equal(y[0], x[0]) and np.array_equal(y[1, :, 4:], x[1, :, 4:])
    a = 3 * f[1]
    assert np.allclose(y[1, 0, 2:4], [x[1, 0, 2] * math.cos(a) - x[1, 0, 3] * math.sin(a), x[1, 0, 3] * math.cos(a) + x[1, 0, 2] * math.sin(a)])


def test_config_reader_and_registry():
    from turboinfer_b200 import models, seq
    sc = {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 128}
    cfg = public_config(make_config([wkv_layer(heads=3, dim=8), attn_layer(heads=6, kv_heads=2, dim=20, vdim=12, window=9, rot_dims=10, scaling=sc, ff=44)],
                                    vocab=55, width=40, loop=(1, 2, 4), eps=1e-4, logit_scale=0.125))
    assert "Binusun" in models.REGISTRY and "llama" in models.REGISTRY
    d, layers = models.binusun_descs(cfg, seq.F32, 300, 3, {"l0.mix.w1": (5, 40)})
    assert (d.vocab, d.width, d.n_layers, d.loop_start, d.loop_stop, d.loop_times, d.max_tokens, d.max_seqs) == (55, 40, 2, 1, 2, 4, 300, 3)
    assert abs(d.norm_eps - 1e-4) < 1e-10 and d.logit_scale == 0.125 and d.mode == seq.F32
    w, a = layers
    assert (w.mixer, w.heads, w.dim, w.decay_rank, w.ff) == (seq.MIXER_WKV, 3, 8, 5, 0)
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.rot_dims, a.rot_scaled, a.ff) == (seq.MIXER_ATTENTION, 6, 2, 20, 12, 9, 10, 1, 44)
    assert (a.rot_factor, a.rot_low, a.rot_high, a.rot_original) == (4.0, 1.0, 2.0, 128.0)
    cfg["loop"] = None
    d, _ = models.binusun_descs(cfg, seq.BF16, 64, 1, {"l0.mix.w1": (5, 40)})
    assert d.loop_times == 0


def test_safetensors_round_trip(tmp_path):
    from turboinfer_b200.safetensors_io import read_safetensors, write_safetensors
    from turboinfer_b200.seq import Bf16Array
    cfg = make_config([wkv_layer()])
    W = random_weights(cfg, seed=4)
    p = os.path.join(tmp_path, "model.safetensors")
    write_safetensors(p, W)
    R = read_safetensors(p)
    assert set(R) == set(W)
    for k, v in W.items():
        assert isinstance(R[k], Bf16Array) and R[k].shape == np.shape(v)
        assert np.array_equal(R[k].to_f32(), np.asarray(v, np.float32))   # the test weights are bf16-representable
    write_safetensors(p, {"a": np.arange(6, dtype=np.float32).reshape(2, 3), "t": np.arange(4)}, bf16=False)
    R = read_safetensors(p)
    assert R["a"].dtype == np.float32 and R["t"].dtype == np.int32 and R["a"].shape == (2, 3)
    with open(p, "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        assert set(json.loads(f.read(n))) == {"a", "t"}
