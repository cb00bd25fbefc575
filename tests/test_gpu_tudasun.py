"""The layered sequence engine on Tudasun models against the plain implementation (tests/tudasun_plain.py): every mechanism
alone, prompts against token-by-token decoding, portions, ragged batches, reuse of pages and state slots, far keys and page
borders with one score made to stand out, the sink, long memory of the recurrences, long decoding, odd sizes, and greedy
generation through the engine's own generation loop and command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tudasun_cases import (build_engine, dense, gla_layer, hgrn2_layer, latent_layer, make_config, moe, public_config, random_weights, rel_err,
                           row_errs, run_schedule, to_bf16_values)
from tudasun_plain import PlainTudasun, norm_one_plus, norm_plain

pytestmark = pytest.mark.gpu

# bf16 mode: products round their inputs to bf16 (relative 4e-3 each); through five layers with cubed activations and capped logits a
# row's error reaches a few percent of the logits' spread, the median stays near one percent
TOL = {"float32": 2e-4, "bfloat16": 1e-1}


def tokens(n, vocab, seed=1):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def whole(m, toks):
    return run_schedule(m, {"a": toks}, [[("a", len(toks))]])["a"]


def check_logits(got, want, dtype):
    assert row_errs(got, want).max() < TOL[dtype]


def weights(cfg, seed, dtype, **kw):
    """In bf16 mode a rounding difference in front of a router could flip a close choice of experts, and the recurrent layers
    behind it would carry the difference to every later token: those comparisons use routers whose choice is fixed by their
    corrections (the fp32 comparisons test the choice itself)."""
    return random_weights(cfg, seed=seed, decisive=(dtype == "bfloat16"), **kw)


# ---- each mechanism alone: residual stream after every layer, and the logits -----------------------------------------------------
MECHANISMS = {
    "gla": make_config([gla_layer()]),
    "gla_wide_keys_one_head": make_config([gla_layer(heads=1, dim=40, vdim=24, tau=3.0, rank=5), gla_layer(heads=2, dim=72, vdim=33, rank=1)], width=40, side=0),
    "gla_many_value_columns": make_config([gla_layer(heads=2, dim=20, vdim=168, rank=3), hgrn2_layer(heads=1, dim=64, vdim=200)], width=40, side=0),
    "gla_state_in_shared_memory": make_config([gla_layer(heads=1, dim=136, vdim=40, rank=3)], width=64),
    "recurrence_128_key_channels": make_config([hgrn2_layer(heads=1, dim=128, vdim=40), gla_layer(heads=2, dim=128, vdim=96, rank=2)], width=64),
    "hgrn2": make_config([hgrn2_layer()]),
    "hgrn2_equal_sizes": make_config([hgrn2_layer(heads=2, dim=32, vdim=32), hgrn2_layer(heads=1, dim=64, vdim=8)], softcap=0),
    "latent": make_config([latent_layer()]),
    "latent_odd_sizes": make_config([latent_layer(heads=3, dim=10, rot_dim=6, vdim=7, kv_rank=17, base=50.0)], width=36, eps=1e-3),
    "latent_no_rotation_part_of_two": make_config([latent_layer(heads=1, dim=16, rot_dim=2, vdim=16, kv_rank=16)]),
    "latent_wide_cache_row": make_config([latent_layer(heads=2, dim=24, rot_dim=16, vdim=12, kv_rank=272)], width=40),
    "latent_shared_cache": make_config([latent_layer(mlp=dense(24)), gla_layer(), latent_layer(heads=4, dim=6, vdim=10, kv_from=0), latent_layer(kv_from=0)]),
    "dense_ff": make_config([hgrn2_layer(mlp=dense(56))]),
    "experts": make_config([gla_layer(mlp=moe())]),
    "experts_no_groups_no_identity_no_shared": make_config([hgrn2_layer(mlp=moe(experts=5, identity=0, top=3, count=0, shared=0))]),
    "experts_one_choice_every_group_kept": make_config([hgrn2_layer(mlp=moe(experts=3, identity=3, top=1, count=2, keep=2, ff=8, shared=8))], side=0),
    "experts_many": make_config([gla_layer(mlp=moe(experts=37, identity=3, top=9, count=8, keep=3, ff=8, shared=0))]),
    "no_side_input_no_cap": make_config([gla_layer(mlp=dense(32)), latent_layer()], side=0, softcap=0),
    "hybrid": make_config([gla_layer(mlp=dense(40)), latent_layer(mlp=moe()), hgrn2_layer(mlp=moe(experts=2, identity=1, top=2, count=3, keep=2)),
                           latent_layer(heads=3, kv_from=1), hgrn2_layer()], vocab=101, width=56, side=7),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_mechanism_layers_and_logits(name, dtype):
    cfg = MECHANISMS[name]
    W = weights(cfg, 3, dtype)
    toks = tokens(37, cfg["vocab"])
    want, layers = PlainTudasun(cfg, W).run(toks)
    m = build_engine(cfg, W, dtype)
    m.debug_layers(True)
    got = whole(m, toks)
    got_layers = m.read_layers(len(toks))
    m.free()
    assert got_layers.shape == layers.shape
    for i in range(layers.shape[0]):
        scale = np.sqrt((layers[i] ** 2).mean())
        assert np.abs(got_layers[i] - layers[i]).max() / scale < TOL[dtype] * 5, f"layer {i}"
    check_logits(got, want, dtype)


# ---- prompts against decoding, portions, batches ---------------------------------------------------------------------------------
HYBRID = make_config([gla_layer(mlp=dense(40)), latent_layer(mlp=moe()), hgrn2_layer(mlp=moe(experts=3, identity=1, top=2, count=2, keep=1)),
                      latent_layer(heads=3, kv_from=1, mlp=dense(24)), gla_layer(heads=3, dim=8, vdim=8, tau=2.0)], side=5)
NO_ROUTER = make_config([hgrn2_layer(mlp=dense(40)), latent_layer(), gla_layer(mlp=dense(16)), latent_layer(kv_from=1, mlp=dense(24))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_token_by_token(dtype):
    W = weights(HYBRID, 5, dtype)
    toks = tokens(150, HYBRID["vocab"], 2)
    want, _ = PlainTudasun(HYBRID, W).run(toks)
    m = build_engine(HYBRID, W, dtype)
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 1)] for _ in toks])["a"]
    m.free()
    check_logits(a, want, dtype)
    check_logits(b, want, dtype)
    check_logits(b, a, dtype)


@pytest.mark.parametrize("rank,rot", [(256, 64), (128, 64), (128, 32)])
def test_latent_prompts_on_the_tensor_cores(rank, rot):
    """bf16 mode, cache rows of 256 + 64, 128 + 64 and 128 + 32: prompt portions of latent attention run on the split-half tensor-core kernel (tiles of
    64 rows, key tiles = pages, both halves of the value columns), single tokens on the row kernels; a large sink on one head."""
    cfg = make_config([latent_layer(heads=3, dim=32, rot_dim=rot, vdim=24, kv_rank=rank, mlp=dense(48)), latent_layer(heads=2, dim=16, rot_dim=rot, vdim=40, kv_rank=rank, kv_from=0)],
                      width=64)
    W = random_weights(cfg, seed=21)
    W["l0.mix.sink"] = to_bf16_values(np.array([2.0, -1.0, 0.5], np.float32))
    toks = tokens(330, cfg["vocab"], 21)
    want, _ = PlainTudasun(cfg, W).run(toks)
    m = build_engine(cfg, W, "bfloat16")
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 130)], [("a", 70)], [("a", 9)], [("a", 100)]] + [[("a", 1)]] * 21)["a"]
    m.free()
    m = build_engine(cfg, W, "float32")
    c = whole(m, toks)
    m.free()
    assert rel_err(a, want) < TOL["bfloat16"] and rel_err(b, want) < TOL["bfloat16"] and rel_err(c, want) < TOL["float32"]
    assert rel_err(b, a) < 2e-2


@pytest.mark.parametrize("sizes", [[2] * 40, [3, 61, 2, 64, 5, 65, 1, 63, 2], [64, 64, 64], [1, 127, 2, 2, 100], [129, 2, 33]])
def test_portions(sizes):
    toks = tokens(sum(sizes), HYBRID["vocab"], 7)
    W = random_weights(HYBRID, seed=6)
    want, _ = PlainTudasun(HYBRID, W).run(toks)
    m = build_engine(HYBRID, W, "float32")
    got = run_schedule(m, {"a": toks}, [[("a", n)] for n in sizes])["a"]
    m.free()
    assert rel_err(got, want) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_ragged_batch_equals_each_alone(dtype):
    cfg = HYBRID if dtype == "float32" else NO_ROUTER
    W = random_weights(cfg, seed=8)
    reqs = {"a": tokens(90, cfg["vocab"], 11), "b": tokens(17, cfg["vocab"], 12), "c": tokens(130, cfg["vocab"], 13), "d": tokens(1, cfg["vocab"], 14)}
    m = build_engine(cfg, W, dtype, max_tokens=448)
    alone = {k: whole(m, v) for k, v in reqs.items()}
    sched = [[("a", 30), ("b", 2)], [("a", 1), ("b", 9), ("c", 64)], [("c", 2), ("a", 1), ("d", 1)], [("b", 6), ("a", 58), ("c", 64)]]
    got = run_schedule(m, reqs, sched)
    m.free()
    oracle = PlainTudasun(cfg, W)
    for k, v in reqs.items():
        assert rel_err(got[k], alone[k]) < TOL[dtype], k
        assert rel_err(got[k], oracle.run(v)[0]) < TOL[dtype], k


def test_pages_and_slots_are_reused():
    """Two slots and three pages for five requests: later requests run in the slots and pages earlier ones gave back, and a
    stale recurrent state or a stale cache row would show in their logits."""
    cfg = NO_ROUTER
    W = random_weights(cfg, seed=9)
    m = build_engine(cfg, W, "float32", max_tokens=192, max_seqs=2)
    oracle = PlainTudasun(cfg, W)
    seen_pages, seen_slots = [], []
    for i, n in enumerate([100, 70, 128, 5, 64]):
        toks = tokens(n, cfg["vocab"], 20 + i)
        s = m.open()
        other = m.open()   # a second live sequence holds the other slot and a page while this one runs
        m.step([(other, tokens(3, cfg["vocab"], 40 + i))], [[]])
        got = np.concatenate([m.step([(s, toks[:n // 2])], [list(range(n // 2))]), m.step([(s, toks[n // 2:])], [list(range(n - n // 2))])])
        seen_pages.append(tuple(m.pages(s)))
        seen_slots.append(s)
        assert rel_err(got, oracle.run(toks)[0]) < TOL["float32"], i
        m.close(s)
        m.close(other)
    assert m.pool_info()["free_pages"] == 3 and m.pool_info()["free_slots"] == 2
    m.free()
    assert len(set(seen_slots)) <= 2
    assert len(set(p for ps in seen_pages for p in ps)) <= 3 and len(seen_pages) == 5


# ---- a key that stands out: far away, at page borders, the first token; in prompts and in decoding -------------------------------
def planted_pair(cfg, W):
    """For a model whose FIRST layer is latent attention: the (key token A, query token B) with the largest unrotated score of
    head 0 over the vocabulary, computed from the design's equations (the mixer input of a first layer depends on the token only)."""
    mx = cfg["layers"][0]["mixer"]
    d, dr, rank, eps = mx["dim"], mx["rot_dim"], mx["kv_rank"], cfg["norm"]["eps"]
    Wd = {k: np.asarray(v, np.float64) for k, v in W.items()}
    h = norm_one_plus(Wd["embed"], Wd["l0.norm1"], eps)                              # [V, D]
    q = (h @ Wd["l0.mix.q"].T)[:, :d]                                                # head 0, unrotated part
    c = norm_plain((h @ Wd["l0.mix.dkv"].T)[:, :rank], Wd["l0.mix.dkv.norm"], eps)
    k = c @ Wd["l0.mix.uk"][:d].T
    s = q @ k.T                                                                       # [query token, key token]
    b, a = np.unravel_index(np.argmax(s), s.shape)
    others = np.argsort(s[b])[: len(s) // 2]                                          # key tokens that score low against B
    return int(a), int(b), [int(t) for t in others if t != a]


@pytest.mark.parametrize("place,n", [(0, 40), (3, 300), (63, 200), (64, 200), (127, 260), (128, 260), (191, 193)])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_stands_out(place, n, decode):
    """Token A sits at `place` among n - 1 tokens that score low against the last token B; the scale is raised so that B's head 0
    puts most of its weight on A.  Leaving that one key out changes B's logits by far more than the tolerance (checked on the
    plain implementation), so an engine that loses the key at a page border, far back or at position 0 cannot pass."""
    cfg = make_config([latent_layer(heads=2, dim=16, rot_dim=2, vdim=16, kv_rank=24, scale=1.5), latent_layer(heads=2, dim=16, rot_dim=2, vdim=16, kv_rank=24, kv_from=0)],
                      width=64, side=0)
    W = random_weights(cfg, seed=13, sink=-2.0)
    A, B, filler = planted_pair(cfg, W)
    rng = np.random.default_rng(place)
    toks = [filler[int(i)] for i in rng.integers(0, len(filler), n)]
    toks[place], toks[-1] = A, B
    oracle = PlainTudasun(cfg, W)
    want, _ = oracle.run(toks)
    st = oracle.new_state()
    for t in toks[:-1]:
        oracle.token(st, t)
    del st["layers"][0]["c"][place], st["layers"][0]["kr"][place]
    without, _ = oracle.token(st, toks[-1])
    assert row_errs(without[None], want[-1:])[0] > 50 * TOL["float32"]
    m = build_engine(cfg, W, "float32")
    if decode:
        got = run_schedule(m, {"a": toks}, [[("a", n - 4)]] + [[("a", 1)]] * 4)["a"]
    else:
        got = whole(m, toks)
    m.free()
    assert rel_err(got, want) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_counts_once_and_only_in_the_denominator(dtype):
    """A large sink takes most of the softmax mass at the first positions: leaving it out (or adding a value for it) would scale
    the attention output by several times there."""
    cfg = make_config([latent_layer(heads=2)], side=0)
    W = random_weights(cfg, seed=14, sink=3.0)
    W["l0.mix.sink"] = to_bf16_values(np.array([3.0, -1.0], np.float32))
    toks = tokens(70, cfg["vocab"], 3)
    want, _ = PlainTudasun(cfg, W).run(toks)
    W0 = dict(W)
    W0["l0.mix.sink"] = np.full(2, -30.0, np.float32)
    assert row_errs(PlainTudasun(cfg, W0).run(toks)[0][:4], want[:4]).max() > 0.5
    m = build_engine(cfg, W, dtype)
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 1)]] * 70)["a"]
    m.free()
    assert rel_err(a, want) < TOL[dtype] and rel_err(b, want) < TOL[dtype]


def test_recurrent_state_long_memory():
    """Decays close to 1 (gla) and lower bounds close to 1 (hgrn2): the first token still moves the last logits after 400 tokens,
    whether the state was carried through one prompt, through portions or through single tokens."""
    cfg = make_config([gla_layer(tau=16.0), hgrn2_layer()], side=0)
    W = random_weights(cfg, seed=15, decay_bias=6.0, lower_hi=0.0)
    W["l1.mix.lower"] = to_bf16_values(np.full(24, 0.996, np.float32))
    toks = tokens(400, cfg["vocab"], 4)
    oracle = PlainTudasun(cfg, W)
    want, _ = oracle.run(toks)
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert row_errs(oracle.run(other)[0][-1:], want[-1:])[0] > 20 * TOL["float32"]
    m = build_engine(cfg, W, "float32")
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 150)], [("a", 2)], [("a", 200)]] + [[("a", 1)]] * 48)["a"]
    m.free()
    assert rel_err(a, want) < TOL["float32"] and rel_err(b, want) < TOL["float32"]


def test_first_tokens_and_single_token_requests():
    W = random_weights(HYBRID, seed=16)
    oracle = PlainTudasun(HYBRID, W)
    m = build_engine(HYBRID, W, "float32")
    for n in (1, 2, 3):
        toks = tokens(n, HYBRID["vocab"], 30 + n)
        assert rel_err(whole(m, toks), oracle.run(toks)[0]) < TOL["float32"]
    m.free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    cfg = NO_ROUTER
    W = random_weights(cfg, seed=17)
    toks = tokens(330, cfg["vocab"], 5)
    want, _ = PlainTudasun(cfg, W).run(toks)
    m = build_engine(cfg, W, dtype)
    got = run_schedule(m, {"a": toks}, [[("a", 10)]] + [[("a", 1)]] * 320)["a"]
    m.free()
    assert rel_err(got, want) < TOL[dtype]


@pytest.mark.parametrize("rows", [1, 3, 8])
def test_wide_model_decode_rows_and_tiles(rows):
    """Widths in whole 32-element chunks (bf16 mode: the decode rows' products run on the tensor-core few-row kernel, prompt
    products on tcgen05), heads of 64 key channels with the state in registers, a cached row of 128 + 32."""
    cfg = make_config([gla_layer(heads=2, dim=64, vdim=64, mlp=dense(264), rank=8), latent_layer(heads=2, dim=64, rot_dim=32, vdim=64, kv_rank=128, mlp=moe(ff=64, shared=96)),
                       hgrn2_layer(heads=2, dim=64, vdim=128), latent_layer(heads=4, dim=32, rot_dim=32, vdim=48, kv_rank=128, kv_from=1)], vocab=203, width=256, side=16)
    W = weights(cfg, 31, "bfloat16")
    lens = [150, 9, 33, 70, 21, 7, 12, 40][:rows]
    reqs = {"r%d" % i: tokens(n, 203, 60 + i) for i, n in enumerate(lens)}
    m = build_engine(cfg, W, "bfloat16", max_tokens=sum((n + 63) // 64 * 64 for n in lens), max_seqs=rows)
    alone = {k: whole(m, v) for k, v in reqs.items()}
    tail = 6
    got = run_schedule(m, reqs, [[(k, len(v) - tail) for k, v in reqs.items()]] + [[(k, 1) for k in reqs]] * tail)
    m.free()
    oracle = PlainTudasun(cfg, W)
    for k, v in reqs.items():
        check_logits(got[k], alone[k], "bfloat16")
        check_logits(alone[k], oracle.run(v)[0], "bfloat16")


# ---- generation through the engine's own loop, and the command line ---------------------------------------------------------------
def plain_greedy(cfg, W, prompt, n_new):
    oracle = PlainTudasun(cfg, W)
    st = oracle.new_state()
    for t in prompt:
        z, _ = oracle.token(st, t)
    out = []
    for _ in range(n_new):
        out.append(int(np.argmax(z)))
        z, _ = oracle.token(st, out[-1])
    return out


def test_greedy_generation_continuous_batching():
    """Six requests through two slots and a pool that holds about two of them: admission, portions of prompts beside decoded
    tokens, and slots / pages handed on, all inside the engine's generation loop."""
    W = random_weights(HYBRID, seed=18)
    prompts = [tokens(n, HYBRID["vocab"], 70 + i) for i, n in enumerate([5, 40, 90, 1, 64, 23])]
    want = [plain_greedy(HYBRID, W, p, 12) for p in prompts]
    m = build_engine(HYBRID, W, "float32", max_tokens=256, max_seqs=2)
    got = m.generate(prompts, 12, step_tokens=48)
    m.free()
    assert got == want


def test_command_line_generate_and_trace_replay(tmp_path):
    from turboinfer_b200.safetensors_io import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = make_config([gla_layer(mlp=moe()), latent_layer(mlp=dense(24)), hgrn2_layer(), latent_layer(kv_from=1)], vocab=53)
    W = random_weights(cfg, seed=19)
    folder = os.path.join(tmp_path, "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(public_config(cfg), f)
    write_safetensors(os.path.join(folder, "model.safetensors"), W)
    prompts = [tokens(7, 53, 3), tokens(30, 53, 4)]
    want = [plain_greedy(cfg, W, p, 6) for p in prompts]
    cmd = [sys.executable, os.path.join(root, "bin", "generate"), "--model", folder, "--dtype", "float32", "--max-new", "6"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(str(t) for t in p)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    assert [json.loads(line)["tokens"] for line in res.stdout.splitlines() if line.startswith("{")] == want
    out = os.path.join(tmp_path, "out")
    os.makedirs(out)
    p = prompts[1]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": p[:11], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": p[11:13], "want": []}, {"id": "b", "tokens": prompts[0], "want": [6]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": p[13:], "want": [0, len(p) - 14]}], "end": ["a"]}]
    res = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out,
                          "--max-tokens", "128"], input="".join(json.dumps(x) + "\n" for x in steps), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    assert [ln for ln in res.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out, "0.f32"))
    oracle = PlainTudasun(cfg, W)
    ref_a, ref_b = oracle.run(p)[0], oracle.run(prompts[0])[0]
    l1 = np.fromfile(os.path.join(out, "1.f32"), "<f4").reshape(1, 53)
    l2 = np.fromfile(os.path.join(out, "2.f32"), "<f4").reshape(2, 53)
    assert rel_err(l1, ref_b[[6]]) < TOL["float32"]
    assert rel_err(l2, ref_a[[13, len(p) - 1]]) < TOL["float32"]


def test_errors_are_reported():
    cfg = make_config([latent_layer(), latent_layer(kv_from=0)])
    W = random_weights(cfg, seed=20)
    bad = dict(W)
    bad["l0.mix.uk"] = W["l0.mix.uk"][:-1]
    with pytest.raises(Exception):
        build_engine(cfg, bad)
    with pytest.raises(Exception):   # a layer cannot read the cache of a layer behind it
        build_engine(make_config([latent_layer(kv_from=1), latent_layer()]), W)
    with pytest.raises(Exception):   # ... nor of a layer that has no cache of its own
        build_engine(make_config([latent_layer(), latent_layer(kv_from=0), latent_layer(kv_from=1)]), W)
