"""The `Domilix` design in the config-driven stack (llm_decoder.hybrid: post-norm wiring, LatentAttentionMixer, gated
dense layers, routed experts weighted on their output; csrc/latent_attention.cu, seq_ops.cu, moe_ops.cu) against the
plain float64 oracle (oracle/domilix_ref.py), on small random models of its own making.

The engine's logits at a position must equal the oracle's full recomputation whatever the cut into steps, the batch
around it, and the pages / slots in use."""
import json
import math
import os
import random
import subprocess

import pytest
import torch

from oracle import domilix_ref as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 4e-4      # max abs error of float32 logits (magnitude of a few units)
BF16_TOL = 0.08     # relative rms error of bfloat16 logits (five layers of two normed sublayers each)


def _model(config, weights, dtype="float32", max_tokens=1024, max_seqs=4, tile_size=16):
    import llm_decoder as ld
    return ld.HybridDecoder(config, weights, dtype, max_tokens=max_tokens, max_seqs=max_seqs, tile_size=tile_size)


def _tokens(n, vocab, seed):
    rnd = random.Random(seed)
    return [rnd.randrange(vocab) for _ in range(n)]


_ORACLE = {}


def _oracle(key, config, weights, tokens):
    k = (key, tuple(tokens))
    if k not in _ORACLE:
        _ORACLE[k] = R.forward(config, weights, tokens)[0]
    return _ORACLE[k]


def _close(got, want, dtype="float32"):
    got, want = got.double().cpu(), want.double()
    if dtype == "float32":
        err = (got - want).abs().max().item()
        assert err < F32_TOL, f"max abs error {err}"
    else:
        # per position; a router decision that bfloat16 rounding flips moves a few positions by much more than rounding
        # does, so the bound is on four positions out of five (float32 carries the exact comparison)
        got, want = got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1])
        rel = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()
        q = rel.sort().values[int(0.8 * (rel.numel() - 1))].item()
        assert q < BF16_TOL, f"relative rms error {q} (80th percentile of the positions)"
        assert rel.max().item() < 1.0


def _feed(engine, rid, tokens, cuts):
    """Feed `tokens` of one request in portions ending at `cuts`; returns logits of ALL positions."""
    outs, lo = [], 0
    for hi in list(cuts) + [len(tokens)]:
        if hi > lo:
            outs.append(engine.step([(rid, tokens[lo:hi], list(range(hi - lo)))]))
            lo = hi
    return torch.cat(outs, 0)


# ---- configurations: sizes and constants unlike each other; rot.dims below rot_dim; more heads than a CTA's rows; top = 1
# and top = experts; widths that are no multiple of 8 ------------------------------------------------------------------
def cfg_attention_only():
    return R.make_config([R.latent_layer()], width=64)


def cfg_dense():
    return R.make_config([R.latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=24, q_rank=16, mlp=R.dense_mlp(80))], width=48)


def cfg_moe():
    return R.make_config([R.latent_layer(heads=2, dim=8, rot_dim=4, vdim=16, kv_rank=32, q_rank=24, mlp=R.moe_mlp(7, 3, 24))], width=40)


def cfg_full():
    """Two pools: layer 1 borrows layer 0's, layers 3 and 4 borrow layer 2's (other sizes, other rotation)."""
    a = dict(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=48, base=1000.0)
    b = dict(heads=5, dim=8, rot_dim=12, vdim=16, kv_rank=72, q_rank=32, base=50.0)
    layers = [R.latent_layer(**a, mlp=R.dense_mlp(96)), R.latent_layer(**a, kv_from=0, mlp=R.moe_mlp(6, 2, 40)),
              R.latent_layer(**b, mlp=R.moe_mlp(5, 5, 16)), R.latent_layer(**b, kv_from=2, mlp=None),
              R.latent_layer(**b, kv_from=2, mlp=R.moe_mlp(9, 1, 24))]
    layers[2]["mixer"]["rot"]["dims"] = 8          # only the first 8 of the 12 entries turn
    layers[3]["mixer"]["rot"]["dims"] = 8
    layers[4]["mixer"]["rot"]["dims"] = 8
    return R.make_config(layers, width=64, vocab=97)


def cfg_wide_heads():
    """40 heads (two chunks of a CTA's 32 rows), a latent of 130 (five 32-column groups), odd width."""
    return R.make_config([R.latent_layer(heads=40, dim=4, rot_dim=2, vdim=6, kv_rank=130, q_rank=20, mlp=R.dense_mlp(30))],
                         width=50, vocab=61, embed_scale=1.0)


CONFIGS = {"attention_only": cfg_attention_only, "dense": cfg_dense, "moe": cfg_moe, "full": cfg_full,
           "wide_heads": cfg_wide_heads}


def _case(name, seed=0):
    config = CONFIGS[name]()
    return config, R.random_weights(config, seed)


# ------------------------------------------------------------------------------------------------------------ CPU tests
def test_oracle_attention_loop_equals_matrix_form():
    config, W = _case("full")
    toks = _tokens(19, config["vocab"], 1)
    a, la = R.forward(config, W, toks, fast_attention=False)
    b, lb = R.forward(config, W, toks, fast_attention=True)
    assert (a - b).abs().max() < 1e-9 and (la - lb).abs().max() < 1e-9


def test_oracle_prefix_property():
    """Causality of the oracle itself: the logits of a prefix do not change when tokens follow."""
    config, W = _case("full")
    toks = _tokens(30, config["vocab"], 2)
    full = R.forward(config, W, toks)[0]
    assert (R.forward(config, W, toks[:11])[0] - full[:11]).abs().max() < 1e-9


def test_oracle_rotation_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(12, generator=g, dtype=torch.float64), torch.randn(12, generator=g, dtype=torch.float64)
    dot = lambda a, b: float((R.rotate_pairs(q, a, 100.0, 8) * R.rotate_pairs(k, b, 100.0, 8)).sum())  # noqa: E731
    assert abs(dot(37, 30) - dot(7, 0)) < 1e-9 and abs(dot(37, 30) - dot(37, 29)) > 1e-3
    assert torch.equal(R.rotate_pairs(q, 5, 100.0, 8)[8:], q[8:])          # entries past rot.dims pass unchanged


def test_oracle_router_weights():
    g = torch.Generator().manual_seed(1)
    h = torch.randn(1, 6, generator=g, dtype=torch.float64)
    wr, b = torch.randn(4, 6, generator=g, dtype=torch.float64), torch.tensor([0., 0., 50., 0.], dtype=torch.float64)
    eye = [(torch.eye(6, dtype=torch.float64), torch.eye(6, dtype=torch.float64))] * 4
    out = R.moe_ff(h, wr, b, eye, 1)
    assert torch.allclose(out, torch.relu(h) ** 2)                          # one expert chosen: weight exactly 1
    ex = [(torch.eye(6, dtype=torch.float64), torch.eye(6, dtype=torch.float64) * (e + 1)) for e in range(4)]
    z = (wr @ h[0]) + b
    top2 = z.topk(2).indices.tolist()
    w = torch.softmax(z[top2], 0)
    want = sum(w[i] * (top2[i] + 1) for i in range(2)) * torch.relu(h) ** 2
    assert top2[0] == 2 and torch.allclose(R.moe_ff(h, wr, b, ex, 2), want)


def test_registry_names_the_design():
    from llm_decoder.hybrid import DESIGNS, FEED_FORWARDS, MIXERS
    from llm_decoder.registry import MODEL_REGISTRY
    assert "Domilix" in MODEL_REGISTRY and "Domilix" in DESIGNS and "Megusun" in DESIGNS
    assert "latent_attention" in MIXERS and set(DESIGNS["Domilix"]["ff"]) <= set(FEED_FORWARDS)


# ------------------------------------------------------------------------------------------------------------ GPU tests
@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_each_mechanism(name, dtype):
    import llm_decoder as ld
    config, W = _case(name)
    toks = _tokens(70, config["vocab"], 3)
    eng = ld.Engine(_model(config, W, dtype))
    _close(_feed(eng, "a", toks, []), _oracle(name, config, W, toks), dtype)


@pytest.mark.gpu
def test_residual_after_every_layer():
    import llm_decoder as ld
    config, W = _case("full")
    toks = _tokens(33, config["vocab"], 6)
    model = _model(config, W)
    seen = []
    model.layer_hook = lambda x: seen.append(x.double().cpu())
    ld.Engine(model).step([("a", toks, [])])
    want = R.forward(config, W, toks)[1]
    assert len(seen) == len(config["layers"])
    for i, x in enumerate(seen):
        assert (x - want[i]).abs().max() < 2e-4, f"layer {i}"


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["full", "attention_only", "moe", "wide_heads"])
def test_prefill_equals_token_by_token(name):
    import llm_decoder as ld
    config, W = _case(name)
    toks = _tokens(45, config["vocab"], 4)
    eng = ld.Engine(_model(config, W))
    _close(_feed(eng, "a", toks, range(1, 45)), _oracle(name, config, W, toks))      # every token a step of its own


@pytest.mark.gpu
@pytest.mark.parametrize("cuts", [[2, 4, 6, 9, 40], [15, 16, 17, 31, 33, 48, 64, 66], [1, 80], [63], [7, 8, 9, 23, 24, 25]])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_many_sizes(cuts, dtype):
    """Cuts at, before and after page borders (16 tokens) and the attention kernels' key steps (32, 64), down to two
    tokens."""
    import llm_decoder as ld
    config, W = _case("full")
    toks = _tokens(90, config["vocab"], 5)
    eng = ld.Engine(_model(config, W, dtype))
    _close(_feed(eng, "a", toks, cuts), _oracle("full", config, W, toks), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_of_unequal_requests(dtype):
    """Four requests of unequal length advance together: portions next to single tokens, one sitting out a step."""
    import llm_decoder as ld
    config, W = _case("full")
    reqs = {r: _tokens(n, config["vocab"], 10 + i) for i, (r, n) in enumerate([("a", 70), ("b", 33), ("c", 5), ("d", 51)])}
    plan = [[("a", 40), ("b", 2)], [("a", 1), ("b", 17), ("c", 5)], [("a", 1), ("d", 30)], [("a", 1), ("b", 1), ("d", 1)],
            [("b", 13), ("d", 20), ("a", 27)]]
    eng = ld.Engine(_model(config, W, dtype))
    at = {r: 0 for r in reqs}
    got = {r: [] for r in reqs}
    for step in plan:
        entries = []
        for r, n in step:
            entries.append((r, reqs[r][at[r]:at[r] + n], list(range(n))))
            at[r] += n
        out = eng.step(entries)
        o = 0
        for r, n in step:
            got[r].append(out[o:o + n])
            o += n
    for r in reqs:
        assert at[r] == len(reqs[r])
        _close(torch.cat(got[r], 0), _oracle("full", config, W, reqs[r]), dtype)


@pytest.mark.gpu
def test_slots_and_pages_are_used_again():
    """A pool of 160 tokens and two slots serves six requests one after another and interleaved: freed pages and slots
    come back (dirty) and the next request must not see what they held -- in the borrowed pools either."""
    import llm_decoder as ld
    config, W = _case("full")
    model = _model(config, W, max_tokens=160, max_seqs=2)
    assert len(model.states._kv) == 2                  # five layers, two pools
    eng = ld.Engine(model)
    seqs = [_tokens(n, config["vocab"], 20 + i) for i, n in enumerate([90, 60, 33, 100, 17, 59])]
    out = eng.step([("r0", seqs[0][:50], list(range(50))), ("r1", seqs[1][:10], list(range(10)))])
    g0, g1 = [out[:50]], [out[50:]]
    out = eng.step([("r1", seqs[1][10:], list(range(50))), ("r0", seqs[0][50:], list(range(40)))])
    g1.append(out[:50])
    g0.append(out[50:])
    _close(torch.cat(g0), _oracle("full", config, W, seqs[0]))
    _close(torch.cat(g1), _oracle("full", config, W, seqs[1]))
    assert model.states.free_slots() == 0 and model.states.free_tokens() == 0
    with pytest.raises(RuntimeError):
        eng.step([("r2", [1], [0])])                 # no slot left
    with pytest.raises(RuntimeError):
        eng.step([("r0", [1] * 7, [0])])             # 97 tokens need a seventh tile: an error, not an eviction
    eng.finish("r0")
    eng.finish("r1")
    assert model.states.free_slots() == 2 and model.states.free_tokens() == 160
    for i in (2, 3, 4, 5):
        _close(_feed(eng, f"r{i}", seqs[i], [len(seqs[i]) // 2]), _oracle("full", config, W, seqs[i]))
        eng.finish(f"r{i}")


def _sharp(W, factor=5.0):
    """Queries scaled up: the softmax concentrates on its best key, so one wrong, missing or extra key (typically a far
    one) moves the output by O(1) instead of O(1/n)."""
    W = dict(W)
    for k in list(W):
        if k.endswith("mix.uq"):
            W[k] = (W[k].float() * factor).to(torch.bfloat16)
    return W


@pytest.mark.gpu
@pytest.mark.parametrize("tile_size", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_and_page_borders_sharp_attention(tile_size, dtype):
    """300 tokens, peaked attention: prompts cut around page borders, then 40 decoded tokens crossing two more."""
    import llm_decoder as ld
    config = R.make_config([R.latent_layer(heads=4, dim=16, rot_dim=8, vdim=32, kv_rank=48, q_rank=40, base=300.0),
                            R.latent_layer(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=48, q_rank=24, base=300.0, kv_from=0)],
                           width=64, vocab=80)
    W = _sharp(R.random_weights(config, 7))
    toks = _tokens(300, config["vocab"], 8)
    want = R.forward(config, W, toks)[0]
    eng = ld.Engine(_model(config, W, dtype, tile_size=tile_size))
    cuts = [63, 64, 65, 127, 129, 192, 255, 256] + list(range(260, 300))
    _close(_feed(eng, "a", toks, cuts), want, dtype)
    eng.finish("a")
    eng = ld.Engine(_model(config, W, dtype, tile_size=tile_size))
    _close(_feed(eng, "b", toks, [5, 290]), want, dtype)


@pytest.mark.gpu
def test_single_far_key_stands_out():
    """A model built so that ONE key far back carries almost all the weight for the last query: a rank-one term added to
    the key map sends the needle token's latent onto the probe token's (unrotated) query."""
    import llm_decoder as ld
    config = R.make_config([R.latent_layer(heads=1, dim=8, rot_dim=2, vdim=16, kv_rank=16, q_rank=12, scale=1.0)],
                           width=32, vocab=40, embed_scale=1.5)
    W = R.random_weights(config, 9)
    needle, probe = 7, 11
    D = {k: v.double() for k, v in W.items()}
    x = D["embed"][[needle, probe]] * 1.5
    c = R.latent_kv(x, D["l0.mix.dkv"], D["l0.mix.dkv.norm"], 16, config["layers"][0]["mixer"]["rot"], 1e-5)[0][0]
    qp = (R.weighted_rms_norm(x[1] @ D["l0.mix.dq"].T, D["l0.mix.dq.norm"], 1e-5) @ D["l0.mix.uq"].T)[:8]
    W["l0.mix.uk"] = (D["l0.mix.uk"] * 0.1 + 14.0 * torch.outer(qp / (qp @ qp), c / (c @ c))).to(torch.bfloat16)
    others = [t for t in range(40) if t not in (needle, probe)]
    rnd = random.Random(3)
    for needle_at in (0, 15, 16, 17, 31, 32, 140):
        toks = [rnd.choice(others) for _ in range(200)] + [probe]
        toks[needle_at] = needle
        want = R.forward(config, W, toks)[0]
        without = list(toks)
        without[needle_at] = others[0]
        assert (R.forward(config, W, without)[0][-1] - want[-1]).abs().max() > 0.3       # the needle matters
        eng = ld.Engine(_model(config, W))
        got = _feed(eng, "a", toks, [150, 200])                                             # probe decoded alone
        _close(got[-1], want[-1])
        _close(got[:-1], want[:-1])


@pytest.mark.gpu
def test_first_tokens():
    import llm_decoder as ld
    config, W = _case("full")
    for n in (1, 2, 3):
        toks = _tokens(n, config["vocab"], 30 + n)
        eng = ld.Engine(_model(config, W))
        _close(_feed(eng, "a", toks, []), _oracle("full", config, W, toks))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_split_keys(dtype):
    """A 560-token portion followed by 150 decoded tokens: single tokens over a long context take the split-key path,
    the same positions inside the portion do not."""
    import llm_decoder as ld
    config, W = _case("full")
    toks = _tokens(710, config["vocab"], 40)
    eng = ld.Engine(_model(config, W, dtype))
    got = _feed(eng, "a", toks, [560] + list(range(561, 710)))
    _close(got, _oracle("full", config, W, toks), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype):
    """Scheduler: five prompts of unequal length on four slots with a small token budget (chunked prompts, continuous
    batching, slot reuse); greedy tokens equal the oracle's argmax at every step (float32), and the teacher-forced
    logits stay close (bfloat16)."""
    import llm_decoder as ld
    config, W = _case("full")
    prompts = [_tokens(n, config["vocab"], 50 + i) for i, n in enumerate([37, 5, 64, 18, 2])]
    model = _model(config, W, dtype, max_tokens=512, max_seqs=4)
    outs = ld.generate(model, prompts, 12, max_batch_tokens=48)
    for p, o in zip(prompts, outs):
        assert o[:len(p)] == p and len(o) == len(p) + 12
        logits = R.forward(config, W, o[:-1])[0]
        if dtype == "float32":
            for t in range(len(p) - 1, len(o) - 1):
                top2 = logits[t].topk(2).values
                if float(top2[0] - top2[1]) > 1e-3:                 # no test on a near tie
                    assert int(logits[t].argmax()) == o[t + 1]
        else:
            chosen = torch.tensor([logits[t, o[t + 1]] for t in range(len(p) - 1, len(o) - 1)])
            best = logits[len(p) - 1:len(o) - 1].max(-1).values
            assert float((best - chosen).max()) < 0.4               # the chosen token is (nearly) the oracle's best: two
            #                                                         bfloat16 logits, each off by up to ~0.15 here


def _random_config(rnd):
    """Layer count, order, which layers borrow which pool, every size and constant drawn at random."""
    layers, owners, shapes = [], [], {}
    for i in range(rnd.randint(2, 6)):
        mlp = rnd.choice([None, "dense", "moe", "moe"])
        if mlp == "dense":
            mlp = R.dense_mlp(rnd.choice([24, 64, 100, 37]))
        elif mlp == "moe":
            experts = rnd.randint(2, 12)
            mlp = R.moe_mlp(experts, rnd.randint(1, experts), rnd.choice([8, 16, 24, 30]))
        own = dict(heads=rnd.randint(1, 9), dim=rnd.choice([8, 16, 24, 12]), vdim=rnd.choice([8, 16, 40, 20]), q_rank=rnd.choice([16, 24, 48, 30]))
        if owners and rnd.random() < 0.5:
            j = rnd.choice(owners)
            layers.append(R.latent_layer(**{**shapes[j], **own}, kv_from=j, mlp=mlp, scale=rnd.uniform(0.1, 0.4)))
        else:
            shapes[i] = dict(own, rot_dim=rnd.choice([2, 4, 8, 16, 24]), kv_rank=rnd.choice([16, 24, 48, 64, 72, 136, 30]),
                             base=rnd.choice([50.0, 1000.0, 20000.0]))
            owners.append(i)
            layers.append(R.latent_layer(**shapes[i], mlp=mlp, scale=rnd.uniform(0.1, 0.4)))
    return R.make_config(layers, width=rnd.choice([40, 64, 72, 96, 50, 128, 200]), vocab=rnd.choice([61, 97, 128]),
                         eps=rnd.choice([1e-5, 1e-6]), embed_scale=rnd.uniform(0.5, 3.0))


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(6))
def test_random_configurations_in_random_schedules(seed):
    """Three requests of a randomly drawn model advance in random portions (1 to 100 tokens, some sitting out) through
    one engine; float32 against the oracle at every position, bfloat16 finite and equal to its own whole-prompt run up
    to rounding."""
    import llm_decoder as ld
    rnd = random.Random(seed)
    config = _random_config(rnd)
    W = R.random_weights(config, seed)
    reqs = {r: _tokens(n, config["vocab"], 100 * seed + i)
            for i, (r, n) in enumerate((("a", rnd.randint(120, 300)), ("b", rnd.randint(2, 90)), ("c", rnd.randint(1, 40))))}
    plan, at = [], {r: 0 for r in reqs}
    while any(at[r] < len(reqs[r]) for r in reqs):
        step = []
        for r in reqs:
            left = len(reqs[r]) - at[r]
            if left and rnd.random() < 0.8:
                n = min(left, rnd.choice([1, 1, 2, 3, 17, 64, 100]))
                step.append((r, at[r], n))
                at[r] += n
        if step:
            plan.append(step)
    outs = {}
    for dtype in ("float32", "bfloat16"):
        eng = ld.Engine(_model(config, W, dtype, max_tokens=640, max_seqs=3))
        got = {r: [] for r in reqs}
        for step in plan:
            out = eng.step([(r, reqs[r][lo:lo + n], list(range(n))) for r, lo, n in step])
            o = 0
            for r, _lo, n in step:
                got[r].append(out[o:o + n])
                o += n
        outs[dtype] = {r: torch.cat(got[r]) for r in reqs}
    for r in reqs:
        _close(outs["float32"][r], R.forward(config, W, reqs[r])[0])
        whole = ld.Engine(_model(config, W, "bfloat16", max_tokens=640, max_seqs=3)).step([(r, reqs[r], list(range(len(reqs[r]))))])
        b16 = outs["bfloat16"][r].double().cpu()
        assert torch.isfinite(b16).all()
        rel = (b16 - whole.double().cpu()).pow(2).mean(-1).sqrt() / whole.double().cpu().pow(2).mean(-1).sqrt()
        assert rel.sort().values[int(0.8 * (rel.numel() - 1))].item() < BF16_TOL


@pytest.mark.gpu
def test_trace_runner_and_generate_cli(tmp_path):
    """bin/trace_run and bin/generate on a model folder: registry -> engine -> files."""
    import numpy as np
    from llm_decoder.safetensors_io import save_file
    config, W = _case("full")
    mdir = tmp_path / "model"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(config))
    save_file(W, str(mdir / "model.safetensors"))
    a, b = _tokens(40, config["vocab"], 70), _tokens(21, config["vocab"], 71)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": []}, {"id": "b", "tokens": b, "want": [20]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:], "want": [8]}], "end": ["a"]}]
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                       capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = R.forward(config, W, a)[0], R.forward(config, W, b)[0]
    V = config["vocab"]
    g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, V))
    g1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V))
    g2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, V))
    _close(g0, wa[[0, 29]])
    _close(g1, wb[[20]])
    _close(g2, wa[[39]])
    p = subprocess.run([os.path.join(ROOT, "bin", "generate"), "--model", str(mdir), "--dtype", "bfloat16", "--prompt",
                        ",".join(map(str, a[:10])), "--max-new-tokens", "4"], text=True, capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    ids = [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]
    assert ids[:10] == a[:10] and len(ids) == 14


@pytest.mark.gpu
def test_config_errors_are_reported():
    config, W = _case("full")
    bad = json.loads(json.dumps(config))
    bad["layers"][1]["mixer"]["kv_from"] = 1           # a layer without a pool of its own
    with pytest.raises(ValueError):
        _model(bad, W)
    bad = json.loads(json.dumps(config))
    bad["layers"][3]["mixer"]["kv_from"] = 0           # other kv_rank than the pool's
    with pytest.raises(ValueError):
        _model(bad, W)


# ---- kernels alone ----------------------------------------------------------------------------------------------------
def _lib():
    from llm_decoder import _cabi
    return _cabi, _cabi.lib(), torch.device("cuda"), _cabi.stream


@pytest.mark.gpu
@pytest.mark.parametrize("elem", [4, 2])
def test_rotation_and_latent_append_kernels(elem):
    """pa_rope_table + pa_rope_rows + pa_latent_kv_append against rotate_pairs / latent_kv at scattered positions (far ones
    too: the angles are exact where float32 products of position and frequency would not be)."""
    cabi, lib, dev, s = _lib()
    dt = torch.float32 if elem == 4 else torch.bfloat16
    g = torch.Generator().manual_seed(5)
    rows, heads, hd, dims, rot_dim, kv_rank, base = 9, 3, 14, 6, 8, 20, 700.0
    pos = torch.tensor([0, 1, 2, 15, 16, 17, 1000, 40000, 31], dtype=torch.int32)
    table = torch.empty(rows, dims // 2, 2, device=dev)
    posd = pos.to(dev)
    cabi.check(lib.pa_rope_table(posd.data_ptr(), rows, dims, base, table.data_ptr(), s()), "table")
    x = torch.randn(rows, 5 + heads * hd, generator=g).to(dt)
    xd = x.to(dev)
    cabi.check(lib.pa_rope_rows(xd.data_ptr(), xd.stride(0), 5 + 4, hd, heads, dims, table.data_ptr(), rows, elem, s()), "rope")
    want = x.double().clone()
    for r in range(rows):
        for h in range(heads):
            o = 5 + h * hd + 4
            want[r, o:o + dims] = R.rotate_pairs(x[r, o:o + dims].double(), int(pos[r]), base, dims)
    tol = 2e-6 if elem == 4 else 1e-2
    assert (xd.cpu().double() - want).abs().max() < tol
    # append: 3 slots x 4 tiles of 16, one row per position; the table maps (slot, tile) -> page
    tile, ntiles, slots, kd = 16, 2600, 2, kv_rank + rot_dim
    pool = torch.zeros(8, tile, kd, dtype=dt, device=dev)
    tbl = torch.full((slots, ntiles), -1, dtype=torch.int32)
    slot = torch.tensor([0, 0, 0, 0, 1, 1, 1, 0, 1], dtype=torch.int32)
    pages = {}
    for r in range(rows):
        key = (int(slot[r]), int(pos[r]) // tile)
        pages.setdefault(key, len(pages))
        tbl[key] = pages[key]
    src = torch.randn(rows, 3 + kd, generator=g).to(dt)
    gain = torch.rand(kv_rank, generator=g) + 0.5
    tbld, srcd, gaind, slotd = tbl.to(dev), src.to(dev), gain.to(dev), slot.to(dev)
    cabi.check(lib.pa_latent_kv_append(pool.data_ptr(), tbld.data_ptr(), slots, ntiles, 8, tile, kv_rank, rot_dim, dims,
                                       srcd.data_ptr(), src.stride(0), 3, gaind.data_ptr(), 1e-5, table.data_ptr(),
                                       slotd.data_ptr(), posd.data_ptr(), rows, elem, s()), "append")
    got = pool.cpu().double()
    for r in range(rows):
        row = got[pages[(int(slot[r]), int(pos[r]) // tile)], int(pos[r]) % tile]
        c = R.weighted_rms_norm(src[r, 3:3 + kv_rank].double(), gain.double(), 1e-5)
        kr = R.rotate_pairs(src[r, 3 + kv_rank:].double(), int(pos[r]), base, dims)
        assert (row - torch.cat([c, kr])).abs().max() < (1e-5 if elem == 4 else 3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("elem", [4, 2])
@pytest.mark.parametrize("heads,K,N,rows", [(3, 16, 40, 70), (1, 7, 5, 3), (5, 130, 66, 129)])
def test_head_linear_and_gate_kernels(elem, heads, K, N, rows):
    cabi, lib, dev, s = _lib()
    dt = torch.float32 if elem == 4 else torch.bfloat16
    g = torch.Generator().manual_seed(K)
    x = torch.randn(rows, heads * (K + 3), generator=g).to(dt)             # head h's K values start at h * (K + 3) + 2
    w = (torch.randn(heads, K, N, generator=g) / math.sqrt(K)).to(dt)
    out = torch.empty(rows, heads * N, dtype=dt, device=dev)
    xd = x.to(dev)
    wdev = w.to(dev)
    cabi.check(lib.pa_head_linear(xd.data_ptr() + 2 * elem, xd.stride(0), K + 3, wdev.data_ptr(), heads, K, N, rows,
                                  out.data_ptr(), heads * N, N, elem, s()), "head_linear")
    want = torch.einsum("rhk,hkn->rhn", x.double().view(rows, heads, K + 3)[:, :, 2:2 + K], w.double())
    tol = 1e-5 if elem == 4 else 2e-2
    assert (out.cpu().double().view(rows, heads, N) - want).abs().max() < tol * max(1.0, want.abs().max().item())
    gate = torch.randn(rows, heads + 4, generator=g).to(dt)
    gd = gate.to(dev)
    og = torch.empty(rows, heads * N, dtype=dt, device=dev)
    cabi.check(lib.pa_head_gate(out.data_ptr(), heads * N, N, gd.data_ptr() + 4 * elem, gd.stride(0), heads, N, rows,
                                og.data_ptr(), elem, s()), "head_gate")
    wantg = out.cpu().double().view(rows, heads, N) * torch.sigmoid(gate.double()[:, 4:, None])
    assert (og.cpu().double().view(rows, heads, N) - wantg).abs().max() < tol * max(1.0, wantg.abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("width,experts,top,elem", [(64, 8, 2, 2), (72, 11, 3, 2), (50, 4, 4, 2), (36, 9, 1, 4), (37, 3, 2, 4)])
def test_router_softmax_over_the_chosen_logits(width, experts, top, elem):
    cabi, lib, dev, s = _lib()
    g = torch.Generator().manual_seed(width)
    rows = 45
    dt = torch.bfloat16 if elem == 2 else torch.float32
    h = torch.randn(rows, width, generator=g).to(dt)
    wr, b = torch.randn(experts, width, generator=g) / math.sqrt(width), torch.randn(experts, generator=g) * 2
    z = h.double() @ wr.double().T + b.double()
    tv, ti = z.topk(top, -1)
    sel_id, sel_w = torch.empty(rows * top, dtype=torch.int32, device=dev), torch.empty(rows * top, device=dev)
    hd, wrd, bd = h.to(dev), wr.to(dev), b.to(dev)
    cabi.check(lib.pa_router_topk(hd.data_ptr(), wrd.data_ptr(), bd.data_ptr(), None, rows, width, experts, top, 2, 0,
                                  sel_id.data_ptr(), sel_w.data_ptr(), None, elem, s()), "router")
    assert torch.equal(sel_id.cpu().view(rows, top).long(), ti)
    assert (sel_w.cpu().view(rows, top).double() - torch.softmax(tv, -1)).abs().max() < 1e-5
    assert (sel_w.cpu().view(rows, top).sum(-1) - 1).abs().max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("rows,experts,top,width,ff,elem", [(300, 4, 2, 64, 48, 2), (300, 4, 2, 64, 48, 4), (20, 6, 3, 72, 40, 2),
                                                              (33, 5, 1, 50, 30, 2), (33, 5, 5, 50, 30, 4)])
def test_plain_experts_with_squared_relu(rows, experts, top, width, ff, elem):
    """pa_moe_up (no gate, relu squared) + pa_moe_down + the weighted sum inside pa_residual_add_norm, on the float kernel,
    the tiled tensor-core kernel (many pairs per expert), the streaming one (few) and the scalar fallback (odd width)."""
    cabi, lib, dev, s = _lib()
    dt = torch.bfloat16 if elem == 2 else torch.float32
    g = torch.Generator().manual_seed(rows + ff)
    h = torch.randn(rows, width, generator=g).to(dt)
    wu = (torch.randn(experts, ff, width, generator=g) / math.sqrt(width)).to(dt)
    wd = (torch.randn(experts, width, ff, generator=g) / math.sqrt(ff)).to(dt)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).to(torch.int32)
    wts = torch.softmax(torch.randn(rows, top, generator=g), -1)
    pairs = rows * top
    sel_id, sel_w = ids.reshape(-1).to(dev), wts.reshape(-1).to(dev)
    order = torch.empty(pairs, dtype=torch.int32, device=dev)
    meta = torch.empty(lib.pa_moe_meta_ints(pairs, experts), dtype=torch.int32, device=dev)
    cabi.check(lib.pa_moe_sort(sel_id.data_ptr(), pairs, experts, order.data_ptr(), meta.data_ptr(), s()), "sort")
    hd, wud, wdd = h.to(dev), wu.to(dev), wd.to(dev)
    act = torch.empty(pairs, ff, dtype=dt, device=dev)
    cabi.check(lib.pa_moe_up(hd.data_ptr(), hd.stride(0), wud.data_ptr(), width, ff, experts, order.data_ptr(), None, top,
                             meta.data_ptr(), pairs, 2, act.data_ptr(), elem, s()), "up")
    routed = torch.empty(pairs, width, device=dev)
    cabi.check(lib.pa_moe_down(act.data_ptr(), wdd.data_ptr(), ff, width, experts, order.data_ptr(), meta.data_ptr(), pairs,
                               routed.data_ptr(), elem, s()), "down")
    x0 = torch.randn(rows, width, generator=g)
    gain = torch.rand(width, generator=g) + 0.5
    x = x0.to(dev)
    nxt = torch.empty(rows, width, dtype=dt, device=dev)
    gaind = gain.to(dev)
    cabi.check(lib.pa_residual_add_norm(x.data_ptr(), rows, width, 1e-5, gaind.data_ptr(), None, routed.data_ptr(),
                                        sel_w.data_ptr(), top, nxt.data_ptr(), elem, s()), "add_norm")
    want = torch.zeros(rows, width, dtype=torch.float64)
    for r in range(rows):
        for k in range(top):
            e = int(ids[r, k])
            want[r] += wts[r, k].double() * (wd[e].double() @ torch.relu(wu[e].double() @ h[r].double()) ** 2)
    want = x0.double() + R.weighted_rms_norm(want, gain.double(), 1e-5)
    tol = 2e-5 if elem == 4 else 3e-2
    assert (x.cpu().double() - want).abs().max() < tol
    assert (nxt.cpu().double() - x.cpu().double()).abs().max() < (1e-6 if elem == 4 else 3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("elem", [4, 2])
@pytest.mark.parametrize("ff", [19, 24])
def test_gated_relu_product_kernel(elem, ff):
    """ff = 24: the bfloat16 form that takes eight values per thread; 19: the element-wise one."""
    cabi, lib, dev, s = _lib()
    dt = torch.bfloat16 if elem == 2 else torch.float32
    gu = torch.randn(37, 2 * ff, generator=torch.Generator().manual_seed(2)).to(dt)
    out = torch.empty(37, ff, dtype=dt, device=dev)
    for act, fn in ((1, torch.relu), (0, torch.nn.functional.silu),
                    (2, lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))):
        gud = gu.to(dev)
        cabi.check(lib.pa_act_mul(gud.data_ptr(), 37, ff, act, out.data_ptr(), elem, s()), "act_mul")
        want = fn(gu.double()[:, :ff]) * gu.double()[:, ff:]
        assert (out.cpu().double() - want).abs().max() < (1e-5 if elem == 4 else 3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,kv_rank,rot_dim,tile_size", [(5, 72, 24, 16), (16, 512, 64, 64), (3, 136, 8, 16), (70, 40, 0, 16),
                                                             (1, 8, 16, 32)])
def test_latent_attention_kernels_alone(heads, kv_rank, rot_dim, tile_size):
    """pa_latent_attention on a pool with scattered pages: the float kernel (float and bfloat16 rows) and the tensor-core
    kernel, portions of several lengths and single tokens over short and long contexts, with and without split keys,
    latent widths that are not a power of two, more heads than a CTA has rows, no rotated part."""
    cabi, lib, dev, s = _lib()
    g = torch.Generator().manual_seed(heads * 1000 + kv_rank)
    kd = kv_rank + rot_dim
    # (slot, tokens held before, new tokens)
    seqs = [(0, 0, 70), (1, 300, 1), (2, 129, 33), (3, 63, 2), (4, 700, 1)]
    ntiles = 64
    pages_needed = sum((before + n + tile_size - 1) // tile_size for _s, before, n in seqs)
    perm = torch.randperm(pages_needed + 3, generator=g).tolist()
    table = torch.full((5, ntiles), -1, dtype=torch.int32)
    pool = torch.randn(pages_needed + 3, tile_size, kd, generator=g)
    used = 0
    for slot, before, n in seqs:
        for t in range((before + n + tile_size - 1) // tile_size):
            table[slot, t] = perm[used]
            used += 1
    R_ = sum(n for _s, _b, n in seqs)
    ql = torch.randn(R_, heads, kv_rank, generator=g) * 0.3
    qr = torch.randn(R_, heads, max(rot_dim, 1), generator=g) * 0.3
    scale = 0.35
    for elem, kind in ((4, 0), (2, 0), (2, 2), (2, 3)):
        dt = torch.float32 if elem == 4 else torch.bfloat16
        if kind >= 2 and not lib.pa_latent_attention_mma_tile_tokens(heads, kv_rank, rot_dim, elem):
            continue
        tt = lib.pa_latent_attention_mma_tile_tokens(heads, kv_rank, rot_dim, elem) if kind == 2 else lib.pa_latent_attention_tile_tokens(heads)
        tt = 1 if kind == 3 else tt                 # kind 3 promises tiles of one token (its key-split form: at most 16 heads)
        poold, qld, qrd, tabled = pool.to(dt).to(dev), ql.to(dt).to(dev), qr.to(dt).to(dev), table.to(dev)
        P, QL, QR = poold.cpu().double(), qld.cpu().double(), qrd.cpu().double()
        want = torch.zeros(R_, heads, kv_rank, dtype=torch.float64)
        tiles, r0 = [], 0
        for slot, before, n in seqs:
            keys = torch.stack([P[table[slot, j // tile_size], j % tile_size] for j in range(before + n)])
            for t in range(n):
                vis = keys[:before + t + 1]
                sc = QL[r0 + t] @ vis[:, :kv_rank].T
                if rot_dim:
                    sc = sc + QR[r0 + t][:, :rot_dim] @ vis[:, kv_rank:].T
                want[r0 + t] = torch.softmax(sc * scale, -1) @ vis[:, :kv_rank]
            for o in range(0, n, tt):
                tiles.append((r0 + o, min(tt, n - o), slot, before + o))
            r0 += n
        td = torch.tensor(tiles, dtype=torch.int32).to(dev)
        for nsplit in (1, 3):
            out = torch.zeros(R_, heads, kv_rank, dtype=dt, device=dev)
            ws = torch.empty(max(1, lib.pa_latent_attention_workspace_bytes(len(tiles), heads, kv_rank, nsplit)), dtype=torch.uint8, device=dev)
            cabi.check(lib.pa_latent_attention(qld.data_ptr(), heads * kv_rank, kv_rank, qrd.data_ptr(), qrd.stride(0), qrd.stride(1),
                                               poold.data_ptr(), tabled.data_ptr(), 5, ntiles, poold.shape[0], tile_size, td.data_ptr(),
                                               len(tiles), heads, kv_rank, rot_dim, scale, out.data_ptr(), heads * kv_rank, kv_rank,
                                               elem, nsplit, kind, ws.data_ptr(), ws.numel(), s()), "latent_attention")
            err = (out.cpu().double() - want).abs().max().item()
            assert err < (2e-5 if elem == 4 else 2e-2), (elem, kind, nsplit, err)
