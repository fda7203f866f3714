"""The config-driven hybrid stack (llm_decoder.hybrid + engine + seq_state; csrc/seq_ops.cu, diff_attention.cu,
moe_ops.cu) against the plain float64 oracle (oracle/hybrid_ref.py), on small random models of its own making.

The engine's logits at a position must equal the oracle's full recomputation whatever the cut into steps, the
batch around it, and the pages / slots in use."""
import functools
import json
import math
import os
import random
import subprocess
import sys

import pytest
import torch

from oracle import hybrid_ref as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 4e-4      # max abs error of float32 logits (magnitude of a few units)
BF16_TOL = 0.06     # relative rms error of bfloat16 logits


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


# ---- configurations: sizes and constants unlike each other, odd widths, several kv heads, top > 1 ---------------------
def cfg_mingru_only():
    return R.make_config([R.mingru_layer(40)], width=72, vocab=61, residual_mult=0.7)


def cfg_attention_only():
    return R.make_config([R.attention_layer(heads=6, kv_heads=2, dim=20, vdim=24, coef=0.5, every=8)], width=72, vocab=61)


def cfg_dense():
    return R.make_config([R.mingru_layer(32, R.dense_mlp(100))], width=48, vocab=50)


def cfg_moe():
    return R.make_config([R.mingru_layer(32, R.moe_mlp(experts=5, top=2, ff=36, shared_ff=44))], width=48, vocab=50)


def cfg_moe_no_shared():
    return R.make_config([R.attention_layer(heads=2, kv_heads=2, dim=8, vdim=40, mlp=R.moe_mlp(3, 3, 20, 0))], width=40, vocab=33)


def cfg_full():
    return R.make_config([R.attention_layer(heads=8, kv_heads=2, dim=16, vdim=40, diff=0.2, coef=0.3, every=32,
                                            mlp=R.moe_mlp(6, 2, 40, 56)),
                          R.mingru_layer(48, R.dense_mlp(96)),
                          R.mingru_layer(80, None),
                          R.attention_layer(heads=3, kv_heads=3, dim=24, vdim=16, scale=0.3, diff=0.4, coef=0.1, every=5,
                                            mlp=R.dense_mlp(64))],
                         width=64, vocab=97, eps=1e-4, residual_mult=0.4)


def cfg_wide_heads():
    # 40 query heads on one kv head: more than the 32 rows of an attention CTA; value rows wider than 128
    return R.make_config([R.attention_layer(heads=40, kv_heads=1, dim=8, vdim=136, every=3)], width=64, vocab=40)


CONFIGS = {f.__name__[4:]: f for f in (cfg_mingru_only, cfg_attention_only, cfg_dense, cfg_moe, cfg_moe_no_shared, cfg_full,
                                       cfg_wide_heads)}


@functools.lru_cache(maxsize=None)
def _case(name, seed=0):
    config = CONFIGS[name]()
    return config, R.random_weights(config, seed)


# ------------------------------------------------------------------------------------------------------------ CPU tests
def test_oracle_attention_loop_equals_matrix_form():
    config, W = _case("attention_only")
    toks = _tokens(19, config["vocab"], 1)
    a = R.forward(config, W, toks, fast_attention=False)[0]
    b = R.forward(config, W, toks, fast_attention=True)[0]
    assert (a - b).abs().max().item() < 1e-10


def test_oracle_prefix_property():
    """Causality of the oracle itself: the logits of a prefix do not change when tokens follow."""
    config, W = _case("full")
    toks = _tokens(24, config["vocab"], 2)
    a = R.forward(config, W, toks)[0]
    b = R.forward(config, W, toks[:11])[0]
    assert (a[:11] - b).abs().max().item() < 1e-10


def test_safetensors_round_trip(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "pagedattention-based-transformer-decoder-inference-framework_b200"))
    from llm_decoder.safetensors_io import load_file, save_file
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "s": torch.tensor(1.5).to(torch.bfloat16),
         "i": torch.arange(7, dtype=torch.int32), "f": torch.randn(2, 2, 2)}
    save_file(t, str(tmp_path / "m.safetensors"))
    back = load_file(str(tmp_path / "m.safetensors"))
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and back[k].shape == t[k].shape and torch.equal(back[k], t[k])


def test_registry_names_the_architectures():
    from llm_decoder.registry import MODEL_REGISTRY
    assert {"Megusun", "CUDADecoder", "INT8Decoder"} <= set(MODEL_REGISTRY)


# ------------------------------------------------------------------------------------------------------------ GPU tests
@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_each_mechanism(name, dtype):
    import llm_decoder as ld
    config, W = _case(name)
    toks = _tokens(70, config["vocab"], 3)
    eng = ld.Engine(_model(config, W, dtype))
    got = _feed(eng, "a", toks, [])
    _close(got, _oracle(name, config, W, toks), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["full", "attention_only", "mingru_only", "moe"])
def test_prefill_equals_token_by_token(name):
    import llm_decoder as ld
    config, W = _case(name)
    toks = _tokens(45, config["vocab"], 4)
    eng = ld.Engine(_model(config, W))
    got = _feed(eng, "a", toks, range(1, 45))          # every token a step of its own, from the first
    _close(got, _oracle(name, config, W, toks))


@pytest.mark.gpu
@pytest.mark.parametrize("cuts", [[2, 4, 6, 9, 40], [15, 16, 17, 31, 33, 48, 64, 66], [1, 80], [63], [7, 8, 9, 23, 24, 25]])
def test_portions_of_many_sizes(cuts):
    """Cuts at, before and after page borders (16 tokens) and temperature steps (every 32 / 5), down to two tokens."""
    import llm_decoder as ld
    config, W = _case("full")
    toks = _tokens(90, config["vocab"], 5)
    eng = ld.Engine(_model(config, W))
    _close(_feed(eng, "a", toks, cuts), _oracle("full", config, W, toks))


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
    come back (dirty) and the next request must not see what they held."""
    import llm_decoder as ld
    config, W = _case("full")
    model = _model(config, W, max_tokens=160, max_seqs=2)
    eng = ld.Engine(model)
    seqs = [_tokens(n, config["vocab"], 20 + i) for i, n in enumerate([90, 60, 33, 100, 17, 59])]
    # 0 and 1 interleaved (90 + 60 tokens: 96 + 64 = the whole pool), then the others reuse their slots and pages
    g0 = [eng.step([("r0", seqs[0][:50], list(range(50))), ("r1", seqs[1][:10], list(range(10)))])]
    g1 = [g0[0][50:]]
    g0 = [g0[0][:50]]
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


def _sharp(W, factor=6.0):
    """Queries scaled up: the softmax of every map concentrates on its best key, so one wrong, missing or extra key
    (typically a far one) moves the output by O(1) instead of O(1/n)."""
    W = dict(W)
    for k in list(W):
        if k.endswith("mix.q"):
            W[k] = (W[k].float() * factor).to(torch.bfloat16)
    return W


@pytest.mark.gpu
@pytest.mark.parametrize("tile_size", [16, 64])
def test_far_keys_and_page_borders_sharp_attention(tile_size):
    """300 tokens, peaked attention: prompts cut around page borders, then 40 decoded tokens crossing two more."""
    import llm_decoder as ld
    config = R.make_config([R.attention_layer(heads=4, kv_heads=2, dim=16, vdim=32, coef=0.6, every=64),
                            R.attention_layer(heads=2, kv_heads=1, dim=32, vdim=16, coef=0.2, every=100)], width=64, vocab=80)
    W = _sharp(R.random_weights(config, 7))
    toks = _tokens(300, config["vocab"], 8)
    want = R.forward(config, W, toks)[0]
    # the peaks are far away for most queries: check the construction, so the test means what it says
    eng = ld.Engine(_model(config, W, tile_size=tile_size))
    cuts = [63, 64, 65, 127, 129, 192, 255, 256] + list(range(260, 300))
    _close(_feed(eng, "a", toks, cuts), want)
    eng.finish("a")
    # one far key made dominant by hand: token 3's key row in map 1 of layer 0 is what query 290 looks for
    eng = ld.Engine(_model(config, W, tile_size=tile_size))
    _close(_feed(eng, "b", toks, [5, 290]), want)


@pytest.mark.gpu
def test_single_far_key_stands_out():
    """A model built so that ONE key far back carries almost all the weight of map 1 for the last query: embedding rows
    are one-hot-like, W_q and W_k make the needle token's key match the probe token's query with a large score."""
    import llm_decoder as ld
    config = R.make_config([R.attention_layer(heads=1, kv_heads=1, dim=8, vdim=16, scale=1.0, diff=0.1, coef=0.0, every=1)],
                           width=32, vocab=40, residual_mult=1.0)
    W = R.random_weights(config, 9, shift=False)
    E = torch.randn(40, 32, generator=torch.Generator().manual_seed(1))
    needle, probe = 7, 11
    W["embed"] = E.to(torch.bfloat16)
    hn = R.unit_rms(W["embed"][needle].double(), 1e-5) * float(W["l0.norm1"])
    hp = R.unit_rms(W["embed"][probe].double(), 1e-5) * float(W["l0.norm1"])
    q = W["l0.mix.q"].double().clone()
    k = W["l0.mix.k"].double().clone()
    q[:8] = 0                            # map 1 scores rest on its first coordinate alone
    k[:8] = 0
    q[0] = 4.0 * hp / (hp @ hp)          # query of the probe = 4
    k[0] = 4.0 * hn / (hn @ hn)          # key of the needle = 4  -> score 16, far above the rest
    W["l0.mix.q"], W["l0.mix.k"] = q.to(torch.bfloat16), k.to(torch.bfloat16)
    others = [t for t in range(40) if t not in (needle, probe)]
    rnd = random.Random(3)
    for needle_at in (0, 15, 16, 17, 140):
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
def test_long_decoding_and_long_portion():
    """A 280-token portion (the chunked recurrent scan and the split-key attention path) followed by 150 decoded
    tokens."""
    import llm_decoder as ld
    config, W = _case("full")
    toks = _tokens(430, config["vocab"], 40)
    eng = ld.Engine(_model(config, W))
    got = _feed(eng, "a", toks, [280] + list(range(281, 430)))
    _close(got, _oracle("full", config, W, toks))


@pytest.mark.gpu
def test_split_keys_equal_unsplit():
    """A single decoded token over a long context takes the split-key path; the same token inside a portion does not."""
    import llm_decoder as ld
    config, W = _case("attention_only")
    toks = _tokens(700, config["vocab"], 41)
    want = _oracle("attention_only", config, W, toks)
    eng = ld.Engine(_model(config, W))
    got = _feed(eng, "a", toks, [690, 699])
    _close(got, want)


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
            assert float((best - chosen).max()) < 0.25              # the chosen token is (nearly) the oracle's best


@pytest.mark.gpu
def test_sampled_generation_is_reproducible():
    import llm_decoder as ld
    config, W = _case("moe")
    prompts = [_tokens(9, config["vocab"], 60), _tokens(4, config["vocab"], 61)]
    a = ld.generate(_model(config, W, "bfloat16"), prompts, 8, temperature=0.8, top_k=5, top_p=0.9, seed=3)
    b = ld.generate(_model(config, W, "bfloat16"), prompts, 8, temperature=0.8, top_k=5, top_p=0.9, seed=3)
    assert a == b and all(len(o) == len(p) + 8 for o, p in zip(a, prompts))


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
    p = subprocess.run([os.path.join(ROOT, "bin", "generate"), "--model", str(mdir), "--dtype", "float32", "--prompt",
                        ",".join(map(str, a[:10])), "--max-new-tokens", "4"], text=True, capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    ids = [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]
    assert ids[:10] == a[:10] and len(ids) == 14


def _check_scan(lib, dev, s, g, width):
    """pa_mingru_scan and pa_mingru_scan_chunked on float rows against the recurrence written out in double."""
    from llm_decoder import _cabi
    # --- recurrence: two portions with non-zero incoming state
    lens = [70, 3]
    zxg = torch.randn(sum(lens), 3 * width, generator=g)
    zb, xb = torch.randn(width, generator=g), torch.randn(width, generator=g)
    st0 = torch.randn(4, width, generator=g)
    want_y, want_s = [], st0.double().clone()
    r0 = 0
    for slot, n in zip((2, 0), lens):
        S = st0[slot].double()
        for t in range(r0, r0 + n):
            z = torch.sigmoid(zxg[t, :width].double() + zb.double())
            u = zxg[t, width:2 * width].double() + xb.double()
            S = (1 - z) * S + z * torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            gt = zxg[t, 2 * width:].double()
            want_y.append(S * gt * torch.sigmoid(gt))
        want_s[slot] = S
        r0 += n
    want_y = torch.stack(want_y)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    for chunked in (False, True):
        state = st0.to(dev).clone()
        y = torch.empty(sum(lens), width, device=dev)
        zd, zbd, xbd = zxg.to(dev), zb.to(dev), xb.to(dev)
        slots, starts, lens_d = i32([2, 0]), i32([0, 70]), i32(lens)     # (kept alive until the kernels have run)
        if chunked:
            cs, cl, c0, cn = i32([0, 16, 32, 48, 64, 70]), i32([16, 16, 16, 16, 6, 3]), i32([0, 5]), i32([5, 1])
            ws = torch.empty(lib.pa_mingru_chunked_workspace_bytes(6, width), dtype=torch.uint8, device=dev)
            st = lib.pa_mingru_scan_chunked(zd.data_ptr(), zbd.data_ptr(), xbd.data_ptr(), width, cs.data_ptr(), cl.data_ptr(), 6,
                                            c0.data_ptr(), cn.data_ptr(), slots.data_ptr(), 2,
                                            state.data_ptr(), y.data_ptr(), 4, ws.data_ptr(), ws.numel(), s())
        else:
            st = lib.pa_mingru_scan(zd.data_ptr(), zbd.data_ptr(), xbd.data_ptr(), width, starts.data_ptr(),
                                    lens_d.data_ptr(), slots.data_ptr(), 2, state.data_ptr(), y.data_ptr(), 4, s())
        torch.cuda.synchronize()
        _cabi.check(st, "mingru")
        assert (y.double().cpu() - want_y).abs().max() < 1e-5
        assert (state.double().cpu() - want_s).abs().max() < 1e-5


@pytest.mark.gpu
def test_kernels_alone_against_the_oracle_functions():
    """minGRU scan (plain and chunked), router top-k and the grouped expert products, each called directly."""
    import llm_decoder as ld
    from llm_decoder import _cabi
    lib, dev, s = _cabi.lib(), torch.device("cuda"), _cabi.stream
    g = torch.Generator().manual_seed(5)
    for width in (40, 37):        # paired channels, and the single-channel form of odd widths
        _check_scan(lib, dev, s, g, width)
    # --- router + grouped experts: 37 rows, 5 experts, top 3, input scaling
    rows, wdt, E, top, ff = 37, 24, 5, 3, 20
    h = torch.randn(rows, wdt, generator=g)
    wr = torch.randn(E, wdt, generator=g) * 0.5
    ex = [(torch.randn(ff, wdt, generator=g) / 5, torch.randn(ff, wdt, generator=g) / 5, torch.randn(wdt, ff, generator=g) / 4)
          for _ in range(E)]
    want = R.moe_ff(h.double(), wr.double(), [tuple(t.double() for t in e) for e in ex], top)
    hd, wrd = h.to(dev), wr.to(dev)
    sel_id, sel_w = torch.empty(rows * top, dtype=torch.int32, device=dev), torch.empty(rows * top, device=dev)
    _cabi.check(lib.pa_router_topk(hd.data_ptr(), wrd.data_ptr(), None, None, rows, wdt, E, top, 0, 0, sel_id.data_ptr(),
                                   sel_w.data_ptr(), None, 4, s()), "router")
    sc = torch.sigmoid(h.double() @ wr.double().T)
    tv, ti = sc.topk(top, -1)
    assert torch.equal(sel_id.cpu().view(rows, top).long(), ti)
    assert (sel_w.cpu().view(rows, top).double() - tv).abs().max() < 1e-6
    order = torch.empty(rows * top, dtype=torch.int32, device=dev)
    meta = torch.empty(lib.pa_moe_meta_ints(rows * top, E), dtype=torch.int32, device=dev)
    _cabi.check(lib.pa_moe_sort(sel_id.data_ptr(), rows * top, E, order.data_ptr(), meta.data_ptr(), s()), "sort")
    assert sorted(order.cpu().tolist()) == list(range(rows * top))
    off = meta.cpu()[:E + 1].tolist()
    assert off[-1] == rows * top and all(int(sel_id[order[i]]) == e for e in range(E) for i in range(off[e], off[e + 1]))
    wgu = torch.stack([torch.cat([a, b], 0) for a, b, _ in ex]).to(dev).contiguous()
    wdn = torch.stack([c for _, _, c in ex]).to(dev).contiguous()
    act = torch.empty(rows * top, ff, device=dev)
    outp = torch.empty(rows * top, wdt, device=dev)
    _cabi.check(lib.pa_moe_gate_up(hd.data_ptr(), wdt, wgu.data_ptr(), wdt, ff, E, order.data_ptr(), sel_w.data_ptr(), top,
                                   meta.data_ptr(), rows * top, act.data_ptr(), 4, s()), "gate_up")
    _cabi.check(lib.pa_moe_down(act.data_ptr(), wdn.data_ptr(), ff, wdt, E, order.data_ptr(), meta.data_ptr(), rows * top,
                                outp.data_ptr(), 4, s()), "down")
    got = outp.view(rows, top, wdt).double().sum(1).cpu()
    assert (got - want).abs().max() < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("rows,experts,top,width,ff", [(20, 6, 2, 72, 40), (9, 3, 1, 64, 24), (300, 6, 2, 72, 40), (130, 2, 2, 40, 136)])
def test_grouped_expert_products_in_bfloat16_both_forms(rows, experts, top, width, ff):
    """pa_moe_gate_up / pa_moe_down on bfloat16 rows: few pairs per expert run the streaming form (weights read straight
    into the fragments), many the tiled form; both against the double oracle with the same rounding points (the scaled
    input row, gate, up and their product are bfloat16 values).  One expert gets no pair, one more than a row tile, and
    the sizes are not multiples of the kernels' tiles."""
    from llm_decoder import _cabi
    lib, dev, s = _cabi.lib(), torch.device("cuda"), _cabi.stream
    g = torch.Generator().manual_seed(rows)
    bf = torch.bfloat16
    rnd = lambda t: t.to(bf).double()  # noqa: E731
    h = torch.randn(rows, width, generator=g).to(bf)
    wgu = (torch.randn(experts, 2 * ff, width, generator=g) / math.sqrt(width)).to(bf)
    wdn = (torch.randn(experts, width, ff, generator=g) / math.sqrt(ff)).to(bf)
    pairs = rows * top
    # expert 1 is never chosen; expert 0 gets at least half of the pairs
    ids = torch.randint(0, experts, (pairs,), generator=g)
    ids[ids == 1] = 0
    ids[: pairs // 2] = 0
    ids = ids[torch.randperm(pairs, generator=g)]
    wts = torch.rand(pairs, generator=g) * 0.9 + 0.1
    want = torch.zeros(pairs, width, dtype=torch.float64)
    for i in range(pairs):
        e = int(ids[i])
        a = rnd(h[i // top].double() * wts[i].double())
        gu = wgu[e].double() @ a
        gt, up = rnd(gu[:ff]), rnd(gu[ff:])
        want[i] = wdn[e].double() @ rnd(gt * torch.sigmoid(gt) * up)
    sel_id, sel_w = ids.to(torch.int32).to(dev), wts.to(dev)
    order = torch.empty(pairs, dtype=torch.int32, device=dev)
    meta = torch.empty(lib.pa_moe_meta_ints(pairs, experts), dtype=torch.int32, device=dev)
    _cabi.check(lib.pa_moe_sort(sel_id.data_ptr(), pairs, experts, order.data_ptr(), meta.data_ptr(), s()), "sort")
    hd, wgud, wdnd = h.to(dev), wgu.to(dev), wdn.to(dev)
    act = torch.empty(pairs, ff, device=dev, dtype=bf)
    outp = torch.full((pairs, width), float("nan"), device=dev)
    _cabi.check(lib.pa_moe_gate_up(hd.data_ptr(), width, wgud.data_ptr(), width, ff, experts, order.data_ptr(), sel_w.data_ptr(),
                                   top, meta.data_ptr(), pairs, act.data_ptr(), 2, s()), "gate_up")
    _cabi.check(lib.pa_moe_down(act.data_ptr(), wdnd.data_ptr(), ff, width, experts, order.data_ptr(), meta.data_ptr(), pairs,
                                outp.data_ptr(), 2, s()), "down")
    got = outp.double().cpu()
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 2e-2 * want.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("width,experts,top,elem", [(64, 8, 2, 2), (72, 11, 3, 2), (50, 4, 4, 2), (36, 9, 1, 4), (37, 3, 2, 4)])
def test_router_scores_and_shared_gate(width, experts, top, elem):
    """pa_router_topk with the shared-expert gate: widths that allow 16-byte pieces and widths that do not, more experts
    than one group of the kernel, top == experts."""
    from llm_decoder import _cabi
    lib, dev, s = _cabi.lib(), torch.device("cuda"), _cabi.stream
    g = torch.Generator().manual_seed(width)
    rows = 45
    dt = torch.bfloat16 if elem == 2 else torch.float32
    h = torch.randn(rows, width, generator=g).to(dt)
    wr, wg = torch.randn(experts, width, generator=g), torch.randn(width, generator=g)
    sc = torch.sigmoid(h.double() @ wr.double().T)
    tv, ti = sc.topk(top, -1)
    hd, wrd, wgd = h.to(dev), wr.to(dev), wg.to(dev)
    sel_id, sel_w = torch.empty(rows * top, dtype=torch.int32, device=dev), torch.empty(rows * top, device=dev)
    gate = torch.empty(rows, device=dev)
    _cabi.check(lib.pa_router_topk(hd.data_ptr(), wrd.data_ptr(), None, wgd.data_ptr(), rows, width, experts, top, 0, 0,
                                   sel_id.data_ptr(), sel_w.data_ptr(), gate.data_ptr(), elem, s()), "router")
    assert torch.equal(sel_id.cpu().view(rows, top).long(), ti)
    assert (sel_w.cpu().view(rows, top).double() - tv).abs().max() < 1e-5
    assert (gate.cpu().double() - torch.sigmoid(h.double() @ wg.double())).abs().max() < 1e-5


# ---- the tensor-core attention kernel (bfloat16 portions of 16 tokens and more) ---------------------------------------
def _selector(rows, cols, first):
    m = torch.zeros(rows, cols, dtype=torch.float64)
    m[torch.arange(rows), first + torch.arange(rows)] = 1.0
    return m


@pytest.mark.gpu
@pytest.mark.parametrize("dim,vdim,heads,kv_heads,tile_size", [(32, 64, 4, 2, 16), (64, 128, 3, 3, 16), (128, 32, 2, 1, 64),
                                                               (64, 64, 6, 2, 8), (48, 80, 6, 3, 16), (24, 40, 2, 2, 16),
                                                               (16, 104, 5, 1, 32), (8, 8, 1, 1, 16)])
def test_tensor_core_attention_kernel_against_the_oracle(dim, vdim, heads, kv_heads, tile_size):
    """pa_diff_attention, tile kind 2, called directly on bfloat16 rows with a peaked softmax (queries scaled up, so a
    key too many or too few at a tile's, a page's or the causal edge moves a row by O(1)): one sequence fed as 150 + 100
    tokens (the second portion starts in the middle of a key tile and of a page), one of 70 tokens from its first token
    in the same launch, on pages that another sequence held before.  The oracle gets the same rounded q / k / v through
    identity projections."""
    from llm_decoder import _cabi
    from llm_decoder.seq_state import SequenceStateCache
    lib, dev = _cabi.lib(), torch.device("cuda")
    assert lib.pa_diff_attention_mma_tile_tokens(dim, vdim, 2) == 64
    assert lib.pa_diff_attention_mma_tile_tokens(dim, vdim, 4) == 0 and lib.pa_diff_attention_mma_tile_tokens(20, vdim, 2) == 0
    assert lib.pa_diff_attention_mma_tile_tokens(dim, 136, 2) == 0
    qc, kc, vc = heads * 2 * dim, kv_heads * 2 * dim, kv_heads * vdim
    cols = qc + kc + vc
    scale, diff, coef, every, eps = 0.9 / math.sqrt(dim), 0.3, 0.4, 48, 1e-5
    lq1, lk1 = torch.zeros(dim, dtype=torch.float64), torch.zeros(dim, dtype=torch.float64)
    lq2, lk2 = lq1.clone(), lk1.clone()
    lq1[0], lk1[0], lq2[1], lk2[1] = 0.2, 1.0, -0.1, 1.0
    lam = math.exp(0.2) - math.exp(-0.1) + diff
    g = torch.Generator().manual_seed(dim + vdim)
    seqs = {"a": torch.randn(250, cols, generator=g), "b": torch.randn(70, cols, generator=g)}
    for t in seqs.values():
        t[:, :qc] *= 3.0
    seqs = {k: v.to(torch.bfloat16) for k, v in seqs.items()}
    states = SequenceStateCache(3, 512, tile_size, dev)
    kv = states.add_kv_layer(kv_heads, 2 * dim, vdim, "bf16")
    old = states.alloc()
    states.extend(old, 40)
    slot = {"a": states.alloc(), "b": states.alloc()}
    states.free(old)
    got = {k: [] for k in seqs}
    fed = {k: 0 for k in seqs}
    for step in ([("a", 150)], [("a", 100), ("b", 70)]):
        batch = states.make_batch([(slot[k], [0] * n) for k, n in step])
        qkv = torch.cat([seqs[k][fed[k]:fed[k] + n] for k, n in step]).to(dev).contiguous()
        kv.append_rows(qkv, qc, qc + kc, batch.row_slot, batch.row_pos)
        tiles, ntiles, _longest = batch.query_tiles(lib.pa_diff_attention_tile_tokens(heads, kv_heads), 64, 16)[2]
        out = torch.zeros(batch.rows, heads * vdim, dtype=torch.bfloat16, device=dev)
        pt = kv.page_table_
        _cabi.check(lib.pa_diff_attention(qkv.data_ptr(), qkv.stride(0), 0, kv.key_buffer_.data_ptr(), kv.value_buffer_.data_ptr(),
                                          pt.device_data().data_ptr(), pt.num_beams_, pt.num_heads_, pt.num_tiles_,
                                          kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles, heads, dim, vdim, scale, coef,
                                          every, lam, 1.0 - diff, eps, out.data_ptr(), 2, 1, 2, None, 0, _cabi.stream()),
                    "pa_diff_attention")
        torch.cuda.synchronize()
        r0 = 0
        for k, n in step:
            got[k].append(out[r0:r0 + n].double().cpu())
            fed[k] += n
            r0 += n
    for k, rows in seqs.items():
        want = R.diff_attention_mixer_fast(rows.double(), _selector(qc, cols, 0), _selector(kc, cols, qc), _selector(vc, cols, qc + kc),
                                           torch.eye(heads * vdim, dtype=torch.float64), lq1, lk1, lq2, lk2, heads, kv_heads, dim,
                                           vdim, scale, diff, coef, every, eps)
        err = (torch.cat(got[k]) - want).abs().max().item()
        assert err < 0.04, f"sequence {k}: max abs error {err}"


@pytest.mark.gpu
@pytest.mark.parametrize("dim,vdim,heads,kv_heads", [(48, 80, 6, 3), (64, 128, 5, 1), (16, 104, 20, 1), (32, 32, 4, 4)])
def test_decoded_tokens_with_heads_as_rows_equal_the_streaming_kernel(dim, vdim, heads, kv_heads):
    """pa_diff_attention tile kind 3 (one token per tile, the heads of a key/value head as the rows of a tensor-core
    tile) against kind 1 (the float streaming kernel, itself held to the oracle elsewhere) on the same pools: sequences
    at their FIRST token, just inside and just past a 64-key step and a page, and far along; peaked softmax."""
    from llm_decoder import _cabi
    from llm_decoder.seq_state import SequenceStateCache
    lib, dev = _cabi.lib(), torch.device("cuda")
    assert lib.pa_diff_attention_mma_head_rows(heads, kv_heads, dim, vdim, 2) == 1
    assert lib.pa_diff_attention_mma_head_rows(heads, kv_heads, dim, vdim, 4) == 0
    assert lib.pa_diff_attention_mma_head_rows(130, 2, dim, vdim, 2) == 0
    qc, kc, vc = heads * 2 * dim, kv_heads * 2 * dim, kv_heads * vdim
    cols = qc + kc + vc
    lens = [1, 16, 17, 64, 65, 129, 300]
    g = torch.Generator().manual_seed(dim * heads)
    states = SequenceStateCache(len(lens), sum(lens) + 16 * len(lens), 16, dev)
    kv = states.add_kv_layer(kv_heads, 2 * dim, vdim, "bf16")
    slots = [states.alloc() for _ in lens]
    # contexts: everything but the last token goes in first (keys and values only), then one token each
    before = [(sl, [0] * (n - 1)) for sl, n in zip(slots, lens) if n > 1]
    b0 = states.make_batch(before)
    ctx = torch.randn(b0.rows, cols, generator=g).to(torch.bfloat16).to(dev)
    kv.append_rows(ctx, qc, qc + kc, b0.row_slot, b0.row_pos)
    b1 = states.make_batch([(sl, [0]) for sl in slots])
    qkv = torch.randn(b1.rows, cols, generator=g)
    qkv[:, :qc] *= 3.0
    qkv = qkv.to(torch.bfloat16).to(dev)
    kv.append_rows(qkv, qc, qc + kc, b1.row_slot, b1.row_pos)
    tiles, ntiles, _longest = b1.query_tiles(lib.pa_diff_attention_tile_tokens(heads, kv_heads))[1]
    pt = kv.page_table_
    outs = {}
    for kind in (1, 3):
        out = torch.full((b1.rows, heads * vdim), float("nan"), dtype=torch.bfloat16, device=dev)
        _cabi.check(lib.pa_diff_attention(qkv.data_ptr(), qkv.stride(0), 0, kv.key_buffer_.data_ptr(), kv.value_buffer_.data_ptr(),
                                          pt.device_data().data_ptr(), pt.num_beams_, pt.num_heads_, pt.num_tiles_,
                                          kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles, heads, dim, vdim,
                                          0.9 / math.sqrt(dim), 0.4, 48, 0.45, 0.7, 1e-5, out.data_ptr(), 2, 1, kind, None, 0,
                                          _cabi.stream()), "pa_diff_attention")
        torch.cuda.synchronize()
        outs[kind] = out.double().cpu()
    assert torch.isfinite(outs[3]).all()
    err = (outs[3] - outs[1]).abs().max().item()
    assert err < 0.04, f"max abs difference {err}"


def cfg_mma_heads():
    # head sizes the tensor-core attention kernel serves in bfloat16
    return R.make_config([R.attention_layer(heads=4, kv_heads=2, dim=32, vdim=64, coef=0.3, every=16, mlp=R.dense_mlp(64)),
                          R.mingru_layer(48, None),
                          R.attention_layer(heads=2, kv_heads=1, dim=64, vdim=32, diff=0.15, coef=0.2, every=50)],
                         width=64, vocab=83, residual_mult=0.6)


CONFIGS["mma_heads"] = cfg_mma_heads


@pytest.mark.gpu
def test_bfloat16_portions_on_the_tensor_cores_equal_small_portions():
    """bfloat16, head sizes of the tensor-core kernel: a 230-token prompt in one step, in portions that switch between
    the tensor-core kernel (16 tokens and more) and the float kernels (shorter, and single tokens), and batched beside
    another request give the same logits up to rounding, and the oracle's."""
    import llm_decoder as ld
    config, W = _case("mma_heads")
    toks = _tokens(230, config["vocab"], 51)
    other = _tokens(90, config["vocab"], 52)
    want = _oracle("mma_heads", config, W, toks)
    whole = _feed(ld.Engine(_model(config, W, "bfloat16")), "a", toks, [])
    _close(whole, want, "bfloat16")
    cut = _feed(ld.Engine(_model(config, W, "bfloat16")), "a", toks, [3, 19, 35, 99, 100, 110, 174, 229])
    eng = ld.Engine(_model(config, W, "bfloat16"))
    outs = [eng.step([("a", toks[:64], list(range(64))), ("b", other[:17], [])])]
    outs.append(eng.step([("b", other[17:], []), ("a", toks[64:65], [0])]))
    outs.append(eng.step([("a", toks[65:], list(range(165)))]))
    mixed = torch.cat(outs, 0)
    for got in (cut, mixed):
        rel = (got.double() - whole.double()).pow(2).mean(-1).sqrt() / whole.double().pow(2).mean(-1).sqrt()
        assert rel.max().item() < 0.03, f"relative rms difference {rel.max().item()}"
