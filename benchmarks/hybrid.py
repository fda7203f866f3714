#!/usr/bin/env python
"""Throughput of the config-driven hybrid stack (llm_decoder.hybrid, design `Megusun`) at layer sizes that resemble a
real model, next to the framework's closest fixed model (CUDADecoder with attention projections) at equal width, layer
count, vocabulary, batch and context; random weights, synthetic tokens.  `python bench.py --hybrid` prints its JSON line.

Per size: prefill tokens/s (PREFILL_SEQS prompts of PREFILL_LEN tokens in one step) and decode tokens/s (DECODE_SEQS
sequences at DECODE_CTX tokens of context, one token each per step), CUDA events around back-to-back steps after
warm-up.  `kernels` times the design's own kernels alone at the largest size against their roofline (algorithmic bytes
over the measured copy bandwidth, or FLOPs over the measured bf16 GEMM rate; MEASURED_PEAKS.json)."""
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "pagedattention-based-transformer-decoder-inference-framework_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

PREFILL_SEQS, PREFILL_LEN = 4, 2048
DECODE_SEQS, DECODE_CTX = 64, 2048
VOCAB = 32768
SIZES = {
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=64, vdim=128, gru=1024, ff=4096, experts=8, top=2, eff=512, sff=1024),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=64, vdim=128, gru=2048, ff=8192, experts=8, top=2, eff=1024, sff=2048),
}


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, "fallback"


def hybrid_config(s):
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "top": s["top"]},
           "shared": {"ff": s["sff"]}}
    gru = lambda mlp: {"type": "mingru", "mixer": {"width": s["gru"]}, "mlp": mlp}  # noqa: E731
    att = {"type": "attention", "mlp": moe,
           "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "diff": 0.3,
                     "scale": s["dim"] ** -0.5, "q_temp": {"coef": 0.3, "every": 256}}}
    return {"architecture": "Megusun", "layers": [gru(dense), gru(moe), att, gru(dense)], "norm": {"eps": 1e-5},
            "residual_mult": 0.3, "vocab": VOCAB, "width": s["width"]}


def hybrid_weights(config, dev):
    g = torch.Generator(device=dev).manual_seed(0)
    Wd = config["width"]
    mat = lambda o, i: (torch.randn(o, i, device=dev, generator=g) / math.sqrt(i)).to(torch.bfloat16)  # noqa: E731
    vec = lambda n: (torch.randn(n, device=dev, generator=g) * 0.3).to(torch.bfloat16)  # noqa: E731
    W = {"embed": torch.randn(config["vocab"], Wd, device=dev, generator=g).to(torch.bfloat16),
         "head": mat(config["vocab"], Wd), "final.norm": torch.tensor(1.0, dtype=torch.bfloat16)}
    for i, lc in enumerate(config["layers"]):
        p, mc = f"l{i}.", lc["mixer"]
        W[p + "norm1"] = torch.tensor(1.0, dtype=torch.bfloat16)
        W[p + "shift"] = torch.rand(Wd, device=dev, generator=g).to(torch.bfloat16)
        if lc["type"] == "mingru":
            for n in "zxg":
                W[p + "mix." + n] = mat(mc["width"], Wd)
            W[p + "mix.z.b"], W[p + "mix.x.b"], W[p + "mix.o"] = vec(mc["width"]), vec(mc["width"]), mat(Wd, mc["width"])
        else:
            H, G, D, V = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(H * 2 * D, Wd), mat(G * 2 * D, Wd), mat(G * V, Wd)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[p + "mix." + n] = vec(D)
            W[p + "mix.o"] = mat(Wd, H * V)
        ml = lc["mlp"]
        if ml["kind"] == "dense":
            W[p + "mlp.up"], W[p + "mlp.down"] = mat(ml["ff"], Wd), mat(Wd, ml["ff"])
        else:
            f = ml["expert"]["ff"]
            for e in range(ml["router"]["experts"]):
                W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = mat(f, Wd), mat(f, Wd), mat(Wd, f)
            W[p + "mlp.router"] = mat(ml["router"]["experts"], Wd)
            f = ml["shared"]["ff"]
            W[p + "mlp.shared.gate"], W[p + "mlp.shared.up"], W[p + "mlp.shared.down"] = mat(f, Wd), mat(f, Wd), mat(Wd, f)
            W[p + "mlp.shared.sg"] = mat(1, Wd)
    return W


def timed(fn, warmup=3, iters=8):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def bench_hybrid(s, dtype, dev):
    import llm_decoder as ld
    config = hybrid_config(s)
    cap = DECODE_SEQS * (DECODE_CTX + 64)
    model = ld.HybridDecoder(config, hybrid_weights(config, dev), dtype, max_tokens=cap, max_seqs=DECODE_SEQS, tile_size=16)
    eng = ld.Engine(model)
    g = torch.Generator().manual_seed(1)
    toks = lambda n: torch.randint(0, VOCAB, (n,), generator=g).tolist()  # noqa: E731
    prompts = [toks(PREFILL_LEN) for _ in range(PREFILL_SEQS)]

    def prefill():
        out = eng.step([(f"p{i}", p, [PREFILL_LEN - 1]) for i, p in enumerate(prompts)])
        for i in range(PREFILL_SEQS):
            eng.finish(f"p{i}")
        return out
    t_pre = timed(prefill, 2, 4)
    # decode: fill DECODE_SEQS sequences to DECODE_CTX, then single-token steps
    for lo in range(0, DECODE_SEQS, 8):
        eng.step([(f"d{i}", toks(DECODE_CTX), []) for i in range(lo, lo + 8)])
    nxt = [toks(1) for _ in range(DECODE_SEQS)]
    t_dec = timed(lambda: eng.step([(f"d{i}", nxt[i], [0]) for i in range(DECODE_SEQS)]), 3, 10)
    for i in range(DECODE_SEQS):
        eng.finish(f"d{i}")
    del model, eng
    torch.cuda.empty_cache()
    return dict(prefill_tok_s=PREFILL_SEQS * PREFILL_LEN / t_pre, prefill_ms=t_pre * 1e3,
                decode_tok_s=DECODE_SEQS / t_dec, decode_ms=t_dec * 1e3)


def bench_fixed(s, dev):
    """CUDADecoder (fp32 activations and weights on the 3xTF32 tcgen05 linear kernel, fp16 K/V pages, tcgen05 prefill
    attention) with Q/K/V/O projections: 4 layers, hidden = width, 128-wide heads, MLP 4 x hidden."""
    import llm_decoder as ld
    hid = s["width"]
    dec = ld.CUDADecoder(4, hid // 128, 128, hid, VOCAB, DECODE_CTX + 64, device=dev, batch_size=DECODE_SEQS)
    g = torch.Generator(device=dev).manual_seed(2)
    rnd = lambda *sh: torch.randn(*sh, device=dev, generator=g) / math.sqrt(sh[0])  # noqa: E731
    dec.embedding = torch.randn(VOCAB, hid, device=dev, generator=g)
    for L in dec.layers:
        L.fc1_w, L.fc2_w = rnd(hid, 4 * hid), rnd(4 * hid, hid)
        L.wq, L.wk, L.wv, L.wo = rnd(hid, hid), rnd(hid, hid), rnd(hid, hid), rnd(hid, hid)
    dec._temperature, dec._sampling = 1.0, None
    prompt = torch.randint(0, VOCAB, (PREFILL_SEQS, PREFILL_LEN), device=dev, dtype=torch.int32)

    def prefill():
        dec._setup_batch(PREFILL_SEQS)
        dec.reset()
        dec._prefill(prompt)
    t_pre = timed(prefill, 2, 4)
    dec._setup_batch(DECODE_SEQS)
    dec.reset()
    dec.positions.fill_(DECODE_CTX)
    dec.ctx_lens.fill_(DECODE_CTX + 1)

    def step():
        dec._step()
        dec.positions.fill_(DECODE_CTX)
        dec.ctx_lens.fill_(DECODE_CTX + 1)
    t_dec = timed(step, 3, 10)
    del dec
    torch.cuda.empty_cache()
    return dict(prefill_tok_s=PREFILL_SEQS * PREFILL_LEN / t_pre, prefill_ms=t_pre * 1e3,
                decode_tok_s=DECODE_SEQS / t_dec, decode_ms=t_dec * 1e3)


def bench_kernels(s, dev):
    """The design's own kernels alone (bfloat16 activations) at the prefill and decode shapes of size `s`."""
    import llm_decoder as ld
    from llm_decoder import _cabi
    from llm_decoder.seq_state import SequenceStateCache
    lib, st = _cabi.lib(), _cabi.stream
    hbm, tfl, how = peaks()
    out = {}
    bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    W, Wr = s["width"], s["gru"]
    H, G, D, V = s["heads"], s["kv_heads"], s["dim"], s["vdim"]

    def rec(name, secs, bytes_=None, flops=None):
        e = dict(us=secs * 1e6)
        if bytes_ is not None:
            e.update(gbs=bytes_ / secs / 1e9, frac_of_hbm=bytes_ / secs / 1e9 / hbm)
        if flops is not None:
            e.update(tflops=flops / secs / 1e12, frac_of_bf16_gemm=flops / secs / 1e12 / tfl)
        out[name] = e

    for tag, nseq, plen, ctx0 in (("prefill", PREFILL_SEQS, PREFILL_LEN, 0), ("decode", DECODE_SEQS, 1, DECODE_CTX)):
        R = nseq * plen
        states = SequenceStateCache(nseq, nseq * (ctx0 + plen + 16), 16, dev)
        prev, gstate = states.add_state(W), states.add_state(Wr)
        kv = states.add_kv_layer(G, 2 * D, V, "bf16")
        slots = [states.alloc() for _ in range(nseq)]
        if ctx0:
            for sl in slots:
                states.extend(sl, ctx0)
        b = states.make_batch([(sl, [1] * plen) for sl in slots])
        x = torch.randn(R, W, device=dev)
        h, hs = torch.empty(R, W, device=dev, dtype=bf), torch.empty(R, W, device=dev, dtype=bf)
        shift = torch.rand(W, device=dev)
        rec(f"rms_norm_shift/{tag}", timed(lambda: lib.pa_rms_norm_shift(
            x.data_ptr(), R, W, 1e-5, 1.0, None, shift.data_ptr(), b.row_prev.data_ptr(), b.row_slot.data_ptr(),
            prev.data_ptr(), h.data_ptr(), hs.data_ptr(), 2, st())), bytes_=R * W * (4 + 4 + 2 + 2))
        zxg = torch.randn(R, 3 * Wr, device=dev).to(bf)
        zb, y = torch.zeros(Wr, device=dev), torch.empty(R, Wr, device=dev, dtype=bf)
        if plen >= 256:
            cs, cl, s0, sn, nch = b.scan_chunks(64)
            ws = torch.empty(lib.pa_mingru_chunked_workspace_bytes(nch, Wr), dtype=torch.uint8, device=dev)
            fn = lambda: lib.pa_mingru_scan_chunked(zxg.data_ptr(), zb.data_ptr(), zb.data_ptr(), Wr, cs.data_ptr(),  # noqa: E731
                                                    cl.data_ptr(), nch, s0.data_ptr(), sn.data_ptr(), b.seq_slot.data_ptr(),
                                                    nseq, gstate.data_ptr(), y.data_ptr(), 2, ws.data_ptr(), ws.numel(), st())
        else:
            fn = lambda: lib.pa_mingru_scan(zxg.data_ptr(), zb.data_ptr(), zb.data_ptr(), Wr, b.seq_start.data_ptr(),  # noqa: E731
                                            b.seq_len.data_ptr(), b.seq_slot.data_ptr(), nseq, gstate.data_ptr(), y.data_ptr(), 2, st())
        rec(f"mingru_scan/{tag}", timed(fn), bytes_=R * Wr * (6 + 2))
        # attention over the pool (pages hold whatever is there: the timing does not depend on the values)
        qkv = torch.randn(R, (H * 2 * D + G * 2 * D + G * V), device=dev).to(bf)
        kv.key_buffer_.normal_()
        kv.value_buffer_.normal_()
        tt = lib.pa_diff_attention_tile_tokens(H, G)
        single = 1 if plen == 1 else 2
        tiles, ntiles, longest = b.query_tiles(tt, lib.pa_diff_attention_mma_tile_tokens(D, V, 2), 16)[single]
        o = torch.empty(R, H * V, device=dev, dtype=bf)
        ctas = ntiles * G
        nsplit = 1
        if single == 1 and ctas >= 148 and lib.pa_diff_attention_mma_head_rows(H, G, D, V, 2):
            single = 3                                     # the engine's rule: heads as rows on the tensor cores
        if single == 1 and ctas < 4 * 148 and longest > 512:
            nsplit = max(1, min(math.ceil(4 * 148 / ctas), longest // 256, 64))
        wsb = lib.pa_diff_attention_workspace_bytes(ntiles, H, G, V, nsplit)
        ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
        pt = kv.page_table_
        table = pt.device_data()
        fn = lambda: lib.pa_diff_attention(qkv.data_ptr(), qkv.stride(0), 0, kv.key_buffer_.data_ptr(),  # noqa: E731
                                           kv.value_buffer_.data_ptr(), table.data_ptr(), pt.num_beams_, pt.num_heads_,
                                           pt.num_tiles_, kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles, H, D, V,
                                           D ** -0.5, 0.3, 256, 0.4, 0.7, 1e-5, o.data_ptr(), 2, nsplit, single,
                                           ws.data_ptr() if wsb else None, wsb, st())
        assert fn() == 0
        if plen > 1:
            flops = nseq * H * (plen * (plen + 1) / 2) * (2 * 2 * D + 2 * 2 * V)     # two maps: q.k and p.v
            rec(f"diff_attention/{tag}", timed(fn, 2, 4), flops=flops)
        else:
            rec(f"diff_attention/{tag}", timed(fn), bytes_=nseq * (ctx0 + 1) * G * (2 * D + V) * 2)
        # routed experts
        E, top, ff = s["experts"], s["top"], s["eff"]
        pairs = R * top
        hb = torch.randn(R, W, device=dev).to(bf)
        wr = torch.randn(E, W, device=dev) / math.sqrt(W)
        sel_id, sel_w = torch.empty(pairs, device=dev, dtype=i32), torch.empty(pairs, device=dev)
        sg, sgw = torch.empty(R, device=dev), torch.randn(W, device=dev)
        rec(f"router_topk/{tag}", timed(lambda: lib.pa_router_topk(hb.data_ptr(), wr.data_ptr(), None, sgw.data_ptr(), R, W, E, top,
                                                                   0, 0, sel_id.data_ptr(), sel_w.data_ptr(), sg.data_ptr(), 2, st())),
            bytes_=R * W * 2)
        order = torch.empty(pairs, device=dev, dtype=i32)
        meta = torch.empty(lib.pa_moe_meta_ints(pairs, E), device=dev, dtype=i32)
        rec(f"moe_sort/{tag}", timed(lambda: lib.pa_moe_sort(sel_id.data_ptr(), pairs, E, order.data_ptr(), meta.data_ptr(), st())))
        wgu = (torch.randn(E, 2 * ff, W, device=dev) / math.sqrt(W)).to(bf)
        wdn = (torch.randn(E, W, ff, device=dev) / math.sqrt(ff)).to(bf)
        act, routed = torch.empty(pairs, ff, device=dev, dtype=bf), torch.empty(pairs, W, device=dev)
        wbytes = E * 3 * ff * W * 2
        t1 = timed(lambda: lib.pa_moe_gate_up(hb.data_ptr(), W, wgu.data_ptr(), W, ff, E, order.data_ptr(), sel_w.data_ptr(), top,
                                              meta.data_ptr(), pairs, act.data_ptr(), 2, st()))
        t2 = timed(lambda: lib.pa_moe_down(act.data_ptr(), wdn.data_ptr(), ff, W, E, order.data_ptr(), meta.data_ptr(), pairs,
                                           routed.data_ptr(), 2, st()))
        if plen > 1:
            rec(f"moe_experts/{tag}", t1 + t2, flops=pairs * 3 * ff * W * 2)
        else:
            rec(f"moe_experts/{tag}", t1 + t2, bytes_=wbytes)
        mix = torch.randn(R, W, device=dev).to(bf)
        rec(f"residual_combine/{tag}", timed(lambda: lib.pa_residual_combine(
            x.data_ptr(), R, W, 0.3, mix.data_ptr(), None, routed.data_ptr(), top, mix.data_ptr(), sg.data_ptr(), 2, st())),
            bytes_=R * W * (8 + 2 + 2 + 4 * top))
        del states, kv
        torch.cuda.empty_cache()
    out["_denominators"] = dict(hbm_gbs=hbm, bf16_tflops=tfl, source=how)
    return out


def run(sizes=None, kernels=True):
    assert torch.cuda.is_available(), "needs a GPU"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    res = {"workload": dict(prefill=f"{PREFILL_SEQS} x {PREFILL_LEN} tokens in one step",
                            decode=f"{DECODE_SEQS} sequences at {DECODE_CTX} tokens, one token each per step",
                            layers="mingru+dense, mingru+moe, attention+moe, mingru+dense", vocab=VOCAB,
                            data="synthetic tokens, random-init weights"), "sizes": {}}
    for name in sizes or SIZES:
        s = SIZES[name]
        res["sizes"][name] = dict(shape=s, hybrid_bf16=bench_hybrid(s, "bfloat16", dev), hybrid_f32=bench_hybrid(s, "float32", dev),
                                  cuda_decoder_f32=bench_fixed(s, dev))
    if kernels:
        res["kernels_w2048_bf16"] = bench_kernels(SIZES["w2048"], dev)
    return res


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "--kernels":     # the kernels alone at one size (a small case for a profiler)
        torch.cuda.set_device(0)
        print(json.dumps({"kernels_" + sys.argv[2]: bench_kernels(SIZES[sys.argv[2]], torch.device("cuda", 0))}, default=float))
    else:
        print(json.dumps(run(), default=float))
