#!/usr/bin/env python
"""Throughput of the `Domilix` design (llm_decoder.hybrid: latent attention, post-norm wiring, gated dense layers, routed
experts weighted on their output) at layer sizes that resemble a real model, next to the framework's closest existing
model -- the same config-driven stack serving `Megusun` -- at equal width, layer count, vocabulary, batch and context;
random weights, synthetic tokens.  `python bench.py --latent` prints its JSON line.

Per size: prefill tokens/s (PREFILL_SEQS prompts of PREFILL_LEN tokens in one step) and decode tokens/s (DECODE_SEQS
sequences at DECODE_CTX tokens of context, one token each per step), CUDA events around back-to-back steps after
warm-up.  `kernels` times the design's own kernels alone at the largest size against their roofline (algorithmic bytes
over the measured copy bandwidth, FLOPs over the measured bf16 GEMM rate; MEASURED_PEAKS.json)."""
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

from benchmarks import hybrid as hy  # noqa: E402

PREFILL_SEQS, PREFILL_LEN = hy.PREFILL_SEQS, hy.PREFILL_LEN
DECODE_SEQS, DECODE_CTX = hy.DECODE_SEQS, hy.DECODE_CTX
VOCAB = hy.VOCAB
SIZES = {
    "w1024": dict(width=1024, heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256, q_rank=384, ff=2816, experts=8, top=2, eff=512),
    "w2048": dict(width=2048, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768, ff=5632, experts=8, top=2, eff=1024),
}
timed, peaks = hy.timed, hy.peaks


def latent_config(s):
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "top": s["top"]}}

    def layer(mlp, kv_from=None):
        m = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot_dim"], "vdim": s["vdim"], "kv_rank": s["kv_rank"],
             "q_rank": s["q_rank"], "rot": {"base": 10000.0, "dims": s["rot_dim"]}, "scale": (s["dim"] + s["rot_dim"]) ** -0.5}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "latent_attention", "mixer": m, "mlp": mlp}
    return {"architecture": "Domilix", "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "vocab": VOCAB, "width": s["width"],
            "layers": [layer(dense), layer(moe), layer(moe, 1), layer(dense, 1)]}


def latent_weights(config, dev):
    g = torch.Generator(device=dev).manual_seed(0)
    Wd = config["width"]
    mat = lambda o, i: (torch.randn(o, i, device=dev, generator=g) / math.sqrt(i)).to(torch.bfloat16)  # noqa: E731
    ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=dev)  # noqa: E731
    W = {"embed": torch.randn(config["vocab"], Wd, device=dev, generator=g).to(torch.bfloat16),
         "head": mat(config["vocab"], Wd), "final.norm": ones(Wd)}
    for i, lc in enumerate(config["layers"]):
        p, mc = f"l{i}.", lc["mixer"]
        H, D, Rt, V, kr, qr = mc["heads"], mc["dim"], mc["rot_dim"], mc["vdim"], mc["kv_rank"], mc["q_rank"]
        W[p + "norm1"], W[p + "norm2"] = ones(Wd), ones(Wd)
        W[p + "mix.dq"], W[p + "mix.dq.norm"], W[p + "mix.uq"] = mat(qr, Wd), ones(qr), mat(H * (D + Rt), qr)
        if "kv_from" not in mc:
            W[p + "mix.dkv"], W[p + "mix.dkv.norm"] = mat(kr + Rt, Wd), ones(kr)
        W[p + "mix.uk"], W[p + "mix.uv"], W[p + "mix.g"], W[p + "mix.o"] = mat(H * D, kr), mat(H * V, kr), mat(H, Wd), mat(Wd, H * V)
        ml = lc["mlp"]
        if ml["kind"] == "dense":
            W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"] = mat(ml["ff"], Wd), mat(ml["ff"], Wd), mat(Wd, ml["ff"])
        else:
            f = ml["expert"]["ff"]
            for e in range(ml["router"]["experts"]):
                W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = mat(f, Wd), mat(Wd, f)
            W[p + "mlp.router"] = mat(ml["router"]["experts"], Wd)
            W[p + "mlp.router.b"] = torch.zeros(ml["router"]["experts"], dtype=torch.bfloat16, device=dev)
    return W


def bench_model(s, dtype, dev):
    import llm_decoder as ld
    config = latent_config(s)
    cap = DECODE_SEQS * (DECODE_CTX + 64)
    model = ld.HybridDecoder(config, latent_weights(config, dev), dtype, max_tokens=cap, max_seqs=DECODE_SEQS, tile_size=16)
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


def bench_kernels(s, dev):
    """The design's own kernels alone (bfloat16 activations) at the prefill and decode shapes of size `s`."""
    from llm_decoder import _cabi
    from llm_decoder.seq_state import SequenceStateCache
    lib, st = _cabi.lib(), _cabi.stream
    hbm, tfl, how = peaks()
    out = {}
    bf, i32 = torch.bfloat16, torch.int32
    W, H, D, Rt, V, kvr, qr = s["width"], s["heads"], s["dim"], s["rot_dim"], s["vdim"], s["kv_rank"], s["q_rank"]
    kd, qd = kvr + Rt, D + Rt

    def rec(name, secs, bytes_=None, flops=None):
        e = dict(us=secs * 1e6)
        if bytes_ is not None:
            e.update(gbs=bytes_ / secs / 1e9, frac_of_hbm=bytes_ / secs / 1e9 / hbm)
        if flops is not None:
            e.update(tflops=flops / secs / 1e12, frac_of_bf16_gemm=flops / secs / 1e12 / tfl)
        if bytes_ is not None and flops is not None:     # the slower of the two floors is the kernel's roofline
            e["frac_of_roofline"] = max(bytes_ / (hbm * 1e9), flops / (tfl * 1e12)) / secs
        out[name] = e

    for tag, nseq, plen, ctx0 in (("prefill", PREFILL_SEQS, PREFILL_LEN, 0), ("decode", DECODE_SEQS, 1, DECODE_CTX)):
        R = nseq * plen
        states = SequenceStateCache(nseq, nseq * (ctx0 + plen + 16), 16, dev)
        kv = states.add_kv_layer(1, kd, 0, "bf16")
        slots = [states.alloc() for _ in range(nseq)]
        if ctx0:
            for sl in slots:
                states.extend(sl, ctx0)
        b = states.make_batch([(sl, [1] * plen) for sl in slots])
        pt = kv.page_table_
        table = pt.device_data()
        kv.key_buffer_.normal_()
        rope = torch.empty(R, Rt // 2, 2, device=dev)
        rec(f"rope_table/{tag}", timed(lambda: lib.pa_rope_table(b.row_pos.data_ptr(), R, Rt, 10000.0, rope.data_ptr(), st())))
        proj = torch.randn(R, qr + kd + H, device=dev).to(bf)
        gain = torch.ones(kvr, device=dev)
        rec(f"latent_kv_append/{tag}", timed(lambda: lib.pa_latent_kv_append(
            kv.key_buffer_.data_ptr(), table.data_ptr(), pt.num_beams_, pt.num_tiles_, kv.total_pages_, kv.tile_size_, kvr, Rt,
            Rt, proj.data_ptr(), proj.stride(0), qr, gain.data_ptr(), 1e-5, rope.data_ptr(), b.row_slot.data_ptr(),
            b.row_pos.data_ptr(), R, 2, st())), bytes_=R * kd * 4)
        cq, qgain = torch.empty(R, qr, device=dev, dtype=bf), torch.ones(qr, device=dev)
        rec(f"rms_norm_rows/{tag}", timed(lambda: lib.pa_rms_norm_rows(proj.data_ptr(), proj.stride(0), 0, qr, 1e-5, qgain.data_ptr(),
                                                                       cq.data_ptr(), qr, R, 2, st())), bytes_=R * qr * 4)
        q = torch.randn(R, H * qd, device=dev).to(bf)
        rec(f"rope_rows/{tag}", timed(lambda: lib.pa_rope_rows(q.data_ptr(), q.stride(0), D, qd, H, Rt, rope.data_ptr(), R, 2, st())),
            bytes_=R * H * Rt * 4)
        w_uk = (torch.randn(H, D, kvr, device=dev) / math.sqrt(D)).to(bf)
        w_uv = (torch.randn(H, kvr, V, device=dev) / math.sqrt(kvr)).to(bf)
        qv = torch.as_strided(q, (H, R, D), (qd, H * qd, 1))
        ql = torch.bmm(qv, w_uk)
        rec(f"head_products_vendor/{tag}", timed(lambda: (torch.bmm(qv, w_uk), torch.bmm(ql, w_uv))),
            flops=2.0 * R * H * kvr * (D + V), bytes_=R * H * (kvr * 4 + (D + V) * 2) + H * kvr * (D + V) * 2)
        lat = torch.empty(H, R, kvr, device=dev, dtype=bf)
        tt = lib.pa_latent_attention_mma_tile_tokens(H, kvr, Rt, 2)
        group = b.query_tiles(tt)[1 if plen == 1 else 0]
        tiles, ntiles, longest = group
        from llm_decoder.hybrid import latent_key_splits
        nsplit = latent_key_splits(ntiles * math.ceil(H / 64), longest, _cabi.device_info()[0])
        wsb = lib.pa_latent_attention_workspace_bytes(ntiles, H, kvr, nsplit)
        ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
        fn = lambda: lib.pa_latent_attention(ql.data_ptr(), kvr, R * kvr, q.data_ptr() + D * 2, q.stride(0), qd,  # noqa: E731
                                             kv.key_buffer_.data_ptr(), table.data_ptr(), pt.num_beams_, pt.num_tiles_,
                                             kv.total_pages_, kv.tile_size_, tiles.data_ptr(), ntiles, H, kvr, Rt, qd ** -0.5,
                                             lat.data_ptr(), kvr, R * kvr, 2, nsplit, 3 if plen == 1 else 2,
                                             ws.data_ptr() if wsb else None, wsb, st())
        assert fn() == 0
        if plen > 1:
            rec(f"latent_attention/{tag}", timed(fn, 2, 4), flops=nseq * H * (plen * (plen + 1) / 2) * (2 * kd + 2 * kvr))
        else:
            rec(f"latent_attention/{tag}", timed(fn), bytes_=nseq * (ctx0 + 1) * kd * 2,
                flops=nseq * (ctx0 + 1) * H * (2 * kd + 2 * kvr))
            out[f"latent_attention/{tag}"]["nsplit"] = nsplit
        ov, og = torch.randn(H, R, V, device=dev).to(bf), torch.empty(R, H * V, device=dev, dtype=bf)
        rec(f"head_gate/{tag}", timed(lambda: lib.pa_head_gate(ov.data_ptr(), V, R * V, proj.data_ptr() + (qr + kd) * 2, proj.stride(0),
                                                               H, V, R, og.data_ptr(), 2, st())), bytes_=R * H * V * 4)
        # feed-forwards
        E, top, ff = s["experts"], s["top"], s["eff"]
        pairs = R * top
        hb = torch.randn(R, W, device=dev).to(bf)
        wr, br = torch.randn(E, W, device=dev) / math.sqrt(W), torch.zeros(E, device=dev)
        sel_id, sel_w = torch.empty(pairs, device=dev, dtype=i32), torch.empty(pairs, device=dev)
        rec(f"router_topk/{tag}", timed(lambda: lib.pa_router_topk(hb.data_ptr(), wr.data_ptr(), br.data_ptr(), None, R, W, E, top, 2, 0,
                                                                   sel_id.data_ptr(), sel_w.data_ptr(), None, 2, st())), bytes_=R * W * 2)
        order = torch.empty(pairs, device=dev, dtype=i32)
        meta = torch.empty(lib.pa_moe_meta_ints(pairs, E), device=dev, dtype=i32)
        rec(f"moe_sort/{tag}", timed(lambda: lib.pa_moe_sort(sel_id.data_ptr(), pairs, E, order.data_ptr(), meta.data_ptr(), st())))
        wup = (torch.randn(E, ff, W, device=dev) / math.sqrt(W)).to(bf)
        wdn = (torch.randn(E, W, ff, device=dev) / math.sqrt(ff)).to(bf)
        act, routed = torch.empty(pairs, ff, device=dev, dtype=bf), torch.empty(pairs, W, device=dev)
        t1 = timed(lambda: lib.pa_moe_up(hb.data_ptr(), W, wup.data_ptr(), W, ff, E, order.data_ptr(), None, top, meta.data_ptr(), pairs,
                                         2, act.data_ptr(), 2, st()))
        t2 = timed(lambda: lib.pa_moe_down(act.data_ptr(), wdn.data_ptr(), ff, W, E, order.data_ptr(), meta.data_ptr(), pairs,
                                           routed.data_ptr(), 2, st()))
        if plen > 1:
            rec(f"moe_experts/{tag}", t1 + t2, flops=pairs * 2 * ff * W * 2)
        else:
            rec(f"moe_experts/{tag}", t1 + t2, bytes_=E * 2 * ff * W * 2)
        x, nxt, g1 = torch.randn(R, W, device=dev), torch.empty(R, W, device=dev, dtype=bf), torch.ones(W, device=dev)
        rec(f"residual_add_norm_routed/{tag}", timed(lambda: lib.pa_residual_add_norm(
            x.data_ptr(), R, W, 1e-5, g1.data_ptr(), None, routed.data_ptr(), sel_w.data_ptr(), top, nxt.data_ptr(), 2, st())),
            bytes_=R * W * (8 + 2 + 4 * top))
        rec(f"residual_add_norm/{tag}", timed(lambda: lib.pa_residual_add_norm(
            x.data_ptr(), R, W, 1e-5, g1.data_ptr(), hb.data_ptr(), None, None, 0, nxt.data_ptr(), 2, st())), bytes_=R * W * (8 + 2 + 2))
        gu, a = torch.randn(R, 2 * s["ff"], device=dev).to(bf), torch.empty(R, s["ff"], device=dev, dtype=bf)
        rec(f"act_mul/{tag}", timed(lambda: lib.pa_act_mul(gu.data_ptr(), R, s["ff"], 1, a.data_ptr(), 2, st())), bytes_=R * s["ff"] * 6)
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
                            layers="latent+dense, latent+moe, latent(borrowed pool)+moe, latent(borrowed pool)+dense", vocab=VOCAB,
                            data="synthetic tokens, random-init weights"), "sizes": {}}
    for name in sizes or SIZES:
        s = SIZES[name]
        res["sizes"][name] = dict(shape=s, latent_bf16=bench_model(s, "bfloat16", dev), latent_f32=bench_model(s, "float32", dev),
                                  megusun_bf16=hy.bench_hybrid(hy.SIZES[name], "bfloat16", dev))
    if kernels:
        res["kernels_w2048_bf16"] = bench_kernels(SIZES["w2048"], dev)
    return res


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "--kernels":     # the kernels alone at one size (a small case for a profiler)
        torch.cuda.set_device(0)
        print(json.dumps({"kernels_" + sys.argv[2]: bench_kernels(SIZES[sys.argv[2]], torch.device("cuda", 0))}, default=float))
    else:
        print(json.dumps(run(), default=float))
