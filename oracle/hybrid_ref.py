"""Test oracle for the config-driven hybrid decoder stack (llm_decoder.hybrid): a plain, slow, float64 restatement of
every mechanism, one function each, that recomputes whole sequences from scratch (no cache, no state, no batching).
It shares no code with the product path; tests compare the engine's logits at any position, however the tokens were
cut into steps and batches, with `forward(config, weights, tokens)` of the full token list.

Also here: `make_config` / `random_weights`, the small random models the tests run."""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, gain, eps):
    return unit_rms(x, eps) * gain


def token_shift(h, shift):
    """Row t becomes h_t + (h_{t-1} - h_t) * shift, with h_{-1} = 0."""
    out = torch.empty_like(h)
    for t in range(h.shape[0]):
        before = h[t - 1] if t > 0 else torch.zeros_like(h[0])
        out[t] = h[t] + (before - h[t]) * shift
    return out


def mingru_mixer(hs, w_z, b_z, w_x, b_x, w_g, w_o):
    state = torch.zeros(w_z.shape[0], dtype=F64)
    rows = []
    for t in range(hs.shape[0]):
        z = torch.sigmoid(w_z @ hs[t] + b_z)
        u = w_x @ hs[t] + b_x
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        state = (1 - z) * state + z * cand
        g = w_g @ hs[t]
        rows.append(w_o @ (state * (g * torch.sigmoid(g))))
    return torch.stack(rows)


def diff_attention_mixer(hs, w_q, w_k, w_v, w_o, lq1, lk1, lq2, lk2, heads, kv_heads, dim, vdim, scale, diff, coef, every,
                         eps):
    n = hs.shape[0]
    lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + diff
    group = heads // kv_heads
    rows = []
    for i in range(n):
        q = (w_q @ hs[i]) * (1 + coef * math.log(math.floor((i + 1) / every) + 1))
        heads_out = []
        for h in range(heads):
            g = h // group
            maps = []
            for part in range(2):
                qv = q[(2 * h + part) * dim:(2 * h + part + 1) * dim]
                scores = torch.stack([(qv * (w_k @ hs[j])[(2 * g + part) * dim:(2 * g + part + 1) * dim]).sum() * scale
                                      for j in range(i + 1)])
                wts = torch.softmax(scores, 0)
                vals = torch.stack([(w_v @ hs[j])[g * vdim:(g + 1) * vdim] for j in range(i + 1)])
                maps.append(wts @ vals)
            o = maps[0] - lam * maps[1]
            heads_out.append(unit_rms(o, eps) * (1 - diff))
        rows.append(w_o @ torch.cat(heads_out))
    return torch.stack(rows)


def diff_attention_mixer_fast(hs, w_q, w_k, w_v, w_o, lq1, lk1, lq2, lk2, heads, kv_heads, dim, vdim, scale, diff, coef,
                              every, eps):
    """The same function with the keys projected once (what the loop above recomputes per query); used for the longer
    test sequences and checked against the loop on short ones."""
    n = hs.shape[0]
    lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + diff
    group = heads // kv_heads
    Q, K, V = hs @ w_q.T, hs @ w_k.T, hs @ w_v.T
    temp = torch.tensor([1 + coef * math.log(math.floor((i + 1) / every) + 1) for i in range(n)], dtype=F64)
    Q = Q * temp[:, None]
    causal = torch.ones(n, n, dtype=torch.bool).tril()
    outs = []
    for h in range(heads):
        g = h // group
        maps = []
        for part in range(2):
            s = Q[:, (2 * h + part) * dim:(2 * h + part + 1) * dim] @ K[:, (2 * g + part) * dim:(2 * g + part + 1) * dim].T
            s = (s * scale).masked_fill(~causal, -math.inf)
            maps.append(torch.softmax(s, -1) @ V[:, g * vdim:(g + 1) * vdim])
        outs.append(unit_rms(maps[0] - lam * maps[1], eps) * (1 - diff))
    return torch.cat(outs, -1) @ w_o.T


def dense_ff(h, w_up, w_down):
    a = h @ w_up.T
    return (0.5 * a * (1 + torch.erf(a / math.sqrt(2)))) @ w_down.T


def gated_expert(a, w_gate, w_up, w_down):
    g = w_gate @ a
    return w_down @ ((g * torch.sigmoid(g)) * (w_up @ a))


def moe_ff(h, w_router, experts, top, shared=None):
    """experts: list of (gate, up, down); shared: None or (gate, up, down, sg or None)."""
    rows = []
    for t in range(h.shape[0]):
        score = torch.sigmoid(w_router @ h[t])
        order = sorted(range(len(experts)), key=lambda e: (-float(score[e]), e))[:top]
        acc = torch.zeros(h.shape[1], dtype=F64)
        for e in order:
            acc = acc + gated_expert(score[e] * h[t], *experts[e])
        if shared is not None:
            s = gated_expert(h[t], *shared[:3])
            acc = acc + (s * torch.sigmoid((shared[3].reshape(-1) * h[t]).sum()) if shared[3] is not None else s)
        rows.append(acc)
    return torch.stack(rows)


def forward(config, weights, tokens, fast_attention=True):
    """Logits [len(tokens), vocab] and the residual after every layer [layers, len(tokens), width], float64."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps, m = config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = W["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    after = []
    for i, lc in enumerate(config["layers"]):
        p = f"l{i}."
        h = scalar_norm(x, W[p + "norm1"], eps)
        hs = token_shift(h, W[p + "shift"]) if p + "shift" in W else h
        mc = lc["mixer"]
        if lc["type"] == "mingru":
            mix = mingru_mixer(hs, W[p + "mix.z"], W[p + "mix.z.b"], W[p + "mix.x"], W[p + "mix.x.b"], W[p + "mix.g"],
                               W[p + "mix.o"])
        elif lc["type"] == "attention":
            fn = diff_attention_mixer_fast if fast_attention else diff_attention_mixer
            mix = fn(hs, W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"], W[p + "mix.o"], W[p + "mix.lq1"], W[p + "mix.lk1"],
                     W[p + "mix.lq2"], W[p + "mix.lk2"], mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"], mc["scale"],
                     mc["diff"], mc["q_temp"]["coef"], mc["q_temp"]["every"], eps)
        else:
            raise ValueError(lc["type"])
        ml = lc.get("mlp")
        if not ml:
            ff = torch.zeros_like(x)
        elif ml["kind"] == "dense":
            ff = dense_ff(h, W[p + "mlp.up"], W[p + "mlp.down"])
        else:
            ex = [(W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"]) for e in range(ml["router"]["experts"])]
            sh = None
            if ml.get("shared"):
                sh = (W[p + "mlp.shared.gate"], W[p + "mlp.shared.up"], W[p + "mlp.shared.down"], W.get(p + "mlp.shared.sg"))
            ff = moe_ff(h, W[p + "mlp.router"], ex, ml["router"]["top"], sh)
        x = x + m * (mix + ff)
        after.append(x.clone())
    logits = scalar_norm(x, W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(after)


# ------------------------------------------------------------------------------------------------- small random models
def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, scale=None, diff=0.25, coef=0.4, every=8, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
                      "scale": dim ** -0.5 if scale is None else scale, "q_temp": {"coef": coef, "every": every}}}


def mingru_layer(width=48, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def dense_mlp(ff=96):
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=6, top=2, ff=40, shared_ff=56):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def make_config(layers, width=64, vocab=97, eps=1e-5, residual_mult=0.5, architecture="Megusun"):
    return {"architecture": architecture, "layers": layers, "norm": {"eps": eps}, "residual_mult": residual_mult,
            "vocab": vocab, "width": width}


def random_weights(config, seed=0, shift=True):
    """bfloat16 tensors under the product's tensor names, scaled so activations stay O(1)."""
    g = torch.Generator().manual_seed(seed)
    Wd, V = config["width"], config["vocab"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s / math.sqrt(i))).to(torch.bfloat16)

    def vec(n, s=1.0, off=0.0):
        return (torch.randn(n, generator=g) * s + off).to(torch.bfloat16)

    W = {"embed": (torch.randn(V, Wd, generator=g)).to(torch.bfloat16), "head": mat(V, Wd),
         "final.norm": torch.tensor(1.1).to(torch.bfloat16)}
    for i, lc in enumerate(config["layers"]):
        p = f"l{i}."
        W[p + "norm1"] = torch.tensor(0.9 + 0.05 * i).to(torch.bfloat16)
        if shift:
            W[p + "shift"] = (torch.rand(Wd, generator=g) * 0.8).to(torch.bfloat16)
        mc = lc["mixer"]
        if lc["type"] == "mingru":
            w = mc["width"]
            W[p + "mix.z"], W[p + "mix.x"], W[p + "mix.g"] = mat(w, Wd, 2.0), mat(w, Wd, 1.5), mat(w, Wd, 1.5)
            W[p + "mix.z.b"], W[p + "mix.x.b"] = vec(w, 0.5), vec(w, 0.5)
            W[p + "mix.o"] = mat(Wd, w)
        else:
            H, G, D, Vd = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(H * 2 * D, Wd, 2.0), mat(G * 2 * D, Wd, 2.0), mat(G * Vd, Wd)
            for nme in ("lq1", "lk1", "lq2", "lk2"):
                W[p + "mix." + nme] = vec(D, 0.3)
            W[p + "mix.o"] = mat(Wd, H * Vd)
        ml = lc.get("mlp")
        if ml and ml["kind"] == "dense":
            W[p + "mlp.up"], W[p + "mlp.down"] = mat(ml["ff"], Wd), mat(Wd, ml["ff"])
        elif ml:
            for e in range(ml["router"]["experts"]):
                f = ml["expert"]["ff"]
                W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = mat(f, Wd, 1.5), mat(f, Wd, 1.5), mat(Wd, f)
            W[p + "mlp.router"] = mat(ml["router"]["experts"], Wd, 3.0)
            if ml.get("shared"):
                f = ml["shared"]["ff"]
                W[p + "mlp.shared.gate"], W[p + "mlp.shared.up"], W[p + "mlp.shared.down"] = mat(f, Wd), mat(f, Wd), mat(Wd, f)
                W[p + "mlp.shared.sg"] = mat(1, Wd, 2.0)
    return W
