"""Test oracle for the `Domilix` design as served by llm_decoder.hybrid: a plain, slow, float64 restatement, one function
per mechanism, that recomputes whole sequences from scratch (no cache, no batching, no absorbed projections).  It shares
no code with the product path; tests compare the engine's logits at any position, however the tokens were cut into steps
and batches, with `forward(config, weights, tokens)` of the full token list.

The design in this file's notation (x_t = residual row of token t, position t counted from 0):

    x_t     = embed[token_t] * s_embed
    x      += N1(mixer(x)),  then  x += N2(ff(x))          N(y) = y / sqrt(mean(y^2) + eps) * w   (no norm on the input)
    logits  = head . N_final(x)

  latent attention   cq = N(Wdq x; w_dq),  q = Wuq cq, head by head [dim plain | rot_dim rotated]
                     [c_raw | kr_raw] = Wdkv x,  c = N(c_raw; w_dkv),  kr = R_t(kr_raw)  (one rotated part for all heads)
                     score_h(t, j) = (q_plain_h(t) . (Wuk_h c_j) + R_t(q_rot_h(t)) . kr_j) * scale,  j <= t, softmax over j
                     o_h(t) = sigmoid(Wg x_t)_h * sum_j p_h(t, j) (Wuv_h c_j),   out = Wo [o_0 | o_1 | ...]
                     a layer with `kv_from: j` uses layer j's (c, kr) rows instead of computing its own
  rotation R_p       pairs (2i, 2i + 1): (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i / dims)
  ff 'dense'         Wdown (relu(Wgate h) * (Wup h))
  ff 'moe'           z = Wr h + b;  the `top` largest z (ties: lower id);  weights = softmax over the chosen z only;
                     sum_e weight_e * Wdown_e relu(Wup_e h)^2

Also here: `make_config` / `random_weights`, the small random models the tests run."""
import math

import torch

F64 = torch.float64


def weighted_rms_norm(y, w, eps):
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps) * w


def rotate_pairs(v, pos, base, dims):
    """Rotate the first `dims` entries of the last axis of v (interleaved pairs) by the angles of position `pos`."""
    out = v.clone()
    for i in range(dims // 2):
        a = pos * base ** (-2.0 * i / dims)
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * math.cos(a) - w * math.sin(a)
        out[..., 2 * i + 1] = w * math.cos(a) + u * math.sin(a)
    return out


def latent_kv(x, w_dkv, w_norm, kv_rank, rot, eps):
    """What a layer with its own down-projection leaves for itself and for the layers that borrow from it:
    (c [n, kv_rank], kr [n, rot_dim] rotated)."""
    both = x @ w_dkv.T
    c = weighted_rms_norm(both[:, :kv_rank], w_norm, eps)
    kr = torch.stack([rotate_pairs(both[t, kv_rank:], t, rot["base"], rot["dims"]) for t in range(x.shape[0])])
    return c, kr


def latent_attention_mixer(x, c, kr, w_dq, w_dq_norm, w_uq, w_uk, w_uv, w_g, w_o, heads, dim, rot_dim, vdim, scale, rot, eps):
    n = x.shape[0]
    cq = weighted_rms_norm(x @ w_dq.T, w_dq_norm, eps)
    q = (cq @ w_uq.T).reshape(n, heads, dim + rot_dim)
    keys = (c @ w_uk.T).reshape(n, heads, dim)
    vals = (c @ w_uv.T).reshape(n, heads, vdim)
    gate = torch.sigmoid(x @ w_g.T)
    rows = []
    for t in range(n):
        parts = []
        for h in range(heads):
            qp = q[t, h, :dim]
            qr = rotate_pairs(q[t, h, dim:], t, rot["base"], rot["dims"])
            s = torch.stack([(qp * keys[j, h]).sum() + (qr * kr[j]).sum() for j in range(t + 1)]) * scale
            p = torch.softmax(s, 0)
            parts.append(gate[t, h] * (p[:, None] * vals[:t + 1, h]).sum(0))
        rows.append(w_o @ torch.cat(parts))
    return torch.stack(rows)


def latent_attention_mixer_fast(x, c, kr, w_dq, w_dq_norm, w_uq, w_uk, w_uv, w_g, w_o, heads, dim, rot_dim, vdim, scale, rot,
                                eps):
    """The same function in matrix form (used for the longer test sequences, checked against the loop on short ones)."""
    n = x.shape[0]
    cq = weighted_rms_norm(x @ w_dq.T, w_dq_norm, eps)
    q = (cq @ w_uq.T).reshape(n, heads, dim + rot_dim)
    qr = torch.stack([rotate_pairs(q[t, :, dim:], t, rot["base"], rot["dims"]) for t in range(n)])
    keys = (c @ w_uk.T).reshape(n, heads, dim)
    vals = (c @ w_uv.T).reshape(n, heads, vdim)
    s = (torch.einsum("thd,jhd->htj", q[:, :, :dim], keys) + torch.einsum("thd,jd->htj", qr, kr)) * scale
    s = s.masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), -math.inf)
    o = torch.einsum("htj,jhv->thv", torch.softmax(s, -1), vals) * torch.sigmoid(x @ w_g.T)[:, :, None]
    return o.reshape(n, heads * vdim) @ w_o.T


def dense_ff(h, w_gate, w_up, w_down):
    return (torch.relu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def moe_ff(h, w_router, b_router, experts, top):
    """experts: list of (up, down)."""
    rows = []
    for t in range(h.shape[0]):
        z = w_router @ h[t] + b_router
        chosen = sorted(range(len(experts)), key=lambda e: (-float(z[e]), e))[:top]
        wts = torch.softmax(torch.stack([z[e] for e in chosen]), 0)
        acc = torch.zeros(h.shape[1], dtype=F64)
        for w, e in zip(wts, chosen):
            up, down = experts[e]
            acc = acc + w * (down @ torch.relu(up @ h[t]) ** 2)
        rows.append(acc)
    return torch.stack(rows)


def forward(config, weights, tokens, fast_attention=True):
    """Logits [len(tokens), vocab] and the residual after every layer [layers, len(tokens), width], float64."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.tensor(list(tokens), dtype=torch.long)] * config["embedding"]["scale"]
    after, kept = [], {}
    for i, lc in enumerate(config["layers"]):
        p, mc = f"l{i}.", lc["mixer"]
        if lc["type"] != "latent_attention":
            raise ValueError(lc["type"])
        if mc.get("kv_from") is None:
            kept[i] = latent_kv(x, W[p + "mix.dkv"], W[p + "mix.dkv.norm"], mc["kv_rank"], mc["rot"], eps)
            c, kr = kept[i]
        else:
            c, kr = kept[mc["kv_from"]]
        fn = latent_attention_mixer_fast if fast_attention else latent_attention_mixer
        mix = fn(x, c, kr, W[p + "mix.dq"], W[p + "mix.dq.norm"], W[p + "mix.uq"], W[p + "mix.uk"],
                 W[p + "mix.uv"], W[p + "mix.g"], W[p + "mix.o"], mc["heads"], mc["dim"], mc["rot_dim"], mc["vdim"], mc["scale"],
                 mc["rot"], eps)
        x = x + weighted_rms_norm(mix, W[p + "norm1"], eps)
        ml = lc.get("mlp")
        if ml:
            if ml["kind"] == "dense":
                ff = dense_ff(x, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"])
            else:
                ex = [(W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"]) for e in range(ml["router"]["experts"])]
                ff = moe_ff(x, W[p + "mlp.router"], W[p + "mlp.router.b"], ex, ml["router"]["top"])
            x = x + weighted_rms_norm(ff, W[p + "norm2"], eps)
        after.append(x.clone())
    logits = weighted_rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(after)


# ------------------------------------------------------------------------------------------------- small random models
def latent_layer(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=48, base=1000.0, scale=None, kv_from=None, mlp=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "rot": {"base": base, "dims": rot_dim}, "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def dense_mlp(ff=96):
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=6, top=2, ff=40):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def make_config(layers, width=64, vocab=97, eps=1e-5, embed_scale=2.0):
    return {"architecture": "Domilix", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


def random_weights(config, seed=0):
    """bfloat16 tensors under the product's tensor names, scaled so activations stay O(1)."""
    g = torch.Generator().manual_seed(seed)
    Wd, V = config["width"], config["vocab"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s / math.sqrt(i))).to(torch.bfloat16)

    def vec(n, s=1.0, off=0.0):
        return (torch.randn(n, generator=g) * s + off).to(torch.bfloat16)

    W = {"embed": (torch.randn(V, Wd, generator=g) * 0.5).to(torch.bfloat16), "head": mat(V, Wd),
         "final.norm": vec(Wd, 0.1, 1.0)}
    for i, lc in enumerate(config["layers"]):
        p, mc = f"l{i}.", lc["mixer"]
        H, D, R, Vd, kr, qr = mc["heads"], mc["dim"], mc["rot_dim"], mc["vdim"], mc["kv_rank"], mc["q_rank"]
        W[p + "norm1"], W[p + "norm2"] = vec(Wd, 0.1, 0.7), vec(Wd, 0.1, 0.7)
        W[p + "mix.dq"], W[p + "mix.dq.norm"], W[p + "mix.uq"] = mat(qr, Wd), vec(qr, 0.1, 1.0), mat(H * (D + R), qr, 2.0)
        if mc.get("kv_from") is None:
            W[p + "mix.dkv"], W[p + "mix.dkv.norm"] = mat(kr + R, Wd, 1.5), vec(kr, 0.1, 1.0)
        W[p + "mix.uk"], W[p + "mix.uv"] = mat(H * D, kr, 2.0), mat(H * Vd, kr)
        W[p + "mix.g"], W[p + "mix.o"] = mat(H, Wd, 2.0), mat(Wd, H * Vd)
        ml = lc.get("mlp")
        if ml and ml["kind"] == "dense":
            W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"] = mat(ml["ff"], Wd, 1.5), mat(ml["ff"], Wd), mat(Wd, ml["ff"])
        elif ml:
            f = ml["expert"]["ff"]
            for e in range(ml["router"]["experts"]):
                W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = mat(f, Wd, 1.5), mat(Wd, f)
            W[p + "mlp.router"], W[p + "mlp.router.b"] = mat(ml["router"]["experts"], Wd, 2.0), vec(ml["router"]["experts"], 0.5)
    return W
