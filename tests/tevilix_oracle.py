"""Plain, slow restatement of the Tevilix design in float64 torch ops, one function per mechanism.  It shares no code with
the product path: tests build small random checkpoints with `random_model` and compare the framework against this.

Notation: x residual stream [T, W]; a layer computes x + mixer(ln(x, w1)) + ff(ln(x, w2)) with both branches reading the
same x; ln is a layer norm with a weight and no bias.  A span of layers may run several times in a row with the same
weights; `layer_runs` lists the order, every run has a state of its own.
"""
import math

import torch

F64 = torch.float64


# ---- norms and activations -----------------------------------------------------------------------------------------
def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def unit_rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def relu_squared(z):
    r = torch.clamp(z, min=0.0)
    return r * r


# ---- attention with mixed head scores ------------------------------------------------------------------------------
def rotary_frequencies(dims, base, factor=1.0):
    return [float(base) ** (-2.0 * i / dims) / float(factor) for i in range(dims // 2)]


def rotate_half(t, pos, dims, base, factor=1.0):
    """t [T, heads, dim]; the first `dims` channels of every head turn by the position: channel i pairs with i + dims / 2."""
    if not dims:
        return t
    half = dims // 2
    f = torch.tensor(rotary_frequencies(dims, base, factor), dtype=F64)
    ang = pos.to(F64)[:, None] * f[None, :]                    # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = t[..., :half], t[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, t[..., dims:]], -1)


def mixed_score_attention(q, k, v, pos_q, pos_k, scale, talk, window):
    """q [Tq, H, D], k [Tk, G, D], v [Tk, G, V].  s[h] = scale * q_h . k_g(h); then every (query, key) pair's H scores are
    mixed by `talk` [H, H] (s'[h] = sum_g talk[h, g] s[g]); key j is seen by query i when 0 <= pos_i - pos_j < window
    (window 0: no limit); plain softmax over the seen keys."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    s = torch.stack([q[:, h] @ k[:, h // rep].T * scale for h in range(H)])           # [H, Tq, Tk]
    if talk is not None:
        s = torch.einsum("hg,gqk->hqk", talk, s)
    d = pos_q[:, None] - pos_k[None, :]
    seen = d >= 0
    if window:
        seen = seen & (d < window)
    s = s.masked_fill(~seen[None], -float("inf"))
    p = torch.softmax(s, -1)
    return torch.stack([p[h] @ v[:, h // rep] for h in range(H)], 1)                 # [Tq, H, V]


def attention_branch(W, p, h, c, eps, pos):
    H, D, V = c["heads"], c["dim"], c["vdim"]
    G = c.get("kv_heads", H)
    T = h.shape[0]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, V)
    q, k = unit_rms(q, eps, W[p + "q.norm"]), unit_rms(k, eps, W[p + "k.norm"])
    rot = c.get("rot") or {}
    dims = int(rot.get("dims", 0))
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q = rotate_half(q, pos, dims, rot.get("base", 10000.0), factor)
    k = rotate_half(k, pos, dims, rot.get("base", 10000.0), factor)
    o = mixed_score_attention(q, k, v, pos, pos, c["scale"], W.get(p + "talk"), int((c.get("mask") or {}).get("size", 0)))
    o = o.reshape(T, H * V) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T + W[p + "o.b"]


# ---- the gated recurrence whose gates read only the current token --------------------------------------------------
def gru_candidate(u):
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def gru_recurrence(z, cand, state=None):
    """S_t = (1 - z_t) S_(t-1) + z_t cand_t, element by element; z, cand [T, width]."""
    S = torch.zeros(z.shape[1], dtype=z.dtype) if state is None else state.clone()
    out = torch.zeros_like(z)
    for t in range(z.shape[0]):
        S = (1 - z[t]) * S + z[t] * cand[t]
        out[t] = S
    return out, S


def gru_branch(W, p, h):
    z = torch.sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    S, _ = gru_recurrence(z, gru_candidate(u))
    g = h @ W[p + "g"].T
    return (S * g * torch.sigmoid(g)) @ W[p + "o"].T


def parallel_mixer(W, p, h, c, eps, pos):
    return c["left_scale"] * attention_branch(W, p + "left.", h, c["left"], eps, pos) + c["right_scale"] * gru_branch(W, p + "right.", h)


# ---- matrix memory ------------------------------------------------------------------------------------------------
def mlstm_gates(h, w_i, b_i, w_f, b_f, cap):
    i = cap * torch.tanh((h @ w_i.T + b_i) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w_f.T + b_f) / cap))
    return i, f


def mlstm_recurrence(q, k, v, ig, fg):
    """q, k [T, H, D] (q already scaled), v [T, H, V], log gates [T, H]; the running maximum starts at 0."""
    T, H, D = q.shape
    V = v.shape[-1]
    S, n, m = torch.zeros(H, D, V, dtype=F64), torch.zeros(H, D, dtype=F64), torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a, b = torch.exp(fg[t] + m - m_new), torch.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    return out


def mlstm_mixer(W, p, h, c, eps):
    H, D, V = c["heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T * D ** -0.5).view(T, H, D)
    k = (h @ W[p + "k"].T).view(T, H, D)
    v = (h @ W[p + "v"].T).view(T, H, V)
    ig, fg = mlstm_gates(h, W[p + "i"], W[p + "i.b"], W[p + "f"], W[p + "f.b"], c["gate_cap"])
    o = unit_rms(mlstm_recurrence(q, k, v, ig, fg), eps).reshape(T, H * V) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# ---- feed-forwards ------------------------------------------------------------------------------------------------
def dense_ff(W, p, h):
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


def route(h, w_router, correction, top, n_groups, keep_groups, scale):
    """(idx [T, top], weights [T, top]).  Scores are sigmoids of the router's outputs; the choice adds `correction`; only the
    `keep_groups` groups of neighbouring experts with the largest sum of their two best choice scores stay eligible; the
    weights are the chosen plain scores over their sum, times `scale`."""
    s = torch.sigmoid(h @ w_router.T)
    choice = s + (correction if correction is not None else 0.0)
    T, E = s.shape
    if n_groups > 1:
        per = E // n_groups
        grouped = choice.view(T, n_groups, per)
        gs = grouped.topk(min(2, per), -1).values.sum(-1)
        kept = gs.topk(keep_groups, -1).indices
        ok = torch.zeros(T, n_groups, dtype=torch.bool)
        ok.scatter_(1, kept, True)
        choice = grouped.masked_fill(~ok[:, :, None], -float("inf")).reshape(T, E)
    idx = choice.topk(top, -1).indices
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20) * scale


def moe_ff(W, p, h, c):
    r = c["router"]
    groups = r.get("groups") or {}
    idx, w = route(h, W[p + "router"], W.get(p + "correction"), r["top"], int(groups.get("count", 1)), int(groups.get("keep", groups.get("count", 1))),
                   float(r.get("scale", 1.0)))
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            y[t] += w[t, j] * (relu_squared(h[t] @ W[f"{p}e{e}.up"].T) @ W[f"{p}e{e}.down"].T)
    return y


# ---- the model ------------------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """Indices of the layers in the order they run: the span [start, stop) `times` times in a row, then the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop.get("times", 1)) == 1:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence run whole."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens)
    pos = torch.arange(tokens.shape[0])
    x = W["embed"][tokens] * cfg["embedding"]["scale"]
    for i in layer_runs(cfg):
        L = cfg["layers"][i]
        p, c = f"l{i}.", L["mixer"]
        h = layer_norm(x, W[p + "norm1"], eps)
        y = mlstm_mixer(W, p + "mix.", h, c, eps) if L["type"] == "mlstm" else parallel_mixer(W, p + "mix.", h, c, eps, pos)
        f = L.get("mlp")
        if f is not None:
            h2 = layer_norm(x, W[p + "norm2"], eps)
            y = y + (dense_ff(W, p + "mlp.", h2) if f["kind"] == "dense" else moe_ff(W, p + "mlp.", h2, f))
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T


def greedy(cfg, W, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]


# ---- small random checkpoints --------------------------------------------------------------------------------------
def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=16, groups=3, keep=2, scale=1.5):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def mlstm_layer(heads=2, dim=8, vdim=12, gate_cap=10.0, mlp="dense"):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap},
            "mlp": dense() if mlp == "dense" else mlp}


def parallel_layer(heads=4, kv_heads=2, dim=12, vdim=10, window=7, rot_dims=8, base=500.0, factor=2.0, scale=None, gru=20,
                   left_scale=0.7, right_scale=1.2, mlp="dense"):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
            "rot": {"base": base, "dims": rot_dims, "scaling": {"factor": factor}}, "scale": scale if scale is not None else dim ** -0.5}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right": {"width": gru}, "right_scale": right_scale},
            "mlp": dense() if mlp == "dense" else mlp}


def make_config(layers, width=32, vocab=53, embed_scale=1.7, eps=1e-5, loop=None):
    cfg = {"architecture": "Tevilix", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale}, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_model(cfg, seed=0, bf16_values=True, talk_off_diagonal=0.3):
    """float64 weights for `cfg`.  With `bf16_values` every weight is exactly representable in bfloat16, so that a checkpoint
    written in bfloat16 holds the same numbers the oracle uses."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]
    W = {}

    def rnd(*shape, std=1.0, mean=0.0):
        t = torch.randn(tuple(shape), generator=g, dtype=F64) * std + mean
        return t.to(torch.bfloat16).to(F64) if bf16_values else t

    lin = lambda o, i: rnd(o, i, std=i ** -0.5)
    W["embed"] = rnd(vocab, width)
    for i, L in enumerate(cfg["layers"]):
        p, c = f"l{i}.", L["mixer"]
        W[p + "norm1"] = rnd(width, std=0.1, mean=1.0)
        if L["type"] == "mlstm":
            H, D, V = c["heads"], c["dim"], c["vdim"]
            m = p + "mix."
            W[m + "q"], W[m + "k"] = lin(H * D, width), lin(H * D, width)
            W[m + "v"], W[m + "g"] = lin(H * V, width), lin(H * V, width)
            W[m + "o"], W[m + "norm"] = lin(width, H * V), rnd(H * V, std=0.1, mean=1.0)
            W[m + "i"], W[m + "i.b"] = lin(H, width) * 2, rnd(H, std=1.0)
            W[m + "f"], W[m + "f.b"] = lin(H, width) * 2, rnd(H, std=1.0, mean=3.0)
        else:
            a, m = c["left"], p + "mix.left."
            H, D, V = a["heads"], a["dim"], a["vdim"]
            G = a.get("kv_heads", H)
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                W[m + n], W[m + n + ".b"] = lin(rows, width), rnd(rows, std=0.3)
            W[m + "q.norm"], W[m + "k.norm"] = rnd(D, std=0.2, mean=1.5), rnd(D, std=0.2, mean=1.5)
            W[m + "talk"] = (torch.eye(H, dtype=F64) + rnd(H, H, std=talk_off_diagonal)).to(torch.bfloat16).to(F64)
            W[m + "g"], W[m + "o"], W[m + "o.b"] = lin(H * V, width), lin(width, H * V), rnd(width, std=0.2)
            r, n = c["right"]["width"], p + "mix.right."
            W[n + "z"], W[n + "z.b"] = lin(r, width) * 2, rnd(r, std=1.0)
            W[n + "x"], W[n + "x.b"] = lin(r, width) * 2, rnd(r, std=0.5)
            W[n + "g"], W[n + "o"] = lin(r, width), lin(width, r)
        f = L.get("mlp")
        if f is not None:
            W[p + "norm2"] = rnd(width, std=0.1, mean=1.0)
            if f["kind"] == "dense":
                W[p + "mlp.up"], W[p + "mlp.down"] = lin(f["ff"], width), lin(width, f["ff"])
            else:
                E, ff = f["router"]["experts"], f["expert"]["ff"]
                for e in range(E):
                    W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = lin(ff, width), lin(width, ff)
                W[p + "mlp.router"], W[p + "mlp.correction"] = lin(E, width) * 2, rnd(E, std=0.3)
    W["final.norm"], W["head"] = rnd(width, std=0.1, mean=1.0), lin(vocab, width)
    return W
