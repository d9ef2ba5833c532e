"""Plain, slow restatement of the Safilorn design in float64 torch ops, one function per mechanism.  It shares no code
with the product path: tests build small random checkpoints with `random_model` and compare the framework against this.

Notation: x residual stream [T, W]; n(x, w) = x / sqrt(mean(x^2) + eps) * (1 + w); a layer is
    x <- x + n(mixer(n(x, w1)), w1b);   x <- x + n(ff(n(x, w2)), w2b)
and with X_0 the embedding output and X_(i+1) the result of layer i, the stream that goes on after layer i is
sum_j a_i[j] X_j (j = 0 .. i + 1).  Everything here recomputes a whole sequence from its first token, so it knows nothing of
caches, slots or batches.
"""
import math

import torch

F64 = torch.float64
SWISH_ALPHA = 1.702   # the experts' gate activation g * sigmoid(1.702 g)
ATTN_FACTOR_COEF = 0.1


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def scaled_frequencies(dims, base, scaling=None):
    """(f_i for i < dims / 2, multiplier of cos and sin).  f_i = base^(-2i/dims); with scaling {factor, original, fast, slow}
    the pairs below `lo` keep f_i, those above `hi` get f_i / factor, a linear ramp lies between."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return out, ATTN_FACTOR_COEF * math.log(factor) + 1.0


def rotate_half(t, pos, freqs, mult):
    """t [T, ..., dims]: coordinate i is paired with i + dims/2 and the pair is turned by pos * f_i; cos and sin times `mult`."""
    half = len(freqs)
    a = torch.tensor([[p * f for f in freqs] for p in pos], dtype=F64)
    while a.dim() < t.dim():
        a = a.unsqueeze(1)
    c, s = torch.cos(a) * mult, torch.sin(a) * mult
    u, v = t[..., :half], t[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, t[..., 2 * half:]], -1)


def softmax_with_sink(scores, sink):
    """scores [n] of the visible keys; the denominator holds one more term exp(sink) that has no value."""
    m = max(float(scores.max()), float(sink))
    e = torch.exp(scores - m)
    return e / (e.sum() + math.exp(float(sink) - m))


def latent_attention(W, p, h, m, eps):
    """h [T, width] of one sequence from its first token -> [T, width]."""
    T = h.shape[0]
    H, D, R, V, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = m["rot"]
    freqs, mult = scaled_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    pos = list(range(T))
    cq = norm_plain(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_half(q[..., D:], pos, freqs, mult)
    dkv = h @ W[p + "dkv"].T
    c = norm_plain(dkv[:, :C], W[p + "dkv.norm"], eps)
    k_rot = rotate_half(dkv[:, C:], pos, freqs, mult)            # [T, R], one for all heads
    k_plain = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, V)
    gate = torch.sigmoid(h @ W[p + "g"].T)                          # [T, H]
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        for hd in range(H):
            s = (k_plain[:i + 1, hd] @ q_plain[i, hd] + k_rot[:i + 1] @ q_rot[i, hd]) * float(m["scale"])
            out[i, hd] = softmax_with_sink(s, W[p + "sink"][hd]) @ v[:i + 1, hd]
    out = out * gate[:, :, None]
    return out.reshape(T, H * V) @ W[p + "o"].T


def decays(W, p, h, m):
    """alpha [T, H, D] = sigmoid(z)^(1/tau), z = A2 (A1 h) + b."""
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    return torch.exp(torch.nn.functional.logsigmoid(z) / float(m["tau"])).view(h.shape[0], int(m["heads"]), int(m["dim"]))


def gla_recurrence(q, k, v, alpha):
    """q, k, alpha [T, H, D], v [T, H, V]: S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=F64)
    out = []
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def gla(W, p, h, m, eps):
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, D)
    v = (h @ W[p + "v"].T).view(T, H, V)
    o = gla_recurrence(q, k, v, decays(W, p, h, m))
    o = norm_plain(o, W[p + "norm"], eps).reshape(T, H * V)
    return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def dense_ff(W, p, h):
    g = h @ W[p + "gate"].T + W[p + "gate.b"]
    u = h @ W[p + "up"].T + W[p + "up.b"]
    return (silu(g) * u) @ W[p + "down"].T + W[p + "down.b"]


def expert(W, p, h, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(SWISH_ALPHA * g) * (u + 1.0)) @ W[p + "down"].T


def route(z, top):
    """z [E] -> (indices of the `top` largest, softmax over those alone)."""
    order = sorted(range(z.shape[0]), key=lambda e: (-float(z[e]), e))[:top]
    return order, torch.softmax(z[order], 0)


def moe_ff(W, p, h, f):
    top, limit = int(f["router"]["top"]), float(f["expert"]["limit"])
    z = h @ W[p + "router"].T + W[p + "router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        idx, wgt = route(z[t], top)
        for e, w in zip(idx, wgt):
            out[t] += w * expert(W, f"{p}e{e}.", h[t], limit)
    return out


def forward(cfg, weights, tokens, trace=None):
    """logits [T, vocab] of one sequence; `trace` (a list) receives each layer's result X_(i+1)."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    results = [x]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mixer = {"latent_attention": latent_attention, "gla": gla}[layer["type"]]
        x = x + norm_around_zero(mixer(W, p + "mix.", norm_around_zero(x, W[p + "norm1"], eps), layer["mixer"], eps), W[p + "norm1b"], eps)
        f = layer.get("mlp")
        if f is not None:
            hin = norm_around_zero(x, W[p + "norm2"], eps)
            y = dense_ff(W, p + "mlp.", hin) if f["kind"] == "dense" else moe_ff(W, p + "mlp.", hin, f)
            x = x + norm_around_zero(y, W[p + "norm2b"], eps)
        results.append(x)
        if trace is not None:
            trace.append(x)
        a = W[p + "dwa"]
        x = sum(a[j] * results[j] for j in range(i + 2))
    return norm_around_zero(x, W["final.norm"], eps) @ W["head"].T


# ---- small random models --------------------------------------------------------------------------------------------
def latent_layer(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=10, q_rank=12, scaling=True, base=1000.0, mlp="dense", ff=24, scale=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 0.5}
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "rot": rot,
         "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
    return {"type": "latent_attention", "mixer": m, "mlp": ff_entry(mlp, ff)}


def gla_layer(heads=2, dim=8, vdim=12, tau=8.0, low_rank=5, mlp="moe", ff=16, experts=5, top=2, limit=1.5):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "low_rank": low_rank},
            "mlp": ff_entry(mlp, ff, experts, top, limit)}


def ff_entry(kind, ff=16, experts=5, top=2, limit=1.5):
    if kind is None:
        return None
    if kind == "dense":
        return {"kind": "dense", "ff": ff}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def make_config(layers, width=40, vocab=61, eps=1e-5, embed_scale=3.0):
    cfg = {"architecture": "Safilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "layers": []}
    for layer in layers:
        layer = dict(layer)
        layer["mixer"] = {k: v for k, v in layer["mixer"].items() if k != "low_rank"}
        cfg["layers"].append(layer)
    cfg["_low_rank"] = [layer["mixer"].get("low_rank", 4) for layer in layers]
    return cfg


def random_model(cfg, seed=0, scale=0.5):
    """bfloat16-representable float32 tensors under the checkpoint's names.  Projections are scaled by fan-in so that activations
    stay of order one; sinks, decays' biases and router biases are spread so that they matter."""
    g = torch.Generator().manual_seed(seed)
    Wd, out = int(cfg["width"]), {}

    def rnd(*shape, s=1.0):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).to(torch.float32)

    def lin(o, i, s=1.0):
        return rnd(o, i, s=s * scale * 2.0 / math.sqrt(i))

    out["embed"] = rnd(int(cfg["vocab"]), Wd, s=0.5)
    out["head"] = lin(int(cfg["vocab"]), Wd)
    out["final.norm"] = rnd(Wd, s=0.2)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm2", "norm1b", "norm2b"):
            out[p + n] = rnd(Wd, s=0.2)
        out[p + "dwa"] = (torch.cat([rnd(i + 1, s=0.3 / (i + 1)), torch.ones(1) + rnd(1, s=0.1)])).to(torch.bfloat16).to(torch.float32)
        if layer["type"] == "latent_attention":
            H, D, R, V, C, Q = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
            out[p + "mix.dq"], out[p + "mix.dq.norm"] = lin(Q, Wd), 1.0 + rnd(Q, s=0.2)
            out[p + "mix.uq"] = lin(H * (D + R), Q, s=2.0)
            out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = lin(C + R, Wd, s=2.0), 1.0 + rnd(C, s=0.2)
            out[p + "mix.uk"], out[p + "mix.uv"] = lin(H * D, C, s=2.0), lin(H * V, C)
            out[p + "mix.sink"] = rnd(H, s=1.5)
            out[p + "mix.g"] = lin(H, Wd, s=2.0)
            out[p + "mix.o"] = lin(Wd, H * V)
        else:
            H, D, V = (int(m[k]) for k in ("heads", "dim", "vdim"))
            r = cfg.get("_low_rank", [4] * len(cfg["layers"]))[i]
            for n, rows in (("q", H * D), ("k", H * D), ("v", H * V), ("g", H * V)):
                out[p + "mix." + n] = lin(rows, Wd, s=1.5)
            out[p + "mix.o"] = lin(Wd, H * V)
            out[p + "mix.norm"] = 1.0 + rnd(V, s=0.2)
            out[p + "mix.a1"], out[p + "mix.a2"] = lin(r, Wd), lin(H * D, r, s=3.0)
            out[p + "mix.a2.b"] = rnd(H * D, s=2.0) + 1.0
        f = layer.get("mlp")
        if f is None:
            continue
        if f["kind"] == "dense":
            ff = int(f["ff"])
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = lin(ff, Wd), lin(ff, Wd), lin(Wd, ff)
            out[p + "mlp.gate.b"], out[p + "mlp.up.b"], out[p + "mlp.down.b"] = rnd(ff, s=0.3), rnd(ff, s=0.3), rnd(Wd, s=0.3)
        else:
            ff, E = int(f["expert"]["ff"]), int(f["router"]["experts"])
            for e in range(E):
                out[f"{p}mlp.e{e}.gate"], out[f"{p}mlp.e{e}.up"], out[f"{p}mlp.e{e}.down"] = lin(ff, Wd, s=2.0), lin(ff, Wd, s=2.0), lin(Wd, ff)
            out[p + "mlp.router"], out[p + "mlp.router.b"] = lin(E, Wd, s=2.0), rnd(E, s=0.5)
    for k in list(out):
        out[k] = out[k].to(torch.bfloat16).to(torch.float32)
    return out
