"""The Safilorn design on the GPU against the float64 oracle (tests/safilorn_oracle.py): each mechanism alone through the
kernels' bindings, then whole models through the step function, the batch engine, the generation engine and bin/trace_run."""
import json
import math
import os
import subprocess

import pytest
import torch

from tests import safilorn_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16, F64 = torch.float32, torch.bfloat16, torch.float64
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def nsq():
    from promptcache_b200 import _native_seq
    _native_seq.load()
    return _native_seq


def dev(t, dtype=F32):
    return t.to(DEV, dtype).contiguous()


def close(got, want, tol, what=""):
    got, want = got.detach().cpu().to(F64), want.to(F64)
    err = float((got - want).abs().max() / (want.abs().max() + 1e-30))
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"
    return err


def close_rows(got, want, tol, what="", share=0.85, worst=0.6):
    """bfloat16 runs of whole models: a rounding can flip a router's choice between two near-equal experts, which moves that
    token's logits by far more than rounding does.  Rows are judged one by one: most within `tol` (relative rms), none beyond `worst`."""
    got, want = got.detach().cpu().to(F64), want.detach().cpu().to(F64)
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()
    ok = float((err <= tol).double().mean())
    assert ok >= share and float(err.max()) <= worst, f"{what}: {ok:.2f} of the rows within {tol:.1e}, worst {float(err.max()):.3e}"


def write_checkpoint(folder, cfg, W):
    from promptcache_b200 import weights as wio
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump({k: v for k, v in cfg.items() if not k.startswith("_")}, fh)
    wio.save_file({k: (v.to(torch.int32) if not v.is_floating_point() else v.to(BF16)) for k, v in W.items()}, os.path.join(folder, "model.safetensors"))


def load(tmp_path, cfg, W, dtype=F32, name="m"):
    from promptcache_b200.model import load_model
    folder = str(tmp_path / name)
    write_checkpoint(folder, cfg, W)
    return load_model(folder, device=DEV, dtype=dtype)


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def batch_of(nsq, slots, pos0, lens):
    return nsq.Batch(slots, pos0, lens, torch.device(DEV))


# ---- mechanisms alone ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("width", [40, 37])
def test_depth_average_and_norms_around_zero(nsq, width):
    g = torch.Generator().manual_seed(width)
    T, n = 9, 4
    xs = torch.randn(n + 1, T, width, generator=g, dtype=F64)
    a, w = torch.randn(n, generator=g, dtype=F64), torch.randn(width, generator=g, dtype=F64) * 0.3
    want = sum(a[j] * xs[j] for j in range(n))
    xo, h = torch.empty(T, width, device=DEV), torch.empty(T, width, device=DEV)
    nsq.depth_mix(dev(xs), n, dev(a), 1e-5, x_out=xo, next_w=dev(w), h_out=h, w_offset=1.0)
    close(xo, want, 2e-6, "weighted sum of the earlier results")
    close(h, O.norm_around_zero(want, w, 1e-5), 2e-6, "norm of the sum")
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    hr = torch.empty(3, width, device=DEV)
    nsq.depth_mix(dev(xs), n, dev(a), 1e-5, next_w=dev(w), h_out=hr, w_offset=1.0, rows=rows)
    close(hr, O.norm_around_zero(want[[7, 0, 3]], w, 1e-5), 2e-6, "only the wanted rows")
    # a sublayer's residual sum riding in the same launch: the newest term is updated in place first
    yv, w3 = torch.randn(T, width, generator=g, dtype=F64), torch.randn(width, generator=g, dtype=F64) * 0.3
    for ydt, wdt in ((F32, F32), (BF16, BF16), (F32, BF16)):
        xs2 = dev(xs)
        xo2, h2 = torch.empty(T, width, device=DEV), torch.empty(T, width, device=DEV, dtype=wdt)
        nsq.depth_mix(xs2, n, dev(a), 1e-5, x_out=xo2, next_w=dev(w, wdt), h_out=h2, w_offset=1.0, y=dev(yv, ydt), y_w=dev(w3, wdt))
        newest = xs[n - 1] + O.norm_around_zero(yv.to(ydt).to(F64), w3.to(wdt).to(F64), 1e-5)
        want2 = sum(a[j] * xs[j] for j in range(n - 1)) + a[n - 1] * newest
        close(xs2[n - 1], newest, 2e-6, "newest term after its residual sum")
        close(xs2[:n - 1], xs[:n - 1].to(F32), 0, "older terms untouched")
        close(xo2, want2, 3e-6, "average over the updated term")
        close(h2, O.norm_around_zero(want2, w.to(wdt).to(F64), 1e-5), 2e-6 if wdt == F32 else 6e-3, "norm of it")
    # the sublayer's output norm, the residual sum and the next input norm, with the 1 added in 32-bit
    x, y, w2 = torch.randn(T, width, generator=g, dtype=F64), torch.randn(T, width, generator=g, dtype=F64), torch.randn(width, generator=g, dtype=F64) * 0.3
    for ydt in (F32, BF16):
        for wdt in ((F32,) if ydt == F32 else (BF16,)):
            xd, hd = dev(x), torch.empty(T, width, device=DEV, dtype=wdt)
            yq, wq, w2q = y.to(ydt).to(F64), w.to(wdt).to(F64), w2.to(wdt).to(F64)
            nsq.gate_norm_add(xd, dev(y, ydt), None, dev(w, wdt), None, 1e-5, dev(w2, wdt), hd, w_offset=1.0)
            xn = x + O.norm_around_zero(yq, wq, 1e-5)
            close(xd, xn, 2e-6, "x += (1 + w) rms(y)")
            close(hd, O.norm_around_zero(xn, w2q, 1e-5), 2e-6 if wdt == F32 else 6e-3, "next input norm")
    # a 32-bit sublayer result under bfloat16 weights (the experts' weighted sum)
    xd = dev(x)
    nsq.gate_norm_add(xd, dev(y), None, dev(w, BF16), None, 1e-5, w_offset=1.0)
    close(xd, x + O.norm_around_zero(y, w.to(BF16).to(F64), 1e-5), 2e-6, "32-bit y, bfloat16 weights")


def test_rescaled_frequencies_match_the_oracle():
    from promptcache_b200.model.safilorn import ramp_scaled_frequencies
    for dims, base, sc in [(8, 1000.0, {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 0.5}), (32, 50000.0, {"factor": 16.0, "original": 512, "fast": 8.0, "slow": 2.0}),
                           (6, 10000.0, None), (4, 100.0, {"factor": 1.0, "original": 8, "fast": 2.0, "slow": 1.0})]:
        f, m = ramp_scaled_frequencies(dims, base, sc)
        fo, mo = O.scaled_frequencies(dims, base, sc)
        assert len(f) == dims // 2 and all(abs(a - b) <= 1e-15 * abs(b) for a, b in zip(f, fo)) and abs(m - mo) < 1e-15
    f, m = ramp_scaled_frequencies(32, 50000.0, {"factor": 16.0, "original": 512, "fast": 8.0, "slow": 2.0})
    plain = [50000.0 ** (-2.0 * i / 32) for i in range(16)]
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 16.0) < 1e-18 and any(p / 16.0 < a < p for a, p in zip(f, plain))   # kept, divided, a ramp between
    assert abs(m - (0.1 * math.log(16.0) + 1.0)) < 1e-15


@pytest.mark.parametrize("C,R,Q,H,D", [(10, 4, 12, 3, 8), (16, 8, 24, 2, 8), (5, 2, 3, 1, 3), (7, 0, 6, 2, 5)])
def test_latent_norms_rotation_and_append(nsq, C, R, Q, H, D):
    g = torch.Generator().manual_seed(C * 100 + R)
    lens, pos0, slots, cap = [5, 3], [0, 9], [2, 0], 16
    T = sum(lens)
    b = batch_of(nsq, slots, pos0, lens)
    pos = list(range(5)) + list(range(9, 12))
    freqs, mult = O.scaled_frequencies(R, 300.0, {"factor": 4.0, "original": 8, "fast": 2.0, "slow": 0.5}) if R else ([], 1.0)
    fr = torch.tensor(freqs, dtype=F64, device=DEV) if R else None
    proj = torch.randn(T, 3 + Q + C + R + 2, generator=g, dtype=F64)
    wq, wc = torch.randn(Q, generator=g, dtype=F64), torch.randn(C, generator=g, dtype=F64)
    pool = torch.full((3, 1, cap, C + R), 7.0, device=DEV)
    cq = torch.empty(T, Q, device=DEV)
    nsq.latent_prep(dev(proj), 3, 3 + Q, Q, C, R, dev(wq), dev(wc), 1e-5, fr, mult, cq, pool, b)
    close(cq, O.norm_plain(proj[:, 3:3 + Q], wq, 1e-5), 2e-6, "query latent")
    c_want = O.norm_plain(proj[:, 3 + Q:3 + Q + C], wc, 1e-5)
    r_want = O.rotate_half(proj[:, 3 + Q + C:3 + Q + C + R], pos, freqs, mult) if R else torch.zeros(T, 0, dtype=F64)
    rows = torch.cat([pool[2, 0, 0:5], pool[0, 0, 9:12]])
    close(rows, torch.cat([c_want, r_want], 1), 2e-6, "appended [latent | rotated part] rows")
    assert float(pool[1].min()) == 7.0 and float(pool[0, 0, :9].min()) == 7.0 and float(pool[2, 0, 5:].min()) == 7.0   # nothing else was written
    # queries: rotated part in place, and packed beside latent-space queries
    q = torch.randn(T, H * (D + R), generator=g, dtype=F64)
    q3 = q.view(T, H, D + R)
    q_want = torch.cat([q3[..., :D], O.rotate_half(q3[..., D:], pos, freqs, mult) if R else q3[..., D:]], -1)
    qd = dev(q)
    assert nsq.latent_q(qd, H, D, R, fr, mult, b) is qd
    close(qd.view(T, H, D + R), q_want, 2e-6, "rotated query parts")
    ql = torch.randn(H, T, C, generator=g, dtype=F64)
    packed = nsq.latent_q(dev(q), H, D, R, fr, mult, b, q_lat=dev(ql).transpose(0, 1))
    close(packed.view(T, H, C + R), torch.cat([ql.transpose(0, 1), q_want[..., D:]], -1), 2e-6, "[latent query | rotated part]")
    # context rows out of the pool and per-head rows into a dense pool
    ctx = batch_of(nsq, slots, [0, 0], [5, 12])
    got = nsq.latent_gather(pool, C, ctx)
    close(got, torch.cat([pool[2, 0, :5, :C], pool[0, 0, :12, :C]]).cpu(), 0, "gathered latents")
    V = 6
    kv = torch.randn(17, H * (D + V), generator=g, dtype=F64)
    kd, vd = torch.zeros(2, H, 64, D + R, device=DEV), torch.zeros(2, H, 64, V, device=DEV)
    nsq.latent_expand(dev(kv), pool, C, R, H, D, V, kd, vd, ctx)
    k3, v3 = kv[:, :H * D].view(17, H, D), kv[:, H * D:].view(17, H, V)
    for e, (n0, n, slot) in enumerate([(0, 5, 2), (5, 12, 0)]):
        close(kd[e, :, :n, :D], k3[n0:n0 + n].transpose(0, 1), 2e-6, "plain key parts")
        close(kd[e, :, :n, D:], pool[slot, 0, :n, C:].cpu().unsqueeze(0).expand(H, n, R), 0, "shared rotated part") if R else None
        close(vd[e, :, :n], v3[n0:n0 + n].transpose(0, 1), 2e-6, "values")


def sink_attention(q, k, v, scale, sink, pos0=0):
    """q [T, H, D] at positions pos0.., k [N, G, D], v [N, G, V] -> [T, H, V] by the oracle's softmax."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        n = pos0 + i + 1
        for h in range(H):
            g = h // (H // G)
            out[i, h] = O.softmax_with_sink((k[:n, g] @ q[i, h]) * scale, sink[h]) @ v[:n, g]
    return out


@pytest.mark.parametrize("dtype,H,D,V,N,T", [(F32, 3, 12, 8, 70, 70), (F32, 2, 10, 7, 45, 3), (BF16, 4, 48, 32, 300, 300), (BF16, 2, 24, 40, 700, 1), (F32, 2, 16, 8, 700, 1),
                                              (BF16, 3, 64, 64, 200, 40), (BF16, 16, 72, 8, 700, 1), (BF16, 20, 40, 8, 130, 3), (BF16, 5, 264, 8, 90, 2)])
def test_attention_with_a_learned_sink_per_head(nsq, dtype, H, D, V, N, T):
    """Multi-head rows (the expanded form) and one shared row per key whose leading numbers are the values (the latent form)."""
    g = torch.Generator().manual_seed(N + T)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=F64).to(dtype).to(F64)
    sink = torch.tensor(([2.5, -1.0, 0.3, 6.0] * 5)[:H], dtype=F64)
    pos0, tol = N - T, (3e-6 if dtype == F32 else 1.2e-2)
    b = batch_of(nsq, [1], [pos0], [T])
    q, k, v = rnd(T, H, D) * 0.7, rnd(N, H, D), rnd(N, H, V)
    kp, vp = torch.zeros(2, H, 768, D, device=DEV, dtype=dtype), torch.zeros(2, H, 768, V, device=DEV, dtype=dtype)
    kp[1, :, :N], vp[1, :, :N] = dev(k.transpose(0, 1), dtype), dev(v.transpose(0, 1), dtype)
    out = torch.empty(T, H * V, device=DEV, dtype=dtype)
    ws = nsq.attn_workspace(T, H, V, torch.device(DEV)) if T <= 16 else None
    nsq.attention(dev(q.reshape(T, H * D), dtype), kp, vp, out, H, 0.3, None, None, True, b, sink_logit=dev(sink), max_keys=768, workspace=ws)
    want = sink_attention(q, k, v, 0.3, sink, pos0)
    close(out.view(T, H, V), want, tol, "per-head rows")
    for impl in (1,):
        nsq.attention(dev(q.reshape(T, H * D), dtype), kp, vp, out, H, 0.3, None, None, True, b, sink_logit=dev(sink), impl=impl)
        close(out.view(T, H, V), want, tol, "per-head rows, plain kernel")
    # one row per key, shared by the heads; the values are its first V numbers
    rows = rnd(N, 1, D)
    pool = torch.zeros(2, 1, 768, D, device=DEV, dtype=dtype)
    pool[1, 0, :N] = dev(rows[:, 0], dtype)
    Vl = D - 8 if D >= 16 else D - 4
    out = torch.empty(T, H * Vl, device=DEV, dtype=dtype)
    ws = nsq.attn_workspace(T, H, Vl, torch.device(DEV)) if T <= 16 else None
    nsq.attention(dev(q.reshape(T, H * D), dtype), pool, pool, out, H, 0.3, None, None, True, b, sink_logit=dev(sink), v_row_stride=D, max_keys=768, workspace=ws)
    close(out.view(T, H, Vl), sink_attention(q, rows, rows[..., :Vl], 0.3, sink, pos0), tol, "shared rows, values inside the key rows")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_far_key_and_sink_decide(nsq, dtype):
    """One key far back answers the query (its score stands out among hundreds); then the sink outweighs every key."""
    H, D, V, N = 2, 16, 8, 600
    g = torch.Generator().manual_seed(5)
    k, v = torch.randn(N, H, D, generator=g, dtype=F64) * 0.1, torch.randn(N, H, V, generator=g, dtype=F64)
    q = torch.randn(1, H, D, generator=g, dtype=F64) * 0.1
    far = 3
    k[far] = q[0] * 300.0
    k, v, q = (t.to(dtype).to(F64) for t in (k, v, q))
    kp, vp = torch.zeros(1, H, 640, D, device=DEV, dtype=dtype), torch.zeros(1, H, 640, V, device=DEV, dtype=dtype)
    kp[0, :, :N], vp[0, :, :N] = dev(k.transpose(0, 1), dtype), dev(v.transpose(0, 1), dtype)
    out = torch.empty(1, H * V, device=DEV, dtype=dtype)
    b = batch_of(nsq, [0], [N - 1], [1])
    ws = nsq.attn_workspace(1, H, V, torch.device(DEV))
    tol = 3e-6 if dtype == F32 else 1e-2
    for sink, what in ((torch.tensor([0.0, -2.0], dtype=F64), "the far key"), (torch.tensor([80.0, 90.0], dtype=F64), "the sink")):
        nsq.attention(dev(q.reshape(1, H * D), dtype), kp, vp, out, H, 1.0, None, None, True, b, sink_logit=dev(sink), max_keys=640, workspace=ws)
        want = sink_attention(q, k, v, 1.0, sink, N - 1)
        close(out.view(1, H, V), want, tol, what)
        if what == "the far key":
            close(out.view(1, H, V), v[far].unsqueeze(0), 0.3, "the result is the far key's value")
        else:
            assert float(out.float().abs().max()) < 1e-3 * float(v.abs().max())   # the sink has no value


def test_head_gate(nsq):
    g = torch.Generator().manual_seed(1)
    o, gt = torch.randn(3, 7, 5, generator=g, dtype=F64), torch.randn(7, 10, generator=g, dtype=F64)
    out = torch.empty(7, 15, device=DEV)
    nsq.head_gate(dev(o).transpose(0, 1), dev(gt)[:, 4:7], out)
    close(out.view(7, 3, 5), o.transpose(0, 1) * torch.sigmoid(gt[:, 4:7])[:, :, None], 2e-6, "sigmoid gate per head")


@pytest.mark.parametrize("dtype,H,D,V,r,tau", [(F32, 2, 8, 12, 5, 8.0), (F32, 3, 7, 5, 3, 2.0), (BF16, 4, 64, 64, 16, 16.0), (F32, 2, 128, 40, 8, 4.0), (BF16, 1, 32, 8, 1, 1.0),
                                                (F32, 1, 260, 16, 4, 16.0)])
def test_gated_linear_attention_in_portions(nsq, dtype, H, D, V, r, tau):
    """The decays and the recurrence against the oracle: a prompt at once, in portions down to one token, two entries in a batch,
    the state carried in the pool; token by token (state in registers / in shared memory) and in chunks of 64 tokens."""
    g = torch.Generator().manual_seed(D + V)
    T = 150
    rq = lambda *s, sc=1.0: (torch.randn(*s, generator=g, dtype=F64) * sc).to(dtype).to(F64)
    proj = rq(T, 2 * H * D + 2 * H * V + r + 8, sc=0.6)
    offs, a_off = (0, H * D, 2 * H * D, 2 * H * D + H * V), 2 * H * D + 2 * H * V + 8
    a2, a2b, nw = rq(H * D, r, sc=1.5), torch.randn(H * D, generator=g, dtype=F64) + 1.0, rq(V, sc=0.3) + 1.0
    a2b = a2b.to(F32).to(F64)
    z = proj[:, a_off:a_off + r] @ a2.T + a2b
    ld_want = torch.nn.functional.logsigmoid(z) / tau
    ld = nsq.gla_decay(dev(proj, dtype)[:, a_off:a_off + r], dev(a2, dtype), dev(a2b), tau)
    close(ld, ld_want, 3e-6, "log decays")
    q, k = proj[:, :H * D].view(T, H, D) * D ** -0.5, proj[:, H * D:2 * H * D].view(T, H, D)
    v, gate = proj[:, offs[2]:offs[2] + H * V].view(T, H, V), proj[:, offs[3]:offs[3] + H * V]
    o = O.gla_recurrence(q, k, v, torch.exp(ld_want).view(T, H, D))
    want = O.norm_plain(o, nw, 1e-5).reshape(T, H * V) * O.silu(gate)
    tol = 2e-5 if dtype == F32 else 1.2e-2
    pd = dev(proj, dtype)
    for impl in (0, 1, 2, 3):
        for cuts in ([T], [1] * T, [17, 2, 1, 130], [2] * 75, [10, 140], [64, 64, 22], [63, 65, 22]):
            if impl in (1, 3) and len(cuts) > 10:
                continue
            pool = torch.full((3, H, D, V), 9.0, device=DEV)   # a slot that was used before: a first token starts from zero all the same
            out, p0 = torch.empty(T, H * V, device=DEV, dtype=dtype), 0
            for n in cuts:
                nsq.gla_scan(pd[p0:p0 + n], offs, ld[p0:p0 + n], dev(nw, dtype), out[p0:p0 + n], pool, 1e-5, batch_of(nsq, [1], [p0], [n]), impl=impl)
                p0 += n
            close(out, want, tol, f"impl {impl}, portions {cuts[:4]}")
    # two entries of unequal length in one launch, the second continuing from a state
    pool = torch.zeros(4, H, D, V, device=DEV)
    out = torch.empty(T, H * V, device=DEV, dtype=dtype)
    for impl in (2, 3):
        nsq.gla_scan(pd[:20], offs, ld[:20], dev(nw, dtype), out[:20], pool, 1e-5, batch_of(nsq, [3], [0], [20]), impl=impl)
        cat = torch.cat([pd[:7], pd[20:]])
        out2 = torch.empty(7 + T - 20, H * V, device=DEV, dtype=dtype)
        nsq.gla_scan(cat, offs, torch.cat([ld[:7], ld[20:]]), dev(nw, dtype), out2, pool, 1e-5, batch_of(nsq, [0, 3], [0, 20], [7, T - 20]), impl=impl)
        close(out2[:7], want[:7], tol, f"a fresh entry beside a continued one (impl {impl})")
        close(out2[7:], want[20:], tol, f"the continued entry (impl {impl})")


def test_decay_separates_channels(nsq):
    """A key channel whose decay is near zero forgets at once, one near one keeps everything: the result shows which is which."""
    H, D, V, T = 1, 4, 4, 30
    proj = torch.zeros(T, 2 * D + 2 * V, dtype=F64)
    proj[:, :D] = 2.0                                   # q: all ones after the D^(-1/2) scale
    proj[0, D:2 * D] = torch.tensor([1.0, 1.0, 0.0, 0.0])   # only the first token writes: channels 0 and 1
    proj[0, 2 * D:2 * D + V] = torch.tensor([1.0, 2.0, 3.0, 4.0])
    proj[:, 2 * D + V:] = 30.0                          # silu gate ~ 30
    ld = torch.zeros(T, D, dtype=F64)
    ld[1:, 0], ld[1:, 1] = -50.0, -1e-4                 # channel 0 forgets, channel 1 keeps
    pool = torch.zeros(1, H, D, V, device=DEV)
    out = torch.empty(T, V, device=DEV)
    o = O.gla_recurrence(proj[:, :D].view(T, 1, D) * 0.5, proj[:, D:2 * D].view(T, 1, D), proj[:, 2 * D:2 * D + V].view(T, 1, V), torch.exp(ld).view(T, 1, D))
    for impl in (2, 3):   # token by token, and in chunks (a decay of e^-50 per token must not overflow any factor)
        pool.zero_()
        nsq.gla_scan(dev(proj), (0, D, 2 * D, 2 * D + V), dev(ld), torch.ones(V, device=DEV), out, pool, 0.0, batch_of(nsq, [0], [0], [T]), impl=impl)
        close(out, O.norm_plain(o, torch.ones(V, dtype=F64), 0.0).reshape(T, V) * O.silu(proj[:, 2 * D + V:]), 1e-5, f"two channels (impl {impl})")
        s = pool[0, 0].cpu().to(F64)
        assert float(s[0].abs().max()) < 1e-30 and abs(float(s[1, 3]) - 4.0 * math.exp(-29e-4)) < 1e-4 and float(s[2:].abs().max()) == 0.0


@pytest.mark.parametrize("E,top,T,W", [(5, 2, 9, 40), (10, 3, 70, 64), (1, 1, 4, 24), (7, 7, 5, 36), (300, 4, 6, 32)])
def test_router_with_bias_and_weights_over_the_chosen(nsq, E, top, T, W):
    g = torch.Generator().manual_seed(E * 10 + top)
    h, wr, b = torch.randn(T, W, generator=g, dtype=F64), torch.randn(E, W, generator=g, dtype=F64) * 0.4, torch.randn(E, generator=g, dtype=F64)
    idx, wgt, _ = nsq.moe_route(dev(h), dev(wr), None, None, top, bias=dev(b), renorm=True)
    z = h @ wr.T + b
    for t in range(T):
        wi, ww = O.route(z[t], top)
        assert idx[t].tolist() == wi, f"token {t}: chosen {idx[t].tolist()}, expected {wi}"
        close(wgt[t], ww, 3e-6, "softmax over the chosen logits")
    # a bias that decides: without it another expert wins
    if E >= 2:
        b2 = torch.zeros(E, dtype=F64)
        b2[E - 1] = 100.0
        idx, wgt, _ = nsq.moe_route(dev(h), dev(wr), None, None, 1, bias=dev(b2), renorm=True)
        assert idx.flatten().tolist() == [E - 1] * T and float((wgt - 1).abs().max()) < 1e-6


@pytest.mark.parametrize("T,ff,W,limit", [(5, 16, 40, 1.5), (3, 13, 30, 0.7), (150, 64, 128, 1.0)])
def test_experts_with_clamped_gate_and_up(nsq, T, ff, W, limit):
    g = torch.Generator().manual_seed(T + ff)
    E, top = 6, 3
    rq = lambda *s, sc=1.0: (torch.randn(*s, generator=g, dtype=F64) * sc).to(BF16).to(F64)
    h, wg, wu, wd = rq(T, W), rq(E, ff, W, sc=0.5), rq(E, ff, W, sc=0.5), rq(E, W, ff, sc=0.3)   # gates and ups reach past the limits
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    Wd = {}
    for e in range(E):
        Wd[f"e{e}.gate"], Wd[f"e{e}.up"], Wd[f"e{e}.down"] = wg[e], wu[e], wd[e]
    want = torch.stack([torch.stack([O.expert(Wd, f"e{int(e)}.", h[t], limit) for e in idx[t]]) for t in range(T)]).view(T * top, W)
    assert float((h @ wg[0].T).max()) > limit and float((h @ wu[0].T).abs().max()) > limit
    act = (nsq.GLU_CLAMPED_SWISH, O.SWISH_ALPHA, limit)
    wgu = torch.cat([wg, wu], 1)
    y, rows = nsq.moe_experts(dev(h), dev(idx, torch.int32), dev(wgu), dev(wd), grouped=False, act=act)
    assert rows is None
    close(y, want, 3e-6, "row kernels, float32")
    if ff % 8 == 0 and W % 8 == 0:
        for mode in ("own", "library"):
            if mode == "library" and not hasattr(torch.nn.functional, "grouped_mm"):
                continue
            y, rows = nsq.moe_experts(dev(h, BF16), dev(idx, torch.int32), dev(wgu, BF16), dev(wd, BF16), grouped=mode, act=act)
            y = y.float() if rows is None else y.float()[rows.long()]
            close(y, want, 1.5e-2, f"grouped products ({mode}), bfloat16")
    gu = torch.randn(T, 2 * ff, generator=g, dtype=F64) * 2
    gg, uu = torch.clamp(gu[:, :ff], max=limit), torch.clamp(gu[:, ff:], -limit, limit)
    close(nsq.glu_mul(dev(gu), ff, act), gg * torch.sigmoid(O.SWISH_ALPHA * gg) * (uu + 1), 3e-6, "clamped swish")
    close(nsq.glu_mul(dev(gu), ff), O.silu(gu[:, :ff]) * gu[:, ff:], 3e-6, "silu(gate) * up")


# ---- whole models ---------------------------------------------------------------------------------------------------
def layer_sets():
    A, G = O.latent_layer, O.gla_layer
    return {
        "mixed": [A(), G(), G(heads=3, dim=8, vdim=8, tau=3.0, mlp="dense", ff=24), A(heads=2, dim=16, rot_dim=8, vdim=8, kv_rank=24, q_rank=16, scaling=False, mlp="moe"),
                  G(mlp=None, tau=20.0)],
        # sizes that are not multiples of the 16-byte pieces: every kernel's plain path; one head, one expert, top = experts
        "odd": [G(heads=1, dim=6, vdim=10, tau=1.0, low_rank=1, mlp="moe", ff=10, experts=3, top=3, limit=0.6), A(heads=1, dim=5, rot_dim=6, vdim=7, kv_rank=9, q_rank=5, mlp="moe", ff=12),
                A(heads=5, dim=6, rot_dim=2, vdim=3, kv_rank=4, q_rank=7, mlp=None), G(heads=3, dim=5, vdim=3, mlp="moe", experts=1, top=1, ff=7)],
        "attention_only": [A(mlp="moe"), A(heads=4, dim=8, rot_dim=8, vdim=16, kv_rank=8, q_rank=8, base=50.0)],
        "recurrent_only": [G(mlp="dense"), G(heads=4, dim=16, vdim=8, low_rank=3)],
        # a latent wider than the decoding kernels' value rows: the expanded form serves decoding too
        "wide_latent": [A(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=520, q_rank=8), G(mlp=None)],
    }


@pytest.mark.parametrize("name,width", [("mixed", 40), ("mixed", 24), ("odd", 30), ("odd", 37), ("attention_only", 64), ("recurrent_only", 48), ("wide_latent", 32)])
def test_model_whole_prompt_against_oracle(tmp_path, name, width):
    cfg = O.make_config(layer_sets()[name], width=width, embed_scale=width ** 0.5)
    W = O.random_model(cfg, seed=width)
    toks = tokens(45, cfg["vocab"], 2)
    trace = []
    want = O.forward(cfg, W, toks, trace)
    for form in ("expanded", "latent"):
        m = load(tmp_path, cfg, W, F32, form)
        m.latent_form, m.layer_trace = form, []
        got = m.step([(m.new_sequence(), toks)], [list(range(len(toks)))])
        for i in range(len(trace)):   # the stream that goes on after layer i: the depth average over X_0 .. X_(i+1)
            a = W[f"l{i}.dwa"].to(F64)
            xs = [W["embed"].to(F64)[torch.tensor(toks)] * cfg["embedding"]["scale"]] + trace
            close(m.layer_trace[i], sum(a[j] * xs[j] for j in range(i + 2)), 3e-5, f"stream after layer {i} ({form})")
        close(got, want, 5e-5, f"logits, float32 ({form})")
    seq = m.new_sequence()   # (the last float32 model) prompt, then token by token
    got = torch.cat([m.step([(seq, toks[:20])], [list(range(20))])] + [m.step([(seq, [t])]) for t in toks[20:]])
    close(got, want, 5e-5, "logits, float32, decoded")
    mb = load(tmp_path, cfg, W, BF16, "b")
    gb = mb.step([(mb.new_sequence(), toks)], [list(range(len(toks)))])
    # (heads of five or six numbers and three-way routers make bfloat16 rounding and flipped choices weigh more in the odd set)
    close_rows(gb, want, 4e-2, "logits, bfloat16", share=0.5 if name == "odd" else 0.7)


@pytest.mark.parametrize("dtype,tol", [(F32, 5e-5), (BF16, 6e-2)])
def test_portions_decoding_batches_and_slot_reuse(tmp_path, dtype, tol):
    """One set of sequences run whole, in portions of several sizes down to two tokens, token by token (through the
    replayed graph), in unequal batches whose shorter members leave early, and through slots that were used before."""
    cfg = O.make_config(layer_sets()["mixed"])
    W = O.random_model(cfg, seed=11)
    V = cfg["vocab"]
    seqs = [tokens(n, V, 20 + n) for n in (61, 9, 30, 1)]
    want = [O.forward(cfg, W, s) for s in seqs]
    m = load(tmp_path, cfg, W, dtype)
    # bfloat16 on heads of eight numbers: a layer adds about one percent of rounding noise, five layers and the depth average
    # two to three, a flipped expert choice more; the float32 run is the sharp one
    cmp = close if dtype == F32 else (lambda g_, w_, t_, s_: close_rows(g_, w_, t_, s_, share=0.7))

    def run(toks, cuts):
        seq, out, p = m.new_sequence(), [], 0
        for n in cuts:
            out.append(m.step([(seq, toks[p:p + n])], [list(range(n))]))
            p += n
        seq.free()
        return torch.cat(out)

    for cuts in ([61], [2] * 30 + [1], [1] * 61, [17, 2, 3, 1, 1, 30, 7], [40] + [1] * 21, [20, 25, 16]):
        cmp(run(seqs[0], cuts), want[0], tol, f"portions {cuts[:6]}...")
    # unequal batch: prompts together, then decoded together; the short ones leave earlier
    from promptcache_b200.batch_engine import BatchEngine
    eng = BatchEngine(m)
    pre = [40, 4, 22, 1]
    got = [[] for _ in seqs]
    lg = eng.step([(f"r{i}", s[:n], list(range(n))) for i, (s, n) in enumerate(zip(seqs, pre))])
    o = 0
    for i, n in enumerate(pre):
        got[i].append(lg[o:o + n])
        o += n
    at = list(pre)
    while any(a < len(s) for a, s in zip(at, seqs)):
        live = [i for i, s in enumerate(seqs) if at[i] < len(s)]
        done = [f"r{i}" for i in live if at[i] + 1 == len(seqs[i])]
        lg = eng.step([(f"r{i}", [seqs[i][at[i]]], [0]) for i in live], done)
        for k_, i in enumerate(live):
            got[i].append(lg[k_:k_ + 1])
            at[i] += 1
    eng.end("r3")
    for i in range(len(seqs)):
        cmp(torch.cat(got[i]), want[i], tol, f"request {i} in a batch")
    # the freed slots are handed out again, to other sequences and in another order
    lg = eng.step([("x", seqs[2], None), ("y", seqs[0], None), ("z", seqs[1], None)], ["x", "y", "z"])
    ref = torch.stack([want[2][-1], want[0][-1], want[1][-1]])
    if dtype == F32:
        close(lg, ref, tol, "reused slots")
    else:
        close_rows(lg, ref, 0.1, "reused slots", share=0.6)


def test_long_decoding_and_pool_growth(tmp_path):
    """300 tokens decoded one by one after a short prompt: the pool grows twice while the sequence lives (captured graphs are
    rebuilt, the decoding attention splits the keys), and a second sequence joins and leaves."""
    cfg = O.make_config([O.latent_layer(), O.gla_layer(tau=6.0), O.latent_layer(heads=2, dim=16, rot_dim=8, vdim=8, kv_rank=24, q_rank=8, mlp=None)])
    W = O.random_model(cfg, seed=3)
    toks = tokens(330, cfg["vocab"], 8)
    want = O.forward(cfg, W, toks)
    m = load(tmp_path, cfg, W, F32)
    seq = m.new_sequence()
    out = [m.step([(seq, toks[:30])], [list(range(30))])]
    other = None
    for p in range(30, 330):
        if p == 100:
            other = m.new_sequence()
            m.step([(other, toks[:50])])
        if other is not None and 100 <= p < 140:
            lg = m.step([(seq, [toks[p]]), (other, [toks[p - 50]])])
            close(lg[1], want[p - 50], 5e-5, f"second sequence at {p - 50}")
            out.append(lg[:1])
        else:
            if other is not None and p == 140:
                other.free()
            out.append(m.step([(seq, [toks[p]])]))
    close(torch.cat(out), want, 5e-5, "long decoding")


def test_medium_model_long_prompt(tmp_path):
    """Sizes at which the other code paths run: 64-wide heads on the tensor-core kernel over twenty key tiles, the register scan,
    decoding that splits the keys, hundreds of pairs per expert through the grouped products."""
    A, G = O.latent_layer, O.gla_layer
    cfg = O.make_config([A(heads=4, dim=48, rot_dim=16, vdim=64, kv_rank=96, q_rank=64, base=10000.0, mlp="moe", ff=128, scale=0.2),
                         G(heads=4, dim=64, vdim=64, tau=12.0, low_rank=8, mlp="moe", ff=128, experts=8, top=2),
                         A(heads=8, dim=16, rot_dim=16, vdim=32, kv_rank=56, q_rank=40, mlp="dense", ff=256, scale=0.25),
                         G(heads=2, dim=128, vdim=128, tau=16.0, low_rank=16, mlp="dense", ff=256)], width=256, vocab=300, embed_scale=16.0)
    cfg["layers"][0]["mlp"] = O.ff_entry("moe", 128, 8, 2, 1.0)
    W = O.random_model(cfg, seed=21)
    toks = tokens(1320, 300, 4)
    rows = list(range(0, 1300, 97)) + [1297, 1298, 1299]
    want = O.forward(cfg, W, toks)
    for dtype in (F32, BF16):
        m = load(tmp_path, cfg, W, dtype, str(dtype)[-4:])
        seq = m.new_sequence()
        got = [m.step([(seq, toks[:1300])], [rows])]
        for p_ in range(1300, 1320):
            got.append(m.step([(seq, [toks[p_]])]))
        got = torch.cat(got)
        ref = want[rows + list(range(1300, 1320))]
        if dtype == F32:
            close(got, ref, 1e-4, "medium model, float32")
        else:
            close_rows(got, ref, 5e-2, "medium model, bfloat16", share=0.7)
        seq.free()


def test_greedy_generation_through_the_engines(tmp_path):
    from promptcache_b200.batch_engine import BatchEngine
    from promptcache_b200.generation_engine import GenerationEngine, GenerationParameters
    from promptcache_b200.model import Safilorn
    cfg = O.make_config(layer_sets()["mixed"][:3], width=48)
    W = O.random_model(cfg, seed=5)
    prompts = [tokens(n, cfg["vocab"], 40 + n) for n in (12, 3, 25)]
    n_new = 10

    def greedy(p):
        s = list(p)
        for _ in range(n_new):
            s.append(int(O.forward(cfg, W, s)[-1].argmax()))
        return s[len(p):]

    want = [greedy(p) for p in prompts]
    folder = str(tmp_path / "g")
    write_checkpoint(folder, cfg, W)
    lm = Safilorn(folder, device=DEV, dtype=F32)
    params = GenerationParameters(temperature=0.0, max_new_tokens=n_new, stop_token_ids=[], stop_str=[])
    assert BatchEngine(lm.hf_model, max_tokens=4096).generate(prompts, params) == want
    for p, w in zip(prompts, want):
        outs = list(GenerationEngine(lm).generate(p, list(range(len(p))), params, None, stream_interval=2))
        assert outs[-1].new_text == lm.decode(w)
    assert not lm.hf_model.pool.rows                         # the engines gave their slots back
    stop = want[2][3]
    stopped = BatchEngine(lm.hf_model, max_tokens=64).generate(prompts, GenerationParameters(temperature=0.0, max_new_tokens=n_new, stop_token_ids=[stop]))
    assert stopped[2] == want[2][:want[2].index(stop) + 1]


def test_trace_replay_end_to_end(tmp_path):
    cfg = O.make_config(layer_sets()["mixed"])
    W = O.random_model(cfg, seed=9)
    folder = str(tmp_path / "t")
    write_checkpoint(folder, cfg, W)
    a, b = tokens(20, cfg["vocab"], 1), tokens(7, cfg["vocab"], 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:15], "want": [0, 14]}, {"id": "b", "tokens": b[:6], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[15:16], "want": [0]}, {"id": "b", "tokens": b[6:], "want": [0]}], "end": ["b"]}] + \
            [{"step": 2 + i, "entries": [{"id": "a", "tokens": [a[16 + i]], "want": [0]}], "end": ["a"] if i == 3 else []} for i in range(4)]
    out = str(tmp_path / "out")
    for dtype, tol in (("float32", 5e-5), ("bfloat16", 0.2)):
        r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out, "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(6)]
        wa, wb = O.forward(cfg, W, a), O.forward(cfg, W, b)
        import numpy as np
        rd = lambda i: torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]).copy())
        cmp = close if dtype == "float32" else (lambda g_, w_, t_, s_: close_rows(g_, w_, t_, s_, share=1.0))
        cmp(rd(0), wa[[0, 14]], tol, "step 0")
        cmp(rd(1), torch.stack([wa[15], wb[6]]), tol, "step 1")
        for i in range(4):
            cmp(rd(2 + i), wa[16 + i:17 + i], tol, f"step {2 + i}")
