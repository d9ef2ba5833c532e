"""The Tevilix design on the GPU against the float64 oracle (tests/tevilix_oracle.py): each mechanism alone through the kernels'
bindings, then whole models through the step function, the batch engine, the generation engine and bin/trace_run."""
import json
import os
import subprocess

import pytest
import torch

from tests import tevilix_oracle as O

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
        json.dump(cfg, fh)
    wio.save_file({k: v.to(BF16) for k, v in W.items()}, os.path.join(folder, "model.safetensors"))


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
@pytest.mark.parametrize("width", [40, 37, 4096 + 8])
def test_residual_sum_and_two_layer_norms(nsq, width):
    g = torch.Generator().manual_seed(width)
    T = 7
    x = torch.randn(T, width, generator=g, dtype=F64) * 3 + 5.0          # a mean far from zero: the variance must come from the deviations
    ys = [torch.randn(T, width, generator=g, dtype=F64) for _ in range(3)]
    w1, w2 = torch.randn(width, generator=g, dtype=F64), torch.randn(width, generator=g, dtype=F64)
    mult = [0.7, 1.3, 1.0]
    for wdt, ydt, tol in ((F32, (F32, F32, F32), 3e-6), (BF16, (BF16, BF16, F32), 6e-3)):
        xd = dev(x)
        h1, h2 = torch.empty(T, width, device=DEV, dtype=wdt), torch.empty(T, width, device=DEV, dtype=wdt)
        yq = [y.to(d).to(F64) for y, d in zip(ys, ydt)]
        nsq.add_layer_norm(xd, [(dev(y, d), m) for y, d, m in zip(ys, ydt, mult)], 1e-5, dev(w1, wdt), h1, dev(w2, wdt), h2)
        xn = x + sum(m * y for m, y in zip(mult, yq))
        close(xd, xn, 2e-6, "stream after the sum of three branches")
        close(h1, O.layer_norm(xn, w1.to(wdt).to(F64), 1e-5), tol, "first norm")
        close(h2, O.layer_norm(xn, w2.to(wdt).to(F64), 1e-5), tol, "second norm")
    # one norm and no addend, on a subset of the rows; the stream stays as it is
    rows = torch.tensor([5, 0, 5, 2], dtype=torch.int32, device=DEV)
    xd, hr = dev(x), torch.empty(4, width, device=DEV)
    nsq.add_layer_norm(xd, [], 1e-5, dev(w1), hr, rows=rows)
    close(hr, O.layer_norm(x[[5, 0, 5, 2]], w1, 1e-5), 3e-6, "only the wanted rows")
    close(xd, x, 1e-7, "stream untouched")
    # only the sum (a model's last layer)
    xd = dev(x)
    nsq.add_layer_norm(xd, [(dev(ys[0]), -2.0)], 1e-5)
    close(xd, x - 2.0 * ys[0], 2e-6, "sum alone")
    # a constant row: zero variance, eps alone under the root
    xc = torch.full((2, width), 3.25, dtype=F64)
    hc = torch.empty(2, width, device=DEV)
    nsq.add_layer_norm(dev(xc), [], 1e-5, dev(w1), hc)
    assert float(hc.abs().max()) < 1e-3


@pytest.mark.parametrize("dtype,H,G,D,V,rot,inter", [(F32, 4, 2, 12, 10, 8, False), (F32, 3, 3, 7, 5, 6, False), (BF16, 8, 2, 32, 16, 16, False), (F32, 2, 1, 8, 8, 8, True),
                                                      (F32, 2, 2, 6, 4, 0, False)])
def test_head_norm_rotation_and_append(nsq, dtype, H, G, D, V, rot, inter):
    g = torch.Generator().manual_seed(H * 100 + D)
    lens, pos0, slots, cap = [5, 3], [0, 4100], [2, 0], 4224
    T = sum(lens)
    b = batch_of(nsq, slots, pos0, lens)
    pos = torch.tensor(list(range(5)) + list(range(4100, 4103)))
    nq, nk, nv = H * D, G * D, G * V
    proj = (torch.randn(T, 3 + nq + nk + nv + 2, generator=g, dtype=F64) * 2).to(dtype).to(F64)
    wq, wk = (torch.randn(D, generator=g, dtype=F64) + 1.5).to(dtype).to(F64), (torch.randn(D, generator=g, dtype=F64) + 1.5).to(dtype).to(F64)
    base, factor = 300.0, 4.0
    freqs = torch.tensor(O.rotary_frequencies(rot, base, factor), dtype=F64, device=DEV) if rot else None
    kp, vp = torch.full((3, G, cap, D), 7.0, device=DEV, dtype=dtype), torch.full((3, G, cap, V), 7.0, device=DEV, dtype=dtype)
    q = torch.empty(T, nq, device=DEV, dtype=dtype)
    nsq.rope_kv_prep(dev(proj, dtype), (3, 3 + nq, 3 + nq + nk), H, G, D, V, freqs, rot, inter, False, 1e-5, q, kp, vp, b, q_norm_w=dev(wq, dtype), k_norm_w=dev(wk, dtype))
    qn = O.unit_rms(proj[:, 3:3 + nq].view(T, H, D), 1e-5, wq)
    kn = O.unit_rms(proj[:, 3 + nq:3 + nq + nk].view(T, G, D), 1e-5, wk)
    if inter:   # neighbouring pairs: the oracle's half layout on a permuted head
        perm = list(range(0, rot, 2)) + list(range(1, rot, 2)) + list(range(rot, D))
        inv = [perm.index(i) for i in range(D)]
        qw = O.rotate_half(qn[..., perm], pos, rot, base, factor)[..., inv]
        kw = O.rotate_half(kn[..., perm], pos, rot, base, factor)[..., inv]
    else:
        qw, kw = O.rotate_half(qn, pos, rot, base, factor), O.rotate_half(kn, pos, rot, base, factor)
    tol = 3e-6 if dtype == F32 else 6e-3
    close(q.view(T, H, D), qw, tol, "queries: head norm, then the turn")
    for i in range(T):
        s = slots[0] if i < 5 else slots[1]
        close(kp[s, :, int(pos[i])], kw[i], tol, f"key row of token {i}")
        close(vp[s, :, int(pos[i])], proj[i, 3 + nq + nk:3 + nq + nk + nv].view(G, V), 1e-7, f"value row of token {i}")
    assert float(kp[1].min()) == 7.0 and float(kp[2, :, 5:].min()) == 7.0      # nothing else was written
    # without head norms the rows are only turned (what other designs get from the same entry point)
    q2 = torch.empty(T, nq, device=DEV, dtype=dtype)
    nsq.rope_kv_prep(dev(proj, dtype), (3, 3 + nq, 3 + nq + nk), H, G, D, V, freqs, rot, inter, False, 1e-5, q2, kp, vp, b)
    if not inter:
        close(q2.view(T, H, D), O.rotate_half(proj[:, 3:3 + nq].view(T, H, D), pos, rot, base, factor), tol, "no head norm")


def _attention_case(nsq, dtype, H, G, D, V, N, T, window, talk, impl=0, gate=True, seed=0):
    g = torch.Generator().manual_seed(seed + H * 1000 + N)
    cap = ((N + 127) // 128) * 128
    q = torch.randn(T, H, D, generator=g, dtype=F64).to(dtype).to(F64)
    k = torch.randn(N, G, D, generator=g, dtype=F64).to(dtype).to(F64)
    v = torch.randn(N, G, V, generator=g, dtype=F64).to(dtype).to(F64)
    og = torch.randn(T, H * V + 3, generator=g, dtype=F64).to(dtype).to(F64)
    kp, vp = torch.zeros(2, G, cap, D, device=DEV, dtype=dtype), torch.zeros(2, G, cap, V, device=DEV, dtype=dtype)
    kp[1, :, :N], vp[1, :, :N] = dev(k, dtype).transpose(0, 1), dev(v, dtype).transpose(0, 1)
    b = batch_of(nsq, [1], [N - T], [T])
    out = torch.empty(T, H * V, device=DEV, dtype=dtype)
    ws = nsq.attn_workspace(T, H, V, DEV) if T <= 16 else None
    ogd = dev(og, dtype)
    nsq.attention(dev(q.reshape(T, H * D), dtype), kp, vp, out, H, 0.3, None, None, False, b, impl=impl, max_keys=min(cap, window) if window else cap, workspace=ws,
                  window=window, talk=dev(talk), out_gate=ogd[:, 3:] if gate else None)
    want = O.mixed_score_attention(q, k, v, torch.arange(N - T, N), torch.arange(N), 0.3, talk, window).reshape(T, H * V)
    if gate:
        want = want * torch.sigmoid(og[:, 3:])
    return out, want


@pytest.mark.parametrize("dtype,H,G,D,V,N,T,window", [(F32, 4, 2, 12, 10, 70, 70, 9), (F32, 3, 1, 7, 5, 45, 3, 0), (F32, 5, 5, 8, 8, 700, 1, 0), (BF16, 8, 2, 32, 16, 300, 300, 45),
                                                       (BF16, 4, 4, 64, 64, 700, 2, 256), (F32, 2, 2, 16, 8, 33, 33, 1), (F32, 6, 3, 24, 20, 900, 4, 600),
                                                       (BF16, 8, 4, 96, 64, 520, 520, 52), (BF16, 16, 4, 64, 64, 400, 400, 128), (BF16, 4, 1, 128, 128, 333, 333, 0),
                                                       (BF16, 12, 3, 48, 80, 200, 200, 33), (BF16, 6, 2, 128, 64, 150, 150, 0), (BF16, 9, 9, 24, 8, 90, 90, 17),
                                                       (F32, 40, 8, 16, 160, 70, 5, 20)])
def test_attention_with_scores_mixed_across_heads(nsq, dtype, H, G, D, V, N, T, window):
    g = torch.Generator().manual_seed(H)
    talk = (torch.eye(H, dtype=F64) + 0.4 * torch.randn(H, H, generator=g, dtype=F64)).to(F32).to(F64)
    for impl in ((0, 1) if dtype == BF16 and T >= 16 else (0,)):    # every kernel that serves the shape; impl 1: the plain one
        out, want = _attention_case(nsq, dtype, H, G, D, V, N, T, window, talk, impl=impl)
        close(out, want, 2e-5 if dtype == F32 else 2e-2, f"mixed scores, window {window}, impl {impl}")
    out, want = _attention_case(nsq, dtype, H, G, D, V, N, T, window, talk, gate=False)
    close(out, want, 2e-5 if dtype == F32 else 2e-2, "without the output gate")


@pytest.mark.parametrize("dtype,H,G,D,V,window", [(BF16, 8, 2, 64, 64, 48), (BF16, 12, 4, 32, 48, 0), (F32, 4, 2, 16, 8, 20), (BF16, 16, 16, 32, 32, 200)])
def test_mixed_score_attention_in_portions_and_unequal_batches(nsq, dtype, H, G, D, V, window):
    """Entries that continue a sequence (their slots already hold rows) beside one that starts, of unequal lengths, in shuffled slots:
    every kernel that serves the shape must see each entry's own rows at its own positions, and nothing of the other slots."""
    g = torch.Generator().manual_seed(H * 7 + D)
    talk = (torch.eye(H, dtype=F64) + 0.3 * torch.randn(H, H, generator=g, dtype=F64)).to(F32).to(F64)
    pos0, lens, slots, cap = [0, 37, 300, 129], [50, 16, 90, 1], [3, 0, 2, 5], 512
    B, T = len(lens), sum(lens)
    ks = [torch.randn(p + n, G, D, generator=g, dtype=F64).to(dtype).to(F64) for p, n in zip(pos0, lens)]
    vs = [torch.randn(p + n, G, V, generator=g, dtype=F64).to(dtype).to(F64) for p, n in zip(pos0, lens)]
    q = torch.randn(T, H, D, generator=g, dtype=F64).to(dtype).to(F64)
    kp = torch.randn(6, G, cap, D, generator=g).to(DEV, dtype) * 3       # other slots and later rows hold numbers that must not show
    vp = torch.randn(6, G, cap, V, generator=g).to(DEV, dtype) * 3
    for s_, k_, v_ in zip(slots, ks, vs):
        kp[s_, :, :k_.shape[0]], vp[s_, :, :v_.shape[0]] = dev(k_, dtype).transpose(0, 1), dev(v_, dtype).transpose(0, 1)
    b = batch_of(nsq, slots, pos0, lens)
    want, o = [], 0
    for p, n, k_, v_ in zip(pos0, lens, ks, vs):
        want.append(O.mixed_score_attention(q[o:o + n], k_, v_, torch.arange(p, p + n), torch.arange(p + n), 0.25, talk, window).reshape(n, H * V))
        o += n
    want = torch.cat(want)
    for impl in ((0, 1) if dtype == BF16 else (0,)):
        out = torch.empty(T, H * V, device=DEV, dtype=dtype)
        nsq.attention(dev(q.reshape(T, H * D), dtype), kp, vp, out, H, 0.25, None, None, False, b, impl=impl, window=window, talk=dev(talk))
        close(out, want, 2e-5 if dtype == F32 else 2e-2, f"portions and unequal entries, impl {impl}")


@pytest.mark.parametrize("dtype,T", [(F32, 1), (F32, 80), (BF16, 1), (BF16, 80)])
def test_window_edge_far_key_and_mixing_decide(nsq, dtype, T):
    """One key carries a score that outweighs every other; whether the last query sees it depends on the window alone, and with the
    mixing matrix it is seen THROUGH ANOTHER HEAD: head 1 gets its large score from head 0's query."""
    H, G, D, V, N, window = 2, 1, 16, 8, 600, 50
    g = torch.Generator().manual_seed(3)
    talk = torch.tensor([[1.0, 0.0], [1.0, 0.05]], dtype=F64)      # head 1 mostly looks where head 0 does
    for special, seen in ((N - window, True), (N - window - 1, False), (N - 1, True), (0, False)):
        q = torch.randn(T, H, D, generator=g, dtype=F64) * 0.1
        k = torch.randn(N, G, D, generator=g, dtype=F64) * 0.1
        v = torch.randn(N, G, V, generator=g, dtype=F64)
        q[-1, 0], k[special, 0] = 0.0, 0.0
        q[-1, 0, 3], k[special, 0, 3] = 8.0, 8.0                     # the last query's head 0 and the special key: score 64 * scale
        v[special, 0] = 50.0
        cap = 640
        kp, vp = torch.zeros(1, G, cap, D, device=DEV, dtype=dtype), torch.zeros(1, G, cap, V, device=DEV, dtype=dtype)
        kp[0, :, :N], vp[0, :, :N] = dev(k, dtype).transpose(0, 1), dev(v, dtype).transpose(0, 1)
        b = batch_of(nsq, [0], [N - T], [T])
        out = torch.empty(T, H * V, device=DEV, dtype=dtype)
        ws = nsq.attn_workspace(T, H, V, DEV) if T <= 16 else None
        nsq.attention(dev(q.reshape(T, H * D), dtype), kp, vp, out, H, 0.5, None, None, False, b, max_keys=window, workspace=ws, window=window, talk=dev(talk))
        qq, kq, vq = (t.to(dtype).to(F64) for t in (q, k, v))
        want = O.mixed_score_attention(qq, kq, vq, torch.arange(N - T, N), torch.arange(N), 0.5, talk, window).reshape(T, H * V)
        close(out, want, 3e-5 if dtype == F32 else 2e-2, f"special key at {special}")
        last = out[-1].float().view(H, V)
        for h in range(H):   # both heads: head 1 only through the mixing
            assert (float(last[h].mean()) > 40.0) == seen, f"key {special} through head {h}: mean {float(last[h].mean()):.2f}, seen {seen}"


@pytest.mark.parametrize("dtype,R,lens,pos0", [(F32, 20, [13, 1, 40], [0, 7, 0]), (F32, 33, [1, 1], [5, 0]), (BF16, 64, [300, 2], [0, 9]), (F32, 7, [2, 3, 90], [0, 0, 4]),
                                               (BF16, 200, [700], [0])])
def test_gated_recurrence_scan(nsq, dtype, R, lens, pos0):
    g = torch.Generator().manual_seed(R)
    T, B = sum(lens), len(lens)
    slots = [2, 0, 3][:B]
    proj = (torch.randn(T, 5 + 3 * R, generator=g, dtype=F64) * 2).to(dtype).to(F64)
    pool = torch.full((4, R), 9.0, device=DEV)
    start = torch.randn(4, R, generator=g, dtype=F64)
    for s, p0 in zip(slots, pos0):
        if p0 > 0:
            pool[s] = start[s].to(DEV, F32)
    keep = pool.clone()
    out = torch.empty(T, R, device=DEV, dtype=dtype)
    nsq.gru_scan(dev(proj, dtype), (5 + R, 5, 5 + 2 * R), R, out, pool, batch_of(nsq, slots, pos0, lens))
    o = 0
    for s, p0, n in zip(slots, pos0, lens):
        rows = proj[o:o + n]
        z, u, gt = torch.sigmoid(rows[:, 5 + R:5 + 2 * R]), rows[:, 5:5 + R], rows[:, 5 + 2 * R:]
        S, last = O.gru_recurrence(z, O.gru_candidate(u), start[s].to(F32).to(F64) if p0 > 0 else None)   # a slot without tokens starts from zero, whatever it holds
        close(out[o:o + n], S * gt * torch.sigmoid(gt), 3e-6 if dtype == F32 else 6e-3, f"entry in slot {s}")
        close(pool[s], last, 3e-6, f"state left in slot {s}")
        o += n
    free = [s for s in range(4) if s not in slots]
    assert torch.equal(pool[free], keep[free])


def test_gated_recurrence_keeps_and_forgets(nsq):
    """A channel whose gate stays shut keeps the state it was given over hundreds of tokens; one whose gate is open holds the
    latest candidate; candidates switch branch at zero."""
    R, n = 4, 500
    proj = torch.zeros(n, 3 * R, dtype=F64)
    proj[:, 0] = -40.0                       # z = 0: keeps
    proj[:, 1] = 40.0                        # z = 1: follows
    proj[:, R + 0] = 3.0
    proj[:, R + 1] = torch.linspace(-2, 2, n, dtype=F64)
    proj[:, 2 * R:] = 30.0                   # silu(30) = 30
    pool = torch.zeros(1, R, device=DEV)
    pool[0, 0] = 1.25
    out = torch.empty(n, R, device=DEV)
    nsq.gru_scan(dev(proj), (0, R, 2 * R), R, out, pool, batch_of(nsq, [0], [3], [n]))
    assert float((out[:, 0] / 30.0 - 1.25).abs().max()) < 1e-5
    u = proj[:, R + 1]
    close(out[:, 1] / 30.0, torch.where(u >= 0, u + 0.5, torch.sigmoid(u)), 1e-5, "open gate follows the candidate")


@pytest.mark.parametrize("E,top,groups,keep,T,W", [(6, 2, 3, 2, 9, 40), (10, 3, 2, 1, 70, 64), (1, 1, 1, 1, 4, 24), (8, 8, 1, 1, 5, 36), (9, 3, 9, 4, 6, 32), (300, 4, 10, 3, 66, 48)])
def test_router_with_sigmoid_scores_and_group_pairs(nsq, E, top, groups, keep, T, W):
    g = torch.Generator().manual_seed(E * 10 + top)
    h = torch.randn(T, W, generator=g, dtype=F64)
    wr = torch.randn(E, W, generator=g, dtype=F64) * W ** -0.5 * 2
    corr = torch.randn(E, generator=g, dtype=F64) * 0.5 - 0.6        # negative choice scores exist: masked experts must not win over them
    idx, wgt, _ = nsq.moe_route(dev(h), dev(wr), dev(corr), None, top, groups, keep, renorm=True, score_fn=nsq.ROUTE_SIGMOID, group_best=2, wgt_scale=1.75, renorm_eps=1e-20)
    wi, ww = O.route(h, wr, corr, top, groups, keep, 1.75)
    # the same experts (order by choice score) with the same weights; rows where the oracle's own margin is tiny are skipped
    s = torch.sigmoid(h @ wr.T) + corr
    for t in range(T):
        got = dict(zip(idx[t].tolist(), wgt[t].tolist()))
        ref = dict(zip(wi[t].tolist(), ww[t].tolist()))
        if set(got) != set(ref):
            srt = s[t].sort(descending=True).values
            assert float((srt[:-1] - srt[1:]).min()) < 1e-5, f"token {t}: chose {sorted(got)}, oracle {sorted(ref)}"
            continue
        for e in ref:
            assert abs(got[e] - ref[e]) <= 3e-6 * 1.75, f"token {t}, expert {e}: weight {got[e]} against {ref[e]}"


def test_router_group_of_the_best_pair_wins(nsq):
    """Three groups of two; the group holding the two SECOND-best experts beats the group of the single best one, which only the
    sum of the two largest choice scores (not the maximum) decides; with the correction the choice changes and the weights do not."""
    W = 8
    h = torch.zeros(1, W, dtype=F64)
    h[0, 0] = 1.0
    z = torch.tensor([-1.0, -2.0, 1.0, 0.9, 1.5, -3.0], dtype=F64)
    wr = torch.zeros(6, W, dtype=F64)
    wr[:, 0] = z
    idx, wgt, _ = nsq.moe_route(dev(h), dev(wr), None, None, 2, 3, 1, renorm=True, score_fn=nsq.ROUTE_SIGMOID, group_best=2, wgt_scale=1.0, renorm_eps=1e-20)
    assert sorted(idx[0].tolist()) == [2, 3]
    idx1, _, _ = nsq.moe_route(dev(h), dev(wr), None, None, 1, 3, 1, renorm=True, score_fn=nsq.ROUTE_SIGMOID, group_best=1)
    assert idx1[0].tolist() == [4]                                   # scored by its maximum, the other group wins
    corr = torch.tensor([0.0, 0.0, -5.0, -5.0, -5.0, 0.4], dtype=F64)
    idx, wgt, _ = nsq.moe_route(dev(h), dev(wr), dev(corr), None, 2, 3, 1, renorm=True, score_fn=nsq.ROUTE_SIGMOID, group_best=2, wgt_scale=3.0, renorm_eps=1e-20)
    assert sorted(idx[0].tolist()) == [0, 1]                         # the only group whose pair is not pushed down
    s = torch.sigmoid(z)
    got = dict(zip(idx[0].tolist(), wgt[0].tolist()))
    assert abs(got[0] - float(3.0 * s[0] / (s[0] + s[1]))) < 1e-5     # weights from the plain scores


@pytest.mark.parametrize("T,ff,W,E,top", [(5, 16, 40, 4, 2), (3, 13, 30, 3, 1), (150, 64, 128, 6, 2)])
def test_experts_without_a_gate_branch(nsq, T, ff, W, E, top):
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, W, generator=g, dtype=F64)
    up, down = torch.randn(E, ff, W, generator=g, dtype=F64) * W ** -0.5, torch.randn(E, W, ff, generator=g, dtype=F64) * ff ** -0.5
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wgt = torch.rand(T, top, generator=g, dtype=F64)
    want = torch.zeros(T, W, dtype=F64)
    for t in range(T):
        for j in range(top):
            e = int(idx[t, j])
            want[t] += wgt[t, j] * (O.relu_squared(h[t] @ up[e].T) @ down[e].T)
    act = (nsq.ACT_RELU2, 0.0, 0.0)
    for dtype, modes, tol in ((F32, (False,), 3e-6), (BF16, (False, "library") if W % 8 == 0 and ff % 8 == 0 else (False,), 3e-2)):
        hq, uq, dq = (t.to(dtype).to(F64) for t in (h, up, down))
        ref = torch.zeros(T, W, dtype=F64)
        for t in range(T):
            for j in range(top):
                e = int(idx[t, j])
                ref[t] += wgt[t, j] * (O.relu_squared(hq[t] @ uq[e].T) @ dq[e].T)
        for mode in modes:
            ye, rows_e = nsq.moe_experts(dev(hq, dtype), idx.to(DEV), dev(uq, dtype), dev(dq, dtype), grouped=mode, act=act)
            y = torch.empty(T, W, device=DEV)
            nsq.moe_combine(y, ye, idx.to(DEV), dev(wgt), dev(hq, dtype), E, 1.0, y_row=rows_e, overwrite=True)
            close(y, ref, tol, f"experts, {dtype}, grouped={mode}")
    # the dense feed-forward's activation through the same entry point
    z = torch.randn(6, 24, generator=g, dtype=F64) * 2
    close(nsq.glu_mul(dev(z), 24, (nsq.ACT_GELU_ERF, 0.0, 0.0)), O.gelu_erf(z), 3e-6, "exact gelu")
    close(nsq.glu_mul(dev(z), 24, act), O.relu_squared(z), 3e-6, "squared relu")


# ---- whole models -------------------------------------------------------------------------------------------------
def layer_sets():
    P, M = O.parallel_layer, O.mlstm_layer
    return {
        "mixed": ([M(), P(mlp=O.moe()), M(mlp=O.moe(experts=4, top=1, groups=2, keep=1, scale=0.7)), P(window=5)], (1, 3, 2)),
        "odd": ([P(heads=3, kv_heads=3, dim=7, vdim=5, window=3, rot_dims=6, gru=9, mlp=O.moe(experts=3, top=3, ff=11, groups=0)),
                 M(heads=1, dim=5, vdim=9, mlp=None), P(heads=1, kv_heads=1, dim=4, vdim=6, window=1, rot_dims=0, gru=1, mlp=None)], None),
        "attention_only": ([P(window=64), P(heads=8, kv_heads=2, dim=16, vdim=16, window=11, rot_dims=16, base=10000.0, factor=1.0, mlp=O.moe(experts=8, top=2, groups=4, keep=2))],
                           (0, 2, 3)),
        "recurrent_only": ([M(), M(heads=4, dim=16, vdim=16, gate_cap=15.0, mlp=O.moe())], (1, 2, 2)),
        "loop_tail": ([P(window=6), M()], (1, 2, 4)),
    }


@pytest.mark.parametrize("name,width", [("mixed", 40), ("mixed", 24), ("odd", 30), ("odd", 37), ("attention_only", 64), ("recurrent_only", 48), ("loop_tail", 32)])
def test_model_whole_prompt_against_oracle(tmp_path, name, width):
    layers, loop = layer_sets()[name]
    cfg = O.make_config(layers, width=width, loop=loop)
    W = O.random_model(cfg, seed=len(name) + width)
    toks = tokens(75, cfg["vocab"], 5)
    lo = []
    want = O.forward(cfg, W, toks, lo)
    m = load(tmp_path, cfg, W, F32)
    assert len(m.state_specs()) == len(O.layer_runs(cfg))
    seq = m.new_sequence()
    m.layer_trace = []
    got = m.step([(seq, toks)], [list(range(len(toks)))])
    for i, (a, b) in enumerate(zip(m.layer_trace, lo)):
        close(a, b, 3e-5, f"{name}: stream after layer run {i}")
    close(got, want, 5e-5, f"{name}: logits")
    m.layer_trace = None
    seq.free()
    mb = load(tmp_path, cfg, W, BF16, "b")
    seq = mb.new_sequence()
    close_rows(mb.step([(seq, toks)], [list(range(len(toks)))]), want, 6e-2, f"{name}: bfloat16 logits", share=0.7)


@pytest.mark.parametrize("dtype,tol", [(F32, 5e-5), (BF16, 6e-2)])
def test_portions_decoding_batches_and_slot_reuse(tmp_path, dtype, tol):
    """One set of sequences run whole, in portions of several sizes down to two tokens, token by token (through the replayed
    graph), in unequal batches whose shorter members leave early, and through slots that were used before.  The windows (5 and
    7 tokens) pass over portion borders and over decoded tokens."""
    layers, loop = layer_sets()["mixed"]
    cfg = O.make_config(layers, loop=loop)
    W = O.random_model(cfg, seed=11)
    V = cfg["vocab"]
    seqs = [tokens(n, V, 20 + n) for n in (61, 9, 30, 1)]
    want = [O.forward(cfg, W, s) for s in seqs]
    m = load(tmp_path, cfg, W, dtype)
    cmp = close if dtype == F32 else (lambda g_, w_, t_, s_: close_rows(g_, w_, t_, s_, share=0.7))

    def run(toks, cuts):
        seq, out, p = m.new_sequence(), [], 0
        for n in cuts:
            out.append(m.step([(seq, toks[p:p + n])], [list(range(n))]))
            p += n
        seq.free()
        return torch.cat(out)

    for cuts in ([61], [2] * 30 + [1], [1] * 61, [17, 2, 3, 1, 1, 30, 7], [40] + [1] * 21, [20, 25, 16], [1, 60]):
        cmp(run(seqs[0], cuts), want[0], tol, f"portions {cuts[:6]}...")
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
    # the freed slots are handed out again, to other sequences and in another order: nothing of the old states shows
    lg = eng.step([("x", seqs[2], None), ("y", seqs[0], None), ("z", seqs[1], None)], ["x", "y", "z"])
    ref = torch.stack([want[2][-1], want[0][-1], want[1][-1]])
    if dtype == F32:
        close(lg, ref, tol, "reused slots")
    else:
        close_rows(lg, ref, 0.3, "reused slots", share=0.6)   # three rows at the sequences' ends, where bfloat16 noise of tiny heads has piled up


@pytest.mark.parametrize("dtype,tol", [(F32, 5e-5), (BF16, 6e-2)])
def test_tensor_core_sizes_in_portions_and_batches(tmp_path, dtype, tol):
    """Head sizes that the tensor-core kernels serve (multiples of 8), prompts cut into portions of 16 tokens and more that continue
    a sequence, and an unequal batch of prompts: the portions' windows (24 and 70 tokens) reach back into rows of earlier steps."""
    P, M = O.parallel_layer, O.mlstm_layer
    cfg = O.make_config([P(heads=8, kv_heads=2, dim=32, vdim=32, window=24, rot_dims=16, gru=40, mlp=O.moe(experts=4, top=2, ff=32, groups=2, keep=1)),
                         M(heads=2, dim=32, vdim=32), P(heads=4, kv_heads=4, dim=64, vdim=16, window=70, rot_dims=64, gru=24)], width=64, loop=(1, 3, 2))
    W = O.random_model(cfg, seed=17)
    seqs = [tokens(n, cfg["vocab"], 70 + n) for n in (150, 33, 80)]
    want = [O.forward(cfg, W, s) for s in seqs]
    m = load(tmp_path, cfg, W, dtype)
    cmp = close if dtype == F32 else (lambda g_, w_, t_, s_: close_rows(g_, w_, t_, s_, share=0.7))
    for cuts in ([150], [40, 17, 64, 29], [16, 16, 100, 2, 16], [149, 1]):
        seq, out, p_ = m.new_sequence(), [], 0
        for n in cuts:
            out.append(m.step([(seq, seqs[0][p_:p_ + n])], [list(range(n))]))
            p_ += n
        seq.free()
        cmp(torch.cat(out), want[0], tol, f"portions {cuts}")
    # three prompts of unequal length as one batch, cut in two steps at different places
    ss = [m.new_sequence() for _ in seqs]
    first = [70, 17, 40]
    a = m.step([(q_, s_[:n]) for q_, s_, n in zip(ss, seqs, first)], [list(range(n)) for n in first])
    b = m.step([(q_, s_[n:]) for q_, s_, n in zip(ss, seqs, first)], [list(range(len(s_) - n)) for s_, n in zip(seqs, first)])
    oa = ob = 0
    for i, (s_, n) in enumerate(zip(seqs, first)):
        got = torch.cat([a[oa:oa + n], b[ob:ob + len(s_) - n]])
        cmp(got, want[i], tol, f"request {i} of the batch")
        oa += n
        ob += len(s_) - n
    for q_ in ss:
        q_.free()


def test_long_decoding_window_passes_over_decoded_tokens(tmp_path):
    """300 tokens decoded one by one after a short prompt: the windows (44 and 130 tokens) leave the prompt behind, the pool grows
    while the sequence lives (captured graphs are rebuilt, the decoding attention splits the keys), a second sequence joins and leaves."""
    P, M = O.parallel_layer, O.mlstm_layer
    cfg = O.make_config([P(window=44), M(), P(heads=2, kv_heads=1, dim=16, vdim=8, window=130, rot_dims=8, mlp=None)], loop=(0, 2, 2))
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
    """Sizes at which the other code paths run: 64-wide heads on the tensor-core kernels over many key tiles with a window that
    ends inside a tile, the chunkwise matrix memory, decoding that splits the keys, hundreds of pairs per expert through the
    grouped product."""
    P, M = O.parallel_layer, O.mlstm_layer
    cfg = O.make_config([M(heads=4, dim=64, vdim=64, gate_cap=15.0, mlp=O.dense(256)),
                         P(heads=8, kv_heads=2, dim=64, vdim=64, window=200, rot_dims=32, base=10000.0, factor=8.0, gru=192, scale=0.2, mlp=O.moe(experts=8, top=2, ff=128, groups=4, keep=2)),
                         P(heads=4, kv_heads=4, dim=48, vdim=32, window=1000, rot_dims=48, gru=64, scale=0.25, mlp=O.dense(256))], width=256, vocab=300, embed_scale=4.0,
                        loop=(0, 2, 2))
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
    from promptcache_b200.model import Tevilix
    layers, loop = layer_sets()["mixed"]
    cfg = O.make_config(layers[:3], width=48, loop=(0, 2, 2))
    W = O.random_model(cfg, seed=5)
    prompts = [tokens(n, cfg["vocab"], 40 + n) for n in (12, 3, 25)]
    n_new = 10
    want = [O.greedy(cfg, W, p, n_new) for p in prompts]
    folder = str(tmp_path / "g")
    write_checkpoint(folder, cfg, W)
    lm = Tevilix(folder, device=DEV, dtype=F32)
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
    layers, loop = layer_sets()["mixed"]
    cfg = O.make_config(layers, loop=loop)
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
