"""Throughput of the slot-pool designs beside the closest existing model at equal sizes: `bench.py --design mutolix`
(against the Llama prompt-cache path), `bench.py --design raritar` (against Mutolix's attention layers with a dense
feed-forward of the same active size, which share the step function, the pool and the attention kernels) and
`bench.py --design safilorn` (against Mutolix with the same order and sizes of recurrent and attention layers) and
`bench.py --design tevilix` (against the same Mutolix model; its four layers run as a loop where Mutolix repeats them).  Random weights, synthetic token ids.  Prefill and decode tokens/s of both models through their own
step / forward, then every kernel of the new design alone against its roofline, next to the like kernel of the Llama path.

Timing: CUDA events on the launching stream, >= 3 warm-up iterations, a 256 MiB write between timed iterations (flushes the
126 MB L2), median of the timed iterations.
"""
from __future__ import annotations

import json
import statistics
from typing import Callable, Dict, List

import torch

SIZES = {
    # width, attention heads / kv heads / dim / vdim, recurrent heads / dim / vdim, ff, layers (pattern repeated), vocab
    "w1024": dict(width=1024, H=8, G=2, D=128, V=128, mH=4, mD=128, mV=256, ff=4096, repeat=1, vocab=8192),
    "w2048": dict(width=2048, H=16, G=4, D=128, V=128, mH=4, mD=256, mV=512, ff=8192, repeat=2, vocab=8192),
}


def mutolix_config(s: dict) -> dict:
    attn = {"type": "attention", "mixer": {"heads": s["H"], "kv_heads": s["G"], "dim": s["D"], "vdim": s["V"], "scale": s["D"] ** -0.5,
                                            "v_mix": True, "q_temp": {"coef": 0.3, "every": 256}}, "mlp": {"kind": "dense", "ff": s["ff"]}}
    rec = {"type": "mlstm", "mixer": {"heads": s["mH"], "dim": s["mD"], "vdim": s["mV"], "gate_cap": 12.0}, "mlp": {"kind": "dense", "ff": s["ff"]}}
    return {"architecture": "Mutolix", "vocab": s["vocab"], "width": s["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "layers": [rec, attn, attn, rec] * s["repeat"]}


def random_tensors(cfg: dict, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bfloat16 tensors with the checkpoint's names and shapes, made on the device."""
    g = torch.Generator(device=device).manual_seed(seed)
    W, t = cfg["width"], {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g, device=device) * std + mean).to(torch.bfloat16)

    lin = lambda o, i: rnd(o, i, std=i ** -0.5)
    t["embed"], t["final.norm"], t["head"] = rnd(cfg["vocab"], W), rnd(W, std=0.05, mean=1.0), lin(cfg["vocab"], W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            t[p + n] = rnd(W, std=0.05, mean=1.0)
        for n in ("ls1", "ls2"):
            t[p + n] = rnd(W, std=0.1, mean=0.5)
        for n in ("rg1", "rg2"):
            t[p + n], t[p + n + ".b"] = lin(W, W), rnd(W, std=0.3)
        if layer["type"] == "mlstm":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.g"] = lin(H * D, W), lin(H * D, W), lin(H * V, W), lin(H * V, W)
            t[p + "mix.o"], t[p + "mix.norm"] = lin(W, H * V), rnd(H * V, std=0.05, mean=1.0)
            t[p + "mix.i"], t[p + "mix.i.b"], t[p + "mix.f"], t[p + "mix.f.b"] = lin(H, W), rnd(H), lin(H, W), rnd(H, mean=3.0)
        else:
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                t[p + "mix." + n], t[p + "mix." + n + ".b"] = lin(rows, W), rnd(rows, std=0.1)
            t[p + "mix.q.norm"], t[p + "mix.k.norm"] = rnd(H * D, std=0.1, mean=1.0), rnd(G * D, std=0.1, mean=1.0)
            t[p + "mix.vmix"], t[p + "mix.o"] = rnd(1, std=0.05, mean=0.4).reshape(()), lin(W, H * V)
            t[p + "mix.r1"], t[p + "mix.r2"] = rnd(H, std=0.05, mean=0.5).abs(), rnd(H, std=0.1, mean=0.5).abs()
        ff = layer["mlp"]["ff"]
        t[p + "mlp.up"], t[p + "mlp.down"], t[p + "mlp.act"] = lin(ff, W), lin(W, ff), rnd(2, std=0.3)
    return t


class Timer:
    def __init__(self, device):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def __call__(self, fn: Callable[[], None], steps: int = 7, warmup: int = 3, setup: Callable[[], None] = None) -> float:
        """Median milliseconds of fn()."""
        ms = []
        for i in range(warmup + steps):
            if setup is not None:
                setup()
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= warmup:
                ms.append(a.elapsed_time(b))
        return statistics.median(ms)


def model_block(name: str, s: dict, dev, timer: Timer, prompt: int, batch: int, ctx: int) -> dict:
    from .model.llama2 import LlamaConfigLite, LlamaForCausalLM
    from .model.mutolix import MutolixConfig, MutolixForCausalLM
    cfg = mutolix_config(s)
    m = MutolixForCausalLM(MutolixConfig(cfg), random_tensors(cfg, dev), device=dev, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    toks = lambda n: torch.randint(0, s["vocab"], (n,), generator=g).tolist()
    out = {"layers": len(cfg["layers"]), "width": s["width"]}
    # ---- the new design: prefill of one prompt, of `batch` prompts, decode of 1 and of `batch` sequences at `ctx` tokens ----
    seqs: List = []

    def fresh(n):
        for q in seqs:
            q.free()
        seqs[:] = [m.new_sequence() for _ in range(n)]

    p1, pb = toks(prompt), [toks(prompt // 2) for _ in range(batch)]
    ms = timer(lambda: m.step([(seqs[0], p1)]), setup=lambda: fresh(1), steps=5)
    out["prefill_1x%d_tok_s" % prompt] = round(prompt / ms * 1e3)
    ms = timer(lambda: m.step([(q, t) for q, t in zip(seqs, pb)]), setup=lambda: fresh(batch), steps=5)
    out["prefill_%dx%d_tok_s" % (batch, prompt // 2)] = round(batch * (prompt // 2) / ms * 1e3)
    for nb in (1, batch):
        fresh(nb)
        m.step([(q, toks(ctx)) for q in seqs])
        for _ in range(3):  # the second one-token step of a batch size captures its graph
            m.step([(q, [1]) for q in seqs])
        ms = timer(lambda: m.step([(q, [1]) for q in seqs]), steps=16)
        out["decode_b%d_ctx%d_tok_s" % (nb, ctx)] = round(nb / ms * 1e3)
        out["decode_b%d_ms_per_step" % nb] = round(ms, 4)
    fresh(0)
    del m
    torch.cuda.empty_cache()
    # ---- the closest prompt-cache model at equal width, depth, heads and feed-forward (fp16, batch of one) ----
    lc = LlamaConfigLite(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"], num_hidden_layers=len(cfg["layers"]),
                         num_attention_heads=s["width"] // 128, num_key_value_heads=s["G"], max_position_embeddings=prompt + ctx + 64)
    ll = LlamaForCausalLM(lc, device=dev)
    ids = torch.tensor([p1], device=dev)
    pos = torch.arange(prompt, device=dev).unsqueeze(0)
    ms = timer(lambda: ll(input_ids=ids, position_ids=pos, use_cache=True, max_position=prompt - 1), steps=5)
    out["llama_prefill_1x%d_tok_s" % prompt] = round(prompt / ms * 1e3)
    cids, cpos = torch.tensor([toks(ctx)], device=dev), torch.arange(ctx, device=dev).unsqueeze(0)
    state = {"past": ll(input_ids=cids, position_ids=cpos, use_cache=True, max_position=ctx - 1).past_key_values, "n": ctx}
    one = torch.tensor([[1]], device=dev)

    def llama_decode():
        o = ll(input_ids=one, position_ids=torch.tensor([[state["n"]]], device=dev), past_key_values=state["past"], use_cache=True,
               max_position=state["n"])
        state["past"], state["n"] = o.past_key_values, state["n"] + 1

    for _ in range(3):
        llama_decode()
    ms = timer(llama_decode, steps=16)
    out["llama_decode_b1_ctx%d_tok_s" % ctx] = round(1 / ms * 1e3)
    out["llama_decode_b1_ms_per_step"] = round(ms, 4)
    del ll
    torch.cuda.empty_cache()
    return out


def kernel_block(s: dict, dev, timer: Timer, prompt: int, ctx: int, hbm_gbs: float, tflops: float) -> dict:
    """Every kernel of the new design alone at this size, achieved / peak, beside the like kernel of the Llama path."""
    from . import _native as nat, _native_seq as nsq
    bf, H, G, D, V, W = torch.bfloat16, s["H"], s["G"], s["D"], s["V"], s["width"]
    out = {}
    cap = ((max(prompt, ctx + 1) + 127) // 128) * 128
    kp, vp = torch.randn(1, G, cap, D, device=dev).to(bf), torch.randn(1, G, cap, V, device=dev).to(bf)
    r1, r2 = torch.full((H,), 0.5, device=dev), torch.full((H,), 0.5, device=dev)
    # attention over a prompt: FLOPs = 2 (D + V) per (query, visible key) pair and head
    b = nsq.Batch([0], [0], [prompt], dev)
    q, o = torch.randn(prompt, H * D, device=dev).to(bf), torch.empty(prompt, H * V, device=dev, dtype=bf)
    ms = timer(lambda: nsq.attention(q, kp, vp, o, H, D ** -0.5, r1, r2, True, b))
    fl = 2.0 * (D + V) * H * prompt * (prompt + 1) / 2
    out["attn_prompt"] = {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1), "of_measured_bf16_peak": round(fl / ms / 1e9 / tflops, 3)}
    ql = torch.randn(H, prompt, 128, device=dev).half()
    kl, vl = torch.randn(G, cap, 128, device=dev).half(), torch.randn(G, cap, 128, device=dev).half()
    ol = torch.empty(prompt, H * 128, device=dev, dtype=torch.half)
    ws = torch.zeros(nat.attn_workspace_bytes(H, prompt, 128), dtype=torch.uint8, device=dev)
    ms = timer(lambda: nat.attention(ql, kl, vl, ol, 0, prompt, H, G, 128, 128 ** -0.5, 0, workspace=ws))
    fl = 4.0 * 128 * H * prompt * (prompt + 1) / 2
    out["llama_attn_prompt"] = {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1), "of_measured_bf16_peak": round(fl / ms / 1e9 / tflops, 3)}
    # attention of one decoded token over ctx keys: bytes = K and V rows of every kv head
    b1 = nsq.Batch([0], [ctx], [1], dev)
    q1, o1 = torch.randn(1, H * D, device=dev).to(bf), torch.empty(1, H * V, device=dev, dtype=bf)
    wsd = nsq.attn_workspace(1, H, V, dev)
    ms = timer(lambda: nsq.attention(q1, kp, vp, o1, H, D ** -0.5, r1, r2, True, b1, max_keys=cap, workspace=wsd), steps=15)
    by = 2.0 * G * (ctx + 1) * (D + V)
    out["attn_decode"] = {"us": round(ms * 1e3, 2), "gb_s": round(by / ms / 1e6, 1), "of_measured_hbm_peak": round(by / ms / 1e6 / hbm_gbs, 4)}
    ql1, ol1 = torch.randn(H, 1, 128, device=dev).half(), torch.empty(1, H * 128, device=dev, dtype=torch.half)
    ws1 = torch.zeros(nat.attn_workspace_bytes(H, 1, 128), dtype=torch.uint8, device=dev)
    ms = timer(lambda: nat.attention(ql1, kl, vl, ol1, ctx, 1, H, G, 128, 128 ** -0.5, 0, workspace=ws1, decode=True), steps=15)
    by = 2.0 * G * (ctx + 1) * 256
    out["llama_attn_decode"] = {"us": round(ms * 1e3, 2), "gb_s": round(by / ms / 1e6, 1), "of_measured_hbm_peak": round(by / ms / 1e6 / hbm_gbs, 4)}
    # gated output norm + residual + next norm over a prompt: reads y, g (2 B), x (4 B), writes x (4 B), h (2 B)
    x, y, gl = torch.randn(prompt, W, device=dev), torch.randn(prompt, W, device=dev).to(bf), torch.randn(prompt, W, device=dev).to(bf)
    wn, h = torch.ones(W, device=dev, dtype=bf), torch.empty(prompt, W, device=dev, dtype=bf)
    ms = timer(lambda: nsq.gate_norm_add(x, y, gl, wn, wn, 1e-5, wn, h))
    by = prompt * W * 14.0
    out["gate_norm_add"] = {"us": round(ms * 1e3, 2), "gb_s": round(by / ms / 1e6, 1), "of_measured_hbm_peak": round(by / ms / 1e6 / hbm_gbs, 4)}
    xh, dh, hh, wh = (torch.randn(prompt, W, device=dev).half(), torch.randn(prompt, W, device=dev).half(),
                      torch.empty(prompt, W, device=dev, dtype=torch.half), torch.ones(W, device=dev, dtype=torch.half))
    ms = timer(lambda: nat.add_rmsnorm(xh, dh, wh, hh, 1e-5))
    by = prompt * W * 8.0
    out["llama_add_rmsnorm"] = {"us": round(ms * 1e3, 2), "gb_s": round(by / ms / 1e6, 1), "of_measured_hbm_peak": round(by / ms / 1e6 / hbm_gbs, 4)}
    # matrix-memory scan over a prompt (sequential in the tokens) and of one decoded token (state read + written once)
    mH, mD, mV = s["mH"], s["mD"], s["mV"]
    proj = (torch.randn(prompt, 2 * mH * mD + 2 * mH * mV, device=dev) * 0.3).to(bf)
    offs = (0, mH * mD, 2 * mH * mD, 2 * mH * mD + mH * mV)
    ig, fg = torch.randn(prompt, mH, device=dev), -torch.rand(prompt, mH, device=dev) * 0.1
    sp, npool, mp = torch.zeros(1, mH, mD, mV, device=dev), torch.zeros(1, mH, mD, device=dev), torch.zeros(1, mH, device=dev)
    nw, om = torch.ones(mH * mV, device=dev, dtype=bf), torch.empty(prompt, mH * mV, device=dev, dtype=bf)
    ms = timer(lambda: nsq.mlstm_scan(proj, offs, ig, fg, nw, om, sp, npool, mp, 1e-5, b), steps=5)
    out["mlstm_scan_prompt"] = {"ms": round(ms, 3), "us_per_token": round(ms * 1e3 / prompt, 3),
                                "gflops": round(4.0 * mH * mD * mV * prompt / ms / 1e6, 1)}
    ms = timer(lambda: nsq.mlstm_scan(proj[:1], offs, ig[:1], fg[:1], nw, om[:1], sp, npool, mp, 1e-5, b1), steps=15)
    by = 8.0 * mH * mD * mV
    out["mlstm_scan_decode"] = {"us": round(ms * 1e3, 2), "gb_s": round(by / ms / 1e6, 1), "of_measured_hbm_peak": round(by / ms / 1e6 / hbm_gbs, 4)}
    return out


# ---- Raritar ----------------------------------------------------------------------------------------------------------
RARITAR_SIZES = {
    # width, heads / kv heads / dim / vdim, window, experts / pass-through / top / groups / expert ff / shared ff, layers, vocab
    "w1024": dict(width=1024, H=8, G=2, D=128, V=128, window=512, keep=8, E=8, I=2, top=2, groups=(2, 1), ff=1024, sff=2048, layers=4, vocab=8192),
    "w2048": dict(width=2048, H=16, G=4, D=128, V=128, window=1024, keep=8, E=16, I=0, top=4, groups=(4, 2), ff=1024, sff=4096, layers=8, vocab=8192),
}


def raritar_config(s: dict) -> dict:
    def layer(kv_from=None):
        mixer = {"heads": s["H"], "kv_heads": s["G"], "dim": s["D"], "vdim": s["V"], "scale": s["D"] ** -0.5, "softcap": 30.0,
                 "mask": {"size": s["window"], "keep_first": s["keep"]},
                 "rot": {"base": 10000.0, "dims": s["D"] // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 4096}}}
        if kv_from is not None:
            mixer["kv_from"] = kv_from
        mlp = {"kind": "moe", "expert": {"ff": s["ff"]}, "shared": {"ff": s["sff"]},
               "router": {"experts": s["E"], "identity": s["I"], "top": s["top"], "groups": {"count": s["groups"][0], "keep": s["groups"][1]}}}
        return {"type": "attention", "mixer": mixer, "mlp": mlp}
    own = s["layers"] - s["layers"] // 4       # the last quarter of the layers reads the rows of the last layer that has its own
    return {"architecture": "Raritar", "vocab": s["vocab"], "width": s["width"], "residual_mult": 0.8, "norm": {"eps": 1e-5},
            "canon": {"taps": 3}, "embedding": {"bigram": {"buckets": 4093, "mul_prev": 29, "mul_cur": 5}},
            "layers": [layer() for _ in range(own)] + [layer(own - 1) for _ in range(s["layers"] - own)]}


def raritar_tensors(cfg: dict, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    W, t = cfg["width"], {}
    rnd = lambda *shape, std=1.0, mean=0.0: (torch.randn(*shape, generator=g, device=device) * std + mean).to(torch.bfloat16)
    lin = lambda o, i: rnd(o, i, std=i ** -0.5)
    t["embed"], t["final.norm"], t["head"] = rnd(cfg["vocab"], W), rnd(1, std=0.05, mean=1.0).reshape(()), lin(cfg["vocab"], W)
    t["bigram"] = rnd(cfg["embedding"]["bigram"]["buckets"] + 1, W, std=0.5)
    for i, layer in enumerate(cfg["layers"]):
        p, m, f = f"l{i}.", layer["mixer"], layer["mlp"]
        t[p + "norm1"], t[p + "norm2"] = rnd(1, std=0.05, mean=1.0).reshape(()), rnd(1, std=0.05, mean=1.0).reshape(())
        t[p + "canon1"] = rnd(W, cfg["canon"]["taps"], std=0.3)
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "mix.q"], t[p + "mix.o"] = lin(H * D, W), lin(W, H * V)
        if "kv_from" not in m:
            t[p + "mix.k"], t[p + "mix.v"] = lin(G * D, W), lin(G * V, W)
        r = f["router"]
        t[p + "mlp.router"], t[p + "mlp.correction"] = rnd(r["experts"] + r["identity"], W, std=3 * W ** -0.5), rnd(r["experts"] + r["identity"], std=0.05)
        for name, ff in [(f"e{e}.", f["expert"]["ff"]) for e in range(r["experts"])] + [("shared.", f["shared"]["ff"])]:
            t[p + "mlp." + name + "gate"], t[p + "mlp." + name + "up"], t[p + "mlp." + name + "down"] = lin(ff, W), lin(ff, W), lin(W, ff)
        t[p + "mlp.shared.sg"] = lin(1, W)
    return t


def _throughput(m, s: dict, timer: Timer, prompt: int, batch: int, ctx: int, out: dict, prefix: str = "") -> None:
    """Prefill of one prompt and of `batch` prompts, decode of 1 and of `batch` sequences at `ctx` tokens, through step()."""
    g = torch.Generator().manual_seed(1)
    toks = lambda n: torch.randint(0, s["vocab"], (n,), generator=g).tolist()
    seqs: List = []

    def fresh(n):
        for q in seqs:
            q.free()
        seqs[:] = [m.new_sequence() for _ in range(n)]

    p1, pb = toks(prompt), [toks(prompt // 2) for _ in range(batch)]
    ms = timer(lambda: m.step([(seqs[0], p1)]), setup=lambda: fresh(1), steps=5)
    out[prefix + "prefill_1x%d_tok_s" % prompt] = round(prompt / ms * 1e3)
    ms = timer(lambda: m.step([(q, t) for q, t in zip(seqs, pb)]), setup=lambda: fresh(batch), steps=5)
    out[prefix + "prefill_%dx%d_tok_s" % (batch, prompt // 2)] = round(batch * (prompt // 2) / ms * 1e3)
    for nb in (1, batch):
        fresh(nb)
        m.step([(q, toks(ctx)) for q in seqs])
        for _ in range(3):  # the second one-token step of a batch size captures its graph
            m.step([(q, [1]) for q in seqs])
        ms = timer(lambda: m.step([(q, [1]) for q in seqs]), steps=16)
        out[prefix + "decode_b%d_ms_per_step" % nb] = round(ms, 4)
    fresh(0)


def raritar_block(s: dict, dev, timer: Timer, prompt: int, batch: int, ctx: int) -> dict:
    from .model.mutolix import MutolixConfig, MutolixForCausalLM
    from .model.raritar import RaritarConfig, RaritarForCausalLM
    cfg = raritar_config(s)
    out = {"layers": len(cfg["layers"]), "width": s["width"], "active_ff": s["top"] * s["ff"] + s["sff"]}
    m = RaritarForCausalLM(RaritarConfig(cfg), raritar_tensors(cfg, dev), device=dev, dtype=torch.bfloat16)
    _throughput(m, s, timer, prompt, batch, ctx, out)
    del m
    torch.cuda.empty_cache()
    # the closest existing model: Mutolix's attention layers (full causal attention, every layer with rows of its own) with a
    # dense feed-forward as wide as this design's active experts
    attn = {"type": "attention", "mixer": {"heads": s["H"], "kv_heads": s["G"], "dim": s["D"], "vdim": s["V"], "scale": s["D"] ** -0.5},
            "mlp": {"kind": "dense", "ff": out["active_ff"]}}
    mc = {"architecture": "Mutolix", "vocab": s["vocab"], "width": s["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
          "layers": [attn] * s["layers"]}
    mm = MutolixForCausalLM(MutolixConfig(mc), random_tensors(mc, dev), device=dev, dtype=torch.bfloat16)
    _throughput(mm, s, timer, prompt, batch, ctx, out, prefix="mutolix_")
    del mm
    torch.cuda.empty_cache()
    return out


def raritar_kernels(s: dict, dev, timer: Timer, prompt: int, ctx: int, hbm_gbs: float, tflops: float) -> dict:
    """Every kernel of the design alone at this size, achieved / peak, beside the like kernel of the closest model."""
    from . import _native_seq as nsq
    bf, H, G, D, V, W = torch.bfloat16, s["H"], s["G"], s["D"], s["V"], s["width"]
    win, keep, E, top, ff = s["window"], s["keep"], s["E"], s["top"], s["ff"]
    out = {}
    gb = lambda by, ms: {"us": round(ms * 1e3, 2), "gb_s": round(by / ms / 1e6, 1), "of_measured_hbm_peak": round(by / ms / 1e6 / hbm_gbs, 4)}
    tf = lambda fl, ms: {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1), "of_measured_bf16_peak": round(fl / ms / 1e9 / tflops, 3)}
    cap = ((max(prompt, ctx + 1) + 127) // 128) * 128
    kp, vp = torch.randn(1, G, cap, D, device=dev).to(bf), torch.randn(1, G, cap, V, device=dev).to(bf)
    b = nsq.Batch([0], [0], [prompt], dev)
    q, o = torch.randn(prompt, H * D, device=dev).to(bf), torch.empty(prompt, H * V, device=dev, dtype=bf)
    # prompt attention: FLOPs = 2 (D + V) per (query, VISIBLE key) pair and head
    pairs = sum(min(i + 1, win) + max(0, min(keep, i + 1 - win)) for i in range(prompt))
    ms = timer(lambda: nsq.attention(q, kp, vp, o, H, D ** -0.5, None, None, False, b, softcap=30.0, window=win, keep_first=keep))
    out["attn_prompt_window"] = tf(2.0 * (D + V) * H * pairs, ms)
    ms = timer(lambda: nsq.attention(q, kp, vp, o, H, D ** -0.5, None, None, False, b, softcap=30.0))
    out["attn_prompt_capped_full"] = tf(2.0 * (D + V) * H * prompt * (prompt + 1) / 2, ms)
    ms = timer(lambda: nsq.attention(q, kp, vp, o, H, D ** -0.5, None, None, False, b))
    out["like_attn_prompt_full"] = tf(2.0 * (D + V) * H * prompt * (prompt + 1) / 2, ms)
    # one decoded token: bytes = visible K and V rows of every kv head
    b1 = nsq.Batch([0], [ctx], [1], dev)
    q1, o1 = torch.randn(1, H * D, device=dev).to(bf), torch.empty(1, H * V, device=dev, dtype=bf)
    wsd = nsq.attn_workspace(1, H, V, dev)
    ms = timer(lambda: nsq.attention(q1, kp, vp, o1, H, D ** -0.5, None, None, False, b1, max_keys=win + keep, workspace=wsd, softcap=30.0, window=win,
                                     keep_first=keep), steps=15)
    out["attn_decode_window"] = gb(2.0 * G * (win + keep) * (D + V), ms)
    ms = timer(lambda: nsq.attention(q1, kp, vp, o1, H, D ** -0.5, None, None, False, b1, max_keys=cap, workspace=wsd), steps=15)
    out["like_attn_decode_full"] = gb(2.0 * G * (ctx + 1) * (D + V), ms)
    # norm + convolution: reads x (4 B, neighbours from L2) and writes h (2 B); like: gated norm + residual + next norm
    x, h = torch.randn(prompt, W, device=dev), torch.empty(prompt, W, device=dev, dtype=bf)
    g1, cw, tail = torch.ones(1, device=dev, dtype=bf), (torch.randn(3, W, device=dev) * 0.3).to(bf), torch.zeros(1, 2, 2, W, device=dev)
    ms = timer(lambda: nsq.norm_conv(x, g1, 1e-5, h, conv_w=cw, tail=tail, batch=b))
    out["norm_conv"] = gb(prompt * W * 6.0, ms)
    y = torch.randn(prompt, W, device=dev).to(bf)
    ms = timer(lambda: nsq.norm_conv(x, g1, 1e-5, h, y=y, y_mult=0.8))
    out["add_norm"] = gb(prompt * W * 12.0, ms)
    wn = torch.ones(W, device=dev, dtype=bf)
    ms = timer(lambda: nsq.gate_norm_add(x, y, None, wn, None, 1e-5, wn, h))
    out["like_gate_norm_add"] = gb(prompt * W * 12.0, ms)
    # rotation + value norm + append: reads the projection row, writes q, k, v (2 B each); like: Mutolix's q/k norm + append
    nq, nk = H * D, G * (D + V)
    proj = torch.randn(prompt, nq + nk, device=dev).to(bf)
    fr = torch.tensor([10000.0 ** (-2.0 * i / (D // 2)) for i in range(D // 4)], dtype=torch.float64, device=dev)
    ms = timer(lambda: nsq.rope_kv_prep(proj, (0, nq, nq + G * D), H, G, D, V, fr, D // 2, True, True, 1e-5, q, kp, vp, b))
    out["rope_kv_prep"] = gb(prompt * (nq + nk) * 4.0, ms)
    qn, kn = torch.ones(nq, device=dev, dtype=bf), torch.ones(G * D, device=dev, dtype=bf)
    ms = timer(lambda: nsq.qk_prep(proj, (0, nq, nq + G * D), qn, kn, 1e-5, H, G, D, V, 0.0, 0, q, kp, vp, None, None, b))
    out["like_qk_prep"] = gb(prompt * (nq + nk) * 4.0, ms)
    # router
    hb = torch.randn(prompt, W, device=dev).to(bf)
    wr, corr, wsg = (torch.randn(E + s["I"], W, device=dev) * 3 * W ** -0.5).to(bf), torch.zeros(E + s["I"], device=dev), torch.randn(W, device=dev).to(bf)
    ms = timer(lambda: nsq.moe_route(hb, wr, corr, wsg, top, s["groups"][0], s["groups"][1]))
    out["moe_route"] = gb(prompt * W * 2.0, ms)
    idx, _, _ = nsq.moe_route(hb, wr, corr, wsg, top, s["groups"][0], s["groups"][1])
    real = int((idx < E).sum())
    # the experts of a prompt: FLOPs = 6 ff W per real pair; like: the dense feed-forward's library products of the same FLOPs
    wgu, wdn = (torch.randn(E, 2 * ff, W, device=dev) * W ** -0.5).to(bf), (torch.randn(E, W, ff, device=dev) * ff ** -0.5).to(bf)
    ms = timer(lambda: nsq.moe_experts(hb, idx, wgu, wdn, grouped="library"))
    out["moe_experts_prompt"] = dict(tf(6.0 * ff * W * real, ms), pairs=real, what="plan + gather + library grouped products + silu_mul")
    ms = timer(lambda: nsq.moe_experts(hb, idx, wgu, wdn, grouped="own"))
    out["moe_experts_prompt_own_kernel"] = tf(6.0 * ff * W * real, ms)
    rows = max(real, 1)
    xa, wa, wb2 = torch.randn(rows, W, device=dev).to(bf), wgu[0], wdn[0]
    ms = timer(lambda: torch.nn.functional.linear(torch.nn.functional.linear(xa, wa)[:, :ff], wb2))
    out["like_dense_ff_products"] = tf(6.0 * ff * W * rows, ms)
    # the experts of one decoded token: bytes = the chosen experts' three matrices; like: the few-row linear kernel on as many bytes
    i1 = idx[:1].contiguous()
    real1 = int((i1 < E).sum())
    ms = timer(lambda: nsq.moe_experts(hb[:1], i1, wgu, wdn, grouped=False), steps=15)
    out["moe_experts_decode"] = gb(real1 * 3.0 * ff * W * 2, ms)
    wl = (torch.randn(real1 * 3 * ff, W, device=dev) * W ** -0.5).to(bf)
    ms = timer(lambda: nsq.linear(hb[:1], wl, kernel=True), steps=15)
    out["like_linear_rows"] = gb(real1 * 3.0 * ff * W * 2, ms)
    ye, wg2, sg, ys = torch.randn(prompt * top, W, device=dev), torch.rand(prompt, top, device=dev), torch.rand(prompt, device=dev), torch.randn(prompt, W, device=dev).to(bf)
    ms = timer(lambda: nsq.moe_combine(x, ye, idx, wg2, hb, E, 0.8, ys=ys, shared_gate=sg))
    out["moe_combine"] = gb(prompt * W * (4.0 * top + 2 + 8), ms)
    return out


# ---- Safilorn ---------------------------------------------------------------------------------------------------------
SAFILORN_SIZES = {
    # the recurrent and attention sizes of SIZES; latent attention: per head dim plain + rot rotated key numbers, kv / q latent ranks;
    # the feed-forward alternates dense (ff) and experts (E of eff, `top` active: the same active size)
    "w1024": dict(SIZES["w1024"], D=96, R=32, C=256, Q=512, rank=16, tau=16.0, E=8, top=2, eff=2048),
    "w2048": dict(SIZES["w2048"], D=96, R=32, C=512, Q=768, rank=32, tau=16.0, E=16, top=4, eff=2048),
}


def safilorn_config(s: dict) -> dict:
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": s["eff"], "limit": 7.0}, "router": {"experts": s["E"], "top": s["top"]}}
    att = lambda mlp: {"type": "latent_attention", "mlp": mlp,
                       "mixer": {"heads": s["H"], "dim": s["D"], "rot_dim": s["R"], "vdim": s["V"], "kv_rank": s["C"], "q_rank": s["Q"], "scale": (s["D"] + s["R"]) ** -0.5,
                                 "rot": {"base": 10000.0, "dims": s["R"], "scaling": {"factor": 8.0, "original": 4096, "fast": 24.0, "slow": 1.5}}}}
    rec = lambda mlp: {"type": "gla", "mixer": {"heads": s["mH"], "dim": s["mD"], "vdim": s["mV"], "tau": s["tau"]}, "mlp": mlp}
    return {"architecture": "Safilorn", "vocab": s["vocab"], "width": s["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "layers": [rec(dense), att(moe), att(dense), rec(moe)] * s["repeat"]}


def safilorn_tensors(cfg: dict, s: dict, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    W, t = cfg["width"], {}
    rnd = lambda *shape, std=1.0, mean=0.0: (torch.randn(*shape, generator=g, device=device) * std + mean).to(torch.bfloat16)
    lin = lambda o, i: rnd(o, i, std=i ** -0.5)
    t["embed"], t["final.norm"], t["head"] = rnd(cfg["vocab"], W), rnd(W, std=0.05), lin(cfg["vocab"], W)
    for i, layer in enumerate(cfg["layers"]):
        p, m, f = f"l{i}.", layer["mixer"], layer["mlp"]
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            t[p + n] = rnd(W, std=0.05)
        t[p + "dwa"] = torch.cat([rnd(i + 1, std=0.1 / (i + 1)), rnd(1, std=0.02, mean=1.0)])
        if layer["type"] == "latent_attention":
            H, D, R, V, C, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"], t[p + "mix.uq"] = lin(Q, W), rnd(Q, std=0.05, mean=1.0), lin(H * (D + R), Q)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = lin(C + R, W), rnd(C, std=0.05, mean=1.0)
            t[p + "mix.uk"], t[p + "mix.uv"], t[p + "mix.sink"] = lin(H * D, C), lin(H * V, C), rnd(H, std=1.0)
            t[p + "mix.g"], t[p + "mix.o"] = lin(H, W), lin(W, H * V)
        else:
            H, D, V = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.g"] = lin(H * D, W), lin(H * D, W), lin(H * V, W), lin(H * V, W)
            t[p + "mix.o"], t[p + "mix.norm"] = lin(W, H * V), rnd(V, std=0.05, mean=1.0)
            t[p + "mix.a1"], t[p + "mix.a2"], t[p + "mix.a2.b"] = lin(s["rank"], W), lin(H * D, s["rank"]), rnd(H * D, std=1.0, mean=3.0)
        if f["kind"] == "dense":
            ff = f["ff"]
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = lin(ff, W), lin(ff, W), lin(W, ff)
            t[p + "mlp.gate.b"], t[p + "mlp.up.b"], t[p + "mlp.down.b"] = rnd(ff, std=0.1), rnd(ff, std=0.1), rnd(W, std=0.1)
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            t[p + "mlp.router"], t[p + "mlp.router.b"] = rnd(E, W, std=3 * W ** -0.5), rnd(E, std=0.1)
            for e in range(E):
                t[f"{p}mlp.e{e}.gate"], t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = lin(ff, W), lin(ff, W), lin(W, ff)
    return t


def safilorn_block(s: dict, dev, timer: Timer, prompt: int, batch: int, ctx: int) -> dict:
    from .model.mutolix import MutolixConfig, MutolixForCausalLM
    from .model.safilorn import SafilornConfig, SafilornForCausalLM
    cfg = safilorn_config(s)
    out = {"layers": len(cfg["layers"]), "width": s["width"], "active_ff": s["ff"]}
    m = SafilornForCausalLM(SafilornConfig(cfg), safilorn_tensors(cfg, s, dev), device=dev, dtype=torch.bfloat16)
    _throughput(m, s, timer, prompt, batch, ctx, out)
    del m
    torch.cuda.empty_cache()
    mc = mutolix_config(s)   # the closest existing model: recurrent and attention layers in the same order, at the same sizes
    mm = MutolixForCausalLM(MutolixConfig(mc), random_tensors(mc, dev), device=dev, dtype=torch.bfloat16)
    _throughput(mm, s, timer, prompt, batch, ctx, out, prefix="mutolix_")
    del mm
    torch.cuda.empty_cache()
    return out


def safilorn_kernels(s: dict, dev, timer: Timer, prompt: int, ctx: int, hbm_gbs: float, tflops: float) -> dict:
    """Every kernel of the design alone at this size, achieved / peak, beside the like kernel of the closest model."""
    from . import _native_seq as nsq
    bf, H, G, D, R, V, C, Q, W = torch.bfloat16, s["H"], s["G"], s["D"], s["R"], s["V"], s["C"], s["Q"], s["width"]
    out = {}
    gb = lambda by, ms: {"us": round(ms * 1e3, 2), "gb_s": round(by / ms / 1e6, 1), "of_measured_hbm_peak": round(by / ms / 1e6 / hbm_gbs, 4)}
    tf = lambda fl, ms: {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1), "of_measured_bf16_peak": round(fl / ms / 1e9 / tflops, 3)}
    cap = ((max(prompt, ctx + 1) + 127) // 128) * 128
    b, b1 = nsq.Batch([0], [0], [prompt], dev), nsq.Batch([0], [ctx], [1], dev)
    sink = torch.randn(H, device=dev)
    r1, r2 = torch.full((H,), 0.5, device=dev), torch.full((H,), 0.5, device=dev)
    # prompt attention over expanded keys (every head its own rows): FLOPs = 2 (D + R + V) per (query, visible key) pair and head
    kd, vd = torch.randn(1, H, cap, D + R, device=dev).to(bf), torch.randn(1, H, cap, V, device=dev).to(bf)
    q, o = torch.randn(prompt, H * (D + R), device=dev).to(bf), torch.empty(prompt, H * V, device=dev, dtype=bf)
    ids = torch.zeros(1, dtype=torch.int32, device=dev)
    ms = timer(lambda: nsq.attention(q, kd, vd, o, H, (D + R) ** -0.5, None, None, True, b, sink_logit=sink, pool_slot=ids))
    out["attn_prompt_expanded"] = tf(2.0 * (D + R + V) * H * prompt * (prompt + 1) / 2, ms)
    kp, vp = torch.randn(1, G, cap, D + R, device=dev).to(bf), torch.randn(1, G, cap, V, device=dev).to(bf)
    ms = timer(lambda: nsq.attention(q, kp, vp, o, H, (D + R) ** -0.5, r1, r2, True, b))
    out["like_attn_prompt"] = tf(2.0 * (D + R + V) * H * prompt * (prompt + 1) / 2, ms)
    # what the expanded form adds per layer: latents out of the pool, one product, per-head rows written (bytes: rows read and written)
    pool = torch.randn(1, 1, cap, C + R, device=dev).to(bf)
    wukv = (torch.randn(H * (D + V), C, device=dev) * C ** -0.5).to(bf)

    def expand():
        kv = nsq.linear(nsq.latent_gather(pool, C, b), wukv)
        nsq.latent_expand(kv, pool, C, R, H, D, V, kd, vd, b)
    ms = timer(expand)
    out["latent_expand_chain"] = dict(tf(2.0 * prompt * C * H * (D + V), ms), **{"gb_s": round(prompt * (2.0 * C * 2 + 4.0 * H * (D + V) + 2.0 * H * (D + R + V)) / ms / 1e6, 1)})
    # decoding in the latent space: every head reads the same rows, bytes = the sequence's cached rows once
    q1, o1 = torch.randn(1, H * (C + R), device=dev).to(bf), torch.empty(1, H * C, device=dev, dtype=bf)
    wsd = nsq.attn_workspace(1, H, C, dev)
    ms = timer(lambda: nsq.attention(q1, pool, pool, o1, H, 0.1, None, None, True, b1, max_keys=cap, workspace=wsd, sink_logit=sink, v_row_stride=C + R), steps=15)
    out["attn_decode_latent"] = dict(gb(2.0 * (ctx + 1) * (C + R), ms), flops_per_byte=round(2.0 * H * (2 * C + R) / (2.0 * (C + R)), 1))
    # the same at four times the context, where the kernels rather than the launches decide: the tensor-core kernel that stages a
    # row once for 16 heads, and the plain kernel (one block per head and split) on the same rows
    ctx4 = 4 * ctx
    cap4 = ((ctx4 + 1 + 127) // 128) * 128
    pool4, b4 = torch.randn(1, 1, cap4, C + R, device=dev).to(bf), nsq.Batch([0], [ctx4], [1], dev)
    for impl, name in ((0, "attn_decode_latent_ctx%d" % ctx4), (2, "attn_decode_latent_plain_kernel_ctx%d" % ctx4)):
        ms = timer(lambda: nsq.attention(q1, pool4, pool4, o1, H, 0.1, None, None, True, b4, impl=impl, max_keys=cap4, workspace=wsd, sink_logit=sink,
                                         v_row_stride=C + R), steps=15)
        out[name] = gb(2.0 * (ctx4 + 1) * (C + R), ms)
    kp4, vp4 = torch.randn(1, G, cap4, D + R, device=dev).to(bf), torch.randn(1, G, cap4, V, device=dev).to(bf)
    qm, om = torch.randn(1, H * (D + R), device=dev).to(bf), torch.empty(1, H * V, device=dev, dtype=bf)
    wsm = nsq.attn_workspace(1, H, V, dev)
    ms = timer(lambda: nsq.attention(qm, kp4, vp4, om, H, 0.1, r1, r2, True, b4, max_keys=cap4, workspace=wsm), steps=15)
    out["like_attn_decode_ctx%d" % ctx4] = gb(2.0 * G * (ctx4 + 1) * (D + R + V), ms)
    del pool4, kp4, vp4
    wsm = nsq.attn_workspace(1, H, V, dev)
    ms = timer(lambda: nsq.attention(qm, kp, vp, om, H, 0.1, r1, r2, True, b1, max_keys=cap, workspace=wsm), steps=15)
    out["like_attn_decode"] = gb(2.0 * G * (ctx + 1) * (D + R + V), ms)
    # norms, rotation and append: reads the projection row, writes the query latent and one cached row
    proj = torch.randn(prompt, Q + C + R + H, device=dev).to(bf)
    fr = torch.tensor([10000.0 ** (-2.0 * i / R) for i in range(R // 2)], dtype=torch.float64, device=dev)
    cq, wq_, wc_ = torch.empty(prompt, Q, device=dev, dtype=bf), torch.ones(Q, device=dev, dtype=bf), torch.ones(C, device=dev, dtype=bf)
    ms = timer(lambda: nsq.latent_prep(proj, 0, Q, Q, C, R, wq_, wc_, 1e-5, fr, 1.2, cq, pool, b))
    out["latent_prep"] = gb(prompt * (Q + C + R) * 4.0, ms)
    ms = timer(lambda: nsq.latent_q(q, H, D, R, fr, 1.2, b))
    out["latent_q_rotation"] = gb(prompt * H * R * 4.0, ms)
    nq, nk = H * (D + R), G * (D + R + V)
    pj = torch.randn(prompt, nq + nk, device=dev).to(bf)
    qn, kn = torch.ones(nq, device=dev, dtype=bf), torch.ones(G * (D + R), device=dev, dtype=bf)
    ms = timer(lambda: nsq.qk_prep(pj, (0, nq, nq + G * (D + R)), qn, kn, 1e-5, H, G, D + R, V, 0.0, 0, q, kp, vp, None, None, b))
    out["like_qk_prep"] = gb(prompt * (nq + nk) * 4.0, ms)
    # the depth average with the next norm: reads n results (4 B), writes the stream (4 B) and h (2 B); like: gated norm + residual + next norm
    n_terms = 5
    xs, h = torch.randn(n_terms + 1, prompt, W, device=dev), torch.empty(prompt, W, device=dev, dtype=bf)
    coef, wn = torch.rand(n_terms, device=dev), torch.zeros(W, device=dev, dtype=bf)
    ms = timer(lambda: nsq.depth_mix(xs, n_terms, coef, 1e-5, x_out=xs[n_terms], next_w=wn, h_out=h, w_offset=1.0))
    out["depth_mix_5_terms"] = gb(prompt * W * (4.0 * n_terms + 6.0), ms)
    x, y = xs[0], torch.randn(prompt, W, device=dev).to(bf)
    ms = timer(lambda: nsq.gate_norm_add(x, y, None, wn, None, 1e-5, wn, h, w_offset=1.0))
    out["norm_add_norm"] = gb(prompt * W * 12.0, ms)
    ms = timer(lambda: nsq.gate_norm_add(x, y, y, wn, wn, 1e-5, wn, h))
    out["like_gate_norm_add"] = gb(prompt * W * 14.0, ms)
    # the recurrence over a prompt (sequential in the tokens) and of one decoded token (state read and written once)
    mH, mD, mV, rk = s["mH"], s["mD"], s["mV"], s["rank"]
    pr = (torch.randn(prompt, 2 * mH * mD + 2 * mH * mV + rk, device=dev) * 0.3).to(bf)
    offs = (0, mH * mD, 2 * mH * mD, 2 * mH * mD + mH * mV)
    a2, a2b = (torch.randn(mH * mD, rk, device=dev) * rk ** -0.5).to(bf), torch.full((mH * mD,), 3.0, device=dev)
    ms = timer(lambda: nsq.gla_decay(pr[:, offs[3] + mH * mV:], a2, a2b, s["tau"]))
    out["gla_decay"] = gb(prompt * mH * mD * 4.0, ms)
    ld = nsq.gla_decay(pr[:, offs[3] + mH * mV:], a2, a2b, s["tau"])
    sp, nw, og = torch.zeros(1, mH, mD, mV, device=dev), torch.ones(mV, device=dev, dtype=bf), torch.empty(prompt, mH * mV, device=dev, dtype=bf)
    ms = timer(lambda: nsq.gla_scan(pr, offs, ld, nw, og, sp, 1e-5, b), steps=5)
    out["gla_scan_prompt"] = {"ms": round(ms, 3), "us_per_token": round(ms * 1e3 / prompt, 3), "gflops": round(4.0 * mH * mD * mV * prompt / ms / 1e6, 1)}
    ms = timer(lambda: nsq.gla_scan(pr[:1], offs, ld[:1], nw, og[:1], sp, 1e-5, b1), steps=15)
    out["gla_scan_decode"] = gb(8.0 * mH * mD * mV, ms)
    ig, fg = torch.randn(prompt, mH, device=dev), -torch.rand(prompt, mH, device=dev) * 0.1
    npool, mp, nwm = torch.zeros(1, mH, mD, device=dev), torch.zeros(1, mH, device=dev), torch.ones(mH * mV, device=dev, dtype=bf)
    ms = timer(lambda: nsq.mlstm_scan(pr, offs, ig, fg, nwm, og, sp, npool, mp, 1e-5, b), steps=5)
    out["like_mlstm_scan_prompt"] = {"ms": round(ms, 3), "us_per_token": round(ms * 1e3 / prompt, 3), "gflops": round(4.0 * mH * mD * mV * prompt / ms / 1e6, 1)}
    ms = timer(lambda: nsq.mlstm_scan(pr, offs, ig, fg, nwm, og, sp, npool, mp, 1e-5, b, impl=2), steps=5)
    out["like_mlstm_scan_prompt_token_by_token"] = {"ms": round(ms, 3), "us_per_token": round(ms * 1e3 / prompt, 3)}
    ms = timer(lambda: nsq.mlstm_scan(pr[:1], offs, ig[:1], fg[:1], nwm, og[:1], sp, npool, mp, 1e-5, b1), steps=15)
    out["like_mlstm_scan_decode"] = gb(8.0 * mH * mD * mV, ms)
    # router and experts
    E, top, ff = s["E"], s["top"], s["eff"]
    hb = torch.randn(prompt, W, device=dev).to(bf)
    wr, br = (torch.randn(E, W, device=dev) * 3 * W ** -0.5).to(bf), torch.zeros(E, device=dev)
    ms = timer(lambda: nsq.moe_route(hb, wr, None, None, top, bias=br, renorm=True))
    out["moe_route"] = gb(prompt * W * 2.0, ms)
    idx, wgt, _ = nsq.moe_route(hb, wr, None, None, top, bias=br, renorm=True)
    act = (nsq.GLU_CLAMPED_SWISH, 1.702, 7.0)
    wgu, wdn = (torch.randn(E, 2 * ff, W, device=dev) * W ** -0.5).to(bf), (torch.randn(E, W, ff, device=dev) * ff ** -0.5).to(bf)
    pairs = prompt * top
    ms = timer(lambda: nsq.moe_experts(hb, idx, wgu, wdn, grouped="library", act=act))
    out["moe_experts_prompt"] = dict(tf(6.0 * ff * W * pairs, ms), what="plan + gather + library grouped products + clamped swish")
    xa = torch.randn(pairs, W, device=dev).to(bf)
    ms = timer(lambda: torch.nn.functional.linear(torch.nn.functional.linear(xa, wgu[0])[:, :ff], wdn[0]))
    out["like_dense_ff_products"] = tf(6.0 * ff * W * pairs, ms)
    i1 = idx[:1].contiguous()
    ms = timer(lambda: nsq.moe_experts(hb[:1], i1, wgu, wdn, grouped=False, act=act), steps=15)
    out["moe_experts_decode"] = gb(top * 3.0 * ff * W * 2, ms)
    wl = (torch.randn(top * 3 * ff, W, device=dev) * W ** -0.5).to(bf)
    ms = timer(lambda: nsq.linear(hb[:1], wl, kernel=True), steps=15)
    out["like_linear_rows"] = gb(top * 3.0 * ff * W * 2, ms)
    return out


def run_safilorn(args, load_peaks, ClockSampler) -> None:
    from . import _native_seq as nsq
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    nsq.load()
    hbm, kind, tfl = load_peaks()
    timer = Timer(dev)
    sampler = ClockSampler(0)
    sampler.start()
    sampler.mark()
    before = nsq.launch_count()
    line = {"design": "safilorn", "compared_with": "mutolix (recurrent and attention layers in the same order, at the same sizes) on the same step function, "
                                                   "pool and kernels",
            "dtype": "bf16", "data": "synthetic", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "kind": kind},
            "timing": "CUDA events, 3 warm-up iterations, 256 MiB L2 flush between iterations, median", "sizes": {}}
    prompt, batch, ctx = 2048, 4, 2048
    for name, s in SAFILORN_SIZES.items():
        blk = safilorn_block(s, dev, timer, prompt, batch, ctx)
        blk["kernels"] = safilorn_kernels(s, dev, timer, prompt, ctx, hbm, tfl)
        line["sizes"][name] = blk
    line["gpu_launches"] = nsq.launch_count() - before
    line["clocks"] = sampler.stop()
    print(json.dumps(line), flush=True)


TEVILIX_SIZES = {
    # the recurrent and attention sizes of SIZES; a sliding window, a partly rotated head, the element-wise recurrence as wide as the model;
    # the feed-forward alternates dense (ff) and experts without a gate branch (E of eff, `top` active: the same active size)
    "w1024": dict(SIZES["w1024"], window=1024, rot=64, gru=1024, E=8, top=2, groups=(4, 2), eff=2048),
    "w2048": dict(SIZES["w2048"], window=1024, rot=64, gru=2048, E=16, top=4, groups=(4, 2), eff=2048),
}


def tevilix_config(s: dict) -> dict:
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["E"], "top": s["top"], "scale": 2.0, "groups": {"count": s["groups"][0], "keep": s["groups"][1]}}}
    par = lambda mlp: {"type": "parallel", "mlp": mlp,
                       "mixer": {"left": {"heads": s["H"], "kv_heads": s["G"], "dim": s["D"], "vdim": s["V"], "scale": s["D"] ** -0.5, "mask": {"size": s["window"]},
                                          "rot": {"base": 10000.0, "dims": s["rot"], "scaling": {"factor": 8.0}}},
                                 "left_scale": 0.7, "right": {"width": s["gru"]}, "right_scale": 0.8}}
    rec = lambda mlp: {"type": "mlstm", "mixer": {"heads": s["mH"], "dim": s["mD"], "vdim": s["mV"], "gate_cap": 15.0}, "mlp": mlp}
    # four layers; the wider size runs them `repeat` times as a loop where the model it is compared with has that many more layers
    return {"architecture": "Tevilix", "vocab": s["vocab"], "width": s["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "loop": {"start": 0, "stop": 4, "times": s["repeat"]}, "layers": [rec(dense), par(moe), par(dense), rec(moe)]}


def tevilix_tensors(cfg: dict, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    W, t = cfg["width"], {}
    rnd = lambda *shape, std=1.0, mean=0.0: (torch.randn(*shape, generator=g, device=device) * std + mean).to(torch.bfloat16)
    lin = lambda o, i: rnd(o, i, std=i ** -0.5)
    t["embed"], t["final.norm"], t["head"] = rnd(cfg["vocab"], W), rnd(W, std=0.05, mean=1.0), lin(cfg["vocab"], W)
    for i, layer in enumerate(cfg["layers"]):
        p, m, f = f"l{i}.", layer["mixer"], layer["mlp"]
        t[p + "norm1"], t[p + "norm2"] = rnd(W, std=0.05, mean=1.0), rnd(W, std=0.05, mean=1.0)
        if layer["type"] == "mlstm":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.g"] = lin(H * D, W), lin(H * D, W), lin(H * V, W), lin(H * V, W)
            t[p + "mix.o"], t[p + "mix.norm"] = lin(W, H * V) * 0.3, rnd(H * V, std=0.05, mean=1.0)
            t[p + "mix.i"], t[p + "mix.i.b"], t[p + "mix.f"], t[p + "mix.f.b"] = lin(H, W), rnd(H), lin(H, W), rnd(H, mean=3.0)
        else:
            a, q, r = m["left"], p + "mix.left.", p + "mix.right."
            H, G, D, V, R = a["heads"], a["kv_heads"], a["dim"], a["vdim"], m["right"]["width"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                t[q + n], t[q + n + ".b"] = lin(rows, W), rnd(rows, std=0.1)
            t[q + "q.norm"], t[q + "k.norm"] = rnd(D, std=0.1, mean=1.0), rnd(D, std=0.1, mean=1.0)
            t[q + "talk"] = (torch.eye(H, device=device) + torch.randn(H, H, generator=g, device=device) * 0.2).to(torch.bfloat16)
            t[q + "g"], t[q + "o"], t[q + "o.b"] = lin(H * V, W), lin(W, H * V) * 0.3, rnd(W, std=0.05)
            t[r + "z"], t[r + "z.b"], t[r + "x"], t[r + "x.b"] = lin(R, W), rnd(R), lin(R, W), rnd(R, std=0.3)
            t[r + "g"], t[r + "o"] = lin(R, W), lin(W, R) * 0.3
        if f["kind"] == "dense":
            t[p + "mlp.up"], t[p + "mlp.down"] = lin(f["ff"], W), lin(W, f["ff"]) * 0.3
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            t[p + "mlp.router"], t[p + "mlp.correction"] = rnd(E, W, std=3 * W ** -0.5), rnd(E, std=0.1)
            for e in range(E):
                t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = lin(ff, W), lin(W, ff) * 0.3
    return t


def tevilix_block(s: dict, dev, timer: Timer, prompt: int, batch: int, ctx: int) -> dict:
    from .model.mutolix import MutolixConfig, MutolixForCausalLM
    from .model.tevilix import TevilixConfig, TevilixForCausalLM
    cfg = tevilix_config(s)
    tc = TevilixConfig(cfg)
    out = {"layers": len(cfg["layers"]), "layer_runs": len(tc.runs), "width": s["width"], "active_ff": s["ff"]}
    m = TevilixForCausalLM(tc, tevilix_tensors(cfg, dev), device=dev, dtype=torch.bfloat16)
    _throughput(m, s, timer, prompt, batch, ctx, out)
    del m
    torch.cuda.empty_cache()
    mc = mutolix_config(s)   # the closest existing model: recurrent and attention layers in the same order, at the same sizes
    mm = MutolixForCausalLM(MutolixConfig(mc), random_tensors(mc, dev), device=dev, dtype=torch.bfloat16)
    _throughput(mm, s, timer, prompt, batch, ctx, out, prefix="mutolix_")
    del mm
    torch.cuda.empty_cache()
    return out


def tevilix_kernels(s: dict, dev, timer: Timer, prompt: int, ctx: int, hbm_gbs: float, tflops: float) -> dict:
    """Every kernel of the design alone at this size, achieved / peak, beside the like kernel of the closest model."""
    from . import _native_seq as nsq
    bf, H, G, D, V, W, R, win = torch.bfloat16, s["H"], s["G"], s["D"], s["V"], s["width"], s["gru"], s["window"]
    out = {}
    gb = lambda by, ms: {"us": round(ms * 1e3, 2), "gb_s": round(by / ms / 1e6, 1), "of_measured_hbm_peak": round(by / ms / 1e6 / hbm_gbs, 4)}
    tf = lambda fl, ms: {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1), "of_measured_bf16_peak": round(fl / ms / 1e9 / tflops, 3)}
    cap = ((max(prompt, ctx + 1) + 127) // 128) * 128
    b, b1 = nsq.Batch([0], [0], [prompt], dev), nsq.Batch([0], [ctx], [1], dev)
    talk = torch.eye(H, device=dev) + torch.randn(H, H, device=dev) * 0.2
    r1, r2 = torch.full((H,), 0.5, device=dev), torch.full((H,), 0.5, device=dev)
    pairs = sum(min(i + 1, win) for i in range(prompt))       # visible (query, key) pairs of the prompt under the window
    kp, vp = torch.randn(1, G, cap, D, device=dev).to(bf), torch.randn(1, G, cap, V, device=dev).to(bf)
    q, o, og = torch.randn(prompt, H * D, device=dev).to(bf), torch.empty(prompt, H * V, device=dev, dtype=bf), torch.randn(prompt, H * V, device=dev).to(bf)
    # prompt attention: FLOPs = 2 (D + V) per visible pair and head (the mixing's 2 H per pair and head comes on top and is not counted)
    ms = timer(lambda: nsq.attention(q, kp, vp, o, H, D ** -0.5, None, None, False, b, window=win, talk=talk, out_gate=og))
    out["attn_prompt_mixed_scores"] = dict(tf(2.0 * (D + V) * H * pairs, ms), uncounted_mixing_flops_share=round(H / (D + V), 3))
    ms = timer(lambda: nsq.attention(q, kp, vp, o, H, D ** -0.5, r1, r2, True, b, window=win))
    out["like_attn_prompt_same_window"] = tf(2.0 * (D + V) * H * pairs, ms)
    ms = timer(lambda: nsq.attention(q, kp, vp, o, H, D ** -0.5, r1, r2, True, b))
    out["like_attn_prompt_full_causal"] = tf(2.0 * (D + V) * H * prompt * (prompt + 1) / 2, ms)
    # decoding: one token over its window; bytes = the window's K and V rows of all key/value heads once
    q1, o1 = torch.randn(1, H * D, device=dev).to(bf), torch.empty(1, H * V, device=dev, dtype=bf)
    ws = nsq.attn_workspace(1, H, V, dev)
    seen = min(win, ctx + 1)
    ms = timer(lambda: nsq.attention(q1, kp, vp, o1, H, D ** -0.5, None, None, False, b1, max_keys=seen, workspace=ws, window=win, talk=talk, out_gate=og[:1]), steps=15)
    out["attn_decode_mixed_scores"] = gb(2.0 * G * seen * (D + V), ms)
    ms = timer(lambda: nsq.attention(q1, kp, vp, o1, H, D ** -0.5, r1, r2, True, b1, max_keys=seen, workspace=ws, window=win), steps=15)
    out["like_attn_decode_same_window"] = gb(2.0 * G * seen * (D + V), ms)
    # head norms + rotation + append, beside Mutolix's whole-projection norms + append (both read the projection row, write q and K/V rows)
    nq, nk = H * D, G * (D + V)
    pj = torch.randn(prompt, nq + nk, device=dev).to(bf)
    fr = torch.tensor([10000.0 ** (-2.0 * i / s["rot"]) / 4.0 for i in range(s["rot"] // 2)], dtype=torch.float64, device=dev)
    hn = torch.ones(D, device=dev, dtype=bf)
    ms = timer(lambda: nsq.rope_kv_prep(pj, (0, nq, nq + G * D), H, G, D, V, fr, s["rot"], False, False, 1e-5, q, kp, vp, b, q_norm_w=hn, k_norm_w=hn))
    out["head_norm_rope_append"] = gb(prompt * (nq + nk) * 4.0, ms)
    qn, kn = torch.ones(nq, device=dev, dtype=bf), torch.ones(G * D, device=dev, dtype=bf)
    ms = timer(lambda: nsq.qk_prep(pj, (0, nq, nq + G * D), qn, kn, 1e-5, H, G, D, V, 0.0, 0, q, kp, vp, None, None, b))
    out["like_qk_prep"] = gb(prompt * (nq + nk) * 4.0, ms)
    # the layer's residual sum of three branch results with both norms of the next layer: reads x (4 B) and three results (2 + 2 + 4 B),
    # writes x (4 B) and two inputs (2 + 2 B); like: gated norm + residual + next norm (reads y, gate, x; writes x, h)
    x, wn = torch.randn(prompt, W, device=dev), torch.ones(W, device=dev, dtype=bf)
    y1, y2, y3 = torch.randn(prompt, W, device=dev).to(bf), torch.randn(prompt, W, device=dev).to(bf), torch.randn(prompt, W, device=dev)
    h1, h2 = torch.empty(prompt, W, device=dev, dtype=bf), torch.empty(prompt, W, device=dev, dtype=bf)
    ms = timer(lambda: nsq.add_layer_norm(x, [(y1, 0.7), (y2, 0.8), (y3, 1.0)], 1e-5, wn, h1, wn, h2))
    out["add3_two_layer_norms"] = gb(prompt * W * 20.0, ms)
    ms = timer(lambda: nsq.gate_norm_add(x, y1, y2, wn, wn, 1e-5, wn, h1))
    out["like_gate_norm_add"] = gb(prompt * W * 14.0, ms)
    # the element-wise recurrence: reads three projections, writes the gated result (2 B each); one decoded token: state read and written
    pr = torch.randn(prompt, 3 * R, device=dev).to(bf)
    sp, go = torch.zeros(1, R, device=dev), torch.empty(prompt, R, device=dev, dtype=bf)
    ms = timer(lambda: nsq.gru_scan(pr, (0, R, 2 * R), R, go, sp, b))
    out["gru_scan_prompt"] = dict(gb(prompt * R * 8.0, ms), us_per_token=round(ms * 1e3 / prompt, 4))
    ms = timer(lambda: nsq.gru_scan(pr[:1], (0, R, 2 * R), R, go[:1], sp, b1), steps=15)
    out["gru_scan_decode"] = gb(R * 16.0, ms)
    # the matrix memory is Mutolix's own kernel (same entry point, same sizes): listed for the step's budget
    mH, mD, mV = s["mH"], s["mD"], s["mV"]
    pm = (torch.randn(prompt, 2 * mH * mD + 2 * mH * mV, device=dev) * 0.3).to(bf)
    offs = (0, mH * mD, 2 * mH * mD, 2 * mH * mD + mH * mV)
    ig, fg = torch.randn(prompt, mH, device=dev), -torch.rand(prompt, mH, device=dev) * 0.1
    spm, npool, mp = torch.zeros(1, mH, mD, mV, device=dev), torch.zeros(1, mH, mD, device=dev), torch.zeros(1, mH, device=dev)
    nwm, om = torch.ones(mH * mV, device=dev, dtype=bf), torch.empty(prompt, mH * mV, device=dev, dtype=bf)
    ms = timer(lambda: nsq.mlstm_scan(pm, offs, ig, fg, nwm, om, spm, npool, mp, 1e-5, b), steps=5)
    out["shared_mlstm_scan_prompt"] = {"ms": round(ms, 3), "us_per_token": round(ms * 1e3 / prompt, 3), "gflops": round(4.0 * mH * mD * mV * prompt / ms / 1e6, 1)}
    ms = timer(lambda: nsq.mlstm_scan(pm[:1], offs, ig[:1], fg[:1], nwm, om[:1], spm, npool, mp, 1e-5, b1), steps=15)
    out["shared_mlstm_scan_decode"] = gb(8.0 * mH * mD * mV, ms)
    # router, experts and the dense feed-forward's activation
    E, top, ff = s["E"], s["top"], s["eff"]
    hb = torch.randn(prompt, W, device=dev).to(bf)
    wr, corr = (torch.randn(E, W, device=dev) * 3 * W ** -0.5).to(bf), torch.randn(E, device=dev) * 0.1
    route = lambda: nsq.moe_route(hb, wr, corr, None, top, s["groups"][0], s["groups"][1], renorm=True, score_fn=nsq.ROUTE_SIGMOID, group_best=2, wgt_scale=2.0, renorm_eps=1e-20)
    ms = timer(route)
    out["moe_route_sigmoid_groups"] = gb(prompt * W * 2.0, ms)
    idx, wgt, _ = route()
    act = (nsq.ACT_RELU2, 0.0, 0.0)
    wup, wdn = (torch.randn(E, ff, W, device=dev) * W ** -0.5).to(bf), (torch.randn(E, W, ff, device=dev) * ff ** -0.5).to(bf)
    n_pairs = prompt * top
    ms = timer(lambda: nsq.moe_experts(hb, idx, wup, wdn, grouped="library", act=act))
    out["moe_experts_prompt"] = dict(tf(4.0 * ff * W * n_pairs, ms), what="plan + gather + library grouped products + squared relu")
    xa = torch.randn(n_pairs, W, device=dev).to(bf)
    ms = timer(lambda: torch.nn.functional.linear(torch.nn.functional.linear(xa, wup[0]), wdn[0]))
    out["like_dense_ff_products"] = tf(4.0 * ff * W * n_pairs, ms)
    i1 = idx[:1].contiguous()
    ms = timer(lambda: nsq.moe_experts(hb[:1], i1, wup, wdn, grouped=False, act=act), steps=15)
    out["moe_experts_decode"] = gb(top * 2.0 * ff * W * 2, ms)
    wl = (torch.randn(top * 2 * ff, W, device=dev) * W ** -0.5).to(bf)
    ms = timer(lambda: nsq.linear(hb[:1], wl, kernel=True), steps=15)
    out["like_linear_rows"] = gb(top * 2.0 * ff * W * 2, ms)
    u = torch.randn(prompt, s["ff"], device=dev).to(bf)
    ms = timer(lambda: nsq.glu_mul(u, s["ff"], (nsq.ACT_GELU_ERF, 0.0, 0.0)))
    out["gelu_erf"] = gb(prompt * s["ff"] * 4.0, ms)
    ua, av = torch.empty_like(u), torch.randn(2, device=dev).to(bf)
    ms = timer(lambda: nsq.xielu(u, ua, av))
    out["like_xielu"] = gb(prompt * s["ff"] * 4.0, ms)
    return out


def run_tevilix(args, load_peaks, ClockSampler) -> None:
    from . import _native_seq as nsq
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    nsq.load()
    hbm, kind, tfl = load_peaks()
    timer = Timer(dev)
    sampler = ClockSampler(0)
    sampler.start()
    sampler.mark()
    before = nsq.launch_count()
    line = {"design": "tevilix", "compared_with": "mutolix (recurrent and attention layers in the same order, at the same sizes; where this design loops over "
                                                  "four layers it has as many layers more) on the same step function, pool and kernels",
            "dtype": "bf16", "data": "synthetic", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "kind": kind},
            "timing": "CUDA events, 3 warm-up iterations, 256 MiB L2 flush between iterations, median", "sizes": {}}
    prompt, batch, ctx = 2048, 4, 2048
    for name, s in TEVILIX_SIZES.items():
        blk = tevilix_block(s, dev, timer, prompt, batch, ctx)
        blk["kernels"] = tevilix_kernels(s, dev, timer, prompt, ctx, hbm, tfl)
        line["sizes"][name] = blk
    line["gpu_launches"] = nsq.launch_count() - before
    line["clocks"] = sampler.stop()
    print(json.dumps(line), flush=True)


def run(args, load_peaks, ClockSampler) -> None:
    if args.design == "tevilix":
        return run_tevilix(args, load_peaks, ClockSampler)
    if args.design == "raritar":
        return run_raritar(args, load_peaks, ClockSampler)
    if args.design == "safilorn":
        return run_safilorn(args, load_peaks, ClockSampler)
    from . import _native as nat, _native_seq as nsq, build as pc_build
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pc_build.build()
    nat.load()
    nsq.load()
    hbm, kind, tfl = load_peaks()
    timer = Timer(dev)
    sampler = ClockSampler(0)
    sampler.start()
    sampler.mark()
    before = nat.launch_count() + nsq.launch_count()
    line = {"design": "mutolix", "compared_with": "llama (fp16 prompt-cache path) at equal width, depth, kv heads and feed-forward",
            "dtype": "bf16", "data": "synthetic", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "kind": kind},
            "timing": "CUDA events, 3 warm-up iterations, 256 MiB L2 flush between iterations, median", "sizes": {}}
    prompt, batch, ctx = 2048, 4, 2048
    for name, s in SIZES.items():
        blk = model_block(name, s, dev, timer, prompt, batch, ctx)
        blk["kernels"] = kernel_block(s, dev, timer, prompt, ctx, hbm, tfl)
        line["sizes"][name] = blk
    line["gpu_launches"] = nat.launch_count() + nsq.launch_count() - before
    line["clocks"] = sampler.stop()
    print(json.dumps(line), flush=True)


def run_raritar(args, load_peaks, ClockSampler) -> None:
    from . import _native_seq as nsq
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    nsq.load()
    hbm, kind, tfl = load_peaks()
    timer = Timer(dev)
    sampler = ClockSampler(0)
    sampler.start()
    sampler.mark()
    before = nsq.launch_count()
    line = {"design": "raritar", "compared_with": "mutolix attention layers (full causal attention, dense feed-forward of the active size) on the same "
                                                  "step function, pool and kernels",
            "dtype": "bf16", "data": "synthetic", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "kind": kind},
            "timing": "CUDA events, 3 warm-up iterations, 256 MiB L2 flush between iterations, median", "sizes": {}}
    prompt, batch, ctx = 2048, 4, 2048
    for name, s in RARITAR_SIZES.items():
        blk = raritar_block(s, dev, timer, prompt, batch, ctx)
        blk["kernels"] = raritar_kernels(s, dev, timer, prompt, ctx, hbm, tfl)
        line["sizes"][name] = blk
    line["gpu_launches"] = nsq.launch_count() - before
    line["clocks"] = sampler.stop()
    print(json.dumps(line), flush=True)
