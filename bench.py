#!/usr/bin/env python
"""Headline benchmark: Llama-2-7B TTFT (ms) and prefill tok/s on the prompt-cache hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--config C1|C2|C3|C4|C5]

One step = one request on BASELINE config C2 (code-generation-game shape: 7 cached segments [24,400x5,24] = 2048
tokens, 16-token uncached suffix): request plan -> splice of ALL segments (retained-prefix shortcut off) -> 32-layer
prefill of the suffix over the spliced cache (per layer: QKV projection with RoPE at position ids + in-place append in
its epilogue, tcgen05 attention, o_proj / MLP as weight-streaming tcgen05 kernels) -> logits.  TTFT = ms_per_step;
value = served prompt tokens/s = n_gpus*(N+q)/TTFT ("effective"); `computed_tok_s` = n_gpus*q/TTFT.  Weights are seeded
random fp16 at the real dims, token ids synthetic (no network).

N>1: one rank per GPU, every rank serves its own prompt against its own HBM-resident segment store (weak scaling, no
data-path collective); NCCL only for the barrier, the max-over-ranks time and the one-time broadcast of the encoded
segment store.  Every line also carries a `c5` block: BASELINE config C5 (B=64 prompts, each 32 of a 64-segment pool
= 8192 cached tokens + 32-token suffix) served through `parallel.serve_batch`'s partition (prompt b -> rank b mod G),
with the NCCL pool broadcast timed against the NVLink peer rate.  At N=1 the line also carries `c4` (Falcon-7B real
dims, parameterized schema), the suffix sweep S and the CPU baseline.

`--impl reference` runs the UNMODIFIED reference (oracle/_ref, staged by oracle/make_ref.py) through its own
CacheEngine.process -> GenerationEngine.generate on the host cores, all layers (cpu_baseline.kind "reference"); only
when the staged copy is missing does it fall back to the oracle port (kind "port").
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

NVLINK_PEER_GBS = 770.0  # measured peer-copy rate per direction (B200_PROFILING.md); denominator of the pool broadcast


def load_traffic(kernel, config):
    """DRAM traffic per launch measured once with `ncu --set full` (committed under profiles/), or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as fh:
            t = json.load(fh).get(kernel)
        return float(t["bytes"]) if t and t.get("config") == config else None
    except Exception:
        return None


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            p = json.load(fh)
        return float(p["hbm_gbs"]), "measured", float(p.get("bf16_tflops", 1590.0))
    except Exception:
        return 6650.0, "fallback", 1590.0


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled DURING the timed region."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines, self.first = index, None, [], 0

    def mark(self):
        """Samples before this point (warm-up) are not reported."""
        self.first = len(self.lines)

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, upto=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines[self.first:upto]:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
SEG_LENS = {"C1": [24] + [92] * 6 + [24], "C2": [24] + [400] * 5 + [24], "C3": [512] * 8}


def build_lm(model_key, dev, layers=None):
    """The CUDA-path LanguageModel of a BASELINE config at real dims, seeded random fp16 weights."""
    from promptcache_b200.model import Falcon, Llama2, LlamaConfigLite, LlamaForCausalLM
    from promptcache_b200.model.falcon import FalconConfigLite, FalconForCausalLM
    from promptcache_b200.synthetic import MODEL_DIMS, IdTokenizer
    md = dict(MODEL_DIMS[model_key])
    if layers:
        md["num_hidden_layers"] = layers
    torch.manual_seed(0)
    tok = IdTokenizer(md["vocab_size"])
    if model_key.startswith("falcon"):
        return Falcon(model_key, model=FalconForCausalLM(FalconConfigLite(**md), device=dev), tokenizer=tok), md
    if model_key.startswith("mpt"):
        from promptcache_b200.model import Mpt
        from promptcache_b200.model.mpt import MptConfigLite, MptForCausalLM
        cfg = MptConfigLite(d_model=md["hidden_size"], n_heads=md["num_attention_heads"], n_layers=md["num_hidden_layers"],
                            vocab_size=md["vocab_size"], max_seq_len=md.get("max_seq_len", 8192))
        return Mpt(model_key, model=MptForCausalLM(cfg, device=dev), tokenizer=tok), md
    return Llama2(model_key, model=LlamaForCausalLM(LlamaConfigLite(**md), device=dev), tokenizer=tok), md


def weight_bytes(md, model_key):
    """fp16 bytes of every matrix one forward streams once (embedding rows excluded: q rows only)."""
    hid, L, V = md["hidden_size"], md["num_hidden_layers"], md["vocab_size"]
    if model_key.startswith("mpt"):
        per = 12 * hid * hid
    elif model_key.startswith("falcon"):
        D = hid // md["num_attention_heads"]
        per = (hid + 2 * D) * hid + hid * hid + 8 * hid * hid
    else:
        per = 4 * hid * hid + 3 * hid * md["intermediate_size"]
    return 2.0 * (L * per + V * hid)


class RequestStep:
    """One request of a flat BASELINE config (C1-C4) on one GPU: device-resident arm and public-API arm."""

    def __init__(self, lm, case, dev, world, rank, seg_lens=None):
        from promptcache_b200 import CacheEngine, GenerationEngine, GenerationParameters, Prompt, parallel
        from promptcache_b200.synthetic import flat_schema
        self.lm, self.case, self.dev = lm, case, dev
        max_ctx = ((case.n_cached + case.q_len + 256 + 127) // 128) * 128
        self.eng = eng = CacheEngine(max_ctx, lm)
        eng.prompt_cache.retain_prefix = False  # every step splices every segment
        self.broadcast = None
        if world > 1:
            # rank 0 encodes the schema once; the segment store reaches the other GPUs over NCCL (NVLink)
            eng.add_schema(case.schema_xml, no_cache=(rank != 0))
            self.broadcast = timed_broadcast(eng.schemas[case.name], dev)
        else:
            eng.add_schema(case.schema_xml)
        prompt_xml = case.prompt_xml
        if world > 1 and seg_lens is not None:  # each rank serves its own prompt (same modules, its own suffix tokens)
            prompt_xml = flat_schema(case.name, seg_lens, case.q_len, lm.hf_tokenizer.vocab_size, seed=1002 + 17 * rank).prompt_xml
        self.prompt = Prompt(prompt_xml)
        self.gen = GenerationEngine(lm)
        self.params = GenerationParameters(temperature=0.0, max_new_tokens=1, stop_token_ids=[], stop_str=[])
        self.full_ids = bool(getattr(lm, "use_full_position_ids", False))  # MPT: ids of the cached rows + the new tokens
        ids, pos, _, _ = eng.process(self.prompt, return_full_position_ids=self.full_ids)
        self.q_len = len(ids)
        self.ids_dev = torch.tensor([ids], device=dev)
        self.pos_dev = torch.tensor([pos], device=dev)
        cached, used, _, _, _, _ = eng.plan(self.prompt, collect_original=False)
        self.seq_caches = [cached.get_cache_l1(s) for s in used if len(s) > 0]
        self.max_pos = max(pos)
        self.splice_ev = []
        # virtual splice (the engine's default whenever the model's short-suffix attention can read the arena in place)
        self.virtual = eng.virtual_splice and 0 < self.q_len <= getattr(lm.hf_model, "virtual_kv_max_q", lambda: 0)()

    def device_step(self, record=False, virtual=None):
        """ids already in HBM, no host sync inside the step."""
        virtual = self.virtual if virtual is None else virtual
        if record:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        self.eng.prompt_cache.update(self.seq_caches, virtual=virtual, slot_rows=self.full_ids)
        if record:
            e1.record()
            self.splice_ev.append((e0, e1))
        return self.lm(input_ids=self.ids_dev, position_ids=self.pos_dev, past_key_values=self.eng.prompt_cache.cache.batched(),
                       use_cache=True, max_position=self.max_pos)

    def e2e_step(self):
        """The public API with host inputs (token lists -> device) and the first token read back."""
        i2, p2, _, cache = self.eng.process(self.prompt, return_full_position_ids=self.full_ids)
        return next(self.gen.generate(i2, p2, self.params, cache, stream_interval=1, use_full_position_ids=self.full_ids))

    def decode_ms_per_token(self, n_tokens=17):
        """Greedy decode after the prefill through the public API; first pass warms up (graph capture), second is reported."""
        from promptcache_b200 import GenerationParameters
        dparams = GenerationParameters(temperature=0.0, max_new_tokens=n_tokens, stop_token_ids=[], stop_str=[])
        outs = []
        for _ in range(2):
            i2, p2, _, cache = self.eng.process(self.prompt, return_full_position_ids=self.full_ids)
            outs = list(self.gen.generate(i2, p2, dparams, cache, use_full_position_ids=self.full_ids))
        return (outs[-1].response_time - outs[0].response_time) / (n_tokens - 1)

    def timed(self, fn, steps, sync_all):
        sync_all()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            fn()
        t1.record()
        sync_all()
        return t0.elapsed_time(t1) / steps


def timed_broadcast(schema_cache, dev):
    """NCCL broadcast of the encoded segment store from rank 0, device-timed, max over ranks."""
    import torch.distributed as dist
    from promptcache_b200 import parallel
    # the first collectives of a process group set up the NCCL communicator and, for large messages, its channels / buffers
    # (~50-100 ms): warm both up, untimed
    warm = torch.zeros(32 << 20, dtype=torch.half, device=dev)
    for _ in range(2):
        dist.broadcast(warm, src=0)
    del warm
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    moved = parallel.broadcast_schema(schema_cache, src=0, device=dev)
    e1.record()
    torch.cuda.synchronize()
    ms = parallel.max_over_ranks(e0.elapsed_time(e1), device=dev)
    gbs = moved["bytes"] / (ms * 1e-3) / 1e9 if ms > 0 else None
    return {"bytes": moved["bytes"], "segments": moved["segments"], "ms": ms, "GB/s": gbs, "peer_peak_GB/s": NVLINK_PEER_GBS,
            "frac_of_peer_peak": (gbs / NVLINK_PEER_GBS) if gbs else None,
            "note": "ONE ncclBroadcast of the schema's segment arena [L,2,Hkv,R,D], rank 0 -> all, device-timed, max over ranks; "
                    "includes the object broadcast of the shape header"}


def c5_block(lm, dev, world, rank, batch=64, pool=64, picks=32, seg_len=256, suffix=32):
    """BASELINE configs[4]: Llama-2-7B, a pool of 64 segments x 256 tokens, B=64 prompts each choosing 32 (seed 5) ->
    N=8192 cached tokens + 32-token suffix, sharded b mod G over the ranks.  Timed through the public calls
    (CacheEngine.process + GenerationEngine.generate(max_new_tokens=1)), host id lists in, token out."""
    import random
    import torch.distributed as dist
    from promptcache_b200 import CacheEngine, GenerationEngine, GenerationParameters, Prompt, parallel
    from promptcache_b200.synthetic import pool_prompt, pool_schema
    vocab = lm.hf_tokenizer.vocab_size
    schema_xml, names = pool_schema("pool", pool, seg_len, vocab, seed=1005)
    n_cached = picks * seg_len
    max_ctx = ((n_cached + suffix + 256 + 127) // 128) * 128
    eng = CacheEngine(max_ctx, lm)
    t0 = time.perf_counter()
    eng.add_schema(schema_xml, no_cache=(world > 1 and rank != 0))
    torch.cuda.synchronize()
    encode_s = time.perf_counter() - t0
    bc = timed_broadcast(eng.schemas["pool"], dev) if world > 1 else None
    rng = random.Random(5)
    prompts = [Prompt(pool_prompt("pool", sorted(rng.sample(names, picks), key=lambda n: int(n[1:])), suffix, vocab, seed=5000 + b))
               for b in range(batch)]
    gen = GenerationEngine(lm)
    params = GenerationParameters(temperature=0.0, max_new_tokens=1, stop_token_ids=[], stop_str=[])

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out = {}
    for mode, virtual, retain in (("virtual_splice", True, False), ("copied_splice", False, False), ("copied_retained_prefix", False, True)):
        eng.virtual_splice = virtual
        eng.prompt_cache.retain_prefix = retain
        for m in eng.schemas["pool"].cache_l1.values():
            m.usage_counter = 0
        eng.prompt_cache.invalidate()
        parallel.serve_batch(eng, gen, prompts[:2 * world], params)  # warm-up: graph capture of the (q, N) shape
        for m in eng.schemas["pool"].cache_l1.values():
            m.usage_counter = 0
        eng.prompt_cache.invalidate()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        served = parallel.serve_batch(eng, gen, prompts, params)
        e1.record()
        sync_all()
        ms = parallel.max_over_ranks(e0.elapsed_time(e1), device=dev)
        ttft = [s.ttft_ms for s in served]
        spliced = sum(s.spliced_rows for s in served)
        out[mode] = {"batch_ms": ms, "tok_s": batch * (n_cached + suffix) / (ms * 1e-3), "computed_tok_s": batch * suffix / (ms * 1e-3),
                     "ttft_ms_mean": statistics.mean(ttft), "ttft_ms_max": max(ttft),
                     "cache_ms_mean": statistics.mean(s.cache_ms for s in served),
                     "prefill_ms_mean": statistics.mean(s.prefill_ms for s in served),
                     "spliced_rows": spliced, "retained_row_fraction": 1.0 - spliced / float(batch * n_cached),
                     "prompts_per_rank": [sum(1 for s in served if s.rank == r) for r in range(world)]}
    L, Hkv, D = lm.get_cache_shape()
    res = {"workload": f"C5: {batch} prompts x ({picks} of a {pool}-segment pool x {seg_len} tokens = {n_cached} cached + {suffix} suffix), "
                       f"prompt b -> rank b mod {world}; public API (process + generate(1)), max over ranks",
           "n_gpus": world, "pool_bytes": 4.0 * L * Hkv * D * pool * seg_len, "encode_s_rank0": encode_s, "broadcast": bc,
           "tok_s": out["virtual_splice"]["tok_s"], "ttft_ms_max": out["virtual_splice"]["ttft_ms_max"], **out,
           "note": "virtual_splice (engine default): attention reads the pool's arena through the request's tile list, nothing is "
                   "copied; copied_splice: every request moves all 8192 rows (8 GiB of HBM traffic, the reference's PromptCache.update); "
                   "copied_retained_prefix: the copy with the usage-ordered layout + retained common prefix (cache_engine.py:121-131)"}
    del eng
    return res


def family_block(model_key, cfg_name, dev, steps, warmup):
    """Another model family on the same engine, one request per step.  C4 = BASELINE configs[3]: Falcon-7B at real dims
    (H=71, Hkv=1, D=64, hidden 4544, 32 layers), parameterized schema: 5 segments = 256 cached tokens, 21-token suffix of
    which 5 sit at interior parameter slots (non-monotone ids).  MPT-7B (ALiBi at key ids, full position ids) is run on
    the C2 schema shape."""
    from promptcache_b200.synthetic import make_case
    lm, md = build_lm(model_key, dev)
    case = make_case(cfg_name, vocab=md["vocab_size"])
    w = RequestStep(lm, case, dev, 1, 0)
    sync = torch.cuda.synchronize
    for _ in range(warmup):
        w.device_step()
    dev_ms = w.timed(lambda: w.device_step(True), steps, sync)
    for _ in range(warmup):
        w.e2e_step()
    e2e_ms = w.timed(w.e2e_step, steps, sync)
    tokens = case.n_cached + case.q_len
    wb = weight_bytes(md, model_key)
    peak, _, _ = load_peaks()
    try:
        decode_ms = w.decode_ms_per_token()
    except Exception as ex:
        decode_ms = f"failed: {type(ex).__name__}: {ex}"
    res = {"workload": f"{cfg_name}: {model_key}, {case.n_segments} cached segments = {case.n_cached} tokens, {case.q_len}-token suffix "
                       f"(suffix position ids {w.pos_dev[0, -case.q_len:][:6].tolist()}...), one request per step",
           "ttft_ms": dev_ms, "tok_s": tokens / (dev_ms * 1e-3), "computed_tok_s": case.q_len / (dev_ms * 1e-3),
           "e2e_ttft_ms": e2e_ms, "e2e_tok_s": tokens / (e2e_ms * 1e-3), "decode_ms_per_token": decode_ms,
           "splice_ms": statistics.mean(a.elapsed_time(b) for a, b in w.splice_ev),
           "roofline_step": {"bound": "hbm", "algorithmic_bytes": wb, "achieved": wb / (dev_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                             "frac": wb / (dev_ms * 1e-3) / 1e9 / peak,
                             "note": "weights only; " + ("cuBLAS linears (the weight-streaming kernel ties with them at Falcon's shapes), "
                                                         "long-suffix attention kernel with the 71 heads folded into M"
                                                         if model_key.startswith("falcon") else
                                                         "weight-streaming linears, virtual splice with ALiBi key ids in tile order")}}
    del w, lm
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------------
# attention micro-benchmarks (kernel alone; the step's own attribution comes from the ablation runs in main)
# ------------------------------------------------------------------------------------------------
def attention_point(nat, dev, H, Hkv, D, q, N, peak, tflops_peak, rounding=None, launches=16):
    """One (q, N) point of pc_prefill_attn timed ALONE: a CUDA graph of `launches` back-to-back launches rotating over
    enough layers of K/V to exceed L2."""
    rounding = nat.PC_ROUND_LLAMA if rounding is None else rounding
    max_ctx = ((N + q + 127) // 128) * 128
    per_layer = 4.0 * Hkv * max_ctx * D
    rot = max(2, min(8, int(300e6 // per_layer) + 1))
    K = torch.randn(rot, Hkv, max_ctx, D, device=dev).half()
    V = torch.randn(rot, Hkv, max_ctx, D, device=dev).half()
    Q = torch.randn(H, q, D, device=dev).half()
    out = torch.empty(q, H * D, dtype=torch.half, device=dev)
    ws = torch.zeros(max(nat.attn_workspace_bytes(H, q, D), 1), dtype=torch.uint8, device=dev)
    state = {"i": 0}

    def run():
        l = state["i"] % rot
        state["i"] += 1
        nat.attention(Q, K[l], V[l], out, N, q, H, Hkv, D, nat.softmax_scale(D), rounding, workspace=ws, decode=(q == 1))

    run()
    torch.cuda.synchronize()
    g, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(st):
        run()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=st):
            for _ in range(launches):
                run()
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    reps = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (reps * launches)
    byts = 4.0 * Hkv * (N + q) * D + 4.0 * H * q * D
    flops = 4.0 * H * D * (q * N + q * (q + 1) / 2)  # causal-aware: key N+t is visible to rows r >= t
    gbs, tf = byts / (ms * 1e-3) / 1e9, flops / (ms * 1e-3) / 1e12
    G = H // Hkv
    return {"q": q, "N": N, "H": H, "Hkv": Hkv, "D": D, "us": ms * 1e3, "GB/s": gbs, "frac_hbm": gbs / peak, "TFLOP/s": tf,
            "frac_tensor": tf / tflops_peak, "bound": "hbm" if G * q < 254 else "tensor",
            "algorithmic_bytes_per_launch": byts, "algorithmic_flops_per_launch": flops}


def suffix_sweep(nat, dev, peak, tflops_peak):
    """q in {16, 64, 256, 1024} over the C2 and C5 cached lengths, no-cache full prefill q=N, and the
    Falcon MQA geometry."""
    pts = []
    for (H, Hkv, D, q, N, rnd, tag) in [(32, 32, 128, 16, 2048, None, "C2"), (32, 32, 128, 64, 2048, None, "C2"),
                                        (32, 32, 128, 256, 2048, None, "C2"), (32, 32, 128, 1024, 2048, None, "C2"),
                                        (32, 32, 128, 2048, 0, None, "C2 no-cache, q=N"), (32, 32, 128, 32, 8192, None, "C5"),
                                        (32, 32, 128, 1024, 8192, None, "C5"), (71, 1, 64, 21, 256, 0, "C4 falcon"),
                                        (71, 1, 64, 256, 2048, 0, "falcon MQA")]:
        try:
            p = attention_point(nat, dev, H, Hkv, D, q, N, peak, tflops_peak, rounding=rnd, launches=8 if q >= 256 else 16)
            p["shape"] = tag
            pts.append(p)
        except Exception as ex:
            pts.append({"q": q, "N": N, "shape": tag, "error": str(ex)})
    return pts


# ------------------------------------------------------------------------------------------------
# CPU arm
# ------------------------------------------------------------------------------------------------
class PortReference:
    """Fallback when oracle/_ref is absent: the oracle restatement, 2 of L layers timed and scaled (kind "port")."""

    kind = "port"

    def __init__(self, dims, n_cached, q_len, seg_lens, sample_layers, threads):
        from oracle import pc_oracle as O
        self.O = O
        torch.set_num_threads(threads)
        self.L, H, hid = dims["L"], dims["H"], dims["hidden"]
        self.sample_layers, self.threads = sample_layers, threads
        D = hid // H
        g = torch.Generator().manual_seed(0)
        self.segs = [[(torch.randn(H, n, D, generator=g).half(), torch.randn(H, n, D, generator=g).half())
                      for _ in range(self.L)] for n in seg_lens]
        self.buf = O.new_prompt_cache(self.L, H, n_cached + 256, D)
        self.sd = O.random_llama_state_dict(dims["vocab"], hid, dims["inter"], sample_layers, H, H, seed=0, dtype=torch.float32)
        rope_rows = max(4096, ((n_cached + q_len + 1023) // 1024) * 1024)
        self.cfg = dict(n_layers=sample_layers, n_heads=H, n_kv_heads=H, eps=1e-5, theta=10000.0, max_pos=rope_rows)
        self.ids = torch.randint(3, dims["vocab"], (1, q_len), generator=g)
        self.pos = torch.arange(n_cached, n_cached + q_len).unsqueeze(0)
        self.cos, self.sin = O.rope_tables(D, rope_rows)
        self.n_cached = n_cached

    def step(self):
        O = self.O
        with torch.inference_mode():
            t0 = time.perf_counter()
            n = O.splice_into(self.buf, self.segs, [0] * len(self.segs))
            t1 = time.perf_counter()
            past = [(self.buf[l][0][:, :n].unsqueeze(0), self.buf[l][1][:, :n].unsqueeze(0)) for l in range(self.sample_layers)]
            t2 = time.perf_counter()
            O.llama_forward(self.sd, self.cfg, self.ids, self.pos, past, cos=self.cos, sin=self.sin)
            t3 = time.perf_counter()
            x = torch.nn.functional.embedding(self.ids, self.sd["model.embed_tokens.weight"])
            torch.nn.functional.linear(O.rms_norm(x, self.sd["model.norm.weight"], 1e-5), self.sd["lm_head.weight"]).float()
            t4 = time.perf_counter()
        head = t4 - t3
        layers = max((t3 - t2) - head, 0.0) * (self.L / self.sample_layers)
        return dict(ttft_s=(t1 - t0) + layers + head, cache_ms=(t1 - t0) * 1e3)

    def describe(self):
        return (f"oracle PORT (oracle/_ref missing): full splice of {self.n_cached} rows x {self.L} layers + {self.sample_layers} of "
                f"{self.L} decoder layers fp32 (time x{self.L // self.sample_layers}) + embedding/norm/lm_head")


class RealReference:
    """The unmodified reference's own classes on the host cores: fp32 weights as `Llama2(name, device_map=None)` loads
    them (eval_sys.py:45-51), fp16 PromptCache (cache_engine.py:104-107), ALL layers, nothing extrapolated."""

    kind = "reference"

    def __init__(self, arch, md, case, threads, synthetic_segments):
        from oracle import ref_runner
        from promptcache_b200.synthetic import IdTokenizer
        torch.set_num_threads(threads)
        t0 = time.perf_counter()
        self.lm = ref_runner.build_reference_lm(arch, md, IdTokenizer(md["vocab_size"]), dtype=torch.float32, device="cpu", seed=0)
        self.build_s = time.perf_counter() - t0
        max_ctx = ((case.n_cached + case.q_len + 256 + 127) // 128) * 128
        self.run = ref_runner.ReferenceTTFT(self.lm, case.schema_xml, case.prompt_xml, max_ctx, device="cpu",
                                            synthetic_segments=synthetic_segments)
        self.synthetic_segments, self.case, self.layers = synthetic_segments, case, md["num_hidden_layers"]

    def step(self):
        import contextlib
        # the reference prints "Prefill latency" on stdout (generation_engine.py:115); stdout carries the one JSON line only
        with torch.inference_mode(), contextlib.redirect_stdout(sys.stderr):
            return self.run.step(invalidate=True)

    def describe(self):
        seg = ("segment K/V synthetic N(0,1) in the reference's own TokenSequenceCache objects (schema encode skipped: it is "
               "outside the TTFT)" if self.synthetic_segments else f"schema encoded by the reference's add_schema ({self.run.encode_s:.0f} s, untimed)")
        return (f"UNMODIFIED reference (oracle/_ref) CacheEngine.process + GenerationEngine.generate(max_new_tokens=1), all "
                f"{self.layers} layers, fp32 weights / fp16 prompt cache on the host cores, every step re-splices all "
                f"{self.case.n_cached} rows; {seg}")


def make_cpu_reference(args, case, md, dims, seg_lens, threads, synthetic_segments):
    from oracle import ref_shim
    arch = "falcon" if args.config == "C4" else "llama"
    want = os.environ.get("PC_BENCH_CPU", "reference")
    if want == "reference" and ref_shim.reference_available():
        return RealReference(arch, md, case, threads, synthetic_segments and arch == "llama")
    if arch != "llama":
        raise RuntimeError("the oracle port covers Llama only")
    return PortReference(dims, case.n_cached, case.q_len, seg_lens, int(os.environ.get("PC_BENCH_CPU_LAYERS", "2")), threads)


def run_reference(args, case, md, dims, seg_lens):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    threads = os.cpu_count() or 1
    ref = make_cpu_reference(args, case, md, dims, seg_lens, threads, synthetic_segments=False)
    recs = []
    for i in range(args.warmup + args.steps):
        r = ref.step()
        if i >= args.warmup:
            recs.append(r)
    ttft = statistics.mean(r["ttft_s"] for r in recs)
    tokens = case.n_cached + case.q_len
    line = {"impl": "reference", "metric": metric_name(args), "value": tokens / ttft, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ttft * 1e3, "ttft_ms": ttft * 1e3,
            "computed_tok_s": case.q_len / ttft, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 weights / f16 cache (CPU)", "data": "synthetic", "config": config_dict(args, case),
            "cpu_baseline": {"value": tokens / ttft, "unit": "tok/s", "cores": threads, "kind": ref.kind, "sample": ref.describe(),
                             "cache_ms": statistics.mean(r["cache_ms"] for r in recs),
                             "ttft_ms_min": min(r["ttft_s"] for r in recs) * 1e3},
            "e2e": {"value": tokens / ttft, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def metric_name(args):
    from promptcache_b200.synthetic import CONFIGS
    model = {"llama2-7b": "Llama-2-7B", "llama2-13b": "Llama-2-13B", "falcon-7b": "Falcon-7B", "mpt-7b": "MPT-7B"}[CONFIGS[args.config]["model"]]
    return f"{model} prefill tok/s (served prompt tokens / TTFT; TTFT = ms_per_step)"


def config_dict(args, case):
    from promptcache_b200.synthetic import CONFIGS
    return {"workload": f"{args.config}: {CONFIGS[args.config]['model']}, {case.n_segments} cached segments = {case.n_cached} tokens, "
                        f"{case.q_len}-token uncached suffix, one request per GPU per step",
            "n_cached": case.n_cached, "q_len": case.q_len, "segments": case.n_segments,
            "l2": "inputs larger than L2 (1 GiB of segments + 13.5 GB of weights stream per step)",
            "parallelism": f"batch partition x{args.gpus} (replicated weights and segment store)",
            "untimed_steps_before_timing": f"{args.warmup} (--warmup) + {max(args.warmup, 48)} after the clock sampler came up"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="C2", choices=["C1", "C2", "C3", "C4", "C5"])
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (marks the line invalid)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the c5 / c4 / sweep / ablation blocks (headline only)")
    ap.add_argument("--design", default=None, choices=["mutolix", "raritar", "safilorn", "tevilix"],
                    help="instead of the headline workload: prefill / decode throughput and per-kernel rooflines of that design "
                         "beside the closest prompt-cache model at equal sizes (one GPU, one JSON line)")
    ap.add_argument("--profile", action="store_true",
                    help="after warm-up run ONE step between cudaProfilerStart/Stop and exit (for ncu --profile-from-start off)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.design in ("mutolix", "raritar", "safilorn", "tevilix"):
        from promptcache_b200 import bench_seq
        bench_seq.run(args, load_peaks, ClockSampler)
        return

    from promptcache_b200.synthetic import CONFIGS, MODEL_DIMS, make_case
    c5_only = args.config == "C5"
    flat_cfg = "C2" if c5_only else args.config
    model_key = CONFIGS[flat_cfg]["model"]
    md = dict(MODEL_DIMS[model_key])
    if args.layers:
        md["num_hidden_layers"] = args.layers
    case = make_case(flat_cfg, vocab=md["vocab_size"])
    seg_lens = SEG_LENS.get(flat_cfg)
    dims = dict(L=md["num_hidden_layers"], H=md["num_attention_heads"], hidden=md["hidden_size"],
                inter=md.get("intermediate_size", 4 * md["hidden_size"]), vocab=md["vocab_size"])
    if args.impl == "reference":
        if c5_only:
            print(json.dumps({"impl": "reference", "unavailable": "C5 on host cores needs a 16384-token fp32 schema encode (34 GB of "
                              "scores per layer); the reference arm runs C1-C4"}), flush=True)
            return
        run_reference(args, case, md, dims, seg_lens)
        return

    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from promptcache_b200 import _native as nat, build as pc_build, parallel
    if rank == 0:
        pc_build.build()
    if world > 1:
        dist.barrier()
    nat.load()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    lm, md = build_lm(model_key, dev, args.layers)
    model = lm.hf_model
    if c5_only:  # C5 as the whole run: print its block as the line
        blk = c5_block(lm, dev, world, rank)
        if rank == 0:
            print(json.dumps({"metric": "Llama-2-7B prefill tok/s, C5 batch (64 prompts x 8224 tokens) over the node", "value": blk["tok_s"],
                              "unit": "tok/s", "n_gpus": world, "higher_is_better": True, "scaling": "strong", "dtype": "f16",
                              "data": "synthetic", "config": {"workload": blk["workload"]}, "c5": blk}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    w = RequestStep(lm, case, dev, world, rank, seg_lens)
    tokens_per_step = case.n_cached + w.q_len

    # The clock sampler (nvidia-smi -lms) is started BEFORE the warm-up: its start-up enumerates every GPU of the box
    # and can hold the driver for tens of ms, which must not land in the timed region.  Only the samples taken from
    # the start of the timed region on are reported.
    sampler = ClockSampler(local)
    if rank == 0 and not args.profile:
        sampler.start()
    for _ in range(args.warmup):
        w.device_step()
    sync_all()
    if args.profile:
        copied = os.environ.get("PC_BENCH_PROFILE_COPIED") == "1"  # profile the step WITH the reference's copy (splice kernel)
        if copied:
            for _ in range(3):
                w.device_step(virtual=False)
            torch.cuda.synchronize()
        torch.cuda.profiler.start()
        w.device_step(virtual=False if copied else None)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return
    if rank == 0:
        deadline = time.time() + 2.0  # give the sampler time to deliver its first line
        while not sampler.lines and time.time() < deadline:
            time.sleep(0.02)
    sync_all()
    # more untimed steps after that wait (the GPU may have idled for up to 2 s: one 3 ms step does not bring clocks and
    # power state back): the timed region starts on a GPU that has been busy for ~0.15 s
    for _ in range(max(args.warmup, 48)):
        w.device_step()
    sync_all()
    sampler.mark()
    launches0 = nat.launch_count()
    ms_per_step = w.timed(lambda: w.device_step(True), args.steps, sync_all)
    launches = nat.launch_count() - launches0
    # the same step with the reference's copy (PromptCache.update moves all N rows): the splice kernel's roofline, and
    # what the virtual splice saves
    w.splice_ev = []
    for _ in range(3):
        w.device_step(virtual=False)
    ms_per_step_copied = w.timed(lambda: w.device_step(True, virtual=False), args.steps, sync_all)
    splice_ms = statistics.mean(a.elapsed_time(b) for a, b in w.splice_ev)
    for _ in range(2):
        w.device_step()

    # ---- end-to-end arm: the public API with host inputs (token lists -> device) and the first token read back ---
    for _ in range(args.warmup):
        w.e2e_step()
    e2e_ms = w.timed(w.e2e_step, args.steps, sync_all)
    n_clock_samples = len(sampler.lines)

    # ---- decode after the prefill (informative; the headline metric is TTFT): 33 greedy tokens through the public API
    decode_ms = None
    try:
        from promptcache_b200 import GenerationParameters
        dparams = GenerationParameters(temperature=0.0, max_new_tokens=33, stop_token_ids=[], stop_str=[])
        for _ in range(2):  # first pass warms up (captures the decode graph of this KV buffer), second is reported
            i2, p2, _, cache = w.eng.process(w.prompt)
            outs = list(w.gen.generate(i2, p2, dparams, cache))
        decode_ms = (outs[-1].response_time - outs[0].response_time) / 32.0
    except Exception:
        pass

    times = torch.tensor([ms_per_step, e2e_ms, ms_per_step_copied], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_per_step, e2e_ms, ms_per_step_copied = float(times[0]), float(times[1]), float(times[2])

    # ---- in-step attribution by ablation (rank-local; same graph machinery, kernel families left out) ------------
    ablation = None
    llama_native = model_key.startswith("llama") and w.q_len <= model.linear_max_q and model.linear_impl == "native"
    if not args.no_extras and llama_native and not args.layers:
        try:
            ablation = {}
            for fam in ("attn", "linear", "norm"):
                model.ablate = frozenset([fam])
                for _ in range(3):
                    w.device_step()
                ablation[fam] = w.timed(w.device_step, 10, torch.cuda.synchronize)
            model.ablate = frozenset()
            for _ in range(2):
                w.device_step()
            ablation["full"] = w.timed(w.device_step, 10, torch.cuda.synchronize)
        except Exception as ex:
            ablation = {"error": str(ex)}
        finally:
            model.ablate = frozenset()

    c5 = None
    if not args.no_extras and model_key == "llama2-7b" and not args.layers:
        try:
            c5 = c5_block(lm, dev, world, rank)
        except Exception as ex:
            c5 = {"error": f"{type(ex).__name__}: {ex}"}

    if rank == 0:
        clocks = sampler.stop(upto=n_clock_samples)
        peak, peak_kind, tflops_peak = load_peaks()
        L, Hkv, D = lm.get_cache_shape()
        H = model.n_heads
        splice_bytes = 8.0 * L * Hkv * case.n_cached * D  # read + write of K and V, fp16
        attn_bytes = L * (4.0 * Hkv * (case.n_cached + w.q_len) * D + 4.0 * H * w.q_len * D)
        wbytes = weight_bytes(md, model_key)
        step_bytes = (0.0 if w.virtual else splice_bytes) + attn_bytes + wbytes
        sp_ach = splice_bytes / (splice_ms * 1e-3) / 1e9
        line = {"metric": metric_name(args), "value": world * tokens_per_step / (ms_per_step * 1e-3), "unit": "tok/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "ttft_ms": ms_per_step,
                "computed_tok_s": world * w.q_len / (ms_per_step * 1e-3),
                "virtual_splice": bool(w.virtual), "ms_per_step_with_copied_splice": ms_per_step_copied,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": config_dict(args, case),
                "e2e": {"value": world * tokens_per_step / (e2e_ms * 1e-3), "unit": "tok/s", "ttft_ms": e2e_ms,
                        "computed_tok_s": world * w.q_len / (e2e_ms * 1e-3),
                        "h2d_bytes_per_step": 2 * 8 * w.q_len, "d2h_bytes_per_step": 8,
                        "note": "CacheEngine.process + GenerationEngine.generate(max_new_tokens=1): token/position id lists go "
                                "host->device, the greedy token comes back; cached segments are HBM-resident by design"},
                "gpu_launches": int(launches), "decode_ms_per_token": decode_ms,
                "roofline_step": {"bound": "hbm", "achieved": step_bytes / (ms_per_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                  "frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak, "algorithmic_bytes_per_step": step_bytes,
                                  "parts": {"weights": wbytes, "splice_read_write": 0.0 if w.virtual else splice_bytes,
                                            "attention_kv_q_o": attn_bytes},
                                  "peak_kind": peak_kind + " (copy, read+write)",
                                  "note": "whole step: every weight matrix once + K/V/Q/O of attention (+ splice read/write when the "
                                          "cached rows are copied; with the virtual splice attention reads the segment arena in place), over ms_per_step"},
                "roofline_splice": {"kernel": "splice_kernel (pc_splice_kv)", "bound": "hbm", "achieved": sp_ach, "peak": peak,
                                    "unit": "GB/s", "frac": sp_ach / peak, "traffic": load_traffic("splice_kernel", args.config),
                                    "algorithmic_bytes_per_launch": splice_bytes, "avg_launch_ms": splice_ms,
                                    "share_of_step": splice_ms / ms_per_step_copied,
                                    "timed": "CUDA events around every launch of a second timed region that runs the step with the "
                                             "reference's copy (virtual splice off); the engine's own path launches no splice"},
                "clocks": clocks}
        if world > 1:
            line["segment_store_broadcast"] = w.broadcast
        if ablation and "error" not in ablation:
            full = ablation["full"]
            n_lin = 4 * L + 1  # qkv, o, gate/up, down per layer + lm_head
            lin_ms = max(full - ablation["linear"], 1e-6)
            att_ms = max(full - ablation["attn"], 1e-6)
            lin_ach = wbytes / (lin_ms * 1e-3) / 1e9
            att_ach = attn_bytes / (att_ms * 1e-3) / 1e9
            line["roofline"] = {"kernel": "linear_small_kernel (pc_linear_small: qkv+RoPE+append, o_proj, gate/up+SiLU, down_proj, lm_head) -- "
                                          "the kernel that owns the step", "bound": "hbm", "achieved": lin_ach, "peak": peak,
                                "unit": "GB/s", "frac": lin_ach / peak, "traffic": load_traffic("linear_small_kernel", args.config),
                                "peak_kind": peak_kind + " (copy, read+write)", "launches_per_step": n_lin,
                                "algorithmic_bytes_per_launch": wbytes / n_lin, "avg_launch_ms": lin_ms / n_lin,
                                "in_step_ms": lin_ms, "share_of_step": lin_ms / full,
                                "timed": "in the step: (full step) - (the same CUDA-graph step with the linear launches left out), "
                                         "CUDA events over 10 steps each; includes the launches' programmatic overlap with their neighbours"}
            line["roofline_attention"] = {"kernel": "attn_small_kernel (pc_prefill_attn)", "bound": "hbm", "achieved": att_ach, "peak": peak,
                                          "unit": "GB/s", "frac": att_ach / peak, "traffic": load_traffic("attn_small_kernel", args.config),
                                          "algorithmic_bytes_per_launch": attn_bytes / L, "avg_launch_ms": att_ms / L, "in_step_ms": att_ms,
                                          "share_of_step": att_ms / full, "timed": "in the step, by ablation (see roofline.timed)"}
            line["step_attribution_ms"] = {"full_step": full, "linears": lin_ms, "attention": att_ms, "norms": full - ablation["norm"],
                                           "splice": 0.0 if w.virtual else splice_ms, "method": "T(full) - T(step without the family); families overlap "
                                           "through PDL, so the parts need not add up to the step"}
        else:
            line["roofline"] = dict(line["roofline_splice"])
            if ablation:
                line["ablation_error"] = ablation["error"]
        if not args.no_extras:
            try:
                alone = attention_point(nat, dev, H, Hkv, D, w.q_len, case.n_cached, peak, tflops_peak,
                                        rounding=getattr(model, "rounding", None))
                line.setdefault("roofline_attention", {})["alone"] = alone
                line["roofline_attention_tensor"] = dict(attention_point(nat, dev, 32, 32, 128, 1024, 8192, peak, tflops_peak, launches=8),
                                                         kernel="attn_pp_kernel (pc_prefill_attn, q=1024 over N=8192)", peak=tflops_peak,
                                                         unit="TFLOP/s")
                line["suffix_sweep"] = suffix_sweep(nat, dev, peak, tflops_peak)
            except Exception as ex:
                line["suffix_sweep"] = {"error": str(ex)}
        if c5 is not None:
            line["c5"] = c5
        if args.layers:
            line["invalid"] = f"debug run with {args.layers} layers"
    if world == 1 and rank == 0 and not args.no_extras and args.config == "C2" and not args.layers:
        try:
            del w
            torch.cuda.empty_cache()
            line["c4"] = family_block("falcon-7b", "C4", dev, max(5, args.steps // 2), 3)
        except Exception as ex:
            line["c4"] = {"error": f"{type(ex).__name__}: {ex}"}
        try:
            line["mpt"] = family_block("mpt-7b", "C2", dev, max(5, args.steps // 2), 3)
        except Exception as ex:
            line["mpt"] = {"error": f"{type(ex).__name__}: {ex}"}
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        try:
            ref = make_cpu_reference(args, case, md, dims, seg_lens, threads, synthetic_segments=True)
            ref.step()
            r = min((ref.step() for _ in range(3)), key=lambda d: d["ttft_s"])
            line["cpu_baseline"] = {"value": tokens_per_step / r["ttft_s"], "unit": "tok/s", "cores": threads, "kind": ref.kind,
                                    "ttft_ms": r["ttft_s"] * 1e3, "cache_ms": r["cache_ms"],
                                    "sample": "best of 3 after 1 warm-up; " + ref.describe()}
        except Exception as ex:  # never lose the GPU line to a host-side OOM
            line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": threads, "kind": "unavailable", "sample": f"failed: {type(ex).__name__}: {ex}"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
