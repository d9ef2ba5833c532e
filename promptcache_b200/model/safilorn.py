"""Safilorn: a decoder-only model that interleaves low-rank (latent) attention layers with gated linear-attention layers,
dense and mixture-of-experts feed-forwards, and a depth-weighted average of all earlier layers' results.

    embedding     token row times a scale                                                            (`pcs_embed`)
    every layer   x += n(mixer(n(x, w1)), w1b);  x += n(ff(n(x, w2)), w2b)   with n(x, w) = rms(x) * (1 + w): weights are stored
                  around zero and the 1 is added in 32-bit                                           (`pcs_gate_norm_add`)
    depth average with X_0 the embedding output and X_(i+1) the result of layer i, layer i hands on sum_j a_i[j] X_j; every X_j of
                  the step is kept, and the sum is fused with the next layer's input norm             (`pcs_depth_mix`)
    latent_attention   queries through a normed low-rank latent; keys and values of all heads are functions of one normed latent
                  per token plus one rotated key part shared by the heads, and only those are cached (`pcs_latent_prep`).  The
                  rotated parts use the rotate-half pairing with frequencies rescaled over a ramp of wavelengths and a common
                  multiplier on cos and sin.  Prompts expand per-head keys and values of the context into a dense pool of the
                  step and run multi-head attention over it; decoding carries the query into the latent space and attends over
                  the cached rows directly (`pcs_latent_q`, `pcs_latent_expand`, `pcs_attn`).  The softmax denominator holds a
                  learned per-head sink term; a per-head sigmoid gate scales the result                (`pcs_head_gate`).
    gla           S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with a decay per key channel,
                  alpha = sigmoid(A2 A1 h + b)^(1/tau); per-head RMS norm, silu gate                 (`pcs_gla_decay`, `pcs_gla_scan`)
    feed-forward  dense: W_down(silu(W_gate h + b) * (W_up h + b)) + b; mixture of experts: router logits with a bias in
                  32-bit, the `top` largest chosen, weights = softmax over the chosen alone; experts with a clamped gate and
                  up branch, g * sigmoid(1.702 g) * (u + 1)                   (`pcs_moe_route`, `pcs_moe_rows_*` / grouped products)

The latent rows and the recurrent states live in the slot pool; sizes, the order of layers and every constant that can differ
between models come from config.json; tensors are named l<i>.norm1, l<i>.mix.dq, l<i>.mlp.e<j>.gate, ... in the checkpoint.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

from .. import _native_seq as nsq
from .. import weights as wio
from ._seqbase import SlotPoolCausalLM
from ._state import DecayStateSpec, LatentKVSpec

SWISH_ALPHA = 1.702        # the experts' gate activation g * sigmoid(SWISH_ALPHA * g)
ATTENTION_FACTOR_COEF = 0.1  # cos and sin are multiplied by ATTENTION_FACTOR_COEF * ln(factor) + 1 when frequencies are rescaled
NORM_WEIGHT_OFFSET = 1.0   # the layers' norm weights are stored around zero


def ramp_scaled_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(angular frequencies of the dims / 2 rotated pairs, multiplier of cos and sin).  Pair i has f_i = base^(-2i/dims).  With
    `scaling` {factor, original, fast, slow}: pair(t) = dims * ln(original / (2 pi t)) / (2 ln base) is the (fractional) pair that
    makes t turns over `original` positions; pairs up to lo = floor(pair(fast)) keep f_i, pairs from hi = ceil(pair(slow)) get
    f_i / factor, and a linear ramp lies between."""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(pair(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, ATTENTION_FACTOR_COEF * math.log(factor) + 1.0


class SafilornConfig:
    """config.json of the design: {"architecture", "vocab", "width", "embedding": {"scale"}, "norm": {"eps"},
    "layers": [{"type": "latent_attention" | "gla", "mixer": {...}, "mlp": {"kind": "dense", "ff"} |
    {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}} | null}]}."""

    def __init__(self, d: dict):
        self.raw = d
        self.architecture = d.get("architecture", "Safilorn")
        self.vocab_size = int(d["vocab"])
        self.width = int(d["width"])
        self.embedding_scale = float((d.get("embedding") or {}).get("scale", 1.0))
        self.eps = float(d["norm"]["eps"])
        self.layers = []
        for i, layer in enumerate(d["layers"]):
            kind = layer["type"]
            if kind not in ("latent_attention", "gla"):
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            self.layers.append({"type": kind, "mixer": dict(layer["mixer"]), "mlp": dict(mlp) if mlp is not None else None})
        self.num_hidden_layers = len(self.layers)

    @classmethod
    def from_dir(cls, path: str) -> "SafilornConfig":
        with open(os.path.join(path, "config.json")) as fh:
            return cls(json.load(fh))


class SafilornForCausalLM(SlotPoolCausalLM):
    def __init__(self, config: SafilornConfig, tensors: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16,
                 max_tokens: Optional[int] = None):
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Safilorn computes in bfloat16 or float32")
        self.config, self.compute_dtype = config, dtype
        self.vocab_size, self.width, self.eps = config.vocab_size, config.width, config.eps
        dev = torch.device(device)
        L = len(config.layers)

        def get(name):
            t = tensors.get(name)
            if t is None:
                raise KeyError(f"the checkpoint has no tensor {name!r}")
            return t.to(dev, dtype).contiguous()

        def f32(name):
            if name not in tensors:
                raise KeyError(f"the checkpoint has no tensor {name!r}")
            return tensors[name].to(dev, torch.float32).contiguous()

        self.embed, self.head, self.final_norm = get("embed"), get("head"), get("final.norm")
        self.blocks: List[dict] = []
        for i, layer in enumerate(config.layers):
            p, m = f"l{i}.", layer["mixer"]
            blk = {"type": layer["type"], "norm1": get(p + "norm1"), "norm1b": get(p + "norm1b"), "depth": f32(p + "dwa").reshape(-1)}
            if blk["depth"].numel() != i + 2:
                raise ValueError(f"layer {i}: the depth average needs {i + 2} coefficients, the checkpoint has {blk['depth'].numel()}")
            if layer["type"] == "latent_attention":
                H, D, R, V, C = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
                rot = m.get("rot") or {}
                if R and int(rot.get("dims", R)) != R:
                    raise ValueError(f"layer {i}: the rotation covers {rot.get('dims')} dimensions, the rotated part has {R}")
                dq, dkv = get(p + "mix.dq"), get(p + "mix.dkv")
                Q = dq.shape[0]
                if dkv.shape[0] != C + R:
                    raise ValueError(f"layer {i}: the key/value down-projection has {dkv.shape[0]} rows, not kv_rank + rot_dim = {C + R}")
                freqs, mult = ramp_scaled_frequencies(R, float(rot.get("base", 10000.0)), rot.get("scaling")) if R else ([], 1.0)
                uk, uv = get(p + "mix.uk"), get(p + "mix.uv")
                blk.update(heads=H, dim=D, rot_dim=R, vdim=V, kv_rank=C, q_rank=Q, scale=float(m["scale"]), rot_mult=float(mult),
                           freqs=torch.tensor(freqs, dtype=torch.float64, device=dev) if R else None,
                           # one product of the mixer's input: query latent, key/value latent with the rotated part, head gates
                           w_in=torch.cat([dq, dkv, get(p + "mix.g")], 0).contiguous(), offs=(0, Q, Q + C + R),
                           cq_norm=get(p + "mix.dq.norm"), ckv_norm=get(p + "mix.dkv.norm"), w_uq=get(p + "mix.uq"),
                           w_ukv=torch.cat([uk, uv], 0).contiguous(),             # latents -> plain key parts of all heads, then values
                           uk_h=uk.view(H, D, C).contiguous(),                    # per head: carries a query into the latent space
                           uv_t=uv.view(H, V, C).transpose(1, 2).contiguous(),    # per head [C, V]: carries a latent result back
                           sink=f32(p + "mix.sink").reshape(-1), w_o=get(p + "mix.o"), spec=LatentKVSpec(C, R),
                           # the latent form's result per head is kv_rank wide: beyond what the decoding kernels hold, only the expanded form runs
                           latent_ok=C <= nsq.ATTN_MAX_VDIM)
            else:
                H, D, V = (int(m[k]) for k in ("heads", "dim", "vdim"))
                a1 = get(p + "mix.a1")
                r = a1.shape[0]
                blk.update(heads=H, dim=D, vdim=V, tau=float(m["tau"]), rank=r,
                           w_in=torch.cat([get(p + "mix.q"), get(p + "mix.k"), get(p + "mix.v"), get(p + "mix.g"), a1], 0).contiguous(),
                           offs=(0, H * D, 2 * H * D, 2 * H * D + H * V), a_off=2 * H * D + 2 * H * V,
                           w_a2=get(p + "mix.a2"), b_a2=f32(p + "mix.a2.b"), mix_norm=get(p + "mix.norm"), w_o=get(p + "mix.o"),
                           spec=DecayStateSpec(H, D, V))
            f = layer["mlp"]
            blk["mlp"] = None if f is None else f["kind"]
            if f is not None:
                blk.update(norm2=get(p + "norm2"), norm2b=get(p + "norm2b"))
                if f["kind"] == "dense":
                    blk.update(ff=int(f["ff"]), w_gu=torch.cat([get(p + "mlp.gate"), get(p + "mlp.up")], 0).contiguous(),
                               b_gu=torch.cat([get(p + "mlp.gate.b"), get(p + "mlp.up.b")]).contiguous(), w_down=get(p + "mlp.down"),
                               b_down=get(p + "mlp.down.b"))
                else:
                    E, top = int(f["router"]["experts"]), int(f["router"]["top"])
                    blk.update(n_experts=E, top=top, act=(nsq.GLU_CLAMPED_SWISH, SWISH_ALPHA, float(f["expert"]["limit"])),
                               w_router=get(p + "mlp.router"), b_router=f32(p + "mlp.router.b"),
                               we_gu=torch.stack([torch.cat([get(f"{p}mlp.e{e}.gate"), get(f"{p}mlp.e{e}.up")], 0) for e in range(E)]).contiguous(),
                               we_down=torch.stack([get(f"{p}mlp.e{e}.down") for e in range(E)]).contiguous())
            self.blocks.append(blk)
        self._one = torch.ones(1, dtype=torch.float32, device=dev)
        # bfloat16 products accumulate in 32-bit all the way (no reduced-precision split-K sums); float32 stays true float32
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.attn_impl = 0
        self.scan_impl = 0
        self.moe_grouped = None      # None: by size; False / "library" / "own" force the row kernels or one of the grouped products
        self.latent_form = None      # None: by step (prompts expanded, decoding in the latent space); "expanded" / "latent" force one
        self.expand_min_len = 16     # steps whose longest entry brings at least this many tokens attend over expanded keys
        self._init_runtime(dev, max_tokens)
        if not all(b.get("latent_ok", True) for b in self.blocks):
            self.use_cuda_graphs = False   # the expanded form describes the step's context on the host: it is not recorded

    def state_specs(self):
        return [b["spec"] for b in self.blocks]

    @classmethod
    def from_pretrained(cls, path: str, device="cuda", dtype=torch.bfloat16, max_tokens: Optional[int] = None, **_):
        """`path`: a folder with config.json and model.safetensors."""
        cfg = SafilornConfig.from_dir(path)
        tensors = wio.load_file(os.path.join(path, "model.safetensors"), device=device)
        return cls(cfg, tensors, device=device, dtype=dtype, max_tokens=max_tokens)

    # ---- the mixers ---------------------------------------------------------------------------------------------
    def _context(self, batch, step):
        """The step's context tokens (every entry's rows from its first one) as a batch description, and the entries' indices as
        the dense pool's slots; built once per step, on the first latent-attention layer that expands."""
        if "ctx" not in step:
            if all(p0 == 0 for p0 in batch.pos0):
                step["ctx"] = batch
            else:
                step["ctx"] = nsq.Batch(batch.slots, [0] * batch.n_seqs, [p0 + n for p0, n in zip(batch.pos0, batch.lens)], self._device)
            step["ids"] = torch.arange(batch.n_seqs, dtype=torch.int32, device=self._device)
        return step["ctx"], step["ids"]

    def _latent_attention(self, h, blk, pool, batch, step):
        T, dt, dev = h.shape[0], self.compute_dtype, self._device
        H, D, R, V, C, Q = blk["heads"], blk["dim"], blk["rot_dim"], blk["vdim"], blk["kv_rank"], blk["q_rank"]
        proj = nsq.linear(h, blk["w_in"])
        cq = torch.empty(T, Q, dtype=dt, device=dev)
        nsq.latent_prep(proj, blk["offs"][0], blk["offs"][1], Q, C, R, blk["cq_norm"], blk["ckv_norm"], self.eps, blk["freqs"], blk["rot_mult"], cq,
                        pool["ckv"], batch)
        q = nsq.linear(cq, blk["w_uq"])                      # [T, H * (D + R)], per head [plain | rotated]
        # a recorded decoding step reads everything that changes from device buffers: only the latent form does
        form = "latent" if torch.cuda.is_current_stream_capturing() else (self.latent_form or ("expanded" if batch.max_len >= self.expand_min_len else "latent"))
        if not blk["latent_ok"]:
            form = "expanded"
        if form == "expanded":
            ctx, ids = self._context(batch, step)
            c_ctx = nsq.latent_gather(pool["ckv"], C, ctx)
            kv = nsq.linear(c_ctx, blk["w_ukv"])             # [N, H * D + H * V]
            cap = ((max(p0 + n for p0, n in zip(batch.pos0, batch.lens)) + 63) // 64) * 64
            kd = torch.empty(batch.n_seqs, H, cap, D + R, dtype=dt, device=dev)
            vd = torch.empty(batch.n_seqs, H, cap, V, dtype=dt, device=dev)
            nsq.latent_expand(kv, pool["ckv"], C, R, H, D, V, kd, vd, ctx)
            nsq.latent_q(q, H, D, R, blk["freqs"], blk["rot_mult"], batch)
            o = torch.empty(T, H * V, dtype=dt, device=dev)
            nsq.attention(q, kd, vd, o, H, blk["scale"], None, None, True, batch, impl=self.attn_impl, sink_logit=blk["sink"], pool_slot=ids)
            o3 = o.view(T, H, V)
        else:
            # q'_h = U_k,h^T q_h: [H, T, D] x [H, D, C]; the rotated parts ride along unchanged
            q_lat = torch.bmm(q.view(T, H, D + R)[:, :, :D].transpose(0, 1), blk["uk_h"]).transpose(0, 1)   # [T, H, C]
            ql = nsq.latent_q(q, H, D, R, blk["freqs"], blk["rot_mult"], batch, q_lat=q_lat)
            o_lat = torch.empty(T, H * C, dtype=dt, device=dev)
            ws = nsq.attn_workspace(T, H, C, dev) if T <= 32 else None
            nsq.attention(ql, pool["ckv"], pool["ckv"], o_lat, H, blk["scale"], None, None, True, batch, impl=self.attn_impl, max_keys=self.pool.cap,
                          workspace=ws, sink_logit=blk["sink"], v_row_stride=C + R)
            o3 = torch.bmm(o_lat.view(T, H, C).transpose(0, 1), blk["uv_t"]).transpose(0, 1)                  # [T, H, V]
        mixed = torch.empty(T, H * V, dtype=dt, device=dev)
        nsq.head_gate(o3, proj[:, blk["offs"][2]:blk["offs"][2] + H], mixed)
        return nsq.linear(mixed, blk["w_o"])

    def _gla(self, h, blk, pool, batch):
        T, dt, dev = h.shape[0], self.compute_dtype, self._device
        H, V = blk["heads"], blk["vdim"]
        proj = nsq.linear(h, blk["w_in"])
        ld = nsq.gla_decay(proj[:, blk["a_off"]:blk["a_off"] + blk["rank"]], blk["w_a2"], blk["b_a2"], blk["tau"])
        mixed = torch.empty(T, H * V, dtype=dt, device=dev)
        nsq.gla_scan(proj, blk["offs"], ld, blk["mix_norm"], mixed, pool["s"], self.eps, batch, impl=self.scan_impl)
        return nsq.linear(mixed, blk["w_o"])

    def _moe(self, h, blk):
        T, W, dev = h.shape[0], self.width, self._device
        idx, wgt, _ = nsq.moe_route(h, blk["w_router"], None, None, blk["top"], bias=blk["b_router"], renorm=True)
        mode = self.moe_grouped
        if mode is None and torch.cuda.is_current_stream_capturing():
            # a recorded decoding step keeps to this library's own kernels: the row kernels, or the grouped one where many pairs fit it
            fits = self.compute_dtype == torch.bfloat16 and W % 8 == 0 and blk["we_down"].shape[2] % 8 == 0
            mode = "own" if (T * blk["top"] > 256 and fits) else False
        ye, rows_e = nsq.moe_experts(h, idx, blk["we_gu"], blk["we_down"], grouped=mode, act=blk["act"])
        y = torch.empty(T, W, dtype=torch.float32, device=dev)
        nsq.moe_combine(y, ye, idx, wgt, h, blk["n_experts"], 1.0, y_row=rows_e, overwrite=True)
        return y

    # ---- the layers over one batch ------------------------------------------------------------------------------
    def _layers(self, ids: torch.Tensor, batch, rows: Optional[torch.Tensor]) -> torch.Tensor:
        T, W, dt, dev, eps, off = ids.shape[0], self.width, self.compute_dtype, self._device, self.eps, NORM_WEIGHT_OFFSET
        L = len(self.blocks)
        # xs[0]: the embedding output; xs[i + 1]: layer i's input, updated in place into its result; all are kept for the depth average
        xs = torch.empty(L + 1, T, W, dtype=torch.float32, device=dev)
        h = torch.empty(T, W, dtype=dt, device=dev)
        step: dict = {}
        nsq.embed(self.embed, ids, xs[0], self.config.embedding_scale)
        if L:
            nsq.depth_mix(xs, 1, self._one, eps, x_out=xs[1], next_w=self.blocks[0]["norm1"], h_out=h, w_offset=off)
        for i, blk in enumerate(self.blocks):
            x, pool = xs[i + 1], self.pool.layers[i]
            y = self._latent_attention(h, blk, pool, batch, step) if blk["type"] == "latent_attention" else self._gla(h, blk, pool, batch)
            kind = blk["mlp"]
            # the layer's last residual sum rides in the depth average's launch (all rows, each once); the last layer's stays a launch of
            # its own because the final average runs on the wanted rows only
            fuse = i + 1 < L
            last_w = blk["norm2b"] if kind else blk["norm1b"]
            if kind:
                nsq.gate_norm_add(x, y, None, blk["norm1b"], None, eps, blk["norm2"], h, w_offset=off)
                if kind == "dense":
                    gu = nsq.linear(h, blk["w_gu"], blk["b_gu"])
                    y = nsq.linear(nsq.glu_mul(gu, blk["ff"]), blk["w_down"], blk["b_down"])
                else:
                    y = self._moe(h, blk)
            if fuse:
                nsq.depth_mix(xs, i + 2, blk["depth"], eps, x_out=xs[i + 2], next_w=self.blocks[i + 1]["norm1"], h_out=h, w_offset=off, y=y, y_w=last_w)
            else:
                nsq.gate_norm_add(x, y, None, last_w, None, eps, w_offset=off)
            if fuse:
                if self.layer_trace is not None:
                    self.layer_trace.append(xs[i + 2].clone())
        if self.layer_trace is not None and L:
            last = torch.empty(T, W, dtype=torch.float32, device=dev)
            nsq.depth_mix(xs, L + 1, self.blocks[-1]["depth"], eps, x_out=last)
            self.layer_trace.append(last)
        if rows is None or rows.numel() == 0:
            return torch.zeros(0, self.vocab_size, dtype=torch.float32, device=dev)
        hw = torch.empty(rows.numel(), W, dtype=dt, device=dev)
        coef = self.blocks[-1]["depth"] if L else self._one
        nsq.depth_mix(xs, L + 1, coef, eps, next_w=self.final_norm, h_out=hw, w_offset=off, rows=rows)   # only the wanted rows go on
        return nsq.linear(hw, self.head).float()
