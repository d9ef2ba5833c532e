"""Tevilix: a decoder-only model whose layers run their mixer and their feed-forward SIDE BY SIDE on the same stream, with a
span of layers that may run several times in a row on the same weights.

    embedding     token row times a scale                                                              (`pcs_embed`)
    every layer   x += mixer(ln(x, w1)) + ff(ln(x, w2)): two layer norms (weight, no bias) of the SAME x; the sum of all branch
                  results and both norms of the next layer are one launch                               (`pcs_add_layer_norm`)
    loop          layers [start, stop) run `times` times in a row; every RUN of a layer owns a state in the slot pool
    parallel      two mixers on the same input, added with two constants:
                  left   attention over grouped heads with biased projections, an RMS norm per query / key head (one weight
                         vector for all heads), a rotate-half turn of the leading coordinates with all frequencies divided by a
                         constant (`pcs_rope_kv_prep`), scores MIXED ACROSS HEADS by an [H, H] matrix before the softmax, a
                         sliding window, and an element-wise sigmoid gate on the concatenated heads     (`pcs_attn` with `talk`)
                  right  an element-wise gated recurrence whose gates read only the current token:
                         S_t = (1 - z_t) S_(t-1) + z_t c_t, result S_t * silu(g_t)                       (`pcs_gru_scan`)
    mlstm         the stabilised matrix-memory recurrence with capped gates, per-head unit RMS, a weight over all heads and a
                  sigmoid gate                                                                   (`pcs_mlstm_gates`, `pcs_mlstm_scan`)
    feed-forward  dense: W_down gelu(W_up h) with the exact (erf) gelu; mixture of experts: router in 32-bit with a sigmoid per
                  expert, choice by score + correction inside the best groups (a group's score: the sum of its two best), weights =
                  the chosen plain scores over their sum times a constant; experts W_down relu(W_up h)^2 without a gate branch
                  (`pcs_moe_route`, `pcs_moe_rows_*` / the library's grouped product, `pcs_glu_mul`, `pcs_moe_combine`)
    output        layer norm of the wanted rows, then the head

K/V rows, matrix memories and the recurrence's vectors live in the slot pool, one set per layer RUN.  Sizes, the order of layers,
the loop and every constant that can differ between models come from config.json; tensors are named l<i>.norm1,
l<i>.mix.left.q, l<i>.mix.right.z, l<i>.mlp.e<j>.up, ... in the checkpoint.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from .. import _native_seq as nsq
from .. import weights as wio
from ._seqbase import SlotPoolCausalLM
from ._state import KVSpec, MatrixMemorySpec, VectorStateSpec

GROUP_BEST = 2          # a group of experts is scored by the sum of this many of its best choice scores
WEIGHT_SUM_EPS = 1e-20  # added to the sum of the chosen scores before the division


def divided_frequencies(dims: int, base: float, factor: float = 1.0) -> List[float]:
    """Angular frequencies of the dims / 2 rotated pairs: base^(-2i/dims), every one divided by `factor` (positions stretched)."""
    return [float(base) ** (-2.0 * i / dims) / float(factor) for i in range(dims // 2)]


def layer_runs(n_layers: int, loop: Optional[dict]) -> List[int]:
    """The layers' indices in the order they run: the span [start, stop) `times` times in a row, then the rest."""
    if not loop:
        return list(range(n_layers))
    a, b, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
    if not (0 <= a <= b <= n_layers) or times < 1:
        raise ValueError(f"loop {loop!r} does not fit {n_layers} layers")
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n_layers))


class TevilixConfig:
    """config.json of the design: {"architecture", "vocab", "width", "embedding": {"scale"}, "norm": {"eps"},
    "loop": {"start", "stop", "times"}, "layers": [{"type": "parallel" | "mlstm", "mixer": {...},
    "mlp": {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale", "groups": {"count", "keep"}}} | null}]}."""

    def __init__(self, d: dict):
        self.raw = d
        self.architecture = d.get("architecture", "Tevilix")
        self.vocab_size = int(d["vocab"])
        self.width = int(d["width"])
        self.embedding_scale = float((d.get("embedding") or {}).get("scale", 1.0))
        self.eps = float(d["norm"]["eps"])
        self.layers = []
        for i, layer in enumerate(d["layers"]):
            kind = layer["type"]
            if kind not in ("parallel", "mlstm"):
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            self.layers.append({"type": kind, "mixer": dict(layer["mixer"]), "mlp": dict(mlp) if mlp is not None else None})
        self.num_hidden_layers = len(self.layers)
        self.loop = dict(d["loop"]) if d.get("loop") else None
        self.runs = layer_runs(len(self.layers), self.loop)

    @classmethod
    def from_dir(cls, path: str) -> "TevilixConfig":
        with open(os.path.join(path, "config.json")) as fh:
            return cls(json.load(fh))


class TevilixForCausalLM(SlotPoolCausalLM):
    def __init__(self, config: TevilixConfig, tensors: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16,
                 max_tokens: Optional[int] = None):
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Tevilix computes in bfloat16 or float32")
        self.config, self.compute_dtype = config, dtype
        self.vocab_size, self.width, self.eps = config.vocab_size, config.width, config.eps
        dev = torch.device(device)

        def get(name, optional=False):
            t = tensors.get(name)
            if t is None:
                if optional:
                    return None
                raise KeyError(f"the checkpoint has no tensor {name!r}")
            return t.to(dev, dtype).contiguous()

        def f32(name, optional=False):
            t = tensors.get(name)
            if t is None:
                if optional:
                    return None
                raise KeyError(f"the checkpoint has no tensor {name!r}")
            return t.to(dev, torch.float32).contiguous()

        def fuse(parts, biases):
            """Rows of several projections of the same input as one matrix; a missing bias is zero."""
            w = torch.cat(parts, 0).contiguous()
            if all(b is None for b in biases):
                return w, None
            b = torch.cat([bb if bb is not None else torch.zeros(p.shape[0], device=dev, dtype=dtype) for p, bb in zip(parts, biases)])
            return w, b.contiguous()

        self.embed, self.head, self.final_norm = get("embed"), get("head"), get("final.norm")
        self.blocks: List[dict] = []
        for i, layer in enumerate(config.layers):
            p, m = f"l{i}.", layer["mixer"]
            blk = {"type": layer["type"], "norm1": get(p + "norm1")}
            if layer["type"] == "mlstm":
                H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
                blk.update(heads=H, dim=D, vdim=V, cap=float(m["gate_cap"]), offs=(0, H * D, 2 * H * D, 2 * H * D + H * V),
                           w_in=torch.cat([get(p + "mix.q"), get(p + "mix.k"), get(p + "mix.v"), get(p + "mix.g")], 0).contiguous(),
                           w_i=get(p + "mix.i"), w_f=get(p + "mix.f"), b_i=f32(p + "mix.i.b"), b_f=f32(p + "mix.f.b"),
                           mix_norm=get(p + "mix.norm"), w_o=get(p + "mix.o"), spec=MatrixMemorySpec(H, D, V))
            else:
                a, q = m["left"], p + "mix.left."
                H, D, V = int(a["heads"]), int(a["dim"]), int(a["vdim"])
                G = int(a.get("kv_heads", H))
                if H % G:
                    raise ValueError(f"layer {i}: {H} heads do not divide into {G} key/value heads")
                rot = a.get("rot") or {}
                rd = int(rot.get("dims", 0))
                if rd % 2 or rd > D:
                    raise ValueError(f"layer {i}: {rd} rotated coordinates do not fit a head of {D}")
                factor = float((rot.get("scaling") or {}).get("factor", 1.0))
                R, r = int(m["right"]["width"]), p + "mix.right."
                parts = [get(q + "q"), get(q + "k"), get(q + "v"), get(q + "g"), get(r + "z"), get(r + "x"), get(r + "g")]
                biases = [get(q + "q.b", True), get(q + "k.b", True), get(q + "v.b", True), None, get(r + "z.b", True), get(r + "x.b", True), None]
                w_in, b_in = fuse(parts, biases)
                o_gate = (H + G) * D + G * V
                talk = f32(q + "talk", True)
                blk.update(heads=H, kv_heads=G, dim=D, vdim=V, scale=float(a.get("scale", D ** -0.5)), window=int((a.get("mask") or {}).get("size", 0)),
                           rot_dims=rd, freqs=torch.tensor(divided_frequencies(rd, float(rot.get("base", 10000.0)), factor), dtype=torch.float64, device=dev) if rd else None,
                           q_norm=get(q + "q.norm", True), k_norm=get(q + "k.norm", True),
                           talk=talk if talk is not None else torch.eye(H, dtype=torch.float32, device=dev),
                           w_in=w_in, b_in=b_in, offs=(0, H * D, (H + G) * D), gate_off=o_gate, gru_offs=(o_gate + H * V, o_gate + H * V + R, o_gate + H * V + 2 * R),
                           gru_width=R, w_o=get(q + "o"), b_o=get(q + "o.b", True), w_ro=get(r + "o"),
                           left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)),
                           spec=(KVSpec(G, D, V), VectorStateSpec(R)))
            f = layer["mlp"]
            blk["mlp"] = None if f is None else f["kind"]
            if f is not None:
                blk["norm2"] = get(p + "norm2")
                if f["kind"] == "dense":
                    blk.update(w_up=get(p + "mlp.up"), w_down=get(p + "mlp.down"))
                    blk["ff"] = blk["w_up"].shape[0]
                else:
                    rt = f["router"]
                    E, groups = int(rt["experts"]), rt.get("groups") or {}
                    blk.update(n_experts=E, top=int(rt["top"]), n_groups=int(groups.get("count", 1)), keep_groups=int(groups.get("keep", groups.get("count", 1))),
                               route_scale=float(rt.get("scale", 1.0)), w_router=get(p + "mlp.router"), correction=f32(p + "mlp.correction", True),
                               we_up=torch.stack([get(f"{p}mlp.e{e}.up") for e in range(E)]).contiguous(),
                               we_down=torch.stack([get(f"{p}mlp.e{e}.down") for e in range(E)]).contiguous())
            self.blocks.append(blk)
        self.runs = list(config.runs)
        # bfloat16 products accumulate in 32-bit all the way (no reduced-precision split-K sums); float32 stays true float32
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.attn_impl = 0
        self.scan_impl = 0
        self.moe_grouped = None   # None: by size; False / "library" force the row kernels or the library's grouped product
        self._init_runtime(dev, max_tokens)

    def state_specs(self):
        """One state per layer RUN: a layer inside the loop keeps as many as it has passes."""
        return [self.blocks[i]["spec"] for i in self.runs]

    @classmethod
    def from_pretrained(cls, path: str, device="cuda", dtype=torch.bfloat16, max_tokens: Optional[int] = None, **_):
        """`path`: a folder with config.json and model.safetensors."""
        cfg = TevilixConfig.from_dir(path)
        tensors = wio.load_file(os.path.join(path, "model.safetensors"), device=device)
        return cls(cfg, tensors, device=device, dtype=dtype, max_tokens=max_tokens)

    # ---- the mixers: each returns the branch results with their multipliers ------------------------------------------
    def _mlstm(self, h, blk, st, batch):
        T, dt, dev = h.shape[0], self.compute_dtype, self._device
        H, V = blk["heads"], blk["vdim"]
        proj = nsq.linear(h, blk["w_in"])
        ig = torch.empty(T, H, dtype=torch.float32, device=dev)
        fg = torch.empty(T, H, dtype=torch.float32, device=dev)
        nsq.mlstm_gates(h, blk["w_i"], blk["w_f"], blk["b_i"], blk["b_f"], ig, fg, blk["cap"])
        mixed = torch.empty(T, H * V, dtype=dt, device=dev)
        nsq.mlstm_scan(proj, blk["offs"], ig, fg, blk["mix_norm"], mixed, st["s"], st["n"], st["m"], self.eps, batch, impl=self.scan_impl)
        return [(nsq.linear(mixed, blk["w_o"]), 1.0)]

    def _parallel(self, h, blk, st, batch):
        T, dt, dev = h.shape[0], self.compute_dtype, self._device
        H, G, D, V, R = blk["heads"], blk["kv_heads"], blk["dim"], blk["vdim"], blk["gru_width"]
        proj = nsq.linear(h, blk["w_in"], blk["b_in"])     # q | k | v | output gate | z | x | g of the recurrence
        q = torch.empty(T, H * D, dtype=dt, device=dev)
        nsq.rope_kv_prep(proj, blk["offs"], H, G, D, V, blk["freqs"], blk["rot_dims"], False, False, self.eps, q, st["k"], st["v"], batch,
                         q_norm_w=blk["q_norm"], k_norm_w=blk["k_norm"])
        mixed = torch.empty(T, H * V, dtype=dt, device=dev)
        # few tokens (decoding): the visible keys are split over more blocks; the bound is the window or the pool's capacity, so
        # that a replayed graph stays valid while the sequences grow
        seen = min(self.pool.cap, blk["window"]) if blk["window"] > 0 else self.pool.cap
        ws = nsq.attn_workspace(T, H, V, dev) if T <= 16 else None
        nsq.attention(q, st["k"], st["v"], mixed, H, blk["scale"], None, None, False, batch, impl=self.attn_impl, max_keys=seen, workspace=ws,
                      window=blk["window"], talk=blk["talk"], out_gate=proj[:, blk["gate_off"]:blk["gate_off"] + H * V])
        left = nsq.linear(mixed, blk["w_o"], blk["b_o"])
        gated = torch.empty(T, R, dtype=dt, device=dev)
        nsq.gru_scan(proj, blk["gru_offs"], R, gated, st["vec"], batch)
        right = nsq.linear(gated, blk["w_ro"])
        return [(left, blk["left_scale"]), (right, blk["right_scale"])]

    def _feed_forward(self, h, blk):
        if blk["mlp"] == "dense":
            a = nsq.glu_mul(nsq.linear(h, blk["w_up"]), blk["ff"], (nsq.ACT_GELU_ERF, 0.0, 0.0))
            return nsq.linear(a, blk["w_down"])
        idx, wgt, _ = nsq.moe_route(h, blk["w_router"], blk["correction"], None, blk["top"], blk["n_groups"], blk["keep_groups"], renorm=True,
                                    score_fn=nsq.ROUTE_SIGMOID, group_best=GROUP_BEST, wgt_scale=blk["route_scale"], renorm_eps=WEIGHT_SUM_EPS)
        mode = self.moe_grouped
        if mode is None and torch.cuda.is_current_stream_capturing():
            mode = False   # a recorded decoding step keeps to this library's own kernels
        ye, rows_e = nsq.moe_experts(h, idx, blk["we_up"], blk["we_down"], grouped=mode, act=(nsq.ACT_RELU2, 0.0, 0.0))
        y = torch.empty(h.shape[0], self.width, dtype=torch.float32, device=self._device)
        nsq.moe_combine(y, ye, idx, wgt, h, blk["n_experts"], 1.0, y_row=rows_e, overwrite=True)
        return y

    # ---- the layers over one batch ------------------------------------------------------------------------------
    def _layers(self, ids: torch.Tensor, batch, rows: Optional[torch.Tensor]) -> torch.Tensor:
        T, W, dt, dev, eps = ids.shape[0], self.width, self.compute_dtype, self._device, self.eps
        x = torch.empty(T, W, dtype=torch.float32, device=dev)     # the residual stream, 32-bit, updated in place
        h1 = torch.empty(T, W, dtype=dt, device=dev)               # the mixer's input of the next layer run
        h2 = torch.empty(T, W, dtype=dt, device=dev)               # its feed-forward's input
        nsq.embed(self.embed, ids, x, self.config.embedding_scale)
        if self.runs:
            first = self.blocks[self.runs[0]]
            nsq.add_layer_norm(x, [], eps, first["norm1"], h1, first.get("norm2"), h2)
        for r, li in enumerate(self.runs):
            blk, st = self.blocks[li], self.pool.layers[r]
            ys = self._mlstm(h1, blk, st, batch) if blk["type"] == "mlstm" else self._parallel(h1, blk, st, batch)
            if blk["mlp"]:
                ys.append((self._feed_forward(h2, blk), 1.0))
            nxt = self.blocks[self.runs[r + 1]] if r + 1 < len(self.runs) else None
            # the sum of all branches and both input norms of the next run in one launch
            nsq.add_layer_norm(x, ys, eps, nxt["norm1"] if nxt else None, h1, nxt.get("norm2") if nxt else None, h2)
            if self.layer_trace is not None:
                self.layer_trace.append(x.clone())
        if rows is None or rows.numel() == 0:
            return torch.zeros(0, self.vocab_size, dtype=torch.float32, device=dev)
        hw = torch.empty(rows.numel(), W, dtype=dt, device=dev)
        nsq.add_layer_norm(x, [], eps, self.final_norm, hw, rows=rows)     # only the wanted rows go on
        return nsq.linear(hw, self.head).float()
