"""Slot pool: the per-sequence memory of models whose layers keep different kinds of state.

The prompt-cache models keep one kind of state, K/V rows of one width, in a `KVBuffer` per sequence (`_kv.py`).  A model
that mixes attention layers (K/V rows whose key and value widths differ) with recurrent layers (a fixed-size state that is
carried from token to token) keeps its sequences in a `SlotPool` instead: every live sequence owns one SLOT, and each
layer has pool tensors whose first dimension is the slot,

    attention layer   K [slots, Hkv, cap, dim]   V [slots, Hkv, cap, vdim]        (compute type)
    low-rank attention  CKV [slots, 1, cap, rank + rot_dim]                        (compute type)
    decaying matrix   S [slots, H, dim, vdim]                                      (float32)
    matrix memory     S [slots, H, dim, vdim]    n [slots, H, dim]    m [slots, H]  (float32)
    short convolution tail [slots, 2, taps - 1, width]                             (float32, double-buffered)
    vector state      vec [slots, width]                                            (float32)

(a layer's spec may be a tuple of these, or None for a layer that reads another layer's rows)

so that one kernel launch serves a whole batch: it gets the slot of every batch entry and the number of tokens the slot
already holds.  A slot that is released is handed out again; nothing is cleared, because every consumer starts a sequence
whose slot holds no tokens from zero (the recurrent kernels) or reads only rows below the sequence's length (attention).
The pool grows (more slots, more rows per slot) by reallocation; `version` changes when it does, which invalidates
captured CUDA graphs that hold its addresses.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch


@dataclass(frozen=True)
class KVSpec:
    """An attention layer's rows: `n_kv_heads` heads of `dim` key and `vdim` value elements per token."""
    n_kv_heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class MatrixMemorySpec:
    """A matrix-memory recurrent layer's state: per head a dim x vdim matrix, a dim vector and a scalar."""
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class LatentKVSpec:
    """A low-rank attention layer's rows: per token ONE row [latent (rank) | rotated key part (rot_dim)] for all heads."""
    rank: int
    rot_dim: int


@dataclass(frozen=True)
class DecayStateSpec:
    """A gated linear-attention layer's state: per head a dim x vdim matrix whose rows decay."""
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class ConvTailSpec:
    """The last `taps - 1` inputs of a causal convolution over time on `width` channels, kept twice: a step reads one copy
    and writes the other (the sequence's step parity says which), so that one launch can do both for a whole batch."""
    taps: int
    width: int


@dataclass(frozen=True)
class VectorStateSpec:
    """An element-wise recurrent layer's state: one number per channel."""
    width: int


class SlotPool:
    def __init__(self, specs: List[object], dtype: torch.dtype, device, n_slots: int = 2, cap: int = 128,
                 max_tokens: Optional[int] = None):
        self.specs, self.dtype, self.device = list(specs), dtype, torch.device(device)
        self.max_tokens = max_tokens  # most tokens live sequences hold at any time (None: unbounded); bounds `cap`
        self.n_slots, self.cap, self.version = 0, 0, 0
        self.layers: List[Dict[str, torch.Tensor]] = [dict() for _ in specs]
        self.rows: Dict[int, int] = {}   # live slot -> tokens it holds
        self._free: List[int] = []
        self._resize(max(1, n_slots), self._round_cap(cap))

    def _round_cap(self, cap: int) -> int:
        cap = ((max(int(cap), 1) + 127) // 128) * 128
        if self.max_tokens is not None:
            cap = min(cap, ((int(self.max_tokens) + 127) // 128) * 128)
        return cap

    def _alloc(self, spec, n_slots: int, cap: int) -> Dict[str, torch.Tensor]:
        if spec is None:  # a layer that keeps nothing (it reads another layer's rows)
            return {}
        if isinstance(spec, (tuple, list)):  # a layer with several kinds of state
            out: Dict[str, torch.Tensor] = {}
            for part in spec:
                out.update(self._alloc(part, n_slots, cap))
            return out
        if isinstance(spec, ConvTailSpec):
            return {"tail": torch.zeros(n_slots, 2, max(spec.taps - 1, 1), spec.width, dtype=torch.float32, device=self.device)}
        if isinstance(spec, KVSpec):
            return {"k": torch.zeros(n_slots, spec.n_kv_heads, cap, spec.dim, dtype=self.dtype, device=self.device),
                    "v": torch.zeros(n_slots, spec.n_kv_heads, cap, spec.vdim, dtype=self.dtype, device=self.device)}
        if isinstance(spec, LatentKVSpec):
            return {"ckv": torch.zeros(n_slots, 1, cap, spec.rank + spec.rot_dim, dtype=self.dtype, device=self.device)}
        if isinstance(spec, VectorStateSpec):
            return {"vec": torch.zeros(n_slots, spec.width, dtype=torch.float32, device=self.device)}
        if isinstance(spec, DecayStateSpec):
            return {"s": torch.zeros(n_slots, spec.heads, spec.dim, spec.vdim, dtype=torch.float32, device=self.device)}
        if isinstance(spec, MatrixMemorySpec):
            return {"s": torch.zeros(n_slots, spec.heads, spec.dim, spec.vdim, dtype=torch.float32, device=self.device),
                    "n": torch.zeros(n_slots, spec.heads, spec.dim, dtype=torch.float32, device=self.device),
                    "m": torch.zeros(n_slots, spec.heads, dtype=torch.float32, device=self.device)}
        raise TypeError(f"unknown layer state {spec!r}")

    def _resize(self, n_slots: int, cap: int) -> None:
        old_slots, old_cap = self.n_slots, self.cap
        new_layers = []
        for spec, old in zip(self.specs, self.layers):
            new = self._alloc(spec, n_slots, cap)
            for name, t in old.items():  # carry every slot over (released ones hold nothing anybody reads)
                if name in ("k", "v", "ckv"):
                    new[name][:old_slots, :, :old_cap].copy_(t)
                else:
                    new[name][:old_slots].copy_(t)
            new_layers.append(new)
        self.layers = new_layers
        self._free += list(range(n_slots - 1, old_slots - 1, -1))  # lowest new slot is handed out first
        self.n_slots, self.cap = n_slots, cap
        self.version += 1

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for layer in self.layers for t in layer.values())

    # ---- slots ---------------------------------------------------------------------------------------------
    def acquire(self) -> int:
        if not self._free:
            self._resize(self.n_slots * 2, self.cap)
        slot = self._free.pop()
        self.rows[slot] = 0
        return slot

    def release(self, slot: int) -> None:
        if slot in self.rows:
            del self.rows[slot]
            self._free.append(slot)

    def reserve(self, slot: int, rows: int) -> None:
        """Make room for `rows` tokens in `slot` (all slots share one capacity)."""
        if rows > self.cap:
            cap = self._round_cap(max(rows, self.cap * 2))
            if rows > cap:
                raise ValueError(f"a sequence of {rows} tokens exceeds the pool's token limit ({self.max_tokens})")
            self._resize(self.n_slots, cap)


class SeqState:
    """One sequence's handle: what a model hands back as `past_key_values` and takes again for the next tokens.  The slot
    goes back to the pool when the handle is freed or garbage-collected."""

    def __init__(self, pool: SlotPool):
        self.pool, self.slot = pool, pool.acquire()
        self.steps = 0           # steps this sequence has run (its parity selects the copy of double-buffered state)
        self.last_token = -1     # the sequence's latest token id (designs whose embedding looks at the previous token)

    @property
    def rows(self) -> int:
        return self.pool.rows.get(self.slot, 0) if self.slot is not None else 0

    def free(self) -> None:
        if self.slot is not None:
            self.pool.release(self.slot)
            self.slot = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
