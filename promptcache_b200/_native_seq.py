"""ctypes binding of libpromptcache_b200_seq.so (the C ABI in include/promptcache_b200_seq.h): the sequence-batch kernels.

Like `_native`, this is the only way the Python host reaches these kernels, and there is no CPU or eager fallback: a
missing library is built on first use (nvcc, sm_100a), a CPU tensor or a failed launch raises `NativeError`.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from ._native import NativeError, note_replayed_launches  # noqa: F401  (one error type for both libraries)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpromptcache_b200_seq.so")
PCS_BF16, PCS_F32 = 0, 1
EXPORTS = ("pcs_version", "pcs_last_error", "pcs_launch_count", "pcs_attn_workspace_floats", "pcs_embed", "pcs_rmsnorm", "pcs_gate_norm_add", "pcs_xielu", "pcs_linear_rows",
           "pcs_qk_prep", "pcs_attn", "pcs_mlstm_gates", "pcs_mlstm_scan", "pcs_embed_bigram", "pcs_norm_conv", "pcs_rope_kv_prep", "pcs_moe_route",
           "pcs_moe_rows_up", "pcs_moe_rows_down", "pcs_moe_plan", "pcs_moe_gather", "pcs_moe_gemm", "pcs_moe_combine", "pcs_silu_mul", "pcs_glu_mul",
           "pcs_depth_mix", "pcs_latent_prep", "pcs_latent_q", "pcs_latent_gather", "pcs_latent_expand", "pcs_head_gate", "pcs_gla_decay", "pcs_gla_scan", "pcs_gla_chunk_prep", "pcs_gla_chunk_scan", "pcs_gla_chunk_out",
           "pcs_add_layer_norm", "pcs_gru_scan")
GLU_SILU, GLU_CLAMPED_SWISH = 0, 1
ACT_RELU2, ACT_GELU_ERF = 2, 3          # activations of a feed-forward without a gate branch
ROUTE_SOFTMAX, ROUTE_SIGMOID = 0, 1


class pcs_gna_params(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("g", C.c_void_p), ("y_stride", C.c_int64), ("g_stride", C.c_int64),
                ("w", C.c_void_p), ("ls", C.c_void_p), ("next_w", C.c_void_p), ("h_out", C.c_void_p),
                ("n_rows", C.c_int32), ("width", C.c_int32), ("eps", C.c_float), ("dtype", C.c_int32),
                ("w_offset", C.c_float), ("y_f32", C.c_int32)]


class pcs_qkprep_params(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("row_stride", C.c_int64), ("q_off", C.c_int32), ("k_off", C.c_int32), ("v_off", C.c_int32),
                ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p), ("eps", C.c_float),
                ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32),
                ("temp_coef", C.c_float), ("temp_every", C.c_int32),
                ("q_out", C.c_void_p), ("k_pool", C.c_void_p), ("v_pool", C.c_void_p), ("cap", C.c_int32),
                ("v_first_pool", C.c_void_p), ("v_lambda", C.c_void_p),
                ("tok_seq", C.c_void_p), ("tok_pos", C.c_void_p), ("seq_slot", C.c_void_p),
                ("n_tokens", C.c_int32), ("dtype", C.c_int32)]


class pcs_attn_params(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k_pool", C.c_void_p), ("v_pool", C.c_void_p), ("out", C.c_void_p),
                ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("cap", C.c_int32),
                ("scale", C.c_float), ("bias_r1", C.c_void_p), ("bias_r2", C.c_void_p), ("sink", C.c_int32),
                ("tok_seq", C.c_void_p), ("tok_pos", C.c_void_p), ("seq_slot", C.c_void_p), ("seq_pos0", C.c_void_p),
                ("seq_len", C.c_void_p), ("seq_off", C.c_void_p),
                ("n_tokens", C.c_int32), ("n_seqs", C.c_int32), ("max_len", C.c_int32), ("dtype", C.c_int32),
                ("impl", C.c_int32), ("max_keys", C.c_int32), ("workspace", C.c_void_p), ("workspace_floats", C.c_int64),
                ("softcap", C.c_float), ("window", C.c_int32), ("keep_first", C.c_int32), ("v_row_stride", C.c_int32),
                ("sink_logit", C.c_void_p), ("pool_slot", C.c_void_p), ("talk", C.c_void_p),
                ("out_gate", C.c_void_p), ("out_gate_stride", C.c_int64)]


class pcs_normconv_params(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("y_stride", C.c_int64), ("y_mult", C.c_float), ("g", C.c_void_p), ("g_len", C.c_int32),
                ("eps", C.c_float), ("conv_w", C.c_void_p), ("taps", C.c_int32), ("tail", C.c_void_p), ("h_out", C.c_void_p),
                ("tok_seq", C.c_void_p), ("tok_pos", C.c_void_p), ("seq_slot", C.c_void_p), ("seq_pos0", C.c_void_p), ("seq_len", C.c_void_p),
                ("seq_par", C.c_void_p), ("n_tokens", C.c_int32), ("width", C.c_int32), ("dtype", C.c_int32), ("reserved", C.c_int32)]


class pcs_rope_params(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("row_stride", C.c_int64), ("q_off", C.c_int32), ("k_off", C.c_int32), ("v_off", C.c_int32),
                ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32),
                ("freqs", C.c_void_p), ("rot_dims", C.c_int32), ("interleaved", C.c_int32), ("v_unit_rms", C.c_int32), ("eps", C.c_float),
                ("q_out", C.c_void_p), ("k_pool", C.c_void_p), ("v_pool", C.c_void_p), ("cap", C.c_int32),
                ("tok_seq", C.c_void_p), ("tok_pos", C.c_void_p), ("seq_slot", C.c_void_p), ("n_tokens", C.c_int32), ("dtype", C.c_int32),
                ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p)]


class pcs_route_params(C.Structure):
    _fields_ = [("h", C.c_void_p), ("h_stride", C.c_int64), ("w_router", C.c_void_p), ("correction", C.c_void_p), ("w_sg", C.c_void_p),
                ("n_tokens", C.c_int32), ("width", C.c_int32), ("n_outputs", C.c_int32), ("top", C.c_int32), ("n_groups", C.c_int32),
                ("keep_groups", C.c_int32), ("idx", C.c_void_p), ("wgt", C.c_void_p), ("shared_gate", C.c_void_p),
                ("dtype", C.c_int32), ("renorm", C.c_int32), ("bias", C.c_void_p),
                ("score_fn", C.c_int32), ("group_best", C.c_int32), ("wgt_scale", C.c_float), ("renorm_eps", C.c_float)]


class pcs_glu_act(C.Structure):
    _fields_ = [("kind", C.c_int32), ("alpha", C.c_float), ("limit", C.c_float)]


class pcs_depthmix_params(C.Structure):
    _fields_ = [("xs", C.c_void_p), ("term_stride", C.c_int64), ("n_terms", C.c_int32), ("coef", C.c_void_p), ("rows", C.c_void_p),
                ("x_out", C.c_void_p), ("next_w", C.c_void_p), ("h_out", C.c_void_p), ("w_offset", C.c_float), ("eps", C.c_float),
                ("n_rows", C.c_int32), ("width", C.c_int32), ("dtype", C.c_int32), ("y_f32", C.c_int32), ("y", C.c_void_p), ("y_stride", C.c_int64),
                ("y_w", C.c_void_p)]


class pcs_latent_prep_params(C.Structure):
    _fields_ = [("proj", C.c_void_p), ("row_stride", C.c_int64), ("cq_off", C.c_int32), ("ckv_off", C.c_int32), ("q_rank", C.c_int32),
                ("kv_rank", C.c_int32), ("rot_dim", C.c_int32), ("cq_norm_w", C.c_void_p), ("ckv_norm_w", C.c_void_p), ("eps", C.c_float),
                ("freqs", C.c_void_p), ("rot_mult", C.c_float), ("cq_out", C.c_void_p), ("pool", C.c_void_p), ("cap", C.c_int32),
                ("tok_seq", C.c_void_p), ("tok_pos", C.c_void_p), ("seq_slot", C.c_void_p), ("n_tokens", C.c_int32), ("dtype", C.c_int32)]


class pcs_latent_q_params(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_out", C.c_void_p), ("q_lat", C.c_void_p), ("lat_tok_stride", C.c_int64), ("lat_head_stride", C.c_int64),
                ("n_heads", C.c_int32), ("dim", C.c_int32), ("rot_dim", C.c_int32), ("kv_rank", C.c_int32), ("freqs", C.c_void_p),
                ("rot_mult", C.c_float), ("tok_pos", C.c_void_p), ("n_tokens", C.c_int32), ("dtype", C.c_int32)]


class pcs_latent_expand_params(C.Structure):
    _fields_ = [("kv", C.c_void_p), ("kv_stride", C.c_int64), ("pool", C.c_void_p), ("cap", C.c_int32), ("kv_rank", C.c_int32),
                ("rot_dim", C.c_int32), ("n_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("k_dense", C.c_void_p),
                ("v_dense", C.c_void_p), ("cap_dense", C.c_int32), ("ctx_seq", C.c_void_p), ("ctx_pos", C.c_void_p), ("seq_slot", C.c_void_p),
                ("n_ctx", C.c_int32), ("dtype", C.c_int32)]


class pcs_gla_params(C.Structure):
    _fields_ = [("proj", C.c_void_p), ("row_stride", C.c_int64), ("q_off", C.c_int32), ("k_off", C.c_int32), ("v_off", C.c_int32), ("g_off", C.c_int32),
                ("ld", C.c_void_p), ("norm_w", C.c_void_p), ("out", C.c_void_p), ("s_pool", C.c_void_p),
                ("heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("q_scale", C.c_float), ("eps", C.c_float),
                ("seq_slot", C.c_void_p), ("seq_pos0", C.c_void_p), ("seq_len", C.c_void_p), ("seq_off", C.c_void_p),
                ("n_seqs", C.c_int32), ("n_tokens", C.c_int32), ("dtype", C.c_int32), ("max_len", C.c_int32), ("impl", C.c_int32), ("o_raw", C.c_void_p)]


class pcs_gla_chunk_params(C.Structure):
    _fields_ = [("proj", C.c_void_p), ("row_stride", C.c_int64), ("q_off", C.c_int32), ("k_off", C.c_int32), ("v_off", C.c_int32), ("g_off", C.c_int32),
                ("ld", C.c_void_p), ("heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("chunk", C.c_int32), ("q_scale", C.c_float), ("eps", C.c_float),
                ("chunk_first", C.c_void_p), ("chunk_len", C.c_void_p), ("n_chunks", C.c_int32), ("n_tokens", C.c_int32), ("dtype", C.c_int32), ("n_seqs", C.c_int32),
                ("qd", C.c_void_p), ("kd", C.c_void_p), ("g", C.c_void_p), ("vf", C.c_void_p), ("a", C.c_void_p), ("u", C.c_void_p), ("s_pool", C.c_void_p),
                ("seq_slot", C.c_void_p), ("seq_pos0", C.c_void_p), ("seq_chunk0", C.c_void_p), ("seq_chunks", C.c_void_p), ("o", C.c_void_p), ("tok_row", C.c_void_p),
                ("norm_w", C.c_void_p), ("out", C.c_void_p)]


class pcs_combine_params(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("idx", C.c_void_p), ("wgt", C.c_void_p), ("h", C.c_void_p), ("h_stride", C.c_int64),
                ("ys", C.c_void_p), ("ys_stride", C.c_int64), ("shared_gate", C.c_void_p), ("mult", C.c_float),
                ("n_tokens", C.c_int32), ("width", C.c_int32), ("top", C.c_int32), ("n_experts", C.c_int32), ("dtype", C.c_int32),
                ("y_dtype", C.c_int32), ("y_row", C.c_void_p), ("overwrite", C.c_int32)]


class pcs_addln_params(C.Structure):
    _fields_ = [("x", C.c_void_p), ("rows", C.c_void_p), ("y", C.c_void_p * 3), ("y_stride", C.c_int64 * 3), ("y_mult", C.c_float * 3),
                ("y_f32", C.c_int32 * 3), ("n_addends", C.c_int32), ("w1", C.c_void_p), ("h1", C.c_void_p), ("w2", C.c_void_p), ("h2", C.c_void_p),
                ("n_rows", C.c_int32), ("width", C.c_int32), ("eps", C.c_float), ("dtype", C.c_int32)]


class pcs_gru_params(C.Structure):
    _fields_ = [("proj", C.c_void_p), ("row_stride", C.c_int64), ("z_off", C.c_int32), ("x_off", C.c_int32), ("g_off", C.c_int32), ("width", C.c_int32),
                ("out", C.c_void_p), ("s_pool", C.c_void_p), ("seq_slot", C.c_void_p), ("seq_pos0", C.c_void_p), ("seq_len", C.c_void_p),
                ("seq_off", C.c_void_p), ("n_seqs", C.c_int32), ("n_tokens", C.c_int32), ("max_len", C.c_int32), ("dtype", C.c_int32)]


class pcs_mlstm_params(C.Structure):
    _fields_ = [("proj", C.c_void_p), ("row_stride", C.c_int64),
                ("q_off", C.c_int32), ("k_off", C.c_int32), ("v_off", C.c_int32), ("g_off", C.c_int32),
                ("ig", C.c_void_p), ("fg", C.c_void_p), ("norm_w", C.c_void_p), ("out", C.c_void_p),
                ("s_pool", C.c_void_p), ("n_pool", C.c_void_p), ("m_pool", C.c_void_p),
                ("heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("q_scale", C.c_float), ("eps", C.c_float),
                ("seq_slot", C.c_void_p), ("seq_pos0", C.c_void_p), ("seq_len", C.c_void_p), ("seq_off", C.c_void_p),
                ("n_seqs", C.c_int32), ("dtype", C.c_int32), ("max_len", C.c_int32), ("impl", C.c_int32),
                ("o_raw", C.c_void_p), ("n_tokens", C.c_int32), ("reserved", C.c_int32)]


_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """dlopen the in-tree library, building it first when it is missing or older than its sources."""
    global _lib
    if _lib is not None:
        return _lib
    from . import build as _build
    try:
        path = _build.build_seq()
    except Exception as e:  # no compiler: a library that travelled with the tree is still usable
        if not os.path.exists(LIB_PATH):
            raise NativeError(f"{LIB_PATH} is missing and could not be built: {e}") from e
        path = LIB_PATH
    lib = C.CDLL(path, mode=C.RTLD_LOCAL)
    lib.pcs_version.restype = C.c_int
    lib.pcs_last_error.restype = C.c_char_p
    lib.pcs_launch_count.restype = C.c_int64
    lib.pcs_embed.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    lib.pcs_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    lib.pcs_gate_norm_add.argtypes = [C.POINTER(pcs_gna_params), C.c_void_p]
    lib.pcs_xielu.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.pcs_linear_rows.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.pcs_qk_prep.argtypes = [C.POINTER(pcs_qkprep_params), C.c_void_p]
    lib.pcs_attn.argtypes = [C.POINTER(pcs_attn_params), C.c_void_p]
    lib.pcs_mlstm_gates.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    lib.pcs_mlstm_scan.argtypes = [C.POINTER(pcs_mlstm_params), C.c_void_p]
    lib.pcs_attn_workspace_floats.argtypes = [C.c_int, C.c_int, C.c_int]
    lib.pcs_attn_workspace_floats.restype = C.c_int64
    lib.pcs_embed_bigram.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64,
                                     C.c_int64, C.c_int, C.c_void_p]
    lib.pcs_norm_conv.argtypes = [C.POINTER(pcs_normconv_params), C.c_void_p]
    lib.pcs_rope_kv_prep.argtypes = [C.POINTER(pcs_rope_params), C.c_void_p]
    lib.pcs_moe_route.argtypes = [C.POINTER(pcs_route_params), C.c_void_p]
    lib.pcs_moe_rows_up.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_void_p, C.c_int, C.c_void_p]
    lib.pcs_moe_rows_down.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    # (the grouped products are declared below)
    lib.pcs_moe_plan_ints.argtypes = [C.c_int, C.c_int]
    lib.pcs_moe_plan_ints.restype = C.c_int64
    lib.pcs_moe_plan.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    lib.pcs_moe_plan_part.argtypes = [C.c_int, C.c_int, C.c_int]
    lib.pcs_moe_plan_part.restype = C.c_int
    lib.pcs_moe_gather.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.pcs_moe_gemm.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                 C.c_void_p, C.c_void_p]
    lib.pcs_moe_combine.argtypes = [C.POINTER(pcs_combine_params), C.c_void_p]
    lib.pcs_silu_mul.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.pcs_glu_mul.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    lib.pcs_depth_mix.argtypes = [C.POINTER(pcs_depthmix_params), C.c_void_p]
    lib.pcs_latent_prep.argtypes = [C.POINTER(pcs_latent_prep_params), C.c_void_p]
    lib.pcs_latent_q.argtypes = [C.POINTER(pcs_latent_q_params), C.c_void_p]
    lib.pcs_latent_gather.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.pcs_latent_expand.argtypes = [C.POINTER(pcs_latent_expand_params), C.c_void_p]
    lib.pcs_head_gate.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.pcs_gla_decay.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    lib.pcs_gla_scan.argtypes = [C.POINTER(pcs_gla_params), C.c_void_p]
    for name in ("pcs_gla_chunk_prep", "pcs_gla_chunk_scan", "pcs_gla_chunk_out"):
        getattr(lib, name).argtypes = [C.POINTER(pcs_gla_chunk_params), C.c_void_p]
    lib.pcs_add_layer_norm.argtypes = [C.POINTER(pcs_addln_params), C.c_void_p]
    lib.pcs_gru_scan.argtypes = [C.POINTER(pcs_gru_params), C.c_void_p]
    for name in EXPORTS[4:]:
        getattr(lib, name).restype = C.c_int
    _lib = lib
    return lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed ({rc}): {load().pcs_last_error().decode('utf-8', 'replace')}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return PCS_BF16
    if dtype == torch.float32:
        return PCS_F32
    raise NativeError(f"the sequence-batch kernels compute in bfloat16 or float32, not {dtype}")


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NativeError("promptcache_b200 kernels take CUDA tensors only (no CPU path exists)")


def _rows2d(t: torch.Tensor, dtype: torch.dtype, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1 or t.dtype != dtype:
        raise NativeError(f"{what}: expected a 2-D {dtype} tensor with a contiguous inner dimension, got {tuple(t.shape)} {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return t.data_ptr() if t is not None else None


def launch_count() -> int:
    return int(load().pcs_launch_count()) if _lib is not None else 0


class Batch:
    """The int32 description of one step's batch on the device (one host-to-device copy): per token its entry and position,
    per entry its slot, the tokens the slot already holds, the number of new tokens, the index of the first one and the
    parity of the sequence's step count (which of two copies of a double-buffered state the step reads)."""

    def __init__(self, slots, pos0, lens, device, parity=None):
        n_seqs, n_tokens = len(slots), int(sum(lens))
        parity = list(parity) if parity is not None else [0] * n_seqs
        offs, tok_seq, tok_pos, o = [], [], [], 0
        for b, (p0, n) in enumerate(zip(pos0, lens)):
            offs.append(o)
            tok_seq += [b] * n
            tok_pos += range(p0, p0 + n)
            o += n
        host = torch.tensor(tok_seq + tok_pos + list(slots) + list(pos0) + list(lens) + offs + parity, dtype=torch.int32)
        self.meta = host.pin_memory().to(device, non_blocking=True) if device.type == "cuda" else host
        T, B = n_tokens, n_seqs
        m = self.meta
        self.tok_seq, self.tok_pos = m[0:T], m[T:2 * T]
        self.seq_slot, self.seq_pos0, self.seq_len, self.seq_off, self.seq_par = (m[2 * T + i * B:2 * T + (i + 1) * B] for i in range(5))
        self.prev_ids = None  # int64 [T] on the device: every token's predecessor in its sequence, -1 for a first token
        self.n_tokens, self.n_seqs, self.max_len = T, B, max(lens) if lens else 0
        self.offsets, self.lens, self.pos0, self.slots = offs, list(lens), list(pos0), list(slots)


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float) -> None:
    _cuda(table, ids, out)
    if ids.dtype != torch.int64 or not ids.is_contiguous() or out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise NativeError("embed: ids must be contiguous int64, out contiguous float32, the table contiguous")
    _check(load().pcs_embed(table.data_ptr(), ids.data_ptr(), out.data_ptr(), ids.numel(), table.shape[1], table.shape[0], float(scale),
                            dtype_code(table.dtype), _stream()), "pcs_embed")


def rmsnorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rms_norm(x[rows[r]]) * w; x is the 32-bit residual stream, out is in the compute type."""
    _cuda(x, w, out, rows)
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or out.dtype != w.dtype:
        raise NativeError("rmsnorm: x must be contiguous float32, out contiguous in the weight's type")
    if rows is not None and (rows.dtype != torch.int32 or not rows.is_contiguous() or rows.numel() != out.shape[0]):
        raise NativeError("rmsnorm: rows must be contiguous int32, one per output row")
    _check(load().pcs_rmsnorm(x.data_ptr(), _ptr(rows), w.data_ptr(), out.data_ptr(), out.shape[0], x.shape[1], float(eps),
                              dtype_code(w.dtype), _stream()), "pcs_rmsnorm")


def gate_norm_add(x: torch.Tensor, y: torch.Tensor, g: Optional[torch.Tensor], w: torch.Tensor, ls: Optional[torch.Tensor], eps: float,
                  next_w: Optional[torch.Tensor] = None, h_out: Optional[torch.Tensor] = None, w_offset: float = 0.0) -> None:
    """x += ls * (w_offset + w) * rms_norm(y * sigmoid(g)); then h_out = rms_norm(x) * (w_offset + next_w) when next_w is given.  y is
    in the weights' type or float32."""
    _cuda(x, y, g, w, ls, next_w, h_out)
    _rows2d(y, torch.float32 if y.dtype == torch.float32 else w.dtype, "gate_norm_add: y")
    if g is not None:
        _rows2d(g, w.dtype, "gate_norm_add: g")
    if x.dtype != torch.float32 or not x.is_contiguous() or x.shape != y.shape:
        raise NativeError("gate_norm_add: x must be contiguous float32 of y's shape")
    if h_out is not None and (not h_out.is_contiguous() or h_out.dtype != w.dtype):
        raise NativeError("gate_norm_add: h_out must be contiguous in the compute type")
    p = pcs_gna_params()
    p.x, p.y, p.g, p.y_stride, p.g_stride = x.data_ptr(), y.data_ptr(), _ptr(g), y.stride(0), g.stride(0) if g is not None else 0
    p.w, p.ls, p.next_w, p.h_out = w.data_ptr(), _ptr(ls), _ptr(next_w), _ptr(h_out)
    p.n_rows, p.width, p.eps, p.dtype = x.shape[0], x.shape[1], float(eps), dtype_code(w.dtype)
    p.w_offset, p.y_f32 = float(w_offset), 1 if (y.dtype == torch.float32 and w.dtype != torch.float32) else 0
    _check(load().pcs_gate_norm_add(C.byref(p), _stream()), "pcs_gate_norm_add")


def xielu(z: torch.Tensor, out: torch.Tensor, a: torch.Tensor) -> None:
    _cuda(z, out, a)
    _rows2d(z, a.dtype, "xielu: z")
    _rows2d(out, a.dtype, "xielu: out")
    _check(load().pcs_xielu(z.data_ptr(), z.stride(0), out.data_ptr(), out.stride(0), a.data_ptr(), z.shape[0], z.shape[1],
                            dtype_code(a.dtype), _stream()), "pcs_xielu")


LINEAR_ROWS_MAX = 8
ATTN_MAX_VDIM = 512   # value columns per head that every attention kernel serves


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, kernel: Optional[bool] = None) -> torch.Tensor:
    """x [M, K] @ w [N, K]^T + bias.  `pcs_linear_rows` streams the weights once for one to eight rows; by default it takes
    the shapes where it was measured faster than the library's product in a replayed decode graph on B200 (at most four
    rows, and few output features or a long K: 4.0 against 8.4 us for 2048 x 2048, 9.8 against 21.3 us for 2048 x 8192 at
    one row); wide outputs over a short K are left to the library, which reaches 3 to 4 TB/s there.  `kernel=True / False`
    forces the choice."""
    M, K = x.shape
    N = w.shape[0]
    fits = (0 < M <= LINEAR_ROWS_MAX and w.is_contiguous() and x.stride(1) == 1 and x.dtype == w.dtype and K % (16 // x.element_size()) == 0 and
            (x.stride(0) * x.element_size()) % 16 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)
    if kernel is None:
        kernel = fits and M <= 4 and (N <= 4096 or K >= 4096)
    if not (kernel and fits):
        return torch.nn.functional.linear(x, w, bias)
    _cuda(x, w, bias)
    out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    _check(load().pcs_linear_rows(x.data_ptr(), x.stride(0), w.data_ptr(), _ptr(bias), out.data_ptr(), out.stride(0), M, N, K,
                                  dtype_code(x.dtype), _stream()), "pcs_linear_rows")
    return out


def qk_prep(qkv: torch.Tensor, offs, q_norm_w, k_norm_w, eps: float, n_heads: int, n_kv_heads: int, dim: int, vdim: int,
            temp_coef: float, temp_every: int, q_out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
            v_first_pool: Optional[torch.Tensor], v_lambda: Optional[torch.Tensor], batch: Batch) -> None:
    """qkv: [T, *] projections with q / k / v at the column offsets `offs`; pools [slots, Hkv, cap, dim | vdim]."""
    _cuda(qkv, q_out, k_pool, v_pool)
    dt = qkv.dtype
    _rows2d(qkv, dt, "qk_prep: qkv")
    if not (k_pool.is_contiguous() and v_pool.is_contiguous() and q_out.is_contiguous()) or k_pool.dtype != dt or v_pool.dtype != dt:
        raise NativeError("qk_prep: pools and q_out must be contiguous tensors of the compute type")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, k_pool.shape[2], dim) or tuple(v_pool.shape[1:]) != (n_kv_heads, k_pool.shape[2], vdim):
        raise NativeError("qk_prep: pool shapes do not match the head sizes")
    if v_first_pool is not None and v_first_pool.shape != v_pool.shape:
        raise NativeError("qk_prep: the mixed-in value pool must have the shape of this layer's value pool")
    p = pcs_qkprep_params()
    p.qkv, p.row_stride = qkv.data_ptr(), qkv.stride(0)
    p.q_off, p.k_off, p.v_off = offs
    p.q_norm_w, p.k_norm_w, p.eps = _ptr(q_norm_w), _ptr(k_norm_w), float(eps)
    p.n_heads, p.n_kv_heads, p.dim, p.vdim = n_heads, n_kv_heads, dim, vdim
    p.temp_coef, p.temp_every = float(temp_coef), int(temp_every)
    p.q_out, p.k_pool, p.v_pool, p.cap = q_out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[2]
    p.v_first_pool, p.v_lambda = _ptr(v_first_pool), _ptr(v_lambda)
    p.tok_seq, p.tok_pos, p.seq_slot = batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.seq_slot.data_ptr()
    p.n_tokens, p.dtype = batch.n_tokens, dtype_code(dt)
    _check(load().pcs_qk_prep(C.byref(p), _stream()), "pcs_qk_prep")


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float,
              r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], sink: bool, batch: Batch, impl: int = 0,
              max_keys: int = 0, workspace: Optional[torch.Tensor] = None, softcap: float = 0.0, window: int = 0,
              keep_first: int = 0, sink_logit: Optional[torch.Tensor] = None, v_row_stride: int = 0,
              pool_slot: Optional[torch.Tensor] = None, talk: Optional[torch.Tensor] = None, out_gate: Optional[torch.Tensor] = None) -> None:
    """q [T, H*dim], out [T, H*vdim]; causal over each entry's own slot rows; r1 / r2 float32 [H] or None.  With a float32
    `workspace` (attn_workspace) and `max_keys` (upper bound of the keys a token sees) few tokens over many keys are run
    as several splits of the keys that a second launch merges.  `softcap` > 0 caps the scaled score by softcap * tanh(s /
    softcap); `window` > 0 limits query i to keys j with i - j < window or j < keep_first.  `sink_logit` (float32 [H], with
    sink=True): the sink's term is exp(sink_logit[h]) instead of exp(0).  `v_row_stride` > 0: a key's value row starts that many
    elements after the previous key's (the values may be a leading part of the key rows: pass the key pool as v_pool too; vdim is
    then out's width per head).  `pool_slot` (int32 [entries]) replaces the batch's slots.  `talk` (float32 [H, H]): every (query, key)
    pair's scaled scores are mixed across heads, s'[h] = sum_g talk[h, g] s[g], before the mask and the softmax; with it, `out_gate`
    ([T, H * vdim], row stride free): out *= sigmoid(out_gate), element by element."""
    _cuda(q, k_pool, v_pool, out, r1, r2, sink_logit, pool_slot, talk)
    if talk is not None and (talk.dtype != torch.float32 or tuple(talk.shape) != (n_heads, n_heads) or not talk.is_contiguous()):
        raise NativeError("attention: talk must be contiguous float32 [H, H]")
    if sink_logit is not None and (sink_logit.dtype != torch.float32 or sink_logit.numel() != n_heads or not sink_logit.is_contiguous()):
        raise NativeError("attention: sink_logit must be float32 [H]")
    if pool_slot is not None and (pool_slot.dtype != torch.int32 or pool_slot.numel() != batch.n_seqs or not pool_slot.is_contiguous()):
        raise NativeError("attention: pool_slot must be int32 [entries]")
    dt = q.dtype
    if not (q.is_contiguous() and out.is_contiguous() and k_pool.is_contiguous() and v_pool.is_contiguous()) or out.dtype != dt \
            or k_pool.dtype != dt or v_pool.dtype != dt:
        raise NativeError("attention: q, out and the pools must be contiguous tensors of one compute type")
    for r in (r1, r2):
        if r is not None and (r.dtype != torch.float32 or r.numel() != n_heads or not r.is_contiguous()):
            raise NativeError("attention: the distance-bias numbers must be float32 [H]")
    p = pcs_attn_params()
    p.q, p.k_pool, p.v_pool, p.out = q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr()
    p.n_heads, p.n_kv_heads, p.dim, p.cap = n_heads, k_pool.shape[1], k_pool.shape[3], k_pool.shape[2]
    p.vdim = out.shape[1] // n_heads if v_row_stride else v_pool.shape[3]
    p.v_row_stride, p.sink_logit, p.pool_slot, p.talk = int(v_row_stride), _ptr(sink_logit), _ptr(pool_slot), _ptr(talk)
    if out_gate is not None:
        _cuda(out_gate)
        if out_gate.dtype != dt or out_gate.dim() != 2 or out_gate.stride(1) != 1 or tuple(out_gate.shape) != tuple(out.shape):
            raise NativeError("attention: out_gate must be [T, H * vdim] in the compute type with a contiguous inner dimension")
        p.out_gate, p.out_gate_stride = out_gate.data_ptr(), out_gate.stride(0)
    p.scale, p.bias_r1, p.bias_r2, p.sink = float(scale), _ptr(r1), _ptr(r2), 1 if sink else 0
    p.tok_seq, p.tok_pos, p.seq_slot = batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.seq_slot.data_ptr()
    p.seq_pos0, p.seq_len, p.seq_off = batch.seq_pos0.data_ptr(), batch.seq_len.data_ptr(), batch.seq_off.data_ptr()
    p.n_tokens, p.n_seqs, p.max_len, p.dtype, p.impl = batch.n_tokens, batch.n_seqs, batch.max_len, dtype_code(dt), impl
    p.softcap, p.window, p.keep_first = float(softcap), int(window), int(keep_first)
    if workspace is not None:
        if workspace.dtype != torch.float32 or not workspace.is_cuda or not workspace.is_contiguous():
            raise NativeError("attention: the workspace must be a contiguous CUDA float32 tensor")
        p.max_keys, p.workspace, p.workspace_floats = int(max_keys), workspace.data_ptr(), workspace.numel()
    _check(load().pcs_attn(C.byref(p), _stream()), "pcs_attn")


def attn_workspace(n_tokens: int, n_heads: int, vdim: int, device) -> torch.Tensor:
    return torch.empty(int(load().pcs_attn_workspace_floats(n_tokens, n_heads, vdim)), dtype=torch.float32, device=device)


def mlstm_gates(h: torch.Tensor, w_i: torch.Tensor, w_f: torch.Tensor, b_i: torch.Tensor, b_f: torch.Tensor, ig: torch.Tensor,
                fg: torch.Tensor, cap: float) -> None:
    _cuda(h, w_i, w_f, b_i, b_f, ig, fg)
    _rows2d(h, w_i.dtype, "mlstm_gates: h")
    if not (w_i.is_contiguous() and w_f.is_contiguous()) or b_i.dtype != torch.float32 or b_f.dtype != torch.float32 \
            or ig.dtype != torch.float32 or fg.dtype != torch.float32 or not ig.is_contiguous() or not fg.is_contiguous():
        raise NativeError("mlstm_gates: weights contiguous, biases and gates float32")
    _check(load().pcs_mlstm_gates(h.data_ptr(), h.stride(0), w_i.data_ptr(), w_f.data_ptr(), b_i.data_ptr(), b_f.data_ptr(),
                                  ig.data_ptr(), fg.data_ptr(), h.shape[0], h.shape[1], w_i.shape[0], float(cap),
                                  dtype_code(w_i.dtype), _stream()), "pcs_mlstm_gates")


def mlstm_scan(proj: torch.Tensor, offs, ig: torch.Tensor, fg: torch.Tensor, norm_w: torch.Tensor, out: torch.Tensor,
               s_pool: torch.Tensor, n_pool: torch.Tensor, m_pool: torch.Tensor, eps: float, batch: Batch, impl: int = 0) -> None:
    """proj [T, *] with q / k / v / output-gate columns at `offs`; state pools float32 [slots, H, dim, vdim], [slots, H, dim],
    [slots, H]; out [T, H*vdim]."""
    _cuda(proj, ig, fg, norm_w, out, s_pool, n_pool, m_pool)
    dt = proj.dtype
    _rows2d(proj, dt, "mlstm_scan: proj")
    if s_pool.dtype != torch.float32 or n_pool.dtype != torch.float32 or m_pool.dtype != torch.float32 \
            or not (s_pool.is_contiguous() and n_pool.is_contiguous() and m_pool.is_contiguous() and out.is_contiguous()):
        raise NativeError("mlstm_scan: the state pools must be contiguous float32")
    p = pcs_mlstm_params()
    p.proj, p.row_stride = proj.data_ptr(), proj.stride(0)
    p.q_off, p.k_off, p.v_off, p.g_off = offs
    p.ig, p.fg, p.norm_w, p.out = ig.data_ptr(), fg.data_ptr(), norm_w.data_ptr(), out.data_ptr()
    p.s_pool, p.n_pool, p.m_pool = s_pool.data_ptr(), n_pool.data_ptr(), m_pool.data_ptr()
    p.heads, p.dim, p.vdim = s_pool.shape[1], s_pool.shape[2], s_pool.shape[3]
    p.q_scale, p.eps = float(p.dim) ** -0.5, float(eps)
    p.seq_slot, p.seq_pos0, p.seq_len, p.seq_off = (batch.seq_slot.data_ptr(), batch.seq_pos0.data_ptr(), batch.seq_len.data_ptr(),
                                                    batch.seq_off.data_ptr())
    p.n_seqs, p.dtype, p.max_len, p.impl = batch.n_seqs, dtype_code(dt), batch.max_len, impl
    # scratch: the recurrence's raw result per token, and the new n / m per entry until the commit launch stores them
    o_raw = torch.empty(batch.n_tokens * p.heads * p.vdim + batch.n_seqs * p.heads * (p.dim + 1), dtype=torch.float32, device=proj.device)
    p.o_raw, p.n_tokens = o_raw.data_ptr(), batch.n_tokens
    _check(load().pcs_mlstm_scan(C.byref(p), _stream()), "pcs_mlstm_scan")


def embed_bigram(table: torch.Tensor, pair: torch.Tensor, ids: torch.Tensor, prev_ids: torch.Tensor, out: torch.Tensor, buckets: int,
                 mul_prev: int, mul_cur: int) -> None:
    """out = table[ids] + pair[(prev * mul_prev + id * mul_cur) mod buckets], the pair table's last row where prev < 0."""
    _cuda(table, pair, ids, prev_ids, out)
    if ids.dtype != torch.int64 or prev_ids.dtype != torch.int64 or not ids.is_contiguous() or not prev_ids.is_contiguous() \
            or prev_ids.numel() != ids.numel() or out.dtype != torch.float32 or not out.is_contiguous():
        raise NativeError("embed_bigram: ids and prev_ids contiguous int64 of one length, out contiguous float32")
    if not (table.is_contiguous() and pair.is_contiguous()) or pair.dtype != table.dtype or pair.shape[0] != buckets + 1 or pair.shape[1] != table.shape[1]:
        raise NativeError("embed_bigram: the pair table must be [buckets + 1, width] in the embedding's type")
    _check(load().pcs_embed_bigram(table.data_ptr(), pair.data_ptr(), ids.data_ptr(), prev_ids.data_ptr(), out.data_ptr(), ids.numel(),
                                   table.shape[1], table.shape[0], int(buckets), int(mul_prev), int(mul_cur), dtype_code(table.dtype), _stream()),
           "pcs_embed_bigram")


def norm_conv(x: torch.Tensor, g: Optional[torch.Tensor], eps: float, h_out: Optional[torch.Tensor], y: Optional[torch.Tensor] = None,
              y_mult: float = 1.0, conv_w: Optional[torch.Tensor] = None, tail: Optional[torch.Tensor] = None, batch: Optional[Batch] = None) -> None:
    """x += y_mult * y (when y is given); h_out = u + causal_conv(u) with u = rms_norm(x) * g (g: one number or [width]).  conv_w is
    [taps, width], the last tap weighing the token itself.  `tail` [slots, 2, taps - 1, width] float32 carries the last inputs
    of every slot from step to step."""
    _cuda(x, g, h_out, y, conv_w, tail)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2:
        raise NativeError("norm_conv: x must be a contiguous float32 matrix")
    dt = h_out.dtype if h_out is not None else y.dtype
    p = pcs_normconv_params()
    p.x, p.eps, p.n_tokens, p.width, p.dtype = x.data_ptr(), float(eps), x.shape[0], x.shape[1], dtype_code(dt)
    if y is not None:
        _rows2d(y, dt, "norm_conv: y")
        if y.shape != x.shape:
            raise NativeError("norm_conv: y must have x's shape")
        p.y, p.y_stride, p.y_mult = y.data_ptr(), y.stride(0), float(y_mult)
    if h_out is not None:
        if g is None or g.dtype != dt or not g.is_contiguous() or g.numel() not in (1, x.shape[1]) or not h_out.is_contiguous() or h_out.shape != x.shape:
            raise NativeError("norm_conv: g is one number or [width] in h_out's type; h_out contiguous of x's shape")
        p.g, p.g_len, p.h_out = g.data_ptr(), g.numel(), h_out.data_ptr()
    if conv_w is not None:
        taps = conv_w.shape[0]
        if conv_w.dtype != dt or not conv_w.is_contiguous() or conv_w.shape[1] != x.shape[1] or batch is None:
            raise NativeError("norm_conv: conv_w must be contiguous [taps, width] in the compute type, with the batch given")
        if taps > 1 and (tail is None or tail.dtype != torch.float32 or not tail.is_contiguous() or tuple(tail.shape[1:]) != (2, taps - 1, x.shape[1])):
            raise NativeError("norm_conv: tail must be contiguous float32 [slots, 2, taps - 1, width]")
        p.conv_w, p.taps, p.tail = conv_w.data_ptr(), taps, _ptr(tail)
        p.tok_seq, p.tok_pos, p.seq_slot = batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.seq_slot.data_ptr()
        p.seq_pos0, p.seq_len, p.seq_par = batch.seq_pos0.data_ptr(), batch.seq_len.data_ptr(), batch.seq_par.data_ptr()
    _check(load().pcs_norm_conv(C.byref(p), _stream()), "pcs_norm_conv")


def rope_kv_prep(qkv: torch.Tensor, offs, n_heads: int, n_kv_heads: int, dim: int, vdim: int, freqs: Optional[torch.Tensor], rot_dims: int,
                 interleaved: bool, v_unit_rms: bool, eps: float, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                 v_pool: Optional[torch.Tensor], batch: Batch, q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None) -> None:
    """qkv [T, *] with q / k / v at the column offsets `offs` (k and v offsets None: the layer appends no rows).  freqs: float64
    [rot_dims / 2] on the device.  `q_norm_w` / `k_norm_w` ([dim], shared by the heads): every query / key head is first divided by
    its root mean square (eps inside the root) and multiplied by the weight."""
    _cuda(qkv, q_out, k_pool, v_pool, freqs, q_norm_w, k_norm_w)
    dt = qkv.dtype
    for w in (q_norm_w, k_norm_w):
        if w is not None and (w.dtype != dt or not w.is_contiguous() or w.numel() != dim):
            raise NativeError("rope_kv_prep: a head norm's weight must be contiguous [dim] in the compute type")
    _rows2d(qkv, dt, "rope_kv_prep: qkv")
    if not q_out.is_contiguous() or q_out.dtype != dt:
        raise NativeError("rope_kv_prep: q_out must be contiguous in the compute type")
    if freqs is not None and (freqs.dtype != torch.float64 or not freqs.is_contiguous() or freqs.numel() < rot_dims // 2):
        raise NativeError("rope_kv_prep: freqs must be contiguous float64 [rot_dims / 2]")
    p = pcs_rope_params()
    p.qkv, p.row_stride = qkv.data_ptr(), qkv.stride(0)
    p.q_off, p.k_off, p.v_off = offs[0], -1 if offs[1] is None else offs[1], -1 if offs[2] is None else offs[2]
    p.n_heads, p.n_kv_heads, p.dim, p.vdim = n_heads, n_kv_heads, dim, vdim
    p.freqs, p.rot_dims, p.interleaved, p.v_unit_rms, p.eps = _ptr(freqs), int(rot_dims), 1 if interleaved else 0, 1 if v_unit_rms else 0, float(eps)
    p.q_out = q_out.data_ptr()
    if offs[1] is not None:
        if k_pool is None or v_pool is None or not (k_pool.is_contiguous() and v_pool.is_contiguous()) or k_pool.dtype != dt or v_pool.dtype != dt \
                or tuple(k_pool.shape[1:]) != (n_kv_heads, k_pool.shape[2], dim) or tuple(v_pool.shape[1:]) != (n_kv_heads, k_pool.shape[2], vdim):
            raise NativeError("rope_kv_prep: pools must be contiguous [slots, Hkv, cap, dim | vdim] in the compute type")
        p.k_pool, p.v_pool, p.cap = k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[2]
    p.tok_seq, p.tok_pos, p.seq_slot = batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.seq_slot.data_ptr()
    p.n_tokens, p.dtype = batch.n_tokens, dtype_code(dt)
    p.q_norm_w, p.k_norm_w = _ptr(q_norm_w), _ptr(k_norm_w)
    _check(load().pcs_rope_kv_prep(C.byref(p), _stream()), "pcs_rope_kv_prep")


def moe_route(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], w_sg: Optional[torch.Tensor], top: int, n_groups: int = 1,
              keep_groups: int = 1, bias: Optional[torch.Tensor] = None, renorm: bool = False, score_fn: int = ROUTE_SOFTMAX, group_best: int = 1,
              wgt_scale: float = 1.0, renorm_eps: float = 0.0):
    """(idx int32 [T, top], wgt float32 [T, top], shared gate float32 [T] or None).  `bias` (float32 [outputs]) is added to the
    router's outputs; `renorm`: the weights are divided by their sum (+ renorm_eps) over the chosen outputs.  `score_fn`: softmax over
    all outputs or a sigmoid of each; `group_best`: a group's score is the sum of that many of its largest choice scores;
    `wgt_scale` multiplies the weights at the end."""
    _cuda(h, w_router, correction, w_sg, bias)
    if bias is not None and (bias.dtype != torch.float32 or not bias.is_contiguous() or bias.numel() != w_router.shape[0]):
        raise NativeError("moe_route: bias must be float32 [outputs]")
    dt = h.dtype
    _rows2d(h, dt, "moe_route: h")
    if w_router.dtype != dt or not w_router.is_contiguous() or w_router.shape[1] != h.shape[1]:
        raise NativeError("moe_route: the router matrix must be contiguous [outputs, width] in h's type")
    if correction is not None and (correction.dtype != torch.float32 or not correction.is_contiguous() or correction.numel() != w_router.shape[0]):
        raise NativeError("moe_route: correction must be float32 [outputs]")
    if w_sg is not None and (w_sg.dtype != dt or not w_sg.is_contiguous() or w_sg.numel() != h.shape[1]):
        raise NativeError("moe_route: the shared gate's weights must be [width] in h's type")
    T = h.shape[0]
    idx = torch.empty(T, top, dtype=torch.int32, device=h.device)
    wgt = torch.empty(T, top, dtype=torch.float32, device=h.device)
    sg = torch.empty(T, dtype=torch.float32, device=h.device) if w_sg is not None else None
    p = pcs_route_params()
    p.h, p.h_stride, p.w_router, p.correction, p.w_sg = h.data_ptr(), h.stride(0), w_router.data_ptr(), _ptr(correction), _ptr(w_sg)
    p.n_tokens, p.width, p.n_outputs, p.top, p.n_groups, p.keep_groups = T, h.shape[1], w_router.shape[0], int(top), int(n_groups), int(keep_groups)
    p.idx, p.wgt, p.shared_gate, p.dtype = idx.data_ptr(), wgt.data_ptr(), _ptr(sg), dtype_code(dt)
    p.renorm, p.bias = 1 if renorm else 0, _ptr(bias)
    p.score_fn, p.group_best, p.wgt_scale, p.renorm_eps = int(score_fn), int(group_best), float(wgt_scale), float(renorm_eps)
    _check(load().pcs_moe_route(C.byref(p), _stream()), "pcs_moe_route")
    return idx, wgt, sg


MOE_ROWS_MAX_PAIRS = 64


def _glu(act):
    """None (silu(g) * u) or (kind, alpha, limit) -> the C struct (pass C.byref of it; None stays None)."""
    if act is None:
        return None
    kind, alpha, limit = act
    return C.byref(pcs_glu_act(int(kind), float(alpha), float(limit)))


def moe_experts(h: torch.Tensor, idx: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, grouped=None, act=None):
    """The chosen experts' results: (y [rows, width], row_of) where pair p = (token p // top, choice p % top) finds its result
    in row row_of[p] of y (row_of None: row p); rows of pass-through choices are not written.  w_gu [E, 2 ff, width] (gate rows,
    then up rows), w_down [E, width, ff].
      grouped=False       the row kernels: every pair streams its expert's weights once (decoding; the 32-bit path); y float32
      grouped="library"   many pairs in bfloat16: pairs sorted by expert on the device (`pcs_moe_plan`), their rows gathered
                          (`pcs_moe_gather`), then the library's grouped product twice with `pcs_silu_mul` between; y bfloat16
                          in the sorted order
      grouped="own"       the same through this library's grouped tensor-core kernel (`pcs_moe_gemm`), activation in its
                          epilogue, y float32 by pair
    None chooses by size: the row kernels up to 64 pairs, otherwise the library's product (or this library's where torch has none).
    `act`: None for silu(gate) * up, or (kind, alpha, limit) of the gated activation (GLU_CLAMPED_SWISH).  With an activation that
    has no gate branch (ACT_RELU2, ACT_GELU_ERF) w_gu is [E, ff, width] and the grouped product of this library is not offered."""
    _cuda(h, idx, w_gu, w_down)
    dt = h.dtype
    _rows2d(h, dt, "moe_experts: h")
    E, ff2, W = w_gu.shape
    gated = act is None or int(act[0]) in (GLU_SILU, GLU_CLAMPED_SWISH)
    ff = ff2 // 2 if gated else ff2
    if w_gu.dtype != dt or w_down.dtype != dt or not (w_gu.is_contiguous() and w_down.is_contiguous()) or tuple(w_down.shape) != (E, W, ff) \
            or idx.dtype != torch.int32 or not idx.is_contiguous() or W != h.shape[1]:
        raise NativeError("moe_experts: weights [E, 2 ff, width] and [E, width, ff] in h's type, idx contiguous int32")
    T, top = idx.shape
    P = T * top
    can_group = dt == torch.bfloat16 and ff % 8 == 0 and W % 8 == 0 and (h.stride(0) * 2) % 16 == 0 and h.data_ptr() % 16 == 0
    has_library = hasattr(torch.nn.functional, "grouped_mm")
    if grouped is True:
        grouped = "own"
    if grouped is None:
        grouped = ("library" if has_library else "own") if (can_group and P > MOE_ROWS_MAX_PAIRS) else False
    if grouped == "own" and ((not can_group and P <= 256) or not gated):
        grouped = False
    if grouped:
        if not can_group:
            raise NativeError("moe_experts: the grouped products need bfloat16 and sizes that are multiples of 8")
        lib = load()
        plan = torch.empty(int(lib.pcs_moe_plan_ints(P, E)), dtype=torch.int32, device=h.device)
        _check(lib.pcs_moe_plan(idx.data_ptr(), P, E, plan.data_ptr(), _stream()), "pcs_moe_plan")
        if grouped == "own":
            y = torch.empty(P, W, dtype=torch.float32, device=h.device)
            a_buf = torch.empty(P, ff, dtype=dt, device=h.device)
            _check(lib.pcs_moe_gemm(0, h.data_ptr(), h.stride(0), w_gu.data_ptr(), plan.data_ptr(), a_buf.data_ptr(), P, top, E, ff, W, _glu(act), _stream()), "pcs_moe_gemm")
            _check(lib.pcs_moe_gemm(1, a_buf.data_ptr(), ff, w_down.data_ptr(), plan.data_ptr(), y.data_ptr(), P, top, E, ff, W, None, _stream()), "pcs_moe_gemm")
            return y, None
        if grouped != "library" or not has_library:
            raise NativeError(f"moe_experts: unknown grouped mode {grouped!r} (or torch has no grouped product)")
        o_ends, o_rows = lib.pcs_moe_plan_part(0, P, E), lib.pcs_moe_plan_part(3, P, E)
        ends, row_of = plan[o_ends:o_ends + E], plan[o_rows:o_rows + P]
        a = torch.empty(P, W, dtype=dt, device=h.device)
        _check(lib.pcs_moe_gather(h.data_ptr(), h.stride(0), plan.data_ptr(), a.data_ptr(), P, top, E, W, _stream()), "pcs_moe_gather")
        gu = torch.nn.functional.grouped_mm(a, w_gu.transpose(1, 2), offs=ends)
        y = torch.nn.functional.grouped_mm(glu_mul(gu, ff, act), w_down.transpose(1, 2), offs=ends)
        return y, row_of
    y = torch.empty(P, W, dtype=torch.float32, device=h.device)
    a_buf = torch.empty(P, ff, dtype=dt, device=h.device)
    _check(load().pcs_moe_rows_up(h.data_ptr(), h.stride(0), w_gu.data_ptr(), idx.data_ptr(), a_buf.data_ptr(), P, top, E, ff, W, _glu(act),
                                  dtype_code(dt), _stream()), "pcs_moe_rows_up")
    _check(load().pcs_moe_rows_down(a_buf.data_ptr(), w_down.data_ptr(), idx.data_ptr(), y.data_ptr(), P, E, ff, W, dtype_code(dt), _stream()),
           "pcs_moe_rows_down")
    return y, None


def moe_combine(x: torch.Tensor, y: Optional[torch.Tensor], idx: torch.Tensor, wgt: torch.Tensor, h: torch.Tensor, n_experts: int, mult: float,
                ys: Optional[torch.Tensor] = None, shared_gate: Optional[torch.Tensor] = None, y_row: Optional[torch.Tensor] = None,
                overwrite: bool = False) -> None:
    """x += mult * (sum_k wgt[:, k] * (y of the choice, or h itself for a choice >= n_experts) + shared_gate * ys).  y is float32 or
    in h's type; `y_row` maps pair t * top + k to its row of y (None: the pair's own index).  `overwrite`: x = mult * (...) instead
    (x may be uninitialised)."""
    _cuda(x, y, idx, wgt, h, ys, shared_gate, y_row)
    dt = h.dtype
    _rows2d(h, dt, "moe_combine: h")
    if x.dtype != torch.float32 or not x.is_contiguous() or x.shape != h.shape:
        raise NativeError("moe_combine: x must be contiguous float32 of h's shape")
    T, top = idx.shape
    if idx.dtype != torch.int32 or wgt.dtype != torch.float32 or not (idx.is_contiguous() and wgt.is_contiguous()) or wgt.shape != idx.shape or T != x.shape[0]:
        raise NativeError("moe_combine: idx int32 and wgt float32 [T, top]")
    if y is not None and (y.dtype not in (torch.float32, dt) or not y.is_contiguous() or y.dim() != 2 or y.shape[1] != x.shape[1]
                          or (y_row is None and y.shape[0] != T * top)):
        raise NativeError("moe_combine: y must be contiguous [rows, width], float32 or in h's type")
    if y_row is not None and (y_row.dtype != torch.int32 or not y_row.is_contiguous() or y_row.numel() != T * top):
        raise NativeError("moe_combine: y_row must be contiguous int32 [T * top]")
    if ys is not None:
        _rows2d(ys, dt, "moe_combine: ys")
    p = pcs_combine_params()
    p.x, p.y, p.idx, p.wgt, p.h, p.h_stride = x.data_ptr(), _ptr(y), idx.data_ptr(), wgt.data_ptr(), h.data_ptr(), h.stride(0)
    p.ys, p.ys_stride, p.shared_gate, p.mult = _ptr(ys), ys.stride(0) if ys is not None else 0, _ptr(shared_gate), float(mult)
    p.n_tokens, p.width, p.top, p.n_experts, p.dtype = T, x.shape[1], top, int(n_experts), dtype_code(dt)
    p.y_dtype, p.y_row = (PCS_F32 if (y is None or y.dtype == torch.float32) else dtype_code(dt)), _ptr(y_row)
    p.overwrite = 1 if overwrite else 0
    _check(load().pcs_moe_combine(C.byref(p), _stream()), "pcs_moe_combine")


def silu_mul(gu: torch.Tensor, ff: int) -> torch.Tensor:
    """silu(gu[:, :ff]) * gu[:, ff:2 ff]."""
    _cuda(gu)
    _rows2d(gu, gu.dtype, "silu_mul: gu")
    out = torch.empty(gu.shape[0], ff, dtype=gu.dtype, device=gu.device)
    _check(load().pcs_silu_mul(gu.data_ptr(), gu.stride(0), out.data_ptr(), gu.shape[0], ff, dtype_code(gu.dtype), _stream()), "pcs_silu_mul")
    return out


def glu_mul(gu: torch.Tensor, ff: int, act=None) -> torch.Tensor:
    """act(gu[:, :ff], gu[:, ff:2 ff]) with `act` None (silu(g) * u) or (kind, alpha, limit); an activation without a gate branch
    (ACT_RELU2, ACT_GELU_ERF) reads gu[:, :ff] alone."""
    _cuda(gu)
    _rows2d(gu, gu.dtype, "glu_mul: gu")
    out = torch.empty(gu.shape[0], ff, dtype=gu.dtype, device=gu.device)
    _check(load().pcs_glu_mul(gu.data_ptr(), gu.stride(0), out.data_ptr(), gu.shape[0], ff, _glu(act), dtype_code(gu.dtype), _stream()), "pcs_glu_mul")
    return out


def depth_mix(xs: torch.Tensor, n_terms: int, coef: torch.Tensor, eps: float, x_out: Optional[torch.Tensor] = None, next_w: Optional[torch.Tensor] = None,
              h_out: Optional[torch.Tensor] = None, w_offset: float = 0.0, rows: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None,
              y_w: Optional[torch.Tensor] = None) -> None:
    """out = sum_{j < n_terms} coef[j] * xs[j] over float32 xs [terms, T, width] (at the rows `rows` when given); x_out gets the sum,
    h_out = rms_norm(out) * (w_offset + next_w).  With y [T, width] (y_w's type or float32) and y_w, xs[n_terms - 1] first takes the
    residual sum xs[n_terms - 1] += (w_offset + y_w) * rms_norm(y) in place (without `rows`: every row once)."""
    _cuda(xs, coef, x_out, next_w, h_out, rows, y, y_w)
    if y is not None:
        if y_w is None or rows is not None or y.dim() != 2 or y.stride(1) != 1 or tuple(y.shape) != tuple(xs.shape[1:]) or y.dtype not in (torch.float32, y_w.dtype) \
                or not y_w.is_contiguous() or y_w.numel() != xs.shape[2] or (next_w is not None and next_w.dtype != y_w.dtype):
            raise NativeError("depth_mix: y must be [T, width] in y_w's type or float32, y_w [width], and no row subset")
    if xs.dtype != torch.float32 or xs.dim() != 3 or not xs.is_contiguous() or not 0 < n_terms <= xs.shape[0]:
        raise NativeError("depth_mix: xs must be contiguous float32 [terms, T, width]")
    if coef.dtype != torch.float32 or not coef.is_contiguous() or coef.numel() < n_terms:
        raise NativeError("depth_mix: coef must be float32 [n_terms]")
    R = rows.numel() if rows is not None else xs.shape[1]
    if rows is not None and (rows.dtype != torch.int32 or not rows.is_contiguous()):
        raise NativeError("depth_mix: rows must be contiguous int32")
    if x_out is not None and (x_out.dtype != torch.float32 or not x_out.is_contiguous() or tuple(x_out.shape) != (R, xs.shape[2])):
        raise NativeError("depth_mix: x_out must be contiguous float32 [rows, width]")
    if next_w is not None and (h_out is None or h_out.dtype != next_w.dtype or not h_out.is_contiguous() or tuple(h_out.shape) != (R, xs.shape[2])
                               or not next_w.is_contiguous() or next_w.numel() != xs.shape[2]):
        raise NativeError("depth_mix: h_out must be contiguous [rows, width] in next_w's type")
    p = pcs_depthmix_params()
    p.xs, p.term_stride, p.n_terms, p.coef, p.rows = xs.data_ptr(), xs.stride(0), int(n_terms), coef.data_ptr(), _ptr(rows)
    p.x_out, p.next_w, p.h_out, p.w_offset, p.eps = _ptr(x_out), _ptr(next_w), _ptr(h_out), float(w_offset), float(eps)
    wt = next_w if next_w is not None else y_w
    p.n_rows, p.width, p.dtype = R, xs.shape[2], dtype_code(wt.dtype if wt is not None else torch.float32)
    if y is not None:
        p.y, p.y_stride, p.y_w, p.y_f32 = y.data_ptr(), y.stride(0), y_w.data_ptr(), 1 if (y.dtype == torch.float32 and y_w.dtype != torch.float32) else 0
    _check(load().pcs_depth_mix(C.byref(p), _stream()), "pcs_depth_mix")


def latent_prep(proj: torch.Tensor, cq_off: int, ckv_off: int, q_rank: int, kv_rank: int, rot_dim: int, cq_norm_w: Optional[torch.Tensor],
                ckv_norm_w: torch.Tensor, eps: float, freqs: Optional[torch.Tensor], rot_mult: float, cq_out: Optional[torch.Tensor], pool: torch.Tensor,
                batch: Batch) -> None:
    """proj [T, *]: the query latent at cq_off, [key/value latent | rotated key part] at ckv_off; pool [slots, 1, cap, kv_rank + rot_dim]."""
    _cuda(proj, cq_norm_w, ckv_norm_w, freqs, cq_out, pool)
    dt = proj.dtype
    _rows2d(proj, dt, "latent_prep: proj")
    if pool.dtype != dt or not pool.is_contiguous() or pool.dim() != 4 or pool.shape[1] != 1 or pool.shape[3] != kv_rank + rot_dim:
        raise NativeError("latent_prep: the pool must be contiguous [slots, 1, cap, kv_rank + rot_dim] in the compute type")
    if cq_out is not None and (cq_out.dtype != dt or not cq_out.is_contiguous() or tuple(cq_out.shape) != (proj.shape[0], q_rank)):
        raise NativeError("latent_prep: cq_out must be contiguous [T, q_rank]")
    if rot_dim and (freqs is None or freqs.dtype != torch.float64 or not freqs.is_contiguous() or freqs.numel() < rot_dim // 2):
        raise NativeError("latent_prep: freqs must be contiguous float64 [rot_dim / 2]")
    p = pcs_latent_prep_params()
    p.proj, p.row_stride, p.cq_off, p.ckv_off = proj.data_ptr(), proj.stride(0), int(cq_off), int(ckv_off)
    p.q_rank, p.kv_rank, p.rot_dim, p.cq_norm_w, p.ckv_norm_w, p.eps = int(q_rank), int(kv_rank), int(rot_dim), _ptr(cq_norm_w), ckv_norm_w.data_ptr(), float(eps)
    p.freqs, p.rot_mult, p.cq_out, p.pool, p.cap = _ptr(freqs), float(rot_mult), _ptr(cq_out), pool.data_ptr(), pool.shape[2]
    p.tok_seq, p.tok_pos, p.seq_slot = batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.seq_slot.data_ptr()
    p.n_tokens, p.dtype = batch.n_tokens, dtype_code(dt)
    _check(load().pcs_latent_prep(C.byref(p), _stream()), "pcs_latent_prep")


def latent_q(q: torch.Tensor, n_heads: int, dim: int, rot_dim: int, freqs: Optional[torch.Tensor], rot_mult: float, batch: Batch,
             q_lat: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H * (dim + rot_dim)]: every head's rotated part is turned by the token's position.  Without q_lat in place (q is
    returned); with q_lat [T, H, kv_rank] (any strides, contiguous last dimension) a new [T, H * (kv_rank + rot_dim)] matrix of
    [q_lat | rotated part] per head is returned."""
    _cuda(q, freqs, q_lat)
    dt = q.dtype
    if not q.is_contiguous() or q.dim() != 2 or q.shape[1] != n_heads * (dim + rot_dim):
        raise NativeError("latent_q: q must be contiguous [T, H * (dim + rot_dim)]")
    p = pcs_latent_q_params()
    out = q
    if q_lat is not None:
        if q_lat.dtype != dt or q_lat.dim() != 3 or q_lat.stride(2) != 1 or q_lat.shape[0] != q.shape[0] or q_lat.shape[1] != n_heads:
            raise NativeError("latent_q: q_lat must be [T, H, kv_rank] with a contiguous last dimension")
        out = torch.empty(q.shape[0], n_heads * (q_lat.shape[2] + rot_dim), dtype=dt, device=q.device)
        p.q_lat, p.lat_tok_stride, p.lat_head_stride, p.kv_rank = q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_lat.shape[2]
    p.q, p.q_out, p.n_heads, p.dim, p.rot_dim = q.data_ptr(), out.data_ptr(), int(n_heads), int(dim), int(rot_dim)
    p.freqs, p.rot_mult, p.tok_pos, p.n_tokens, p.dtype = _ptr(freqs), float(rot_mult), batch.tok_pos.data_ptr(), q.shape[0], dtype_code(dt)
    _check(load().pcs_latent_q(C.byref(p), _stream()), "pcs_latent_q")
    return out


def latent_gather(pool: torch.Tensor, width: int, ctx: Batch) -> torch.Tensor:
    """The first `width` numbers of the pool rows of every context token of `ctx` (a Batch whose entries start at position 0)."""
    _cuda(pool)
    out = torch.empty(ctx.n_tokens, width, dtype=pool.dtype, device=pool.device)
    _check(load().pcs_latent_gather(pool.data_ptr(), pool.shape[2], pool.shape[3], int(width), out.data_ptr(), ctx.tok_seq.data_ptr(), ctx.tok_pos.data_ptr(),
                                    ctx.seq_slot.data_ptr(), ctx.n_tokens, dtype_code(pool.dtype), _stream()), "pcs_latent_gather")
    return out


def latent_expand(kv: torch.Tensor, pool: torch.Tensor, kv_rank: int, rot_dim: int, n_heads: int, dim: int, vdim: int, k_dense: torch.Tensor,
                  v_dense: torch.Tensor, ctx: Batch) -> None:
    """kv [N, H * (dim + vdim)] (plain key parts of all heads, then values) of the context tokens -> k_dense [B, H, cap', dim + rot_dim],
    v_dense [B, H, cap', vdim], indexed by the batch entry."""
    _cuda(kv, pool, k_dense, v_dense)
    dt = kv.dtype
    _rows2d(kv, dt, "latent_expand: kv")
    if not (k_dense.is_contiguous() and v_dense.is_contiguous()) or k_dense.dtype != dt or v_dense.dtype != dt or pool.dtype != dt \
            or tuple(k_dense.shape[1:]) != (n_heads, k_dense.shape[2], dim + rot_dim) or tuple(v_dense.shape[1:]) != (n_heads, k_dense.shape[2], vdim):
        raise NativeError("latent_expand: dense pools must be contiguous [B, H, cap, dim + rot_dim | vdim] in the compute type")
    p = pcs_latent_expand_params()
    p.kv, p.kv_stride, p.pool, p.cap, p.kv_rank, p.rot_dim = kv.data_ptr(), kv.stride(0), pool.data_ptr(), pool.shape[2], int(kv_rank), int(rot_dim)
    p.n_heads, p.dim, p.vdim, p.k_dense, p.v_dense, p.cap_dense = int(n_heads), int(dim), int(vdim), k_dense.data_ptr(), v_dense.data_ptr(), k_dense.shape[2]
    p.ctx_seq, p.ctx_pos, p.seq_slot, p.n_ctx, p.dtype = ctx.tok_seq.data_ptr(), ctx.tok_pos.data_ptr(), ctx.seq_slot.data_ptr(), ctx.n_tokens, dtype_code(dt)
    _check(load().pcs_latent_expand(C.byref(p), _stream()), "pcs_latent_expand")


def head_gate(o: torch.Tensor, g: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, h * vdim + c] = o[t, h, c] * sigmoid(g[t, h]); o [T, H, vdim] with any token / head strides."""
    _cuda(o, g, out)
    dt = out.dtype
    if o.dim() != 3 or o.stride(2) != 1 or o.dtype != dt or g.dtype != dt or g.dim() != 2 or g.stride(1) != 1 or not out.is_contiguous():
        raise NativeError("head_gate: o [T, H, vdim] and g [T, H] with contiguous last dimensions, out contiguous, one type")
    T, H, V = o.shape
    _check(load().pcs_head_gate(o.data_ptr(), o.stride(0), o.stride(1), g.data_ptr(), g.stride(0), out.data_ptr(), T, H, V, dtype_code(dt), _stream()),
           "pcs_head_gate")


def gla_decay(a: torch.Tensor, a2: torch.Tensor, a2_b: Optional[torch.Tensor], tau: float) -> torch.Tensor:
    """float32 [T, channels]: logsigmoid(a2 a + a2_b) / tau; a [T, rank] (row stride free), a2 [channels, rank]."""
    _cuda(a, a2, a2_b)
    _rows2d(a, a2.dtype, "gla_decay: a")
    if not a2.is_contiguous() or a2.shape[1] != a.shape[1] or (a2_b is not None and (a2_b.dtype != torch.float32 or a2_b.numel() != a2.shape[0])):
        raise NativeError("gla_decay: a2 contiguous [channels, rank], the bias float32 [channels]")
    ld = torch.empty(a.shape[0], a2.shape[0], dtype=torch.float32, device=a.device)
    _check(load().pcs_gla_decay(a.data_ptr(), a.stride(0), a2.data_ptr(), _ptr(a2_b), ld.data_ptr(), a.shape[0], a2.shape[0], a2.shape[1], float(tau),
                                dtype_code(a2.dtype), _stream()), "pcs_gla_decay")
    return ld


GLA_CHUNK = 64          # tokens per chunk of the chunkwise form
GLA_CHUNK_MIN_LEN = 32  # steps whose longest entry brings fewer tokens go token by token (decoding, tails of a prompt)


def _gla_chunk_plan(batch: Batch, chunk: int):
    """The step's entries cut into chunks, as device arrays (made once per step and kept on the batch)."""
    plan = getattr(batch, "_gla_plan", None)
    if plan is not None and plan["chunk"] == chunk:
        return plan
    first, length, seq0, seqn, tok_row = [], [], [], [], []
    for off, n in zip(batch.offsets, batch.lens):
        seq0.append(len(first))
        seqn.append((n + chunk - 1) // chunk)
        for c in range(0, n, chunk):
            tok_row += range(len(first) * chunk, len(first) * chunk + min(chunk, n - c))
            first.append(off + c)
            length.append(min(chunk, n - c))
    nc = len(first)
    host = torch.tensor(first + length + seq0 + seqn + tok_row, dtype=torch.int32)
    dev = host.pin_memory().to(batch.meta.device, non_blocking=True)
    B = batch.n_seqs
    plan = {"chunk": chunk, "n_chunks": nc, "first": dev[:nc], "len": dev[nc:2 * nc], "seq0": dev[2 * nc:2 * nc + B], "seqn": dev[2 * nc + B:2 * nc + 2 * B],
            "tok_row": dev[2 * nc + 2 * B:], "all": dev}
    batch._gla_plan = plan
    return plan


def gla_scan_chunked(proj: torch.Tensor, offs, ld: torch.Tensor, norm_w: torch.Tensor, out: torch.Tensor, s_pool: torch.Tensor, eps: float, batch: Batch,
                     chunk: int = GLA_CHUNK) -> None:
    """The recurrence of `gla_scan` in chunks: the factors that carry decays are formed by `pcs_gla_chunk_prep` (32-bit, every
    exponent <= 0), the sums over tokens and channels are three batched float32 matrix products, the chunks' start states come
    from one pass over the chunks (`pcs_gla_chunk_scan`)."""
    H, D, V = s_pool.shape[1:]
    dt, dev = proj.dtype, proj.device
    plan = _gla_chunk_plan(batch, chunk)
    nc = plan["n_chunks"]
    f32 = dict(dtype=torch.float32, device=dev)
    qd, kd = torch.empty(nc * H, chunk, D, **f32), torch.empty(nc * H, chunk, D, **f32)
    g, vf, a = torch.empty(nc * H, D, **f32), torch.empty(nc * H, chunk, V, **f32), torch.empty(nc * H, chunk, chunk, **f32)
    p = pcs_gla_chunk_params()
    p.proj, p.row_stride = proj.data_ptr(), proj.stride(0)
    p.q_off, p.k_off, p.v_off, p.g_off = offs
    p.ld, p.heads, p.dim, p.vdim, p.chunk, p.q_scale, p.eps = ld.data_ptr(), H, D, V, chunk, float(D) ** -0.5, float(eps)
    p.chunk_first, p.chunk_len, p.n_chunks, p.n_tokens, p.dtype, p.n_seqs = plan["first"].data_ptr(), plan["len"].data_ptr(), nc, batch.n_tokens, dtype_code(dt), batch.n_seqs
    p.qd, p.kd, p.g, p.vf, p.a = qd.data_ptr(), kd.data_ptr(), g.data_ptr(), vf.data_ptr(), a.data_ptr()
    _check(load().pcs_gla_chunk_prep(C.byref(p), _stream()), "pcs_gla_chunk_prep")
    u = torch.bmm(kd.transpose(1, 2), vf)                  # [chunks * H, dim, vdim]: every chunk's own sum of k v^T, decayed to its end
    p.u, p.s_pool = u.data_ptr(), s_pool.data_ptr()
    p.seq_slot, p.seq_pos0, p.seq_chunk0, p.seq_chunks = batch.seq_slot.data_ptr(), batch.seq_pos0.data_ptr(), plan["seq0"].data_ptr(), plan["seqn"].data_ptr()
    _check(load().pcs_gla_chunk_scan(C.byref(p), _stream()), "pcs_gla_chunk_scan")   # u now holds the state every chunk starts from
    o = torch.baddbmm(torch.bmm(a, vf), qd, u)             # [chunks * H, chunk, vdim]
    p.o, p.tok_row, p.norm_w, p.out = o.data_ptr(), plan["tok_row"].data_ptr(), norm_w.data_ptr(), out.data_ptr()
    _check(load().pcs_gla_chunk_out(C.byref(p), _stream()), "pcs_gla_chunk_out")


def gla_scan(proj: torch.Tensor, offs, ld: torch.Tensor, norm_w: torch.Tensor, out: torch.Tensor, s_pool: torch.Tensor, eps: float, batch: Batch,
             impl: int = 0) -> None:
    """proj [T, *] with q / k / v / gate columns at `offs`; ld float32 [T, H * dim] log decays; state pool float32 [slots, H, dim, vdim];
    out [T, H * vdim].  impl 0: by step (prompts in chunks, short steps token by token); 1: token by token with the state in shared
    memory; 2: token by token (registers where the sizes allow); 3: in chunks."""
    _cuda(proj, ld, norm_w, out, s_pool)
    dt = proj.dtype
    _rows2d(proj, dt, "gla_scan: proj")
    if s_pool.dtype != torch.float32 or not s_pool.is_contiguous() or s_pool.dim() != 4 or not out.is_contiguous() or out.dtype != dt:
        raise NativeError("gla_scan: the state pool must be contiguous float32 [slots, H, dim, vdim], out contiguous in the compute type")
    H, D, V = s_pool.shape[1:]
    if ld.dtype != torch.float32 or not ld.is_contiguous() or tuple(ld.shape) != (proj.shape[0], H * D) or norm_w.dtype != dt or norm_w.numel() != V:
        raise NativeError("gla_scan: ld float32 [T, H * dim], norm_w [vdim] in the compute type")
    chunk_fits = 3 * GLA_CHUNK * (D + 1) * 4 <= 220 * 1024
    if impl == 3 or (impl == 0 and batch.max_len >= GLA_CHUNK_MIN_LEN and chunk_fits and not torch.cuda.is_current_stream_capturing()):
        return gla_scan_chunked(proj, offs, ld, norm_w, out, s_pool, eps, batch)
    p = pcs_gla_params()
    p.proj, p.row_stride = proj.data_ptr(), proj.stride(0)
    p.q_off, p.k_off, p.v_off, p.g_off = offs
    p.ld, p.norm_w, p.out, p.s_pool = ld.data_ptr(), norm_w.data_ptr(), out.data_ptr(), s_pool.data_ptr()
    p.heads, p.dim, p.vdim, p.q_scale, p.eps = H, D, V, float(D) ** -0.5, float(eps)
    p.seq_slot, p.seq_pos0, p.seq_len, p.seq_off = (batch.seq_slot.data_ptr(), batch.seq_pos0.data_ptr(), batch.seq_len.data_ptr(),
                                                    batch.seq_off.data_ptr())
    p.n_seqs, p.n_tokens, p.dtype, p.max_len, p.impl = batch.n_seqs, batch.n_tokens, dtype_code(dt), batch.max_len, 1 if impl == 1 else 0
    o_raw = torch.empty(batch.n_tokens, H * V, dtype=torch.float32, device=proj.device)
    p.o_raw = o_raw.data_ptr()
    _check(load().pcs_gla_scan(C.byref(p), _stream()), "pcs_gla_scan")


def add_layer_norm(x: torch.Tensor, addends, eps: float, w1: Optional[torch.Tensor] = None, h1: Optional[torch.Tensor] = None,
                   w2: Optional[torch.Tensor] = None, h2: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """x += sum_i mult_i * y_i for `addends` = [(y_i [T, width] in the compute type or float32, mult_i)] (at most three), then
    h1 = ln(x) * w1 and h2 = ln(x) * w2 with ln(x) = (x - mean) / sqrt(var + eps) (each optional).  With `rows` (int32) only
    those rows are normed (no addends) and h1 / h2 have one row per entry of `rows`."""
    addends = list(addends or [])
    _cuda(x, w1, h1, w2, h2, rows, *[y for y, _ in addends])
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2 or len(addends) > 3:
        raise NativeError("add_layer_norm: x must be a contiguous float32 matrix, with at most three addends")
    wt = w1 if w1 is not None else w2
    dt = wt.dtype if wt is not None else next((y.dtype for y, _ in addends if y.dtype != torch.float32), torch.float32)
    R = rows.numel() if rows is not None else x.shape[0]
    if rows is not None and (rows.dtype != torch.int32 or not rows.is_contiguous() or addends):
        raise NativeError("add_layer_norm: rows must be contiguous int32, and a row subset takes no addends")
    p = pcs_addln_params()
    p.x, p.rows, p.n_addends = x.data_ptr(), _ptr(rows), len(addends)
    for j, (y, mult) in enumerate(addends):
        if y.dim() != 2 or y.stride(1) != 1 or tuple(y.shape) != tuple(x.shape) or y.dtype not in (torch.float32, dt):
            raise NativeError("add_layer_norm: an addend must be [T, width] in the compute type or float32")
        p.y[j], p.y_stride[j], p.y_mult[j], p.y_f32[j] = y.data_ptr(), y.stride(0), float(mult), 1 if (y.dtype == torch.float32 and dt != torch.float32) else 0
    for w, h in ((w1, h1), (w2, h2)):
        if w is not None and (h is None or w.dtype != dt or h.dtype != dt or not (w.is_contiguous() and h.is_contiguous()) or w.numel() != x.shape[1]
                              or tuple(h.shape) != (R, x.shape[1])):
            raise NativeError("add_layer_norm: a weight [width] needs its output [rows, width], both in the compute type")
    p.w1, p.h1, p.w2, p.h2 = _ptr(w1), _ptr(h1) if w1 is not None else None, _ptr(w2), _ptr(h2) if w2 is not None else None
    p.n_rows, p.width, p.eps, p.dtype = R, x.shape[1], float(eps), dtype_code(dt)
    _check(load().pcs_add_layer_norm(C.byref(p), _stream()), "pcs_add_layer_norm")


def gru_scan(proj: torch.Tensor, offs, width: int, out: torch.Tensor, s_pool: torch.Tensor, batch: Batch) -> None:
    """proj [T, *] with the gate's pre-activation, the candidate's input and the output gate's pre-activation at the column offsets
    `offs` = (z, x, g), `width` channels each; state pool float32 [slots, width]; out [T, width] = S_t * silu(g_t)."""
    _cuda(proj, out, s_pool)
    dt = proj.dtype
    _rows2d(proj, dt, "gru_scan: proj")
    if s_pool.dtype != torch.float32 or not s_pool.is_contiguous() or s_pool.dim() != 2 or s_pool.shape[1] != width or out.dtype != dt \
            or not out.is_contiguous() or tuple(out.shape) != (proj.shape[0], width):
        raise NativeError("gru_scan: the state pool must be contiguous float32 [slots, width], out contiguous [T, width] in the compute type")
    p = pcs_gru_params()
    p.proj, p.row_stride = proj.data_ptr(), proj.stride(0)
    p.z_off, p.x_off, p.g_off = offs
    p.width, p.out, p.s_pool = int(width), out.data_ptr(), s_pool.data_ptr()
    p.seq_slot, p.seq_pos0, p.seq_len, p.seq_off = (batch.seq_slot.data_ptr(), batch.seq_pos0.data_ptr(), batch.seq_len.data_ptr(),
                                                    batch.seq_off.data_ptr())
    p.n_seqs, p.n_tokens, p.max_len, p.dtype = batch.n_seqs, batch.n_tokens, batch.max_len, dtype_code(dt)
    _check(load().pcs_gru_scan(C.byref(p), _stream()), "pcs_gru_scan")
