"""ctypes binding of the C ABI in include/cc_b200.h.

There is NO CPU fallback: if libcc_b200.so is missing or does not export every declared symbol,
loading fails loudly.  On a machine without a GPU the library still loads (so the symbol table
can be checked) but every compute call returns CC_ERR_NO_DEVICE / CC_ERR_CUDA.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
import os

SO_PATH = Path(os.environ.get("CC_B200_LIB", PKG / "libcc_b200.so"))  # override: A/B builds in profiles/

ABI_VERSION = 1
CC_OK = 0
POLICY_EXTERNAL, POLICY_RECENT_GLOBAL, POLICY_L2, POLICY_HEAVY_HITTER, POLICY_HYBRID = range(5)
ATTN_MATH_FP32, ATTN_NAIVE_BF16 = 0, 1
PHASE_EVICT_FILL, PHASE_ATTEND, PHASE_SCORE, PHASE_ALL = 1, 2, 4, 7
FLAG_OVERLAP_PREDECESSOR = 1
FLAG_VIA_TOKEN_KERNEL = 2
HYB_FULL, HYB_WINDOW, HYB_HEAVY_HITTER, HYB_SPECIAL, HYB_PUNC = 1, 2, 4, 8, 16

_STATE_INTS = ("policy", "attn_mode", "n_kv_heads", "q_per_kv", "head_dim", "max_cache_length",
               "global_tokens", "recent_window", "history_window", "pos_heads", "cts_heads", "attn_thresholding")
_STATE_PTRS = ("k_cache", "v_cache", "pos", "mask", "cache_cts", "attn_history_num", "attn_history_denom",
               "attn_counter", "attn_history_sum", "key_norm", "hyb_strategy_bits", "hyb_recent_window", "hyb_heavy_budget",
               "special_mask", "punc_mask", "num_special", "num_punc", "sync_words")


class CcCacheState(C.Structure):
    _fields_ = [(n, C.c_int32) for n in _STATE_INTS] + [(n, C.c_void_p) for n in _STATE_PTRS]


class CcDecodeArgs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("q", "k_new", "v_new", "input_pos", "y", "fill_idx", "probs")] + [
        ("is_punc", C.c_int32), ("phases", C.c_int32), ("flags", C.c_int32), ("n_prefetch", C.c_int32)] + [
        (f"prefetch{i}_{f}", t) for i in range(3) for f, t in (("ptr", C.c_void_p), ("bytes", C.c_uint64))] + [
        ("is_punc_dev", C.c_void_p)]


class CcTpLink(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("world", "rank", "dim", "n_ops")] + [
        (n, C.c_void_p) for n in ("peer_buf", "peer_flag", "cta_done", "epoch")]


class CcTpArgs(C.Structure):
    _fields_ = [("link", C.POINTER(CcTpLink)), ("send_op", C.c_int32), ("recv_op", C.c_int32), ("recv_out", C.c_void_p)]


class CcPrefillAttnArgs(C.Structure):
    _fields_ = [f for t in "qkvy" for f in ((t, C.c_void_p), (f"{t}_stride_s", C.c_int64), (f"{t}_stride_h", C.c_int64))] + [
        (n, C.c_int32) for n in ("seq_len", "n_kv_heads", "q_per_kv", "head_dim", "attn_mode", "obs_len", "n_windows")] + [
        ("windows", C.c_int32 * 4), ("reserved0", C.c_int32)] + [
        (n, C.c_void_p) for n in ("col_sum", "obs_sum", "band_sum", "workspace")] + [("workspace_bytes", C.c_uint64)]


class CcTokenLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attention_norm", "wqkv", "bqkv", "wo", "ffn_norm", "w1", "w3", "w2")] + [
        ("attention_norm_eps", C.c_float), ("ffn_norm_eps", C.c_float), ("cache", CcCacheState),
        ("fill_idx", C.c_void_p), ("probs", C.c_void_p)]


class CcTokenModel(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "dim", "n_q_heads", "n_kv_heads", "head_dim", "intermediate", "vocab")] + [
        ("norm_eps", C.c_float), ("layers", C.POINTER(CcTokenLayer))] + [
        (n, C.c_void_p) for n in ("tok_embeddings", "norm", "output", "freqs_cis")] + [
        ("world", C.c_int32), ("rank", C.c_int32), ("scratch_peers", C.POINTER(C.c_uint64)), ("scratch_bytes", C.c_uint64)]


# every symbol include/cc_b200.h declares: name -> (restype, argtypes)
EXPORTS = {
    "cc_abi_version": (C.c_int, []),
    "cc_build_info": (C.c_char_p, []),
    "cc_last_error": (C.c_char_p, []),
    "cc_sync_words": (C.c_int, []),
    "cc_decode_step": (C.c_int, [C.POINTER(CcCacheState), C.POINTER(CcDecodeArgs), C.c_void_p]),
    "cc_decode_cluster_size": (C.c_int, [C.POINTER(CcCacheState)]),
    "cc_debug_set_trace": (None, [C.c_void_p]),
    "cc_key_norms": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "cc_prefill_gather": (C.c_int, [C.POINTER(CcCacheState), C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "cc_requantize_cache": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32] + [C.c_void_p] * 7),
    "cc_prefill_attention_workspace": (C.c_uint64, [C.c_int32] * 5),
    "cc_prefill_attention": (C.c_int, [C.POINTER(CcPrefillAttnArgs), C.c_void_p]),
    "cc_token_scratch_bytes": (C.c_uint64, [C.POINTER(CcTokenModel)]),
    "cc_token_plan_create": (C.c_int, [C.POINTER(CcTokenModel), C.POINTER(C.c_void_p)]),
    "cc_token_plan_destroy": (C.c_int, [C.c_void_p]),
    "cc_decode_token": (C.c_int, [C.c_void_p] * 7),
    "cc_token_buffer": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_uint64), C.POINTER(C.c_int32)]),
    "cc_token_set_trace": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cc_token_info": (C.c_int, [C.c_void_p] + [C.POINTER(C.c_int32)] * 4),
    "cc_rmsnorm_qkv_rope": (C.c_int, [C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                      C.c_int32, C.c_int32, C.POINTER(CcTpArgs), C.c_void_p]),
    "cc_gemv_residual": (C.c_int, [C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_int32, C.c_int32, C.POINTER(CcTpArgs), C.c_void_p]),
    "cc_rmsnorm_ffn_gate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_int32, C.c_int32, C.POINTER(CcTpArgs), C.c_void_p]),
}

_lib = None


class CcError(RuntimeError):
    pass


def load() -> C.CDLL:
    """Load the CUDA library; raises if it has not been built (python -m cold_compress_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not SO_PATH.exists():
        raise CcError(f"{SO_PATH} is missing: build it with `python -m cold_compress_b200.build` "
                      "(nvcc, sm_100a). There is no CPU or PyTorch fallback for the decode path.")
    lib = C.CDLL(str(SO_PATH))
    for name, (restype, argtypes) in EXPORTS.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
        fn.restype, fn.argtypes = restype, argtypes
    if lib.cc_abi_version() != ABI_VERSION:
        raise CcError(f"ABI mismatch: library {lib.cc_abi_version()} vs binding {ABI_VERSION}")
    _lib = lib
    return lib


def check(rc: int, what: str = "") -> int:
    if rc < 0:
        raise CcError(f"{what or 'cc call'} failed ({rc}): {load().cc_last_error().decode()}")
    return rc


# --------------------------------------------------------------------------- libcc_b200_seq.so (include/cc_b200_seq.h)
SEQ_SO_PATH = Path(os.environ.get("CC_B200_SEQ_LIB", PKG / "libcc_b200_seq.so"))
SEQ_ABI_VERSION = 4
DT_F32, DT_BF16 = 0, 1
SINK_NONE, SINK_LEARNED, SINK_ZERO = 0, 1, 2


class CcSeqAttn(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("q", "k_new", "v_new", "k_cache", "v_cache", "pos", "mask", "cache_cts",
                                          "input_pos", "y", "sink")] + [
        (n, C.c_int32) for n in ("T", "H", "G", "Dk", "Dv", "L", "window", "sink_mode", "cache_dtype", "y_dtype")] + [
        ("scale", C.c_float), ("append", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64),
        ("block", C.c_int32), ("keep_first", C.c_int32), ("softcap", C.c_float), ("dist_a", C.c_void_p), ("dist_b", C.c_void_p)]


class CcSeqGemv(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x_dtype", C.c_int32), ("in_norm_w", C.c_void_p), ("W", C.c_void_p), ("w_dtype", C.c_int32),
                ("bias", C.c_void_p), ("res", C.c_void_p), ("res_norm_w", C.c_void_p), ("alpha", C.c_float), ("eps", C.c_float),
                ("limit", C.c_float), ("slope", C.c_float), ("mode", C.c_int32), ("out", C.c_void_p), ("out_dtype", C.c_int32),
                ("N", C.c_int32), ("K", C.c_int32)]


GEMV_PLAIN, GEMV_RESIDUAL, GEMV_GLU = 0, 1, 2
_i32, _f32, _vp = C.c_int32, C.c_float, C.c_void_p
SEQ_EXPORTS = {
    "cc_seq_gemv": (C.c_int, [C.POINTER(CcSeqGemv), C.c_void_p]),
    "cc_seq_abi_version": (C.c_int, []),
    "cc_seq_last_error": (C.c_char_p, []),
    "cc_seq_embed": (C.c_int, [_vp] * 8 + [_i32, _i32, _f32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "cc_seq_qkv_prepare": (C.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32,
                                     _f32, _i32, _f32, _i32, _vp]),
    "cc_seq_attention": (C.c_int, [C.POINTER(CcSeqAttn), _vp]),
    "cc_seq_attention_decode": (C.c_int, [C.POINTER(CcSeqAttn), _vp]),
    "cc_seq_decode_workspace": (C.c_uint64, [_i32] * 5),
    "cc_seq_cache_append": (C.c_int, [C.POINTER(CcSeqAttn), _vp]),
    "cc_seq_residual_norm": (C.c_int, [_vp, _vp, _i32, _vp, _f32, _f32, _vp, _i32, _i32, _i32, _vp]),
    "cc_seq_clamped_glu": (C.c_int, [_vp, _vp, _i32, _i32, _f32, _f32, _i32, _i32, _vp]),
}

# ---- second part of the header: state-carrying layers (csrc/seq/mix_kernels.cu)
ACT_NONE, ACT_GELU_TANH, ACT_SILU, ACT_TANH, ACT_SIGMOID, ACT_RELU_SQ = range(6)
_i64 = C.c_int64


class CcSeqGatedNorm(C.Structure):
    _fields_ = [("x", _vp), ("a", _vp), ("lda", _i64), ("ga", _vp), ("ldga", _i64), ("ba", _vp),
                ("b", _vp), ("ldb", _i64), ("gb", _vp), ("ldgb", _i64), ("bb", _vp), ("w", _vp),
                ("h", _vp), ("h_act", _vp), ("act_dtype", _i32), ("rows", _vp), ("T", _i32), ("E", _i32), ("groups", _i32),
                ("eps", _f32), ("shift_state", _vp), ("shift_mu", _vp), ("hs_act", _vp), ("mix_state", _vp), ("mix_mu", _vp),
                ("mixes", _vp), ("n_mix", _i32)]


GEMV_MAX_JOBS = 6


class CcSeqGemvJob(C.Structure):
    _fields_ = [("x", _vp), ("W", _vp), ("out", _vp)] + [(n, _i32) for n in ("x_dtype", "kind", "off_gate", "off_up", "N", "K")]


class CcSeqGemvMulti(C.Structure):
    _fields_ = [("job", CcSeqGemvJob * GEMV_MAX_JOBS), ("n_jobs", _i32), ("w_dtype", _i32)]


class CcSeqLatentPrep(C.Structure):
    _fields_ = [("inp", _vp), ("ld", _i64)] + [(n, _i32) for n in ("off_q", "q_rank", "off_kv", "kv_rank", "rot_dim", "rot_dims")] + [
        (n, _vp) for n in ("wq", "wkv", "inv_freq", "input_pos", "cq", "krow", "vrow")] + [("dtype", _i32), ("T", _i32), ("eps", _f32),
                                                                                      ("interleaved", _i32)]


class CcSeqLatentExpand(C.Structure):
    _fields_ = [("kv_old", _vp), ("kv_new", _vp), ("ld_kv", _i64), ("lat_old", _vp), ("lat_new", _vp), ("ld_lat", _i64)] + [
        (n, _vp) for n in ("k_old", "v_old", "k_new", "v_new")] + [
        (n, _i32) for n in ("dtype", "n_old", "n_new", "H", "D", "V", "R", "kv_rank")]


class CcSeqLatentDecode(C.Structure):
    _fields_ = [(n, _vp) for n in ("q", "k_new", "k_cache", "pos", "mask", "cache_cts", "input_pos", "y")] + [
        (n, _i32) for n in ("H", "Dk", "C", "L", "cache_dtype", "y_dtype")] + [("scale", _f32), ("append", _i32),
                                                                               ("workspace", _vp), ("workspace_bytes", C.c_uint64),
                                                                               ("sink", _vp)]


class CcSeqWkv(C.Structure):
    _fields_ = [(n, _vp) for n in ("r", "k", "v", "wraw", "w0", "u", "state", "o")] + [(n, _i32) for n in ("T", "H", "D")]


class CcSeqMoeCombine(C.Structure):
    _fields_ = [(n, _vp) for n in ("ids", "wts", "slot", "y", "h", "shared", "sg")] + [("ld_sg", _i64), ("out", _vp)] + [
        (n, _i32) for n in ("T", "E", "top", "n_real")]


SEQ_EXPORTS.update({
    "cc_seq_embed_rows": (C.c_int, [_vp, _vp, _i32, _vp, _i32, _i32, _f32, _vp]),
    "cc_seq_gated_group_norm": (C.c_int, [C.POINTER(CcSeqGatedNorm), _vp]),
    "cc_seq_token_shift": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _vp, _i32, _i32, _i32, _vp]),
    "cc_seq_gated_unit": (C.c_int, [_vp, _i64, _i32, _i32, _vp, _i32, _i32, _i32, _i32, _vp]),
    "cc_seq_latent_prepare": (C.c_int, [C.POINTER(CcSeqLatentPrep), _vp]),
    "cc_seq_rope_heads": (C.c_int, [_vp, _i64, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i64, _i32, _i32, _vp]),
    "cc_seq_latent_expand": (C.c_int, [C.POINTER(CcSeqLatentExpand), _vp]),
    "cc_seq_latent_decode": (C.c_int, [C.POINTER(CcSeqLatentDecode), _vp]),
    "cc_seq_latent_decode_workspace": (C.c_uint64, [_i32, _i32, _i32]),
    "cc_seq_gemv_multi": (C.c_int, [C.POINTER(CcSeqGemvMulti), _vp]),
    "cc_seq_head_gate": (C.c_int, [_vp, _i32, _vp, _i64, _i32, _i32, _i32, _vp]),
    "cc_seq_head_gemv": (C.c_int, [_vp, _i32, _vp, _i32, _i64, _vp, _i32, _i64, _vp, _i32, _i32, _i32, _vp]),
    "cc_seq_wkv": (C.c_int, [C.POINTER(CcSeqWkv), _vp]),
    "cc_seq_head_norm_gate": (C.c_int, [_vp, _vp, _i64, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _vp]),
    "cc_seq_moe_route": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp]),
    "cc_seq_moe_group": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "cc_seq_gather_rows": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "cc_seq_moe_expert_tokens": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "cc_seq_moe_combine": (C.c_int, [C.POINTER(CcSeqMoeCombine), _vp]),
})

# ---- third part of the header: post-sum norms, short convolutions, matrix-state scans, rotations (csrc/seq/scan_kernels.cu)
class CcSeqSumNorm(C.Structure):
    _fields_ = [("x", _vp), ("y", _vp), ("ldy", _i64), ("y_norm_w", _vp), ("y2", _vp), ("ldy2", _i64), ("y2_norm_w", _vp),
                ("y_coef", _f32), ("y_scale", _vp), ("w", _vp), ("alpha", _f32), ("eps", _f32), ("gain_offset", _f32),
                ("center", _i32), ("out", _vp), ("stack", _vp), ("stack_stride", _i64), ("n_prev", _i32), ("coef", _vp),
                ("mix", _vp), ("out_act", _vp), ("act_dtype", _i32), ("rows", _vp), ("T", _i32), ("E", _i32)]


class CcSeqSsdScan(C.Structure):
    _fields_ = [("x", _vp), ("ldx", _i64), ("B", _vp), ("C", _vp), ("ldbc", _i64), ("dt_raw", _vp), ("lddt", _i64),
                ("dt_bias", _vp), ("A_log", _vp), ("D", _vp), ("state", _vp), ("y", _vp)] + [
        (n, _i32) for n in ("T", "H", "G", "N", "V")]


class CcSeqDeltaScan(C.Structure):
    _fields_ = [("q", _vp), ("k", _vp), ("ldqk", _i64), ("v", _vp), ("ldv", _i64), ("beta_raw", _vp), ("ldb", _i64),
                ("a_raw", _vp), ("lda", _i64), ("dt_bias", _vp), ("A_log", _vp), ("state", _vp), ("o", _vp)] + [
        (n, _i32) for n in ("T", "H", "G", "D", "V")] + [("q_scale", _f32), ("unit_eps", _f32), ("qk", _vp), ("prepared", _i32)]


class CcSeqQkvRope(C.Structure):
    _fields_ = [("inp", _vp), ("ld", _i64)] + [(n, _i32) for n in ("off_q", "off_k", "off_v", "H", "G", "Dk", "Dv")] + [
        ("q_norm_w", _vp), ("k_norm_w", _vp), ("eps", _f32), ("rot_dims", _i32), ("interleaved", _i32), ("inv_freq", _vp),
        ("v_inv_freq", _vp), ("input_pos", _vp), ("q_out", _vp), ("k_out", _vp), ("v_out", _vp), ("out_dtype", _i32), ("T", _i32)]


SEQ_EXPORTS.update({
    "cc_seq_sum_norm": (C.c_int, [C.POINTER(CcSeqSumNorm), _vp]),
    "cc_seq_short_conv": (C.c_int, [_vp, _i64, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp]),
    "cc_seq_ssd_scan": (C.c_int, [C.POINTER(CcSeqSsdScan), _vp]),
    "cc_seq_delta_scan": (C.c_int, [C.POINTER(CcSeqDeltaScan), _vp]),
    "cc_seq_delta_prepare": (C.c_int, [C.POINTER(CcSeqDeltaScan), _vp, _vp, _vp, _vp, _vp, _vp]),
    "cc_seq_gated_rms_groups": (C.c_int, [_vp, _vp, _i64, _i32, _i32, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _f32, _vp]),
    "cc_seq_qkv_rope": (C.c_int, [C.POINTER(CcSeqQkvRope), _vp]),
    "cc_seq_turn_heads_gate": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _f32, _vp, _i64, _vp, _i32, _i32, _i32, _i32, _vp]),
    "cc_seq_softcap": (C.c_int, [_vp, _i64, _f32, _vp]),
})

# ---- fourth part of the header: sublayers on norms of one stream, whole-row q / k norms, polynomial activation (csrc/seq/par_kernels.cu)
PAR_MAX_OUT = 4


class CcSeqParNorm(C.Structure):
    _fields_ = [("x", _vp), ("a", _vp), ("lda", _i64), ("b", _vp), ("ldb", _i64), ("add", _vp), ("rinv", _vp), ("x_out", _vp), ("tail", _vp),
                ("gain", _vp * PAR_MAX_OUT), ("conv_w", _vp * PAR_MAX_OUT), ("out", _vp * PAR_MAX_OUT)] + [
        (n, _i32) for n in ("n_out", "act_dtype", "T", "E", "taps")] + [("eps", _f32)]


class CcSeqQkRowNorm(C.Structure):
    _fields_ = [("inp", _vp), ("ld", _i64)] + [(n, _i32) for n in ("off_q", "nq", "off_k", "nk", "off_v", "nv")] + [
        (n, _vp) for n in ("wq", "wk", "q_out", "k_out", "v_out")] + [("out_dtype", _i32), ("T", _i32), ("eps", _f32)]


SEQ_EXPORTS.update({
    "cc_seq_par_norm": (C.c_int, [C.POINTER(CcSeqParNorm), _vp]),
    "cc_seq_qk_row_norm": (C.c_int, [C.POINTER(CcSeqQkRowNorm), _vp]),
    "cc_seq_poly_norm": (C.c_int, [_vp, _i64, _vp, _vp, _i32, _i32, _i32, _f32, _vp]),
})

_seq_lib = None


def load_seq() -> C.CDLL:
    """Load the sequence-kernel library; raises if it has not been built (python -m cold_compress_b200.build)."""
    global _seq_lib
    if _seq_lib is not None:
        return _seq_lib
    if not SEQ_SO_PATH.exists():
        raise CcError(f"{SEQ_SO_PATH} is missing: build it with `python -m cold_compress_b200.build --only=seq` "
                      "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these kernels.")
    lib = C.CDLL(str(SEQ_SO_PATH))
    for name, (restype, argtypes) in SEQ_EXPORTS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = restype, argtypes
    if lib.cc_seq_abi_version() != SEQ_ABI_VERSION:
        raise CcError(f"ABI mismatch: library {lib.cc_seq_abi_version()} vs binding {SEQ_ABI_VERSION}")
    _seq_lib = lib
    return lib


def check_seq(rc: int, what: str = "") -> int:
    if rc < 0:
        raise CcError(f"{what or 'cc_seq call'} failed ({rc}): {load_seq().cc_seq_last_error().decode()}")
    return rc
