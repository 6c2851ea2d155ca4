"""ctypes binding of libdllama_b200_cuda.so (C ABI declared in include/dllama_b200.h).

The library is built in-tree by ``build.py`` and MUST be present on a GPU box: every op fails
loudly (``NativeLibraryError``) instead of silently falling back to PyTorch.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_LIB_PATH = os.path.join(_PKG, "lib", "libdllama_b200_cuda.so")
HOST_LIB_PATH = os.path.join(_PKG, "lib", "libdllama_b200_host.so")
LAYERS_LIB_PATH = os.path.join(_PKG, "lib", "libdllama_b200_layers.so")

DL_MAX_PEERS = 8
EPI_STORE, EPI_QKV_ROPE, EPI_SILU_MUL, EPI_DENSE = 0, 1, 2, 3


class NativeLibraryError(RuntimeError):
    pass


class DlEpilogue(C.Structure):
    """Mirror of ``DlEpilogue`` in include/dllama_b200.h (field order and types must match)."""
    _fields_ = [
        ("kind", C.c_int),
        ("dst", C.c_void_p * DL_MAX_PEERS),
        ("n_dst", C.c_int),
        ("ld", C.c_int),
        ("dst_off", C.c_longlong),
        ("q80_roundtrip", C.c_int),
        ("residual", C.c_void_p),
        ("residual_ld", C.c_int),
        ("flag", C.c_void_p * DL_MAX_PEERS),
        ("step_counter", C.c_void_p),
        ("flag_mul", C.c_uint32),
        ("flag_add", C.c_uint32),
        ("cta_counter", C.c_void_p),
        ("q_out", C.c_void_p),
        ("q_dim", C.c_int),
        ("kv_dim", C.c_int),
        ("head_size", C.c_int),
        ("rope_freqs", C.c_void_p),
        ("pos", C.c_void_p),
        ("slot", C.c_void_p),
        ("block_table", C.c_void_p),
        ("max_pages", C.c_int),
        ("page_size", C.c_int),
        ("n_kv_heads", C.c_int),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("kv_f32", C.c_int),
        ("xq_out", C.c_void_p),
        ("xh_out", C.c_void_p),
        ("out_mcap", C.c_int),
        ("act_gelu", C.c_int),
        ("ll", C.c_int),
        ("dense_op", C.c_int),
        ("dense_param", C.c_float),
        ("dense_aux", C.c_void_p),
        ("dense_aux_ld", C.c_longlong),
        ("dense_param2", C.c_float),
    ]


class DlNormProlog(C.Structure):
    """Mirror of ``DlNormProlog`` in include/dllama_b200.h."""
    _fields_ = [
        ("x_in", C.c_void_p),
        ("x_out", C.c_void_p),
        ("partials", C.c_void_p),
        ("n_src", C.c_int),
        ("src_stride", C.c_longlong),
        ("flags", C.c_void_p),
        ("step_counter", C.c_void_p),
        ("flag_mul", C.c_uint32),
        ("flag_add", C.c_uint32),
        ("norm_w", C.c_void_p),
        ("eps", C.c_float),
        ("ll", C.c_int),
    ]


class DlDecodeLayer(C.Structure):
    """Mirror of ``DlDecodeLayer`` (per-layer device pointers of the persistent decode kernel)."""
    _fields_ = [("qkv", C.c_void_p), ("wo", C.c_void_p), ("w13", C.c_void_p), ("w2", C.c_void_p),
                ("rms_att", C.c_void_p), ("rms_ffn", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


class DlDecodeArgs(C.Structure):
    """Mirror of ``DlDecodeArgs`` in include/dllama_b200.h (field order and types must match)."""
    _fields_ = [
        ("n_layers", C.c_int), ("dim", C.c_int), ("q_dim", C.c_int), ("kv_dim", C.c_int), ("hid", C.c_int),
        ("vocab_loc", C.c_int), ("vocab", C.c_int), ("head_size", C.c_int), ("n_heads", C.c_int),
        ("n_kv_heads", C.c_int),
        ("rank", C.c_int), ("world", C.c_int),
        ("eps", C.c_float),
        ("act_gelu", C.c_int),
        ("q80_sync", C.c_int),
        ("layers", C.c_void_p),
        ("rms_final", C.c_void_p),
        ("wcls", C.c_void_p),
        ("embedding", C.c_void_p),
        ("rope_freqs", C.c_void_p),
        ("M", C.c_int), ("row0", C.c_int),
        ("tokens", C.c_void_p),
        ("pos", C.c_void_p),
        ("slot", C.c_void_p),
        ("block_table", C.c_void_p),
        ("max_pages", C.c_int),
        ("x", C.c_void_p * 2),
        ("q", C.c_void_p),
        ("h", C.c_void_p),
        ("att_o", C.c_void_p),
        ("att_ml", C.c_void_p),
        ("max_splits", C.c_int),
        ("att_splits", C.c_int),
        ("cta_best", C.c_void_p),
        ("grid_bar", C.c_void_p),
        ("step_counter", C.c_void_p),
        ("ll_att", C.c_void_p * DL_MAX_PEERS),
        ("ll_ffn", C.c_void_p * DL_MAX_PEERS),
        ("ll_tok", C.c_void_p * DL_MAX_PEERS),
        ("logits", C.c_void_p * DL_MAX_PEERS),
        ("flag_logits", C.c_void_p * DL_MAX_PEERS),
        ("greedy", C.c_int),
        ("tokens_out", C.c_void_p),
        ("advance", C.c_int),
        ("history", C.c_void_p),
        ("history_cap", C.c_int),
        ("timeout_ns", C.c_ulonglong),
        ("debug", C.c_void_p),
        ("trace", C.c_void_p),
        ("trace_cta", C.c_int),
        ("dbg", C.c_int),
        ("pf_dist", C.c_int),
    ]


_cuda = None


def cuda_lib():
    """Load (once) and return the CUDA library with argtypes set."""
    global _cuda
    if _cuda is not None:
        return _cuda
    if not os.path.exists(CUDA_LIB_PATH):
        raise NativeLibraryError(
            f"{CUDA_LIB_PATH} is missing: run `python build.py` (nvcc, sm_100a) before using GPU ops")
    L = C.CDLL(CUDA_LIB_PATH)
    vp, i32, i64, u32, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_uint32, C.c_float
    L.dl_last_error.restype = C.c_char_p
    L.dl_device_sm_count.restype = i32
    L.dl_q40t_bytes.restype = i64
    L.dl_q40t_bytes.argtypes = [i32, i32]
    L.dl_q40_repack.argtypes = [vp, i32, i32, vp, i32, i32, i32, vp]
    L.dl_q40t_dequant.argtypes = [vp, i32, i32, vp, vp]
    L.dl_reduce_norm_quant.argtypes = [vp, vp, vp, i32, i32, vp, vp, u32, u32, i32, vp, f32, i32, i32, i32,
                                       vp, vp, vp, i32, vp]
    L.dl_quant_q80.argtypes = [vp, i32, i32, i32, vp, vp, vp]
    L.dl_embedding.argtypes = [vp, vp, vp, i32, i32, vp, vp]
    L.dl_sample_rows.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, vp]
    L.dl_gemm_f32.argtypes = [vp, i32, i32, i64, vp, i32, i32, vp, i32, i32, vp]
    L.dl_gemv_q40.argtypes = [vp, i32, i32, vp, i32, i32, i32, i32, C.POINTER(DlNormProlog), C.POINTER(DlEpilogue), i32, vp]
    L.dl_gemv_q40_smem_bytes.restype = i64
    L.dl_gemv_q40_smem_bytes.argtypes = [i32, i32, i32]
    L.dl_gemm_q40_tc.argtypes = [vp, i32, i32, vp, i32, i32, i32, C.POINTER(DlEpilogue), i32, vp]
    L.dl_wh_bytes.restype = i64
    L.dl_wh_bytes.argtypes = [i32, i32]
    L.dl_q40t_to_wh.argtypes = [vp, i32, i32, vp, vp]
    L.dl_gemm_wh_tc.argtypes = [vp, i32, i32, vp, i32, i32, C.POINTER(DlEpilogue), i32, i32, vp]
    L.dl_attention_scratch_bytes.restype = i64
    L.dl_attention_scratch_bytes.argtypes = [i32, i32, i32, i32]
    L.dl_attention.argtypes = [vp, i32, i32, i32, i32, vp, vp, i32, vp, vp, vp, i32, i32, i32, vp, vp, vp,
                               i32, vp, vp, i32, vp]
    L.dl_attention_prefill.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, i32, i32, vp, vp, vp, i32, vp, i32, vp]
    L.dl_attention_prefill_tc.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, i32, i32, vp, vp, vp, i32, vp, i32, i32, vp]
    L.dl_argmax.argtypes = [vp, i32, i32, i32, vp, vp, i32, vp, u32, u32, vp, vp, i32, vp, i32, vp]
    L.dl_argmax_scratch_bytes.restype = i64
    L.dl_argmax_scratch_bytes.argtypes = [i32]
    L.dl_wait_flags.argtypes = [vp, i32, vp, u32, u32, vp]
    L.dl_ipc_alloc.argtypes = [C.POINTER(vp), i64, vp]
    L.dl_ipc_open.argtypes = [vp, C.POINTER(vp)]
    L.dl_ipc_close.argtypes = [vp]
    L.dl_ipc_free.argtypes = [vp]
    L.dl_peer_barrier.argtypes = [C.POINTER(vp), vp, i32, i32, u32, vp]
    L.dl_f32_rope_kv.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, i32, vp, vp, vp, i32, vp]
    L.dl_f32_silu_mul.argtypes = [vp, vp, vp, i64, i32, vp]
    L.dl_f32_push.argtypes = [vp, i32, i32, i32, C.POINTER(vp), i32, i64, i32, C.POINTER(vp), vp, u32, u32, vp, vp]
    for name in ("dl_f32_rope_kv", "dl_f32_silu_mul", "dl_f32_push"):
        getattr(L, name).restype = i32
    L.dl_decode_mega_supported.argtypes = [C.POINTER(DlDecodeArgs), i32]
    L.dl_decode_mega_supported.restype = i32
    L.dl_decode_mega.argtypes = [C.POINTER(DlDecodeArgs), i32, vp]
    L.dl_decode_mega.restype = i32
    L.dl_decode_mega_plan.argtypes = [i32, i32, i32, i32, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]
    L.dl_decode_mega_plan.restype = i32
    for name in ("dl_q40_repack", "dl_q40t_dequant", "dl_reduce_norm_quant", "dl_quant_q80", "dl_embedding",
                 "dl_sample_rows", "dl_gemm_f32", "dl_gemv_q40", "dl_gemm_q40_tc", "dl_q40t_to_wh", "dl_gemm_wh_tc", "dl_attention", "dl_attention_prefill", "dl_attention_prefill_tc", "dl_argmax", "dl_ipc_alloc", "dl_ipc_open",
                 "dl_ipc_close", "dl_ipc_free", "dl_peer_barrier", "dl_wait_flags"):
        getattr(L, name).restype = i32
    _cuda = L
    return L


def check(rc: int, what: str = ""):
    if rc != 0:
        msg = cuda_lib().dl_last_error().decode("utf-8", "replace")
        raise NativeLibraryError(f"{what} failed ({rc}): {msg}")


# ---- libdllama_b200_layers.so: kernels of layer-list models (dense weights, latent and windowed attention, Mamba-2,
# ---- hyper-connections, routed experts)
T_F32, T_BF16 = 0, 1
DENSE_STORE, DENSE_RELU2, DENSE_SIGMOID_MUL, DENSE_SOFTCAP, DENSE_SILU, DENSE_GLU_CLAMP = 0, 1, 2, 3, 4, 5
DENSE_MUL, DENSE_XIELU, DENSE_ROWGATE_ADD, DENSE_GLU_SILU = 6, 7, 8, 9


class DlDenseArgs(C.Structure):
    """Mirror of ``DlDenseArgs`` in include/dllama_b200.h."""
    _fields_ = [("W", C.c_void_p), ("wtype", C.c_int), ("ldw", C.c_longlong), ("w_bs", C.c_longlong),
                ("X", C.c_void_p), ("ldx", C.c_longlong), ("x_bs", C.c_longlong),
                ("Y", C.c_void_p), ("ldy", C.c_longlong), ("y_bs", C.c_longlong),
                ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("batch", C.c_int),
                ("round_x", C.c_int), ("epi", C.c_int),
                ("aux", C.c_void_p), ("ld_aux", C.c_longlong), ("aux_bs", C.c_longlong),
                ("param", C.c_float), ("param2", C.c_float)]


class DlNormArgs(C.Structure):
    """Mirror of ``DlNormArgs``."""
    _fields_ = [("x", C.c_void_p), ("ldx", C.c_longlong), ("gate", C.c_void_p), ("ld_gate", C.c_longlong),
                ("w", C.c_void_p), ("y", C.c_void_p), ("ldy", C.c_longlong), ("rows", C.c_void_p),
                ("M", C.c_int), ("dim", C.c_int), ("groups", C.c_int), ("eps", C.c_float),
                ("plus_one", C.c_int), ("accumulate", C.c_int)]


class DlLatentKvArgs(C.Structure):
    """Mirror of ``DlLatentKvArgs``."""
    _fields_ = [("kv", C.c_void_p), ("ld", C.c_longlong), ("norm_w", C.c_void_p), ("eps", C.c_float),
                ("rank", C.c_int), ("rot", C.c_int), ("rope_dims", C.c_int), ("freqs", C.c_void_p),
                ("pos", C.c_void_p), ("slot", C.c_void_p), ("block_table", C.c_void_p),
                ("max_pages", C.c_int), ("page_size", C.c_int), ("cache", C.c_void_p), ("ctype", C.c_int),
                ("interleaved", C.c_int)]


class DlLatentAttnArgs(C.Structure):
    """Mirror of ``DlLatentAttnArgs``."""
    _fields_ = [("q_lat", C.c_void_p), ("q", C.c_void_p), ("ldq", C.c_longlong), ("q_head_stride", C.c_int),
                ("q_rot_offset", C.c_int), ("out", C.c_void_p), ("n_heads", C.c_int), ("rank", C.c_int),
                ("rot", C.c_int), ("scale", C.c_float), ("pos", C.c_void_p), ("slot", C.c_void_p),
                ("block_table", C.c_void_p), ("max_pages", C.c_int), ("page_size", C.c_int),
                ("cache", C.c_void_p), ("ctype", C.c_int),
                ("window", C.c_int), ("sink", C.c_void_p), ("gate", C.c_void_p), ("ld_gate", C.c_longlong)]


class DlLatentTiles(C.Structure):
    """Mirror of ``DlLatentTiles``."""
    _fields_ = [("tile_rows", C.c_void_p), ("n_tiles", C.c_int), ("rq", C.c_int), ("n_splits", C.c_int),
                ("partial", C.c_void_p), ("d_pad", C.c_int)]


class DlMambaBatch(C.Structure):
    """Mirror of ``DlMambaBatch``."""
    _fields_ = [("pos", C.c_void_p), ("row_seq", C.c_void_p), ("seq_start", C.c_void_p), ("seq_rows", C.c_void_p),
                ("seq_slot", C.c_void_p), ("seq_pos0", C.c_void_p)]


class DlMambaScanArgs(C.Structure):
    """Mirror of ``DlMambaScanArgs``."""
    _fields_ = [("xbc", C.c_void_p), ("ld_xbc", C.c_longlong), ("dt", C.c_void_p), ("ld_dt", C.c_longlong),
                ("dt_bias", C.c_void_p), ("A_log", C.c_void_p), ("D", C.c_void_p),
                ("y", C.c_void_p), ("ld_y", C.c_longlong), ("ssm_state", C.c_void_p),
                ("n_heads", C.c_int), ("vdim", C.c_int), ("state", C.c_int), ("groups", C.c_int)]


class DlMambaChunks(C.Structure):
    """Mirror of ``DlMambaChunks``."""
    _fields_ = [("chunk_seq", C.c_void_p), ("chunk_off", C.c_void_p), ("n_chunks", C.c_int), ("chunk", C.c_int),
                ("state", C.c_void_p), ("decay", C.c_void_p), ("cum", C.c_void_p)]


class DlHyperArgs(C.Structure):
    """Mirror of ``DlHyperArgs``."""
    _fields_ = [("x", C.c_void_p), ("ldx", C.c_longlong), ("streams", C.c_int), ("dim", C.c_int), ("M", C.c_int),
                ("y", C.c_void_p), ("ldy", C.c_longlong), ("mix", C.c_void_p), ("w_out", C.c_void_p), ("mult", C.c_float),
                ("w_in", C.c_void_p), ("norm_w", C.c_void_p), ("eps", C.c_float), ("rows", C.c_void_p),
                ("h", C.c_void_p), ("ldh", C.c_longlong), ("u_out", C.c_void_p)]


class DlWindowKvArgs(C.Structure):
    """Mirror of ``DlWindowKvArgs``."""
    _fields_ = [("k", C.c_void_p), ("ld", C.c_longlong), ("q", C.c_void_p), ("ldq", C.c_longlong), ("q_heads", C.c_int),
                ("kv_heads", C.c_int), ("dim", C.c_int), ("rope_dims", C.c_int),
                ("freqs", C.c_void_p), ("rope_scale", C.c_float),
                ("pos", C.c_void_p), ("slot", C.c_void_p), ("block_table", C.c_void_p),
                ("max_pages", C.c_int), ("page_size", C.c_int), ("cache", C.c_void_p), ("ctype", C.c_int),
                ("v", C.c_void_p), ("ldv", C.c_longlong), ("vdim", C.c_int), ("qk_norm", C.c_int), ("eps", C.c_float),
                ("rope_half", C.c_int), ("talk", C.c_void_p), ("q_mixed", C.c_void_p), ("ld_qm", C.c_longlong)]


class DlWindowAttnArgs(C.Structure):
    """Mirror of ``DlWindowAttnArgs``."""
    _fields_ = [("q", C.c_void_p), ("ldq", C.c_longlong), ("out", C.c_void_p), ("ldo", C.c_longlong),
                ("heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("rope_dims", C.c_int),
                ("scale", C.c_float), ("softcap", C.c_float), ("window", C.c_int),
                ("pos", C.c_void_p), ("slot", C.c_void_p), ("block_table", C.c_void_p),
                ("max_pages", C.c_int), ("page_size", C.c_int), ("cache", C.c_void_p), ("ctype", C.c_int),
                ("vdim", C.c_int), ("chunk", C.c_int), ("sink", C.c_void_p), ("key_heads", C.c_int)]


class DlConvArgs(C.Structure):
    """Mirror of ``DlConvArgs``."""
    _fields_ = [("in_", C.c_void_p), ("ld", C.c_longlong), ("in_off", C.c_int),
                ("w", C.c_void_p), ("bias", C.c_void_p), ("wtype", C.c_int), ("conv_state", C.c_void_p),
                ("out", C.c_void_p), ("ld_out", C.c_longlong),
                ("channels", C.c_int), ("taps", C.c_int), ("act", C.c_int), ("residual", C.c_int)]


class DlLightningArgs(C.Structure):
    """Mirror of ``DlLightningArgs``."""
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
                ("ldq", C.c_longlong), ("ldk", C.c_longlong), ("ldv", C.c_longlong),
                ("decay", C.c_void_p), ("y", C.c_void_p), ("ld_y", C.c_longlong), ("state", C.c_void_p),
                ("n_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int)]


class DlMoeSelectArgs(C.Structure):
    """Mirror of ``DlMoeSelectArgs``."""
    _fields_ = [("z", C.c_void_p), ("ldz", C.c_longlong), ("M", C.c_int), ("experts", C.c_int), ("top", C.c_int),
                ("groups", C.c_int), ("keep", C.c_int), ("group_top", C.c_int), ("renorm", C.c_int),
                ("sel", C.c_void_p), ("wgt", C.c_void_p), ("score", C.c_int), ("scale", C.c_float),
                ("bias", C.c_void_p)]


class DlMoeArgs(C.Structure):
    """Mirror of ``DlMoeArgs``."""
    _fields_ = [("w_up", C.c_void_p), ("w_down", C.c_void_p), ("wtype", C.c_int),
                ("width", C.c_int), ("ff", C.c_int), ("top", C.c_int), ("M", C.c_int), ("round_x", C.c_int),
                ("x", C.c_void_p), ("ldx", C.c_longlong), ("sel", C.c_void_p), ("wgt", C.c_void_p),
                ("act", C.c_void_p), ("y", C.c_void_p), ("ldy", C.c_longlong), ("w_gate", C.c_void_p), ("limit", C.c_float),
                ("gate_act", C.c_int)]


class DlMoePlanArgs(C.Structure):
    """Mirror of ``DlMoePlanArgs``."""
    _fields_ = [("sel", C.c_void_p), ("M", C.c_int), ("top", C.c_int), ("experts", C.c_int), ("cap", C.c_int),
                ("cnt", C.c_void_p), ("grp", C.c_void_p), ("slot_row", C.c_void_p), ("pair_pos", C.c_void_p)]


_layers = None


def layers_lib():
    """Load (once) and return the layer-list model library with argtypes set."""
    global _layers
    if _layers is not None:
        return _layers
    if not os.path.exists(LAYERS_LIB_PATH):
        raise NativeLibraryError(
            f"{LAYERS_LIB_PATH} is missing: run `python build.py layers` (nvcc, sm_100a) before using GPU ops")
    L = C.CDLL(LAYERS_LIB_PATH)
    vp, i32, i64, u32 = C.c_void_p, C.c_int, C.c_longlong, C.c_uint32
    L.dl_last_error.restype = C.c_char_p
    L.dl_device_sm_count.restype = i32
    L.dl_dense.argtypes = [C.POINTER(DlDenseArgs), vp]
    L.dl_embed_rows.argtypes = [vp, i32, vp, vp, i32, i32, C.c_float, i32, vp]
    L.dl_rms_norm.argtypes = [C.POINTER(DlNormArgs), vp]
    L.dl_latent_kv_write.argtypes = [C.POINTER(DlLatentKvArgs), i32, vp]
    L.dl_rope_rows.argtypes = [vp, i64, i32, i32, i32, i32, i32, vp, vp, i32, C.c_float, vp]
    L.dl_latent_attention.argtypes = [C.POINTER(DlLatentAttnArgs), i32, vp]
    L.dl_latent_attention_tc.argtypes = [C.POINTER(DlLatentAttnArgs), C.POINTER(DlLatentTiles), vp]
    L.dl_latent_attention_tc_supported.argtypes = [i32, i32, i32, i32, i32]
    L.dl_latent_attention_tc_supported.restype = i32
    L.dl_latent_tc_partial_floats.argtypes = [i32, i32, i32]
    L.dl_latent_tc_partial_floats.restype = i64
    L.dl_hyper_step.argtypes = [C.POINTER(DlHyperArgs), vp]
    L.dl_window_kv_write.argtypes = [C.POINTER(DlWindowKvArgs), i32, vp]
    L.dl_window_attention.argtypes = [C.POINTER(DlWindowAttnArgs), i32, vp]
    L.dl_moe_select.argtypes = [C.POINTER(DlMoeSelectArgs), vp]
    L.dl_moe_rows.argtypes = [C.POINTER(DlMoeArgs), vp]
    L.dl_moe_plan.argtypes = [C.POINTER(DlMoePlanArgs), vp]
    L.dl_moe_combine.argtypes = [vp, i64, vp, vp, i32, i32, i32, vp, i64, vp]
    L.dl_xh_gather_rows.argtypes = [vp, i64, vp, i32, i32, i32, vp, vp]
    L.dl_gemm_wh_tc_grouped.argtypes = [vp, i64, i32, vp, i32, i32, vp, i32, i32, C.POINTER(DlEpilogue), i32, vp]
    L.dl_window_tc_rows.argtypes = [i32, i32]
    L.dl_window_attention_tc_supported.argtypes = [i32, i32, i32, i32, i32]
    L.dl_window_attention_tc.argtypes = [C.POINTER(DlWindowAttnArgs), vp, i32, i32, i32, vp, vp]
    L.dl_window_tc_partial_floats.argtypes = [i32, i32, i32, i32]
    L.dl_window_tc_partial_floats.restype = i64
    L.dl_talk_attention_tc_supported.argtypes = [i32, i32, i32, i32, i32, i32]
    L.dl_talk_attention_tc.argtypes = [C.POINTER(DlWindowAttnArgs), vp, i32, i32, i32, vp, vp]
    L.dl_talk_tc_partial_floats.argtypes = [i32, i32, i32, i32, i32]
    L.dl_talk_tc_tile_rows.argtypes = [i32, i32, i32, i32, i32, i32]
    L.dl_talk_tc_partial_floats.restype = i64
    L.dl_mamba_conv.argtypes = [C.POINTER(DlMambaBatch), i32, i32, vp, i64, i32, vp, vp, i32, vp, vp, i32, i32, vp]
    L.dl_mamba_scan.argtypes = [C.POINTER(DlMambaBatch), i32, C.POINTER(DlMambaScanArgs), vp]
    L.dl_mamba_scan_chunked.argtypes = [C.POINTER(DlMambaBatch), C.POINTER(DlMambaScanArgs), C.POINTER(DlMambaChunks), vp]
    L.dl_mamba_scan_chunked_supported.argtypes = [i32, i32]
    L.dl_mamba_scan_chunked_supported.restype = i32
    L.dl_causal_conv.argtypes = [C.POINTER(DlMambaBatch), i32, i32, C.POINTER(DlConvArgs), vp]
    L.dl_poly_norm.argtypes = [vp, i64, vp, i64, i32, i32, vp, C.c_float, vp]
    L.dl_lightning_scan.argtypes = [C.POINTER(DlMambaBatch), i32, C.POINTER(DlLightningArgs), vp]
    L.dl_lightning_scan_chunked.argtypes = [C.POINTER(DlMambaBatch), i32, i32, C.POINTER(DlLightningArgs), vp, vp]
    L.dl_lightning_scan_chunked_supported.argtypes = [i32, i32]
    L.dl_lightning_scan_chunked_supported.restype = i32
    L.dl_lightning_chunk_floats.argtypes = [i32, i32, i32, i32, i32]
    L.dl_lightning_chunk_floats.restype = i64
    L.dl_wh_bytes.restype = i64
    L.dl_wh_bytes.argtypes = [i32, i32]
    L.dl_wh_from_dense.argtypes = [vp, i32, i32, i64, vp, vp]
    L.dl_xh_from_rows.argtypes = [vp, i64, i32, i32, i32, vp, vp]
    L.dl_gemm_wh_tc.argtypes = [vp, i32, i32, vp, i32, i32, C.POINTER(DlEpilogue), i32, i32, vp]
    L.dl_sample_rows.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, vp]
    L.dl_argmax.argtypes = [vp, i32, i32, i32, vp, vp, i32, vp, u32, u32, vp, vp, i32, vp, i32, vp]
    L.dl_argmax_scratch_bytes.restype = i64
    L.dl_argmax_scratch_bytes.argtypes = [i32]
    for name in ("dl_dense", "dl_embed_rows", "dl_rms_norm", "dl_latent_kv_write", "dl_rope_rows", "dl_latent_attention", "dl_latent_attention_tc",
                 "dl_mamba_conv", "dl_mamba_scan", "dl_mamba_scan_chunked", "dl_sample_rows", "dl_argmax", "dl_wh_from_dense", "dl_xh_from_rows",
                 "dl_gemm_wh_tc", "dl_hyper_step", "dl_window_kv_write", "dl_window_attention", "dl_moe_select", "dl_moe_rows", "dl_moe_plan",
                 "dl_moe_combine", "dl_xh_gather_rows", "dl_gemm_wh_tc_grouped", "dl_window_tc_rows", "dl_window_attention_tc_supported",
                 "dl_window_attention_tc", "dl_talk_attention_tc_supported", "dl_talk_attention_tc", "dl_talk_tc_tile_rows", "dl_causal_conv", "dl_poly_norm", "dl_lightning_scan", "dl_lightning_scan_chunked"):
        getattr(L, name).restype = i32
    _layers = L
    return L


def check_layers(rc: int, what: str = ""):
    if rc != 0:
        msg = layers_lib().dl_last_error().decode("utf-8", "replace")
        raise NativeLibraryError(f"{what} failed ({rc}): {msg}")


# kernels launched by this process (bench.py reports it as gpu_launches)
launch_count = 0


def count_launch(n: int = 1):
    global launch_count
    launch_count += n
