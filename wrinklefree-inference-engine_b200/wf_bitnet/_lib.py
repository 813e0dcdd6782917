"""ctypes binding of libwf_bitnet.so (C ABI: include/wf_bitnet.h).

The library is the product: there is NO fallback.  If it is missing, or no sm_100 device is
present when a compute entry point is called, we raise — loudly.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG_ROOT = Path(__file__).resolve().parent.parent
LIB_PATH = Path(os.environ.get("WF_BITNET_LIB", _PKG_ROOT / "libwf_bitnet.so"))

WF_OK, WF_ERR_INVALID, WF_ERR_UNSUPPORTED, WF_ERR_CUDA = 0, -1, -2, -3
WF_F32, WF_BF16, WF_F16, WF_I8 = 0, 1, 2, 3
WF_W_I2S, WF_W_TILE = 0, 1
WF_OUT_I32_PLUS1, WF_OUT_I32, WF_OUT_COMPAT_F32, WF_OUT_LINEAR = 0, 1, 2, 3
WF_EPI_RESIDUAL, WF_EPI_RELU2_MUL = 1, 2
BITNET_BLOCK_SIZE = 128


class WfError(RuntimeError):
    pass


class LinearArgs(C.Structure):
    _fields_ = [
        ("w", C.c_void_p), ("w_layout", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("q", C.c_void_p), ("M", C.c_int), ("ldq", C.c_int),
        ("rowsum", C.c_void_p), ("act_scale", C.c_void_p), ("act_scale_per_token", C.c_int),
        ("w_scale", C.c_void_p), ("nseg", C.c_int), ("seg_end", C.c_int * 4),
        ("host_scale", C.c_float), ("out_mode", C.c_int), ("epi_flags", C.c_int), ("out_dtype", C.c_int),
        ("out", C.c_void_p), ("ldo", C.c_int), ("residual", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("algo", C.c_int),
    ]


class KvLayout(C.Structure):
    _fields_ = [
        ("pool", C.c_void_p), ("max_pages", C.c_int), ("layers", C.c_int), ("kv_heads", C.c_int),
        ("page_size", C.c_int), ("head_dim", C.c_int), ("dtype", C.c_int),
    ]


class ModelConfig(C.Structure):
    _fields_ = [
        ("hidden", C.c_int), ("layers", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int), ("head_dim", C.c_int),
        ("ffn", C.c_int), ("vocab", C.c_int), ("rope_theta", C.c_float), ("eps", C.c_float),
        ("max_seq", C.c_int), ("page_size", C.c_int), ("max_batch", C.c_int), ("max_pages", C.c_int),
        ("tp_rank", C.c_int), ("tp_size", C.c_int), ("kv_dtype", C.c_int),
    ]


# every symbol include/wf_bitnet.h declares: name -> (restype, argtypes)
_vp, _i, _f, _sz, _u64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint64
SYMBOLS = {
    "wf_bitnet_available": (_i, []),
    "wf_last_error": (C.c_char_p, []),
    "wf_sm_count": (_i, []),
    "wf_version": (C.c_char_p, []),
    "wf_copy_d2d": (_i, [_vp, _vp, _sz, _vp]),
    "wf_pack_ternary": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "wf_unpack_i2s": (_i, [_vp, _i, _i, _vp, _vp]),
    "wf_hf_to_i2s": (_i, [_vp, _i, _i, _vp, _vp]),
    "wf_tile_bytes": (_sz, [_i, _i]),
    "wf_repack_i2s_to_tile": (_i, [_vp, _i, _i, _vp, _vp]),
    "wf_repack_tile_to_i2s": (_i, [_vp, _i, _i, _vp, _vp]),
    "wf_interleave_rows16": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "wf_act_quant_i8": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "wf_linear_workspace_bytes": (_sz, [_i, _i, _i]),
    "wf_ternary_linear": (_i, [C.POINTER(LinearArgs), _vp]),
    "wf_bitnet_gemv": (_i, [_vp, _vp, _f, _i, _i, _vp, _vp, _sz, _vp]),
    "wf_bitnet_gemm": (_i, [_vp, _vp, _f, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "wf_static_workspace_max_bytes": (_sz, []),
    "wf_bitnet_gemm_static": (_i, [_vp, _vp, _f, _i, _i, _i, _vp, _vp]),
    "wf_kv_pool_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "wf_kv_scatter": (_i, [C.POINTER(KvLayout), _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "wf_kv_gather": (_i, [C.POINTER(KvLayout), _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "wf_rope_kv_append": (_i, [_vp, _i, _i, C.POINTER(KvLayout), _i, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp]),
    "wf_attn_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "wf_paged_decode_attn": (_i, [_vp, C.POINTER(KvLayout), _i, _vp, _i, _vp, _i, _i, _f, _vp, _i, _vp, _sz, _vp]),
    "wf_rmsnorm_quant": (_i, [_vp, _vp, _f, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "wf_embed": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "wf_lm_head_workspace_bytes": (_sz, [_i, _i]),
    "wf_lm_head_argmax": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "wf_engine_create": (_i, [C.POINTER(ModelConfig), C.POINTER(_vp)]),
    "wf_engine_destroy": (None, [_vp]),
    "wf_engine_device_bytes": (_sz, [_vp]),
    "wf_engine_set_linear": (_i, [_vp, _i, C.c_char_p, _vp, _f, _i]),
    "wf_engine_set_tensor": (_i, [_vp, _i, C.c_char_p, _vp, _sz, _i]),
    "wf_engine_init_synthetic": (_i, [_vp, _u64]),
    "wf_engine_finalize_weights": (_i, [_vp]),
    "wf_engine_reset": (_i, [_vp]),
    "wf_engine_set_context": (_i, [_vp, _i, _i, _i]),
    "wf_engine_decode": (_i, [_vp, _vp, _i, _vp]),
    "wf_engine_decode_device": (_i, [_vp, _i, _i]),
    "wf_engine_sync": (_i, [_vp]),
    "wf_engine_stream": (_vp, [_vp]),
    "wf_engine_tp_handle_bytes": (_sz, []),
    "wf_engine_tp_export": (_i, [_vp, _vp]),
    "wf_engine_tp_attach": (_i, [_vp, _vp]),
    "wf_engine_buffer": (_vp, [_vp, C.c_char_p]),
    "wf_engine_launches_per_step": (_i, [_vp]),
    "wf_engine_time_kernel": (_i, [_vp, C.c_char_p, _i, _i, C.POINTER(_f)]),
    "wf_bench_gemv": (_i, [_i, _i, _i, _i, _i, C.POINTER(_f)]),
    "wf_gemm_stream_acc": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _i, _vp]),
}

_lib = None

# ---- libwf_seq.so (include/wf_seq.h): the engine for layer-stack sequence models ------------------------------------------------
SEQ_LIB_PATH = Path(os.environ.get("WF_SEQ_LIB", _PKG_ROOT / "libwf_seq.so"))
WF_SEQ_F32, WF_SEQ_BF16 = 0, 1
WF_SEQ_LATENT_ATTENTION, WF_SEQ_DELTA, WF_SEQ_GQA_ATTENTION, WF_SEQ_SSD, WF_SEQ_MINGRU, WF_SEQ_MLSTM = 0, 1, 2, 3, 4, 5
WF_SEQ_BLOCK_SANDWICH, WF_SEQ_BLOCK_POST, WF_SEQ_BLOCK_PARALLEL = 0, 1, 2
WF_SEQ_FF_NONE, WF_SEQ_FF_ROUTED, WF_SEQ_FF_DENSE = 0, 1, 2
WF_SEQ_ACT_SILU, WF_SEQ_ACT_CLAMPED, WF_SEQ_ACT_GELU_TANH, WF_SEQ_ACT_RELU2 = 0, 1, 2, 3
WF_SEQ_QKNORM_NONE, WF_SEQ_QKNORM_UNIT, WF_SEQ_QKNORM_HEAD, WF_SEQ_QKNORM_FULL = 0, 1, 2, 3


class SeqLayer(C.Structure):
    _fields_ = [
        ("type", C.c_int), ("heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int),
        ("rot_dim", C.c_int), ("kv_rank", C.c_int), ("window", C.c_int), ("rope_dims", C.c_int),
        ("scale", C.c_float), ("rope_base", C.c_float),
        ("kv_heads", C.c_int), ("conv", C.c_int),
        ("has_ff", C.c_int), ("experts", C.c_int), ("identity", C.c_int), ("top", C.c_int), ("groups", C.c_int), ("keep", C.c_int),
        ("ff", C.c_int),
        ("qk_norm", C.c_int), ("v_norm", C.c_int), ("proj_bias", C.c_int), ("head_gate", C.c_int), ("kv_from", C.c_int),
        ("dist_exp", C.c_float),
        ("ff_act", C.c_int), ("ff_limit", C.c_float), ("router_act", C.c_int), ("group_top", C.c_int), ("router_norm", C.c_int),
        ("router_scale", C.c_float), ("shared_ff", C.c_int), ("shared_limit", C.c_float),
        ("rope_interleaved", C.c_int), ("chunk", C.c_int), ("rel_rows", C.c_int), ("sink", C.c_int),
        ("softcap", C.c_float), ("rel_far", C.c_float),
        ("decay_channels", C.c_int), ("decay_rank", C.c_int), ("gate_rank", C.c_int), ("gate_act", C.c_int),
        ("out_norm_groups", C.c_int),
        ("pair", C.c_int), ("mix_scale", C.c_float), ("pair_scale", C.c_float),
        ("tied", C.c_int), ("tied_to", C.c_int),
        ("q_rank", C.c_int),
        ("rope_factor", C.c_float), ("rope_orig", C.c_float), ("rope_fast", C.c_float), ("rope_slow", C.c_float),
        ("v_is_k", C.c_int), ("gate_cap", C.c_float),
    ]

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        if "kv_from" not in kw:
            self.kv_from = -1
        if "router_scale" not in kw:
            self.router_scale = 1.0


class SeqConfig(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("vocab", C.c_int), ("width", C.c_int), ("n_layers", C.c_int), ("eps", C.c_float),
        ("norm_groups", C.c_int), ("canon_taps", C.c_int), ("page_size", C.c_int), ("max_pages", C.c_int), ("slots", C.c_int),
        ("max_step_tokens", C.c_int),
        ("block_form", C.c_int), ("residual_mult", C.c_float), ("pos_embed", C.c_int), ("pos_base", C.c_float),
        ("n_extra", C.c_int), ("embed_scale", C.c_float), ("norm_weights", C.c_int), ("tied_head", C.c_int),
        ("norm_offset", C.c_float),
    ]


_ip, _fp = C.POINTER(C.c_int32), C.POINTER(C.c_float)
SEQ_SYMBOLS = {
    "wf_last_error": (C.c_char_p, []),
    "wf_seq_available": (_i, []),
    "wf_seq_create": (_i, [C.POINTER(SeqConfig), C.POINTER(SeqLayer), C.POINTER(_vp)]),
    "wf_seq_destroy": (None, [_vp]),
    "wf_seq_device_bytes": (_sz, [_vp]),
    "wf_seq_set_tensor": (_i, [_vp, C.c_char_p, _vp, _sz, _i]),
    "wf_seq_tensor_count": (_i, [_vp]),
    "wf_seq_tensor_name": (C.c_char_p, [_vp, _i, C.POINTER(_sz), C.POINTER(_i)]),
    "wf_seq_finalize": (_i, [_vp]),
    "wf_seq_admit": (_i, [_vp, C.POINTER(_i)]),
    "wf_seq_release": (_i, [_vp, _i]),
    "wf_seq_length": (_i, [_vp, _i]),
    "wf_seq_free_pages": (_i, [_vp]),
    "wf_seq_free_slots": (_i, [_vp]),
    "wf_seq_step": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp]),
    "wf_seq_sample": (_i, [_vp, _i, _f, _i, _f, _vp, _vp]),
    "wf_seq_logits_device": (_vp, [_vp]),
    "wf_seq_launches_last_step": (_i, [_vp]),
    "wf_seq_set_layer_tap": (_i, [_vp, _vp]),
    "wf_seq_run_part": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "wf_seq_time_step": (_i, [_vp, _i, _vp, _vp, _i, _fp]),
    "wf_seq_profile_step": (_i, [_vp, _i, _vp, _vp, _i, C.c_char_p, _sz]),
    "wf_seq_set_length": (_i, [_vp, _i, _i]),
    "wf_seq_op_gemm": (_i, [_i, _vp, _i, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp, C.c_longlong, _i, _i, _vp]),
}
_seq_lib = None


def build_seq_lib() -> None:
    """Compile libwf_seq.so in-tree (make target `seq`: the sequence-model sources only)."""
    import subprocess
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    subprocess.run(["make", "-C", str(_PKG_ROOT / "csrc"), "seq", "-j8"], check=True, env=env, stdout=subprocess.DEVNULL)


def seq_lib(build: bool = False) -> C.CDLL:
    """Load libwf_seq.so and bind every symbol of include/wf_seq.h.  build=True compiles it first when it is absent."""
    global _seq_lib
    if _seq_lib is None:
        if not SEQ_LIB_PATH.exists():
            if not build:
                raise WfError(f"{SEQ_LIB_PATH} not found: build it with `make -C {_PKG_ROOT / 'csrc'} seq`. There is no CPU fallback.")
            build_seq_lib()
        L = C.CDLL(str(SEQ_LIB_PATH))
        for name, (res, args) in SEQ_SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _seq_lib = L
    return _seq_lib


def seq_check(rc: int) -> None:
    if rc == WF_OK:
        return
    msg = seq_lib().wf_last_error().decode("utf-8", "replace")
    if rc == WF_ERR_INVALID:
        raise ValueError(msg)
    if rc == WF_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise WfError(msg)


def lib() -> C.CDLL:
    """Load libwf_bitnet.so and bind every declared symbol.  Raises if the library is absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise WfError(
                f"{LIB_PATH} not found: build it with `make -C {_PKG_ROOT / 'csrc'}` (or __graft_entry__.build()). "
                "There is no CPU fallback."
            )
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)   # AttributeError here == header/library mismatch
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().wf_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Map a C status to the reference's Python error behaviour (ValueError for bad arguments)."""
    if rc == WF_OK:
        return
    msg = last_error()
    if rc == WF_ERR_INVALID:
        raise ValueError(msg)
    if rc == WF_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise WfError(msg)


def available() -> bool:
    try:
        return bool(lib().wf_bitnet_available())
    except WfError:
        return False


def require_gpu() -> None:
    if not lib().wf_bitnet_available():
        raise WfError("no compute-capability-10.x CUDA device visible; the BitNet kernels are sm_100a-only and there is no CPU fallback")
