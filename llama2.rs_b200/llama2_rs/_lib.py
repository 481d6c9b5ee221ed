"""ctypes binding of libllama2_b200.so (the C ABI declared in include/llama2_b200.h).

The library is looked up next to this package and is never replaced by a Python or CPU
implementation: if it is missing, importing this module raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# LLAMA2_B200_LIB names another build of the same library (for example one with the debugging clock stamps compiled in)
LIB_PATH = os.environ.get("LLAMA2_B200_LIB") or os.path.join(os.path.dirname(_HERE), "libllama2_b200.so")


class L2Error(RuntimeError):
    def __init__(self, code, message):
        super().__init__("llama2_b200 error %d: %s" % (code, message))
        self.code = code


class Config(C.Structure):
    """The reference's Config (src/constants.rs:77-91) plus the compile-time group size."""
    _fields_ = [(n, C.c_int32) for n in
                ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "seq_len", "group_size")]

    def __repr__(self):
        return "Config { " + ", ".join("%s: %d" % (n, getattr(self, n)) for n, _ in self._fields_) + " }"


class Options(C.Structure):
    _fields_ = [("model_size", C.c_char_p), ("group_size", C.c_int32), ("attn_groups", C.c_int32),
                ("device", C.c_int32), ("debug", C.c_int32), ("max_batch", C.c_int32), ("flags", C.c_int32),
                ("tp_rank", C.c_int32), ("tp_world", C.c_int32), ("poll_limit_log2", C.c_int32)]


FLAG_NO_GRAPH = 1
FLAG_NO_PDL = 2

if not os.path.exists(LIB_PATH):
    raise ImportError("libllama2_b200.so is not built (%s); run `python llama2.rs_b200/build.py`" % LIB_PATH)
lib = C.CDLL(LIB_PATH)

_p = C.POINTER
_i32p, _f32p, _u64p, _vp = _p(C.c_int32), _p(C.c_float), _p(C.c_uint64), C.c_void_p

# name -> (restype, argtypes); every symbol of include/llama2_b200.h
SIGNATURES = {
    "l2_last_error": (C.c_char_p, []),
    "l2_launch_count": (C.c_uint64, []),
    "l2_preset_config": (C.c_int, [C.c_char_p, C.c_int, _p(Config)]),
    "l2_checkpoint_bytes": (C.c_size_t, [_p(Config)]),
    "l2_synth_fill": (C.c_int, [_p(Config), C.c_uint64, _vp, C.c_size_t, C.c_int]),
    "l2_synth_write_file": (C.c_int, [_p(Config), C.c_uint64, C.c_char_p, C.c_int]),
    "l2_model_open": (C.c_int, [C.c_char_p, _p(Options), _p(_vp)]),
    "l2_model_open_blob": (C.c_int, [_p(Config), _vp, C.c_size_t, _p(Options), _p(_vp)]),
    "l2_model_open_synthetic": (C.c_int, [_p(Config), C.c_uint64, _p(Options), _p(_vp)]),
    "l2_model_close": (None, [_vp]),
    "l2_model_config": (C.c_int, [_vp, _p(Config)]),
    "l2_model_prefill": (C.c_int, [_vp]),
    "l2_model_set_stream": (C.c_int, [_vp, _vp]),
    "l2_model_decode_bytes": (C.c_uint64, [_vp]),
    "l2_tp_unique_id": (C.c_int, [_vp]),
    "l2_model_tp_connect": (C.c_int, [_vp, _vp]),
    "l2_tp_rows": (C.c_int, [C.c_int, C.c_int, C.c_int, _p(C.c_int), _p(C.c_int)]),
    "l2_model_tp_pool_handle": (C.c_int, [_vp, _vp]),
    "l2_model_tp_pool_attach": (C.c_int, [_vp, C.c_int, _vp]),
    "l2_model_tp_pool_bytes": (C.c_size_t, [_vp]),
    "l2_model_tp_pool_attach_ptr": (C.c_int, [_vp, C.c_int, _vp]),
    "l2_state_new": (C.c_int, [_vp, _p(_vp)]),
    "l2_state_reset": (C.c_int, [_vp]),
    "l2_state_free": (None, [_vp]),
    "l2_state_read_kv": (C.c_int, [_vp, C.c_int, _f32p, _f32p]),
    "l2_forward": (C.c_int, [_vp, _vp, _i32p, _i32p, C.c_int, _f32p]),
    "l2_prefill": (C.c_int, [_vp, _vp, _i32p, C.c_int, C.c_int, _i32p]),
    "l2_decode_step": (C.c_int, [_vp, _vp, C.c_int32, C.c_int32, C.c_float, _u64p, C.c_int32, _i32p, _f32p]),
    "l2_decode_run": (C.c_int, [_vp, _vp, _i32p, C.c_int, C.c_int32, C.c_int32, C.c_float, _u64p, _i32p]),
    "l2_generate_ids": (C.c_int, [_vp, _i32p, C.c_int, C.c_int, C.c_float, _u64p, C.c_int, _i32p, _i32p, _f32p,
                                  _p(C.c_double), _p(C.c_double), _p(C.c_double)]),
    "l2_qlinear_create": (C.c_int, [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _f32p, _i32p, C.c_int, _p(_vp)]),
    "l2_qlinear_matvec": (C.c_int, [_vp, _f32p, _f32p, C.c_int]),
    "l2_qlinear_matvec_dev": (C.c_int, [_vp, _vp, _vp, C.c_int, _vp]),
    "l2_qlinear_free": (None, [_vp]),
    "l2_rope_table": (C.c_int, [C.c_int, _f32p, _f32p]),
    "l2_attention_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "l2_attention_decode_dev": (C.c_int, [C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _vp]),
    "l2_attention_decode_noalloc": (C.c_int, [C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "l2_bench_projection": (C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int]),
    "l2_projection_bytes": (C.c_uint64, [_vp, C.c_int]),
    "l2_debug_trace": (C.c_int, [C.c_int, _p(C.c_uint64), C.c_int]),
    "l2_debug_token_trace": (C.c_int, [C.c_void_p, C.c_int, _p(C.c_uint64), C.c_size_t]),
    "l2_random_u32": (C.c_uint32, [_u64p]),
    "l2_random_f32": (C.c_float, [_u64p]),
    "l2_tokenizer_open": (C.c_int, [C.c_char_p, C.c_int, _p(_vp)]),
    "l2_tokenizer_free": (None, [_vp]),
    "l2_tokenizer_encode": (C.c_int, [_vp, C.c_char_p, _i32p, C.c_int]),
    "l2_tokenizer_vocab": (C.c_char_p, [_vp, C.c_int32]),
    "l2_tokenizer_piece": (C.c_char_p, [_vp, C.c_int32, C.c_int32]),
    "l2_debug_repack": (C.c_int, [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _f32p, _i32p,
                                  _p(_p(C.c_uint32)), _p(C.c_int), _p(C.c_int)]),
    "l2_host_free": (None, [_vp]),
}
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def check(rc):
    """Raises L2Error for a negative return code; passes non-negative values through."""
    if rc < 0:
        raise L2Error(rc, (lib.l2_last_error() or b"").decode("utf-8", "replace"))
    return rc


def as_i32p(a):
    return a.ctypes.data_as(_i32p)


def as_f32p(a):
    return a.ctypes.data_as(_f32p)
FLAG_NO_L2_PREFETCH = 4
FLAG_NO_TOKEN_KERNEL = 8
