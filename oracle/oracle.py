"""ctypes wrapper of the CPU oracle (oracle/liboracle.so) -- TEST INFRASTRUCTURE ONLY.

Used by tests/, the smoke check and bench.py's CPU-baseline legs; never by the product."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liboracle.so")


def build(force=False):
    src = [os.path.join(HERE, f) for f in ("llama2_oracle.c", "llama2_oracle.h", "Makefile")]
    if force or not os.path.exists(LIB_PATH) or any(os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in src):
        subprocess.check_call(["make", "-C", HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return LIB_PATH


class Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "seq_len", "group_size")]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        p, i32p, f32p, vp = C.POINTER, C.POINTER(C.c_int32), C.POINTER(C.c_float), C.c_void_p
        sig = {
            "orc_weights_bytes": (C.c_size_t, [p(Config)]),
            "orc_model_map": (vp, [p(Config), vp, C.c_size_t]),
            "orc_model_open": (vp, [C.c_char_p, C.c_int, C.c_int]),
            "orc_model_close": (None, [vp]),
            "orc_model_config": (p(Config), [vp]),
            "orc_state_new": (vp, [vp]),
            "orc_state_free": (None, [vp]),
            "orc_state_key_cache": (f32p, [vp]),
            "orc_state_value_cache": (f32p, [vp]),
            "orc_qlinear_matvec": (None, [C.c_int, C.c_int, C.c_int, i32p, i32p, f32p, i32p, C.c_int, f32p, f32p]),
            "orc_linear_matvec": (None, [C.c_int, C.c_int, f32p, C.c_int, f32p, f32p]),
            "orc_rmsnorm": (None, [f32p, f32p, f32p, C.c_int, C.c_float]),
            "orc_softmax": (None, [f32p, C.c_int]),
            "orc_silu": (None, [f32p, f32p, C.c_int]),
            "orc_rope": (None, [f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int]),
            "orc_attention": (None, [f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int]),
            "orc_transformer": (None, [vp, vp, C.c_int, i32p, i32p, f32p]),
            "orc_argmax": (C.c_int32, [f32p, C.c_int]),
            "orc_random_u32": (C.c_uint32, [p(C.c_uint64)]),
            "orc_random_f32": (C.c_float, [p(C.c_uint64)]),
            "orc_sample": (C.c_int32, [p(C.c_uint64), f32p, C.c_int]),
            "orc_generate_ids": (C.c_int, [vp, i32p, C.c_int, C.c_int, C.c_float, p(C.c_uint64), C.c_int, i32p, i32p, f32p,
                                           p(C.c_double), p(C.c_double)]),
            "orc_num_threads": (C.c_int, []),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _f(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def make_config(**kw):
    c = Config()
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def copy_config(src):
    """Config from any object with the same field names (e.g. the product's Config)."""
    return make_config(**{n: getattr(src, n) for n, _ in Config._fields_})


def weights_bytes(cfg):
    return lib().orc_weights_bytes(C.byref(cfg))


def qlinear_matvec(qweight, qzeros, scales, g_index, group_size, x):
    """QLinear::matvec<B>: arrays in the checkpoint layout; x [B][IN] -> [B][OUT]."""
    qweight = np.ascontiguousarray(qweight, np.int32)
    qzeros = np.ascontiguousarray(qzeros, np.int32)
    scales = np.ascontiguousarray(scales, np.float32)
    g_index = np.ascontiguousarray(g_index, np.int32)
    x = np.ascontiguousarray(x, np.float32)
    out_f, in_f = qweight.shape[0], qweight.shape[1] * 8
    xb = x.reshape(-1, in_f)
    y = np.zeros((xb.shape[0], out_f), np.float32)
    # the restated matvec<B> holds at most 64 rows (the reference's largest prefill chunk); rows are independent of one another
    for b0 in range(0, xb.shape[0], 64):
        part = np.ascontiguousarray(xb[b0:b0 + 64])
        out = np.zeros((part.shape[0], out_f), np.float32)
        lib().orc_qlinear_matvec(in_f, out_f, group_size, _i(qweight), _i(qzeros), _f(scales), _i(g_index), part.shape[0], _f(part), _f(out))
        y[b0:b0 + 64] = out
    return y[0] if x.ndim == 1 else y


class Model:
    """View over a checkpoint payload (numpy uint8 array kept alive by this object)."""

    def __init__(self, cfg, payload):
        self.cfg = copy_config(cfg)
        self.payload = payload
        self.h = lib().orc_model_map(C.byref(self.cfg), payload.ctypes.data_as(C.c_void_p), payload.nbytes)
        if not self.h:
            raise ValueError("payload size does not match the configuration")
        self._owned = True

    @classmethod
    def open(cls, path, attn_groups, group_size):
        self = cls.__new__(cls)
        self.payload = None
        self.h = lib().orc_model_open(str(path).encode(), attn_groups, group_size)
        if not self.h:
            raise ValueError("cannot open %s with these options" % path)
        self.cfg = copy_config(lib().orc_model_config(self.h).contents)
        return self

    def transformer(self, state, tokens, pos):
        t = np.ascontiguousarray(tokens, np.int32)
        p = np.ascontiguousarray(pos, np.int32)
        logits = np.zeros(self.cfg.vocab_size, np.float32)
        lib().orc_transformer(self.h, state.h, t.size, _i(t), _i(p), _f(logits))
        return logits if t.size == 1 else None

    def generate_ids(self, prompt, steps, temperature=0.0, seed=0, use_prefill=True, trace_logits=False):
        pr = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(max(steps, 1), np.int32)
        pos0 = C.c_int32(0)
        s = C.c_uint64(seed)
        trace = np.zeros((max(steps, 1), self.cfg.vocab_size), np.float32) if trace_logits else None
        el, pf = C.c_double(0), C.c_double(0)
        n = lib().orc_generate_ids(self.h, _i(pr), pr.size, steps, temperature, C.byref(s), int(use_prefill), _i(out),
                                   C.byref(pos0), _f(trace) if trace_logits else None, C.byref(el), C.byref(pf))
        if n < 0:
            raise ValueError("steps exceeds SEQ_LEN")
        return {"tokens": out[:n].copy(), "pos0": pos0.value, "logits": trace[:n] if trace_logits else None,
                "elapsed_ms": el.value, "prefill_ms": pf.value, "seed": s.value}

    def __del__(self):
        try:
            if self.h:
                lib().orc_model_close(self.h)
        except Exception:
            pass


class State:
    def __init__(self, model):
        self.model = model
        self.h = lib().orc_state_new(model.h)

    def kv(self, layer):
        c = self.model.cfg
        hs = c.dim // c.n_heads
        n = c.seq_len * c.n_kv_heads * hs
        k = np.ctypeslib.as_array(lib().orc_state_key_cache(self.h), shape=(c.n_layers * n,))
        v = np.ctypeslib.as_array(lib().orc_state_value_cache(self.h), shape=(c.n_layers * n,))
        shape = (c.seq_len, c.n_kv_heads, hs)
        return k[layer * n:(layer + 1) * n].reshape(shape).copy(), v[layer * n:(layer + 1) * n].reshape(shape).copy()

    def __del__(self):
        try:
            if self.h:
                lib().orc_state_free(self.h)
        except Exception:
            pass
