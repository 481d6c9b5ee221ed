"""llama2_rs -- the reference's Python surface (python/llama2_rs/__init__.py,
python/llama2_rs/llama2_rs_pylib.pyi, src/lib.rs:111-131) over the B200 C-ABI library.

    model = llama2_rs.LlamaModel("llama2_7b_4_128act.bin", False)
    tokenizer = llama2_rs.Tokenizer("tokenizer.bin")
    random = llama2_rs.Random()
    ms, pieces = llama2_rs.generate(model, tokenizer, "prompt", 50, random, 0.0)

What the reference fixes at compile time with cargo features is passed to LlamaModel as
keyword arguments (model_size="7B"|"13B"|"70B", group_size=32|64|128); without model_size
the shape is taken from the checkpoint header.
"""
import ctypes as C
import time

import numpy as np

from . import _lib
from ._lib import Config, L2Error, Options, check, lib

START = 1  # python/llama2_rs/__init__.py:4
RET = 13   # python/llama2_rs/__init__.py:5

__all__ = ["LlamaModel", "Tokenizer", "Random", "Config", "generate", "generate_ids", "RunState", "QLinear",
           "START", "RET", "preset_config", "checkpoint_bytes", "synth_fill", "synth_write_file", "L2Error"]


def tp_unique_id():
    """128-byte NCCL id made on rank 0, to be handed to every rank's LlamaModel.tp_connect."""
    buf = C.create_string_buffer(128)
    check(lib.l2_tp_unique_id(buf))
    return buf.raw


def preset_config(model_size, group_size):
    c = Config()
    check(lib.l2_preset_config(model_size.encode(), group_size, C.byref(c)))
    return c


def checkpoint_bytes(config):
    return lib.l2_checkpoint_bytes(C.byref(config))


def synth_fill(config, seed, threads=0):
    """The seeded synthetic checkpoint payload (bytes after the header) as a numpy uint8 array."""
    n = checkpoint_bytes(config)
    buf = np.empty(n, dtype=np.uint8)
    check(lib.l2_synth_fill(C.byref(config), seed, buf.ctypes.data_as(C.c_void_p), n, threads))
    return buf


def synth_write_file(config, seed, path, threads=0):
    check(lib.l2_synth_write_file(C.byref(config), seed, str(path).encode(), threads))


def _options(model_size, group_size, attn_groups, device, debug, max_batch, flags, tp=(0, 1), poll_limit_log2=0):
    o = Options()
    o.model_size = model_size.encode() if model_size else None
    o.group_size = group_size
    o.attn_groups = attn_groups
    o.device = device
    o.debug = int(bool(debug))
    o.max_batch = max_batch
    o.flags = flags
    o.tp_rank, o.tp_world = tp
    o.poll_limit_log2 = poll_limit_log2
    return o


class LlamaModel:
    """LlamaModel (src/lib.rs:28-77): LlamaModel(checkpoint, debug=False)."""

    def __init__(self, checkpoint=None, debug=False, *, model_size=None, group_size=128, attn_groups=1, device=-1,
                 max_batch=0, flags=0, tp=(0, 1), _handle=None):
        self._h = C.c_void_p()
        if _handle is not None:
            self._h = _handle
        else:
            o = _options(model_size, group_size, attn_groups, device, debug, max_batch, flags, tp)
            check(lib.l2_model_open(str(checkpoint).encode(), C.byref(o), C.byref(self._h)))
        self.config = Config()
        check(lib.l2_model_config(self._h, C.byref(self.config)))

    @classmethod
    def from_file(cls, checkpoint, debug=False, **kw):
        return cls(checkpoint, debug, **kw)

    @classmethod
    def from_blob(cls, config, payload, *, device=-1, debug=False, max_batch=0, flags=0, tp=(0, 1), poll_limit_log2=0):
        """The same on the bytes after the header (numpy uint8 array in the export.py layout)."""
        h = C.c_void_p()
        o = _options(None, config.group_size, config.n_heads // config.n_kv_heads, device, debug, max_batch, flags, tp, poll_limit_log2)
        check(lib.l2_model_open_blob(C.byref(config), payload.ctypes.data_as(C.c_void_p), payload.nbytes, C.byref(o), C.byref(h)))
        return cls(_handle=h)

    @classmethod
    def synthetic(cls, config, seed, *, device=-1, debug=False, max_batch=0, flags=0, tp=(0, 1)):
        """Seeded synthetic checkpoint generated tensor by tensor straight onto the device."""
        h = C.c_void_p()
        o = _options(None, config.group_size, config.n_heads // config.n_kv_heads, device, debug, max_batch, flags, tp)
        check(lib.l2_model_open_synthetic(C.byref(config), seed, C.byref(o), C.byref(h)))
        return cls(_handle=h)

    def prefill(self):
        return bool(lib.l2_model_prefill(self._h))

    def tp_connect(self, id_bytes):
        """Joins the NCCL communicator of a tensor-parallel model; id_bytes comes from tp_unique_id() on rank 0."""
        buf = C.create_string_buffer(bytes(id_bytes), 128)
        check(lib.l2_model_tp_connect(self._h, buf))

    def tp_pool_handle(self):
        """64-byte CUDA IPC handle of this rank's activation pool (tensor parallelism over peer memory)."""
        buf = C.create_string_buffer(64)
        check(lib.l2_model_tp_pool_handle(self._h, buf))
        return buf.raw

    def tp_pool_attach(self, rank, handle_bytes):
        """Maps rank `rank`'s pool; when every rank's pool is attached the token path needs no NCCL."""
        buf = C.create_string_buffer(bytes(handle_bytes), 64)
        check(lib.l2_model_tp_pool_attach(self._h, rank, buf))

    def tp_pool_bytes(self):
        return int(lib.l2_model_tp_pool_bytes(self._h))

    def tp_pool_attach_ptr(self, rank, device_ptr):
        """Attaches a pool that lives in this process (device pointer) as rank `rank`'s."""
        check(lib.l2_model_tp_pool_attach_ptr(self._h, rank, C.c_void_p(device_ptr)))

    def set_stream(self, cuda_stream):
        check(lib.l2_model_set_stream(self._h, C.c_void_p(cuda_stream)))

    @property
    def decode_bytes(self):
        return int(lib.l2_model_decode_bytes(self._h))

    def close(self):
        if self._h:
            lib.l2_model_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class RunState:
    """RunState (src/models.rs:29-42): the device-resident KV cache of one sequence."""

    def __init__(self, model):
        self.model = model
        self._h = C.c_void_p()
        check(lib.l2_state_new(model._h, C.byref(self._h)))

    def reset(self):
        check(lib.l2_state_reset(self._h))

    def read_kv(self, layer):
        c = self.model.config
        shape = (c.seq_len, c.n_kv_heads, c.dim // c.n_heads)
        k = np.empty(shape, np.float32)
        v = np.empty(shape, np.float32)
        check(lib.l2_state_read_kv(self._h, layer, _lib.as_f32p(k), _lib.as_f32p(v)))
        return k, v

    def close(self):
        if self._h:
            lib.l2_state_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            if self.model._h:
                self.close()
        except Exception:
            pass


def transformer(model, state, tokens, pos, want_logits=True):
    """transformer<B> (src/models.rs:178-298): logits (numpy, VOCAB) when B == 1, else None."""
    t = np.ascontiguousarray(tokens, np.int32)
    p = np.ascontiguousarray(pos, np.int32)
    B = t.size
    logits = np.empty(model.config.vocab_size, np.float32) if (B == 1 and want_logits) else None
    check(lib.l2_forward(model._h, state._h, _lib.as_i32p(t), _lib.as_i32p(p), B,
                         _lib.as_f32p(logits) if logits is not None else None))
    return logits


def prefill(model, state, prompt, chunk=0):
    """prefill<A> ladder (src/inference.rs:16-44, 78-127); returns the next position."""
    pr = np.ascontiguousarray(prompt, np.int32)
    pos = C.c_int32(0)
    check(lib.l2_prefill(model._h, state._h, _lib.as_i32p(pr), pr.size, chunk, C.byref(pos)))
    return pos.value


def decode_step(model, state, token, pos, temperature=0.0, random=None, forced_next=-1, want_logits=False):
    seed = C.c_uint64(random.seed if random is not None else 0)
    nxt = C.c_int32(0)
    logits = np.empty(model.config.vocab_size, np.float32) if want_logits else None
    check(lib.l2_decode_step(model._h, state._h, token, pos, temperature, C.byref(seed), forced_next, C.byref(nxt),
                             _lib.as_f32p(logits) if want_logits else None))
    if random is not None:
        random.seed = seed.value
    return nxt.value, logits


def decode_run(model, state, prompt, pos0, steps, temperature=0.0, random=None):
    pr = np.ascontiguousarray(prompt, np.int32)
    seed = C.c_uint64(random.seed if random is not None else 0)
    out = np.zeros(max(0, steps - pos0), np.int32)
    check(lib.l2_decode_run(model._h, state._h, _lib.as_i32p(pr), pr.size, pos0, steps, temperature, C.byref(seed), _lib.as_i32p(out)))
    if random is not None:
        random.seed = seed.value
    return out


def generate_ids(model, prompt_ids, steps, random=None, temperature=0.0, use_prefill=True, trace_logits=False):
    """generate() on token ids (src/inference.rs:49-193 with bpe_encode factored out).

    Returns a dict: tokens (the `next` of every B=1 iteration, forced ones included), pos0,
    logits ([n][VOCAB] or None), elapsed_ms / prefill_ms / decode_ms (device times)."""
    pr = np.ascontiguousarray(prompt_ids, np.int32)
    V = model.config.vocab_size
    out = np.zeros(max(steps, 1), np.int32)
    pos0 = C.c_int32(0)
    seed = C.c_uint64(random.seed if random is not None else 0)
    trace = np.zeros((max(steps, 1), V), np.float32) if trace_logits else None
    el, pf, dc = C.c_double(0), C.c_double(0), C.c_double(0)
    n = check(lib.l2_generate_ids(model._h, _lib.as_i32p(pr), pr.size, steps, temperature, C.byref(seed), int(use_prefill),
                                  _lib.as_i32p(out), C.byref(pos0), _lib.as_f32p(trace) if trace_logits else None,
                                  C.byref(el), C.byref(pf), C.byref(dc)))
    if random is not None:
        random.seed = seed.value
    return {"tokens": out[:n].copy(), "pos0": pos0.value, "logits": trace[:n] if trace_logits else None,
            "elapsed_ms": el.value, "prefill_ms": pf.value, "decode_ms": dc.value}


class Tokenizer:
    """Tokenizer (src/tokenizer.rs:13-44): Tokenizer(filename).bpe_encode(text) -> list[int]."""

    def __init__(self, filename, vocab_size=32000):
        self._h = C.c_void_p()
        check(lib.l2_tokenizer_open(str(filename).encode(), vocab_size, C.byref(self._h)))

    def bpe_encode(self, text):
        data = text.encode("utf-8")
        cap = max(16, len(data) + 1)
        ids = np.zeros(cap, np.int32)
        n = check(lib.l2_tokenizer_encode(self._h, data, _lib.as_i32p(ids), cap))
        return [int(i) for i in ids[:n]]

    def piece(self, prev, nxt):
        s = lib.l2_tokenizer_piece(self._h, prev, nxt)
        return s.decode("utf-8", "replace") if s is not None else ""

    def __del__(self):
        try:
            if self._h:
                lib.l2_tokenizer_free(self._h)
        except Exception:
            pass


class Random:
    """Random (src/util.rs:55-83): xorshift* seeded with the unix time in seconds."""

    def __init__(self, seed=None):
        self.seed = int(time.time()) if seed is None else int(seed)

    def random_u32(self):
        s = C.c_uint64(self.seed)
        r = lib.l2_random_u32(C.byref(s))
        self.seed = s.value
        return r

    def random(self):
        s = C.c_uint64(self.seed)
        r = lib.l2_random_f32(C.byref(s))
        self.seed = s.value
        return r


def generate(model, tokenizer, prompt, steps, random, temperature=0.0, print_tokens=False):
    """generate (src/inference.rs:49-57) -> (elapsed ms, list of token strings)."""
    ids = tokenizer.bpe_encode(" " + prompt.strip()) if prompt else []  # :62-67
    r = generate_ids(model, ids, steps, random, temperature, use_prefill=model.prefill())
    pieces = []
    # the token fed at the first B=1 position (src/inference.rs:128-132)
    token = START if r["pos0"] == 0 else ids[r["pos0"] - 1]
    for nxt in r["tokens"]:
        pieces.append(tokenizer.piece(token, int(nxt)))  # get_token, src/util.rs:116-123
        token = int(nxt)
    if print_tokens:
        print("".join(pieces), end="", flush=True)
    return int(r["elapsed_ms"]), pieces


class QLinear:
    """One quantised linear layer on the device (src/gptq.rs:68-84, src/gptq_cuda.rs:93-110).

    Arrays are in the checkpoint layout: qweight [OUT][IN/8] i32, qzeros [OUT/8][GROUPS] i32,
    scales [OUT][GROUPS] f32, g_index [IN] i32."""

    def __init__(self, qweight, qzeros, scales, g_index, group_size, device=-1):
        qweight = np.ascontiguousarray(qweight, np.int32)
        qzeros = np.ascontiguousarray(qzeros, np.int32)
        scales = np.ascontiguousarray(scales, np.float32)
        g_index = np.ascontiguousarray(g_index, np.int32)
        self.out_features, self.in_features = qweight.shape[0], qweight.shape[1] * 8
        self._h = C.c_void_p()
        check(lib.l2_qlinear_create(self.in_features, self.out_features, group_size, _lib.as_i32p(qweight), _lib.as_i32p(qzeros),
                                    _lib.as_f32p(scales), _lib.as_i32p(g_index), device, C.byref(self._h)))

    def matvec(self, x):
        """QLinear::matvec<B> (src/gptq.rs:94): x [B][IN] (or [IN]) f32 -> [B][OUT]."""
        x = np.ascontiguousarray(x, np.float32)
        one = x.ndim == 1
        xb = x.reshape(-1, self.in_features)
        out = np.empty((xb.shape[0], self.out_features), np.float32)
        check(lib.l2_qlinear_matvec(self._h, _lib.as_f32p(xb), _lib.as_f32p(out), xb.shape[0]))
        return out[0] if one else out

    def matvec_dev(self, x_ptr, out_ptr, B, stream=0):
        check(lib.l2_qlinear_matvec_dev(self._h, C.c_void_p(x_ptr), C.c_void_p(out_ptr), B, C.c_void_p(stream)))

    def __del__(self):
        try:
            if self._h:
                lib.l2_qlinear_free(self._h)
        except Exception:
            pass
