// Checkpoint layout (export.py:83-119, src/gptq.rs:34-84), presets (src/constants.rs:7-41)
// and thread-local error reporting for the C ABI.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "host_common.h"

namespace l2 {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}
void clear_error() { g_err[0] = 0; }
const char* last_error() { return g_err; }

int default_threads() {
    unsigned n = std::thread::hardware_concurrency();
    return n ? (int)std::min(n, 64u) : 4;
}

void Shape::qdims(int t, int* in, int* out) const {
    const int D = c.dim, H = c.hidden_dim, KV = kv_dim();
    switch (t) {
        case T_WQ: case T_WO: *in = D; *out = D; break;
        case T_WK: case T_WV: *in = D; *out = KV; break;
        case T_W1: case T_W3: *in = D; *out = H; break;
        case T_W2: *in = H; *out = D; break;
        default: *in = *out = 0;
    }
}

size_t Shape::sub_words(int t, int sub) const {
    if (is_qlinear(t)) {
        int in, out;
        qdims(t, &in, &out);
        const size_t g = groups(in, c.group_size);
        switch (sub) {
            case S_QWEIGHT: return (size_t)out * (in / 32 * BITS);
            case S_QZEROS: return (size_t)(out / 32 * BITS) * g;
            case S_SCALES: return (size_t)out * g;
            case S_GINDEX: return (size_t)in;
        }
        return 0;
    }
    const size_t D = c.dim, L = c.n_layers, V = c.vocab_size, S = c.seq_len, HS = head_size();
    switch (t) {
        case T_RMS_EPS: return 1;
        case T_TOK_EMB: case T_WCLS: return V * D;
        case T_RMS_ATT: case T_RMS_FFN: return L * D;
        case T_RMS_FINAL: return D;
        case T_FREQ_REAL: case T_FREQ_IMAG: return S * (HS / 2);
    }
    return 0;
}

size_t Shape::qlinear_words(int t) const {
    return sub_words(t, S_QWEIGHT) + sub_words(t, S_QZEROS) + sub_words(t, S_SCALES) + sub_words(t, S_GINDEX);
}

size_t Shape::tensor_words(int t) const {
    return is_qlinear(t) ? qlinear_words(t) * (size_t)c.n_layers : sub_words(t, S_DENSE);
}

size_t Shape::tensor_offset_words(int t) const {
    size_t off = 0;
    for (int i = 0; i < t; i++) off += tensor_words(i);
    return off;
}

size_t Shape::total_words() const { return tensor_offset_words(T_COUNT); }

size_t Shape::offset_words(int t, int layer, int sub) const {
    size_t off = tensor_offset_words(t);
    if (!is_qlinear(t)) {
        // per-layer dense tensors are [L][DIM]
        if (t == T_RMS_ATT || t == T_RMS_FFN) off += (size_t)layer * c.dim;
        return off;
    }
    off += (size_t)layer * qlinear_words(t);
    for (int s = 0; s < sub; s++) off += sub_words(t, s);
    return off;
}

int validate_config(const l2_config& c) {
    if (c.dim <= 0 || c.hidden_dim <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 ||
        c.vocab_size <= 0 || c.seq_len <= 0)
        return fail(L2_EINVAL, "config: non-positive field");
    if (c.group_size != 32 && c.group_size != 64 && c.group_size != 128)
        return fail(L2_EINVAL, "config: group_size %d is not 32, 64 or 128", c.group_size);
    if (c.dim % c.n_heads || c.n_heads % c.n_kv_heads)
        return fail(L2_EINVAL, "config: heads do not divide dim / kv heads do not divide heads");
    if (c.dim / c.n_heads != 128) return fail(L2_EINVAL, "config: head size %d unsupported (128 only)", c.dim / c.n_heads);
    if (c.dim % c.group_size || c.hidden_dim % c.group_size)
        return fail(L2_EINVAL, "config: group size must divide dim and hidden_dim");
    if (c.dim % 32 || c.hidden_dim % 32 || c.vocab_size % 8)
        return fail(L2_EINVAL, "config: dim/hidden_dim must be multiples of 32, vocab of 8");
    if (c.n_heads / c.n_kv_heads > 8) return fail(L2_EINVAL, "config: more than 8 query heads per kv head");
    {
        const int ag = c.n_heads / c.n_kv_heads;  // the attention kernels are instantiated for these
        if (ag != 1 && ag != 2 && ag != 4 && ag != 8) return fail(L2_EINVAL, "config: %d query heads per kv head (1, 2, 4 or 8 supported)", ag);
    }
    return L2_OK;
}

}  // namespace l2

using namespace l2;

extern "C" const char* l2_last_error(void) { return l2::last_error(); }

extern "C" int l2_preset_config(const char* model_size, int group_size, l2_config* out) {
    if (!model_size || !out) return fail(L2_EINVAL, "l2_preset_config: null argument");
    l2_config c{};
    c.seq_len = 2048;
    c.vocab_size = 32000;
    c.group_size = group_size;
    if (!strcmp(model_size, "7B")) {  // src/constants.rs:31-41
        c.dim = 4096; c.hidden_dim = 11008; c.n_layers = 32; c.n_heads = 32; c.n_kv_heads = 32;
    } else if (!strcmp(model_size, "13B")) {  // :19-29
        c.dim = 5120; c.hidden_dim = 13824; c.n_layers = 40; c.n_heads = 40; c.n_kv_heads = 40;
    } else if (!strcmp(model_size, "70B")) {  // :7-17, ATTN_GROUPS = 8
        c.dim = 8192; c.hidden_dim = 28672; c.n_layers = 80; c.n_heads = 64; c.n_kv_heads = 8;
    } else {
        return fail(L2_EINVAL, "unknown model size '%s' (7B, 13B or 70B)", model_size);
    }
    if (int rc = validate_config(c)) return rc;
    *out = c;
    return L2_OK;
}

extern "C" size_t l2_checkpoint_bytes(const l2_config* c) {
    if (!c) return 0;
    Shape s{*c};
    return s.total_words() * 4;
}

extern "C" void l2_host_free(void* p) { free(p); }
