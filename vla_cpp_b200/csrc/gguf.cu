// GGUF reader (versions 2 and 3) for the reference's checkpoint files, and the action-expert loader on
// top of it.  Host code only.  The reference reads its checkpoints through ggml's gguf_* API and a thin
// wrapper (src/gguf_reader.h:60-200: typed metadata getters, read_raw / read_f32 / read_convert with the
// Gemma-norm "+1", src/loader.cpp:131-180); ggml is not part of this library, so the container format is
// parsed here directly: header, metadata key/values, tensor directory, aligned data section (mmap'ed).
//
// File layout (little endian): magic "GGUF", u32 version, u64 n_tensors, u64 n_kv; n_kv x {string key,
// u32 type, value}; n_tensors x {string name, u32 n_dims, u64 dims[n_dims] (fastest first), u32 ggml type,
// u64 offset}; padding to general.alignment (default 32); tensor data at data_start + offset.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "host_common.h"

namespace vb {

enum GgufValueType { GV_U8 = 0, GV_I8, GV_U16, GV_I16, GV_U32, GV_I32, GV_F32, GV_BOOL, GV_STR, GV_ARR, GV_U64, GV_I64, GV_F64 };
// ggml tensor types this reader knows the size of
enum GgmlType { GT_F32 = 0, GT_F16 = 1, GT_Q4_0 = 2, GT_Q8_0 = 8, GT_I8 = 24, GT_I16 = 25, GT_I32 = 26, GT_I64 = 27, GT_F64 = 28, GT_BF16 = 30 };

struct GgufValue {
    uint32_t type = 0;
    uint64_t u = 0;      // integers and bool
    double f = 0.0;      // floats
    std::string s;       // strings
    uint32_t arr_type = 0;
    uint64_t arr_n = 0;
    size_t arr_off = 0;  // file offset of the first array element
};

struct GgufTensor {
    uint32_t type = 0, n_dims = 0;
    int64_t dims[4] = {1, 1, 1, 1};
    uint64_t offset = 0, n_bytes = 0;
    int64_t n_elems = 1;
};

// bytes of n elements of a ggml type; 0 = unknown type or n not a multiple of the block size
static uint64_t ggml_bytes(uint32_t type, int64_t n) {
    switch (type) {
        case GT_F32: case GT_I32: return (uint64_t)n * 4;
        case GT_F16: case GT_BF16: case GT_I16: return (uint64_t)n * 2;
        case GT_I8: return (uint64_t)n;
        case GT_I64: case GT_F64: return (uint64_t)n * 8;
        case GT_Q8_0: return n % 32 ? 0 : (uint64_t)(n / 32) * 34;
        case GT_Q4_0: return n % 32 ? 0 : (uint64_t)(n / 32) * 18;
        default: return 0;
    }
}

static float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { ++e; man <<= 1; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

static uint16_t float_to_bf16(float f) {  // round to nearest even; NaN stays NaN
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

}  // namespace vb

struct vlab200_gguf {
    int fd = -1;
    const uint8_t *base = nullptr;
    size_t size = 0, data_start = 0;
    uint32_t version = 0;
    std::map<std::string, vb::GgufValue> kv;
    std::map<std::string, vb::GgufTensor> tensors;
    std::vector<std::string> order;  // tensor names in file order
};

namespace vb {

// Cursor over the mapped file; every read is bounds-checked (a truncated or corrupt file is an error,
// never an out-of-range access).
struct Cursor {
    const uint8_t *b;
    size_t n, pos = 0;
    bool ok = true;
    template <typename T> T get() {
        T v{};
        if (!ok || n - pos < sizeof(T)) { ok = false; return v; }
        std::memcpy(&v, b + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t len = get<uint64_t>();
        if (!ok || len > n - pos || len > (1u << 20)) { ok = false; return {}; }
        std::string s(reinterpret_cast<const char *>(b + pos), (size_t)len);
        pos += (size_t)len;
        return s;
    }
    void skip(uint64_t bytes) {
        if (!ok || bytes > n - pos) ok = false;
        else pos += (size_t)bytes;
    }
};

static size_t scalar_size(uint32_t t) {
    switch (t) {
        case GV_U8: case GV_I8: case GV_BOOL: return 1;
        case GV_U16: case GV_I16: return 2;
        case GV_U32: case GV_I32: case GV_F32: return 4;
        case GV_U64: case GV_I64: case GV_F64: return 8;
        default: return 0;
    }
}

static bool read_value(Cursor &c, uint32_t type, GgufValue &v) {
    v.type = type;
    switch (type) {
        case GV_U8: v.u = c.get<uint8_t>(); break;
        case GV_I8: v.u = (uint64_t)(int64_t)c.get<int8_t>(); break;
        case GV_U16: v.u = c.get<uint16_t>(); break;
        case GV_I16: v.u = (uint64_t)(int64_t)c.get<int16_t>(); break;
        case GV_U32: v.u = c.get<uint32_t>(); break;
        case GV_I32: v.u = (uint64_t)(int64_t)c.get<int32_t>(); break;
        case GV_U64: v.u = c.get<uint64_t>(); break;
        case GV_I64: v.u = (uint64_t)c.get<int64_t>(); break;
        case GV_BOOL: v.u = c.get<uint8_t>() != 0; break;
        case GV_F32: v.f = c.get<float>(); break;
        case GV_F64: v.f = c.get<double>(); break;
        case GV_STR: v.s = c.str(); break;
        case GV_ARR: {
            v.arr_type = c.get<uint32_t>();
            v.arr_n = c.get<uint64_t>();
            v.arr_off = c.pos;
            if (v.arr_type == GV_STR) {
                for (uint64_t i = 0; c.ok && i < v.arr_n; ++i) c.skip(c.get<uint64_t>());
            } else {
                const size_t es = scalar_size(v.arr_type);
                if (!es || (v.arr_n && es > (c.n - c.pos) / v.arr_n)) c.ok = false;
                else c.skip(v.arr_n * es);
            }
            break;
        }
        default: c.ok = false;
    }
    return c.ok;
}

static bool parse(vlab200_gguf *g) {
    Cursor c{g->base, g->size};
    if (c.get<uint32_t>() != 0x46554747u) return set_last_error("gguf: bad magic"), false;
    g->version = c.get<uint32_t>();
    if (g->version != 2 && g->version != 3) return set_last_error("gguf: unsupported version %u", g->version), false;
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return set_last_error("gguf: bad header"), false;
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        GgufValue v;
        if (!c.ok || !read_value(c, type, v)) return set_last_error("gguf: bad metadata entry %llu", (unsigned long long)i), false;
        g->kv[key] = v;
    }
    for (uint64_t i = 0; i < n_tensors; ++i) {
        std::string name = c.str();
        GgufTensor t;
        t.n_dims = c.get<uint32_t>();
        if (!c.ok || t.n_dims > 4) return set_last_error("gguf: bad tensor entry %llu", (unsigned long long)i), false;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            t.dims[d] = (int64_t)c.get<uint64_t>();
            if (t.dims[d] <= 0 || t.dims[d] > (int64_t)1 << 40 || t.n_elems > ((int64_t)1 << 46) / t.dims[d])
                return set_last_error("gguf: bad dims of %s", name.c_str()), false;
            t.n_elems *= t.dims[d];
        }
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) return set_last_error("gguf: truncated tensor directory"), false;
        // quantised rows are blocked along dims[0]
        t.n_bytes = (t.type == GT_Q8_0 || t.type == GT_Q4_0) && t.dims[0] % 32 ? 0 : ggml_bytes(t.type, t.n_elems);
        g->tensors[name] = t;
        g->order.push_back(name);
    }
    uint64_t align = 32;
    auto it = g->kv.find("general.alignment");
    if (it != g->kv.end() && it->second.type == GV_U32 && it->second.u) align = it->second.u;
    g->data_start = (c.pos + align - 1) / align * align;
    for (auto &e : g->tensors) {
        const GgufTensor &t = e.second;
        if (t.n_bytes && (g->data_start > g->size || t.offset > g->size - g->data_start ||
                          t.n_bytes > g->size - g->data_start - t.offset))
            return set_last_error("gguf: tensor %s lies outside the file", e.first.c_str()), false;
    }
    return true;
}

static const GgufTensor *find_tensor(const vlab200_gguf *g, const char *name) {
    if (!g || !name) return nullptr;
    auto it = g->tensors.find(name);
    return it == g->tensors.end() ? nullptr : &it->second;
}

}  // namespace vb

// ------------------------------------------------------------------------------------------ C ABI

extern "C" {

vlab200_gguf *vlab200_gguf_open(const char *path) {
    if (!path) return vb::set_last_error("gguf: null path"), nullptr;
    vlab200_gguf *g = new vlab200_gguf();
    g->fd = ::open(path, O_RDONLY);
    struct stat st;
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) {
        vb::set_last_error("gguf: cannot open %s", path);
        vlab200_gguf_close(g);
        return nullptr;
    }
    g->size = (size_t)st.st_size;
    void *m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) {
        vb::set_last_error("gguf: mmap of %s failed", path);
        vlab200_gguf_close(g);
        return nullptr;
    }
    g->base = static_cast<const uint8_t *>(m);
    if (!vb::parse(g)) {
        vlab200_gguf_close(g);
        return nullptr;
    }
    return g;
}

void vlab200_gguf_close(vlab200_gguf *g) {
    if (!g) return;
    if (g->base) munmap(const_cast<uint8_t *>(g->base), g->size);
    if (g->fd >= 0) ::close(g->fd);
    delete g;
}

int64_t vlab200_gguf_n_tensors(const vlab200_gguf *g) { return g ? (int64_t)g->order.size() : -1; }

const char *vlab200_gguf_tensor_name(const vlab200_gguf *g, int64_t index) {
    return (g && index >= 0 && index < (int64_t)g->order.size()) ? g->order[(size_t)index].c_str() : nullptr;
}

int32_t vlab200_gguf_tensor_info(const vlab200_gguf *g, const char *name, int32_t *type, int32_t *n_dims,
                                 int64_t dims[4], uint64_t *n_bytes) {
    const vb::GgufTensor *t = vb::find_tensor(g, name);
    if (!t) return VLAB200_ERR_ARG;
    if (type) *type = (int32_t)t->type;
    if (n_dims) *n_dims = (int32_t)t->n_dims;
    if (dims) for (int d = 0; d < 4; ++d) dims[d] = t->dims[d];
    if (n_bytes) *n_bytes = t->n_bytes;
    return VLAB200_OK;
}

const void *vlab200_gguf_tensor_data(const vlab200_gguf *g, const char *name) {
    const vb::GgufTensor *t = vb::find_tensor(g, name);
    return (t && t->n_bytes) ? g->base + g->data_start + t->offset : nullptr;
}

int32_t vlab200_gguf_read_f32(const vlab200_gguf *g, const char *name, float *dst, int64_t n_elems,
                              int32_t gemma_norm) {
    const vb::GgufTensor *t = vb::find_tensor(g, name);
    if (!t || !dst) return vb::set_last_error("gguf: missing tensor %s", name ? name : "(null)"), VLAB200_ERR_ARG;
    if (t->n_elems != n_elems)
        return vb::set_last_error("gguf: tensor %s has %lld elements, caller expects %lld", name, (long long)t->n_elems,
                                  (long long)n_elems), VLAB200_ERR_ARG;
    const uint8_t *src = g->base + g->data_start + t->offset;
    if (t->type == vb::GT_F32) std::memcpy(dst, src, (size_t)n_elems * 4);
    else if (t->type == vb::GT_BF16) {
        for (int64_t i = 0; i < n_elems; ++i) {
            uint16_t h;
            std::memcpy(&h, src + 2 * i, 2);
            const uint32_t u = (uint32_t)h << 16;
            std::memcpy(dst + i, &u, 4);
        }
    } else if (t->type == vb::GT_F16) {
        for (int64_t i = 0; i < n_elems; ++i) {
            uint16_t h;
            std::memcpy(&h, src + 2 * i, 2);
            dst[i] = vb::half_to_float(h);
        }
    } else {
        return vb::set_last_error("gguf: tensor %s has type %u, not f32 / f16 / bf16", name, t->type), VLAB200_ERR_UNSUPPORTED;
    }
    if (gemma_norm) for (int64_t i = 0; i < n_elems; ++i) dst[i] += 1.0f;
    return VLAB200_OK;
}

static const vb::GgufValue *find_kv(const vlab200_gguf *g, const char *key) {
    if (!g || !key) return nullptr;
    auto it = g->kv.find(key);
    return it == g->kv.end() ? nullptr : &it->second;
}

int32_t vlab200_gguf_meta_u32(const vlab200_gguf *g, const char *key, uint32_t *out) {
    const vb::GgufValue *v = find_kv(g, key);
    if (!v || !out || v->type != vb::GV_U32) return VLAB200_ERR_ARG;
    *out = (uint32_t)v->u;
    return VLAB200_OK;
}

int32_t vlab200_gguf_meta_f64(const vlab200_gguf *g, const char *key, double *out) {
    const vb::GgufValue *v = find_kv(g, key);
    if (!v || !out || (v->type != vb::GV_F32 && v->type != vb::GV_F64)) return VLAB200_ERR_ARG;
    *out = v->f;
    return VLAB200_OK;
}

int32_t vlab200_gguf_meta_str(const vlab200_gguf *g, const char *key, char *buf, int32_t cap) {
    const vb::GgufValue *v = find_kv(g, key);
    if (!v || !buf || cap <= 0 || v->type != vb::GV_STR) return VLAB200_ERR_ARG;
    std::snprintf(buf, (size_t)cap, "%s", v->s.c_str());
    return VLAB200_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ action expert from a pi0 GGUF

namespace vb {

// One tensor of the checkpoint on the device: matrices as bf16, vectors as float32.
struct Upload {
    std::vector<DevBuf> bufs;
    std::vector<float> tmp;
    std::vector<uint16_t> tmp16;
    bool ok = true;

    // Reads `name` (f32 / f16 / bf16), checks its shape ([d1][d0], d1 == 1 for vectors, d1 < 0: d0 elements of any
    // shape), optional Gemma "+1",
    // converts matrices to bf16 (round to nearest even) and copies to the device.
    const void *get(const vlab200_gguf *g, const std::string &name, int64_t d0, int64_t d1, bool as_bf16, bool gemma) {
        if (!ok) return nullptr;
        const GgufTensor *t = find_tensor(g, name.c_str());
        if (!t) return fail("gguf: missing tensor %s", name);
        if (d1 < 0) {  // any shape with d0 elements in all (a convolution kernel kept as the file lays it out)
            if (t->dims[0] * t->dims[1] * t->dims[2] * t->dims[3] != d0) {
                set_last_error("gguf: tensor %s has %lld elements, expected %lld", name.c_str(),
                               (long long)(t->dims[0] * t->dims[1] * t->dims[2] * t->dims[3]), (long long)d0);
                ok = false;
                return nullptr;
            }
            d1 = 1;
        } else if (t->dims[0] != d0 || t->dims[1] != d1 || t->dims[2] != 1 || t->dims[3] != 1) {
            set_last_error("gguf: tensor %s is [%lld][%lld], expected [%lld][%lld]", name.c_str(), (long long)t->dims[1],
                           (long long)t->dims[0], (long long)d1, (long long)d0);
            ok = false;
            return nullptr;
        }
        const int64_t n = d0 * d1;
        tmp.resize((size_t)n);
        if (vlab200_gguf_read_f32(g, name.c_str(), tmp.data(), n, gemma ? 1 : 0) != VLAB200_OK) {
            ok = false;
            return nullptr;
        }
        bufs.emplace_back();
        DevBuf &b = bufs.back();
        const void *src = tmp.data();
        size_t bytes = (size_t)n * 4;
        if (as_bf16) {
            tmp16.resize((size_t)n);
            for (int64_t i = 0; i < n; ++i) tmp16[(size_t)i] = float_to_bf16(tmp[(size_t)i]);
            src = tmp16.data();
            bytes = (size_t)n * 2;
        }
        if (b.alloc(bytes) != VLAB200_OK || cudaMemcpy(b.p, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
            if (b.p) cuda_fail(cudaGetLastError(), "cudaMemcpy (gguf upload)");
            ok = false;
            return nullptr;
        }
        return b.p;
    }
    const void *fail(const char *fmt, const std::string &name) {
        set_last_error(fmt, name.c_str());
        ok = false;
        return nullptr;
    }
};

// One tensor onto the device for other translation units (same checks and conversions as Upload::get).
int gguf_upload(const vlab200_gguf *g, const char *name, int64_t d0, int64_t d1, bool as_bf16, bool gemma, DevBuf *out) {
    Upload up;
    const void *p = up.get(g, name, d0, d1, as_bf16, gemma);
    if (!p || !up.ok) return VLAB200_ERR_ARG;
    *out = std::move(up.bufs.back());
    return VLAB200_OK;
}

}  // namespace vb

extern "C" vlab200_engine *vlab200_engine_create_from_gguf(const vlab200_gguf *g, int32_t max_obs, int32_t prefix_len) {
    if (!g) return vb::set_last_error("gguf: null handle"), nullptr;
    char arch[32] = "";
    vlab200_gguf_meta_str(g, "general.architecture", arch, sizeof arch);
    const bool pi05 = std::strcmp(arch, "pi05") == 0;
    const bool pi0 = std::strcmp(arch, "pi0") == 0, smol = std::strcmp(arch, "smolvla") == 0;
    if (!pi0 && !smol && !pi05)
        return vb::set_last_error("gguf: general.architecture is '%s'; pi0, pi05 and smolvla checkpoints are mapped to the engine", arch), nullptr;
    const std::string pfx = std::string(arch) + ".";
    // metadata keys of src/models/pi0.cpp:267-293, src/models/pi05.cpp:292-326 and src/models/smolvla.cpp:604-632
    uint32_t n_layers, H, n_q, n_kv, hd, inter, chunk, steps, sdim, adim, self_every = 1;
    const struct { const char *key; uint32_t *dst; } u32s[] = {
        {"n_layers", &n_layers}, {"expert_h", &H}, {"n_q_heads", &n_q}, {"n_kv_heads", &n_kv},
        {"head_dim", &hd}, {"expert_inter", &inter}, {"chunk_size", &chunk}, {"num_steps", &steps},
        {"max_state_dim", &sdim}, {"max_action_dim", &adim}};
    for (const auto &e : u32s)
        if (vlab200_gguf_meta_u32(g, (pfx + e.key).c_str(), e.dst) != VLAB200_OK)
            return vb::set_last_error("gguf: missing u32 metadata %s%s", pfx.c_str(), e.key), nullptr;
    if (smol && vlab200_gguf_meta_u32(g, "smolvla.self_attn_every_n_layers", &self_every) != VLAB200_OK)
        return vb::set_last_error("gguf: missing u32 metadata smolvla.self_attn_every_n_layers"), nullptr;
    vlab200_policy_config cfg{};
    cfg.model = pi0 ? 0 : (pi05 ? 2 : 1);
    cfg.n_layers = (int32_t)n_layers; cfg.H = (int32_t)H; cfg.n_q = (int32_t)n_q; cfg.n_kv = (int32_t)n_kv;
    cfg.head_dim = (int32_t)hd; cfg.inter = (int32_t)inter; cfg.chunk = (int32_t)chunk;
    cfg.action_dim = (int32_t)adim; cfg.state_dim = pi05 ? 0 : (int32_t)sdim; cfg.steps = (int32_t)steps;
    cfg.self_every = (int32_t)self_every;
    double v;
    // SmolVLA fixes both constants in code (smolvla.cpp:622-624); pi0 reads them when present (pi0.cpp:289-293)
    cfg.rms_eps = smol ? 1e-5f : (vlab200_gguf_meta_f64(g, (pfx + "rms_norm_eps").c_str(), &v) == VLAB200_OK ? (float)v : 1e-6f);
    cfg.rope_base = (!smol && vlab200_gguf_meta_f64(g, (pfx + "rope_theta").c_str(), &v) == VLAB200_OK) ? (float)v : 10000.0f;
    uint32_t cond_dim = 0;
    if (pi05 && vlab200_gguf_meta_u32(g, "pi05.adarms_cond_dim", &cond_dim) == VLAB200_OK) cfg.cond_dim = (int32_t)cond_dim;
    const int64_t Hc = cfg.cond_dim > 0 ? cfg.cond_dim : (int64_t)H;
    if (vlab200_gguf_meta_f64(g, (pfx + "min_period").c_str(), &cfg.min_period) != VLAB200_OK ||
        vlab200_gguf_meta_f64(g, (pfx + "max_period").c_str(), &cfg.max_period) != VLAB200_OK)
        return vb::set_last_error("gguf: missing %smin_period / %smax_period", pfx.c_str(), pfx.c_str()), nullptr;
    if (n_layers == 0 || n_layers > 1024) return vb::set_last_error("gguf: %sn_layers = %u", pfx.c_str(), n_layers), nullptr;

    // tensor names of src/modules/gemma_expert.h:46-62 / src/models/pi0.cpp:431-437 and, for SmolVLA, of
    // hf_to_gguf (src/models/smolvla.cpp:648-703) and the projection heads (smolvla.cpp:1226-1236); only Gemma
    // norms carry the "+1"
    vb::Upload up;
    const int64_t qd = (int64_t)n_q * hd, kvd = (int64_t)n_kv * hd;
    std::vector<const void *> wq(n_layers), wk(n_layers), wv(n_layers), wo(n_layers), wg(n_layers), wu(n_layers), wd(n_layers);
    std::vector<const float *> ln_in(n_layers), ln_post(n_layers), ada_in_b(n_layers), ada_post_b(n_layers);
    for (uint32_t l = 0; l < n_layers; ++l) {
        const std::string b = "aex.blk." + std::to_string(l) + ".";
        // SmolVLA cross-attention layers project the VLM's K / V rows ([n_kv*hd] wide) instead of the expert's
        const bool cross = smol && self_every > 1 && l % self_every != 0;
        const int64_t kv_in = cross ? kvd : (int64_t)H;
        if (pi05) {  // the norms are dense maps of the time conditioning: [3H][cond] + [3H] (src/models/pi05.cpp:467-474)
            ln_in[l] = static_cast<const float *>(up.get(g, b + "attn_norm.weight", Hc, 3 * (int64_t)H, false, false));
            ada_in_b[l] = static_cast<const float *>(up.get(g, b + "attn_norm.bias", 3 * (int64_t)H, 1, false, false));
            ln_post[l] = static_cast<const float *>(up.get(g, b + "ffn_norm.weight", Hc, 3 * (int64_t)H, false, false));
            ada_post_b[l] = static_cast<const float *>(up.get(g, b + "ffn_norm.bias", 3 * (int64_t)H, 1, false, false));
        } else {
            ln_in[l] = static_cast<const float *>(up.get(g, b + "attn_norm.weight", H, 1, false, pi0));
            ln_post[l] = static_cast<const float *>(up.get(g, b + "ffn_norm.weight", H, 1, false, pi0));
        }
        wq[l] = up.get(g, b + "attn_q.weight", H, qd, true, false);
        wk[l] = up.get(g, b + "attn_k.weight", kv_in, kvd, true, false);
        wv[l] = up.get(g, b + "attn_v.weight", kv_in, kvd, true, false);
        wo[l] = up.get(g, b + "attn_o.weight", qd, H, true, false);
        wg[l] = up.get(g, b + "ffn_gate.weight", H, inter, true, false);
        wu[l] = up.get(g, b + "ffn_up.weight", H, inter, true, false);
        wd[l] = up.get(g, b + "ffn_down.weight", inter, H, true, false);
    }
    vlab200_policy_weights w{};
    w.wq = wq.data(); w.wk = wk.data(); w.wv = wv.data(); w.wo = wo.data();
    w.wgate = wg.data(); w.wup = wu.data(); w.wdown = wd.data();
    auto vec = [&](const char *name, int64_t n) { return static_cast<const float *>(up.get(g, name, n, 1, false, false)); };
    if (pi05) {
        w.ada_in_w = ln_in.data(); w.ada_in_b = ada_in_b.data(); w.ada_post_w = ln_post.data(); w.ada_post_b = ada_post_b.data();
        w.ada_final_w = static_cast<const float *>(up.get(g, "aex.output_norm.weight", Hc, 3 * (int64_t)H, false, false));
        w.ada_final_b = vec("aex.output_norm.bias", 3 * (int64_t)H);
        w.w_tin = static_cast<const float *>(up.get(g, "time_mlp_in.weight", H, Hc, false, false));   w.b_tin = vec("time_mlp_in.bias", Hc);
        w.w_tout = static_cast<const float *>(up.get(g, "time_mlp_out.weight", Hc, Hc, false, false)); w.b_tout = vec("time_mlp_out.bias", Hc);
    } else {
        w.ln_in = ln_in.data(); w.ln_post = ln_post.data();
        w.out_norm = static_cast<const float *>(up.get(g, "aex.output_norm.weight", H, 1, false, pi0));
    }
    if (pi0) {  // SmolVLA's state token belongs to the prefix (smolvla.cpp:1103-1104), not to the denoise loop
        w.w_sp = up.get(g, "state_proj.weight", sdim, H, true, false);
        w.b_sp = vec("state_proj.bias", H);
    }
    w.w_ain = up.get(g, "action_in_proj.weight", adim, H, true, false);       w.b_ain = vec("action_in_proj.bias", H);
    if (!pi05) {
        w.w_at1 = up.get(g, "action_time_mlp_in.weight", 2 * (int64_t)H, H, true, false);
        w.b_at1 = vec("action_time_mlp_in.bias", H);
        w.w_at2 = up.get(g, "action_time_mlp_out.weight", H, H, true, false);     w.b_at2 = vec("action_time_mlp_out.bias", H);
    }
    w.w_aout = up.get(g, "action_out_proj.weight", H, adim, true, false);     w.b_aout = vec("action_out_proj.bias", adim);
    if (!up.ok) return nullptr;
    // the engine keeps its own prepared copies; the uploads are released when `up` goes out of scope
    return vlab200_engine_create(&cfg, &w, max_obs, prefix_len);
}
