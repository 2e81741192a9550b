// On-disk EXL3 checkpoints: a safetensors reader (header parse + validation as src/safetensors.rs:64-171 performs them,
// positional reads straight into pinned staging and from there into device memory) and Linear::load
// (src/modules.rs:97-165: key scheme <key>.trellis/.suh/.svh/.mcg/.mul1/.bias, or <key>.weight for a dense layer, features
// padded to multiples of 128).  Host code plus two small copy kernels; nothing here runs on the decode path.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>
#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>
#include "common.cuh"

namespace {

constexpr uint64_t MAX_HEADER = 100ull << 20;      // src/safetensors.rs:15
constexpr size_t STAGE_BYTES = 32u << 20;          // pinned staging buffer: tensors larger than this go in pieces

struct Entry { std::string dtype; std::vector<int64_t> shape; uint64_t begin = 0, end = 0; };

int dtype_size(const std::string& dt)              // src/safetensors.rs:42-57
{
    if (dt == "F16" || dt == "BF16" || dt == "I16") return 2;
    if (dt == "F32" || dt == "I32") return 4;
    if (dt == "I64") return 8;
    if (dt == "I8" || dt == "U8" || dt == "F8_E4M3" || dt == "F8_E8M0") return 1;
    return 0;
}

// ---- a JSON reader for the header: objects, arrays, strings, integers; values it has no use for are skipped
struct Json {
    const char* p; const char* end; bool ok = true;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool eat(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
    bool str(std::string& out)
    {
        ws();
        if (p >= end || *p != '"') return ok = false;
        ++p; out.clear();
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return ok = false;
                switch (*p) {
                    case 'n': out += '\n'; break; case 't': out += '\t'; break; case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break; case 'f': out += '\f'; break;
                    case 'u': {                        // keep the escape as written: tensor names are compared byte for byte
                        if (end - p < 5) return ok = false;
                        out += "\\u"; out.append(p + 1, 4); p += 4; break;
                    }
                    default: out += *p;
                }
                ++p;
            } else out += *p++;
        }
        if (p >= end) return ok = false;
        ++p;
        return true;
    }
    bool integer(int64_t& v, bool& is_int)
    {
        ws();
        const char* s = p;
        if (p < end && (*p == '-' || *p == '+')) ++p;
        while (p < end && *p >= '0' && *p <= '9') ++p;
        is_int = true;
        if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) {       // a float: not a valid shape or offset
            is_int = false;
            while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) ++p;
        }
        if (p == s) return ok = false;
        if (is_int) {
            if (p - s > 19) { is_int = false; return true; }
            v = strtoll(std::string(s, p).c_str(), nullptr, 10);
        }
        return true;
    }
    bool skip()                                         // any value
    {
        ws();
        if (p >= end) return ok = false;
        if (*p == '"') { std::string t; return str(t); }
        if (*p == '{' || *p == '[') {
            const char close = *p == '{' ? '}' : ']';
            const bool obj = *p == '{';
            ++p;
            if (eat(close)) return true;
            for (;;) {
                if (obj) { std::string k; if (!str(k) || !eat(':')) return ok = false; }
                if (!skip()) return false;
                if (eat(',')) continue;
                return eat(close) ? true : (ok = false);
            }
        }
        if (!strncmp(p, "true", std::min<size_t>(4, end - p))) { p += 4; return true; }
        if (!strncmp(p, "false", std::min<size_t>(5, end - p))) { p += 5; return true; }
        if (!strncmp(p, "null", std::min<size_t>(4, end - p))) { p += 4; return true; }
        int64_t v; bool ii;
        return integer(v, ii);
    }
};

}  // namespace

struct exl3_checkpoint {
    int fd = -1;
    uint64_t file_size = 0, data_offset = 0;
    std::unordered_map<std::string, Entry> entries;
    std::vector<std::string> names;                  // in file order of the header
    void* pinned = nullptr;
    char err[256] = {0};
};

namespace {

int ck_fail(exl3_checkpoint* ck, int code, const std::string& msg)
{
    if (ck) { strncpy(ck->err, msg.c_str(), sizeof(ck->err) - 1); ck->err[sizeof(ck->err) - 1] = 0; }
    return code;
}

// one tensor entry {"dtype": .., "shape": [..], "data_offsets": [b, e]} with the checks of validate_header
int parse_entry(exl3_checkpoint* ck, Json& j, const std::string& key, Entry& e)
{
    if (!j.eat('{')) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid entry for " + key);
    bool have_shape = false, have_offs = false;
    if (!j.eat('}')) {
        for (;;) {
            std::string f;
            if (!j.str(f) || !j.eat(':')) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid entry for " + key);
            if (f == "dtype") { if (!j.str(e.dtype)) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid dtype for " + key); }
            else if (f == "shape" || f == "data_offsets") {
                std::vector<int64_t> v;
                if (!j.eat('[')) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid " + f + " for " + key);
                if (!j.eat(']')) {
                    for (;;) {
                        int64_t x; bool ii;
                        if (!j.integer(x, ii) || !ii || x < 0) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid " + f + " for " + key);
                        v.push_back(x);
                        if (j.eat(',')) continue;
                        if (!j.eat(']')) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid " + f + " for " + key);
                        break;
                    }
                }
                if (f == "shape") { e.shape = v; have_shape = true; }
                else {
                    if (v.size() != 2 || v[0] > v[1]) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid data_offsets for " + key);
                    e.begin = (uint64_t)v[0]; e.end = (uint64_t)v[1]; have_offs = true;
                }
            } else if (!j.skip()) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid entry for " + key);
            if (j.eat(',')) continue;
            if (!j.eat('}')) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid entry for " + key);
            break;
        }
    }
    if (!have_shape) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid shape for " + key);
    if (!have_offs) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid data_offsets for " + key);
    if (ck->data_offset + e.end > ck->file_size) return ck_fail(ck, EXL3_ERR_INVALID, "Tensor " + key + " extends past end of file");
    const int es = dtype_size(e.dtype);
    if (es) {
        // product with overflow check: a shape must not be able to wrap around to the span's size
        unsigned __int128 n = (unsigned)es;
        for (int64_t d : e.shape) { n *= (unsigned __int128)d; if (n > ((unsigned __int128)1 << 62)) return ck_fail(ck, EXL3_ERR_INVALID, "Size mismatch for " + key); }
        if ((uint64_t)n != e.end - e.begin) return ck_fail(ck, EXL3_ERR_INVALID, "Size mismatch for " + key);
    }
    e.begin += ck->data_offset; e.end += ck->data_offset;
    return EXL3_OK;
}

bool pread_all(int fd, void* dst, size_t n, uint64_t off)
{
    uint8_t* d = (uint8_t*)dst;
    while (n) {
        const ssize_t r = pread(fd, d, n, (off_t)off);
        if (r <= 0) return false;
        d += r; n -= (size_t)r; off += (uint64_t)r;
    }
    return true;
}

// dst[i][o] (fp16, [in_pad, out_pad], zero padded) = src[o][i] (checkpoint order [out, in]); F16, BF16 or F32 source
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<half>(half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<uint16_t>(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }    // bf16 bits

template <typename T>
__global__ void __launch_bounds__(256) transpose_pad_kernel(const T* __restrict__ src, half* __restrict__ dst, int out_f, int in_f,
                                                            int in_pad, int out_pad)
{
    __shared__ float tile[32][33];
    const int o0 = blockIdx.x * 32, i0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int o = o0 + r, i = i0 + tx;
        tile[r][tx] = (o < out_f && i < in_f) ? to_f<T>(src[(size_t)o * in_f + i]) : 0.0f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int i = i0 + r, o = o0 + tx;
        if (i < in_pad && o < out_pad) dst[(size_t)i * out_pad + o] = __float2half_rn(tile[tx][r]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) to_half_pad_kernel(const T* __restrict__ src, half* __restrict__ dst, int n, int n_pad)
{
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < n_pad) dst[i] = i < n ? __float2half_rn(to_f<T>(src[i])) : __float2half(0.0f);
}

}  // namespace

extern "C" int exl3_checkpoint_open(const char* path, exl3_checkpoint** out)
{
    if (!path || !out) return EXL3_ERR_INVALID;
    *out = nullptr;
    exl3_checkpoint* ck = new (std::nothrow) exl3_checkpoint;
    if (!ck) return EXL3_ERR_NOMEM;
    *out = ck;                                       // kept on failure so that exl3_checkpoint_error can be read; close it anyway
    ck->fd = open(path, O_RDONLY);
    struct stat sb;
    if (ck->fd < 0 || fstat(ck->fd, &sb) != 0) return ck_fail(ck, EXL3_ERR_INVALID, std::string("cannot open ") + path);
    ck->file_size = (uint64_t)sb.st_size;
    if (ck->file_size < 8) return ck_fail(ck, EXL3_ERR_INVALID, "too small to be a safetensors file");
    uint64_t hs = 0;
    if (!pread_all(ck->fd, &hs, 8, 0)) return ck_fail(ck, EXL3_ERR_INVALID, "cannot read the header size");
    if (!(hs > 0 && hs <= MAX_HEADER)) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid safetensors header size");
    if (8 + hs > ck->file_size) return ck_fail(ck, EXL3_ERR_INVALID, "Truncated safetensors header");
    std::vector<char> buf((size_t)hs);
    if (!pread_all(ck->fd, buf.data(), (size_t)hs, 8)) return ck_fail(ck, EXL3_ERR_INVALID, "cannot read the header");
    ck->data_offset = 8 + hs;
    Json j{buf.data(), buf.data() + buf.size()};
    if (!j.eat('{')) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid safetensors header");
    if (!j.eat('}')) {
        for (;;) {
            std::string key;
            if (!j.str(key) || !j.eat(':')) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid safetensors header");
            if (key == "__metadata__") { if (!j.skip()) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid safetensors header"); }
            else {
                Entry e;
                const int rc = parse_entry(ck, j, key, e);
                if (rc) return rc;
                if (ck->entries.emplace(key, e).second) ck->names.push_back(key);
            }
            if (j.eat(',')) continue;
            if (!j.eat('}')) return ck_fail(ck, EXL3_ERR_INVALID, "Invalid safetensors header");
            break;
        }
    }
    return EXL3_OK;
}

extern "C" void exl3_checkpoint_close(exl3_checkpoint* ck)
{
    if (!ck) return;
    if (ck->fd >= 0) close(ck->fd);
    if (ck->pinned) cudaFreeHost(ck->pinned);
    delete ck;
}

extern "C" const char* exl3_checkpoint_error(const exl3_checkpoint* ck) { return ck ? ck->err : "null checkpoint"; }
extern "C" int exl3_checkpoint_count(const exl3_checkpoint* ck) { return ck ? (int)ck->names.size() : 0; }
extern "C" const char* exl3_checkpoint_name(const exl3_checkpoint* ck, int i)
{
    return (ck && i >= 0 && i < (int)ck->names.size()) ? ck->names[i].c_str() : nullptr;
}
extern "C" int exl3_checkpoint_has(const exl3_checkpoint* ck, const char* name)
{
    return ck && name && ck->entries.count(name) ? 1 : 0;
}

extern "C" int exl3_checkpoint_info(const exl3_checkpoint* ck, const char* name, char* dtype, int dtype_cap, int64_t* shape,
                                    int shape_cap, int* ndim, uint64_t* bytes)
{
    if (!ck || !name) return EXL3_ERR_INVALID;
    auto it = ck->entries.find(name);
    if (it == ck->entries.end()) return EXL3_ERR_INVALID;
    const Entry& e = it->second;
    if (dtype && dtype_cap > 0) { strncpy(dtype, e.dtype.c_str(), dtype_cap - 1); dtype[dtype_cap - 1] = 0; }
    if (ndim) *ndim = (int)e.shape.size();
    if (shape) for (int i = 0; i < shape_cap && i < (int)e.shape.size(); ++i) shape[i] = e.shape[i];
    if (bytes) *bytes = e.end - e.begin;
    return EXL3_OK;
}

// Reads a tensor's bytes into device memory (dst_device, at least `capacity` bytes): positional reads into a pinned
// buffer, one cudaMemcpyAsync per piece on `stream`, the host waiting for each piece before it reuses the buffer.
extern "C" int exl3_checkpoint_read(exl3_checkpoint* ck, const char* name, void* dst_device, size_t capacity, exl3_stream stream)
{
    if (!ck || !name || !dst_device) return EXL3_ERR_INVALID;
    auto it = ck->entries.find(name);
    if (it == ck->entries.end()) return ck_fail(ck, EXL3_ERR_INVALID, std::string("no tensor ") + name);
    const Entry& e = it->second;
    const uint64_t n = e.end - e.begin;
    if (n > capacity) return ck_fail(ck, EXL3_ERR_INVALID, std::string("destination too small for ") + name);
    if (!ck->pinned && cudaMallocHost(&ck->pinned, STAGE_BYTES) != cudaSuccess) { cudaGetLastError(); return ck_fail(ck, EXL3_ERR_NOMEM, "no pinned staging memory"); }
    cudaStream_t st = (cudaStream_t)stream;
    for (uint64_t off = 0; off < n; off += STAGE_BYTES) {
        const size_t piece = (size_t)std::min<uint64_t>(STAGE_BYTES, n - off);
        if (!pread_all(ck->fd, ck->pinned, piece, e.begin + off)) return ck_fail(ck, EXL3_ERR_INVALID, std::string("short read in ") + name);
        if (cudaMemcpyAsync((uint8_t*)dst_device + off, ck->pinned, piece, cudaMemcpyHostToDevice, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess) { cudaGetLastError(); return ck_fail(ck, EXL3_ERR_CUDA, std::string("copy failed for ") + name); }
    }
    return EXL3_OK;
}

// Linear::load (src/modules.rs:97-165).  Tries `key`, then `alt_key` (may be NULL).  An EXL3 layer needs
// <k>.trellis [k/16, n/16, 16 K] I16 with <k>.suh [k] and <k>.svh [n] F16 (the packed sign form <k>.su is not supported,
// as in the reference's port); the presence of <k>.mcg / <k>.mul1 selects the codebook; <k>.bias is optional.  A dense
// layer is <k>.weight [out, in] (F16, BF16 or F32), stored transposed and zero-padded as fp16 [in_pad, out_pad].  All
// device memory of the layer is one allocation owned by it (exl3_linear_free).
namespace {

// `find(name)` returns the opened file that holds tensor `name`, or NULL; errors are reported into `rep`'s buffer
template <typename Find>
int linear_load_impl(Find find, exl3_checkpoint* rep, exl3_stream stream, const char* key, const char* alt_key, int in_features,
                     int out_features, int trim_padded_out, float softcap, exl3_linear_layer* out)
{
    exl3_checkpoint* ck = rep;
    if (!ck || !key || !out || in_features <= 0 || out_features <= 0) return EXL3_ERR_INVALID;
    memset(out, 0, sizeof(*out));
    const int inf = (in_features + 127) / 128 * 128, outf = (out_features + 127) / 128 * 128;
    cudaStream_t st = (cudaStream_t)stream;
    const char* keys[2] = {key, alt_key};
    for (const char* k : keys) {
        if (!k) continue;
        const std::string base(k);
        auto has = [&](const char* suf) { return find(base + suf) != nullptr; };
        auto entry = [&](const char* suf) -> const Entry& { return find(base + suf)->entries.at(base + suf); };
        auto bytes_of = [&](const char* suf) { const Entry& e = entry(suf); return (size_t)(e.end - e.begin); };
        auto read = [&](const char* suf, void* dst, size_t cap) {
            exl3_checkpoint* src = find(base + suf);
            const int rc = exl3_checkpoint_read(src, (base + suf).c_str(), dst, cap, stream);
            if (rc && src != ck) ck_fail(ck, rc, src->err);
            return rc;
        };
        auto align = [](size_t x) { return (x + 255) & ~(size_t)255; };
        if (has(".trellis")) {
            const Entry& tr = entry(".trellis");
            if (tr.dtype != "I16" || tr.shape.size() != 3 || tr.shape[2] % 16 != 0 || tr.shape[2] < 16 || tr.shape[2] > 128)
                return ck_fail(ck, EXL3_ERR_INVALID, base + ".trellis: expected I16 [k/16, n/16, 16 K]");
            if (tr.shape[0] * 16 != inf || tr.shape[1] * 16 != outf)
                return ck_fail(ck, EXL3_ERR_INVALID, base + ".trellis does not match the padded features");
            if (!has(".suh")) return ck_fail(ck, EXL3_ERR_UNSUPPORTED, base + ": only unpacked suh/svh supported");
            if (!has(".svh")) return ck_fail(ck, EXL3_ERR_INVALID, base + ".svh missing");
            const Entry& su = entry(".suh"); const Entry& sv = entry(".svh");
            if (su.dtype != "F16" || sv.dtype != "F16" || bytes_of(".suh") != (size_t)inf * 2 || bytes_of(".svh") != (size_t)outf * 2)
                return ck_fail(ck, EXL3_ERR_INVALID, base + ": suh/svh must be F16 of the padded sizes");
            if (has(".mcg") && has(".mul1")) return ck_fail(ck, EXL3_ERR_INVALID, base + ": both mcg and mul1");
            const bool bias = has(".bias");
            if (bias && (entry(".bias").dtype != "F16" || bytes_of(".bias") > (size_t)outf * 2))
                return ck_fail(ck, EXL3_ERR_INVALID, base + ".bias: expected F16 of at most the padded width");
            const size_t o_tr = 0, o_su = align(bytes_of(".trellis")), o_sv = o_su + align((size_t)inf * 2), o_b = o_sv + align((size_t)outf * 2);
            const size_t total = o_b + (bias ? align((size_t)outf * 2) : 0);
            uint8_t* mem = nullptr;
            if (cudaMalloc(&mem, total) != cudaSuccess) { cudaGetLastError(); return ck_fail(ck, EXL3_ERR_NOMEM, "device memory for " + base); }
            int rc = read(".trellis", mem + o_tr, bytes_of(".trellis"));
            if (!rc) rc = read(".suh", mem + o_su, (size_t)inf * 2);
            if (!rc) rc = read(".svh", mem + o_sv, (size_t)outf * 2);
            if (!rc && bias) {
                if (cudaMemsetAsync(mem + o_b, 0, (size_t)outf * 2, st) != cudaSuccess) rc = EXL3_ERR_CUDA;
                if (!rc) rc = read(".bias", mem + o_b, (size_t)outf * 2);
            }
            if (rc) { cudaFree(mem); return rc; }
            out->w.trellis = mem + o_tr; out->w.suh = mem + o_su; out->w.svh = mem + o_sv;
            out->w.k = inf; out->w.n = outf; out->w.K = (int)(tr.shape[2] / 16);
            out->w.cb = has(".mcg") ? 1 : (has(".mul1") ? 2 : 0);
            out->bias = bias ? mem + o_b : nullptr;
            out->in_unpadded = in_features; out->out_unpadded = out_features;
            out->trim_padded_out = trim_padded_out; out->softcap = softcap;
            return EXL3_OK;
        }
        if (has(".weight")) {
            const Entry& w = entry(".weight");
            const int es = dtype_size(w.dtype);
            if (w.shape.size() != 2 || !(w.dtype == "F16" || w.dtype == "BF16" || w.dtype == "F32") || w.shape[0] > outf || w.shape[1] > inf)
                return ck_fail(ck, EXL3_ERR_INVALID, base + ".weight: expected a float matrix [out, in] within the padded sizes");
            const int wo = (int)w.shape[0], wi = (int)w.shape[1];
            const bool bias = has(".bias");
            const Entry* be = bias ? &entry(".bias") : nullptr;
            if (bias && (!(be->dtype == "F16" || be->dtype == "BF16" || be->dtype == "F32") || be->shape.size() != 1 || be->shape[0] > outf))
                return ck_fail(ck, EXL3_ERR_INVALID, base + ".bias: expected a float vector of at most the padded width");
            const size_t o_w = 0, o_b = align((size_t)inf * outf * 2), o_raw = o_b + align((size_t)outf * 2);
            const size_t raw_bytes = std::max(bytes_of(".weight"), bias ? bytes_of(".bias") : (size_t)0);
            uint8_t* mem = nullptr;
            if (cudaMalloc(&mem, o_raw + align(raw_bytes)) != cudaSuccess) { cudaGetLastError(); return ck_fail(ck, EXL3_ERR_NOMEM, "device memory for " + base); }
            int rc = read(".weight", mem + o_raw, raw_bytes);
            if (!rc) {
                const dim3 grid((outf + 31) / 32, (inf + 31) / 32);
                if (es == 4) transpose_pad_kernel<float><<<grid, 256, 0, st>>>((const float*)(mem + o_raw), (half*)(mem + o_w), wo, wi, inf, outf);
                else if (w.dtype == "BF16") transpose_pad_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)(mem + o_raw), (half*)(mem + o_w), wo, wi, inf, outf);
                else transpose_pad_kernel<half><<<grid, 256, 0, st>>>((const half*)(mem + o_raw), (half*)(mem + o_w), wo, wi, inf, outf);
                if (cudaStreamSynchronize(st) != cudaSuccess) rc = EXL3_ERR_CUDA;
            }
            if (!rc && bias) {
                rc = read(".bias", mem + o_raw, raw_bytes);
                if (!rc) {
                    const int nb = (int)be->shape[0];
                    if (be->dtype == "F32") to_half_pad_kernel<float><<<(outf + 255) / 256, 256, 0, st>>>((const float*)(mem + o_raw), (half*)(mem + o_b), nb, outf);
                    else if (be->dtype == "BF16") to_half_pad_kernel<uint16_t><<<(outf + 255) / 256, 256, 0, st>>>((const uint16_t*)(mem + o_raw), (half*)(mem + o_b), nb, outf);
                    else to_half_pad_kernel<half><<<(outf + 255) / 256, 256, 0, st>>>((const half*)(mem + o_raw), (half*)(mem + o_b), nb, outf);
                    if (cudaStreamSynchronize(st) != cudaSuccess) rc = EXL3_ERR_CUDA;
                }
            }
            if (rc) { cudaGetLastError(); cudaFree(mem); return ck_fail(ck, rc, "loading " + base + " failed"); }
            out->w.trellis = nullptr; out->w.k = inf; out->w.n = outf; out->w.K = 0; out->w.cb = 0;
            out->dense = mem + o_w; out->bias = bias ? mem + o_b : nullptr;
            out->in_unpadded = in_features; out->out_unpadded = out_features;
            out->trim_padded_out = trim_padded_out; out->softcap = softcap;
            return EXL3_OK;
        }
    }
    return ck_fail(ck, EXL3_ERR_INVALID, std::string("No supported quant tensors for ") + key);
}

}  // namespace

extern "C" int exl3_linear_load(exl3_checkpoint* ck, exl3_stream stream, const char* key, const char* alt_key, int in_features,
                                int out_features, int trim_padded_out, float softcap, exl3_linear_layer* out)
{
    if (!ck) return EXL3_ERR_INVALID;
    auto find = [ck](const std::string& name) -> exl3_checkpoint* { return ck->entries.count(name) ? ck : nullptr; };
    return linear_load_impl(find, ck, stream, key, alt_key, in_features, out_features, trim_padded_out, softcap, out);
}

extern "C" void exl3_linear_free(exl3_linear_layer* layer)
{
    if (!layer) return;
    // the layer's tensors live in one allocation that starts at the trellis (EXL3) or at the dense weight
    void* base = layer->w.trellis ? const_cast<void*>(layer->w.trellis) : const_cast<void*>(layer->dense);
    if (base) cudaFree(base);
    memset(layer, 0, sizeof(*layer));
}

// ---------------------------------------------------------------------------------------------- whole dense model
// Model::load for the dense transformer family of the step runner (src/model.rs:262-420, src/modules.rs:470-490,985-1000):
// <pfx>.embed_tokens.weight, <pfx>.layers.<i>.{input_layernorm, post_attention_layernorm}.weight,
// .self_attn.{q,k,v,o}_proj, .self_attn.{q,k}_norm.weight (optional), .mlp.{gate,up,down}_proj, <pfx>.norm.weight, lm_head.
// Projections must be EXL3 tensors (the step runner has no dense projection path); vectors and the embedding table may
// be F16, BF16 or F32 and are kept as fp16.  Tensors may be spread over several files.
struct exl3_loaded_model {
    exl3_model model;
    std::vector<exl3_layer> layers;
    std::vector<exl3_linear_layer> linears;      // owners of the projections' device memory
    std::vector<void*> buffers;                  // norms, embedding, rotary frequencies
    char err[256] = {0};
};

namespace {

struct Shards {
    exl3_checkpoint* const* ck; int n;
    exl3_checkpoint* find(const std::string& name) const
    {
        for (int i = 0; i < n; ++i) if (ck[i] && ck[i]->entries.count(name)) return ck[i];
        return nullptr;
    }
};

int lm_fail(exl3_loaded_model* m, int code, const std::string& msg)
{
    strncpy(m->err, msg.c_str(), sizeof(m->err) - 1); m->err[sizeof(m->err) - 1] = 0;
    return code;
}

// a float tensor of exactly `numel` elements as fp16 on the device
int load_half(exl3_loaded_model* m, const Shards& sh, cudaStream_t st, const std::string& name, size_t numel, void** out)
{
    exl3_checkpoint* ck = sh.find(name);
    if (!ck) return lm_fail(m, EXL3_ERR_INVALID, "missing tensor " + name);
    const Entry& e = ck->entries.at(name);
    const int es = dtype_size(e.dtype);
    if (!(e.dtype == "F16" || e.dtype == "BF16" || e.dtype == "F32") || (size_t)(e.end - e.begin) != numel * es)
        return lm_fail(m, EXL3_ERR_INVALID, name + ": expected " + std::to_string(numel) + " float elements");
    uint8_t* dst = nullptr;
    const size_t half_bytes = (numel * 2 + 255) & ~(size_t)255;
    if (cudaMalloc(&dst, half_bytes + (e.dtype == "F16" ? 0 : numel * es)) != cudaSuccess) { cudaGetLastError(); return lm_fail(m, EXL3_ERR_NOMEM, "device memory for " + name); }
    m->buffers.push_back(dst);
    int rc = exl3_checkpoint_read(ck, name.c_str(), e.dtype == "F16" ? dst : dst + half_bytes, numel * es, (exl3_stream)st);
    if (rc) return lm_fail(m, rc, ck->err);
    if (e.dtype != "F16") {
        if (numel > 0x7fffffffull) return lm_fail(m, EXL3_ERR_UNSUPPORTED, name + ": too large to convert");
        const unsigned grid = (unsigned)((numel + 255) / 256);
        if (e.dtype == "F32") to_half_pad_kernel<float><<<grid, 256, 0, st>>>((const float*)(dst + half_bytes), (half*)dst, (int)numel, (int)numel);
        else to_half_pad_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)(dst + half_bytes), (half*)dst, (int)numel, (int)numel);
        if (cudaStreamSynchronize(st) != cudaSuccess) { cudaGetLastError(); return lm_fail(m, EXL3_ERR_CUDA, "conversion of " + name + " failed"); }
    }
    *out = dst;
    return EXL3_OK;
}

int load_proj(exl3_loaded_model* m, const Shards& sh, cudaStream_t st, const std::string& key, int in_f, int out_f, exl3_linear* out)
{
    exl3_checkpoint* ck = sh.find(key + ".trellis");
    if (!ck) return lm_fail(m, sh.find(key + ".weight") ? EXL3_ERR_UNSUPPORTED : EXL3_ERR_INVALID,
                            key + ": the step runner needs an EXL3 tensor here");
    if (in_f % 128 || out_f % 128) return lm_fail(m, EXL3_ERR_UNSUPPORTED, key + ": features must be multiples of 128");
    exl3_linear_layer L;
    auto find = [&sh](const std::string& name) { return sh.find(name); };
    const int rc = linear_load_impl(find, ck, (exl3_stream)st, key.c_str(), nullptr, in_f, out_f, 0, 0.0f, &L);
    if (rc) return lm_fail(m, rc, ck->err);
    m->linears.push_back(L);
    if (L.bias) return lm_fail(m, EXL3_ERR_UNSUPPORTED, key + ": projections with a bias are not supported by the step runner");
    *out = L.w;
    return EXL3_OK;
}

}  // namespace

extern "C" int exl3_model_load(exl3_checkpoint* const* shards, int n_shards, exl3_stream stream, const char* prefix, int n_layers,
                               int hidden, int nq, int nkv, int hd, int inter, int vocab, float norm_eps, float rope_theta,
                               const exl3_pool* pool, exl3_loaded_model** out)
{
    if (!shards || n_shards <= 0 || !prefix || !pool || !out) return EXL3_ERR_INVALID;
    if (n_layers <= 0 || hidden <= 0 || nq <= 0 || nkv <= 0 || hd <= 0 || hd % 2 || inter <= 0 || vocab <= 0 || rope_theta <= 0.0f)
        return EXL3_ERR_INVALID;
    exl3_loaded_model* m = new (std::nothrow) exl3_loaded_model;
    if (!m) return EXL3_ERR_NOMEM;
    *out = m;                                        // kept on failure for exl3_model_error; free it in either case
    memset(&m->model, 0, sizeof(m->model));
    const Shards sh{shards, n_shards};
    cudaStream_t st = (cudaStream_t)stream;
    const std::string pfx(prefix);
    int k_bits = 0, v_bits = 0;
    exl3_pool_kv_bits(pool, &k_bits, &v_bits);
    if (k_bits != v_bits) return lm_fail(m, EXL3_ERR_UNSUPPORTED, "the step runner needs equal K and V code widths");
    m->layers.resize(n_layers);
    m->linears.reserve((size_t)n_layers * 7 + 1);
    int rc;
    void* p = nullptr;
    if ((rc = load_half(m, sh, st, pfx + ".embed_tokens.weight", (size_t)vocab * hidden, &p))) return rc;
    m->model.embed = p;
    for (int i = 0; i < n_layers; ++i) {
        const std::string key = pfx + ".layers." + std::to_string(i);
        exl3_layer& L = m->layers[i];
        memset(&L, 0, sizeof(L));
        if ((rc = load_half(m, sh, st, key + ".input_layernorm.weight", hidden, &p))) return rc;
        L.attn_norm = p;
        if ((rc = load_half(m, sh, st, key + ".post_attention_layernorm.weight", hidden, &p))) return rc;
        L.mlp_norm = p;
        if (sh.find(key + ".self_attn.q_norm.weight")) {
            if ((rc = load_half(m, sh, st, key + ".self_attn.q_norm.weight", hd, &p))) return rc;
            L.q_norm = p;
            if ((rc = load_half(m, sh, st, key + ".self_attn.k_norm.weight", hd, &p))) return rc;
            L.k_norm = p;
        }
        if ((rc = load_proj(m, sh, st, key + ".self_attn.q_proj", hidden, nq * hd, &L.q_proj))) return rc;
        if ((rc = load_proj(m, sh, st, key + ".self_attn.k_proj", hidden, nkv * hd, &L.k_proj))) return rc;
        if ((rc = load_proj(m, sh, st, key + ".self_attn.v_proj", hidden, nkv * hd, &L.v_proj))) return rc;
        if ((rc = load_proj(m, sh, st, key + ".self_attn.o_proj", nq * hd, hidden, &L.o_proj))) return rc;
        if ((rc = load_proj(m, sh, st, key + ".mlp.gate_proj", hidden, inter, &L.gate_proj))) return rc;
        if ((rc = load_proj(m, sh, st, key + ".mlp.up_proj", hidden, inter, &L.up_proj))) return rc;
        if ((rc = load_proj(m, sh, st, key + ".mlp.down_proj", inter, hidden, &L.down_proj))) return rc;
        void *k = nullptr, *v = nullptr, *sk = nullptr, *sv = nullptr;
        if (exl3_pool_layer(pool, i, &k, &v, &sk, &sv) != EXL3_OK) return lm_fail(m, EXL3_ERR_INVALID, "the pool has fewer layers than the model");
        if (k_bits == 0) { L.k_cache = k; L.v_cache = v; }
        else { L.qk = k; L.qv = v; L.sk = sk; L.sv = sv; }
    }
    if ((rc = load_half(m, sh, st, pfx + ".norm.weight", hidden, &p))) return rc;
    m->model.final_norm = p;
    if ((rc = load_proj(m, sh, st, "lm_head", hidden, vocab, &m->model.lm_head))) return rc;
    // rotary frequencies theta^(-2i/hd), i < hd/2 (src/rope.rs:82-86)
    std::vector<float> inv(hd / 2);
    for (int i = 0; i < hd / 2; ++i) inv[i] = 1.0f / powf(rope_theta, (float)(2 * i) / (float)hd);
    float* dinv = nullptr;
    if (cudaMalloc(&dinv, inv.size() * 4) != cudaSuccess) { cudaGetLastError(); return lm_fail(m, EXL3_ERR_NOMEM, "device memory for the rotary table"); }
    m->buffers.push_back(dinv);
    if (cudaMemcpyAsync(dinv, inv.data(), inv.size() * 4, cudaMemcpyHostToDevice, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return lm_fail(m, EXL3_ERR_CUDA, "copy of the rotary table failed");
    }
    exl3_model& M = m->model;
    M.n_layers = n_layers; M.hidden = hidden; M.nq = nq; M.nkv = nkv; M.hd = hd; M.inter = inter; M.vocab = vocab;
    M.kv_bits = k_bits; M.pages = exl3_pool_num_pages(pool); M.norm_eps = norm_eps; M.attn_factor = 1.0f;
    M.rope_mode = EXL3_ROPE_NEOX; M.n_freq = hd / 2; M.inv_freq = dinv; M.layers = m->layers.data();
    return EXL3_OK;
}

extern "C" const exl3_model* exl3_model_get(const exl3_loaded_model* m) { return m ? &m->model : nullptr; }
extern "C" const char* exl3_model_error(const exl3_loaded_model* m) { return m ? m->err : "null model"; }
extern "C" void exl3_model_free(exl3_loaded_model* m)
{
    if (!m) return;
    for (auto& L : m->linears) exl3_linear_free(&L);
    for (void* b : m->buffers) cudaFree(b);
    delete m;
}

