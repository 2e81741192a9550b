// Paged KV pools and the page allocator: the host-side state of a continuous batch.
//
// Follows the reference's pools (src/paged.rs:18-92: one K and one V plane per layer, [pages,256,nkv,hd] fp16, or packed
// int32 codes [pages,256,groups*bits] + fp16 scales [pages,256,groups] per layer) and its page table
// (src/paged.rs:330-506: free list, a reference count per physical page, chained content hashes of complete pages so that
// later sequences with the same prompt prefix share pages, least-recently-released eviction of unreferenced hashed
// pages).  The pools live in device memory owned by this object; the page table is plain host state.
#include "common.cuh"
#include <deque>
#include <new>
#include <unordered_map>
#include <vector>

namespace {

struct PageHash {
    uint64_t a, b;
    bool operator==(const PageHash& o) const { return a == o.a && b == o.b; }
};
struct PageHashHasher { size_t operator()(const PageHash& h) const { return (size_t)(h.a ^ (h.b * 0x9E3779B97F4A7C15ull)); } };

// two independent 64-bit mixes over (seed, previous page's hash, the page's 256 token ids)
uint64_t mix64(uint64_t x)
{
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}
PageHash chain_hash(const PageHash* prev, const int64_t* ids, int n)
{
    auto run = [&](uint64_t seed) {
        uint64_t h = mix64(seed);
        h = mix64(h ^ (prev ? prev->a : 0x5151515151515151ull));
        h = mix64(h ^ (prev ? prev->b : 0xA3A3A3A3A3A3A3A3ull));
        for (int i = 0; i < n; ++i) h = mix64(h ^ (uint64_t)ids[i]) + seed;
        return h;
    };
    return PageHash{run(0x9E3779B97F4A7C15ull), run(0xC2B2AE3D27D4EB4Full)};
}

}  // namespace

struct exl3_pool {
    int device, n_layers, pages, nkv, hd, k_bits, v_bits;
    std::vector<void*> k, v, sk, sv;         // per layer: fp16 planes (k, v) or codes (k, v) + scales (sk, sv)
    // page table
    std::vector<int32_t> free_list;          // popped from the back: pages are handed out in ascending order at first
    std::vector<uint32_t> rc;
    std::vector<uint8_t> hashed;
    std::vector<PageHash> hash;
    std::unordered_map<PageHash, int32_t, PageHashHasher> by_hash;
    std::deque<int32_t> reclaimable;         // rc == 0 pages that still carry a hash, oldest first
    std::vector<int32_t> evicted;            // hashed pages repurposed since the last drain
    int dedup;
    uint64_t cached_tokens, prompt_tokens;

    int num_free() const { return (int)(free_list.size() + reclaimable.size()); }
    int32_t take_one()
    {
        int32_t id;
        if (!free_list.empty()) { id = free_list.back(); free_list.pop_back(); }
        else {
            id = reclaimable.front(); reclaimable.pop_front();
            if (hashed[id]) {
                auto it = by_hash.find(hash[id]);
                if (it != by_hash.end() && it->second == id) by_hash.erase(it);
                evicted.push_back(id);
            }
        }
        rc[id] = 1; hashed[id] = 0;
        return id;
    }
    void acquire(int32_t id)
    {
        if (rc[id] == 0)
            for (auto it = reclaimable.begin(); it != reclaimable.end(); ++it)
                if (*it == id) { reclaimable.erase(it); break; }
        rc[id]++;
    }
};

extern "C" int exl3_pool_create(int device, int n_layers, int pages, int nkv, int hd, int k_bits, int v_bits, exl3_pool** out)
{
    if (!out) return EXL3_ERR_INVALID;
    *out = nullptr;
    if (n_layers < 0 || pages <= 0 || nkv <= 0 || hd <= 0 || (nkv * hd) % 32) return EXL3_ERR_INVALID;
    const bool quant = k_bits != 0 || v_bits != 0;
    if (quant && (k_bits < 2 || k_bits > 8 || v_bits < 2 || v_bits > 8)) return EXL3_ERR_INVALID;
    // n_layers = 0: a page table without planes (no device is touched)
    if (n_layers > 0 && cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return EXL3_ERR_CUDA; }
    exl3_pool* p = new (std::nothrow) exl3_pool();
    if (!p) return EXL3_ERR_NOMEM;
    p->device = device; p->n_layers = n_layers; p->pages = pages; p->nkv = nkv; p->hd = hd; p->k_bits = k_bits; p->v_bits = v_bits;
    p->dedup = 0; p->cached_tokens = p->prompt_tokens = 0;
    const size_t tokens = (size_t)pages * EXL3_PAGE, groups = (size_t)nkv * hd / 32;
    const size_t kb = quant ? tokens * groups * k_bits * 4 : tokens * nkv * hd * 2;
    const size_t vb = quant ? tokens * groups * v_bits * 4 : tokens * nkv * hd * 2;
    const size_t sb = quant ? tokens * groups * 2 : 0;
    bool ok = true;
    auto take = [&](std::vector<void*>& dst, size_t bytes) {
        void* ptr = nullptr;
        if (ok && bytes) ok = cudaMalloc(&ptr, bytes) == cudaSuccess && cudaMemset(ptr, 0, bytes) == cudaSuccess;
        dst.push_back(ptr);
    };
    for (int l = 0; l < n_layers; ++l) { take(p->k, kb); take(p->v, vb); take(p->sk, sb); take(p->sv, sb); }
    if (!ok) { cudaGetLastError(); exl3_pool_destroy(p); return EXL3_ERR_NOMEM; }
    p->rc.assign(pages, 0); p->hashed.assign(pages, 0); p->hash.assign(pages, PageHash{0, 0});
    p->free_list.reserve(pages);
    for (int i = pages - 1; i >= 0; --i) p->free_list.push_back(i);
    *out = p;
    return EXL3_OK;
}

extern "C" void exl3_pool_destroy(exl3_pool* p)
{
    if (!p) return;
    if (p->n_layers > 0) cudaSetDevice(p->device);
    for (auto* vec : {&p->k, &p->v, &p->sk, &p->sv})
        for (void* ptr : *vec) if (ptr) cudaFree(ptr);
    delete p;
}

extern "C" int exl3_pool_layer(const exl3_pool* p, int layer, void** k, void** v, void** sk, void** sv)
{
    if (!p || layer < 0 || layer >= p->n_layers) return EXL3_ERR_INVALID;
    if (k) *k = p->k[layer];
    if (v) *v = p->v[layer];
    if (sk) *sk = p->sk[layer];
    if (sv) *sv = p->sv[layer];
    return EXL3_OK;
}

extern "C" int exl3_pool_num_pages(const exl3_pool* p) { return p ? p->pages : 0; }
extern "C" void exl3_pool_kv_bits(const exl3_pool* p, int* k_bits, int* v_bits)
{
    if (k_bits) *k_bits = p ? p->k_bits : 0;
    if (v_bits) *v_bits = p ? p->v_bits : 0;
}
extern "C" int exl3_pool_num_free(const exl3_pool* p) { return p ? p->num_free() : 0; }
extern "C" int exl3_pool_refcount(const exl3_pool* p, int page) { return (p && page >= 0 && page < p->pages) ? (int)p->rc[page] : -1; }
extern "C" void exl3_pool_set_dedup(exl3_pool* p, int on) { if (p) p->dedup = on ? 1 : 0; }

extern "C" int exl3_pool_alloc(exl3_pool* p, int n, int32_t* out_pages)
{
    if (!p || n < 0 || (n > 0 && !out_pages)) return EXL3_ERR_INVALID;
    if (p->num_free() < n) return EXL3_ERR_NOMEM;
    for (int i = 0; i < n; ++i) out_pages[i] = p->take_one();
    return EXL3_OK;
}

extern "C" int exl3_pool_alloc_prefix(exl3_pool* p, const int64_t* prompt_ids, int n_ids, int gen_reserve, int32_t* out_block,
                                      int block_capacity, int* out_count, int64_t* out_matched_tokens)
{
    if (!p || n_ids < 0 || gen_reserve < 0 || (n_ids > 0 && !prompt_ids) || !out_block || !out_count) return EXL3_ERR_INVALID;
    const int need = (int)(((int64_t)n_ids + gen_reserve + EXL3_PAGE - 1) / EXL3_PAGE);
    if (need > block_capacity) return EXL3_ERR_INVALID;
    std::vector<int32_t> hits;
    if (p->dedup) {
        PageHash prev; bool have_prev = false;
        for (int pg = 0; pg < n_ids / EXL3_PAGE; ++pg) {
            const PageHash h = chain_hash(have_prev ? &prev : nullptr, prompt_ids + (size_t)pg * EXL3_PAGE, EXL3_PAGE);
            auto it = p->by_hash.find(h);
            if (it == p->by_hash.end()) break;
            hits.push_back(it->second); prev = h; have_prev = true;
        }
    }
    // a prefix hit on a reclaimable page takes it off the list the fresh pages would come from
    int revive = 0;
    for (int32_t id : hits) if (p->rc[id] == 0) ++revive;
    if (p->num_free() - revive < need - (int)hits.size()) return EXL3_ERR_NOMEM;
    for (int32_t id : hits) p->acquire(id);
    int cnt = 0;
    for (int32_t id : hits) out_block[cnt++] = id;
    while (cnt < need) out_block[cnt++] = p->take_one();
    *out_count = cnt;
    if (out_matched_tokens) *out_matched_tokens = (int64_t)hits.size() * EXL3_PAGE;
    p->cached_tokens += (uint64_t)hits.size() * EXL3_PAGE;
    p->prompt_tokens += (uint64_t)n_ids;
    return EXL3_OK;
}

extern "C" int exl3_pool_register_page_hash(exl3_pool* p, int page, int prev_page, const int64_t* token_ids, int n_ids)
{
    if (!p || page < 0 || page >= p->pages || !token_ids) return EXL3_ERR_INVALID;
    if (p->hashed[page] || n_ids != EXL3_PAGE) return EXL3_OK;               // idempotent; only complete pages are hashed
    const PageHash* prev = nullptr;
    if (prev_page >= 0) {
        if (prev_page >= p->pages || !p->hashed[prev_page]) return EXL3_ERR_INVALID;
        prev = &p->hash[prev_page];
    }
    const PageHash h = chain_hash(prev, token_ids, n_ids);
    p->hash[page] = h; p->hashed[page] = 1;
    p->by_hash.emplace(h, page);                                             // first page registered for a hash keeps it
    return EXL3_OK;
}

extern "C" int exl3_pool_release(exl3_pool* p, const int32_t* pages, int n)
{
    if (!p || n < 0 || (n > 0 && !pages)) return EXL3_ERR_INVALID;
    for (int i = 0; i < n; ++i) {
        const int32_t id = pages[i];
        if (id < 0 || id >= p->pages) return EXL3_ERR_INVALID;
        if (p->rc[id] > 0 && --p->rc[id] == 0) {
            if (p->hashed[id]) p->reclaimable.push_back(id);
            else p->free_list.push_back(id);
        }
    }
    return EXL3_OK;
}

extern "C" int exl3_pool_drain_evicted(exl3_pool* p, int32_t* out_pages, int capacity)
{
    if (!p || capacity < 0) return EXL3_ERR_INVALID;
    const int n = (int)p->evicted.size() < capacity ? (int)p->evicted.size() : capacity;
    for (int i = 0; i < n; ++i) out_pages[i] = p->evicted[i];
    p->evicted.erase(p->evicted.begin(), p->evicted.begin() + n);
    return n;
}

extern "C" void exl3_pool_prefix_stats(const exl3_pool* p, uint64_t* cached_tokens, uint64_t* prompt_tokens)
{
    if (cached_tokens) *cached_tokens = p ? p->cached_tokens : 0;
    if (prompt_tokens) *prompt_tokens = p ? p->prompt_tokens : 0;
}
