// Host-side life cycle of a paged KV cache: a page allocator with reference counts and a
// prefix cache whose entries share pages instead of copying rows.
//
// The reference keeps contiguous caches and snapshots a prompt prefix by copying the first
// prefix_len rows of every head into a fresh buffer (src/model/executor.rs:1136-1262), restores
// by copying them back (:1264-1350), and keeps at most METALLIC_KV_PREFIX_CACHE_ENTRIES snapshots
// (default 8, clamped to 1..64, :266-279) in a deque: a store replaces the entry with the same
// key (or, without key, the same tokens) and drops the oldest entry when full (:1584-1636); a
// lookup without key takes the longest snapshot that is a prefix of the prompt, the later entry
// on ties (:1352-1375); a keyed lookup takes, among the entries of that key that are not longer
// than the prompt, the longest common prefix, zero excluded, later entry on ties (:1425-1515);
// a hit moves the entry to the back (:1388-1398, :1535-1546).  The same rules are kept here; what
// changes is the payload: with pages a snapshot is a list of page ids whose reference count is
// raised, a restore hands the ids to the new sequence, and only a page that the new sequence
// will write into (the last one when the matched prefix ends inside it) has to be copied first.
#include <cstring>
#include <deque>
#include <string>
#include <vector>

#include <new>

#include "../../include/metallic_cuda.h"

struct MfPagePool {
    std::vector<uint32_t> refs;       // per page
    std::vector<uint32_t> free_list;  // stack; low ids are handed out first
};

struct PrefixEntry {
    std::vector<uint32_t> tokens;
    std::vector<uint32_t> pages;
    bool has_key = false;
    std::string key;
};

struct MfPrefixCache {
    MfPagePool *pool = nullptr;
    uint32_t page_size = 0;
    uint32_t max_entries = 0;
    std::deque<PrefixEntry> entries;
};

namespace {

void release_pages(MfPagePool *pool, const uint32_t *ids, uint32_t n)
{
    for (uint32_t i = 0; i < n; ++i) {
        const uint32_t id = ids[i];
        if (id < pool->refs.size() && pool->refs[id] > 0 && --pool->refs[id] == 0) pool->free_list.push_back(id);
    }
}

}  // namespace

extern "C" {

mf_status mf_page_pool_create(uint32_t n_pages, MfPagePool **out)
{
    if (!out) return MF_ERR_INPUT_NOT_FOUND;
    *out = nullptr;
    if (n_pages == 0) return MF_ERR_INVALID_OPERATION;
    MfPagePool *p = new (std::nothrow) MfPagePool();
    if (!p) return MF_ERR_OUT_OF_MEMORY;
    p->refs.assign(n_pages, 0);
    p->free_list.reserve(n_pages);
    for (uint32_t i = n_pages; i-- > 0;) p->free_list.push_back(i);
    *out = p;
    return MF_OK;
}

void mf_page_pool_destroy(MfPagePool *pool) { delete pool; }

mf_status mf_page_pool_alloc(MfPagePool *pool, uint32_t n, uint32_t *ids_out)
{
    if (!pool || (n && !ids_out)) return MF_ERR_INPUT_NOT_FOUND;
    if (n > pool->free_list.size()) return MF_ERR_OUT_OF_MEMORY;  // all or nothing
    for (uint32_t i = 0; i < n; ++i) {
        const uint32_t id = pool->free_list.back();
        pool->free_list.pop_back();
        pool->refs[id] = 1;
        ids_out[i] = id;
    }
    return MF_OK;
}

mf_status mf_page_pool_retain(MfPagePool *pool, const uint32_t *ids, uint32_t n)
{
    if (!pool || (n && !ids)) return MF_ERR_INPUT_NOT_FOUND;
    for (uint32_t i = 0; i < n; ++i)
        if (ids[i] >= pool->refs.size() || pool->refs[ids[i]] == 0) return MF_ERR_INVALID_OPERATION;  // not live
    for (uint32_t i = 0; i < n; ++i) ++pool->refs[ids[i]];
    return MF_OK;
}

mf_status mf_page_pool_release(MfPagePool *pool, const uint32_t *ids, uint32_t n)
{
    if (!pool || (n && !ids)) return MF_ERR_INPUT_NOT_FOUND;
    for (uint32_t i = 0; i < n; ++i)
        if (ids[i] >= pool->refs.size() || pool->refs[ids[i]] == 0) return MF_ERR_INVALID_OPERATION;
    release_pages(pool, ids, n);
    return MF_OK;
}

uint32_t mf_page_pool_free_count(const MfPagePool *pool) { return pool ? (uint32_t)pool->free_list.size() : 0; }

uint32_t mf_page_pool_refcount(const MfPagePool *pool, uint32_t id)
{
    return (pool && id < pool->refs.size()) ? pool->refs[id] : 0;
}

uint32_t mf_prefix_cache_default_entries(void) { return 8; }  // executor.rs:267

mf_status mf_prefix_cache_create(MfPagePool *pool, uint32_t page_size, uint32_t max_entries, MfPrefixCache **out)
{
    if (!out) return MF_ERR_INPUT_NOT_FOUND;
    *out = nullptr;
    if (!pool) return MF_ERR_INPUT_NOT_FOUND;
    if (page_size == 0) return MF_ERR_INVALID_OPERATION;
    MfPrefixCache *c = new (std::nothrow) MfPrefixCache();
    if (!c) return MF_ERR_OUT_OF_MEMORY;
    c->pool = pool;
    c->page_size = page_size;
    c->max_entries = max_entries < 1 ? 1 : (max_entries > 64 ? 64 : max_entries);  // clamp(1, 64), executor.rs:268-277
    *out = c;
    return MF_OK;
}

void mf_prefix_cache_destroy(MfPrefixCache *cache)
{
    if (!cache) return;
    for (auto &e : cache->entries) release_pages(cache->pool, e.pages.data(), (uint32_t)e.pages.size());
    delete cache;
}

uint32_t mf_prefix_cache_entries(const MfPrefixCache *cache) { return cache ? (uint32_t)cache->entries.size() : 0; }

mf_status mf_prefix_cache_store(MfPrefixCache *cache, const uint32_t *tokens, uint32_t n_tokens, const char *key,
                                const uint32_t *page_ids, uint32_t n_pages)
{
    if (!cache || !tokens || !page_ids) return MF_ERR_INPUT_NOT_FOUND;
    if (n_tokens == 0) return MF_OK;  // nothing to keep (executor.rs:1591)
    if (n_pages != (n_tokens + cache->page_size - 1) / cache->page_size) return MF_ERR_INVALID_SHAPE;
    mf_status st = mf_page_pool_retain(cache->pool, page_ids, n_pages);
    if (st != MF_OK) return st;
    PrefixEntry e;
    e.tokens.assign(tokens, tokens + n_tokens);
    e.pages.assign(page_ids, page_ids + n_pages);
    if (key) {
        e.has_key = true;
        e.key = key;
    }
    // replace the entry of the same key, or without key of the same tokens
    for (size_t i = 0; i < cache->entries.size(); ++i) {
        const PrefixEntry &o = cache->entries[i];
        const bool same = key ? (o.has_key && o.key == e.key) : (o.tokens == e.tokens);
        if (same) {
            release_pages(cache->pool, o.pages.data(), (uint32_t)o.pages.size());
            cache->entries.erase(cache->entries.begin() + (long)i);
            break;
        }
    }
    if (cache->entries.size() >= cache->max_entries) {
        const PrefixEntry &old = cache->entries.front();
        release_pages(cache->pool, old.pages.data(), (uint32_t)old.pages.size());
        cache->entries.pop_front();
    }
    cache->entries.push_back(std::move(e));
    return MF_OK;
}

mf_status mf_prefix_cache_lookup(MfPrefixCache *cache, const uint32_t *prompt, uint32_t n_prompt, const char *key,
                                 uint32_t *matched_out, uint32_t *page_ids_out, uint32_t page_ids_cap,
                                 uint32_t *n_pages_out)
{
    if (!cache || !matched_out || !n_pages_out) return MF_ERR_INPUT_NOT_FOUND;
    *matched_out = 0;
    *n_pages_out = 0;
    if (n_prompt == 0 || !prompt) return MF_OK;
    if (key && !*key) return MF_OK;  // an empty key never matches (executor.rs:1432)
    long best = -1;
    uint32_t best_len = 0;
    for (size_t i = 0; i < cache->entries.size(); ++i) {
        const PrefixEntry &e = cache->entries[i];
        const uint32_t len = (uint32_t)e.tokens.size();
        if (len == 0 || len > n_prompt) continue;
        if (key) {
            if (!e.has_key || e.key != key) continue;
            uint32_t m = 0;
            while (m < len && e.tokens[m] == prompt[m]) ++m;
            if (m == 0) continue;
            if (m >= best_len) {
                best = (long)i;
                best_len = m;
            }
        } else {
            if (std::memcmp(e.tokens.data(), prompt, (size_t)len * 4) == 0 && len >= best_len) {
                best = (long)i;
                best_len = len;
            }
        }
    }
    if (best < 0) return MF_OK;
    const uint32_t n_pages = (best_len + cache->page_size - 1) / cache->page_size;
    if (n_pages > page_ids_cap || !page_ids_out) return MF_ERR_OUT_OF_MEMORY;
    PrefixEntry e = std::move(cache->entries[(size_t)best]);
    cache->entries.erase(cache->entries.begin() + best);
    std::memcpy(page_ids_out, e.pages.data(), (size_t)n_pages * 4);
    // the caller's sequence now also refers to these pages
    mf_status st = mf_page_pool_retain(cache->pool, page_ids_out, n_pages);
    cache->entries.push_back(std::move(e));  // most recently used goes to the back
    if (st != MF_OK) return st;
    *matched_out = best_len;
    *n_pages_out = n_pages;
    return MF_OK;
}

}  // extern "C"
