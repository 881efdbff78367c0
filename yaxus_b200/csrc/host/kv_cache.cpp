// C entry points over yxh::KvCache for ctypes harnesses.  Errors (the reference's `Err`) come
// back as -1 with the message in yxh_last_error().
#include "kv_cache.hpp"

#include <string.h>

#include <string>

namespace {
thread_local std::string g_error;
struct Handle {
    yxh::KvCache cache;
    yxh::PassMeta meta;                 // of the last append
    std::vector<yxh::PageCopy> copies;  // pending, in order
    Handle(size_t pages, size_t max_pos) : cache(pages, max_pos) {}
};
template <typename F>
int64_t guarded(F f) {
    try {
        return f();
    } catch (const std::exception &e) {
        g_error = e.what();
        return -1;
    }
}
}  // namespace

extern "C" {

const char *yxh_last_error(void) { return g_error.c_str(); }

void *yxh_kvcache_new(uint64_t pages, uint64_t max_pos) { return new Handle(pages, max_pos); }
void yxh_kvcache_free(void *h) { delete (Handle *)h; }
void yxh_set_prefix_reuse(void *h, int on) { ((Handle *)h)->cache.set_prefix_reuse(on != 0); }
int64_t yxh_new_seq(void *h) { return (int64_t)((Handle *)h)->cache.new_seq(); }
void yxh_free_seq(void *h, uint64_t id) { ((Handle *)h)->cache.free_seq(id); }
void yxh_finish(void *h, uint64_t id) { ((Handle *)h)->cache.finish(id); }
int64_t yxh_seq_len(void *h, uint64_t id) { return (int64_t)((Handle *)h)->cache.seq_len(id); }
int64_t yxh_free_pages(void *h) { return (int64_t)((Handle *)h)->cache.free_pages(); }
int64_t yxh_total_pages(void *h) { return (int64_t)((Handle *)h)->cache.total_pages(); }
int64_t yxh_page_refs(void *h, uint32_t p) { return ((Handle *)h)->cache.page_refs(p); }

int64_t yxh_seq_pages(void *h, uint64_t id, uint32_t *out, uint64_t cap) {
    const auto &p = ((Handle *)h)->cache.seq_pages(id);
    for (size_t i = 0; i < p.size() && i < cap; i++) out[i] = p[i];
    return (int64_t)p.size();
}
int64_t yxh_seq_tokens(void *h, uint64_t id, uint32_t *out, uint64_t cap) {
    const auto &t = ((Handle *)h)->cache.seq_tokens(id);
    for (size_t i = 0; i < t.size() && i < cap; i++) out[i] = t[i];
    return (int64_t)t.size();
}

// Returns the sequence id; *reused gets the prompt tokens already in it.
int64_t yxh_begin(void *h, const uint32_t *prompt, uint64_t n, uint64_t *reused) {
    Handle *H = (Handle *)h;
    return guarded([&]() -> int64_t {
        auto r = H->cache.begin(std::vector<uint32_t>(prompt, prompt + n), H->copies);
        if (reused) *reused = r.second;
        return (int64_t)r.first;
    });
}
int64_t yxh_fork(void *h, uint64_t id, uint64_t len) {
    Handle *H = (Handle *)h;
    return guarded([&]() -> int64_t { return (int64_t)H->cache.fork(id, len, H->copies); });
}
int64_t yxh_truncate(void *h, uint64_t id, uint64_t len) {
    Handle *H = (Handle *)h;
    return guarded([&]() -> int64_t {
        H->cache.truncate(id, len);
        return 0;
    });
}

// items: seq_ids[n_items], counts[n_items], tokens concatenated.  Returns the rows of the pass.
int64_t yxh_append(void *h, uint64_t n_items, const uint64_t *seq_ids, const uint64_t *counts, const uint32_t *tokens) {
    Handle *H = (Handle *)h;
    return guarded([&]() -> int64_t {
        std::vector<std::pair<uint64_t, std::vector<uint32_t>>> items;
        size_t at = 0;
        for (uint64_t i = 0; i < n_items; i++) {
            items.push_back({seq_ids[i], std::vector<uint32_t>(tokens + at, tokens + at + counts[i])});
            at += counts[i];
        }
        H->meta = H->cache.append(items, H->copies);
        return (int64_t)H->meta.pos.size();
    });
}
int64_t yxh_meta_pages(void *h) { return (int64_t)((Handle *)h)->meta.pages.size(); }
// Copies the last pass's arrays out (each may be null).
void yxh_meta_get(void *h, uint32_t *ids, uint32_t *pos, uint32_t *kv_slot, uint32_t *pt_off, uint32_t *pages,
                  uint32_t *last) {
    const yxh::PassMeta &m = ((Handle *)h)->meta;
    auto put = [](uint32_t *dst, const std::vector<uint32_t> &v) {
        if (dst && !v.empty()) memcpy(dst, v.data(), v.size() * 4);
    };
    put(ids, m.ids);
    put(pos, m.pos);
    put(kv_slot, m.kv_slot);
    put(pt_off, m.pt_off);
    put(pages, m.pages);
    put(last, m.last);
}
int64_t yxh_meta_items(void *h) { return (int64_t)((Handle *)h)->meta.last.size(); }

// Pending page copies, in the order they must be made; taking them clears the list.
int64_t yxh_copies_pending(void *h) { return (int64_t)((Handle *)h)->copies.size(); }
int64_t yxh_copies_take(void *h, uint32_t *src, uint32_t *dst, uint64_t cap) {
    Handle *H = (Handle *)h;
    size_t n = std::min<size_t>(cap, H->copies.size());
    for (size_t i = 0; i < n; i++) {
        src[i] = H->copies[i].src;
        dst[i] = H->copies[i].dst;
    }
    H->copies.clear();
    return (int64_t)n;
}

}  // extern "C"
