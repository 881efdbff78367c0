// Host-side paged KV bookkeeping: a C++ restatement of yaxus-model's `KvCache`
// (crates/yaxus-model/src/kv.rs:49-353) for harnesses that have no Rust toolchain.  In a real
// integration yaxus-model's own KvCache is used unchanged and this file is not needed; it
// exists so that tests and benchmarks can drive the CUDA library with the page tables, forks
// and copy-on-write page copies the reference would produce.
//
// Behaviour kept from the reference: pages are handed out in ascending order first and then
// last-freed-first (kv.rs:55-71); whole pages of a common prefix are shared by reference
// count and a partly used last page is copied (fork, kv.rs:277-295); a shared page is copied
// right before the first write into it (reserve, kv.rs:299-326); finished sequences are kept
// for prefix reuse, at most 32, least recently used evicted first (kv.rs:27, 230-238); a
// prefix shorter than 16 tokens is not reused (kv.rs:25).
#pragma once

#include <stdint.h>

#include <algorithm>
#include <stdexcept>
#include <unordered_map>
#include <utility>
#include <vector>

namespace yxh {

constexpr size_t PAGE = 128;
constexpr size_t MIN_REUSE = 16;
constexpr size_t MAX_CACHED = 32;

inline size_t slot(const uint32_t *pages, size_t pos) { return (size_t)pages[pos / PAGE] * PAGE + pos % PAGE; }

struct PageCopy {
    uint32_t src, dst;
};

// PassMeta (crates/yaxus-model/src/lib.rs:63-75).
struct PassMeta {
    std::vector<uint32_t> ids, pos, kv_slot, pt_off, pages;
    std::vector<uint32_t> last;   // row of each item's last token (PassRows::last, kv.rs:124-127)
};

class KvCache {
  public:
    KvCache(size_t pages, size_t max_pos) : refs_(pages, 0), max_pos_(max_pos) {
        for (size_t p = pages; p-- > 0;) free_.push_back((uint32_t)p);
    }

    void set_prefix_reuse(bool on) {
        reuse_ = on;
        if (!on) clear_prefix_cache();
    }
    uint64_t new_seq() { return insert(Seq{}); }
    void free_seq(uint64_t id) {
        forget(id);
        auto it = seqs_.find(id);
        if (it == seqs_.end()) return;
        for (uint32_t p : it->second.pages) release(p);
        seqs_.erase(it);
    }
    void clear_prefix_cache() {
        while (evict_one()) {
        }
    }
    size_t seq_len(uint64_t id) const {
        auto it = seqs_.find(id);
        return it == seqs_.end() ? 0 : it->second.len;
    }
    const std::vector<uint32_t> &seq_tokens(uint64_t id) const {
        static const std::vector<uint32_t> none;
        auto it = seqs_.find(id);
        return it == seqs_.end() ? none : it->second.tokens;
    }
    const std::vector<uint32_t> &seq_pages(uint64_t id) const {
        static const std::vector<uint32_t> none;
        auto it = seqs_.find(id);
        return it == seqs_.end() ? none : it->second.pages;
    }
    size_t free_pages() const { return free_.size(); }
    size_t total_pages() const { return refs_.size(); }
    size_t max_pos() const { return max_pos_; }

    // kv.rs:189-212.  Returns (sequence, prompt tokens already in it).
    std::pair<uint64_t, size_t> begin(const std::vector<uint32_t> &prompt, std::vector<PageCopy> &copies) {
        if (prompt.empty()) throw std::runtime_error("empty prompt");
        uint64_t src;
        size_t keep;
        if (!best_prefix(prompt, src, keep)) return {new_seq(), 0};
        bool kept = forget(src);
        if (keep % PAGE != 0) {
            ensure_free(1);
            if (free_.empty()) keep = keep / PAGE * PAGE;
        }
        if (kept) touch(src);
        if (keep >= MIN_REUSE) {
            try {
                return {fork(src, keep, copies), keep};
            } catch (const std::runtime_error &) {
            }
        }
        return {new_seq(), 0};
    }

    // kv.rs:230-238.
    void finish(uint64_t id) {
        if (!reuse_ || seq_len(id) < MIN_REUSE) {
            free_seq(id);
            return;
        }
        touch(id);
        while (kept_.size() > MAX_CACHED && evict_one()) {
        }
    }

    // kv.rs:265-273.
    void truncate(uint64_t id, size_t len) {
        auto it = seqs_.find(id);
        if (it == seqs_.end()) return;
        Seq &s = it->second;
        if (len > s.len) throw std::runtime_error("truncate beyond the end");
        s.len = len;
        s.tokens.resize(len);
        size_t keep_pages = (len + PAGE - 1) / PAGE;
        for (size_t i = keep_pages; i < s.pages.size(); i++) release(s.pages[i]);
        s.pages.resize(std::min(keep_pages, s.pages.size()));
    }

    // kv.rs:277-295.
    uint64_t fork(uint64_t id, size_t len, std::vector<PageCopy> &copies) {
        auto it = seqs_.find(id);
        if (it == seqs_.end()) throw std::runtime_error("unknown sequence");
        const Seq &src = it->second;
        if (len > src.len) throw std::runtime_error("fork beyond the end");
        size_t full = len / PAGE;
        bool has_partial = len % PAGE != 0;
        uint32_t partial = 0;
        if (has_partial && !alloc(partial)) throw std::runtime_error("KV cache is full");
        Seq s;
        s.pages.assign(src.pages.begin(), src.pages.begin() + full);
        for (uint32_t p : s.pages) refs_[p]++;
        if (has_partial) {
            copies.push_back({src.pages[full], partial});
            s.pages.push_back(partial);
        }
        s.len = len;
        s.tokens.assign(src.tokens.begin(), src.tokens.begin() + len);
        return insert(std::move(s));
    }

    // kv.rs:330-352.  items[i] = (sequence, tokens).
    PassMeta append(const std::vector<std::pair<uint64_t, std::vector<uint32_t>>> &items, std::vector<PageCopy> &copies) {
        for (const auto &it : items) reserve(it.first, it.second.size(), copies);
        PassMeta meta;
        for (const auto &it : items) {
            Seq &s = seqs_.at(it.first);
            uint32_t off = (uint32_t)meta.pages.size();
            meta.pages.insert(meta.pages.end(), s.pages.begin(), s.pages.end());
            for (size_t j = 0; j < it.second.size(); j++) {
                size_t pos = s.len + j;
                meta.ids.push_back(it.second[j]);
                meta.pos.push_back((uint32_t)pos);
                meta.kv_slot.push_back((uint32_t)slot(s.pages.data(), pos));
                meta.pt_off.push_back(off);
            }
            s.len += it.second.size();
            s.tokens.insert(s.tokens.end(), it.second.begin(), it.second.end());
            meta.last.push_back((uint32_t)meta.ids.size() - 1);
        }
        return meta;
    }

    uint32_t page_refs(uint32_t p) const { return refs_[p]; }

  private:
    struct Seq {
        std::vector<uint32_t> pages;
        size_t len = 0;
        std::vector<uint32_t> tokens;
    };

    uint64_t insert(Seq s) {
        uint64_t id = next_id_++;
        seqs_.emplace(id, std::move(s));
        return id;
    }
    bool alloc(uint32_t &p) {
        if (free_.empty()) return false;
        p = free_.back();
        free_.pop_back();
        refs_[p] = 1;
        return true;
    }
    void release(uint32_t p) {
        if (--refs_[p] == 0) free_.push_back(p);
    }
    bool shared(uint32_t p) const { return refs_[p] > 1; }

    // The kept (finished) sequences, by last use.
    void touch(uint64_t id) {
        forget(id);
        kept_.push_back({id, ++clock_});
    }
    bool forget(uint64_t id) {
        size_t before = kept_.size();
        kept_.erase(std::remove_if(kept_.begin(), kept_.end(), [&](const auto &e) { return e.first == id; }), kept_.end());
        return kept_.size() != before;
    }
    bool evict_one() {
        if (kept_.empty()) return false;
        auto lru = std::min_element(kept_.begin(), kept_.end(), [](const auto &a, const auto &b) { return a.second < b.second; });
        free_seq(lru->first);
        return true;
    }
    void ensure_free(size_t n) {
        while (free_.size() < n && evict_one()) {
        }
    }

    // kv.rs:216-227: the kept sequence with the longest common prefix (first of equals).
    bool best_prefix(const std::vector<uint32_t> &prompt, uint64_t &src, size_t &keep) const {
        if (!reuse_) return false;
        bool have = false;
        size_t best = 0;
        for (const auto &e : kept_) {
            const std::vector<uint32_t> &t = seqs_.at(e.first).tokens;
            size_t lcp = 0;
            while (lcp < t.size() && lcp < prompt.size() && t[lcp] == prompt[lcp]) lcp++;
            if (!have || lcp > best) {
                have = true;
                best = lcp;
                src = e.first;
            }
        }
        if (!have) return false;
        keep = std::min(best, prompt.size() - 1);
        return keep >= MIN_REUSE;
    }

    // kv.rs:299-326.
    void reserve(uint64_t id, size_t n, std::vector<PageCopy> &copies) {
        size_t need = 0;
        {
            auto it = seqs_.find(id);
            if (it == seqs_.end()) throw std::runtime_error("unknown sequence");
            const Seq &s = it->second;
            size_t end = s.len + n;
            // Checked before anything is evicted: a pass that cannot run must not flush the cache.
            if (end > max_pos_) throw std::runtime_error("context length exceeds the limit");
            for (size_t pi = s.len / PAGE; pi < (end + PAGE - 1) / PAGE; pi++)
                if (pi >= s.pages.size() || shared(s.pages[pi])) need++;
        }
        ensure_free(need);
        Seq &s = seqs_.at(id);
        for (size_t pi = s.len / PAGE; pi < (s.len + n + PAGE - 1) / PAGE; pi++) {
            if (pi < s.pages.size()) {
                uint32_t p = s.pages[pi];
                if (shared(p)) {
                    uint32_t q;
                    if (!alloc(q)) throw std::runtime_error("KV cache is full");
                    copies.push_back({p, q});
                    release(p);
                    s.pages[pi] = q;
                }
            } else {
                uint32_t q;
                if (!alloc(q)) throw std::runtime_error("KV cache is full");
                s.pages.push_back(q);
            }
        }
    }

    std::vector<uint32_t> refs_;
    std::vector<uint32_t> free_;
    std::unordered_map<uint64_t, Seq> seqs_;
    uint64_t next_id_ = 0;
    size_t max_pos_;
    std::vector<std::pair<uint64_t, uint64_t>> kept_;   // (sequence, last use)
    uint64_t clock_ = 0;
    bool reuse_ = true;
};

}  // namespace yxh
