// Native page allocator with prefix sharing: the C++ counterpart of the reference engine's
// BlockManager / Block / Sequence (infer/engine/block_mannager.py:26-133,
// infer/engine/sequence.py:15-84).  Same observable behaviour, page id for page id: pages
// leave the front of a FIFO free list, a full page is keyed by the XXH64 digest (seed 0) of
// the previous page's digest (8 bytes, little endian) followed by its token ids as int64, a
// request whose leading pages carry known digests and the same token ids re-uses those pages
// and bumps their reference counts, and a page returns to the back of the free list when its
// count reaches zero.  The free list supports O(1) removal of a revived page (the reference
// removes from a deque in O(n)).  Host-only: the attention kernels see the block tables.
#pragma once

#include <cstdint>
#include <cstring>
#include <list>
#include <stdexcept>
#include <unordered_map>
#include <vector>

namespace infer {

// XXH64 of a byte string, seed 0 (the published algorithm of the xxHash project).
inline uint64_t xxh64(const void* data, size_t len) {
    constexpr uint64_t P1 = 11400714785074694791ull, P2 = 14029467366897019727ull, P3 = 1609587929392839161ull,
                       P4 = 9650029242287828579ull, P5 = 2870177450012600261ull;
    auto rotl = [](uint64_t x, int r) { return (x << r) | (x >> (64 - r)); };
    auto rd64 = [](const uint8_t* p) { uint64_t v; std::memcpy(&v, p, 8); return v; };
    auto rd32 = [](const uint8_t* p) { uint32_t v; std::memcpy(&v, p, 4); return uint64_t(v); };
    auto round = [&](uint64_t acc, uint64_t in) { return rotl(acc + in * P2, 31) * P1; };
    const uint8_t* p = static_cast<const uint8_t*>(data);
    const uint8_t* end = p + len;
    uint64_t h;
    if (len >= 32) {
        uint64_t v1 = P1 + P2, v2 = P2, v3 = 0, v4 = 0 - P1;
        for (; p + 32 <= end; p += 32) {
            v1 = round(v1, rd64(p));
            v2 = round(v2, rd64(p + 8));
            v3 = round(v3, rd64(p + 16));
            v4 = round(v4, rd64(p + 24));
        }
        h = rotl(v1, 1) + rotl(v2, 7) + rotl(v3, 12) + rotl(v4, 18);
        for (uint64_t v : {v1, v2, v3, v4}) h = (h ^ round(0, v)) * P1 + P4;
    } else {
        h = P5;
    }
    h += uint64_t(len);
    for (; p + 8 <= end; p += 8) h = rotl(h ^ round(0, rd64(p)), 27) * P1 + P4;
    if (p + 4 <= end) {
        h = rotl(h ^ (rd32(p) * P1), 23) * P2 + P3;
        p += 4;
    }
    for (; p < end; ++p) h = rotl(h ^ (uint64_t(*p) * P5), 11) * P1;
    h ^= h >> 33;
    h *= P2;
    h ^= h >> 29;
    h *= P3;
    h ^= h >> 32;
    return h;
}

// A request as the allocator sees it: token ids and the logical -> physical page list.
struct PagedSequence {
    std::vector<int64_t> token_ids;
    std::vector<int32_t> block_table;
    size_t num_cached_tokens = 0;

    size_t size() const { return token_ids.size(); }
    size_t num_blocks(size_t block_size) const { return (token_ids.size() + block_size - 1) / block_size; }
    size_t last_block_num_tokens(size_t block_size) const {
        return token_ids.size() - (num_blocks(block_size) - 1) * block_size;
    }
    void append_token(int64_t t) { token_ids.push_back(t); }
};

class BlockManager {
public:
    struct Block {
        int32_t block_id = 0;
        int ref_count = 0;
        bool has_hash = false;
        uint64_t hash = 0;
        std::vector<int64_t> token_ids;
    };

    BlockManager(size_t num_blocks, size_t block_size) : block_size_(block_size), blocks_(num_blocks), where_(num_blocks) {
        if (num_blocks == 0) throw std::invalid_argument("BlockManager: num_blocks must be positive");
        for (size_t i = 0; i < num_blocks; ++i) {
            blocks_[i].block_id = static_cast<int32_t>(i);
            where_[i] = free_.insert(free_.end(), static_cast<int32_t>(i));
        }
    }

    // digest chain (infer/engine/block_mannager.py:54-60)
    static uint64_t compute_hash(const int64_t* tokens, size_t n, bool has_prefix, uint64_t prefix) {
        std::vector<uint8_t> buf((has_prefix ? 8 : 0) + n * 8);
        size_t at = 0;
        if (has_prefix) {
            std::memcpy(buf.data(), &prefix, 8);     // little-endian hosts only, like the kernels' target
            at = 8;
        }
        std::memcpy(buf.data() + at, tokens, n * 8);
        return xxh64(buf.data(), buf.size());
    }

    bool can_allocate(const PagedSequence& seq) const { return free_.size() >= seq.num_blocks(block_size_); }

    // whole-prompt allocation (infer/engine/block_mannager.py:76-103)
    void allocate(PagedSequence& seq) {
        if (!seq.block_table.empty()) throw std::runtime_error("BlockManager::allocate: sequence already has pages");
        bool have = false, missed = false;
        uint64_t digest = 0;
        const size_t nb = seq.num_blocks(block_size_);
        for (size_t i = 0; i < nb; ++i) {
            const size_t lo = i * block_size_, n = std::min(block_size_, seq.size() - lo);
            const int64_t* tok = seq.token_ids.data() + lo;
            const bool full = n == block_size_;
            if (full) {
                digest = compute_hash(tok, n, have, digest);
                have = true;
            } else {
                have = false;
            }
            int32_t hit = -1;
            if (have) {
                auto it = hash_to_block_.find(digest);
                if (it != hash_to_block_.end()) hit = it->second;
            }
            if (hit < 0 || !same_tokens(blocks_[hit], tok, n)) missed = true;   // once one page misses, all later ones are fresh
            Block* page;
            if (missed) {
                hit = free_.front();
                page = &take(hit);
            } else {
                seq.num_cached_tokens += block_size_;
                if (blocks_[hit].ref_count > 0) {
                    page = &blocks_[hit];
                    ++page->ref_count;
                } else {
                    page = &take(hit);               // the digest survived a free: revive the page
                }
            }
            if (have) {
                page->has_hash = true;
                page->hash = digest;
                page->token_ids.assign(tok, tok + n);
                hash_to_block_[digest] = hit;
            }
            seq.block_table.push_back(hit);
        }
    }

    void deallocate(PagedSequence& seq) {
        for (auto it = seq.block_table.rbegin(); it != seq.block_table.rend(); ++it) {
            Block& page = blocks_[*it];
            if (--page.ref_count == 0) where_[*it] = free_.insert(free_.end(), *it);
        }
        seq.num_cached_tokens = 0;
        seq.block_table.clear();
    }

    // one-token growth (infer/engine/block_mannager.py:114-133)
    bool can_append(const PagedSequence& seq) const { return free_.size() >= (seq.size() % block_size_ == 1 ? 1u : 0u); }

    void may_append(PagedSequence& seq) {
        Block& tail = blocks_[seq.block_table.back()];
        const size_t rem = seq.size() % block_size_;
        if (rem == 1) {                              // first token of a new page
            if (!tail.has_hash) throw std::runtime_error("BlockManager::may_append: previous page was never sealed");
            if (free_.empty()) throw std::runtime_error("BlockManager::may_append: out of pages");
            const int32_t fresh = free_.front();
            take(fresh);
            seq.block_table.push_back(fresh);
        } else if (rem == 0) {                       // page just filled: seal it with its digest
            if (tail.has_hash) throw std::runtime_error("BlockManager::may_append: page sealed twice");
            const size_t lo = (seq.num_blocks(block_size_) - 1) * block_size_;
            const bool has_prev = seq.block_table.size() > 1;
            const Block* prev = has_prev ? &blocks_[seq.block_table[seq.block_table.size() - 2]] : nullptr;
            const bool chain = prev && prev->has_hash;
            const uint64_t digest = compute_hash(seq.token_ids.data() + lo, block_size_, chain, chain ? prev->hash : 0);
            tail.has_hash = true;
            tail.hash = digest;
            tail.token_ids.assign(seq.token_ids.begin() + lo, seq.token_ids.begin() + lo + block_size_);
            hash_to_block_[digest] = tail.block_id;
        } else if (tail.has_hash) {
            throw std::runtime_error("BlockManager::may_append: open page carries a digest");
        }
    }

    // A page without token ids (no digest, never shared): for callers that track lengths only.
    int32_t take_anonymous() {
        if (free_.empty()) throw std::runtime_error("BlockManager: out of pages");
        const int32_t id = free_.front();
        take(id);
        return id;
    }
    // Drops one reference; the page returns to the back of the free list at zero.
    void release(int32_t block_id) {
        Block& page = blocks_.at(block_id);
        if (page.ref_count <= 0) throw std::runtime_error("BlockManager::release: page is not in use");
        if (--page.ref_count == 0) where_[block_id] = free_.insert(free_.end(), block_id);
    }

    // Replaces the order of the free list (every page must be free and appear once): lets a
    // workload generator scatter the pages of its sequences over the pool.
    void set_free_order(const int32_t* ids, size_t n) {
        if (n != blocks_.size() || free_.size() != blocks_.size())
            throw std::runtime_error("BlockManager::set_free_order: needs every page, all of them free");
        std::vector<char> seen(n, 0);
        for (size_t i = 0; i < n; ++i) {
            if (ids[i] < 0 || size_t(ids[i]) >= n || seen[ids[i]]) throw std::runtime_error("BlockManager::set_free_order: not a permutation");
            seen[ids[i]] = 1;
        }
        free_.clear();
        for (size_t i = 0; i < n; ++i) where_[ids[i]] = free_.insert(free_.end(), ids[i]);
    }

    size_t block_size() const { return block_size_; }
    size_t num_free() const { return free_.size(); }
    const std::list<int32_t>& free_block_ids() const { return free_; }
    int ref_count(int32_t block_id) const { return blocks_.at(block_id).ref_count; }
    size_t num_blocks() const { return blocks_.size(); }

private:
    static bool same_tokens(const Block& b, const int64_t* tok, size_t n) {
        return b.token_ids.size() == n && std::memcmp(b.token_ids.data(), tok, n * 8) == 0;
    }
    Block& take(int32_t id) {
        Block& page = blocks_[id];
        if (page.ref_count != 0) throw std::runtime_error("BlockManager: page is still referenced");
        page.ref_count = 1;
        page.has_hash = false;
        page.token_ids.clear();
        free_.erase(where_[id]);
        return page;
    }

    size_t block_size_;
    std::vector<Block> blocks_;
    std::unordered_map<uint64_t, int32_t> hash_to_block_;
    std::list<int32_t> free_;
    std::vector<std::list<int32_t>::iterator> where_;
};

}  // namespace infer
