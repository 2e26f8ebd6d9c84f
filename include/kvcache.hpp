// KVCachePool<T>: the reference's KV-cache class (include/kvcache.hpp:12-97,
// src/kvcache.cc:7-305), re-backed by pages.
//
// The reference keeps one contiguous [len, heads, head_size] tensor per sequence and layer
// and grows it by reallocate-and-copy.  Here a sequence owns a list of fixed-size pages of
// the per-layer pools [num_blocks, block_size, heads, head_size] that the attention kernels
// read through block tables; growing a sequence appends page ids, nothing is copied.  The
// class does host bookkeeping only: it never allocates device memory - the caller attaches
// the pool memory of every layer (attach_layer) - and keeps one library handle per layer.
// Method names and the config struct follow the reference; every public method takes the
// pool mutex once (the reference's extend_sequence/prefetch_sequence lock it recursively and
// deadlock, src/kvcache.cc:73-80,143-149).
//
// Pages come from the native BlockManager (block_manager.hpp), so the pool also offers what the
// reference's Python engine does with its allocator (infer/engine/block_mannager.py:76-133,
// infer/engine/scheduler.py:24-61): a prompt given by its token ids shares the pages of a known
// prefix (allocate_prompt), a decoded token seals or opens pages (append_token), and a
// sequence can give its pages up and take them back later (preempt / resume).
#pragma once

#include <algorithm>
#include <iostream>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "block_manager.hpp"
#include "infer_b200.h"
#include "tensor.hpp"

namespace infer {

struct KVCachePoolConfig {
    size_t block_size;   // tokens per page (a multiple of 256)
    size_t head_size;    // 128
    size_t num_heads;    // KV heads held by this pool (this GPU's shard)
    size_t num_layers;
    bool use_mla;        // value cache aliases the key cache (kept from the reference)
    size_t num_blocks;   // pages per layer pool

    KVCachePoolConfig(size_t blk_size = 256, size_t h_size = 128, size_t n_heads = 8, size_t n_layers = 1,
                      bool mla = false, size_t n_blocks = 0)
        : block_size(blk_size), head_size(h_size), num_heads(n_heads), num_layers(n_layers), use_mla(mla),
          num_blocks(n_blocks) {}
};

template <typename T>
class KVCachePool {
public:
    explicit KVCachePool(const KVCachePoolConfig& config, void* stream = nullptr)
        : config_(config), stream_(stream), layers_(config.num_layers) {
        static_assert(sizeof(T) == 1 || sizeof(T) == 2, "KVCachePool holds bf16 (2-byte) or e4m3 (1-byte) elements");
        if (config.block_size == 0 || config.block_size % 256 != 0)
            throw std::invalid_argument("KVCachePool: block_size must be a multiple of 256");
        if (config.head_size != 128) throw std::invalid_argument("KVCachePool: head_size must be 128");
        if (config.num_blocks > 0) pages_.reset(new BlockManager(config.num_blocks, config.block_size));
    }
    ~KVCachePool() {
        for (auto& l : layers_)
            if (l.handle) infer_kv_pool_destroy(l.handle);
    }
    KVCachePool(const KVCachePool&) = delete;
    KVCachePool& operator=(const KVCachePool&) = delete;

    // Hands the pool the device memory of one layer: k and v pools
    // [num_blocks, block_size, num_heads, head_size] (and, for 1-byte T, the fp32 scales
    // [num_blocks, num_heads]).  Builds the library handle (TMA descriptors) for the layer.
    void attach_layer(size_t layer_idx, T* k_pool, T* v_pool, float* k_scale = nullptr, float* v_scale = nullptr) {
        std::lock_guard<std::mutex> lock(mutex_);
        check_layer(layer_idx);
        Layer& l = layers_[layer_idx];
        if (l.handle) {
            infer_kv_pool_destroy(l.handle);
            l.handle = nullptr;
        }
        const int rc = infer_kv_pool_create(&l.handle, k_pool, config_.use_mla ? k_pool : v_pool, k_scale, v_scale,
                                            static_cast<int64_t>(config_.num_blocks), static_cast<int>(config_.block_size),
                                            static_cast<int>(config_.num_heads), static_cast<int>(config_.head_size),
                                            sizeof(T) == 2 ? INFER_KV_BF16 : INFER_KV_E4M3);
        if (rc != INFER_OK) throw std::runtime_error(std::string("KVCachePool::attach_layer: ") + infer_strerror(rc));
        l.k = k_pool;
        l.v = config_.use_mla ? k_pool : v_pool;
    }

    // The layer's whole key (value) pool; the pages of `sequence_id` inside it are block_table().
    Tensor<T> get_key_cache(size_t sequence_id, size_t layer_idx) {
        std::lock_guard<std::mutex> lock(mutex_);
        find(sequence_id);
        check_layer(layer_idx);
        return Tensor<T>(layers_[layer_idx].k, pool_shape());
    }
    Tensor<T> get_value_cache(size_t sequence_id, size_t layer_idx) {
        std::lock_guard<std::mutex> lock(mutex_);
        find(sequence_id);
        check_layer(layer_idx);
        return Tensor<T>(layers_[layer_idx].v, pool_shape());
    }

    // Grows (never shrinks) a sequence to new_length tokens, taking pages from the free list;
    // creates the sequence if it does not exist (as the reference does).
    void extend_sequence(size_t sequence_id, size_t new_length) {
        std::lock_guard<std::mutex> lock(mutex_);
        grow(sequence_id, new_length);
    }
    void prefetch_sequence(size_t sequence_id, size_t initial_length) {
        std::lock_guard<std::mutex> lock(mutex_);
        grow(sequence_id, initial_length);
    }
    void free_sequence(size_t sequence_id) {
        std::lock_guard<std::mutex> lock(mutex_);
        auto it = sequences_.find(sequence_id);
        if (it == sequences_.end()) return;
        give_back(it->second);
        sequences_.erase(it);
    }

    // ---- sequences known by their token ids: prefix sharing, sealing, preemption
    // True when a prompt of these tokens fits (counted without sharing, as the reference's
    // scheduler does before it admits a request, infer/engine/scheduler.py:31).
    bool can_allocate(const std::vector<int64_t>& token_ids) const {
        std::lock_guard<std::mutex> lock(mutex_);
        return pages_ && pages_->num_free() >= (token_ids.size() + config_.block_size - 1) / config_.block_size;
    }
    // Creates a sequence from its prompt.  Leading full pages whose content is already cached
    // are shared; returns the number of tokens whose KV is therefore already in the pool (the
    // reference's num_cached_tokens: those rows need no append and no prefill compute).
    size_t allocate_prompt(size_t sequence_id, const std::vector<int64_t>& token_ids) {
        std::lock_guard<std::mutex> lock(mutex_);
        if (sequences_.count(sequence_id)) throw std::runtime_error("KVCachePool: sequence exists: " + std::to_string(sequence_id));
        if (token_ids.empty()) throw std::invalid_argument("KVCachePool::allocate_prompt: empty prompt");
        Sequence s;
        s.tokens.token_ids = token_ids;
        if (!pages_ || !pages_->can_allocate(s.tokens)) throw std::runtime_error("KVCachePool: out of pages");
        pages_->allocate(s.tokens);
        s.by_tokens = true;
        s.length = token_ids.size();
        const size_t cached = s.tokens.num_cached_tokens;
        sequences_.emplace(sequence_id, std::move(s));
        return cached;
    }
    bool can_append(size_t sequence_id) const {
        std::lock_guard<std::mutex> lock(mutex_);
        const Sequence& s = find(sequence_id);
        // the next token opens a new page exactly when the current length fills its pages
        return !(s.length % config_.block_size == 0) || pages_->num_free() >= 1;
    }
    // One decoded token: opens a page when the token is the first of one, seals the page with
    // its digest when the token fills it.
    void append_token(size_t sequence_id, int64_t token_id) {
        std::lock_guard<std::mutex> lock(mutex_);
        Sequence& s = find(sequence_id);
        if (!s.by_tokens || s.preempted) throw std::runtime_error("KVCachePool::append_token: sequence holds no token pages");
        if (s.length % config_.block_size == 0 && pages_->num_free() == 0) throw std::runtime_error("KVCachePool: out of pages");
        s.tokens.append_token(token_id);
        pages_->may_append(s.tokens);
        s.length = s.tokens.size();
    }
    // Gives up the pages but keeps the tokens (the scheduler's preemption,
    // infer/engine/scheduler.py:57-61); sealed pages keep their digests while they sit in
    // the free list, so resume() finds them again unless they were handed out meanwhile.
    void preempt(size_t sequence_id) {
        std::lock_guard<std::mutex> lock(mutex_);
        Sequence& s = find(sequence_id);
        if (!s.by_tokens) throw std::runtime_error("KVCachePool::preempt: sequence was not created from token ids");
        if (s.preempted) return;
        pages_->deallocate(s.tokens);
        s.preempted = true;
    }
    // Takes pages again for a preempted sequence; returns the tokens found cached.
    size_t resume(size_t sequence_id) {
        std::lock_guard<std::mutex> lock(mutex_);
        Sequence& s = find(sequence_id);
        if (!s.preempted) throw std::runtime_error("KVCachePool::resume: sequence is not preempted");
        if (!pages_->can_allocate(s.tokens)) throw std::runtime_error("KVCachePool: out of pages");
        pages_->allocate(s.tokens);
        s.preempted = false;
        return s.tokens.num_cached_tokens;
    }
    int page_ref_count(int32_t page) const {
        std::lock_guard<std::mutex> lock(mutex_);
        if (!pages_) throw std::runtime_error("KVCachePool: no pages");
        return pages_->ref_count(page);
    }
    // Returns pages a sequence holds beyond ceil(length / block_size) (none are ever taken in
    // advance here, so this only matters after truncate()).
    void optimize_memory() {
        std::lock_guard<std::mutex> lock(mutex_);
        for (auto& kv : sequences_) trim(kv.second);
    }
    void truncate(size_t sequence_id, size_t new_length) {
        std::lock_guard<std::mutex> lock(mutex_);
        Sequence& s = find(sequence_id);
        if (s.by_tokens) throw std::runtime_error("KVCachePool::truncate: sequence was created from token ids");
        if (new_length < s.length) s.length = new_length;
    }

    // ---- paged accessors used to build the step metadata
    std::vector<int32_t> block_table(size_t sequence_id) const {
        std::lock_guard<std::mutex> lock(mutex_);
        return find(sequence_id).tokens.block_table;
    }
    size_t length(size_t sequence_id) const {
        std::lock_guard<std::mutex> lock(mutex_);
        return find(sequence_id).length;
    }
    // flat slot of token `pos`: block_table[pos / block_size] * block_size + pos % block_size
    int32_t slot_of(size_t sequence_id, size_t pos) const {
        std::lock_guard<std::mutex> lock(mutex_);
        const Sequence& s = find(sequence_id);
        if (pos >= s.length || s.preempted) throw std::out_of_range("KVCachePool::slot_of: position beyond the sequence");
        return static_cast<int32_t>(s.tokens.block_table[pos / config_.block_size] * config_.block_size + pos % config_.block_size);
    }
    infer_kv_pool_t* handle(size_t layer_idx) const {
        std::lock_guard<std::mutex> lock(mutex_);
        check_layer(layer_idx);
        if (!layers_[layer_idx].handle) throw std::runtime_error("KVCachePool: layer has no pool memory attached");
        return layers_[layer_idx].handle;
    }
    size_t free_blocks() const {
        std::lock_guard<std::mutex> lock(mutex_);
        return free_count();
    }
    size_t active_sequences() const {
        std::lock_guard<std::mutex> lock(mutex_);
        return sequences_.size();
    }
    const KVCachePoolConfig& config() const { return config_; }
    void* stream() const { return stream_; }

    void print_memory_stats(std::ostream& os = std::cout) const {
        std::lock_guard<std::mutex> lock(mutex_);
        const size_t used = config_.num_blocks - free_count();
        const size_t page_bytes = config_.block_size * config_.num_heads * config_.head_size * sizeof(T) *
                                  (config_.use_mla ? 1 : 2) * config_.num_layers;
        size_t total_len = 0, max_len = 0;
        for (const auto& kv : sequences_) {
            total_len += kv.second.length;
            max_len = std::max(max_len, kv.second.length);
        }
        os << "KV Cache Pool Memory Stats:" << std::endl;
        os << "  Pages used / total: " << used << " / " << config_.num_blocks << std::endl;
        os << "  Total Allocated Memory: " << (used * page_bytes) / (1024 * 1024) << " MB" << std::endl;
        os << "  Active Sequences: " << sequences_.size() << std::endl;
        os << "  Max Sequence Length: " << max_len << std::endl;
        if (!sequences_.empty())
            os << "  Average Sequence Length: " << static_cast<double>(total_len) / sequences_.size() << " tokens" << std::endl;
    }

private:
    struct Sequence {
        PagedSequence tokens;        // block_table always; token_ids only for sequences created from a prompt
        size_t length = 0;
        bool by_tokens = false;
        bool preempted = false;
    };
    struct Layer {
        T* k = nullptr;
        T* v = nullptr;
        infer_kv_pool_t* handle = nullptr;
    };

    std::vector<size_t> pool_shape() const {
        return {config_.num_blocks, config_.block_size, config_.num_heads, config_.head_size};
    }
    void check_layer(size_t layer_idx) const {
        if (layer_idx >= layers_.size())
            throw std::runtime_error("Layer index out of bounds: " + std::to_string(layer_idx));
    }
    Sequence& find(size_t id) {
        auto it = sequences_.find(id);
        if (it == sequences_.end()) throw std::runtime_error("Sequence ID not found: " + std::to_string(id));
        return it->second;
    }
    const Sequence& find(size_t id) const {
        auto it = sequences_.find(id);
        if (it == sequences_.end()) throw std::runtime_error("Sequence ID not found: " + std::to_string(id));
        return it->second;
    }
    size_t free_count() const { return pages_ ? pages_->num_free() : 0; }
    void give_back(Sequence& s) {
        if (s.by_tokens) {
            if (!s.preempted) pages_->deallocate(s.tokens);
            return;
        }
        std::vector<int32_t>& pages = s.tokens.block_table;
        for (auto p = pages.rbegin(); p != pages.rend(); ++p) pages_->release(*p);
        pages.clear();
    }
    void grow(size_t id, size_t new_length) {
        Sequence& s = sequences_[id];
        if (s.by_tokens) throw std::runtime_error("KVCachePool: sequence was created from token ids; use append_token");
        if (new_length <= s.length) return;
        std::vector<int32_t>& pages = s.tokens.block_table;
        const size_t need = (new_length + config_.block_size - 1) / config_.block_size;
        if (need > pages.size() && need - pages.size() > free_count()) {
            if (pages.empty() && s.length == 0) sequences_.erase(id);
            throw std::runtime_error("KVCachePool: out of pages");
        }
        while (pages.size() < need) pages.push_back(pages_->take_anonymous());
        s.length = new_length;
    }
    void trim(Sequence& s) {
        if (s.by_tokens) return;
        std::vector<int32_t>& pages = s.tokens.block_table;
        const size_t need = (s.length + config_.block_size - 1) / config_.block_size;
        while (pages.size() > need) {
            pages_->release(pages.back());
            pages.pop_back();
        }
    }

    KVCachePoolConfig config_;
    void* stream_;
    std::vector<Layer> layers_;
    std::unordered_map<size_t, Sequence> sequences_;
    std::unique_ptr<BlockManager> pages_;
    mutable std::mutex mutex_;
};

}  // namespace infer
