// C ABI over the native page allocator (include/block_manager.hpp): what the Python host side
// binds in place of a Python allocator.  Host-only code; it lives in this library so that one
// shared object carries the whole path.  Sequences are kept inside the manager under the
// caller's 64-bit ids; no C++ exception crosses the boundary.
#include <memory>
#include <string>
#include <unordered_map>

#include "../../include/block_manager.hpp"
#include "../../include/infer_b200.h"

struct infer_block_manager {
    infer::BlockManager mgr;
    std::unordered_map<int64_t, infer::PagedSequence> seqs;
    std::string last_error;
    infer_block_manager(size_t n, size_t bs) : mgr(n, bs) {}
};

namespace {

template <typename F>
int guarded(infer_block_manager* m, F&& body) {
    try {
        return body();
    } catch (const std::exception& e) {
        m->last_error = e.what();
        return INFER_ERR_STATE;
    }
}

infer::PagedSequence* find(infer_block_manager* m, int64_t id) {
    auto it = m->seqs.find(id);
    if (it == m->seqs.end()) {
        m->last_error = "unknown sequence id";
        return nullptr;
    }
    return &it->second;
}

}  // namespace

extern "C" {

int infer_block_manager_create(infer_block_manager_t** out, int64_t num_blocks, int block_size) {
    if (!out) return INFER_ERR_NULL;
    *out = nullptr;
    if (num_blocks <= 0 || block_size <= 0 || num_blocks >= (int64_t(1) << 31)) return INFER_ERR_GEOMETRY;
    try {
        *out = new infer_block_manager(size_t(num_blocks), size_t(block_size));
    } catch (const std::exception&) {
        return INFER_ERR_STATE;
    }
    return INFER_OK;
}

int infer_block_manager_destroy(infer_block_manager_t* m) {
    delete m;
    return INFER_OK;
}

const char* infer_block_manager_last_error(const infer_block_manager_t* m) { return m ? m->last_error.c_str() : ""; }

int64_t infer_block_manager_num_free(const infer_block_manager_t* m) { return m ? int64_t(m->mgr.num_free()) : INFER_ERR_NULL; }

int64_t infer_block_manager_free_ids(const infer_block_manager_t* m, int32_t* out, int64_t cap) {
    if (!m || (!out && cap > 0)) return INFER_ERR_NULL;
    int64_t n = 0;
    for (int32_t id : m->mgr.free_block_ids()) {
        if (n < cap) out[n] = id;
        ++n;
    }
    return n;
}

int infer_block_manager_set_free_order(infer_block_manager_t* m, const int32_t* ids, int64_t n) {
    if (!m || !ids) return INFER_ERR_NULL;
    return guarded(m, [&] {
        m->mgr.set_free_order(ids, size_t(n));
        return INFER_OK;
    });
}

int64_t infer_block_manager_ref_counts(const infer_block_manager_t* m, int32_t* out, int64_t cap) {
    if (!m || (!out && cap > 0)) return INFER_ERR_NULL;
    const int64_t n = int64_t(m->mgr.num_blocks());
    for (int64_t i = 0; i < n && i < cap; ++i) out[i] = m->mgr.ref_count(int32_t(i));
    return n;
}

int infer_block_manager_can_allocate(const infer_block_manager_t* m, int64_t n_tokens) {
    if (!m) return INFER_ERR_NULL;
    if (n_tokens < 0) return INFER_ERR_GEOMETRY;
    const size_t bs = m->mgr.block_size();
    return m->mgr.num_free() >= (size_t(n_tokens) + bs - 1) / bs ? 1 : 0;
}

int64_t infer_block_manager_allocate(infer_block_manager_t* m, int64_t seq_id, const int64_t* token_ids, int64_t n_tokens) {
    if (!m || !token_ids) return INFER_ERR_NULL;
    if (n_tokens <= 0) return INFER_ERR_GEOMETRY;
    if (m->seqs.count(seq_id)) {
        m->last_error = "sequence already has pages";
        return INFER_ERR_STATE;
    }
    if (infer_block_manager_can_allocate(m, n_tokens) != 1) {
        m->last_error = "out of pages";
        return INFER_ERR_STATE;
    }
    int64_t cached = 0;
    const int rc = guarded(m, [&] {
        infer::PagedSequence seq;
        seq.token_ids.assign(token_ids, token_ids + n_tokens);
        m->mgr.allocate(seq);
        cached = int64_t(seq.num_cached_tokens);
        m->seqs.emplace(seq_id, std::move(seq));
        return INFER_OK;
    });
    return rc == INFER_OK ? cached : rc;
}

int infer_block_manager_can_append(const infer_block_manager_t* m, int64_t seq_id) {
    if (!m) return INFER_ERR_NULL;
    auto it = m->seqs.find(seq_id);
    if (it == m->seqs.end()) return INFER_ERR_STATE;
    return m->mgr.can_append(it->second) ? 1 : 0;
}

int infer_block_manager_append(infer_block_manager_t* m, int64_t seq_id, const int64_t* token_ids, int64_t n_new) {
    if (!m || (!token_ids && n_new > 0)) return INFER_ERR_NULL;
    if (n_new < 0) return INFER_ERR_GEOMETRY;
    infer::PagedSequence* seq = find(m, seq_id);
    if (!seq) return INFER_ERR_STATE;
    return guarded(m, [&] {
        if (n_new == 0) m->mgr.may_append(*seq);
        for (int64_t i = 0; i < n_new; ++i) {
            seq->append_token(token_ids[i]);
            m->mgr.may_append(*seq);
        }
        return INFER_OK;
    });
}

int64_t infer_block_manager_block_table(const infer_block_manager_t* m, int64_t seq_id, int32_t* out, int64_t cap) {
    if (!m || (!out && cap > 0)) return INFER_ERR_NULL;
    auto it = m->seqs.find(seq_id);
    if (it == m->seqs.end()) return INFER_ERR_STATE;
    const auto& table = it->second.block_table;
    for (size_t i = 0; i < table.size() && int64_t(i) < cap; ++i) out[i] = table[i];
    return int64_t(table.size());
}

int64_t infer_block_manager_num_tokens(const infer_block_manager_t* m, int64_t seq_id) {
    if (!m) return INFER_ERR_NULL;
    auto it = m->seqs.find(seq_id);
    return it == m->seqs.end() ? int64_t(INFER_ERR_STATE) : int64_t(it->second.size());
}

int infer_block_manager_deallocate(infer_block_manager_t* m, int64_t seq_id) {
    if (!m) return INFER_ERR_NULL;
    infer::PagedSequence* seq = find(m, seq_id);
    if (!seq) return INFER_ERR_STATE;
    return guarded(m, [&] {
        m->mgr.deallocate(*seq);
        m->seqs.erase(seq_id);
        return INFER_OK;
    });
}

}  // extern "C"
