// Exercises the C++ operator surface (include/*.hpp) without torch.
//   surface_test cpu                 host-only checks: registry, KVCachePool bookkeeping, error paths
//   surface_test gpu <in> <out>      append + paged decode + dense attention on the GPU through
//                                    UnifiedOp / KVCachePool; inputs and outputs are raw files
//                                    exchanged with the Python test, which checks them against
//                                    the CPU oracle.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <thread>

#include "unifiedOp.hpp"

using infer::bfloat16;
using infer::Tensor;

#define EXPECT(cond)                                                          \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                         \
        }                                                                     \
    } while (0)

template <typename F>
static bool throws(F f, const char* needle = nullptr) {
    try {
        f();
    } catch (const std::exception& e) {
        return !needle || std::strstr(e.what(), needle) != nullptr;
    }
    return false;
}

static int run_cpu() {
    using namespace infer;
    // ---- registry
    EXPECT(OperatorFactory::getFlashAttnOperator<bfloat16>() == nullptr);
    UnifiedOp<bfloat16> ops;
    auto fa = OperatorFactory::getFlashAttnOperator<bfloat16>();
    EXPECT(fa && fa->type() == OperatorType::FLASHATTENTION && fa->name() == "FLASHATTENTION");
    EXPECT(OperatorFactory::getKVAppendOperator<bfloat16>()->name() == "KV_APPEND");
    EXPECT(OperatorFactory::getPagedDecodeOperator<bfloat16>()->type() == OperatorType::PAGED_DECODE);
    EXPECT(OperatorFactory::getPagedPrefillOperator<bfloat16>()->type() == OperatorType::PAGED_PREFILL);
    EXPECT(OperatorFactory::getFlashAttnOperator<float>() == nullptr);          // keyed by element type
    EXPECT(OperatorRegistry::getInstance().size() == 4);
    UnifiedOp<bfloat16> again;                                                   // re-registration replaces, not duplicates
    EXPECT(OperatorRegistry::getInstance().size() == 4);
    std::ostringstream listing;
    OperatorRegistry::getInstance().listRegisteredOperators(listing);
    EXPECT(listing.str().find("PAGED_DECODE") != std::string::npos);
    EXPECT(static_cast<int>(OperatorType::FLASHATTENTION) == 4);                // reference ids unchanged

    // ---- operator argument checks (no GPU work is reached)
    Tensor<bfloat16> q(reinterpret_cast<bfloat16*>(0x1000), {1, 4, 64, 128}), bad(reinterpret_cast<bfloat16*>(0x1000), {1, 4, 64, 64});
    EXPECT(throws([&] { ops.attention(&q, &q, nullptr, &q); }, "null"));
    EXPECT(throws([&] { ops.attention(&bad, &bad, &bad, &bad); }, "expected"));
    UnifiedOp<float> fops;
    Tensor<float> fq(reinterpret_cast<float*>(0x1000), {1, 4, 64, 128});
    EXPECT(throws([&] { fops.attention(&fq, &fq, &fq, &fq); }, "bf16"));

    // ---- KVCachePool bookkeeping
    EXPECT(throws([] { KVCachePool<bfloat16> p(KVCachePoolConfig(100)); }, "multiple of 256"));
    EXPECT(throws([] { KVCachePool<bfloat16> p(KVCachePoolConfig(256, 64)); }, "head_size"));
    KVCachePool<bfloat16> pool(KVCachePoolConfig(256, 128, 8, 2, false, 10));
    EXPECT(pool.free_blocks() == 10);
    pool.prefetch_sequence(7, 600);                                              // 3 pages
    EXPECT((pool.block_table(7) == std::vector<int32_t>{0, 1, 2}));
    pool.extend_sequence(9, 256);                                                // creates the sequence: 1 page
    EXPECT((pool.block_table(9) == std::vector<int32_t>{3}));
    pool.extend_sequence(7, 768);                                                // still 3 pages
    EXPECT(pool.block_table(7).size() == 3 && pool.length(7) == 768);
    pool.extend_sequence(7, 769);                                                // crosses into a 4th page
    EXPECT((pool.block_table(7) == std::vector<int32_t>{0, 1, 2, 4}));
    pool.prefetch_sequence(7, 100);                                              // never shrinks
    EXPECT(pool.length(7) == 769);
    EXPECT(pool.slot_of(7, 0) == 0 && pool.slot_of(7, 300) == 256 + 44 && pool.slot_of(7, 768) == 4 * 256);
    EXPECT(throws([&] { pool.slot_of(7, 769); }));
    EXPECT(throws([&] { pool.block_table(1234); }, "Sequence ID not found"));
    EXPECT(throws([&] { pool.get_key_cache(7, 5); }, "Layer index"));
    EXPECT(throws([&] { pool.handle(0); }, "no pool memory"));
    EXPECT(pool.free_blocks() == 5 && pool.active_sequences() == 2);
    EXPECT(throws([&] { pool.extend_sequence(11, 256 * 6); }, "out of pages"));
    EXPECT(pool.active_sequences() == 2 && pool.free_blocks() == 5);             // a failed create leaves nothing behind
    pool.free_sequence(9);
    EXPECT(pool.free_blocks() == 6);
    pool.extend_sequence(12, 10);                                                // FIFO: oldest free page first
    EXPECT((pool.block_table(12) == std::vector<int32_t>{5}));
    pool.truncate(7, 300);
    pool.optimize_memory();
    EXPECT((pool.block_table(7) == std::vector<int32_t>{0, 1}) && pool.free_blocks() == 7);
    std::ostringstream stats;
    pool.print_memory_stats(stats);
    EXPECT(stats.str().find("Active Sequences: 2") != std::string::npos);
    // many threads growing and freeing their own sequences: the single mutex must hold up
    KVCachePool<bfloat16> big(KVCachePoolConfig(256, 128, 8, 1, false, 4096));
    std::vector<std::thread> ts;
    for (int t = 0; t < 8; ++t)
        ts.emplace_back([&big, t] {
            for (int i = 0; i < 200; ++i) {
                big.extend_sequence(t, 256 * (1 + i % 7) + 1);
                if (i % 5 == 4) big.free_sequence(t);
            }
            big.free_sequence(t);
        });
    for (auto& t : ts) t.join();
    EXPECT(big.free_blocks() == 4096 && big.active_sequences() == 0);
    // ---- pages by token ids: prefix sharing, sealing, preemption (the reference engine's allocator behaviour)
    {
        KVCachePool<bfloat16> shared(KVCachePoolConfig(256, 128, 8, 1, false, 8));
        std::vector<int64_t> prompt(600);
        for (size_t i = 0; i < prompt.size(); ++i) prompt[i] = int64_t(i * 7 + 3);
        EXPECT(shared.can_allocate(prompt));
        EXPECT(shared.allocate_prompt(1, prompt) == 0);
        EXPECT(shared.allocate_prompt(2, prompt) == 512);                            // two full pages found by digest
        EXPECT((shared.block_table(1) == std::vector<int32_t>{0, 1, 2}));
        EXPECT((shared.block_table(2) == std::vector<int32_t>{0, 1, 3}));            // the open tail page is never shared
        EXPECT(shared.page_ref_count(0) == 2 && shared.page_ref_count(1) == 2 && shared.page_ref_count(2) == 1);
        EXPECT(shared.free_blocks() == 4 && shared.length(2) == 600);
        EXPECT(throws([&] { shared.allocate_prompt(2, prompt); }, "exists"));
        EXPECT(throws([&] { shared.extend_sequence(1, 700); }, "token ids"));
        // decode: 168 tokens fill page 3 (sealed at 768), the 169th opens a new page
        for (int i = 0; i < 168; ++i) shared.append_token(2, 9000 + i);
        EXPECT(shared.length(2) == 768 && shared.block_table(2).size() == 3);
        EXPECT(shared.can_append(2));
        shared.append_token(2, 1);
        EXPECT(shared.block_table(2).size() == 4 && shared.block_table(2)[3] == 4 && shared.free_blocks() == 3);
        EXPECT(shared.slot_of(2, 768) == 4 * 256);
        // preemption gives the pages up; shared pages stay with sequence 1; resuming finds all three sealed pages again
        shared.preempt(2);
        EXPECT(shared.free_blocks() == 5 && shared.page_ref_count(0) == 1);
        EXPECT(throws([&] { shared.slot_of(2, 0); }, "beyond"));
        EXPECT(shared.resume(2) == 768);
        EXPECT((shared.block_table(2)[0] == 0) && (shared.block_table(2)[1] == 1) && (shared.block_table(2)[2] == 3));
        EXPECT(shared.page_ref_count(0) == 2 && shared.free_blocks() == 3);
        // a different prompt that fits nowhere
        std::vector<int64_t> big_prompt(256 * 4, 5);
        EXPECT(!shared.can_allocate(big_prompt));
        EXPECT(throws([&] { shared.allocate_prompt(3, big_prompt); }, "out of pages"));
        shared.free_sequence(1);
        shared.free_sequence(2);
        EXPECT(shared.free_blocks() == 8 && shared.active_sequences() == 0);
        // digests survive in the free list: the same prompt is served from cache again
        EXPECT(shared.allocate_prompt(4, prompt) == 512);
    }
    std::printf("surface cpu ok\n");
    return 0;
}

#define CUDA_OK(x)                                                                       \
    do {                                                                                 \
        cudaError_t e_ = (x);                                                            \
        if (e_ != cudaSuccess) {                                                         \
            std::fprintf(stderr, "CUDA %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            return 1;                                                                    \
        }                                                                                \
    } while (0)

// in : int32 header {B, Hq, Hkv, num_blocks, S_dense, lens[B]}, then bf16 q [B,Hq,128],
//      per sequence bf16 k then v [len, Hkv, 128], then dense Q,K,V [1,Hq|Hkv,S,128]
// out: int32 {W, block_tables[B*W]}, bf16 decode out [B,Hq,128], bf16 dense out [1,Hq,S,128]
static int run_gpu(const char* in_path, const char* out_path) {
    using namespace infer;
    std::ifstream in(in_path, std::ios::binary);
    std::vector<char> blob((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
    const int32_t* hdr = reinterpret_cast<const int32_t*>(blob.data());
    const int B = hdr[0], Hq = hdr[1], Hkv = hdr[2], nb = hdr[3], S = hdr[4];
    std::vector<int32_t> lens(hdr + 5, hdr + 5 + B);
    const char* cur = blob.data() + (5 + B) * 4;
    auto upload = [&](size_t bytes, void** dev) -> cudaError_t {
        cudaError_t e = cudaMalloc(dev, bytes);
        if (e != cudaSuccess) return e;
        e = cudaMemcpy(*dev, cur, bytes, cudaMemcpyHostToDevice);
        cur += bytes;
        return e;
    };
    const size_t row = size_t(Hkv) * 128 * 2;
    void *d_q, *d_kpool, *d_vpool, *d_out, *d_ws;
    CUDA_OK(upload(size_t(B) * Hq * 128 * 2, &d_q));
    CUDA_OK(cudaMalloc(&d_kpool, size_t(nb) * 256 * row));
    CUDA_OK(cudaMalloc(&d_vpool, size_t(nb) * 256 * row));
    CUDA_OK(cudaMemset(d_kpool, 0, size_t(nb) * 256 * row));
    CUDA_OK(cudaMemset(d_vpool, 0, size_t(nb) * 256 * row));
    CUDA_OK(cudaMalloc(&d_out, size_t(B) * Hq * 128 * 2));

    KVCachePool<bfloat16> cache(KVCachePoolConfig(256, 128, Hkv, 1, false, nb));
    cache.attach_layer(0, static_cast<bfloat16*>(d_kpool), static_cast<bfloat16*>(d_vpool));
    UnifiedOp<bfloat16> ops;

    // sequences arrive interleaved in two rounds so that their pages interleave too
    size_t W = 0;
    std::vector<std::pair<void*, void*>> kv(B);
    for (int b = 0; b < B; ++b) {
        CUDA_OK(upload(size_t(lens[b]) * row, &kv[b].first));
        CUDA_OK(upload(size_t(lens[b]) * row, &kv[b].second));
    }
    for (int round = 0; round < 2; ++round)
        for (int b = 0; b < B; ++b) {
            const size_t lo = round == 0 ? 0 : lens[b] / 2, hi = round == 0 ? lens[b] / 2 : lens[b];
            if (hi == lo) continue;
            cache.extend_sequence(b, hi);
            std::vector<int32_t> slots;
            for (size_t p = lo; p < hi; ++p) slots.push_back(cache.slot_of(b, p));
            int32_t* d_slots;
            CUDA_OK(cudaMalloc(&d_slots, slots.size() * 4));
            CUDA_OK(cudaMemcpy(d_slots, slots.data(), slots.size() * 4, cudaMemcpyHostToDevice));
            Tensor<bfloat16> k(reinterpret_cast<bfloat16*>(static_cast<char*>(kv[b].first) + lo * row), {hi - lo, size_t(Hkv), 128});
            Tensor<bfloat16> v(reinterpret_cast<bfloat16*>(static_cast<char*>(kv[b].second) + lo * row), {hi - lo, size_t(Hkv), 128});
            Tensor<int32_t> sm(d_slots, {hi - lo});
            ops.kv_append(cache, 0, &k, &v, &sm);
            CUDA_OK(cudaDeviceSynchronize());
            CUDA_OK(cudaFree(d_slots));
        }
    for (int b = 0; b < B; ++b) W = std::max(W, cache.block_table(b).size());
    std::vector<int32_t> bt(size_t(B) * W, -1);
    for (int b = 0; b < B; ++b) {
        auto t = cache.block_table(b);
        std::copy(t.begin(), t.end(), bt.begin() + b * W);
    }
    int32_t *d_bt, *d_cl;
    CUDA_OK(cudaMalloc(&d_bt, bt.size() * 4));
    CUDA_OK(cudaMemcpy(d_bt, bt.data(), bt.size() * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMalloc(&d_cl, B * 4));
    CUDA_OK(cudaMemcpy(d_cl, lens.data(), B * 4, cudaMemcpyHostToDevice));
    const size_t ws_bytes = PagedDecodeOperator<bfloat16>::workspace_bytes(cache.handle(0), B, Hq);
    CUDA_OK(cudaMalloc(&d_ws, ws_bytes));
    CUDA_OK(cudaMemset(d_ws, 0, ws_bytes));
    Tensor<bfloat16> q(static_cast<bfloat16*>(d_q), {size_t(B), size_t(Hq), 128}), out(static_cast<bfloat16*>(d_out), {size_t(B), size_t(Hq), 128});
    Tensor<int32_t> cl(d_cl, {size_t(B)}), btt(d_bt, {size_t(B), W});
    Tensor<uint8_t> ws(static_cast<uint8_t*>(d_ws), {ws_bytes});
    ops.paged_decode(cache, 0, &q, &cl, &btt, 1.0f / std::sqrt(128.0f), &ws, &out);
    CUDA_OK(cudaDeviceSynchronize());
    EXPECT(infer_paged_decode_status(d_ws, nullptr) == INFER_OK);

    // dense op through UnifiedOp::attention
    void *d_Q, *d_K, *d_V, *d_O;
    CUDA_OK(upload(size_t(Hq) * S * 128 * 2, &d_Q));
    CUDA_OK(upload(size_t(Hkv) * S * 128 * 2, &d_K));
    CUDA_OK(upload(size_t(Hkv) * S * 128 * 2, &d_V));
    CUDA_OK(cudaMalloc(&d_O, size_t(Hq) * S * 128 * 2));
    Tensor<bfloat16> Q(static_cast<bfloat16*>(d_Q), {1, size_t(Hq), size_t(S), 128}), K(static_cast<bfloat16*>(d_K), {1, size_t(Hkv), size_t(S), 128}),
        V(static_cast<bfloat16*>(d_V), {1, size_t(Hkv), size_t(S), 128}), O(static_cast<bfloat16*>(d_O), {1, size_t(Hq), size_t(S), 128});
    ops.attention(&Q, &K, &V, &O);
    CUDA_OK(cudaDeviceSynchronize());

    std::ofstream os(out_path, std::ios::binary);
    const int32_t w32 = static_cast<int32_t>(W);
    os.write(reinterpret_cast<const char*>(&w32), 4);
    os.write(reinterpret_cast<const char*>(bt.data()), bt.size() * 4);
    std::vector<char> host(std::max(size_t(B) * Hq * 128 * 2, size_t(Hq) * S * 128 * 2));
    CUDA_OK(cudaMemcpy(host.data(), d_out, size_t(B) * Hq * 128 * 2, cudaMemcpyDeviceToHost));
    os.write(host.data(), size_t(B) * Hq * 128 * 2);
    CUDA_OK(cudaMemcpy(host.data(), d_O, size_t(Hq) * S * 128 * 2, cudaMemcpyDeviceToHost));
    os.write(host.data(), size_t(Hq) * S * 128 * 2);
    std::printf("surface gpu ok\n");
    return 0;
}

int main(int argc, char** argv) {
    try {
        if (argc >= 2 && std::strcmp(argv[1], "cpu") == 0) return run_cpu();
        if (argc >= 4 && std::strcmp(argv[1], "gpu") == 0) return run_gpu(argv[2], argv[3]);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "exception: %s\n", e.what());
        return 2;
    }
    std::fprintf(stderr, "usage: surface_test cpu | gpu <in> <out>\n");
    return 64;
}
