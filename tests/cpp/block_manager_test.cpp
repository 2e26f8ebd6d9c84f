// Replays an allocator scenario through include/block_manager.hpp and prints one JSON line per
// snapshot; the Python test builds the scenario from the golden fixture that the reference's
// own BlockManager produced and compares page for page.
//   block_manager_test <scenario>      lines: "N blocks block_size" | "A n t0 t1 ..." | "T idx tok" | "D idx" | "S"
//   block_manager_test hash            reads "n t0 t1 ... [prefix]" lines from stdin, prints digests
#include <cstdio>
#include <fstream>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>

#include "block_manager.hpp"

int main(int argc, char** argv) {
    using namespace infer;
    if (argc < 2) return 64;
    if (std::string(argv[1]) == "hash") {
        std::string line;
        while (std::getline(std::cin, line)) {
            std::istringstream is(line);
            size_t n;
            is >> n;
            std::vector<int64_t> t(n);
            for (auto& x : t) is >> x;
            uint64_t prefix;
            const bool has = static_cast<bool>(is >> prefix);
            std::printf("%llu\n", static_cast<unsigned long long>(BlockManager::compute_hash(t.data(), n, has, has ? prefix : 0)));
        }
        return 0;
    }
    std::ifstream in(argv[1]);
    std::unique_ptr<BlockManager> mgr;
    std::vector<PagedSequence> seqs;
    std::string line;
    try {
        while (std::getline(in, line)) {
            std::istringstream is(line);
            char op;
            is >> op;
            if (op == 'N') {
                size_t nb, bs;
                is >> nb >> bs;
                mgr = std::make_unique<BlockManager>(nb, bs);
            } else if (op == 'A') {
                size_t n;
                is >> n;
                PagedSequence s;
                s.token_ids.resize(n);
                for (auto& x : s.token_ids) is >> x;
                if (!mgr->can_allocate(s)) throw std::runtime_error("cannot allocate");
                mgr->allocate(s);
                seqs.push_back(std::move(s));
            } else if (op == 'T') {
                size_t idx;
                int64_t tok;
                is >> idx >> tok;
                seqs[idx].append_token(tok);
                if (!mgr->can_append(seqs[idx])) throw std::runtime_error("cannot append");
                mgr->may_append(seqs[idx]);
            } else if (op == 'D') {
                size_t idx;
                is >> idx;
                mgr->deallocate(seqs[idx]);
            } else if (op == 'S') {
                std::ostringstream os;
                os << "{\"tables\": [";
                for (size_t i = 0; i < seqs.size(); ++i) {
                    os << (i ? ", [" : "[");
                    for (size_t j = 0; j < seqs[i].block_table.size(); ++j) os << (j ? ", " : "") << seqs[i].block_table[j];
                    os << "]";
                }
                os << "], \"cached\": [";
                for (size_t i = 0; i < seqs.size(); ++i) os << (i ? ", " : "") << seqs[i].num_cached_tokens;
                os << "], \"lens\": [";
                for (size_t i = 0; i < seqs.size(); ++i) os << (i ? ", " : "") << seqs[i].size();
                os << "], \"ref_counts\": [";
                for (size_t i = 0; i < mgr->num_blocks(); ++i) os << (i ? ", " : "") << mgr->ref_count(int32_t(i));
                os << "], \"free\": [";
                bool first = true;
                for (int32_t b : mgr->free_block_ids()) {
                    os << (first ? "" : ", ") << b;
                    first = false;
                }
                os << "]}";
                std::puts(os.str().c_str());
            }
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "exception: %s\n", e.what());
        return 2;
    }
    return 0;
}
