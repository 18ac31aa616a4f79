// The step function's packing on the host: the index arrays that describe one step (a batch of requests, each with
// its next tokens) and the block tables of the requests' slots, laid out for ONE copy to the device.
// (The reference packs per call in compiled code too: crates/ai-engine-candle/src/paged/engine.rs:62-237.)
#pragma once
#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "runtime.hpp"

namespace aie {

// Segments lie back to back in one int32 buffer, each starting at a multiple of 4 ints (16 bytes).
inline int pad4(int n) { return (n + 3) / 4 * 4; }

struct StepShape {
    int T = 0, R = 0, N = 0;                // tokens, requests, wanted rows
    int max_q_len = 0, max_total_len = 0;   // most tokens an entry brings; most it holds after the step
    int width = 0;                          // block-table entries per request
    bool has_src = false;                   // some entry's token is still on the device
    std::vector<int> lengths;               // of the segments, in order
    int total = 0;                          // ints of the packed buffer
};

// Order of the segments: token_ids, positions, token_req [T]; q_start, q_len, ctx_len, slots, live [R];
// logit_rows [N]; token_src [T]; then one block table [R, width] per cache group.
enum { SEG_TOKEN_IDS, SEG_POSITIONS, SEG_TOKEN_REQ, SEG_Q_START, SEG_Q_LEN, SEG_CTX_LEN, SEG_SLOTS, SEG_LIVE,
       SEG_LOGIT_ROWS, SEG_TOKEN_SRC, SEG_TABLES };

// Checks the entries and works out the sizes.  `srcs[r] < 0`: the entry's tokens come from the host.
inline StepShape step_shape(const CacheManager& cache, const std::vector<int>& starts,
                            const std::vector<std::vector<long long>>& tokens,
                            const std::vector<std::vector<int>>& wants, const std::vector<int>& srcs,
                            int page_size, bool bucket_width) {
    StepShape s;
    s.R = (int)tokens.size();
    if (s.R == 0) throw std::invalid_argument("a step needs at least one entry and every entry at least one token");
    if ((int)starts.size() != s.R || (int)wants.size() != s.R || (int)srcs.size() != s.R)
        throw std::invalid_argument("pack_step: the entries' fields differ in number");
    for (int r = 0; r < s.R; ++r) {
        const int n = (int)tokens[r].size();
        if (n < 1) throw std::invalid_argument("a step needs at least one entry and every entry at least one token");
        if (srcs[r] >= 0) {
            if (n != 1) throw std::invalid_argument("only an entry of one token can take it from the device");
            s.has_src = true;
        }
        for (long long id : tokens[r])
            if (id < 0 || id > 2147483647LL) throw std::invalid_argument("token ids must be non-negative 32-bit integers");
        for (int w : wants[r])
            if (w < 0 || w >= n)
                throw std::invalid_argument("wanted place " + std::to_string(w) + " is outside the entry's " +
                                            std::to_string(n) + " tokens");
        s.T += n;
        s.N += (int)wants[r].size();
        s.max_q_len = std::max(s.max_q_len, n);
        s.max_total_len = std::max(s.max_total_len, starts[r] + n);
    }
    int width = std::max(1, (s.max_total_len + page_size - 1) / page_size);
    if (bucket_width) {         // few distinct widths, so layouts (and captured graphs) are reused
        int w = 64;
        while (w < width) w *= 2;
        width = w;
    }
    s.width = width;
    s.lengths = {s.T, s.T, s.T, s.R, s.R, s.R, s.R, s.R, s.N, s.T};
    for (int g = 0; g < cache.num_groups(); ++g) s.lengths.push_back(s.R * width);
    for (int n : s.lengths) s.total += pad4(n);
    s.total = std::max(s.total, 4);
    return s;
}

// Fills `out` (s.total ints).  Rows from `n_live` on only round the batch up (live = 0); n_live < 0: all are live.
inline void pack_step(const CacheManager& cache, const StepShape& s, const std::vector<int>& slots,
                      const std::vector<int>& starts, const std::vector<std::vector<long long>>& tokens,
                      const std::vector<std::vector<int>>& wants, const std::vector<int>& srcs, int n_live,
                      int32_t* out) {
    std::vector<int32_t*> seg(s.lengths.size());
    int o = 0;
    for (size_t i = 0; i < s.lengths.size(); ++i) {
        seg[i] = out + o;
        const int n = s.lengths[i], p = pad4(n);
        for (int k = n; k < p; ++k) out[o + k] = 0;      // the padding is copied too: keep it defined
        o += p;
    }
    int t = 0, row = 0;
    for (int r = 0; r < s.R; ++r) {
        const int n = (int)tokens[r].size();
        seg[SEG_Q_START][r] = t;
        seg[SEG_Q_LEN][r] = n;
        seg[SEG_CTX_LEN][r] = starts[r];
        seg[SEG_SLOTS][r] = slots[r];
        seg[SEG_LIVE][r] = (n_live < 0 || r < n_live) ? 1 : 0;
        for (int w : wants[r]) seg[SEG_LOGIT_ROWS][row++] = t + w;
        for (int i = 0; i < n; ++i) {
            seg[SEG_TOKEN_IDS][t + i] = (int32_t)tokens[r][i];
            seg[SEG_POSITIONS][t + i] = starts[r] + i;
            seg[SEG_TOKEN_REQ][t + i] = r;
            seg[SEG_TOKEN_SRC][t + i] = -1;
        }
        if (srcs[r] >= 0) seg[SEG_TOKEN_SRC][t] = srcs[r];
        t += n;
    }
    for (int g = 0; g < cache.num_groups(); ++g)
        cache.fill_block_table(g, slots.data(), s.R, s.width, seg[SEG_TABLES + g]);
}

// The work lists of the attention kernels, derived from a step's q_len / ctx_len / q_start (what
// parts/attention.py:AttentionWork hands to the kernels): rows of the lone tokens, longest context first; the
// other tokens; the tiles of `tile` tokens of the longer entries by the keys they read, fewest first; the same in
// units of two tiles.
struct AttentionLists {
    std::vector<int32_t> decode_tokens, other_tokens, tiles, pairs;      // tiles, pairs: (request row, offset) pairs
    int n_decode = 0, max_decode_len = 0;
};

inline AttentionLists attention_lists(const int32_t* q_start, const int32_t* q_len, const int32_t* ctx_len, int R,
                                      int tile) {
    AttentionLists a;
    std::vector<int> dec;
    for (int r = 0; r < R; ++r) {
        if (q_len[r] == 1) {
            dec.push_back(r);
            a.max_decode_len = std::max(a.max_decode_len, ctx_len[r] + 1);
        } else {
            for (int i = 0; i < q_len[r]; ++i) a.other_tokens.push_back(q_start[r] + i);
        }
    }
    std::stable_sort(dec.begin(), dec.end(), [&](int x, int y) { return ctx_len[x] > ctx_len[y]; });
    for (int r : dec) a.decode_tokens.push_back(q_start[r]);
    a.n_decode = (int)dec.size();
    struct Tile { int keys, r, o; };
    std::vector<Tile> ts;
    for (int r = 0; r < R; ++r)
        if (q_len[r] != 1)
            for (int o = 0; o < q_len[r]; o += tile) ts.push_back({ctx_len[r] + o, r, o});
    std::sort(ts.begin(), ts.end(), [](const Tile& x, const Tile& y) {
        return x.keys != y.keys ? x.keys < y.keys : (x.r != y.r ? x.r < y.r : x.o < y.o);
    });
    for (const Tile& t : ts) {
        a.tiles.push_back(t.r);
        a.tiles.push_back(t.o);
        if (t.o % (2 * tile) == 0) {
            a.pairs.push_back(t.r);
            a.pairs.push_back(t.o);
        }
    }
    return a;
}

}  // namespace aie
