// Lays out what the kernels need to know about one step's batch as one int32 buffer (the caller
// copies it to the device in one transfer), with the reference's batch checks
// (crates/kernels/src/lib.rs:407-474: empty batch, empty sequence, length beyond the limit, too few
// pages, id outside the vocabulary, a request twice).  One call for the whole batch: the block
// tables and write slots come straight from the cache manager's leases.
#include <cstring>
#include <string>
#include <unordered_set>
#include <vector>

#include "cache_manager.h"

#define API extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string g_step_error;
inline int64_t align4(int64_t n) { return (n + 3) & ~int64_t(3); }
constexpr int kNeedMore = -7;
}  // namespace

API const char* mrs_step_last_error() { return g_step_error.c_str(); }

// Inputs: n_seq sequences (request id, first position, token count), their tokens and wanted places
// (flat, in sequence order).  pad_to > 0 (single tokens only): the batch is filled up to pad_to
// sequences with rows that write nothing, every row's logits are wanted, block tables are
// fixed_width wide.  pad_rows > 0 (with pad_to > 0; any batch): the step is filled up to pad_to
// sequences and pad_rows token rows; the added sequences have no rows, the added rows (token 0 at
// position 0 of the last sequence) write nothing and belong to no attention tile, and there are pad_to
// wanted rows: the real ones first (at most one a sequence), then row 0 again and again.  The shapes
// of such a step depend on pad_to, pad_rows and fixed_width alone.
// Output: buf (capacity cap ints) and layout:
//   [0] tokens T  [1] sequences B  [2] wanted rows R  [3] 1 when every sequence brings one token
//   [4..11] offsets of ids, pos, seq, q_start, ctx_len, state slot, want, tiles
//   [12 + 3g ..] per group: offset of the table, its width, offset of the write slots
//   [12 + 3G] longest context after the step   [13 + 3G] longest run of tokens of a sequence
// Returns the ints used, kNeedMore (-7) with the need in layout[0], or kInvalid (-6) with a message.
API int64_t mrs_step_build_padded(void* cache, int n_seq, const int64_t* requests, const int64_t* start_pos,
                                  const int32_t* counts, const int32_t* tokens, const int32_t* want_counts,
                                  const int32_t* want, int pad_to, int pad_rows, int fixed_width, int64_t max_seq_len,
                                  int64_t vocab, int32_t* buf, int64_t cap, int64_t* layout) {
    try {
        auto* m = static_cast<mrs::CacheManager*>(cache);
        const int G = m->num_groups();
        const int S = m->page_size();
        if (n_seq <= 0) {
            g_step_error = "empty batch or KV pool";
            return mrs::kInvalid;
        }
        std::unordered_set<int64_t> seen;
        std::vector<const mrs::Lease*> leases((size_t)n_seq);
        int64_t real_tokens = 0, wanted = 0, longest = 0, longest_run = 0;
        bool decode = true;
        std::vector<int64_t> widths((size_t)G, 1);
        for (int i = 0; i < n_seq; ++i) {
            const int64_t n = counts[i], start = start_pos[i];
            if (n <= 0 || start < 0 || start + n > max_seq_len) {
                g_step_error = "batch sequence length/page coverage mismatch";
                return mrs::kInvalid;
            }
            if (!seen.insert(requests[i]).second) {
                g_step_error = "aliased KV write slots in batch: a request appears twice";
                return mrs::kInvalid;
            }
            const mrs::Lease* lease = m->find(requests[i]);
            if (!lease) {
                g_step_error = "block table of request " + std::to_string(requests[i]) + ": unknown request";
                return mrs::kInvalid;
            }
            leases[(size_t)i] = lease;
            const int64_t need_pages = (start + n + S - 1) / S;
            for (int g = 0; g < G; ++g) {
                const auto& table = lease->tables[(size_t)g];
                if ((int64_t)table.size() < need_pages) {
                    g_step_error = "batch sequence length/page coverage mismatch";
                    return mrs::kInvalid;
                }
                for (int64_t p = start / S; p < need_pages; ++p)
                    if (table[(size_t)p] < 0) {
                        g_step_error = "a page to be written was given back already";
                        return mrs::kInvalid;
                    }
                if ((int64_t)table.size() > widths[(size_t)g]) widths[(size_t)g] = (int64_t)table.size();
            }
            for (int w = 0; w < want_counts[i]; ++w) {
                const int place = want[wanted + w];
                if (place < 0 || place >= n) {
                    g_step_error = "wanted place " + std::to_string(place) + " outside the " + std::to_string(n) + " tokens of the step";
                    return mrs::kInvalid;
                }
            }
            for (int64_t t = 0; t < n; ++t) {
                const int32_t id = tokens[real_tokens + t];
                if (id < 0 || id >= vocab) {
                    g_step_error = "token or page ID out of range";
                    return mrs::kInvalid;
                }
            }
            if (pad_rows > 0 && want_counts[i] > 1) {
                g_step_error = "a step padded to fixed shapes takes at most one wanted place a sequence";
                return mrs::kInvalid;
            }
            wanted += want_counts[i];
            real_tokens += n;
            if (n != 1) decode = false;
            if (start + n > longest) longest = start + n;
            if (n > longest_run) longest_run = n;
        }
        const bool fixed_rows = pad_rows > 0;
        if (fixed_rows) decode = false;            // a list of attention tiles is planned for such a step by its mixers
        const int64_t B = pad_to > 0 ? pad_to : n_seq;
        const int64_t pads = B - n_seq;
        if (pads < 0 || (pads > 0 && !decode && !fixed_rows)) {
            g_step_error = "only batches of single decoded tokens can be padded";
            return mrs::kInvalid;
        }
        if (fixed_rows && (pad_to <= 0 || pad_rows < real_tokens)) {
            g_step_error = "a step padded to fixed shapes needs pad_to sequences and at least its own rows";
            return mrs::kInvalid;
        }
        const int64_t T = fixed_rows ? pad_rows : real_tokens + pads;
        const int64_t R = pad_to > 0 ? B : wanted;
        if (fixed_width > 0)
            for (int g = 0; g < G; ++g) {
                if (widths[(size_t)g] > fixed_width) {
                    g_step_error = "batch sequence length/page coverage mismatch";
                    return mrs::kInvalid;
                }
                widths[(size_t)g] = fixed_width;
            }
        int64_t cursor = 0;
        auto take = [&](int64_t n) {
            const int64_t at = cursor;
            cursor += align4(n);
            return at;
        };
        const int64_t off_ids = take(T), off_pos = take(T), off_seq = take(T), off_q = take(B + 1), off_ctx = take(B),
                      off_slot = take(B), off_want = take(R), off_tiles = take(decode ? 4 * B : 0);
        std::vector<int64_t> off_table((size_t)G), off_slots((size_t)G);
        for (int g = 0; g < G; ++g) {
            off_table[(size_t)g] = take(B * widths[(size_t)g]);
            off_slots[(size_t)g] = take(T);
        }
        layout[0] = T, layout[1] = B, layout[2] = R, layout[3] = decode ? 1 : 0;
        layout[4] = off_ids, layout[5] = off_pos, layout[6] = off_seq, layout[7] = off_q, layout[8] = off_ctx;
        layout[9] = off_slot, layout[10] = off_want, layout[11] = off_tiles;
        for (int g = 0; g < G; ++g) {
            layout[12 + 3 * g] = off_table[(size_t)g];
            layout[13 + 3 * g] = widths[(size_t)g];
            layout[14 + 3 * g] = off_slots[(size_t)g];
        }
        layout[12 + 3 * G] = longest;
        layout[13 + 3 * G] = longest_run;
        if (cursor > cap) {
            layout[0] = cursor;
            return kNeedMore;
        }
        int32_t *ids = buf + off_ids, *pos = buf + off_pos, *seq = buf + off_seq, *q_start = buf + off_q,
                *ctx_len = buf + off_ctx, *slot = buf + off_slot, *want_rows = buf + off_want, *tiles = buf + off_tiles;
        std::memcpy(ids, tokens, (size_t)real_tokens * sizeof(int32_t));
        int64_t row = 0, w = 0;
        q_start[0] = 0;
        for (int i = 0; i < n_seq; ++i) {
            const int64_t n = counts[i], start = start_pos[i];
            for (int64_t t = 0; t < n; ++t) {
                pos[row + t] = (int32_t)(start + t);
                seq[row + t] = i;
            }
            if (pad_to <= 0 || fixed_rows)
                for (int k = 0; k < want_counts[i]; ++k) want_rows[w + k] = (int32_t)(row + want[w + k]);
            w += want_counts[i];
            ctx_len[i] = (int32_t)(start + n);
            slot[i] = leases[(size_t)i]->slot;
            row += n;
            q_start[i + 1] = (int32_t)row;
        }
        if (fixed_rows) {
            for (int64_t i = n_seq; i < B; ++i) {  // sequences without rows
                ctx_len[i] = 0, slot[i] = -1;
                q_start[i + 1] = (int32_t)row;
            }
            for (int64_t r = row; r < T; ++r) ids[r] = 0, pos[r] = 0, seq[r] = (int32_t)(B - 1);
            for (int64_t k = w; k < R; ++k) want_rows[k] = 0;
        } else {
            for (int64_t i = n_seq; i < B; ++i) {  // rows that write nothing: token 0 at position 0, state slot -1
                ids[row] = 0, pos[row] = 0, seq[row] = (int32_t)i;
                ctx_len[i] = 1, slot[i] = -1;
                ++row;
                q_start[i + 1] = (int32_t)row;
            }
            if (pad_to > 0)
                for (int64_t i = 0; i < B; ++i) want_rows[i] = (int32_t)i;
        }
        if (decode) {                              // one attention tile a sequence; none for a padding row
            std::memset(tiles, 0, (size_t)(4 * B) * sizeof(int32_t));
            for (int i = 0; i < n_seq; ++i) tiles[4 * i] = i, tiles[4 * i + 1] = i, tiles[4 * i + 2] = 1;
        }
        for (int g = 0; g < G; ++g) {
            int32_t* table = buf + off_table[(size_t)g];
            int32_t* slots = buf + off_slots[(size_t)g];
            const int64_t width = widths[(size_t)g];
            int64_t r = 0;
            for (int i = 0; i < n_seq; ++i) {
                const auto& t = leases[(size_t)i]->tables[(size_t)g];
                int32_t* dst = table + (int64_t)i * width;
                if (!t.empty()) std::memcpy(dst, t.data(), t.size() * sizeof(int32_t));
                for (int64_t c = (int64_t)t.size(); c < width; ++c) dst[c] = -1;
                for (int64_t k = 0; k < counts[i]; ++k) {
                    const int64_t p = start_pos[i] + k;
                    slots[r + k] = (int32_t)((int64_t)t[(size_t)(p / S)] * S + p % S);
                }
                r += counts[i];
            }
            for (int64_t i = n_seq; i < B; ++i) {  // a padding row reads page 0 and its result is dropped
                std::memset(table + i * width, 0, (size_t)width * sizeof(int32_t));
                if (!fixed_rows) slots[r++] = -1;
            }
            for (; fixed_rows && r < T; ++r) slots[r] = -1;
        }
        return cursor;
    } catch (const std::exception& e) {
        g_step_error = e.what();
        return -100;
    }
}

API int64_t mrs_step_build(void* cache, int n_seq, const int64_t* requests, const int64_t* start_pos, const int32_t* counts,
                           const int32_t* tokens, const int32_t* want_counts, const int32_t* want, int pad_to,
                           int fixed_width, int64_t max_seq_len, int64_t vocab, int32_t* buf, int64_t cap,
                           int64_t* layout) {
    return mrs_step_build_padded(cache, n_seq, requests, start_pos, counts, tokens, want_counts, want, pad_to, 0,
                                 fixed_width, max_seq_len, vocab, buf, cap, layout);
}
