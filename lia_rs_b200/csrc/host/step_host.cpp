// The step function's host side, native: the checks on a batch of (request slot, its next tokens, wanted places) and
// the layout of the step's metadata, written straight into the pinned buffer that one copy takes to the device.
// No CUDA in this file.  The Python class `engine.StepRuntime` is its face: it flattens the entries, calls
// `lia_step_stage`, issues the copy and builds the step's context from the counts that come back.
//
// The checks are the reference's before a paged forward (src/inference/paging.rs:120-172): no request twice in a
// step, every position covered by reserved pages, every token id inside the vocabulary, every wanted place among the
// entry's tokens, the step within its buffers.
//
// Layout of the metadata, 32-bit words, n rows of the batch (padding rows included), n_out wanted rows:
//   [tokens n][positions n][slots n][wanted rows n_out][rows of single tokens][rows of portions][portions: row, start, count]
// A step of more than `pad_above` entries that are all single tokens gets rows of nobody at its end, up to a multiple
// of `pad_to` rows while `max_batch_tokens` has room: token 0, position 0, slot -1, listed among the wanted rows and
// the rows of single tokens (the kernels skip a negative slot wherever a cache is touched).
#include "cache_host.h"

#define LIA_HOST_EXPORT extern "C" __attribute__((visibility("default")))

using namespace lia_host;

// Rows of nobody that a step of `n_tokens` tokens in `n_entries` entries gets.
LIA_HOST_EXPORT int lia_step_padding(int n_tokens, int n_entries, int pad_above, int pad_to, int max_batch_tokens) {
    if (n_entries != n_tokens || n_tokens <= pad_above || pad_to <= 0) return 0;
    const int padded = (n_tokens + pad_to - 1) / pad_to * pad_to;
    return padded <= max_batch_tokens ? padded - n_tokens : 0;
}

// `slots`, `starts`, `counts`, `want_counts`: one per entry; `tokens`: the entries' tokens one after the other;
// `wants`: their wanted places (indices among the entry's own tokens) one after the other.  `cache`: the native cache
// (lia_cache_create), asked up to where each slot has pages.  `meta`: room for `capacity` words.
// `summary` (6 words): rows of the batch, wanted rows, rows of nobody among both, rows of single tokens, portions,
// words written.  Returns 0, or a negative code with the message in lia_host_error (nothing is promised about `meta`
// then).
LIA_HOST_EXPORT int lia_step_stage(void* cache, int n_entries, const int* slots, const int* starts, const int* counts,
                                   const int* tokens, const int* want_counts, const int* wants, int vocab,
                                   int max_batch_tokens, int pad_above, int pad_to, int32_t* meta, long long capacity,
                                   int* summary) {
    Cache* c = static_cast<Cache*>(cache);
    if (!c || n_entries < 0 || !meta || !summary) return refuse("lia_step_stage: missing argument");
    // ---- the checks, entry by entry ----
    long long real = 0, wanted = 0;
    int portions = 0;
    static thread_local std::vector<char> seen;
    seen.assign((size_t)c->max_slots, 0);
    const int* token_at = tokens;
    const int* want_at = wants;
    for (int i = 0; i < n_entries; ++i) {
        const int slot = slots[i], start = starts[i], count = counts[i];
        if (count <= 0) return refuse("a step entry brings no tokens");
        const bool known = !c->bad_slot(slot);
        if (known && seen[(size_t)slot]) return refuse("request slot " + std::to_string(slot) + " appears twice in one step");
        if (known) seen[(size_t)slot] = 1;
        const int upto = (known && c->live[(size_t)slot]) ? c->length[(size_t)slot] : -1;
        if (upto < 0) return refuse("request slot " + std::to_string(slot) + " is not live");
        if (start < 0 || (long long)start + count > upto)
            return refuse("slot " + std::to_string(slot) + ": positions [" + std::to_string(start) + ", " +
                          std::to_string((long long)start + count) + ") have no reserved pages (reserved up to " +
                          std::to_string(upto) + ")");
        int low = token_at[0], high = token_at[0];
        for (int t = 1; t < count; ++t) {
            low = std::min(low, token_at[t]);
            high = std::max(high, token_at[t]);
        }
        if (low < 0 || high >= vocab)
            return refuse("token id " + std::to_string(low < 0 ? low : high) + " is outside the vocabulary of " + std::to_string(vocab));
        for (int w = 0; w < want_counts[i]; ++w)
            if (want_at[w] < 0 || want_at[w] >= count)
                return refuse("wanted index " + std::to_string(want_at[w]) + " is outside the entry's " + std::to_string(count) + " tokens");
        real += count;
        wanted += want_counts[i];
        portions += count > 1;
        token_at += count;
        want_at += want_counts[i];
    }
    if (real > max_batch_tokens)
        return refuse(std::to_string(real) + " tokens in one step exceed max_batch_tokens=" + std::to_string(max_batch_tokens));
    const int padding = lia_step_padding((int)real, n_entries, pad_above, pad_to, max_batch_tokens);
    const long long n = real + padding, n_out = wanted + padding;
    const long long total = 4 * n + n_out + 3LL * portions;
    if (total > capacity) return refuse("the step's metadata does not fit its staging buffer");
    // ---- the layout ----
    int32_t* token_part = meta;
    int32_t* position_part = meta + n;
    int32_t* slot_part = meta + 2 * n;
    int32_t* out_rows = meta + 3 * n;
    int32_t* single_rows = out_rows + n_out;
    int32_t* portion_rows = single_rows + (n_entries - portions) + padding;
    int32_t* portion_list = meta + 4 * n + n_out;
    token_at = tokens;
    want_at = wants;
    int row = 0;
    for (int i = 0; i < n_entries; ++i) {
        const int slot = slots[i], start = starts[i], count = counts[i];
        for (int w = 0; w < want_counts[i]; ++w) *out_rows++ = row + want_at[w];
        if (count == 1) {
            *single_rows++ = row;
        } else {
            for (int t = 0; t < count; ++t) *portion_rows++ = row + t;
            *portion_list++ = row;
            *portion_list++ = start;
            *portion_list++ = count;
        }
        for (int t = 0; t < count; ++t) {
            token_part[row + t] = token_at[t];
            position_part[row + t] = start + t;
            slot_part[row + t] = slot;
        }
        row += count;
        token_at += count;
        want_at += want_counts[i];
    }
    for (int k = 0; k < padding; ++k, ++row) {
        token_part[row] = 0;
        position_part[row] = 0;
        slot_part[row] = -1;
        *out_rows++ = row;
        *single_rows++ = row;
    }
    summary[0] = (int)n;
    summary[1] = (int)n_out;
    summary[2] = padding;
    summary[3] = n_entries - portions + padding;
    summary[4] = portions;
    summary[5] = (int)total;
    return 0;
}
