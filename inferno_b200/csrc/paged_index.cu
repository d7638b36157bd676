// Host-side page bookkeeping: the logical-token -> (physical page, offset) map of the reference's
// PagedKvCache (crates/cache/src/paged.rs:40-72, 219-315) for many sequences over one shared pool.
// Pure host code (no CUDA calls): it produces the int32 page table and length arrays that the
// kernels read, allocates pages from a free list, and supports cheap checkpoints (pages are
// immutable once full, so a checkpoint is a length: metal/f16_attention.rs:120-210 only has to copy
// storage because its ring overwrites).
#include <string.h>

#include <string>
#include <vector>

#include "../../include/inferno_attn.h"

struct inf_paged_index {
    int num_pages, page_size, max_seqs, max_pages;
    std::vector<int32_t> table;  // [max_seqs][max_pages], -1 = unmapped
    std::vector<int32_t> lens;   // [max_seqs]
    std::vector<int32_t> mapped; // page slots in use per sequence: slots [trimmed, mapped) hold pages
    std::vector<int32_t> trimmed;  // leading page slots whose pages went back to the pool (inf_paged_index_trim)
    std::vector<int32_t> checkpoint;  // saved length per sequence, -1 = none
    std::vector<int32_t> free_list;   // stack of free physical pages (lowest id on top at start)
    std::string err;
};

static int pi_fail(inf_paged_index* p, int code, const std::string& msg) {
    if (p) p->err = msg;
    return code;
}

extern "C" {

int32_t inf_paged_index_create(int32_t num_pages, int32_t page_size, int32_t max_seqs, int32_t max_pages_per_seq,
                               inf_paged_index** out) {
    if (!out) return INF_E_ARG;
    *out = nullptr;
    // PagedKvCacheSpec::validate (crates/cache/src/paged.rs:16-36)
    if (num_pages <= 0 || page_size <= 0 || max_seqs <= 0 || max_pages_per_seq <= 0) return INF_E_CACHE;
    inf_paged_index* p = new inf_paged_index();
    p->num_pages = num_pages;
    p->page_size = page_size;
    p->max_seqs = max_seqs;
    p->max_pages = max_pages_per_seq;
    p->table.assign((size_t)max_seqs * max_pages_per_seq, -1);
    p->lens.assign(max_seqs, 0);
    p->mapped.assign(max_seqs, 0);
    p->trimmed.assign(max_seqs, 0);
    p->checkpoint.assign(max_seqs, -1);
    p->free_list.resize(num_pages);
    for (int i = 0; i < num_pages; ++i) p->free_list[i] = num_pages - 1 - i;  // pop() yields 0, 1, 2, ...
    *out = p;
    return INF_OK;
}

int32_t inf_paged_index_destroy(inf_paged_index* p) {
    delete p;
    return INF_OK;
}

const char* inf_paged_index_last_error(inf_paged_index* p) { return p ? p->err.c_str() : "null index"; }

int32_t inf_paged_index_append(inf_paged_index* p, int32_t seq, int32_t tokens, int32_t* start_position,
                               int32_t* allocated_pages) {
    if (!p) return INF_E_ARG;
    if (seq < 0 || seq >= p->max_seqs) return pi_fail(p, INF_E_CACHE, "sequence index out of range");
    if (tokens <= 0) return pi_fail(p, INF_E_CACHE, "append needs at least one token");
    const long long end = (long long)p->lens[seq] + tokens;
    const long long need = (end + p->page_size - 1) / p->page_size;
    if (need > p->max_pages)
        return pi_fail(p, INF_E_CACHE, "sequence would exceed max_context (" + std::to_string(end) + " tokens)");
    const int fresh = (int)need - p->mapped[seq];
    if (fresh > (int)p->free_list.size())
        return pi_fail(p, INF_E_CACHE, "page pool exhausted: need " + std::to_string(fresh) + " pages, " +
                                           std::to_string(p->free_list.size()) + " free");
    for (int i = 0; i < fresh; ++i) {
        p->table[(size_t)seq * p->max_pages + p->mapped[seq]] = p->free_list.back();
        p->free_list.pop_back();
        ++p->mapped[seq];
    }
    if (start_position) *start_position = p->lens[seq];
    if (allocated_pages) *allocated_pages = fresh;
    p->lens[seq] = (int32_t)end;
    return INF_OK;
}

int32_t inf_paged_index_locate(inf_paged_index* p, int32_t seq, int32_t token, int32_t* page, int32_t* offset) {
    if (!p) return INF_E_ARG;
    if (seq < 0 || seq >= p->max_seqs) return pi_fail(p, INF_E_CACHE, "sequence index out of range");
    if (token < 0 || token >= p->lens[seq])
        return pi_fail(p, INF_E_CACHE, "token index " + std::to_string(token) + " is outside cached token count " +
                                           std::to_string(p->lens[seq]));
    if (token / p->page_size < p->trimmed[seq])
        return pi_fail(p, INF_E_CACHE, "token index " + std::to_string(token) + " lies in a page that was trimmed away");
    if (page) *page = p->table[(size_t)seq * p->max_pages + token / p->page_size];
    if (offset) *offset = token % p->page_size;
    return INF_OK;
}

int32_t inf_paged_index_len(inf_paged_index* p, int32_t seq) {
    if (!p || seq < 0 || seq >= p->max_seqs) return -1;
    return p->lens[seq];
}

int32_t inf_paged_index_page_count(inf_paged_index* p, int32_t seq) {
    if (!p || seq < 0 || seq >= p->max_seqs) return -1;
    return p->mapped[seq] - p->trimmed[seq];
}

int32_t inf_paged_index_free_pages(inf_paged_index* p) { return p ? (int32_t)p->free_list.size() : -1; }

static void pi_truncate(inf_paged_index* p, int seq, int new_len) {
    const int keep = (new_len + p->page_size - 1) / p->page_size;
    while (p->mapped[seq] > keep) {
        --p->mapped[seq];
        int32_t& slot = p->table[(size_t)seq * p->max_pages + p->mapped[seq]];
        if (slot >= 0) p->free_list.push_back(slot);
        slot = -1;
    }
    if (p->trimmed[seq] > p->mapped[seq]) p->trimmed[seq] = p->mapped[seq];
    p->lens[seq] = new_len;
}

// The sliding-window ring on pages (the reference bounds a sliding layer's cache at 512 slots and overwrites slot
// abs % capacity, crates/backend/src/metal/f16_attention.rs:120-210): once no future query can see a row, its page
// goes back to the pool.  Logical positions do not move: the page-table slots of the released pages become -1 and
// the kernels, which mask everything below the window, never resolve them.
int32_t inf_paged_index_trim(inf_paged_index* p, int32_t seq, int32_t first_visible, int32_t* released_pages) {
    if (!p) return INF_E_ARG;
    if (seq < 0 || seq >= p->max_seqs) return pi_fail(p, INF_E_CACHE, "sequence index out of range");
    if (first_visible < 0) return pi_fail(p, INF_E_CACHE, "first visible token must not be negative");
    if (first_visible > p->lens[seq]) first_visible = p->lens[seq];
    if (p->checkpoint[seq] >= 0 && first_visible > p->checkpoint[seq])
        return pi_fail(p, INF_E_CACHE, "trim would release rows a checkpoint at " + std::to_string(p->checkpoint[seq]) +
                                           " tokens still covers; drop or renew the checkpoint first");
    const int upto = first_visible / p->page_size;  // pages wholly below the first visible token
    int released = 0;
    while (p->trimmed[seq] < upto && p->trimmed[seq] < p->mapped[seq]) {
        int32_t& slot = p->table[(size_t)seq * p->max_pages + p->trimmed[seq]];
        if (slot >= 0) {
            p->free_list.push_back(slot);
            ++released;
        }
        slot = -1;
        ++p->trimmed[seq];
    }
    if (released_pages) *released_pages = released;
    return INF_OK;
}

int32_t inf_paged_index_release(inf_paged_index* p, int32_t seq) {
    if (!p) return INF_E_ARG;
    if (seq < 0 || seq >= p->max_seqs) return pi_fail(p, INF_E_CACHE, "sequence index out of range");
    pi_truncate(p, seq, 0);
    p->trimmed[seq] = 0;
    p->checkpoint[seq] = -1;
    return INF_OK;
}

int32_t inf_paged_index_checkpoint(inf_paged_index* p, int32_t seq) {
    if (!p) return INF_E_ARG;
    if (seq < 0 || seq >= p->max_seqs) return pi_fail(p, INF_E_CACHE, "sequence index out of range");
    p->checkpoint[seq] = p->lens[seq];
    return INF_OK;
}

int32_t inf_paged_index_restore(inf_paged_index* p, int32_t seq) {
    if (!p) return INF_E_ARG;
    if (seq < 0 || seq >= p->max_seqs) return pi_fail(p, INF_E_CACHE, "sequence index out of range");
    if (p->checkpoint[seq] < 0) return pi_fail(p, INF_E_CACHE, "sequence has no checkpoint");
    if (p->checkpoint[seq] > p->lens[seq]) return pi_fail(p, INF_E_CACHE, "checkpoint is ahead of the sequence");
    if (p->checkpoint[seq] < (long long)p->trimmed[seq] * p->page_size)
        return pi_fail(p, INF_E_CACHE, "checkpoint lies below the rows that were trimmed away");
    pi_truncate(p, seq, p->checkpoint[seq]);
    return INF_OK;
}

int32_t inf_paged_index_arrays(inf_paged_index* p, const int32_t** pages, const int32_t** lens, int32_t* max_seqs,
                               int32_t* max_pages) {
    if (!p) return INF_E_ARG;
    if (pages) *pages = p->table.data();
    if (lens) *lens = p->lens.data();
    if (max_seqs) *max_seqs = p->max_seqs;
    if (max_pages) *max_pages = p->max_pages;
    return INF_OK;
}

}  // extern "C"
