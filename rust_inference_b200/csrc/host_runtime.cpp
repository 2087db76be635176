// The host side of the runtime that runs at every step: the books of the cache (slots, pages,
// lengths) and the packing of a step's batch into the int32 arrays the kernels read.  Plain C++
// with a C ABI, no CUDA; the Python classes in cache/pager.py and engine/context.py are its faces.
//
// The reference keeps one cache per layer for its single sequence, with a length counter, an
// append that asserts on overflow and a clear (kv_cache.rs:40-75, :122-124), and passes each
// token's position by hand (model.rs:361-363, :431-433).  Here a slot stands for one sequence of
// a batch; its keys and values live in pages of `page_size` positions taken from a shared pool;
// a step's tokens, positions and places are laid out once per step for every kernel.
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <vector>

#define RI_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

// ---------------------------------------------------------------------------------------------
// Slots, pages and lengths.
// ---------------------------------------------------------------------------------------------
enum PagerError {
    PG_FULL = -1,            // no free slot, or not enough free pages
    PG_NO_SUCH_SLOT = -2,
    PG_SLOT_NOT_LIVE = -3,   // never allocated, or freed already
    PG_TOO_LONG = -4,        // beyond max_seq_len
    PG_BAD_LENGTH = -5,      // a length beyond the slot's reserved pages
    PG_SMALL_BUFFER = -6,
};

struct Pager {
    int n_slots, n_pages, page_size, max_seq_len;
    std::vector<int> free_slots, free_pages;       // handed out from the end: low numbers first
    std::vector<char> live;
    std::vector<int> length;
    std::vector<std::vector<int>> pages;

    int check(int slot) const {
        if (slot < 0 || slot >= n_slots) return fail(PG_NO_SUCH_SLOT, "slot %d does not exist (0..%d)", slot, n_slots - 1);
        if (!live[slot]) return fail(PG_SLOT_NOT_LIVE, "slot %d is not in use (never allocated, or freed already)", slot);
        return 0;
    }
    int pages_needed(int slot, int new_length) const {
        const int want = (new_length + page_size - 1) / page_size;
        return std::max(0, want - (int)pages[slot].size());
    }
};

Pager* as_pager(void* p) { return static_cast<Pager*>(p); }

}  // namespace

RI_API const char* ri_last_error() { return g_error; }

RI_API void* ri_pager_create(int n_slots, int n_pages, int page_size, int max_seq_len) {
    if (n_slots <= 0 || n_pages <= 0 || page_size <= 0 || max_seq_len <= 0) {
        fail(0, "cache sizes must be positive");
        return nullptr;
    }
    Pager* p = new Pager{n_slots, n_pages, page_size, max_seq_len, {}, {}, {}, {}, {}};
    p->free_slots.resize(n_slots);
    p->free_pages.resize(n_pages);
    for (int i = 0; i < n_slots; ++i) p->free_slots[i] = n_slots - 1 - i;
    for (int i = 0; i < n_pages; ++i) p->free_pages[i] = n_pages - 1 - i;
    p->live.assign(n_slots, 0);
    p->length.assign(n_slots, 0);
    p->pages.assign(n_slots, {});
    return p;
}

RI_API void ri_pager_destroy(void* h) { delete as_pager(h); }

RI_API int ri_pager_alloc_slot(void* h) {
    Pager* p = as_pager(h);
    if (p->free_slots.empty()) return fail(PG_FULL, "all %d cache slots are in use", p->n_slots);
    const int s = p->free_slots.back();
    p->free_slots.pop_back();
    p->live[s] = 1;
    p->length[s] = 0;
    return s;
}

RI_API int ri_pager_free_slot(void* h, int slot) {
    Pager* p = as_pager(h);
    if (int rc = p->check(slot)) return rc;
    // the slot's pages go back so that the one taken last is handed out first again
    for (auto it = p->pages[slot].rbegin(); it != p->pages[slot].rend(); ++it) p->free_pages.push_back(*it);
    p->pages[slot].clear();
    p->length[slot] = 0;
    p->live[slot] = 0;
    p->free_slots.push_back(slot);
    return 0;
}

RI_API int ri_pager_length(void* h, int slot) {
    Pager* p = as_pager(h);
    if (int rc = p->check(slot)) return rc;
    return p->length[slot];
}

RI_API int ri_pager_page_count(void* h, int slot) {
    Pager* p = as_pager(h);
    if (int rc = p->check(slot)) return rc;
    return (int)p->pages[slot].size();
}

// The slot's pages, in order, into out[0..cap); returns how many there are.
RI_API int ri_pager_pages(void* h, int slot, int* out, int cap) {
    Pager* p = as_pager(h);
    if (int rc = p->check(slot)) return rc;
    const int n = (int)p->pages[slot].size();
    if (n > cap) return fail(PG_SMALL_BUFFER, "slot %d holds %d pages, the buffer %d", slot, n, cap);
    std::copy(p->pages[slot].begin(), p->pages[slot].end(), out);
    return n;
}

RI_API int ri_pager_pages_needed(void* h, int slot, int new_length) {
    Pager* p = as_pager(h);
    if (int rc = p->check(slot)) return rc;
    return p->pages_needed(slot, new_length);
}

// Room for positions < new_lengths[i] in slots[i], for all n pairs or for none.  The pages added go,
// pair after pair, to added_pages[0..cap) and their numbers per pair to added_counts[0..n); returns
// how many pages were added in all.
RI_API int ri_pager_reserve_many(void* h, int n, const int* slots, const int* new_lengths, int* added_counts,
                                 int* added_pages, int cap) {
    Pager* p = as_pager(h);
    long long total = 0;
    for (int i = 0; i < n; ++i) {
        if (int rc = p->check(slots[i])) return rc;
        if (new_lengths[i] > p->max_seq_len)
            return fail(PG_TOO_LONG, "slot %d: %d positions exceed max_seq_len %d", slots[i], new_lengths[i], p->max_seq_len);
    }
    // a slot may be named twice: count against what the earlier pairs will have added
    std::vector<int> planned(n, 0);
    for (int i = 0; i < n; ++i) {
        int have = (int)p->pages[slots[i]].size();
        for (int j = 0; j < i; ++j)
            if (slots[j] == slots[i]) have += planned[j];
        const int want = (new_lengths[i] + p->page_size - 1) / p->page_size;
        planned[i] = std::max(0, want - have);
        total += planned[i];
    }
    if (total > (long long)p->free_pages.size()) {
        if (n == 1)
            return fail(PG_FULL, "cache is full: slot %d needs %lld more pages of %d positions, %d of %d are free", slots[0],
                        total, p->page_size, (int)p->free_pages.size(), p->n_pages);
        return fail(PG_FULL, "cache is full: the step needs %lld more pages of %d positions, %d of %d are free", total,
                    p->page_size, (int)p->free_pages.size(), p->n_pages);
    }
    if (total > cap) return fail(PG_SMALL_BUFFER, "the step adds %lld pages, the buffer holds %d", total, cap);
    int k = 0;
    for (int i = 0; i < n; ++i) {
        added_counts[i] = planned[i];
        for (int j = 0; j < planned[i]; ++j) {
            const int page = p->free_pages.back();
            p->free_pages.pop_back();
            p->pages[slots[i]].push_back(page);
            added_pages[k++] = page;
        }
    }
    return k;
}

RI_API int ri_pager_set_length(void* h, int slot, int length) {
    Pager* p = as_pager(h);
    if (int rc = p->check(slot)) return rc;
    if ((long long)length > (long long)p->pages[slot].size() * p->page_size)
        return fail(PG_BAD_LENGTH, "slot %d: length %d exceeds its reserved pages", slot, length);
    p->length[slot] = length;
    return 0;
}

RI_API int ri_pager_free_slot_count(void* h) { return (int)as_pager(h)->free_slots.size(); }
RI_API int ri_pager_free_page_count(void* h) { return (int)as_pager(h)->free_pages.size(); }

// The slots in use, ascending, into out[0..n_slots); returns how many.
RI_API int ri_pager_live_slots(void* h, int* out) {
    Pager* p = as_pager(h);
    int k = 0;
    for (int s = 0; s < p->n_slots; ++s)
        if (p->live[s]) out[k++] = s;
    return k;
}

// Hand out the highest page numbers first from now on (the free pages in reverse order): for tests
// that want a sequence at the far end of the pool.
RI_API void ri_pager_prefer_high_pages(void* h) {
    Pager* p = as_pager(h);
    std::sort(p->free_pages.begin(), p->free_pages.end());
}

// Every slot and every page is either free or held, exactly once: 0, or a negative code with the
// finding in ri_last_error.
RI_API int ri_pager_audit(void* h) {
    Pager* p = as_pager(h);
    std::vector<int> seen(p->n_pages, 0);
    for (int pg : p->free_pages) {
        if (pg < 0 || pg >= p->n_pages) return fail(-1, "page accounting broken: a page is lost or held twice");
        ++seen[pg];
    }
    for (int s = 0; s < p->n_slots; ++s)
        for (int pg : p->pages[s]) {
            if (pg < 0 || pg >= p->n_pages) return fail(-1, "page accounting broken: a page is lost or held twice");
            ++seen[pg];
        }
    for (int c : seen)
        if (c != 1) return fail(-1, "page accounting broken: a page is lost or held twice");
    std::vector<int> slot_seen(p->n_slots, 0);
    for (int s : p->free_slots) {
        if (s < 0 || s >= p->n_slots) return fail(-1, "slot accounting broken: a slot is lost or held twice");
        ++slot_seen[s];
    }
    for (int s = 0; s < p->n_slots; ++s) {
        if (p->live[s]) ++slot_seen[s];
        if (slot_seen[s] != 1) return fail(-1, "slot accounting broken: a slot is lost or held twice");
        if (!p->live[s] && (!p->pages[s].empty() || p->length[s] != 0))
            return fail(-1, "free slot %d still holds pages or a length", s);
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// A step's batch as int32 arrays: T tokens of B sequences, sequence after sequence, no padding.
//
//   token_ids[T] token_pos[T] token_seq[T] seq_slot[B] seq_start[B] seq_len[B] cu_seqlens[B+1] logit_rows[R]
//
// in this order in `meta` (T + T + T + B + B + B + B + 1 + R entries).  starts[b]: positions already
// cached for sequence b; counts[b] and tokens: its new tokens, one sequence after the other;
// want_counts[b] and wants: places among its tokens whose logits are wanted; slots may be null
// (the caller fills them in).  scalars receives {most tokens a sequence brings, longest sequence
// after the step, 1 if every sequence brings exactly one token}.  Returns the entries written.
// ---------------------------------------------------------------------------------------------
RI_API long long ri_pack_step(int n_seqs, const int* starts, const int* counts, const int* tokens, const int* slots,
                              const int* want_counts, const int* wants, int* meta, long long meta_cap, int* scalars) {
    long long T = 0, R = 0;
    for (int b = 0; b < n_seqs; ++b) {
        if (counts[b] < 0 || want_counts[b] < 0) return fail(-1, "sequence %d: negative count", b);
        T += counts[b];
        R += want_counts[b];
    }
    const long long need = 3 * T + 4LL * n_seqs + 1 + R;
    if (need > meta_cap) return fail(-2, "the step needs %lld entries, the buffer holds %lld", need, meta_cap);
    if (T > 0x7fffffffLL) return fail(-3, "a step of %lld tokens exceeds the index range", T);
    int* ids = meta;
    int* pos = ids + T;
    int* seq = pos + T;
    int* slot = seq + T;
    int* start = slot + n_seqs;
    int* len = start + n_seqs;
    int* cu = len + n_seqs;
    int* rows = cu + n_seqs + 1;
    long long t = 0, r = 0, w = 0;
    int max_new = 0, max_len = 0, all_single = n_seqs > 0 ? 1 : 0;
    for (int b = 0; b < n_seqs; ++b) {
        const int c = counts[b];
        cu[b] = (int)t;
        for (int i = 0; i < c; ++i) {
            ids[t + i] = tokens[t + i];
            pos[t + i] = starts[b] + i;
            seq[t + i] = b;
        }
        for (int i = 0; i < want_counts[b]; ++i) {
            const int place = wants[w + i];
            if (place < 0 || place >= c) return fail(-4, "sequence %d: wanted place %d is outside its %d tokens", b, place, c);
            rows[r++] = (int)t + place;
        }
        w += want_counts[b];
        slot[b] = slots ? slots[b] : 0;
        start[b] = starts[b];
        len[b] = starts[b] + c;
        max_new = std::max(max_new, c);
        max_len = std::max(max_len, starts[b] + c);
        if (c != 1) all_single = 0;
        t += c;
    }
    cu[n_seqs] = (int)t;
    scalars[0] = max_new;
    scalars[1] = max_len;
    scalars[2] = all_single;
    return need;
}

// The lengths of n slots at once, and n slots moved on by counts[i] positions (a step's commit).
RI_API int ri_pager_lengths(void* h, int n, const int* slots, int* out) {
    Pager* p = as_pager(h);
    for (int i = 0; i < n; ++i) {
        if (int rc = p->check(slots[i])) return rc;
        out[i] = p->length[slots[i]];
    }
    return 0;
}

RI_API int ri_pager_advance(void* h, int n, const int* slots, const int* counts) {
    Pager* p = as_pager(h);
    for (int i = 0; i < n; ++i) {
        if (int rc = p->check(slots[i])) return rc;
        const long long length = (long long)p->length[slots[i]] + counts[i];
        if (counts[i] < 0 || length > (long long)p->pages[slots[i]].size() * p->page_size)
            return fail(PG_BAD_LENGTH, "slot %d: length %lld exceeds its reserved pages", slots[i], length);
    }
    for (int i = 0; i < n; ++i) p->length[slots[i]] += counts[i];
    return 0;
}
