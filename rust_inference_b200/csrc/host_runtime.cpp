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
#include <unordered_set>

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
// The generation loop's books: what every request has generated so far and whether it goes on.
//
// The reference's loop serves one prompt (model.rs:332-478): it samples, breaks BEFORE emitting when
// the token is a stop id (model.rs:383-387), emits, and runs at most max_tokens iterations
// (model.rs:373); it keeps every token of prompt and generation for the repetition window
// (model.rs:357, :364, :440).  Here the same rules are kept per request of a batch, with one change:
// a sequence that has no position left in the cache ends with reason "length" instead of a panic
// (kv_cache.rs:54-59).  The loop in Python launches steps and reads tokens; every decision about a
// request is made here.
// ---------------------------------------------------------------------------------------------
namespace {

enum Finish { GEN_LIVE = 0, GEN_STOP = 1, GEN_LENGTH = 2 };

struct GenRequest {
    int prompt_len = 0;
    int finished = GEN_LIVE;
    std::vector<int> tokens;      // generated, stop ids not among them
    std::vector<int> history;     // prompt and generated tokens, kept only when a sampler wants them
};

struct GenBooks {
    int max_tokens, max_seq_len;
    bool keep_history;
    std::unordered_set<int> stop_ids;
    std::vector<GenRequest> reqs;

    // Will the request certainly be stepped again after its `drawn`-th token?  Length limits are known
    // in advance; stop tokens are not.
    bool goes_on(const GenRequest& r, int drawn) const {
        return drawn < max_tokens && r.prompt_len + drawn <= max_seq_len;
    }
};

GenBooks* as_books(void* p) { return static_cast<GenBooks*>(p); }

int check_request(const GenBooks* g, int i) {
    if (i < 0 || i >= (int)g->reqs.size()) return fail(-1, "request %d does not exist (0..%d)", i, (int)g->reqs.size() - 1);
    return 0;
}

}  // namespace

RI_API void* ri_gen_create(int max_tokens, int max_seq_len, const int* stop_ids, int n_stop, int keep_history) {
    if (max_seq_len <= 0) {
        fail(0, "max_seq_len must be positive");
        return nullptr;
    }
    GenBooks* g = new GenBooks{max_tokens, max_seq_len, keep_history != 0, {}, {}};
    for (int i = 0; i < n_stop; ++i) g->stop_ids.insert(stop_ids[i]);
    return g;
}

RI_API void ri_gen_destroy(void* h) { delete as_books(h); }

// A new request; returns its index.
RI_API int ri_gen_add(void* h, const int* prompt, int prompt_len) {
    GenBooks* g = as_books(h);
    if (prompt_len <= 0) return fail(-1, "request %d: empty prompt", (int)g->reqs.size());
    if (prompt_len > g->max_seq_len)
        return fail(-2, "request %d: prompt of %d tokens exceeds max_seq_len %d", (int)g->reqs.size(), prompt_len, g->max_seq_len);
    GenRequest r;
    r.prompt_len = prompt_len;
    if (g->keep_history) r.history.assign(prompt, prompt + prompt_len);
    g->reqs.push_back(std::move(r));
    return (int)g->reqs.size() - 1;
}

// How many requests, starting at `first`, fit the cache together: every admitted request has pages for
// its prompt plus all the tokens it may generate, so a batch never runs out of room half way.
// max_batch <= 0: no limit.  Returns the count (>= 1), or a negative code if even one does not fit.
RI_API int ri_gen_admit(void* h, void* pager, int first, int max_batch) {
    GenBooks* g = as_books(h);
    Pager* p = as_pager(pager);
    long long free_pages = (long long)p->free_pages.size(), free_slots = (long long)p->free_slots.size();
    int n = 0;
    while (first + n < (int)g->reqs.size()) {
        if (max_batch > 0 && n >= max_batch) break;
        const int length = std::min(g->reqs[first + n].prompt_len + g->max_tokens, g->max_seq_len);
        const int need = (length + p->page_size - 1) / p->page_size;
        if (need > free_pages || free_slots == 0) break;
        free_pages -= need;
        free_slots -= 1;
        ++n;
    }
    if (n == 0 && first < (int)g->reqs.size())
        return fail(-3, "request %d (prompt of %d tokens, up to %d more) does not fit the cache even alone", first,
                    g->reqs[first].prompt_len, g->max_tokens);
    return n;
}

// flags[i] = 1 if request idx[i] will certainly be stepped again after its drawn[i]-th token.  Returns how many.
RI_API int ri_gen_goes_on(void* h, int n, const int* idx, const int* drawn, int* flags) {
    GenBooks* g = as_books(h);
    int count = 0;
    for (int i = 0; i < n; ++i) {
        if (int rc = check_request(g, idx[i])) return rc;
        flags[i] = g->goes_on(g->reqs[idx[i]], drawn[i]) ? 1 : 0;
        count += flags[i];
    }
    return count;
}

// Books one sampled token per listed request.  status[i]: 0 the request goes on (the token is to be fed),
// 1 it sampled a stop id (not emitted, not fed back), 2 it ends by length (the token is its last).
// Returns how many go on.
RI_API int ri_gen_book(void* h, int n, const int* idx, const int* tokens, int* status) {
    GenBooks* g = as_books(h);
    int going = 0;
    for (int i = 0; i < n; ++i) {
        if (int rc = check_request(g, idx[i])) return rc;
        GenRequest& r = g->reqs[idx[i]];
        if (r.finished != GEN_LIVE) return fail(-4, "request %d has ended already", idx[i]);
        if (g->stop_ids.count(tokens[i])) {
            r.finished = GEN_STOP;
        } else {
            r.tokens.push_back(tokens[i]);
            if (g->keep_history) r.history.push_back(tokens[i]);
            const int made = (int)r.tokens.size();
            if (made >= g->max_tokens || r.prompt_len + made > g->max_seq_len) r.finished = GEN_LENGTH;   // no position left to feed it at
        }
        status[i] = r.finished;
        going += r.finished == GEN_LIVE;
    }
    return going;
}

RI_API int ri_gen_token_count(void* h, int i) {
    GenBooks* g = as_books(h);
    if (int rc = check_request(g, i)) return rc;
    return (int)g->reqs[i].tokens.size();
}

RI_API int ri_gen_finish(void* h, int i) {
    GenBooks* g = as_books(h);
    if (int rc = check_request(g, i)) return rc;
    return g->reqs[i].finished;
}

// The request's generated tokens into out[0..cap); returns how many there are.
RI_API int ri_gen_tokens(void* h, int i, int* out, int cap) {
    GenBooks* g = as_books(h);
    if (int rc = check_request(g, i)) return rc;
    const std::vector<int>& t = g->reqs[i].tokens;
    for (int k = 0; k < (int)t.size() && k < cap; ++k) out[k] = t[k];
    return (int)t.size();
}

// The last `keep` ids of each listed request's history (prompt and generated tokens) as rows of
// `width` ints, left-aligned, with their counts: what the sampler's repetition window is filled from.
RI_API int ri_gen_recent(void* h, int n, const int* idx, int keep, int width, int* counts, int* rows) {
    GenBooks* g = as_books(h);
    if (!g->keep_history) return fail(-5, "these books keep no history");
    if (keep > width) return fail(-6, "a row of %d ids cannot hold %d", width, keep);
    for (int i = 0; i < n; ++i) {
        if (int rc = check_request(g, idx[i])) return rc;
        const std::vector<int>& hist = g->reqs[idx[i]].history;
        const int take = std::max(0, std::min(keep, (int)hist.size()));
        counts[i] = take;
        for (int k = 0; k < take; ++k) rows[(size_t)i * width + k] = hist[hist.size() - take + k];
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

// ---------------------------------------------------------------------------------------------
// Safetensors files: an 8-byte little-endian header length, a JSON header
// {name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {..}} and the raw
// little-endian data, which is mapped, not read.  The role is the one gguf.rs plays in the
// reference (name -> type, shape, bytes; errors on a bad header: gguf.rs:255-341); the format
// itself is the model folder's.
// ---------------------------------------------------------------------------------------------
#include <cctype>
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <utility>

namespace {

struct StEntry {
    std::string name, dtype;
    std::vector<long long> shape;
    long long begin = 0, end = 0;
};

struct StFile {
    int fd = -1;
    void* map = nullptr;
    size_t size = 0, data_start = 0;
    std::vector<StEntry> entries;
    std::vector<std::pair<std::string, std::string>> metadata;
};

// The little of JSON that a header uses: objects, arrays, strings, integers, and any other value skipped.
struct Json {
    const char* s;
    size_t n, i = 0;
    std::string err;

    bool bad(const char* what) {
        if (err.empty()) err = std::string(what) + " at byte " + std::to_string(i);
        return false;
    }
    void ws() {
        while (i < n && (s[i] == ' ' || s[i] == '\t' || s[i] == '\n' || s[i] == '\r')) ++i;
    }
    bool eat(char c) {
        ws();
        if (i < n && s[i] == c) { ++i; return true; }
        return false;
    }
    bool peek(char c) {
        ws();
        return i < n && s[i] == c;
    }
    static void utf8(std::string& out, unsigned cp) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
        else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    }
    bool hex4(unsigned& v) {
        if (i + 4 > n) return bad("short \\u escape");
        v = 0;
        for (int k = 0; k < 4; ++k) {
            const char c = s[i++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (unsigned)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (unsigned)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (unsigned)(c - 'A' + 10);
            else return bad("bad \\u escape");
        }
        return true;
    }
    bool string(std::string& out) {
        out.clear();
        if (!eat('"')) return bad("expected a string");
        while (i < n) {
            const unsigned char c = (unsigned char)s[i++];
            if (c == '"') return true;
            if (c < 0x20) return bad("control character in a string");
            if (c != '\\') { out += (char)c; continue; }
            if (i >= n) break;
            const char e = s[i++];
            switch (e) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    unsigned cp = 0;
                    if (!hex4(cp)) return false;
                    if (cp >= 0xD800 && cp < 0xDC00 && i + 6 <= n && s[i] == '\\' && s[i + 1] == 'u') {
                        i += 2;
                        unsigned lo;
                        if (!hex4(lo)) return false;
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: return bad("bad escape in a string");
            }
        }
        return bad("unterminated string");
    }
    bool integer(long long& v) {
        ws();
        size_t j = i;
        if (j < n && s[j] == '-') ++j;
        if (j >= n || s[j] < '0' || s[j] > '9') return bad("expected an integer");
        long long x = 0;
        const bool neg = s[i] == '-';
        for (; j < n && s[j] >= '0' && s[j] <= '9'; ++j) {
            if (x > (0x7fffffffffffffffLL - 9) / 10) return bad("integer too large");
            x = x * 10 + (s[j] - '0');
        }
        if (j < n && (s[j] == '.' || s[j] == 'e' || s[j] == 'E')) return bad("expected an integer");
        i = j;
        v = neg ? -x : x;
        return true;
    }
    bool int_array(std::vector<long long>& out) {
        out.clear();
        if (!eat('[')) return bad("expected an array");
        if (eat(']')) return true;
        do {
            long long v;
            if (!integer(v)) return false;
            out.push_back(v);
        } while (eat(','));
        return eat(']') || bad("expected ] or ,");
    }
    // any value, unread
    bool skip(int depth = 0) {
        if (depth > 64) return bad("nested too deeply");
        ws();
        if (i >= n) return bad("unexpected end");
        const char c = s[i];
        if (c == '"') { std::string t; return string(t); }
        if (c == '{') {
            ++i;
            if (eat('}')) return true;
            do {
                std::string k;
                if (!string(k) || !(eat(':') || bad("expected :")) || !skip(depth + 1)) return false;
            } while (eat(','));
            return eat('}') || bad("expected } or ,");
        }
        if (c == '[') {
            ++i;
            if (eat(']')) return true;
            do {
                if (!skip(depth + 1)) return false;
            } while (eat(','));
            return eat(']') || bad("expected ] or ,");
        }
        size_t j = i;
        while (j < n && (isalnum((unsigned char)s[j]) || s[j] == '-' || s[j] == '+' || s[j] == '.')) ++j;
        if (j == i) return bad("unexpected character");
        const std::string tok(s + i, j - i);
        const bool word = tok == "true" || tok == "false" || tok == "null";
        const bool number = !word && (tok[0] == '-' || (tok[0] >= '0' && tok[0] <= '9'));
        if (!word && !number) return bad("unexpected token");
        i = j;
        return true;
    }
};

long long dtype_bytes(const std::string& d) {
    if (d == "F32" || d == "I32") return 4;
    if (d == "BF16" || d == "F16") return 2;
    if (d == "I64") return 8;
    return 0;                                  // not one this library reads
}

std::string shape_text(const std::vector<long long>& shape) {
    std::string t = "[";
    for (size_t k = 0; k < shape.size(); ++k) t += (k ? ", " : "") + std::to_string(shape[k]);
    return t + "]";
}

void st_release(StFile* f) {
    if (f->map) munmap(f->map, f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
}

}  // namespace

// Opens and maps a file and reads its header; null with the reason in ri_last_error.
RI_API void* ri_st_open(const char* path) {
    StFile* f = new StFile;
    auto give_up = [&](const std::string& why) -> void* {
        fail(0, "%s: %s", path, why.c_str());
        st_release(f);
        return nullptr;
    };
    f->fd = open(path, O_RDONLY | O_CLOEXEC);
    if (f->fd < 0) return give_up(strerror(errno));
    struct stat st;
    if (fstat(f->fd, &st) != 0) return give_up(strerror(errno));
    f->size = (size_t)st.st_size;
    if (f->size < 8) return give_up("too short to hold a safetensors header");
    void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) return give_up(std::string("cannot map the file: ") + strerror(errno));
    f->map = m;
    const unsigned char* bytes = static_cast<const unsigned char*>(m);
    unsigned long long hlen = 0;
    for (int k = 7; k >= 0; --k) hlen = (hlen << 8) | bytes[k];
    if (hlen == 0 || hlen > f->size - 8)
        return give_up("header length " + std::to_string(hlen) + " does not fit a file of " + std::to_string(f->size) + " bytes");
    f->data_start = 8 + (size_t)hlen;
    const long long data_len = (long long)(f->size - f->data_start);

    Json js{reinterpret_cast<const char*>(bytes + 8), (size_t)hlen, 0, std::string()};
    auto bad_json = [&]() { return give_up("header is not valid JSON: " + js.err); };
    js.ws();
    if (js.i < js.n && js.s[js.i] != '{') {
        if (!js.skip()) return bad_json();
        return give_up("header must be a JSON object");
    }
    if (!js.eat('{')) { js.bad("expected {"); return bad_json(); }
    if (!js.eat('}')) {
        do {
            std::string name;
            if (!js.string(name) || !(js.eat(':') || js.bad("expected :"))) return bad_json();
            if (name == "__metadata__") {
                if (js.peek('{')) {
                    js.eat('{');
                    if (!js.eat('}')) {
                        do {
                            std::string k, v;
                            if (!js.string(k) || !(js.eat(':') || js.bad("expected :"))) return bad_json();
                            if (js.peek('"')) {
                                if (!js.string(v)) return bad_json();
                                f->metadata.emplace_back(k, v);
                            } else if (!js.skip()) {
                                return bad_json();
                            }
                        } while (js.eat(','));
                        if (!js.eat('}')) { js.bad("expected } or ,"); return bad_json(); }
                    }
                } else if (!js.skip()) {
                    return bad_json();
                }
                continue;
            }
            StEntry e;
            e.name = name;
            bool has_dtype = false, has_shape = false, has_offsets = false, malformed = false;
            if (!js.peek('{')) {
                if (!js.skip()) return bad_json();
                malformed = true;
            } else {
                js.eat('{');
                if (!js.eat('}')) {
                    do {
                        std::string k;
                        if (!js.string(k) || !(js.eat(':') || js.bad("expected :"))) return bad_json();
                        const size_t at = js.i;
                        if (k == "dtype" && js.peek('"')) {
                            if (!js.string(e.dtype)) return bad_json();
                            has_dtype = true;
                        } else if (k == "shape" && js.peek('[')) {
                            if (js.int_array(e.shape)) has_shape = true;
                            else { js.i = at; js.err.clear(); if (!js.skip()) return bad_json(); malformed = true; }
                        } else if (k == "data_offsets" && js.peek('[')) {
                            std::vector<long long> o;
                            if (js.int_array(o) && o.size() == 2) { e.begin = o[0]; e.end = o[1]; has_offsets = true; }
                            else { js.i = at; js.err.clear(); if (!js.skip()) return bad_json(); malformed = true; }
                        } else {
                            if (k == "dtype" || k == "shape" || k == "data_offsets") malformed = true;
                            if (!js.skip()) return bad_json();
                        }
                    } while (js.eat(','));
                    if (!js.eat('}')) { js.bad("expected } or ,"); return bad_json(); }
                }
            }
            if (malformed || !has_dtype || !has_shape || !has_offsets) return give_up("malformed header entry for '" + name + "'");
            const long long unit = dtype_bytes(e.dtype);
            if (unit > 0) {
                long long want = unit;
                for (long long d : e.shape) {
                    if (d < 0 || (d > 0 && want > 0x7fffffffffffffffLL / d)) return give_up("malformed header entry for '" + name + "'");
                    want *= d;
                }
                if (e.end - e.begin != want)
                    return give_up("'" + name + "' has " + std::to_string(e.end - e.begin) + " bytes, shape " + shape_text(e.shape) +
                                   " of " + e.dtype + " needs " + std::to_string(want));
            }
            if (e.begin < 0 || e.end < e.begin || e.end > data_len)
                return give_up("'" + name + "' data_offsets [" + std::to_string(e.begin) + ", " + std::to_string(e.end) +
                               ") lie outside the " + std::to_string(data_len) + " data bytes");
            f->entries.push_back(std::move(e));
        } while (js.eat(','));
        if (!js.eat('}')) { js.bad("expected } or ,"); return bad_json(); }
    }
    js.ws();
    if (js.i != js.n) { js.bad("text after the header object"); return bad_json(); }
    return f;
}

RI_API void ri_st_close(void* h) {
    if (h) st_release(static_cast<StFile*>(h));
}

RI_API int ri_st_count(void* h) { return (int)static_cast<StFile*>(h)->entries.size(); }

// Entry i: its name and dtype (UTF-8, valid until the file is closed), its shape, and where its bytes lie
// among the data.
RI_API int ri_st_entry(void* h, int i, const char** name, const char** dtype, int* ndim, const long long** shape,
                       long long* begin, long long* end) {
    StFile* f = static_cast<StFile*>(h);
    if (i < 0 || i >= (int)f->entries.size()) return fail(-1, "no entry %d", i);
    const StEntry& e = f->entries[i];
    *name = e.name.c_str();
    *dtype = e.dtype.c_str();
    *ndim = (int)e.shape.size();
    *shape = e.shape.data();
    *begin = e.begin;
    *end = e.end;
    return 0;
}

// The mapped data (what data_offsets count from) and its length.
RI_API const void* ri_st_data(void* h, long long* length) {
    StFile* f = static_cast<StFile*>(h);
    if (length) *length = (long long)(f->size - f->data_start);
    return static_cast<const unsigned char*>(f->map) + f->data_start;
}

RI_API int ri_st_metadata_count(void* h) { return (int)static_cast<StFile*>(h)->metadata.size(); }

RI_API int ri_st_metadata(void* h, int i, const char** key, const char** value) {
    StFile* f = static_cast<StFile*>(h);
    if (i < 0 || i >= (int)f->metadata.size()) return fail(-1, "no metadata entry %d", i);
    *key = f->metadata[i].first.c_str();
    *value = f->metadata[i].second.c_str();
    return 0;
}
