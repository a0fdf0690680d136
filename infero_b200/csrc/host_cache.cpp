// Host-side bookkeeping of the paged cache, and the builder of a step's device inputs.
//
// Who holds which page of which layer group, one block table per request and group, the
// rule by which a window group gives pages back, and the state slots: the same job as the
// reference's KvPool / SeqState (crates/model/src/cache.rs:100-249, :320-339, :567-594,
// :656-679), with pages of page_size tokens instead of one-token slots, and a group per kind
// of cache.  Plain C++ without CUDA; the Python class infero_b200.cache.CacheManager is a thin
// wrapper over the C functions at the end of this file.
//
// Rules.  A page is free or held by exactly one request.  reserve() takes the pages n more
// tokens need in every group, or none at all.  commit() advances the length and, in a group
// with window W, returns every page whose last position is <= length - W (the next query, at
// position >= length, sees keys j > p - W only); its table entry becomes -1.  abort() drops
// what was reserved and not committed.  close() returns everything.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

struct Group {
    int window = 0;                          // 0: every key is kept
    int num_pages = 0;                       // this group's own pool
    std::vector<int> free_stack;             // lowest page on top, so the first request gets page 0 upward
    std::vector<uint8_t> held, ever_held;
};

struct Request {
    bool open = false, fresh = true;
    int length = 0, reserved = 0;
    std::vector<std::vector<int>> tables;    // per group: logical page -> page id, -1 once given back
    std::vector<int> first_live;             // per group: first logical page still held
};

struct Cache {
    int page_size = 0, max_requests = 0, max_blocks = 0;   // max_blocks 0: no limit
    std::vector<Group> groups;
    std::vector<Request> reqs;
    std::vector<int> free_slots;             // lowest slot on top
    // device-bound copy of the tables: per group [max_requests, width], -1 where nothing is held
    int width = 1;
    std::vector<std::vector<int>> mirror;
    long long reclaimed = 0, reused = 0;
    std::string error;

    void grow(int need) {
        if (need <= width) return;
        int w = std::max(need, 2 * width);
        for (auto& m : mirror) {
            std::vector<int> wider((size_t)max_requests * w, -1);
            for (int r = 0; r < max_requests; ++r)
                std::copy(m.begin() + (size_t)r * width, m.begin() + (size_t)(r + 1) * width, wider.begin() + (size_t)r * w);
            m.swap(wider);
        }
        width = w;
    }
    int pages_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
    void give_back(int g, int page) {
        Group& G = groups[g];
        G.held[page] = 0;
        G.free_stack.push_back(page);
    }
};

bool valid_slot(const Cache* c, int slot) { return slot >= 0 && slot < c->max_requests && c->reqs[slot].open; }

}  // namespace

extern "C" {

// Every group has a pool of its own, of num_pages[g] pages: a group that keeps a window of keys needs
// far fewer than one that keeps them all.
void* infero_cache_new(int n_groups, const int* windows, const int* pages_per_group, int page_size, int max_requests,
                       int max_blocks) {
    if (n_groups < 0 || page_size <= 0 || max_requests <= 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (pages_per_group[g] <= 0) return nullptr;
    Cache* c = new Cache();
    c->page_size = page_size; c->max_requests = max_requests; c->max_blocks = max_blocks;
    c->groups.resize(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        Group& G = c->groups[g];
        G.window = windows[g];
        G.num_pages = pages_per_group[g];
        const int num_pages = G.num_pages;
        G.free_stack.resize(num_pages);
        for (int p = 0; p < num_pages; ++p) G.free_stack[p] = num_pages - 1 - p;
        G.held.assign(num_pages, 0);
        G.ever_held.assign(num_pages, 0);
    }
    c->reqs.resize(max_requests);
    c->free_slots.resize(max_requests);
    for (int s = 0; s < max_requests; ++s) c->free_slots[s] = max_requests - 1 - s;
    c->width = max_blocks > 0 ? max_blocks : 1;
    c->mirror.assign(n_groups, std::vector<int>((size_t)max_requests * c->width, -1));
    return c;
}

void infero_cache_delete(void* h) { delete static_cast<Cache*>(h); }

// -> slot, or -1 when every slot is taken
int infero_cache_open(void* h) {
    Cache* c = static_cast<Cache*>(h);
    if (c->free_slots.empty()) return -1;
    const int slot = c->free_slots.back();
    c->free_slots.pop_back();
    Request& r = c->reqs[slot];
    r = Request();
    r.open = true;
    r.tables.assign(c->groups.size(), {});
    r.first_live.assign(c->groups.size(), 0);
    for (auto& m : c->mirror) std::fill(m.begin() + (size_t)slot * c->width, m.begin() + (size_t)(slot + 1) * c->width, -1);
    return slot;
}

int infero_cache_close(void* h, int slot) {
    Cache* c = static_cast<Cache*>(h);
    if (!valid_slot(c, slot)) return 1;
    Request& r = c->reqs[slot];
    for (size_t g = 0; g < c->groups.size(); ++g)
        for (int p : r.tables[g])
            if (p >= 0) c->give_back((int)g, p);
    r.open = false;
    r.tables.clear();
    c->free_slots.push_back(slot);
    return 0;
}

int infero_cache_length(void* h, int slot) { return static_cast<Cache*>(h)->reqs[slot].length; }
int infero_cache_reserved(void* h, int slot) { return static_cast<Cache*>(h)->reqs[slot].reserved; }
int infero_cache_fresh(void* h, int slot) { return static_cast<Cache*>(h)->reqs[slot].fresh ? 1 : 0; }
int infero_cache_num_free(void* h, int group) { return (int)static_cast<Cache*>(h)->groups[group].free_stack.size(); }
int infero_cache_table_len(void* h, int group, int slot) { return (int)static_cast<Cache*>(h)->reqs[slot].tables[group].size(); }
int infero_cache_first_live(void* h, int group, int slot) { return static_cast<Cache*>(h)->reqs[slot].first_live[group]; }
// n_groups, pages of the largest pool, page_size, max_requests
void infero_cache_geometry(void* h, int* out) {
    Cache* c = static_cast<Cache*>(h);
    int most = 0;
    for (const Group& G : c->groups) most = std::max(most, G.num_pages);
    out[0] = (int)c->groups.size(); out[1] = most; out[2] = c->page_size; out[3] = c->max_requests;
}
int infero_cache_group_pages(void* h, int group) { return static_cast<Cache*>(h)->groups[group].num_pages; }
int infero_cache_group_window(void* h, int group) { return static_cast<Cache*>(h)->groups[group].window; }
// Pages of group g that the request in `slot` holds now (a window group's table also lists, as -1, what it gave back).
int infero_cache_held_by(void* h, int group, int slot) {
    Cache* c = static_cast<Cache*>(h);
    const Request& r = c->reqs[slot];
    return (int)r.tables[group].size() - r.first_live[group];
}
// The most pages of group g a request of n_tokens ever holds at once when it is fed in portions of at
// most max_chunk tokens: all of them in a group that keeps every key; in a group with window W what
// covers the W - 1 keys before a portion and the portion itself.
int infero_cache_most_pages(void* h, int group, int n_tokens, int max_chunk) {
    Cache* c = static_cast<Cache*>(h);
    const int all = c->pages_for(n_tokens), W = c->groups[group].window;
    if (W <= 0) return all;
    return std::min(all, c->pages_for(W - 1 + std::max(1, max_chunk)) + 1);
}
int infero_cache_width(void* h) { return static_cast<Cache*>(h)->width; }
const int* infero_cache_mirror(void* h, int group) { return static_cast<Cache*>(h)->mirror[group].data(); }
long long infero_cache_counter(void* h, int which) {
    Cache* c = static_cast<Cache*>(h);
    return which == 0 ? c->reclaimed : c->reused;
}
const char* infero_cache_error(void* h) { return static_cast<Cache*>(h)->error.c_str(); }

// out[g] = new pages group g would need for n_new more tokens
void infero_cache_pages_needed(void* h, int slot, int n_new, int* out) {
    Cache* c = static_cast<Cache*>(h);
    const Request& r = c->reqs[slot];
    const int want = c->pages_for(r.length + r.reserved + n_new);
    for (size_t g = 0; g < c->groups.size(); ++g) out[g] = std::max(0, want - (int)r.tables[g].size());
}

// 0: done.  1: a group is short (info = group, wanted, free).  2: the request would exceed
// max_blocks pages (info = -1, wanted, max_blocks).  Nothing is taken unless 0 is returned.
int infero_cache_reserve(void* h, int slot, int n_new, int* info) {
    Cache* c = static_cast<Cache*>(h);
    Request& r = c->reqs[slot];
    const int want = c->pages_for(r.length + r.reserved + n_new);
    if (c->max_blocks > 0 && want > c->max_blocks) {
        info[0] = -1; info[1] = want; info[2] = c->max_blocks;
        return 2;
    }
    const int G = (int)c->groups.size();
    for (int g = 0; g < G; ++g) {
        const int need = std::max(0, want - (int)r.tables[g].size());
        if (need > (int)c->groups[g].free_stack.size()) {
            info[0] = g; info[1] = need; info[2] = (int)c->groups[g].free_stack.size();
            return 1;
        }
    }
    c->grow(want);
    for (int g = 0; g < G; ++g) {
        Group& grp = c->groups[g];
        int* row = c->mirror[g].data() + (size_t)slot * c->width;
        while ((int)r.tables[g].size() < want) {
            const int p = grp.free_stack.back();
            grp.free_stack.pop_back();
            grp.held[p] = 1;
            if (grp.ever_held[p]) ++c->reused;
            grp.ever_held[p] = 1;
            row[r.tables[g].size()] = p;
            r.tables[g].push_back(p);
        }
    }
    r.reserved += n_new;
    return 0;
}

// 0: done.  1: more tokens than were reserved.
int infero_cache_commit(void* h, int slot, int n_new) {
    Cache* c = static_cast<Cache*>(h);
    Request& r = c->reqs[slot];
    if (n_new > r.reserved) return 1;
    r.reserved -= n_new;
    r.length += n_new;
    r.fresh = false;
    const int P = c->page_size;
    for (size_t g = 0; g < c->groups.size(); ++g) {
        const int W = c->groups[g].window;
        if (W <= 0) continue;
        // logical page k covers [kP, kP + P - 1]; it is dead iff kP + P - 1 <= length - W
        const int live_from = r.length - W + 1;
        const int dead_upto = live_from > 0 ? live_from / P : 0;
        std::vector<int>& t = r.tables[g];
        int* row = c->mirror[g].data() + (size_t)slot * c->width;
        int k = r.first_live[g];
        while (k < dead_upto && k < (int)t.size()) {
            if (t[k] >= 0) {
                c->give_back((int)g, t[k]);
                t[k] = -1;
                row[k] = -1;
                ++c->reclaimed;
            }
            ++k;
        }
        r.first_live[g] = k;
    }
    return 0;
}

// Forget the tokens from position `length` on (the reference's KvPool::truncate,
// crates/model/src/cache.rs:656-679): pages that lie wholly behind the new end go back, the rest
// stays.  0: done.  1: nothing to cut (length above what is cached), or a step is in flight.
// 2: a window group has already given back pages that a query at `length` would see, so the
// request cannot go back that far.  Nothing changes unless 0 is returned.
int infero_cache_truncate(void* h, int slot, int length) {
    Cache* c = static_cast<Cache*>(h);
    if (!valid_slot(c, slot)) return 1;
    Request& r = c->reqs[slot];
    if (length < 0 || length > r.length || r.reserved != 0) return 1;
    const int P = c->page_size;
    for (size_t g = 0; g < c->groups.size(); ++g) {
        const int W = c->groups[g].window;
        if (W <= 0) continue;
        // at the new length, pages whose last position is <= length - W may be missing, no others
        const int live_from = length - W + 1;
        const int may_be_dead = live_from > 0 ? live_from / P : 0;
        if (r.first_live[g] > may_be_dead) return 2;
    }
    const int keep = c->pages_for(length);
    for (size_t g = 0; g < c->groups.size(); ++g) {
        std::vector<int>& t = r.tables[g];
        int* row = c->mirror[g].data() + (size_t)slot * c->width;
        for (int k = keep; k < (int)t.size(); ++k) {
            if (t[k] >= 0) c->give_back((int)g, t[k]);
            row[k] = -1;
        }
        if ((int)t.size() > keep) t.resize(keep);
        if (r.first_live[g] > keep) r.first_live[g] = keep;
    }
    r.length = length;
    if (length == 0) r.fresh = true;
    return 0;
}

void infero_cache_abort(void* h, int slot) {
    Cache* c = static_cast<Cache*>(h);
    Request& r = c->reqs[slot];
    if (r.reserved == 0) return;
    const int keep = c->pages_for(r.length);
    for (size_t g = 0; g < c->groups.size(); ++g) {
        std::vector<int>& t = r.tables[g];
        int* row = c->mirror[g].data() + (size_t)slot * c->width;
        for (int k = keep; k < (int)t.size(); ++k) {
            if (t[k] >= 0) c->give_back((int)g, t[k]);
            row[k] = -1;
        }
        if ((int)t.size() > keep) t.resize(keep);
    }
    r.reserved = 0;
}

// The pages group g holds, ascending; returns how many (out may be null to count).
int infero_cache_held(void* h, int group, int* out, int cap) {
    Cache* c = static_cast<Cache*>(h);
    int n = 0;
    for (int p = 0; p < c->groups[group].num_pages; ++p)
        if (c->groups[group].held[p]) {
            if (out && n < cap) out[n] = p;
            ++n;
        }
    return n;
}

// 0 when every invariant holds; else 1 and infero_cache_error() says which one broke.
int infero_cache_check(void* h) {
    Cache* c = static_cast<Cache*>(h);
    char buf[256];
    for (size_t g = 0; g < c->groups.size(); ++g) {
        const Group& G = c->groups[g];
        const int num_pages = G.num_pages;
        std::vector<uint8_t> seen(num_pages, 0);
        int held = 0;
        for (int s = 0; s < c->max_requests; ++s) {
            const Request& r = c->reqs[s];
            if (!r.open) continue;
            const int* row = c->mirror[g].data() + (size_t)s * c->width;
            for (size_t k = 0; k < r.tables[g].size(); ++k) {
                const int p = r.tables[g][k];
                if (row[k] != p) {
                    snprintf(buf, sizeof buf, "group %zu: the table copy of slot %d is out of date at block %zu", g, s, k);
                    c->error = buf;
                    return 1;
                }
                if (p < 0) continue;
                if (p >= num_pages || seen[p]) {
                    snprintf(buf, sizeof buf, "group %zu: page %d is held twice", g, p);
                    c->error = buf;
                    return 1;
                }
                seen[p] = 1;
                ++held;
            }
            for (int k = (int)r.tables[g].size(); k < c->width; ++k)
                if (row[k] != -1) {
                    snprintf(buf, sizeof buf, "group %zu: the table copy of slot %d has an entry past its end", g, s);
                    c->error = buf;
                    return 1;
                }
        }
        for (int p = 0; p < num_pages; ++p)
            if ((seen[p] != 0) != (G.held[p] != 0)) {
                snprintf(buf, sizeof buf, "group %zu: page %d lost or leaked (tables and allocator disagree)", g, p);
                c->error = buf;
                return 1;
            }
        if (held + (int)G.free_stack.size() != num_pages) {
            snprintf(buf, sizeof buf, "group %zu: %d held + %zu free != %d", g, held, G.free_stack.size(), num_pages);
            c->error = buf;
            return 1;
        }
        std::vector<uint8_t> on_free(num_pages, 0);
        for (int p : G.free_stack) {
            if (on_free[p] || G.held[p]) {
                snprintf(buf, sizeof buf, "group %zu: page %d is on the free list twice, or free and held", g, p);
                c->error = buf;
                return 1;
            }
            on_free[p] = 1;
        }
    }
    std::vector<uint8_t> slot_seen(c->max_requests, 0);
    int open = 0;
    for (int s = 0; s < c->max_requests; ++s) open += c->reqs[s].open ? 1 : 0;
    for (int s : c->free_slots) {
        if (slot_seen[s] || c->reqs[s].open) { c->error = "a state slot is held twice"; return 1; }
        slot_seen[s] = 1;
    }
    if (open + (int)c->free_slots.size() != c->max_requests) { c->error = "a state slot was lost"; return 1; }
    return 0;
}

// The int32 arrays of a step, written one after the other into out (capacity cap ints):
//   token ids [T] (a negative id -1 of a single-token entry becomes -(slot + 1): "from the device"),
//   positions [T], token -> entry [T], then per entry first row, row count, cached length, slot [E each],
//   the rows whose logits are wanted [R], and per group the block table [E, table_width].
// sizes[0 .. 7 + n_groups] receives the section sizes.  Returns the total, or -1 when cap is too small
// or a request holds more than table_width pages.
//
// n_pad more entries follow the real ones (a captured step is replayed with fewer requests than it was
// captured for): each feeds token 0 at position 0 of a request that does not exist, in state slot
// pad_slot, with a block table of a single page, and wants its logits (which nobody reads).  That page
// is, in every group, the one past the group's pool (id = the group's page count): the device arrays
// hold one page more than the bookkeeping hands out.
long long infero_step_layout(void* h, int n_entries, const int* slots, const int* n_tokens, const int* tokens,
                             const int* want_counts, const int* wants, int table_width, int* out, long long cap,
                             long long* sizes, int n_pad, int pad_slot) {
    Cache* c = static_cast<Cache*>(h);
    const int real = n_entries, E = n_entries + n_pad, G = (int)c->groups.size();
    long long T = n_pad, R = n_pad;
    for (int e = 0; e < real; ++e) { T += n_tokens[e]; R += want_counts[e]; }
    const long long total = 3 * T + 4LL * E + R + (long long)G * std::max(1, E) * table_width;
    if (total > cap) return -1;
    int* tok = out;
    int* pos = tok + T;
    int* ent = pos + T;
    int* q_start = ent + T;
    int* q_len = q_start + E;
    int* pos0 = q_len + E;
    int* slot_out = pos0 + E;
    int* rows = slot_out + E;
    int* tab = rows + R;
    long long t = 0, r = 0, w = 0;
    for (int e = real; e < E; ++e) {                     // the pads' rows come after the real ones'
        const long long tp = T - n_pad + (e - real);
        q_start[e] = (int)tp; q_len[e] = 1; pos0[e] = 0; slot_out[e] = pad_slot;
        rows[R - n_pad + (e - real)] = (int)tp;
        tok[tp] = 0; pos[tp] = 0; ent[tp] = e;
    }
    for (int e = 0; e < real; ++e) {
        const Request& rq = c->reqs[slots[e]];
        const int base = rq.length;                  // tokens already in the cache (this step's are only reserved)
        q_start[e] = (int)t;
        q_len[e] = n_tokens[e];
        pos0[e] = base;
        slot_out[e] = slots[e];
        for (int i = 0; i < want_counts[e]; ++i) rows[r++] = (int)t + wants[w++];
        for (int i = 0; i < n_tokens[e]; ++i, ++t) {
            int id = tokens[t];
            if (id < 0) id = -(slots[e] + 1);
            tok[t] = id;
            pos[t] = base + i;
            ent[t] = e;
        }
    }
    for (int g = 0; g < G; ++g) {
        int* dst = tab + (long long)g * std::max(1, E) * table_width;
        if (E == 0) std::fill(dst, dst + table_width, -1);
        for (int e = real; e < E; ++e) {
            std::fill(dst + (long long)e * table_width, dst + (long long)(e + 1) * table_width, -1);
            dst[(long long)e * table_width] = c->groups[g].num_pages;
        }
        for (int e = 0; e < real; ++e) {
            const Request& rq = c->reqs[slots[e]];
            if ((int)rq.tables[g].size() > table_width) return -1;
            const int* row = c->mirror[g].data() + (size_t)slots[e] * c->width;
            const int n = std::min(table_width, c->width);
            std::copy(row, row + n, dst + (long long)e * table_width);
            std::fill(dst + (long long)e * table_width + n, dst + (long long)(e + 1) * table_width, -1);
        }
    }
    sizes[0] = T; sizes[1] = T; sizes[2] = T;
    sizes[3] = E; sizes[4] = E; sizes[5] = E; sizes[6] = E;
    sizes[7] = R;
    for (int g = 0; g < G; ++g) sizes[8 + g] = (long long)std::max(1, E) * table_width;
    return total;
}

}  // extern "C"
