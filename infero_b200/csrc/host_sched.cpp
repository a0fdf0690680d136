// The scheduler's decisions (host only, no CUDA): who is admitted, what a step runs, who is
// preempted when pages run out, when a request ends, and whether the next step may be launched
// before this one's tokens are known.  It keeps counters only; token ids, samplers and outputs
// stay with the caller, which identifies requests by the integer this code hands out.
//
// The rules follow the reference's scheduler (crates/server/src/scheduler.rs): FIFO admission
// while a request's tokens plus one fit the free cache and a sequence row is free, the head of
// the queue staying in front otherwise (:1854-1957); decodes first (:2076-2098); prompt portions
// under the token budget, several prompts may share a step (:2105-2127); a request ends on an
// end-of-sequence token (not appended, :2151-2153), on its generation budget or when the context
// is full (:2170-2178).  The reference never preempts (:1042-1055); here the youngest running
// request is preempted by recompute when a step can move nothing.
#include <algorithm>
#include <cstdint>
#include <deque>
#include <vector>

extern "C" {
// host_cache.cpp
int infero_cache_open(void* h);
int infero_cache_close(void* h, int slot);
int infero_cache_length(void* h, int slot);
int infero_cache_reserved(void* h, int slot);
int infero_cache_num_free(void* h, int group);
int infero_cache_table_len(void* h, int group, int slot);
void infero_cache_pages_needed(void* h, int slot, int n_new, int* out);
void infero_cache_geometry(void* h, int* out);
int infero_cache_group_pages(void* h, int group);
int infero_cache_held_by(void* h, int group, int slot);
int infero_cache_most_pages(void* h, int group, int n_tokens, int max_chunk);
}

namespace {

struct Req {
    bool used = false, finished = false, has_pending = false, needs_host_token = false;
    int prompt_len = 0, n_tokens = 0, fed = 0, n_generated = 0, max_new = 0, slot = -1, preemptions = 0;
    long long admitted_at = 0;
};

struct Sched {
    void* cache;
    int max_seqs, max_batch_tokens, ctx, max_prefill_chunk;
    int n_groups, page_size;
    std::vector<Req> reqs;
    std::vector<int> free_ids;
    std::deque<int> waiting;
    std::vector<int> running;
    long long clock = 0;
    long long stats[6] = {0, 0, 0, 0, 0, 0};     // preemptions, decode tokens, prefill tokens, rejected, finished, dropped
    std::vector<int> need, used;

    int pages_for(int n_tokens) const { return (n_tokens + page_size - 1) / page_size; }
    int free_pages(int g) const { return infero_cache_num_free(cache, g); }
    // Pages of group g a request of n tokens has to hold at once, at least: all of them where every key
    // is kept; where a window is kept, what a token-by-token feed holds (larger portions hold more for
    // a step, and the planner cuts portions to the pages that are free).
    int least_need(int g, int n_tokens) const { return infero_cache_most_pages(cache, g, n_tokens, 1); }
    // pages of group g the running requests still have to take to hold their tokens plus one
    int outstanding(int g) const {
        int total = 0;
        for (int id : running) {
            const Req& r = reqs[id];
            total += std::max(0, least_need(g, r.n_tokens + 1) - infero_cache_held_by(cache, g, r.slot));
        }
        return total;
    }
    void drop_running(int id) {
        auto it = std::find(running.begin(), running.end(), id);
        if (it != running.end()) running.erase(it);
    }
    void finish(int id) {
        Req& r = reqs[id];
        if (r.finished) return;
        r.finished = true;
        drop_running(id);
        if (r.slot >= 0) {
            infero_cache_close(cache, r.slot);
            r.slot = -1;
        }
        ++stats[4];
    }
};

}  // namespace

extern "C" {

void* infero_sched_new(void* cache, int max_seqs, int max_batch_tokens, int ctx, int max_prefill_chunk) {
    if (!cache || max_seqs <= 0 || max_batch_tokens <= 0 || ctx <= 0) return nullptr;
    Sched* s = new Sched();
    s->cache = cache;
    s->max_seqs = max_seqs;
    s->max_batch_tokens = max_batch_tokens;
    s->ctx = ctx;
    s->max_prefill_chunk = max_prefill_chunk;
    int geo[4];
    infero_cache_geometry(cache, geo);
    s->n_groups = geo[0];
    s->page_size = geo[2];
    s->need.assign(std::max(1, s->n_groups), 0);
    s->used.assign(std::max(1, s->n_groups), 0);
    return s;
}

void infero_sched_delete(void* h) { delete static_cast<Sched*>(h); }

// A new request at the back of the queue.  Returns its id, -1 for an empty prompt, -2 for a prompt
// that leaves no room for one generated token in the context.
int infero_sched_enqueue(void* h, int prompt_len, int max_new, int needs_host_token) {
    Sched* s = static_cast<Sched*>(h);
    if (prompt_len <= 0) { ++s->stats[3]; return -1; }
    if (prompt_len + 1 > s->ctx) { ++s->stats[3]; return -2; }
    int id;
    if (!s->free_ids.empty()) {
        id = s->free_ids.back();
        s->free_ids.pop_back();
    } else {
        id = (int)s->reqs.size();
        s->reqs.emplace_back();
    }
    Req& r = s->reqs[id];
    r = Req();
    r.used = true;
    r.prompt_len = r.n_tokens = prompt_len;
    r.max_new = max_new;
    r.needs_host_token = needs_host_token != 0;
    s->waiting.push_back(id);
    return id;
}

// The caller has read everything it wants of a finished request: its id may be given out again.
void infero_sched_release(void* h, int id) {
    Sched* s = static_cast<Sched*>(h);
    if (id < 0 || id >= (int)s->reqs.size() || !s->reqs[id].used) return;
    s->reqs[id].used = false;
    s->free_ids.push_back(id);
}

// Admit from the front of the queue.  out receives triples (id, code, value): code 0 = admitted, value
// is its cache slot; code 1 = a new request that can never fit the pool, code 2 = a preempted one that
// no longer can (both finished here; value is the pages it would need).  Returns the number of triples.
int infero_sched_admit(void* h, int* out, int cap) {
    Sched* s = static_cast<Sched*>(h);
    int n = 0;
    while (!s->waiting.empty() && (int)s->running.size() < s->max_seqs && n < cap) {
        const int id = s->waiting.front();
        Req& r = s->reqs[id];
        // every group has a pool of its own: the request must fit each, and each must have the room now
        int need = 0;
        bool never = false, not_now = false;
        for (int g = 0; g < s->n_groups; ++g) {
            const int need_g = s->least_need(g, r.n_tokens + 1);
            if (need_g > infero_cache_group_pages(s->cache, g)) { never = true; need = std::max(need, need_g); }
            else if (need_g > s->free_pages(g) - s->outstanding(g)) not_now = true;
        }
        if (never) {
            s->waiting.pop_front();
            const bool resumed = r.preemptions > 0;
            r.finished = true;
            ++s->stats[3];
            out[3 * n] = id; out[3 * n + 1] = resumed ? 2 : 1; out[3 * n + 2] = need;
            ++n;
            continue;
        }
        if (not_now) break;                                      // stays at the front; tried again next step
        const int slot = infero_cache_open(s->cache);
        if (slot < 0) break;
        s->waiting.pop_front();
        r.slot = slot;
        r.admitted_at = s->clock++;
        s->running.push_back(id);
        out[3 * n] = id; out[3 * n + 1] = 0; out[3 * n + 2] = slot;
        ++n;
    }
    return n;
}

// What the next step runs.  out receives (id, first token, count, samples, is_decode) per item: a decode
// item feeds the pending token (first token = -1); a prompt portion feeds tokens[first .. first + count).
int infero_sched_plan(void* h, int* out, int cap) {
    Sched* s = static_cast<Sched*>(h);
    int budget = s->max_batch_tokens, n = 0;
    const int G = s->n_groups, P = s->page_size;
    std::fill(s->used.begin(), s->used.end(), 0);
    auto left = [&](int g) { return s->free_pages(g) - s->used[g]; };
    // decodes first
    for (int id : s->running) {
        const Req& r = s->reqs[id];
        if (!r.has_pending || r.fed < r.n_tokens || budget <= 0 || n >= cap) continue;
        infero_cache_pages_needed(s->cache, r.slot, 1, s->need.data());
        bool fits = true;
        for (int g = 0; g < G; ++g) fits = fits && s->need[g] <= left(g);
        if (!fits) continue;
        for (int g = 0; g < G; ++g) s->used[g] += s->need[g];
        int* o = out + 5 * n++;
        o[0] = id; o[1] = -1; o[2] = 1; o[3] = 1; o[4] = 1;
        --budget;
    }
    // then prompt portions, in running order
    for (int id : s->running) {
        if (budget <= 0 || n >= cap) break;
        const Req& r = s->reqs[id];
        const int remaining = r.n_tokens - r.fed;
        if (remaining <= 0) continue;
        const int filled = infero_cache_length(s->cache, r.slot) + infero_cache_reserved(s->cache, r.slot);
        const int slack = (P - filled % P) % P;                    // free rows in its last page
        int min_left = G ? left(0) : 0;
        for (int g = 1; g < G; ++g) min_left = std::min(min_left, left(g));
        const long long room = slack + (long long)std::max(0, min_left) * P;
        long long cnt = std::min<long long>(std::min(remaining, budget), room);
        if (s->max_prefill_chunk > 0) cnt = std::min<long long>(cnt, s->max_prefill_chunk);
        if (cnt <= 0) continue;
        infero_cache_pages_needed(s->cache, r.slot, (int)cnt, s->need.data());
        for (int g = 0; g < G; ++g) s->used[g] += s->need[g];
        int* o = out + 5 * n++;
        o[0] = id; o[1] = r.fed; o[2] = (int)cnt; o[3] = cnt == remaining ? 1 : 0; o[4] = 0;
        budget -= (int)cnt;
    }
    return n;
}

// Free the youngest running request and put it back at the front of the queue: what it generated
// so far becomes part of the tokens it recomputes.  Returns its id, or -1 when at most one runs.
int infero_sched_preempt_youngest(void* h) {
    Sched* s = static_cast<Sched*>(h);
    if (s->running.size() <= 1) return -1;
    int victim = s->running[0];
    for (int id : s->running)
        if (s->reqs[id].admitted_at > s->reqs[victim].admitted_at) victim = id;
    s->drop_running(victim);
    Req& r = s->reqs[victim];
    infero_cache_close(s->cache, r.slot);
    r.slot = -1;
    r.n_tokens = r.prompt_len + r.n_generated;
    r.has_pending = false;            // the pending token is the last generated one: fed with the recompute
    r.fed = 0;
    ++r.preemptions;
    ++s->stats[0];
    s->waiting.push_front(victim);
    return victim;
}

// May a step that decodes one more token for exactly these requests (the items of the step in
// flight, each with its `samples` flag) be launched before that step's tokens are known?
int infero_sched_can_run_ahead(void* h, int n_items, const int* ids, const int* samples) {
    Sched* s = static_cast<Sched*>(h);
    if (!s->waiting.empty() || n_items != (int)s->running.size() || n_items > s->max_batch_tokens) return 0;
    std::fill(s->used.begin(), s->used.end(), 0);
    for (int i = 0; i < n_items; ++i) {
        const Req& r = s->reqs[ids[i]];
        if (!samples[i] || r.finished) return 0;                       // a prompt is still being fed
        if (r.needs_host_token) return 0;                              // e.g. a repetition penalty
        if (r.n_generated + 2 > r.max_new || r.prompt_len + r.n_generated + 2 > s->ctx) return 0;   // ends now or next
        infero_cache_pages_needed(s->cache, r.slot, 1, s->need.data());
        for (int g = 0; g < s->n_groups; ++g) s->used[g] += s->need[g];
    }
    for (int g = 0; g < s->n_groups; ++g)
        if (s->used[g] > s->free_pages(g)) return 0;
    return 1;
}

// One item of a completed step.  Returns 0: a prompt portion without a sample; 1: a token was generated
// and the request goes on; 2: it ended on an end-of-sequence token (not kept); 3: it ended on its
// generation budget (token kept); 4: it ended because the context is full (token kept); 5: it had
// ended a step earlier and this item ran a token too far (dropped).
int infero_sched_complete(void* h, int id, int count, int is_decode, int samples, int is_eos) {
    Sched* s = static_cast<Sched*>(h);
    Req& r = s->reqs[id];
    if (r.finished) { ++s->stats[5]; return 5; }
    if (is_decode) {
        r.has_pending = false;
        r.n_tokens += 1;
        r.fed += 1;
        ++s->stats[1];
    } else {
        r.fed += count;
        s->stats[2] += count;
    }
    if (!samples) return 0;
    if (is_eos) { s->finish(id); return 2; }
    ++r.n_generated;
    if (r.n_generated >= r.max_new) { s->finish(id); return 3; }
    if (r.prompt_len + r.n_generated >= s->ctx) { s->finish(id); return 4; }
    r.has_pending = true;
    return 1;
}

// End a request from outside (the cache is exhausted for it, or the engine gives up).
void infero_sched_finish(void* h, int id) { static_cast<Sched*>(h)->finish(id); }

// Take a waiting request out of the queue (the engine gives up); returns -1 when none waits.
int infero_sched_pop_waiting(void* h) {
    Sched* s = static_cast<Sched*>(h);
    if (s->waiting.empty()) return -1;
    const int id = s->waiting.front();
    s->waiting.pop_front();
    s->reqs[id].finished = true;
    return id;
}

int infero_sched_num_waiting(void* h) { return (int)static_cast<Sched*>(h)->waiting.size(); }
int infero_sched_num_running(void* h) { return (int)static_cast<Sched*>(h)->running.size(); }
int infero_sched_running(void* h, int* out, int cap) {
    Sched* s = static_cast<Sched*>(h);
    int n = 0;
    for (int id : s->running)
        if (n < cap) out[n++] = id;
    return n;
}
int infero_sched_waiting(void* h, int* out, int cap) {
    Sched* s = static_cast<Sched*>(h);
    int n = 0;
    for (int id : s->waiting)
        if (n < cap) out[n++] = id;
    return n;
}
long long infero_sched_stat(void* h, int which) {
    Sched* s = static_cast<Sched*>(h);
    return which >= 0 && which < 6 ? s->stats[which] : -1;
}
int infero_sched_slot(void* h, int id) { return static_cast<Sched*>(h)->reqs[id].slot; }
int infero_sched_preemptions(void* h, int id) { return static_cast<Sched*>(h)->reqs[id].preemptions; }

}  // extern "C"
