// The scheduler's decisions: which requests run in the next step, with how many tokens.
//
// LitInfer's engine has no admission control, no token budget and no portions: every unfinished request runs each
// step, a new one with its entire prompt (src/llaisys/models/qwen2.cpp:934-941), and when pages run out it throws in
// mid-step with some requests already advanced (qwen2.cpp:839-844).  Decided here instead:
//
//  * requests wait in FIFO order and are admitted while a state slot is free, fewer than max_num_seqs run, budget is
//    left and at least one of their tokens fits into free pages;
//  * a step spends at most max_tokens_per_step tokens: one for every running request that is decoding, then portions of
//    prompts (at most prefill_chunk tokens each, and no more than the free pages hold) for running requests in
//    admission order, then for newly admitted ones;
//  * when pages run out for a decoding request, the most recently admitted running request is preempted: its pages and
//    slot go back and it returns to the head of the waiting queue, to be recomputed later.  A portion of a prompt
//    preempts nobody; it shrinks or waits.  If nothing at all can run, the youngest is preempted so that the oldest can;
//  * finishing follows LitInfer (qwen2.cpp:1060-1066): an end-of-sequence token ends the request and is not part of its
//    output; otherwise it ends after exactly max_new_tokens tokens.  Pages go back at once.
//
// The scheduler knows requests by id and by their counts of tokens; the tokens themselves stay with the caller.  What
// it did to the caller's picture of the requests (admitted with which slot, preempted) comes back as a list of events.
#include <deque>

#include "runtime.h"

using namespace li_host;

namespace {

enum { kWaiting = 0, kRunning = 1, kFinished = 2 };
enum { kNone = 0, kEos = 1, kLength = 2, kMaxPositions = 3, kAborted = 4 };
enum { kEventAdmitted = 1, kEventPreempted = 2 };

struct SReq {
    int id = 0, prompt_len = 0, generated = 0, max_new = 0;
    int status = kWaiting, reason = kNone, preemptions = 0;
};

struct Event {
    int kind, id, arg;
};

struct Scheduler {
    Manager* m;
    int max_num_seqs, max_tokens_per_step, prefill_chunk, max_positions;
    std::unordered_set<int> eos;
    std::deque<int> waiting;
    std::vector<int> running;
    std::unordered_map<int, SReq> reqs;
    int num_preemptions = 0;
    std::vector<Event> events;

    SReq* find(int id) {
        auto it = reqs.find(id);
        return it == reqs.end() ? nullptr : &it->second;
    }
    int num_tokens(const SReq& r) const { return r.prompt_len + r.generated; }
    int num_cached(const SReq& r) const {
        Request* rc = m->find(r.id);
        return rc ? rc->length : 0;
    }
    void remove_running(int id) { running.erase(std::remove(running.begin(), running.end(), id), running.end()); }
    void give_back(SReq& r) {
        if (m->find(r.id)) cm_release(m, r.id);
    }
    void preempt(SReq& r) {
        remove_running(r.id);
        give_back(r);
        r.status = kWaiting;
        ++r.preemptions;
        ++num_preemptions;
        waiting.push_front(r.id);
        events.push_back({kEventPreempted, r.id, 0});
    }
    // how many of the next `want` tokens fit into the free pages of every group
    int fit(const SReq& r, int want) const {
        Request* rc = m->find(r.id);
        int most = want;
        for (size_t g = 0; g < m->pools.size(); ++g) {
            const int have = (int)rc->tables[g].size() * m->page_size - rc->length;
            most = std::min(most, have + m->pools[g].num_free() * m->page_size);
        }
        return most > 0 ? most : 0;
    }
};

struct Item {
    int id, start, count, wants;
};

int schedule(Scheduler* s, std::vector<Item>& items) {
    const int preempted_before = s->num_preemptions;
    for (;;) {
        int budget = s->max_tokens_per_step;
        items.clear();
        std::unordered_set<int> picked;
        // 1. decoding requests, oldest first; preempt the youngest when a page is missing
        const std::vector<int> snapshot = s->running;
        for (int id : snapshot) {
            SReq& r = *s->find(id);
            if (r.status != kRunning || budget <= 0) continue;
            const int cached = s->num_cached(r);
            if (s->num_tokens(r) - cached != 1) continue;
            for (;;) {
                const int rc = cm_extend(s->m, id, cached + 1);
                if (rc == LI_HOST_OK) break;
                if (rc != LI_HOST_OUT_OF_PAGES) return rc;
                SReq& victim = *s->find(s->running.back());
                s->preempt(victim);
                if (victim.id == id) break;
            }
            if (r.status != kRunning) continue;
            items.push_back({id, cached, 1, 1});
            picked.insert(id);
            --budget;
        }
        // 2. portions of the prompts of running requests
        for (int id : s->running) {
            if (budget <= 0) break;
            if (picked.count(id)) continue;
            SReq& r = *s->find(id);
            const int cached = s->num_cached(r), left = s->num_tokens(r) - cached;
            const int n = s->fit(r, std::min(left, std::min(s->prefill_chunk, budget)));
            if (n <= 0) continue;
            if (int rc = cm_extend(s->m, id, cached + n)) return rc;
            items.push_back({id, cached, n, n == left ? 1 : 0});
            picked.insert(id);
            budget -= n;
        }
        // 3. admit waiting requests, in order
        while (!s->waiting.empty() && budget > 0 && (int)s->running.size() < s->max_num_seqs && s->m->slots.num_free() > 0) {
            if (s->num_preemptions != preempted_before) break;        // a request was just preempted for lack of pages: admit nobody this step
            SReq& r = *s->find(s->waiting.front());
            int slot = 0;
            if (int rc = cm_admit(s->m, r.id, &slot)) return rc;
            const int n = s->fit(r, std::min(s->num_tokens(r), std::min(s->prefill_chunk, budget)));
            if (n <= 0) {
                s->give_back(r);
                break;
            }
            s->waiting.pop_front();
            r.status = kRunning;
            s->running.push_back(r.id);
            s->events.push_back({kEventAdmitted, r.id, slot});
            if (int rc = cm_extend(s->m, r.id, n)) return rc;
            items.push_back({r.id, 0, n, n == s->num_tokens(r) ? 1 : 0});
            picked.insert(r.id);
            budget -= n;
        }
        if (!items.empty() || s->running.empty()) return LI_HOST_OK;
        // nothing can run although requests are live: free the youngest one's pages
        s->preempt(*s->find(s->running.back()));
    }
}

}  // namespace

LI_HOST_EXPORT void* li_sched_create(void* manager, int max_num_seqs, int max_tokens_per_step, int prefill_chunk, int max_positions) {
    if (!manager || max_num_seqs <= 0 || max_tokens_per_step <= 0 || prefill_chunk <= 0) return nullptr;
    Scheduler* s = new Scheduler();
    s->m = static_cast<Manager*>(manager);
    s->max_num_seqs = max_num_seqs;
    s->max_tokens_per_step = max_tokens_per_step;
    s->prefill_chunk = prefill_chunk;
    s->max_positions = max_positions;
    return s;
}
LI_HOST_EXPORT void li_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

LI_HOST_EXPORT int li_sched_set_eos(void* h, const int* ids, int n) {
    Scheduler* s = static_cast<Scheduler*>(h);
    s->eos.clear();
    for (int i = 0; i < n; ++i) s->eos.insert(ids[i]);
    return LI_HOST_OK;
}

// a new request at the end of the waiting queue (its sizes were checked by the caller)
LI_HOST_EXPORT int li_sched_add(void* h, int id, int prompt_len, int max_new_tokens) {
    Scheduler* s = static_cast<Scheduler*>(h);
    if (s->find(id)) return fail(LI_HOST_VALUE, "request %d exists already", id);
    if (prompt_len <= 0 || max_new_tokens <= 0) return fail(LI_HOST_VALUE, "request %d: bad sizes", id);
    SReq r;
    r.id = id;
    r.prompt_len = prompt_len;
    r.max_new = max_new_tokens;
    s->reqs.emplace(id, r);
    s->waiting.push_back(id);
    return LI_HOST_OK;
}

LI_HOST_EXPORT int li_sched_counts(void* h, int* waiting, int* running, int* preemptions) {
    Scheduler* s = static_cast<Scheduler*>(h);
    *waiting = (int)s->waiting.size();
    *running = (int)s->running.size();
    *preemptions = s->num_preemptions;
    return LI_HOST_OK;
}

// Picks the next step's items and allocates their pages.  items: up to item_cap rows of (id, start, count, wants logits);
// events: up to event_cap rows of (kind, id, arg) in the order they happened: 1 admitted (arg: its state slot),
// 2 preempted.
LI_HOST_EXPORT int li_sched_schedule(void* h, int* items, int item_cap, int* n_items, int* events, int event_cap, int* n_events) {
    Scheduler* s = static_cast<Scheduler*>(h);
    s->events.clear();
    std::vector<Item> picked;
    const int rc = schedule(s, picked);
    *n_events = (int)s->events.size();
    if (*n_events > event_cap) return fail(LI_HOST_RUNTIME, "%d scheduler events do not fit %d", *n_events, event_cap);
    for (int i = 0; i < *n_events; ++i) {
        events[3 * i] = s->events[(size_t)i].kind;
        events[3 * i + 1] = s->events[(size_t)i].id;
        events[3 * i + 2] = s->events[(size_t)i].arg;
    }
    if (rc) return rc;
    *n_items = (int)picked.size();
    if (*n_items > item_cap) return fail(LI_HOST_RUNTIME, "%d scheduled items do not fit %d", *n_items, item_cap);
    for (int i = 0; i < *n_items; ++i) {
        items[4 * i] = picked[(size_t)i].id;
        items[4 * i + 1] = picked[(size_t)i].start;
        items[4 * i + 2] = picked[(size_t)i].count;
        items[4 * i + 3] = picked[(size_t)i].wants;
    }
    return LI_HOST_OK;
}

// After the step: tokens[i] was drawn for request ids[i].  outcome[i]: 1 the token is part of the output, 0 it is the
// dropped end-of-sequence token; reason[i]: 0 the request goes on, else why it ended (1 eos, 2 length, 3 positions).
// A request that ends gives its pages and slot back here.
LI_HOST_EXPORT int li_sched_update(void* h, int n, const int* ids, const int* tokens, int* outcome, int* reason) {
    Scheduler* s = static_cast<Scheduler*>(h);
    for (int i = 0; i < n; ++i) {
        SReq* r = s->find(ids[i]);
        if (!r || r->status != kRunning) return fail(LI_HOST_VALUE, "request %d is not running", ids[i]);
        if (s->eos.count(tokens[i])) {
            outcome[i] = 0;
            r->reason = kEos;                                      // the token is dropped (qwen2.cpp:1060-1062)
        } else {
            outcome[i] = 1;
            ++r->generated;
            if (r->generated >= r->max_new) r->reason = kLength;
            else if (s->num_tokens(*r) > s->max_positions) r->reason = kMaxPositions;
        }
        reason[i] = r->reason;
        if (r->reason != kNone) {
            s->remove_running(r->id);
            s->give_back(*r);
            r->status = kFinished;
        }
    }
    return LI_HOST_OK;
}

// was_running: whether the request held pages and a slot (given back here)
LI_HOST_EXPORT int li_sched_abort(void* h, int id, int* was_running) {
    Scheduler* s = static_cast<Scheduler*>(h);
    SReq* r = s->find(id);
    if (!r) return fail(LI_HOST_VALUE, "request %d is not known", id);
    *was_running = 0;
    if (r->status == kFinished) return LI_HOST_OK;
    if (r->status == kRunning) {
        *was_running = 1;
        s->remove_running(id);
        s->give_back(*r);
    } else {
        s->waiting.erase(std::remove(s->waiting.begin(), s->waiting.end(), id), s->waiting.end());
    }
    r->status = kFinished;
    r->reason = kAborted;
    return LI_HOST_OK;
}

LI_HOST_EXPORT int li_sched_forget(void* h, int id) {
    Scheduler* s = static_cast<Scheduler*>(h);
    SReq* r = s->find(id);
    if (!r) return fail(LI_HOST_VALUE, "request %d is not known", id);
    if (r->status != kFinished) return fail(LI_HOST_VALUE, "request %d is not finished", id);
    s->reqs.erase(id);
    return LI_HOST_OK;
}
