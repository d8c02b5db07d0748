// The host side of the engine's memory: pools of pages and slots, the block tables of the live requests, and the
// packer that turns a step's items into the one int32 buffer the kernels read.  Plain C++17 behind a C interface
// (no CUDA, no Python): it is compiled with g++ into a library of its own, so that it also runs where there is no GPU.
//
// LitInfer keeps the same bookkeeping in C++, per layer: a free list and a block table for every layer
// (src/llaisys/kv_cache/block_kv_cache.hpp:34-81) and a block table rebuilt and uploaded per layer and step
// (src/llaisys/models/qwen2.cpp:993-1007).  Here a group of layers with equal needs shares one page-id space, a page
// cannot be freed twice or by a request that does not hold it, and a step's metadata is packed once.
//
// Every function returns 0 or an error class (LI_HOST_* below) and leaves the message for li_host_last_error().
#include "runtime.h"

namespace li_host {

static thread_local char g_error[512] = "";

char* error_text() { return g_error; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace li_host

using namespace li_host;

LI_HOST_EXPORT const char* li_host_last_error() { return error_text(); }

// ---- a pool by itself ---------------------------------------------------------------------------------------------

LI_HOST_EXPORT void* li_pool_create(int pages, const char* what) { return pages > 0 ? new Pool(pages, what ? what : "page") : nullptr; }
LI_HOST_EXPORT void li_pool_destroy(void* p) { delete static_cast<Pool*>(p); }
LI_HOST_EXPORT int li_pool_alloc(void* p, int owner, int* page) { return static_cast<Pool*>(p)->alloc(owner, page); }
LI_HOST_EXPORT int li_pool_free(void* p, int page, int owner) { return static_cast<Pool*>(p)->release(page, owner); }
LI_HOST_EXPORT int li_pool_num_free(void* p) { return static_cast<Pool*>(p)->num_free(); }
LI_HOST_EXPORT int li_pool_owner(void* p, int page) {
    Pool* pool = static_cast<Pool*>(p);
    return page >= 0 && page < pool->n ? pool->owner[(size_t)page] : -2;
}
LI_HOST_EXPORT int li_pool_check(void* p) { return static_cast<Pool*>(p)->check(); }

// ---- the manager ----------------------------------------------------------------------------------------------------

// windows[g] <= 0: the group keeps every key
LI_HOST_EXPORT void* li_cm_create(int groups, const int* windows, int num_pages, int page_size, int max_requests) {
    if (groups < 0 || num_pages <= 0 || max_requests <= 0 || page_size < 1) return nullptr;
    return new Manager(groups, windows, num_pages, page_size, max_requests);
}
LI_HOST_EXPORT void li_cm_destroy(void* h) { delete static_cast<Manager*>(h); }

// which: -1 the state slots, else a group's pages
static Pool* pool_of(Manager* m, int which) {
    if (which < 0) return &m->slots;
    return which < (int)m->pools.size() ? &m->pools[(size_t)which] : nullptr;
}
LI_HOST_EXPORT int li_cm_num_free(void* h, int which) {
    Pool* p = pool_of(static_cast<Manager*>(h), which);
    return p ? p->num_free() : -1;
}
LI_HOST_EXPORT int li_cm_owner(void* h, int which, int page) {
    Pool* p = pool_of(static_cast<Manager*>(h), which);
    return p && page >= 0 && page < p->n ? p->owner[(size_t)page] : -2;
}
LI_HOST_EXPORT int li_cm_pool_check(void* h, int which) {
    Pool* p = pool_of(static_cast<Manager*>(h), which);
    return p ? p->check() : fail(LI_HOST_POOL, "no pool %d", which);
}

int li_host::cm_admit(Manager* m, int id, int* slot) {
    if (m->find(id)) return fail(LI_HOST_POOL, "request %d is already admitted", id);
    if (int rc = m->slots.alloc(id, slot)) return rc;
    Request r;
    r.id = id;
    r.slot = *slot;
    r.tables.resize(m->pools.size());
    r.sent.assign(m->pools.size(), 0);
    r.trash_sent.assign(m->pools.size(), 0);
    m->live.emplace(id, std::move(r));
    return LI_HOST_OK;
}

// pages each group lacks for positions up to new_length
LI_HOST_EXPORT int li_cm_pages_needed(void* h, int id, int new_length, int* need) {
    Manager* m = static_cast<Manager*>(h);
    FIND(m, r, id);
    const int want = m->blocks(new_length);
    for (size_t g = 0; g < m->pools.size(); ++g) {
        const int have = (int)r->tables[g].size();
        need[g] = want > have ? want - have : 0;
    }
    return LI_HOST_OK;
}

// pages for positions up to new_length in every group; all or nothing
int li_host::cm_extend(Manager* m, int id, int new_length) {
    FIND(m, r, id);
    const int want = m->blocks(new_length);
    for (size_t g = 0; g < m->pools.size(); ++g) {
        const int n = want - (int)r->tables[g].size();
        if (n > m->pools[g].num_free())
            return fail(LI_HOST_OUT_OF_PAGES, "request %d needs %d pages, %d are free", id, n, m->pools[g].num_free());
    }
    for (size_t g = 0; g < m->pools.size(); ++g)
        while ((int)r->tables[g].size() < want) {
            int page = 0;
            if (int rc = m->pools[g].alloc(id, &page)) return rc;
            r->tables[g].push_back(page);
        }
    return LI_HOST_OK;
}

// the step has written positions below new_length: pages of windowed groups that no further query can read go back
LI_HOST_EXPORT int li_cm_commit(void* h, int id, int new_length) {
    Manager* m = static_cast<Manager*>(h);
    FIND(m, r, id);
    if (new_length < r->length) return fail(LI_HOST_POOL, "a request's length never shrinks");
    r->length = new_length;
    for (size_t g = 0; g < m->pools.size(); ++g) {
        if (m->windows[g] <= 0) continue;
        std::vector<int>& t = r->tables[g];
        const int upto = std::min(m->first_needed_page((int)g, new_length), (int)t.size());
        for (int lp = 0; lp < upto; ++lp)
            if (t[(size_t)lp] != kReleased) {
                if (int rc = m->pools[g].release(t[(size_t)lp], id)) return rc;
                t[(size_t)lp] = kReleased;
            }
    }
    return LI_HOST_OK;
}

// li_cm_commit for the requests of a step at once
LI_HOST_EXPORT int li_cm_commit_many(void* h, int n, const int* ids, const int* new_lengths) {
    for (int i = 0; i < n; ++i)
        if (int rc = li_cm_commit(h, ids[i], new_lengths[i])) return rc;
    return LI_HOST_OK;
}

int li_host::cm_release(Manager* m, int id) {
    FIND(m, r, id);
    for (size_t g = 0; g < m->pools.size(); ++g) {
        // last page first, so that a request admitted next gets them in ascending order
        std::vector<int>& t = r->tables[g];
        for (size_t i = t.size(); i-- > 0;)
            if (t[i] != kReleased)
                if (int rc = m->pools[g].release(t[i], id)) return rc;
        t.clear();
    }
    if (int rc = m->slots.release(r->slot, id)) return rc;
    m->live.erase(id);
    return LI_HOST_OK;
}

LI_HOST_EXPORT int li_cm_admit(void* h, int id, int* slot) { return cm_admit(static_cast<Manager*>(h), id, slot); }
LI_HOST_EXPORT int li_cm_extend(void* h, int id, int new_length) { return cm_extend(static_cast<Manager*>(h), id, new_length); }
LI_HOST_EXPORT int li_cm_release(void* h, int id) { return cm_release(static_cast<Manager*>(h), id); }

LI_HOST_EXPORT int li_cm_length(void* h, int id) {
    Request* r = static_cast<Manager*>(h)->find(id);
    return r ? r->length : -1;
}

// a request's block table of one group: its length, and up to cap entries into out
LI_HOST_EXPORT int li_cm_table(void* h, int id, int group, int* out, int cap) {
    Manager* m = static_cast<Manager*>(h);
    Request* r = m->find(id);
    if (!r || group < 0 || group >= (int)m->pools.size()) return -1;
    const std::vector<int>& t = r->tables[(size_t)group];
    const int n = (int)t.size();
    if (out && cap > 0) std::memcpy(out, t.data(), sizeof(int) * (size_t)std::min(n, cap));
    return n;
}

// no page lost, held twice, or held by a request that is not live
LI_HOST_EXPORT int li_cm_check(void* h) {
    Manager* m = static_cast<Manager*>(h);
    if (int rc = m->slots.check()) return rc;
    for (size_t g = 0; g < m->pools.size(); ++g) {
        if (int rc = m->pools[g].check()) return rc;
        std::unordered_map<int, int> held;
        for (const auto& kv : m->live)
            for (int p : kv.second.tables[g]) {
                if (p == kReleased) continue;
                auto it = held.find(p);
                if (it != held.end()) return fail(LI_HOST_POOL, "page %d of group %d is held by requests %d and %d", p, (int)g, it->second, kv.first);
                held.emplace(p, kv.first);
                if (m->pools[g].owner[(size_t)p] != kv.first)
                    return fail(LI_HOST_POOL, "page %d of group %d: table of %d, pool says %d", p, (int)g, kv.first, m->pools[g].owner[(size_t)p]);
            }
        const int used = m->num_pages - m->pools[g].num_free();
        if ((int)held.size() != used) return fail(LI_HOST_POOL, "group %d: %d pages in use, %d in block tables", (int)g, used, (int)held.size());
    }
    return LI_HOST_OK;
}

// ---- the packer -----------------------------------------------------------------------------------------------------
//
// Fills the packed int32 buffer of a step (engine/batch.py describes the layout; `offsets` gives where each field
// starts: token_ids, positions, seq_of_token, q_start, ctx_lens, old_lens, state_slots, logit_rows, then per group
// slot_mapping and block_table).  Items: request ids, token counts, tokens and wanted places, flattened.
// starts[i] / olds[i] (or -1: the request's cached length): the position of the item's first token, and how many of the
// request's keys were cached before the step; they differ from the cached length when a portion is given as single
// tokens.  The batch is padded to S sequences, T tokens and R rows (their meaning as in batch.py: with pad_tokens the
// padding sequences are empty but the last, else they hold one token each and want its row).  The buffer must be
// zeroed and sized by the caller; T, S, R and the width of the block tables are the caller's too, checked here.
//
// Resident tables (update_cap >= 0): the device keeps a copy of every request's tables, a row per state slot, and the
// step's sequences name their row by state_slots.  The field that would hold a group's block tables then holds what
// that copy lacks for the step's requests: a count, then triples (slot, logical page, page id; the sink page for a page
// that was given back), at most update_cap of them (li_cm_table_updates_bound says how many it can be).  What is written
// counts as sent: the caller uploads the buffer and applies it (kernels.table_gather) before anything else is packed.
LI_HOST_EXPORT int li_cm_table_updates_bound(void* h, int n_items, const int* request_ids, const int* q_lens, const int* starts, int* bound) {
    Manager* m = static_cast<Manager*>(h);
    const int G = (int)m->pools.size();
    long long most = 0;
    for (int g = 0; g < G; ++g) {
        long long n = 0;
        for (int s = 0; s < n_items; ++s) {
            FIND(m, r, request_ids[s]);
            const int start = starts && starts[s] >= 0 ? starts[s] : r->length;
            const int nb = m->blocks(start + q_lens[s]);
            n += std::max(0, nb - std::min(r->sent[(size_t)g], nb));
            n += std::max(0, std::min(m->first_needed_page(g, r->length), nb) - r->trash_sent[(size_t)g]);
        }
        most = std::max(most, n);
    }
    *bound = (int)std::min<long long>(most, 1 << 30);
    return LI_HOST_OK;
}

LI_HOST_EXPORT int li_cm_pack_step(void* h, int n_items, const int* request_ids, const int* q_lens, const int* starts, const int* olds,
                                   const int* tokens, const int* want_counts, const int* wants, int vocab, int S, int T, int R,
                                   int pad_tokens, int max_blocks, int allow_repeat, int trash_page, int trash_slot, const int* offsets,
                                   int* buf, long long buf_len, int* info /* R_real, max_q_len, max_ctx_len, singles */, int update_cap) {
    Manager* m = static_cast<Manager*>(h);
    const int G = (int)m->pools.size(), page = m->page_size;
    if (n_items <= 0) return fail(LI_HOST_VALUE, "a step needs at least one item");
    if (S < n_items) return fail(LI_HOST_VALUE, "%d items do not fit %d sequences", n_items, S);
    long long t_real = 0, r_real = 0;
    for (int i = 0; i < n_items; ++i) {
        if (q_lens[i] <= 0) return fail(LI_HOST_VALUE, "an item without tokens");
        t_real += q_lens[i];
        r_real += want_counts[i];
    }
    const int pad_seq = S - n_items;
    long long t_pad = 0;                                // tokens of the padding sequences
    if (pad_tokens) {
        t_pad = (long long)T - t_real;
        if (t_pad < 0 || (t_pad > 0 && pad_seq == 0))
            return fail(LI_HOST_VALUE, "%lld tokens in %d sequences cannot be padded to %d tokens in %d", t_real, n_items, T, S);
        if (r_real > R) return fail(LI_HOST_VALUE, "%lld wanted rows do not fit the %d of the padded step", r_real, R);
    } else {
        t_pad = pad_seq;
        if (t_real + t_pad != T || r_real + pad_seq != R) return fail(LI_HOST_VALUE, "the step's sizes do not match its items");
    }
    const bool resident = update_cap >= 0;
    // the fields must fit the buffer
    const int n_fields = 8 + 2 * G;
    const long long sizes[8] = {T, T, T, (long long)S + 1, S, S, S, R};
    for (int f = 0; f < n_fields; ++f) {
        const long long len = f < 8 ? sizes[f] : ((f - 8) % 2 == 0 ? (long long)T : (resident ? 1 + 3LL * update_cap : (long long)S * max_blocks));
        if (offsets[f] < 0 || offsets[f] + len > buf_len) return fail(LI_HOST_VALUE, "field %d does not fit the step's buffer", f);
    }
    int* token_ids = buf + offsets[0];
    int* positions = buf + offsets[1];
    int* seq_of = buf + offsets[2];
    int* q_start = buf + offsets[3];
    int* ctx_lens = buf + offsets[4];
    int* old_lens = buf + offsets[5];
    int* state_slots = buf + offsets[6];
    int* logit_rows = buf + offsets[7];

    std::unordered_set<int> seen;
    int tok = 0, row = 0, max_q = 0, max_ctx = 0, singles = 0, tok_in = 0, want_in = 0;
    q_start[0] = 0;
    for (int s = 0; s < n_items; ++s) {
        const int id = request_ids[s], n = q_lens[s];
        FIND(m, r, id);
        if (!seen.insert(id).second && !allow_repeat) return fail(LI_HOST_VALUE, "request %d appears twice in one step", id);
        const int start = starts && starts[s] >= 0 ? starts[s] : r->length;
        const int old = olds && olds[s] >= 0 ? olds[s] : r->length;
        for (int j = 0; j < n; ++j) {
            const int t = tokens[tok_in + j];
            if (t < 0 || t >= vocab) return fail(LI_HOST_INDEX, "request %d: token id outside [0, %d)", id, vocab);
            token_ids[tok + j] = t;
            positions[tok + j] = start + j;
            seq_of[tok + j] = s;
        }
        for (int w = 0; w < want_counts[s]; ++w) {
            const int place = wants[want_in + w];
            if (place < 0 || place >= n) return fail(LI_HOST_INDEX, "request %d: wanted place %d is outside its %d tokens", id, place, n);
            logit_rows[row++] = tok + place;
        }
        const int ctx = start + n;
        ctx_lens[s] = ctx;
        old_lens[s] = old;
        state_slots[s] = r->slot;
        const int nb = m->blocks(ctx);
        if (nb > max_blocks) return fail(LI_HOST_VALUE, "request %d: %d pages do not fit block tables of %d", id, nb, max_blocks);
        for (int g = 0; g < G; ++g) {
            const std::vector<int>& table = r->tables[(size_t)g];
            if ((int)table.size() < nb)
                return fail(LI_HOST_RUNTIME, "request %d: pages for %d tokens are not allocated (group %d)", id, ctx, g);
            if (resident) {
                int* upd = buf + offsets[8 + 2 * g + 1];           // [0]: count so far, then the triples
                int& given_back = r->trash_sent[(size_t)g];
                int& sent = r->sent[(size_t)g];
                auto emit = [&](int b, int pg) {
                    if (upd[0] >= update_cap) return false;
                    int* t3 = upd + 1 + 3 * upd[0]++;
                    t3[0] = r->slot, t3[1] = b, t3[2] = pg;
                    return true;
                };
                bool room = true;
                while (room && given_back < nb && table[(size_t)given_back] == kReleased) {
                    if (given_back < sent) room = emit(given_back, trash_page);      // else the loop below sends it, as given back
                    if (room) ++given_back;
                }
                while (room && sent < nb) {
                    room = emit(sent, table[(size_t)sent] == kReleased ? trash_page : table[(size_t)sent]);
                    if (room) ++sent;
                }
                if (!room) return fail(LI_HOST_VALUE, "request %d: more than %d changes of its block table in one step (group %d)", id, update_cap, g);
            } else {
                int* bt = buf + offsets[8 + 2 * g + 1] + (size_t)s * max_blocks;
                for (int b = 0; b < nb; ++b) bt[b] = table[(size_t)b] == kReleased ? trash_page : table[(size_t)b];
                for (int b = nb; b < max_blocks; ++b) bt[b] = trash_page;
            }
            int* sm = buf + offsets[8 + 2 * g] + tok;
            for (int j = 0; j < n; ++j) {
                const int pos = start + j, pg = table[(size_t)(pos / page)];
                if (pg == kReleased) return fail(LI_HOST_RUNTIME, "request %d: a new token falls on a page that was given back (group %d)", id, g);
                sm[j] = pg * page + pos % page;
            }
        }
        if (n > max_q) max_q = n;
        if (ctx > max_ctx) max_ctx = ctx;
        if (n == 1) ++singles;
        tok += n;
        tok_in += n;
        want_in += want_counts[s];
        q_start[s + 1] = tok;
    }
    const int r_real_i = row;
    // padding: sequences at position 0 on the sink page
    for (int s = n_items; s < S; ++s) {
        int n = pad_tokens ? 0 : 1;
        if (pad_tokens && s == S - 1) n = (int)t_pad;
        for (int j = 0; j < n; ++j) {
            token_ids[tok + j] = 0;
            positions[tok + j] = j;
            seq_of[tok + j] = s;
            for (int g = 0; g < G; ++g) buf[offsets[8 + 2 * g] + tok + j] = trash_page * page + j % page;
        }
        ctx_lens[s] = n;
        old_lens[s] = 0;
        state_slots[s] = trash_slot;
        for (int g = 0; g < G && !resident; ++g) {
            int* bt = buf + offsets[8 + 2 * g + 1] + (size_t)s * max_blocks;
            for (int b = 0; b < max_blocks; ++b) bt[b] = trash_page;
        }
        if (!pad_tokens) logit_rows[row++] = tok;       // padded items want a row too: the layout depends on S alone
        if (n > max_q) max_q = n;
        if (n > max_ctx) max_ctx = n;
        tok += n;
        q_start[s + 1] = tok;
    }
    if (pad_tokens)
        while (row < R) logit_rows[row++] = T - 1;
    if (tok != T || row != R) return fail(LI_HOST_VALUE, "the step's sizes do not match its items (%d tokens, %d rows)", tok, row);
    info[0] = r_real_i;
    info[1] = max_q;
    info[2] = max_ctx;
    info[3] = max_q > 1 ? singles : 0;
    return LI_HOST_OK;
}
