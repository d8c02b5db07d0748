/* The C interface of the host runtime (liblitinfer_host_*.so): page pools, the block tables of the live requests, the
 * packer of a step's metadata and the scheduler's decisions.  Plain host code: no CUDA, all pointers are host pointers.
 * litinfer_b200/cache and litinfer_b200/engine/scheduler.py call it through ctypes.
 *
 * Every int-returning function that can fail returns one of the classes below and leaves the message for
 * li_host_last_error().  Not thread-safe per object; different objects may be used from different threads.
 * LitInfer's counterparts: src/llaisys/kv_cache/block_kv_cache.hpp and the engine_* entries of include/llaisys/models/qwen2.h.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

enum { LI_HOST_OK = 0, LI_HOST_POOL = 1, LI_HOST_OUT_OF_PAGES = 2, LI_HOST_VALUE = 3, LI_HOST_INDEX = 4, LI_HOST_RUNTIME = 5 };

/* ---- runtime.cpp ---- */
/* The calling thread's message of the last call that returned non-zero. */
const char* li_host_last_error();

/* A pool by itself: `pages` ids, page 0 comes out first, a page just given back is the next one handed out. */
void* li_pool_create(int pages, const char* what);

void li_pool_destroy(void* p);

/* A free id for `owner` (>= 0). */
int li_pool_alloc(void* p, int owner, int* page);

/* Give `page` back; refused if it is free already or held by another owner. */
int li_pool_free(void* p, int page, int owner);

int li_pool_num_free(void* p);

/* The owner of `page`, -1 if it is free, -2 if it is outside the pool. */
int li_pool_owner(void* p, int page);

/* Every id is either free exactly once or owned. */
int li_pool_check(void* p);

/* A manager of `groups` page-id spaces of `num_pages` pages of `page_size` tokens and `max_requests` state slots;
 * windows[g] <= 0: the group keeps every key. */
void* li_cm_create(int groups, const int* windows, int num_pages, int page_size, int max_requests);

void li_cm_destroy(void* h);

/* Free ids of a pool; which: -1 the state slots, else a group's pages. */
int li_cm_num_free(void* h, int which);

/* The request that holds a page (-1 free, -2 outside). */
int li_cm_owner(void* h, int which, int page);

int li_cm_pool_check(void* h, int which);

/* Pages each group lacks for positions up to new_length */
int li_cm_pages_needed(void* h, int id, int new_length, int* need);

/* The step has written positions below new_length: pages of windowed groups that no further query can read go back */
int li_cm_commit(void* h, int id, int new_length);

/* li_cm_commit for the requests of a step at once. */
int li_cm_commit_many(void* h, int n, const int* ids, const int* new_lengths);

/* A new live request: takes a state slot. */
int li_cm_admit(void* h, int id, int* slot);

/* Pages for positions up to new_length in every group; all or nothing (LI_HOST_OUT_OF_PAGES changes nothing). */
int li_cm_extend(void* h, int id, int new_length);

/* All pages (last first) and the slot go back; the request is no longer live. */
int li_cm_release(void* h, int id);

/* Tokens whose keys and values are cached (-1: not live). */
int li_cm_length(void* h, int id);

/* A request's block table of one group: its length, and up to cap entries into out */
int li_cm_table(void* h, int id, int group, int* out, int cap);

/* No page lost, held twice, or held by a request that is not live */
int li_cm_check(void* h);

/* The packer.  Fills the packed int32 buffer of a step (engine/batch.py describes the layout; `offsets` gives where each
 * field starts: token_ids, positions, seq_of_token, q_start, ctx_lens, old_lens, state_slots, logit_rows, then per group
 * slot_mapping and block_table).  Items: request ids, token counts, tokens and wanted places, flattened.  starts[i] /
 * olds[i] (or -1: the request's cached length): the position of the item's first token, and how many of the request's
 * keys were cached before the step; they differ from the cached length when a portion is given as single tokens.  The
 * batch is padded to S sequences, T tokens and R rows (with pad_tokens the padding sequences are empty but the last,
 * else they hold one token each and want its row).  The buffer must be zeroed and sized by the caller; T, S, R and the
 * width of the block tables are the caller's too, checked here. */
int li_cm_pack_step(void* h, int n_items, const int* request_ids, const int* q_lens, const int* starts, const int*
    olds, const int* tokens, const int* want_counts, const int* wants, int vocab, int S, int T, int R, int pad_tokens,
    int max_blocks, int allow_repeat, int trash_page, int trash_slot, const int* offsets, int* buf, long long buf_len,
    int* info /* R_real, max_q_len, max_ctx_len, singles */, int update_cap);

/* Resident tables (li_cm_pack_step with update_cap >= 0: the field of a group's block tables then holds a count and
 * triples (state slot, logical page, page id) that bring the device's copy of the step's requests' tables up to date,
 * and what is written counts as sent): an upper bound of how many triples a group can need for these items. */
int li_cm_table_updates_bound(void* h, int n_items, const int* request_ids, const int* q_lens, const int* starts, int* bound);

/* ---- scheduler.cpp ---- */
/* A scheduler over a manager (which must outlive it). */
void* li_sched_create(void* manager, int max_num_seqs, int max_tokens_per_step, int prefill_chunk, int max_positions);

void li_sched_destroy(void* h);

/* The token ids that end a request and are dropped from its output. */
int li_sched_set_eos(void* h, const int* ids, int n);

/* A new request at the end of the waiting queue (its sizes were checked by the caller) */
int li_sched_add(void* h, int id, int prompt_len, int max_new_tokens);

/* Requests waiting and running, and preemptions so far. */
int li_sched_counts(void* h, int* waiting, int* running, int* preemptions);

/* Picks the next step's items and allocates their pages.  items: up to item_cap rows of (id, start, count, wants
 * logits); events: up to event_cap rows of (kind, id, arg) in the order they happened: 1 admitted (arg: its state
 * slot), 2 preempted. */
int li_sched_schedule(void* h, int* items, int item_cap, int* n_items, int* events, int event_cap, int* n_events);

/* After the step: tokens[i] was drawn for request ids[i].  outcome[i]: 1 the token is part of the output, 0 it is
 * the dropped end-of-sequence token; reason[i]: 0 the request goes on, else why it ended (1 eos, 2 length, 3
 * positions). A request that ends gives its pages and slot back here. */
int li_sched_update(void* h, int n, const int* ids, const int* tokens, int* outcome, int* reason);

/* Aborts a request that has not finished; was_running: whether the request held pages and a slot (given back here) */
int li_sched_abort(void* h, int id, int* was_running);

/* Drop a finished request's record. */
int li_sched_forget(void* h, int id);

#ifdef __cplusplus
}
#endif
