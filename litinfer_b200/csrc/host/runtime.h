// Types of the host runtime shared by its files: error classes, the pool, a request's tables, the manager.
#pragma once
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#define LI_HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace li_host {

enum { LI_HOST_OK = 0, LI_HOST_POOL = 1, LI_HOST_OUT_OF_PAGES = 2, LI_HOST_VALUE = 3, LI_HOST_INDEX = 4, LI_HOST_RUNTIME = 5 };

char* error_text();                           // the calling thread's last message (512 bytes)
int fail(int code, const char* fmt, ...);     // stores the message, returns the code

constexpr int kFree = -1;          // owner of a page nobody holds
constexpr int kReleased = -1;      // block-table entry of a page that was given back behind a window

// A LIFO free list with ownership: page 0 comes out first, a page just given back is the next one handed out.
struct Pool {
    int n = 0;
    std::string what;
    std::vector<int> free_list;
    std::vector<int> owner;

    Pool(int pages, const char* name) : n(pages), what(name), owner((size_t)pages, kFree) {
        free_list.reserve((size_t)pages);
        for (int p = pages - 1; p >= 0; --p) free_list.push_back(p);
    }
    int num_free() const { return (int)free_list.size(); }
    int alloc(int who, int* page) {
        if (who < 0) return fail(LI_HOST_POOL, "owner ids are non-negative");
        if (free_list.empty()) return fail(LI_HOST_OUT_OF_PAGES, "no free %s (all %d in use)", what.c_str(), n);
        *page = free_list.back();
        free_list.pop_back();
        owner[(size_t)*page] = who;
        return LI_HOST_OK;
    }
    int release(int page, int who) {
        if (page < 0 || page >= n) return fail(LI_HOST_POOL, "%s %d is outside the pool of %d", what.c_str(), page, n);
        const int held_by = owner[(size_t)page];
        if (held_by == kFree) return fail(LI_HOST_POOL, "%s %d freed twice", what.c_str(), page);
        if (held_by != who) return fail(LI_HOST_POOL, "%s %d is held by %d, not by %d", what.c_str(), page, held_by, who);
        owner[(size_t)page] = kFree;
        free_list.push_back(page);
        return LI_HOST_OK;
    }
    // every page is either free exactly once or owned, never both
    int check() const {
        std::vector<char> seen((size_t)n, 0);
        for (int p : free_list) {
            if (seen[(size_t)p]) return fail(LI_HOST_POOL, "%s %d is on the free list twice", what.c_str(), p);
            if (owner[(size_t)p] != kFree) return fail(LI_HOST_POOL, "%s %d is free and owned by %d", what.c_str(), p, owner[(size_t)p]);
            seen[(size_t)p] = 1;
        }
        for (int p = 0; p < n; ++p)
            if (owner[(size_t)p] == kFree && !seen[(size_t)p]) return fail(LI_HOST_POOL, "%s %d is lost: neither free nor owned", what.c_str(), p);
        return LI_HOST_OK;
    }
};

struct Request {
    int id = 0, slot = 0, length = 0;
    std::vector<std::vector<int>> tables;          // per group: logical page -> page id, kReleased once given back
    // What the device's resident copy of the tables holds of this request (li_cm_pack_step in resident mode): per group,
    // logical pages below sent[g] have been sent with the page id they had then, and those below trash_sent[g] have been
    // sent again as given back (pages go back as a growing prefix, li_cm_commit).
    std::vector<int> sent, trash_sent;
};

struct Manager {
    int page_size, num_pages, max_requests;
    std::vector<int> windows;                      // per group: keys a query still reads, 0 = all of them
    std::vector<Pool> pools;
    Pool slots;
    std::unordered_map<int, Request> live;

    Manager(int groups, const int* win, int pages, int page, int requests)
        : page_size(page), num_pages(pages), max_requests(requests), windows(win, win + groups), slots(requests, "state slot") {
        for (int g = 0; g < groups; ++g) pools.emplace_back(pages, "page");
    }
    Request* find(int id) {
        auto it = live.find(id);
        return it == live.end() ? nullptr : &it->second;
    }
    int blocks(int tokens) const { return (tokens + page_size - 1) / page_size; }
    // first logical page that a query at a position >= length can still read
    int first_needed_page(int g, int length) const {
        if (windows[(size_t)g] <= 0) return 0;
        const int first_key = length - windows[(size_t)g] + 1;
        return first_key > 0 ? first_key / page_size : 0;
    }
};

#define FIND(m, r, id)                                                                \
    Request* r = (m)->find(id);                                                       \
    if (!r) return fail(LI_HOST_POOL, "request %d is not live", id)


int cm_admit(Manager* m, int id, int* slot);
int cm_extend(Manager* m, int id, int new_length);
int cm_release(Manager* m, int id);

}  // namespace li_host
