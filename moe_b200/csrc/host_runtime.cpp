// The host side of a step, in C++: who holds which cache slot and which pages, the
// all-or-nothing reservation of a step, and the packing of a step's index arrays into the
// pinned staging buffer.  No CUDA here: the library builds with the host compiler alone and is
// tested on a machine without a GPU.
//
// A slot belongs to one sequence from its first step until it is released; a page holds
// PAGE_TOKENS consecutive positions of one sequence for every layer of one cache group.  Page 0
// of every pool is never handed out: padding rows of a batch point at it.  The reference keeps
// one flat array of ctx positions per layer and sequence (src/model.rs:140-153) and a pool of
// sessions in its server (src/serve.rs:419-443); slots and pages are this library's own.
//
// Every entry point returns a negative code on failure and leaves a message for
// moe_host_error(): -1 for the cache's own errors (full, not held, freed twice), -2 for a bad
// argument.  A failed call changes nothing.
#include <algorithm>
#include <cstdint>
#include <string>
#include <vector>

#define MOE_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int PAGE_TOKENS = 64;
constexpr int ERR_CACHE = -1, ERR_VALUE = -2;

thread_local std::string g_error;

int fail(int code, std::string msg) {
    g_error = std::move(msg);
    return code;
}

struct SlotPool {
    int num_slots;
    std::vector<int> free_list;      // back() is handed out next: the lowest slot first
    std::vector<char> held;
    explicit SlotPool(int n) : num_slots(n), held(n, 0) {
        for (int s = n - 1; s >= 0; s--) free_list.push_back(s);
    }
    int acquire() {
        if (free_list.empty()) return fail(ERR_CACHE, "all " + std::to_string(num_slots) + " slots are in use");
        const int s = free_list.back();
        free_list.pop_back();
        held[s] = 1;
        return s;
    }
    int release(int s) {
        if (s < 0 || s >= num_slots) return fail(ERR_CACHE, "slot " + std::to_string(s) + " does not exist");
        if (!held[s]) return fail(ERR_CACHE, "slot " + std::to_string(s) + " is not held (released twice?)");
        held[s] = 0;
        free_list.push_back(s);
        return 0;
    }
    bool is_held(int s) const { return s >= 0 && s < num_slots && held[s]; }
};

struct PagePool {
    int num_pages;
    std::vector<int> free_list;
    std::vector<char> held;
    explicit PagePool(int n) : num_pages(n), held(n, 0) {
        for (int p = n - 1; p >= 1; p--) free_list.push_back(p);      // page 0 is the scratch page
    }
    int num_free() const { return (int)free_list.size(); }
    int alloc(int n, int* out) {
        if (n > num_free())
            return fail(ERR_CACHE, "the cache is full: " + std::to_string(n) + " more pages of " +
                                       std::to_string(PAGE_TOKENS) + " tokens wanted, " + std::to_string(num_free()) +
                                       " free of " + std::to_string(num_pages - 1));
        for (int i = 0; i < n; i++) {
            out[i] = free_list.back();
            free_list.pop_back();
            held[out[i]] = 1;
        }
        return n;
    }
    int free_pages(const int* pages, int n) {
        for (int i = 0; i < n; i++) {
            const int p = pages[i];
            if (p <= 0 || p >= num_pages) return fail(ERR_CACHE, "page " + std::to_string(p) + " does not exist");
            if (!held[p]) return fail(ERR_CACHE, "page " + std::to_string(p) + " is not held (freed twice?)");
            for (int j = 0; j < i; j++)
                if (pages[j] == p) return fail(ERR_CACHE, "page " + std::to_string(p) + " is named twice");
        }
        for (int i = 0; i < n; i++) {
            held[pages[i]] = 0;
            free_list.push_back(pages[i]);
        }
        return 0;
    }
};

int pages_for(long long length, int ring_pages) {
    const long long n = (length + PAGE_TOKENS - 1) / PAGE_TOKENS;
    return (int)(ring_pages ? std::min<long long>(n, ring_pages) : n);
}

struct Group {
    PagePool pool;
    int ring_pages;                              // 0: grows with the sequence
    std::vector<std::vector<int>> pages;         // per slot
    Group(int num_pages, int ring, int num_slots) : pool(num_pages), ring_pages(ring), pages(num_slots) {}
};

struct Ledger {
    SlotPool slots;
    std::vector<Group> groups;
    std::vector<int> length;                     // per slot; meaningful while held
    Ledger(int num_slots, int num_groups, const int* group_pages, const int* ring_pages)
        : slots(num_slots), length(num_slots, 0) {
        for (int g = 0; g < num_groups; g++) groups.emplace_back(group_pages[g], ring_pages[g], num_slots);
    }
    // pages each group must add for `slot` to hold new_length tokens
    int need(int g, int slot, long long new_length) const {
        return std::max(0, pages_for(new_length, groups[g].ring_pages) - (int)groups[g].pages[slot].size());
    }
    // hand out the pages (the caller has checked that every pool has enough); appends (g, slot, index, page)
    int grow(int slot, int new_length, int* updates, int cap, int at) {
        for (int g = 0; g < (int)groups.size(); g++) {
            const int n = need(g, slot, new_length);
            if (!n) continue;
            std::vector<int> got(n);
            groups[g].pool.alloc(n, got.data());
            const int base = (int)groups[g].pages[slot].size();
            for (int i = 0; i < n; i++) {
                groups[g].pages[slot].push_back(got[i]);
                if (at < cap) {
                    int* u = updates + 4 * at;
                    u[0] = g, u[1] = slot, u[2] = base + i, u[3] = got[i];
                }
                at++;
            }
        }
        length[slot] = new_length;
        return at;
    }
};

}  // namespace

MOE_API const char* moe_host_error() { return g_error.c_str(); }
MOE_API int moe_host_page_tokens() { return PAGE_TOKENS; }

// ---- the pools alone ---------------------------------------------------------------------------
MOE_API void* moe_slotpool_new(int n) {
    if (n <= 0) {
        fail(ERR_CACHE, "a cache needs at least one slot");
        return nullptr;
    }
    return new SlotPool(n);
}
MOE_API void moe_slotpool_delete(void* p) { delete static_cast<SlotPool*>(p); }
MOE_API int moe_slotpool_acquire(void* p) { return static_cast<SlotPool*>(p)->acquire(); }
MOE_API int moe_slotpool_release(void* p, int s) { return static_cast<SlotPool*>(p)->release(s); }
MOE_API int moe_slotpool_is_held(void* p, int s) { return static_cast<SlotPool*>(p)->is_held(s) ? 1 : 0; }
MOE_API int moe_slotpool_num_free(void* p) { return (int)static_cast<SlotPool*>(p)->free_list.size(); }

MOE_API void* moe_pagepool_new(int n) {
    if (n < 2) {
        fail(ERR_CACHE, "a page pool needs the scratch page and at least one more");
        return nullptr;
    }
    return new PagePool(n);
}
MOE_API void moe_pagepool_delete(void* p) { delete static_cast<PagePool*>(p); }
MOE_API int moe_pagepool_alloc(void* p, int n, int* out) { return n < 0 ? fail(ERR_VALUE, "negative count") : static_cast<PagePool*>(p)->alloc(n, out); }
MOE_API int moe_pagepool_free(void* p, const int* pages, int n) { return static_cast<PagePool*>(p)->free_pages(pages, n); }
MOE_API int moe_pagepool_num_free(void* p) { return static_cast<PagePool*>(p)->num_free(); }

// ---- the ledger ----------------------------------------------------------------------------------
MOE_API void* moe_ledger_new(int num_slots, int num_groups, const int* group_pages, const int* ring_pages) {
    if (num_slots <= 0) {
        fail(ERR_CACHE, "a cache needs at least one slot");
        return nullptr;
    }
    for (int g = 0; g < num_groups; g++)
        if (group_pages[g] < 2) {
            fail(ERR_CACHE, "a page pool needs the scratch page and at least one more");
            return nullptr;
        }
    return new Ledger(num_slots, num_groups, group_pages, ring_pages);
}
MOE_API void moe_ledger_delete(void* p) { delete static_cast<Ledger*>(p); }

MOE_API int moe_ledger_acquire(void* p) {
    Ledger& L = *static_cast<Ledger*>(p);
    const int s = L.slots.acquire();
    if (s >= 0) {
        L.length[s] = 0;
        for (auto& g : L.groups) g.pages[s].clear();
    }
    return s;
}

MOE_API int moe_ledger_release(void* p, int slot) {
    Ledger& L = *static_cast<Ledger*>(p);
    if (!L.slots.is_held(slot)) return fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not held (released twice?)");
    for (auto& g : L.groups) {
        const int rc = g.pool.free_pages(g.pages[slot].data(), (int)g.pages[slot].size());
        if (rc) return rc;
        g.pages[slot].clear();
    }
    L.length[slot] = 0;
    return L.slots.release(slot);
}

MOE_API int moe_ledger_is_held(void* p, int slot) { return static_cast<Ledger*>(p)->slots.is_held(slot) ? 1 : 0; }

MOE_API int moe_ledger_length(void* p, int slot) {
    Ledger& L = *static_cast<Ledger*>(p);
    if (!L.slots.is_held(slot)) return fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not held");
    return L.length[slot];
}

// what: 0 free slots, 1 held slots, 2 free pages of `group`, 3 pages of `group` in all, 4 ring pages of `group`
MOE_API int moe_ledger_count(void* p, int what, int group) {
    Ledger& L = *static_cast<Ledger*>(p);
    if (what >= 2 && (group < 0 || group >= (int)L.groups.size())) return fail(ERR_VALUE, "no such cache group");
    switch (what) {
        case 0: return (int)L.slots.free_list.size();
        case 1: return L.slots.num_slots - (int)L.slots.free_list.size();
        case 2: return L.groups[group].pool.num_free();
        case 3: return L.groups[group].pool.num_pages;
        case 4: return L.groups[group].ring_pages;
        default: return fail(ERR_VALUE, "no such count");
    }
}

// the pages of `slot` in `group`, in order; returns how many there are (out gets at most cap)
MOE_API int moe_ledger_pages(void* p, int group, int slot, int* out, int cap) {
    Ledger& L = *static_cast<Ledger*>(p);
    if (group < 0 || group >= (int)L.groups.size()) return fail(ERR_VALUE, "no such cache group");
    if (!L.slots.is_held(slot)) return fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not held");
    const auto& v = L.groups[group].pages[slot];
    for (int i = 0; i < (int)v.size() && i < cap; i++) out[i] = v[i];
    return (int)v.size();
}

// Room for new_length tokens in `slot`: every group gets its pages or none does.  Writes the
// page-table entries that changed as (group, slot, index, page) and returns their number.
MOE_API int moe_ledger_extend(void* p, int slot, int new_length, int* updates, int cap) {
    Ledger& L = *static_cast<Ledger*>(p);
    if (!L.slots.is_held(slot)) return fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not held");
    if (new_length < L.length[slot]) return fail(ERR_CACHE, "extend cannot shrink a sequence; use truncate");
    for (int g = 0; g < (int)L.groups.size(); g++) {
        const int n = L.need(g, slot, new_length);
        if (n > L.groups[g].pool.num_free())
            return fail(ERR_CACHE, "the cache is full: slot " + std::to_string(slot) + " needs " + std::to_string(n) +
                                       " more pages of " + std::to_string(PAGE_TOKENS) + " tokens, " +
                                       std::to_string(L.groups[g].pool.num_free()) + " free");
    }
    return L.grow(slot, new_length, updates, cap, 0);
}

// Forget everything at or after new_length (src/model.rs:176-189).  Pages are kept.  A ring holds
// the last `ring` positions only: once it has wrapped, a rewind is possible only while the keys that
// the token at new_length will look back on, [new_length + 1 - window, new_length), are still in it.
// windows[g]: the window of group g (0 or a null array: unknown, any rewind of a wrapped ring is refused).
MOE_API int moe_ledger_truncate(void* p, int slot, int new_length, const int* windows) {
    Ledger& L = *static_cast<Ledger*>(p);
    if (!L.slots.is_held(slot)) return fail(ERR_CACHE, "slot " + std::to_string(slot) + " is not held");
    const int cur = L.length[slot];
    if (new_length > cur) return fail(ERR_CACHE, "truncate cannot lengthen a sequence");
    if (new_length < 0) return fail(ERR_VALUE, "negative length");
    for (size_t gi = 0; gi < L.groups.size(); gi++) {
        const auto& g = L.groups[gi];
        const int ring = g.ring_pages * PAGE_TOKENS;
        if (!g.ring_pages || new_length == cur || cur <= ring) continue;
        const int w = windows ? windows[gi] : 0;
        const int oldest_needed = w > 0 ? std::max(0, new_length + 1 - w) : 0;
        if (w <= 0 || oldest_needed < cur - ring)
            return fail(ERR_CACHE, "a windowed cache no longer holds the keys before position " +
                                       std::to_string(new_length) + ": it cannot be rewound that far");
    }
    L.length[slot] = new_length;
    return 0;
}

// tokens the live sequences hold, each rounded up to whole pages
MOE_API long long moe_ledger_tokens_held(void* p) {
    Ledger& L = *static_cast<Ledger*>(p);
    long long n = 0;
    for (int s = 0; s < L.slots.num_slots; s++)
        if (L.slots.held[s]) n += (long long)pages_for(L.length[s], 0) * PAGE_TOKENS;
    return n;
}

// The reservation of a whole step: sequence i (in slots[i]) brings counts[i] more tokens.  Either
// every sequence gets its room in every group or nothing changes.  table_cap[g]: the most pages a
// sequence may hold in group g (its page table's width; 0: no limit).  Writes each sequence's
// length before the step to starts[] and the changed page-table entries to updates[] as
// (group, slot, index, page); returns their number (which may exceed cap: call again with more).
// What a step needs, without changing anything: 0 if every sequence finds its room in every group
// (total_updates: the page-table entries that would change), else the error of moe_ledger_reserve.
static int check_step(Ledger& L, int B, const int* slots, const int* counts, const int* table_cap, long long max_tokens,
                      long long* total_updates) {
    const int G = (int)L.groups.size();
    std::vector<char> seen(L.slots.num_slots, 0);
    std::vector<long long> need(G, 0);
    *total_updates = 0;
    for (int i = 0; i < B; i++) {
        const int s = slots[i];
        if (!L.slots.is_held(s)) return fail(ERR_CACHE, "slot " + std::to_string(s) + " is not held");
        if (seen[s]) return fail(ERR_VALUE, "a slot appears twice in one step");
        seen[s] = 1;
        if (counts[i] <= 0) return fail(ERR_VALUE, "every sequence of a step brings at least one token");
        const long long end = (long long)L.length[s] + counts[i];
        if (end > INT32_MAX) return fail(ERR_VALUE, "a sequence would outgrow 2^31 positions");
        for (int g = 0; g < G; g++) {
            need[g] += L.need(g, s, end);
            if (!L.groups[g].ring_pages && table_cap && table_cap[g] > 0 && pages_for(end, 0) > table_cap[g])
                return fail(ERR_CACHE, "a sequence would outgrow the page table");
        }
    }
    for (int g = 0; g < G; g++) {
        if (need[g] > L.groups[g].pool.num_free())
            return fail(ERR_CACHE, "the cache is full: this step needs " + std::to_string(need[g]) + " more pages of " +
                                       std::to_string(PAGE_TOKENS) + " tokens, " + std::to_string(L.groups[g].pool.num_free()) +
                                       " are free (max_tokens = " + std::to_string(max_tokens) + ")");
        *total_updates += need[g];
    }
    return 0;
}

MOE_API int moe_ledger_reserve(void* p, int B, const int* slots, const int* counts, const int* table_cap, int* starts,
                               int* updates, int cap, long long max_tokens) {
    Ledger& L = *static_cast<Ledger*>(p);
    long long total_updates = 0;
    const int rc = check_step(L, B, slots, counts, table_cap, max_tokens, &total_updates);
    if (rc) return rc;
    if (total_updates > cap) return (int)std::min<long long>(total_updates, INT32_MAX);   // nothing changed yet
    int at = 0;
    for (int i = 0; i < B; i++) {
        starts[i] = L.length[slots[i]];
        at = L.grow(slots[i], L.length[slots[i]] + counts[i], updates, cap, at);
    }
    return at;
}

// Would moe_ledger_reserve succeed?  0, or its error; nothing changes either way.  (A step that the
// engine runs in several pieces asks this first, so that it fails before its first piece or not at all.)
MOE_API int moe_ledger_check(void* p, int B, const int* slots, const int* counts, const int* table_cap,
                             long long max_tokens) {
    long long total_updates = 0;
    return check_step(*static_cast<Ledger*>(p), B, slots, counts, table_cap, max_tokens, &total_updates);
}

// ---- packing a step ------------------------------------------------------------------------------
// The index arrays of a step, one after another in `buf` (int32):
//   token_ids[T] seq_of_token[T] pos[T] cu_seqlens[B + 1] slots[B] seq_start[B] seq_end[B] want_rows[max(W, 1)]
// tokens: the sequences' tokens one after another; want: for each sequence want_counts[i] places
// among its tokens.  offsets[8]: where each array begins.  facts[7]: T, B, W, max_new, max_end,
// all_decode, all_fresh.  Returns the ints used.
MOE_API long long moe_pack_step(int* buf, long long cap, int B, const int* slots, const int* starts, const int* counts,
                                const int* tokens, const int* want_counts, const int* want, int* offsets, int* facts) {
    long long T = 0, W = 0;
    for (int i = 0; i < B; i++) {
        if (counts[i] <= 0) return fail(ERR_VALUE, "every sequence of a step brings at least one token");
        T += counts[i];
        W += want_counts[i];
    }
    const long long sizes[8] = {T, T, T, B + 1, B, B, B, std::max<long long>(W, 1)};
    long long o = 0;
    for (int k = 0; k < 8; k++) {
        if (o > INT32_MAX) return fail(ERR_VALUE, "step too large");
        offsets[k] = (int)o;
        o += sizes[k];
    }
    if (o > cap) return fail(ERR_VALUE, "staging buffer too small");
    int *tok = buf + offsets[0], *sot = buf + offsets[1], *pos = buf + offsets[2], *cu = buf + offsets[3];
    int *sl = buf + offsets[4], *st = buf + offsets[5], *en = buf + offsets[6], *wr = buf + offsets[7];
    int at = 0, wi = 0, max_new = 0, max_end = 0, all_decode = 1, all_fresh = 1;
    const int* w = want;
    for (int i = 0; i < B; i++) {
        const int n = counts[i];
        for (int j = 0; j < n; j++) {
            tok[at + j] = tokens[at + j];
            sot[at + j] = i;
            pos[at + j] = starts[i] + j;
        }
        cu[i] = at, sl[i] = slots[i], st[i] = starts[i], en[i] = starts[i] + n;
        for (int j = 0; j < want_counts[i]; j++, w++) {
            if (*w < 0 || *w >= n)
                return fail(ERR_VALUE, "wanted place " + std::to_string(*w) + " is not among the " + std::to_string(n) +
                                           " tokens of this step");
            wr[wi++] = at + *w;
        }
        max_new = std::max(max_new, n), max_end = std::max(max_end, starts[i] + n);
        all_decode &= n == 1, all_fresh &= starts[i] == 0;
        at += n;
    }
    cu[B] = at;
    if (W == 0) wr[0] = 0;
    facts[0] = (int)T, facts[1] = B, facts[2] = (int)W, facts[3] = max_new, facts[4] = max_end;
    facts[5] = all_decode, facts[6] = all_fresh;
    return o;
}

// Any step, padded for a captured graph to `tp` token rows, `bb` sequences and `wb` wanted places:
// rows past the tokens belong to no sequence (seq_of_token -1, position 0, token 0), sequences past B
// are empty and sit in the padding slot, wanted places past the real ones repeat row 0 (the caller
// drops them).  Layout: token_ids[tp] seq_of_token[tp] pos[tp] cu_seqlens[bb + 1] slots[bb]
// seq_start[bb] seq_end[bb] want_rows[wb], then per cache group `upd_cap` page-table updates at
// upd_off[g], padded as in moe_pack_decode.  starts, want_counts, want: as in moe_pack_step.
MOE_API int moe_pack_padded(int* buf, int tp, int bb, int wb, int B, const int* slots, const int* starts,
                            const int* counts, const int* tokens, const int* want_counts, const int* want,
                            int pad_slot, int num_groups, const int* upd_off, int upd_cap, const int* updates,
                            int num_updates) {
    if (B > bb || B < 0) return fail(ERR_VALUE, "more sequences than the bucket holds");
    long long T = 0, W = 0;
    for (int i = 0; i < B; i++) {
        if (counts[i] <= 0) return fail(ERR_VALUE, "every sequence of a step brings at least one token");
        T += counts[i], W += want_counts[i];
    }
    if (T > tp) return fail(ERR_VALUE, "more tokens than the bucket holds");
    if (W > wb) return fail(ERR_VALUE, "more wanted places than the bucket holds");
    int* tok = buf;
    int *sot = tok + tp, *pos = sot + tp, *cu = pos + tp, *sl = cu + bb + 1, *st = sl + bb, *en = st + bb;
    int* wr = en + bb;
    int at = 0, wi = 0;
    const int* w = want;
    for (int i = 0; i < bb; i++) {
        const int n = i < B ? counts[i] : 0, s0 = i < B ? starts[i] : 0;
        for (int j = 0; j < n; j++) tok[at + j] = tokens[at + j], sot[at + j] = i, pos[at + j] = s0 + j;
        cu[i] = at, sl[i] = i < B ? slots[i] : pad_slot, st[i] = s0, en[i] = s0 + n;
        for (int j = 0; i < B && j < want_counts[i]; j++, w++) {
            if (*w < 0 || *w >= n)
                return fail(ERR_VALUE, "wanted place " + std::to_string(*w) + " is not among the " + std::to_string(n) +
                                           " tokens of this step");
            wr[wi++] = at + *w;
        }
        at += n;
    }
    cu[bb] = at;
    for (; wi < wb; wi++) wr[wi] = 0;
    for (int t = at; t < tp; t++) tok[t] = 0, sot[t] = -1, pos[t] = 0;
    for (int g = 0; g < num_groups; g++) {
        int* u = buf + upd_off[g];
        int n = 0;
        for (int k = 0; k < num_updates; k++) {
            const int* e = updates + 4 * k;
            if (e[0] != g) continue;
            if (n >= upd_cap) return fail(ERR_VALUE, "more page-table updates than the bucket holds");
            u[3 * n] = e[1], u[3 * n + 1] = e[2], u[3 * n + 2] = e[3];
            n++;
        }
        for (; n < upd_cap; n++) u[3 * n] = pad_slot, u[3 * n + 1] = 0, u[3 * n + 2] = 0;
    }
    return 0;
}

// A step of one token per sequence, padded to `size` rows for a captured graph: rows past B belong
// to no sequence (seq_of_token -1, the padding slot, position 0).  After the eight arrays of
// moe_pack_step (each `size` long, cu_seqlens size + 1) come, per cache group, `size` page-table
// updates (slot, index, page) at upd_off[g]; unused ones rewrite the padding slot's first entry
// with 0, which changes nothing.  updates: (group, slot, index, page) as moe_ledger_reserve wrote them.
MOE_API int moe_pack_decode(int* buf, int size, int B, const int* slots, const int* starts, const int* tokens,
                            int pad_slot, int num_groups, const int* upd_off, const int* updates, int num_updates) {
    if (B > size || B < 0) return fail(ERR_VALUE, "more sequences than the bucket holds");
    int* tok = buf;
    int *sot = tok + size, *pos = sot + size, *cu = pos + size, *sl = cu + size + 1, *st = sl + size, *en = st + size;
    int* wr = en + size;
    for (int i = 0; i < size; i++) {
        const bool live = i < B;
        tok[i] = live ? tokens[i] : 0;
        sot[i] = live ? i : -1;
        pos[i] = live ? starts[i] : 0;
        cu[i] = live ? i : B;
        sl[i] = live ? slots[i] : pad_slot;
        st[i] = live ? starts[i] : 0;
        en[i] = live ? starts[i] + 1 : 1;
        wr[i] = i;
    }
    cu[size] = B;
    for (int g = 0; g < num_groups; g++) {
        int* u = buf + upd_off[g];
        int n = 0;
        for (int k = 0; k < num_updates; k++) {
            const int* e = updates + 4 * k;
            if (e[0] != g) continue;
            if (n >= size) return fail(ERR_VALUE, "more page-table updates than the bucket holds");
            u[3 * n] = e[1], u[3 * n + 1] = e[2], u[3 * n + 2] = e[3];
            n++;
        }
        for (; n < size; n++) u[3 * n] = pad_slot, u[3 * n + 1] = 0, u[3 * n + 2] = 0;
    }
    return 0;
}
