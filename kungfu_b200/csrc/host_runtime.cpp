// Host-side runtime of the engine, in C++: the page pools and block tables of the cache manager, the builder of the
// integer block every step sends to the device, and the scheduler that plans each step.  The Python classes of
// kungfu_b200/cache, kungfu_b200/engine/step.py and kungfu_b200/engine/scheduler.py are thin wrappers over the functions
// exported here (C ABI, called through ctypes).
//
// The reference keeps the corresponding state in Rust (per-slot ring caches sized at plan time,
// crates/kf-core/src/plan.rs:59-64 and crates/kf-backend-cuda/src/exec.rs:1466-1498; per-pass integer inputs staged
// in one pinned buffer, exec.rs:2922-2944).  Here the unit is a page, a request owns a block table per cache group,
// and a windowed group gives pages back as soon as no later query can reach them.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <deque>
#include <unordered_map>
#include <vector>

#define KF_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

struct Pool {
  int n = 0;
  std::vector<int> free_list;           // pop_back hands out low ids first
  std::vector<char> held;
  long n_taken = 0;                     // pages handed out so far (more than n: pages were used again)
  explicit Pool(int n_pages) : n(n_pages), held(n_pages, 0) {
    free_list.reserve(n_pages);
    for (int i = n_pages - 1; i >= 0; --i) free_list.push_back(i);
  }
  int n_free() const { return (int)free_list.size(); }
  int take() {
    if (free_list.empty()) return -1;
    const int p = free_list.back();
    free_list.pop_back();
    held[p] = 1;
    ++n_taken;
    return p;
  }
  bool give_back(int p) {
    if (p < 0 || p >= n || !held[p]) return false;
    held[p] = 0;
    free_list.push_back(p);
    return true;
  }
};

struct Group {
  int window;                            // -1: none
  Pool pool;
  std::vector<int> mirror;               // [max_requests][width]: block tables by state slot, -1 where no page
  Group(int w, int n_pages) : window(w), pool(n_pages) {}
};

struct Request {
  int slot = 0;
  int length = 0;                        // tokens committed
  int reserved = 0;                      // tokens reserved beyond the committed length
  std::vector<int> n_entries;            // per group: entries of the block table in use (absolute page index)
  std::vector<int> first_live;           // per group: first page index still held
};

struct Cache {
  int page_size, max_requests, max_context, max_pages, width;
  std::vector<Group> groups;
  std::unordered_map<int64_t, Request> reqs;
  std::vector<int> free_slots;
  int* row(int g, int slot) { return groups[g].mirror.data() + (size_t)slot * width; }
};

enum { OK = 0, E_NOT_LIVE = 1, E_ALREADY_LIVE = 2, E_NO_SLOT = 3, E_OUT_OF_PAGES = 4, E_CONTEXT = 5, E_COMMIT = 6,
       E_PAGE_NOT_HELD = 7, E_INCONSISTENT = 8 };

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int align4(int n) { return (n + 3) & ~3; }

}  // namespace

// ---- page pool (exported on its own for its unit test) -----------------------------------------------------------
KF_HOST_API void* kf_pool_create(int n_pages) { return new Pool(n_pages); }
KF_HOST_API void kf_pool_destroy(void* p) { delete (Pool*)p; }
KF_HOST_API int kf_pool_take(void* p) { return ((Pool*)p)->take(); }
KF_HOST_API int kf_pool_give_back(void* p, int page) { return ((Pool*)p)->give_back(page) ? OK : E_PAGE_NOT_HELD; }
KF_HOST_API int kf_pool_n_free(void* p) { return ((Pool*)p)->n_free(); }
KF_HOST_API int kf_pool_is_held(void* p, int page) { Pool* q = (Pool*)p; return page >= 0 && page < q->n && q->held[page]; }

// ---- cache manager ---------------------------------------------------------------------------------------------------
KF_HOST_API void* kf_cache_create(int n_groups, const int* windows, const int* n_pages, int page_size, int max_requests,
                                  int max_context) {
  Cache* c = new Cache();
  c->page_size = page_size;
  c->max_requests = max_requests;
  c->max_context = max_context;
  c->max_pages = ceil_div(max_context, page_size);
  c->width = align4(c->max_pages);
  for (int g = 0; g < n_groups; ++g) {
    c->groups.emplace_back(windows[g], n_pages[g]);
    c->groups.back().mirror.assign((size_t)max_requests * c->width, -1);
  }
  for (int s = max_requests - 1; s >= 0; --s) c->free_slots.push_back(s);
  return c;
}
KF_HOST_API void kf_cache_destroy(void* h) { delete (Cache*)h; }
KF_HOST_API int kf_cache_width(void* h) { return ((Cache*)h)->width; }
KF_HOST_API int kf_cache_n_live(void* h) { return (int)((Cache*)h)->reqs.size(); }
KF_HOST_API int kf_cache_contains(void* h, int64_t req) { return ((Cache*)h)->reqs.count(req) ? 1 : 0; }
KF_HOST_API int kf_cache_length(void* h, int64_t req) {
  auto& m = ((Cache*)h)->reqs;
  auto it = m.find(req);
  return it == m.end() ? -1 : it->second.length;
}
KF_HOST_API int kf_cache_state_slot(void* h, int64_t req) {
  auto& m = ((Cache*)h)->reqs;
  auto it = m.find(req);
  return it == m.end() ? -1 : it->second.slot;
}
KF_HOST_API int kf_cache_pool_n_free(void* h, int g) { return ((Cache*)h)->groups[g].pool.n_free(); }
KF_HOST_API int kf_cache_pool_is_held(void* h, int g, int page) {
  Pool& p = ((Cache*)h)->groups[g].pool;
  return page >= 0 && page < p.n && p.held[page];
}
KF_HOST_API long kf_cache_pool_n_taken(void* h, int g) { return ((Cache*)h)->groups[g].pool.n_taken; }
KF_HOST_API const int* kf_cache_mirror(void* h, int g) { return ((Cache*)h)->groups[g].mirror.data(); }

// state slot (>= 0) or -(error code)
KF_HOST_API int kf_cache_add_request(void* h, int64_t req) {
  Cache* c = (Cache*)h;
  if (c->reqs.count(req)) return -E_ALREADY_LIVE;
  if (c->free_slots.empty()) return -E_NO_SLOT;
  Request r;
  r.slot = c->free_slots.back();
  c->free_slots.pop_back();
  r.n_entries.assign(c->groups.size(), 0);
  r.first_live.assign(c->groups.size(), 0);
  for (size_t g = 0; g < c->groups.size(); ++g) std::fill(c->row((int)g, r.slot), c->row((int)g, r.slot) + c->width, -1);
  c->reqs.emplace(req, std::move(r));
  return c->reqs[req].slot;
}

// pages each group must still take so that the request can hold n_new more tokens
KF_HOST_API int kf_cache_pages_needed(void* h, int64_t req, int n_new, int* out) {
  Cache* c = (Cache*)h;
  auto it = c->reqs.find(req);
  if (it == c->reqs.end()) return E_NOT_LIVE;
  const Request& r = it->second;
  const int want = ceil_div(r.length + r.reserved + n_new, c->page_size);
  for (size_t g = 0; g < c->groups.size(); ++g) out[g] = std::max(0, want - r.n_entries[g]);
  return OK;
}

// all-or-nothing: OK, or E_OUT_OF_PAGES / E_CONTEXT with nothing taken
KF_HOST_API int kf_cache_reserve(void* h, int64_t req, int n_new) {
  Cache* c = (Cache*)h;
  auto it = c->reqs.find(req);
  if (it == c->reqs.end()) return E_NOT_LIVE;
  Request& r = it->second;
  if (r.length + r.reserved + n_new > c->max_context) return E_CONTEXT;
  const int want = ceil_div(r.length + r.reserved + n_new, c->page_size);
  for (size_t g = 0; g < c->groups.size(); ++g)
    if (std::max(0, want - r.n_entries[g]) > c->groups[g].pool.n_free()) return E_OUT_OF_PAGES;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    int* row = c->row((int)g, r.slot);
    while (r.n_entries[g] < want) row[r.n_entries[g]++] = c->groups[g].pool.take();
  }
  r.reserved += n_new;
  return OK;
}

KF_HOST_API int kf_cache_cancel_reservation(void* h, int64_t req) {
  Cache* c = (Cache*)h;
  auto it = c->reqs.find(req);
  if (it == c->reqs.end()) return E_NOT_LIVE;
  Request& r = it->second;
  r.reserved = 0;
  const int keep = ceil_div(r.length, c->page_size);
  for (size_t g = 0; g < c->groups.size(); ++g) {
    int* row = c->row((int)g, r.slot);
    while (r.n_entries[g] > keep) {
      const int p = row[--r.n_entries[g]];
      row[r.n_entries[g]] = -1;
      if (p >= 0 && !c->groups[g].pool.give_back(p)) return E_PAGE_NOT_HELD;
    }
  }
  return OK;
}

// the step that wrote n_new reserved tokens succeeded: advance, and give back the pages a window has passed
KF_HOST_API int kf_cache_commit(void* h, int64_t req, int n_new) {
  Cache* c = (Cache*)h;
  auto it = c->reqs.find(req);
  if (it == c->reqs.end()) return E_NOT_LIVE;
  Request& r = it->second;
  if (n_new > r.reserved) return E_COMMIT;
  r.reserved -= n_new;
  r.length += n_new;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    const int w = c->groups[g].window;
    if (w < 0) continue;
    // a query at position p reads keys >= p - w + 1; the next query sits at r.length
    const int dead = std::min(std::max(0, r.length - w + 1) / c->page_size, r.n_entries[g]);
    int* row = c->row((int)g, r.slot);
    for (int i = r.first_live[g]; i < dead; ++i) {
      if (row[i] >= 0) {
        if (!c->groups[g].pool.give_back(row[i])) return E_PAGE_NOT_HELD;
        row[i] = -1;
      }
    }
    r.first_live[g] = std::max(r.first_live[g], dead);
  }
  return OK;
}

KF_HOST_API int kf_cache_release(void* h, int64_t req) {
  Cache* c = (Cache*)h;
  auto it = c->reqs.find(req);
  if (it == c->reqs.end()) return E_NOT_LIVE;
  Request& r = it->second;
  int rc = OK;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    int* row = c->row((int)g, r.slot);
    for (int i = 0; i < r.n_entries[g]; ++i)
      if (row[i] >= 0 && !c->groups[g].pool.give_back(row[i])) rc = E_PAGE_NOT_HELD;
    std::fill(row, row + c->width, -1);
  }
  c->free_slots.push_back(r.slot);
  c->reqs.erase(it);
  return rc;
}

// the request's block table of group g (absolute page index -> page id or -1); returns its length
KF_HOST_API int kf_cache_table(void* h, int g, int64_t req, int* out, int cap) {
  Cache* c = (Cache*)h;
  auto it = c->reqs.find(req);
  if (it == c->reqs.end()) return -1;
  const int n = it->second.n_entries[g];
  const int* row = c->row(g, it->second.slot);
  for (int i = 0; i < n && i < cap; ++i) out[i] = row[i];
  return n;
}

// every page is either free or in exactly one table: OK or E_INCONSISTENT
KF_HOST_API int kf_cache_check(void* h) {
  Cache* c = (Cache*)h;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    Pool& pool = c->groups[g].pool;
    std::vector<char> seen(pool.n, 0);
    int n_seen = 0;
    for (auto& kv : c->reqs) {
      const Request& r = kv.second;
      const int* row = c->row((int)g, r.slot);
      for (int i = 0; i < c->width; ++i) {
        const int p = row[i];
        if (i >= r.n_entries[g]) { if (p != -1) return E_INCONSISTENT; continue; }
        if (p < 0) continue;
        if (p >= pool.n || seen[p] || !pool.held[p]) return E_INCONSISTENT;
        seen[p] = 1;
        ++n_seen;
      }
    }
    int n_held = 0;
    for (int p = 0; p < pool.n; ++p) n_held += pool.held[p];
    if (n_held != n_seen || n_held + pool.n_free() != pool.n) return E_INCONSISTENT;
  }
  return OK;
}

// ---- the step's integer block ------------------------------------------------------------------------------------------
// Sections, each starting on a 16-byte boundary, in this order (n = ints):
//   tokens T | positions T | row_req T | logit_rows max(n_out,1) | dec_rows T | pre_rows T | tile_row0, tile_nrows
//   (T/64 + B + 1 each) | wide_row0, wide_nrows (T/128 + B + 1 each) | req_row_start, req_n_rows, req_kv_len,
//   req_state_slot (B each) | logit_req max(n_out,1): the request whose logits row i of the output is, -1 for none |
//   one block table [B][width] per group.
// `info` receives: [0] total ints, [1] T, [2] B, [3] n_out, [4] width, [5] n_dec, [6] n_pre, [7] n_tiles, [8] n_wide,
// [9] max_kv, [10] max rows of a request, then the offset of every section in the order above (15 + n_groups).
// Layouts (steps of one layout can be replayed from one CUDA graph, because nothing but the block's contents changes):
//   bucket = 0, pre = 0   the entries as they are, tables as wide as the longest request needs;
//   bucket > 0, pre = 0   `bucket` single-row requests with full-width tables; rows beyond the real entries are padding
//                         (request -1) that every kernel skips;
//   bucket < 0, pre = 0   the entries as they are but with full-width tables and the longest context as max_kv;
//   pre > 0               a mixed step: `bucket` (>= 0) rows of single-token requests first, then `pre` rows for up to
//                         `pre_reqs` prompt portions; entries must come in that order; every count a kernel is launched
//                         with (rows, requests, tiles, wanted rows) is the bucket's, unused rows are padding, unused
//                         tiles have no rows, and a portion has one output row (its last row if wanted).
enum { SEC_TOKENS, SEC_POSITIONS, SEC_ROW_REQ, SEC_LOGIT_ROWS, SEC_DEC_ROWS, SEC_PRE_ROWS, SEC_TILE_ROW0, SEC_TILE_NROWS,
       SEC_WIDE_ROW0, SEC_WIDE_NROWS, SEC_REQ_ROW_START, SEC_REQ_N_ROWS, SEC_REQ_KV_LEN, SEC_REQ_STATE_SLOT, SEC_LOGIT_REQ,
       SEC_TABLE0 };
constexpr int INFO_FIXED = 11;

// Size of the block for a step, so that the caller can provide the buffer: returns total ints, fills info[0..].
KF_HOST_API int kf_step_layout(void* h, int n_entries, const int64_t* reqs, const int* n_tokens, const int* n_want, int bucket,
                               int pre, int pre_reqs, int* info) {
  Cache* c = (Cache*)h;
  const int G = (int)c->groups.size();
  int T = 0, n_out = 0, width = 1;
  int n_single = 0, n_multi = 0, multi_rows = 0;
  bool ordered = true;
  for (int e = 0; e < n_entries; ++e) {
    T += n_tokens[e];
    n_out += n_want[e];
    auto it = c->reqs.find(reqs[e]);
    if (it == c->reqs.end()) return -E_NOT_LIVE;
    width = std::max(width, ceil_div(it->second.length + n_tokens[e], c->page_size));
    if (n_tokens[e] == 1) { ++n_single; if (n_multi > 0) ordered = false; }
    else { ++n_multi; multi_rows += n_tokens[e]; }
  }
  int B = n_entries;
  if (pre > 0) {
    if (!ordered || bucket < 0 || n_single > bucket || multi_rows > pre || n_multi > pre_reqs) return -E_INCONSISTENT;
    T = bucket + pre; B = bucket + pre_reqs; n_out = B; width = c->max_pages;
  } else {
    if (bucket > 0) { T = B = n_out = bucket; width = c->max_pages; }
    if (bucket < 0) width = c->max_pages;
  }
  width = align4(width);
  const int sizes[SEC_TABLE0] = {T, T, T, std::max(n_out, 1), T, T, T / 64 + B + 1, T / 64 + B + 1, T / 128 + B + 1,
                                 T / 128 + B + 1, B, B, B, B, std::max(n_out, 1)};
  int o = 0;
  for (int s = 0; s < SEC_TABLE0; ++s) { info[INFO_FIXED + s] = o; o += align4(sizes[s]); }
  for (int g = 0; g < G; ++g) { info[INFO_FIXED + SEC_TABLE0 + g] = o; o += align4(B * width); }
  info[0] = o; info[1] = T; info[2] = B; info[3] = n_out; info[4] = width;
  return o;
}

// Fill `block` (info from kf_step_layout).  tokens / wants are the entries' lists laid end to end.
KF_HOST_API int kf_step_fill(void* h, int n_entries, const int64_t* reqs, const int* n_tokens, const int* tokens,
                             const int* n_want, const int* wants, int bucket, int pre, int pre_reqs, int* info, int* block) {
  Cache* c = (Cache*)h;
  const int G = (int)c->groups.size();
  const int total = info[0], T = info[1], B = info[2], width = info[4];
  const int* off = info + INFO_FIXED;
  memset(block, 0, (size_t)total * sizeof(int));
  const bool mixed = pre > 0;
  if (bucket > 0 || mixed) {
    for (int t = 0; t < T; ++t) block[off[SEC_ROW_REQ] + t] = -1;              // real rows are overwritten below
  }
  for (int i = 0; i < std::max(info[3], 1); ++i) block[off[SEC_LOGIT_REQ] + i] = -1;
  for (int g = 0; g < G; ++g) std::fill(block + off[SEC_TABLE0 + g], block + off[SEC_TABLE0 + g] + (size_t)B * width, -1);
  int r = 0, k = 0, tok_at = 0, want_at = 0, n_dec = 0, n_pre = 0, n_tiles = 0, n_wide = 0, max_kv = 0, max_rows = 0;
  int n_single = 0, n_multi = 0;
  for (int e = 0; e < n_entries; ++e) {
    auto it = c->reqs.find(reqs[e]);
    if (it == c->reqs.end()) return E_NOT_LIVE;
    const Request& rq = it->second;
    const int n = n_tokens[e], start = rq.length;
    int ri = e;                                                               // the entry's request index in the block
    if (mixed) {
      if (n == 1) { ri = n_single; r = n_single; ++n_single; }
      else { ri = bucket + n_multi; if (n_multi == 0) r = bucket; ++n_multi; }
    }
    for (int i = 0; i < n; ++i) {
      block[off[SEC_TOKENS] + r + i] = tokens[tok_at + i];
      block[off[SEC_POSITIONS] + r + i] = start + i;
      block[off[SEC_ROW_REQ] + r + i] = ri;
    }
    tok_at += n;
    block[off[SEC_REQ_ROW_START] + ri] = r;
    block[off[SEC_REQ_N_ROWS] + ri] = n;
    block[off[SEC_REQ_KV_LEN] + ri] = start + n;
    block[off[SEC_REQ_STATE_SLOT] + ri] = rq.slot;
    if (mixed) {                                                              // one output row per request slot of the bucket
      if (n_want[e] > 1 || (n_want[e] == 1 && wants[want_at] != n - 1)) return E_INCONSISTENT;
      if (n_want[e] == 1) { block[off[SEC_LOGIT_ROWS] + ri] = r + n - 1; block[off[SEC_LOGIT_REQ] + ri] = ri; }
    } else {
      for (int i = 0; i < n_want[e]; ++i) { block[off[SEC_LOGIT_ROWS] + k] = r + wants[want_at + i]; block[off[SEC_LOGIT_REQ] + k++] = ri; }
    }
    want_at += n_want[e];
    for (int g = 0; g < G; ++g)
      memcpy(block + off[SEC_TABLE0 + g] + (size_t)ri * width, c->row(g, rq.slot), (size_t)std::min(width, c->width) * sizeof(int));
    max_rows = std::max(max_rows, n);
    max_kv = std::max(max_kv, start + n);
    if (n == 1) {
      block[off[SEC_DEC_ROWS] + n_dec++] = r;
    } else {
      for (int i = 0; i < n; ++i) block[off[SEC_PRE_ROWS] + n_pre++] = r + i;
      for (int a = 0; a < n; a += 64) {                  // tiles of up to 64 consecutive rows of one request
        block[off[SEC_TILE_ROW0] + n_tiles] = r + a;
        block[off[SEC_TILE_NROWS] + n_tiles++] = std::min(64, n - a);
      }
      for (int a = 0; a < n; a += 128) {                 // and of up to 128 rows
        block[off[SEC_WIDE_ROW0] + n_wide] = r + a;
        block[off[SEC_WIDE_NROWS] + n_wide++] = std::min(128, n - a);
      }
    }
    r += n;
  }
  if (bucket > 0 && !mixed) {                             // every row of the bucket is a decode row that wants its logits
    n_dec = bucket;
    for (int t = 0; t < bucket; ++t) {
      block[off[SEC_DEC_ROWS] + t] = t;
      block[off[SEC_LOGIT_ROWS] + t] = t;
    }
    max_kv = c->max_context;                              // a captured graph's split plan must not depend on the step
  }
  if (mixed) {
    // counts are the bucket's: decode rows 0..bucket-1, prompt rows bucket..T-1, and as many tiles as `pre` rows in
    // `pre_reqs` portions can ever make; tiles beyond the real ones have no rows (their first row is the first prompt row)
    for (int t = 0; t < bucket; ++t) block[off[SEC_DEC_ROWS] + t] = t;
    for (int t = 0; t < pre; ++t) block[off[SEC_PRE_ROWS] + t] = bucket + t;
    const int tiles_fixed = pre / 64 + pre_reqs, wide_fixed = pre / 128 + pre_reqs;
    for (int t = n_tiles; t < tiles_fixed; ++t) { block[off[SEC_TILE_ROW0] + t] = bucket; block[off[SEC_TILE_NROWS] + t] = 0; }
    for (int t = n_wide; t < wide_fixed; ++t) { block[off[SEC_WIDE_ROW0] + t] = bucket; block[off[SEC_WIDE_NROWS] + t] = 0; }
    n_dec = bucket; n_pre = pre; n_tiles = tiles_fixed; n_wide = wide_fixed;
    max_kv = c->max_context;
    max_rows = std::max(max_rows, 2);
  }
  if (bucket < 0 && !mixed) max_kv = c->max_context;
  info[5] = n_dec; info[6] = n_pre; info[7] = n_tiles; info[8] = n_wide; info[9] = max_kv; info[10] = max_rows;
  return OK;
}


// ---- scheduler -------------------------------------------------------------------------------------------------------
// Plans one mixed step at a time over the requests it knows by 64-bit key (the keys of the cache manager above):
//   1. every decoding request gets its one token, oldest first; out of pages -> the request admitted last is preempted
//      (everything given back, to be recomputed from its prompt and its own output) and the request tries again;
//   2. the rest of the token budget goes to prompt portions of running requests, in order of admission;
//   3. waiting requests are admitted first come first served while a state slot and the pages of their whole pending
//      prompt are free; nothing is admitted in a step that had to preempt.
// A request that cannot fit with the whole pool to itself finishes with "no_fit".  The reference plans per pass in
// Rust too (crates/kf-serve/src/engine.rs:396-430 admit / prefill chunk / decode / retire); there prompt rows and decode
// rows never share a pass and a context that cannot fit is refused at plan time (crates/kf-engine/src/plan.rs:213-215).
// Token values stay with the caller: the scheduler needs counts only.
namespace {

enum { ST_WAITING = 0, ST_RUNNING = 1, ST_FINISHED = 2 };
enum { EV_ADMITTED = 1, EV_PREEMPTED = 2, EV_NO_FIT = 3 };
enum { FIN_NONE = 0, FIN_EOS = 1, FIN_LENGTH = 2, FIN_CONTEXT = 3 };

struct SReq {
  int64_t key = 0;
  int prompt_len = 0, out_len = 0, n_cached = 0, max_tokens = 0, status = ST_WAITING, n_preempted = 0;
};
struct SPortion {
  int64_t key;
  int start, n, wants;
};
struct Sched {
  Cache* cache = nullptr;
  int max_batch_tokens = 0, max_requests = 0;
  // 1: a step's decode rows count towards the budget as the next power of two (the step function pads them to that
  // when it replays steps from captured graphs), so that decode rows and prompt rows together stay within the budget
  int pad_decode_rows = 0;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;                      // in order of admission
  std::unordered_map<int64_t, SReq> reqs;
  long n_preemptions = 0;
  std::vector<SPortion> plan;
  std::vector<int64_t> events;                       // (code, key, argument) triples of the last schedule()

  int G() const { return (int)cache->groups.size(); }
  static int n_pending(const SReq& r) { return r.prompt_len + r.out_len - r.n_cached; }
  static bool decoding(const SReq& r) { return r.status == ST_RUNNING && n_pending(r) == 1 && r.out_len > 0; }
  std::vector<int> free_pages() const {
    std::vector<int> f(cache->groups.size());
    for (size_t g = 0; g < f.size(); ++g) f[g] = cache->groups[g].pool.n_free();
    return f;
  }
  std::vector<int> pages_needed(int64_t key, int n) const {
    std::vector<int> out(cache->groups.size(), 0);
    kf_cache_pages_needed(cache, key, n, out.data());
    return out;
  }
  static bool covers(const std::vector<int>& need, const std::vector<int>& free) {
    for (size_t g = 0; g < need.size(); ++g)
      if (need[g] > free[g]) return false;
    return true;
  }
  static bool take(const std::vector<int>& need, std::vector<int>& free) {
    if (!covers(need, free)) return false;
    for (size_t g = 0; g < need.size(); ++g) free[g] -= need[g];
    return true;
  }
  void event(int code, int64_t key, int64_t arg) { events.push_back(code); events.push_back(key); events.push_back(arg); }

  bool fits_at_all(const SReq& r) const {
    int total = r.prompt_len + r.max_tokens;
    if (total > cache->max_context) total = cache->max_context;
    if (r.prompt_len >= cache->max_context) return false;
    const int P = cache->page_size;
    for (const Group& g : cache->groups) {
      int need = total;
      if (g.window >= 0) need = std::min(total, g.window + P + std::min(max_batch_tokens, r.prompt_len));
      if (ceil_div(need, P) > g.pool.n) return false;
    }
    return true;
  }
  std::vector<int> admission_pages(const SReq& r) const {
    const int P = cache->page_size;
    std::vector<int> out;
    for (const Group& g : cache->groups) {
      int need = n_pending(r);
      if (g.window >= 0) need = std::min(need, g.window + P + std::min(max_batch_tokens, n_pending(r)));
      out.push_back(ceil_div(need, P));
    }
    return out;
  }
  // the most recently admitted running request other than `keep` goes back to the front of the waiting queue
  int64_t preempt_last(int64_t keep) {
    for (int i = (int)running.size() - 1; i >= 0; --i) {
      const int64_t key = running[i];
      if (key == keep) continue;
      running.erase(running.begin() + i);
      kf_cache_release(cache, key);
      SReq& r = reqs[key];
      r.status = ST_WAITING;
      r.n_cached = 0;
      r.n_preempted += 1;
      n_preemptions += 1;
      waiting.push_front(key);
      event(EV_PREEMPTED, key, 0);
      return key;
    }
    return 0;
  }
  void finish(int64_t key) {
    SReq& r = reqs[key];
    auto it = std::find(running.begin(), running.end(), key);
    if (it != running.end()) {
      running.erase(it);
      kf_cache_release(cache, key);
    } else {
      auto iw = std::find(waiting.begin(), waiting.end(), key);
      if (iw != waiting.end()) waiting.erase(iw);
    }
    r.status = ST_FINISHED;
  }
  // the most tokens (<= n_max) of a running request whose pages the free counts still cover
  int largest_portion(int64_t key, int n_max, const std::vector<int>& free) const {
    const int P = cache->page_size;
    int n = n_max;
    while (n > 0) {
      if (covers(pages_needed(key, n), free)) return n;
      const int have = kf_cache_length(cache, key);
      n = std::min(n - 1, ((have + n - 1) / P) * P - have);     // the largest count that needs one page fewer
    }
    return 0;
  }
  bool planned(int64_t key) const {
    for (const SPortion& p : plan)
      if (p.key == key) return true;
    return false;
  }

  void schedule() {
    events.clear();
    for (;;) {
      plan.clear();
      std::vector<int> free = free_pages();
      int budget = max_batch_tokens;
      bool preempted = false;
      // 1. decoding requests
      size_t i = 0;
      while (i < running.size()) {
        const int64_t key = running[i];
        const SReq& r = reqs[key];
        if (!decoding(r)) { ++i; continue; }
        if (budget <= 0) break;
        if (take(pages_needed(key, 1), free)) {
          plan.push_back({key, r.n_cached, 1, 1});
          --budget;
          ++i;
          continue;
        }
        const int64_t victim = preempt_last(key);
        if (victim == 0) {                                       // alone and still no page
          finish(key);
          event(EV_NO_FIT, key, 0);
          continue;
        }
        preempted = true;
        for (size_t k = 0; k < plan.size();) {                   // it had been planned in this very call: undo
          if (plan[k].key == victim) { budget += plan[k].n; plan.erase(plan.begin() + k); } else ++k;
        }
        free = free_pages();
        for (const SPortion& p : plan) {                         // re-apply what is already planned
          const std::vector<int> need = pages_needed(p.key, p.n);
          for (size_t g = 0; g < need.size(); ++g) free[g] -= need[g];
        }
        i = (size_t)(std::find(running.begin(), running.end(), key) - running.begin());
      }
      if (pad_decode_rows && !plan.empty()) {
        int padded = 1;
        while (padded < (int)plan.size()) padded *= 2;
        // (only while the padded rows leave at least half of the budget: prompts must not starve behind many decoders)
        if (2 * padded <= max_batch_tokens) budget = std::min(budget, max_batch_tokens - padded);
      }
      // 2. prompt portions of running requests
      for (const int64_t key : running) {
        if (budget <= 0) break;
        const SReq& r = reqs[key];
        if (decoding(r) || n_pending(r) == 0 || planned(key)) continue;
        const int n = largest_portion(key, std::min(budget, n_pending(r)), free);
        if (n <= 0) continue;
        take(pages_needed(key, n), free);
        plan.push_back({key, r.n_cached, n, n == n_pending(r) ? 1 : 0});
        budget -= n;
      }
      // 3. admission
      while (!waiting.empty() && budget > 0 && (int)running.size() < max_requests) {
        const int64_t key = waiting.front();
        SReq& r = reqs[key];
        if (!fits_at_all(r)) {
          waiting.pop_front();
          finish(key);
          event(EV_NO_FIT, key, 0);
          continue;
        }
        if (preempted || !covers(admission_pages(r), free)) break;
        const int n = std::min(budget, n_pending(r));
        waiting.pop_front();
        const int slot = kf_cache_add_request(cache, key);
        if (slot < 0) { waiting.push_front(key); break; }        // no state slot after all
        r.status = ST_RUNNING;
        running.push_back(key);
        event(EV_ADMITTED, key, slot);
        take(pages_needed(key, n), free);
        plan.push_back({key, 0, n, n == n_pending(r) ? 1 : 0});
        budget -= n;
      }
      if (plan.empty() && !running.empty()) {
        bool any_decoding = false;
        for (const int64_t key : running) any_decoding = any_decoding || decoding(reqs[key]);
        if (!any_decoding) {
          // every running request is mid-prompt and none can get a page: free the youngest so that the oldest moves
          if (running.size() > 1) {
            preempt_last(running[0]);
            continue;
          }
          const int64_t key = running[0];
          finish(key);
          event(EV_NO_FIT, key, 0);
        }
      }
      return;
    }
  }
};

}  // namespace

KF_HOST_API void* kf_sched_create(void* cache, int max_batch_tokens, int max_requests) {
  Sched* s = new Sched();
  s->cache = (Cache*)cache;
  s->max_batch_tokens = max_batch_tokens;
  s->max_requests = max_requests;
  return s;
}
KF_HOST_API void kf_sched_destroy(void* h) { delete (Sched*)h; }
KF_HOST_API void kf_sched_pad_decode_rows(void* h, int on) { ((Sched*)h)->pad_decode_rows = on ? 1 : 0; }

KF_HOST_API int kf_sched_add(void* h, int64_t key, int prompt_len, int out_len, int max_tokens) {
  Sched* s = (Sched*)h;
  if (s->reqs.count(key)) return E_ALREADY_LIVE;
  SReq r;
  r.key = key; r.prompt_len = prompt_len; r.out_len = out_len; r.max_tokens = max_tokens;
  s->reqs.emplace(key, r);
  s->waiting.push_back(key);
  return OK;
}
// a request that already holds its cache (admitted and filled by the caller): joins the running list as it is
KF_HOST_API int kf_sched_adopt(void* h, int64_t key, int prompt_len, int out_len, int n_cached, int max_tokens) {
  Sched* s = (Sched*)h;
  if (s->reqs.count(key) || !s->cache->reqs.count(key)) return E_NOT_LIVE;
  SReq r;
  r.key = key; r.prompt_len = prompt_len; r.out_len = out_len; r.n_cached = n_cached; r.max_tokens = max_tokens;
  r.status = ST_RUNNING;
  s->reqs.emplace(key, r);
  s->running.push_back(key);
  return OK;
}
KF_HOST_API void kf_sched_forget(void* h, int64_t key) { ((Sched*)h)->reqs.erase(key); }

// Plans a step.  portions: up to cap_portions x 4 values (key, start, n, wants logits); events: up to cap_events x 3
// values (code 1 admitted / 2 preempted / 3 finished with no_fit, key, state slot for admissions).  counts[0], [1].
KF_HOST_API int kf_sched_schedule(void* h, int64_t* portions, int cap_portions, int64_t* events, int cap_events, int* counts) {
  Sched* s = (Sched*)h;
  s->schedule();
  const int np = (int)s->plan.size(), ne = (int)s->events.size() / 3;
  counts[0] = np;
  counts[1] = ne;
  if (np > cap_portions || ne > cap_events) return E_INCONSISTENT;
  for (int i = 0; i < np; ++i) {
    portions[4 * i] = s->plan[i].key; portions[4 * i + 1] = s->plan[i].start;
    portions[4 * i + 2] = s->plan[i].n; portions[4 * i + 3] = s->plan[i].wants;
  }
  memcpy(events, s->events.data(), s->events.size() * sizeof(int64_t));
  return OK;
}
KF_HOST_API int kf_sched_advance(void* h, int64_t key, int n) {
  Sched* s = (Sched*)h;
  auto it = s->reqs.find(key);
  if (it == s->reqs.end()) return E_NOT_LIVE;
  it->second.n_cached += n;
  return OK;
}
// A sampled token: returns 0, or the finish reason (1 eos, 2 length, 3 context) after finishing and freeing the request.
KF_HOST_API int kf_sched_on_token(void* h, int64_t key, int is_eos) {
  Sched* s = (Sched*)h;
  auto it = s->reqs.find(key);
  if (it == s->reqs.end()) return -E_NOT_LIVE;
  SReq& r = it->second;
  r.out_len += 1;
  int reason = FIN_NONE;
  if (is_eos) reason = FIN_EOS;
  else if (r.out_len >= r.max_tokens) reason = FIN_LENGTH;
  else if (r.prompt_len + r.out_len >= s->cache->max_context) reason = FIN_CONTEXT;
  if (reason != FIN_NONE) s->finish(key);
  return reason;
}
KF_HOST_API int kf_sched_finish(void* h, int64_t key) {
  Sched* s = (Sched*)h;
  if (!s->reqs.count(key)) return E_NOT_LIVE;
  s->finish(key);
  return OK;
}
KF_HOST_API int64_t kf_sched_preempt_last(void* h, int64_t keep) {
  Sched* s = (Sched*)h;
  s->events.clear();
  return s->preempt_last(keep);
}
KF_HOST_API long kf_sched_n_preemptions(void* h) { return ((Sched*)h)->n_preemptions; }
KF_HOST_API int kf_sched_counts(void* h, int* n_waiting, int* n_running) {
  Sched* s = (Sched*)h;
  *n_waiting = (int)s->waiting.size();
  *n_running = (int)s->running.size();
  return OK;
}
// the queues in order: waiting first, then running (caps as given by kf_sched_counts)
KF_HOST_API int kf_sched_lists(void* h, int64_t* waiting, int64_t* running) {
  Sched* s = (Sched*)h;
  std::copy(s->waiting.begin(), s->waiting.end(), waiting);
  std::copy(s->running.begin(), s->running.end(), running);
  return OK;
}
// (status, n_cached, n_preempted, out_len) of a request
KF_HOST_API int kf_sched_state(void* h, int64_t key, int* out) {
  Sched* s = (Sched*)h;
  auto it = s->reqs.find(key);
  if (it == s->reqs.end()) return E_NOT_LIVE;
  out[0] = it->second.status; out[1] = it->second.n_cached; out[2] = it->second.n_preempted; out[3] = it->second.out_len;
  return OK;
}
