// Host-side runtime of the engine, in C++: the page pools and block tables of the cache manager, and the builder of
// the integer block every step sends to the device.  The Python classes of kungfu_b200/cache and
// kungfu_b200/engine/step.py are thin wrappers over the functions exported here (C ABI, called through ctypes).
//
// The reference keeps the corresponding state in Rust (per-slot ring caches sized at plan time,
// crates/kf-core/src/plan.rs:59-64 and crates/kf-backend-cuda/src/exec.rs:1466-1498; per-pass integer inputs staged
// in one pinned buffer, exec.rs:2922-2944).  Here the unit is a page, a request owns a block table per cache group,
// and a windowed group gives pages back as soon as no later query can reach them.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <unordered_map>
#include <vector>

#define KF_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

struct Pool {
  int n = 0;
  std::vector<int> free_list;           // pop_back hands out low ids first
  std::vector<char> held;
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
//   req_state_slot (B each) | one block table [B][width] per group.
// `info` receives: [0] total ints, [1] T, [2] B, [3] n_out, [4] width, [5] n_dec, [6] n_pre, [7] n_tiles, [8] n_wide,
// [9] max_kv, [10] max rows of a request, then the offset of every section in the order above (14 + n_groups).
// With bucket > 0 the layout is that of `bucket` single-row requests with full-width tables; rows beyond the real
// entries are padding (request -1).
enum { SEC_TOKENS, SEC_POSITIONS, SEC_ROW_REQ, SEC_LOGIT_ROWS, SEC_DEC_ROWS, SEC_PRE_ROWS, SEC_TILE_ROW0, SEC_TILE_NROWS,
       SEC_WIDE_ROW0, SEC_WIDE_NROWS, SEC_REQ_ROW_START, SEC_REQ_N_ROWS, SEC_REQ_KV_LEN, SEC_REQ_STATE_SLOT, SEC_TABLE0 };
constexpr int INFO_FIXED = 11;

// Size of the block for a step, so that the caller can provide the buffer: returns total ints, fills info[0..].
KF_HOST_API int kf_step_layout(void* h, int n_entries, const int64_t* reqs, const int* n_tokens, const int* n_want, int bucket,
                               int* info) {
  Cache* c = (Cache*)h;
  const int G = (int)c->groups.size();
  int T = 0, n_out = 0, width = 1;
  for (int e = 0; e < n_entries; ++e) {
    T += n_tokens[e];
    n_out += n_want[e];
    auto it = c->reqs.find(reqs[e]);
    if (it == c->reqs.end()) return -E_NOT_LIVE;
    width = std::max(width, ceil_div(it->second.length + n_tokens[e], c->page_size));
  }
  int B = n_entries;
  if (bucket > 0) { T = B = n_out = bucket; width = c->max_pages; }
  width = align4(width);
  const int sizes[SEC_TABLE0] = {T, T, T, std::max(n_out, 1), T, T, T / 64 + B + 1, T / 64 + B + 1, T / 128 + B + 1,
                                 T / 128 + B + 1, B, B, B, B};
  int o = 0;
  for (int s = 0; s < SEC_TABLE0; ++s) { info[INFO_FIXED + s] = o; o += align4(sizes[s]); }
  for (int g = 0; g < G; ++g) { info[INFO_FIXED + SEC_TABLE0 + g] = o; o += align4(B * width); }
  info[0] = o; info[1] = T; info[2] = B; info[3] = n_out; info[4] = width;
  return o;
}

// Fill `block` (info from kf_step_layout).  tokens / wants are the entries' lists laid end to end.
KF_HOST_API int kf_step_fill(void* h, int n_entries, const int64_t* reqs, const int* n_tokens, const int* tokens,
                             const int* n_want, const int* wants, int bucket, int* info, int* block) {
  Cache* c = (Cache*)h;
  const int G = (int)c->groups.size();
  const int total = info[0], T = info[1], B = info[2], width = info[4];
  const int* off = info + INFO_FIXED;
  memset(block, 0, (size_t)total * sizeof(int));
  if (bucket > 0) {
    for (int t = n_entries; t < T; ++t) block[off[SEC_ROW_REQ] + t] = -1;
  }
  for (int g = 0; g < G; ++g) std::fill(block + off[SEC_TABLE0 + g], block + off[SEC_TABLE0 + g] + (size_t)B * width, -1);
  int r = 0, k = 0, tok_at = 0, want_at = 0, n_dec = 0, n_pre = 0, n_tiles = 0, n_wide = 0, max_kv = 0, max_rows = 0;
  for (int e = 0; e < n_entries; ++e) {
    auto it = c->reqs.find(reqs[e]);
    if (it == c->reqs.end()) return E_NOT_LIVE;
    const Request& rq = it->second;
    const int n = n_tokens[e], start = rq.length;
    for (int i = 0; i < n; ++i) {
      block[off[SEC_TOKENS] + r + i] = tokens[tok_at + i];
      block[off[SEC_POSITIONS] + r + i] = start + i;
      block[off[SEC_ROW_REQ] + r + i] = e;
    }
    tok_at += n;
    block[off[SEC_REQ_ROW_START] + e] = r;
    block[off[SEC_REQ_N_ROWS] + e] = n;
    block[off[SEC_REQ_KV_LEN] + e] = start + n;
    block[off[SEC_REQ_STATE_SLOT] + e] = rq.slot;
    for (int i = 0; i < n_want[e]; ++i) block[off[SEC_LOGIT_ROWS] + k++] = r + wants[want_at + i];
    want_at += n_want[e];
    for (int g = 0; g < G; ++g)
      memcpy(block + off[SEC_TABLE0 + g] + (size_t)e * width, c->row(g, rq.slot), (size_t)std::min(width, c->width) * sizeof(int));
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
  if (bucket > 0) {                                       // every row of the bucket is a decode row that wants its logits
    n_dec = bucket;
    for (int t = 0; t < bucket; ++t) {
      block[off[SEC_DEC_ROWS] + t] = t;
      block[off[SEC_LOGIT_ROWS] + t] = t;
    }
    max_kv = c->max_context;                              // a captured graph's split plan must not depend on the step
  }
  info[5] = n_dec; info[6] = n_pre; info[7] = n_tiles; info[8] = n_wide; info[9] = max_kv; info[10] = max_rows;
  return OK;
}
