// Paged KV bookkeeping on the host: a ref-counted page pool plus per-sequence page lists with
// transactional length publication, prefix forking (shared full pages + private copy of the tail
// page), truncation for speculative rollback, and block-table export.
//
// This is the paged analogue of the reference's VMM KV planes: grow-on-append
// (native/hip/src/public_runtime.hip.cpp:578-614), read-only page sharing with a copy-on-write tail
// (:654-809) and published_length / rewind (:863-989, include/sllm/hip.h:1569).  Device memory itself
// is owned by the caller (one tensor per layer); this module only hands out page indices.
#include "host_api.h"

#include <algorithm>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

struct Seq {
  std::vector<int> pages;
  long long published = 0;   // tokens visible to readers
  long long reserved = 0;    // tokens with storage (>= published while a step is in flight)
};

struct Pool {
  int page_size = 16;
  std::vector<int> free_list;   // LIFO
  std::vector<int> refcnt;
  std::unordered_map<int, Seq> seqs;
  int next_seq = 1;
  long long high_water = 0;
  std::mutex mu;
  int fail_after = -1;  // fault injection: allocation number that fails (-1 = never)
  long long alloc_calls = 0;
};

std::mutex g_mu;
std::unordered_map<int, Pool*> g_pools;
int g_next_pool = 1;

Pool* find_pool(int h) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_pools.find(h);
  return it == g_pools.end() ? nullptr : it->second;
}

bool take_pages(Pool* p, int n, std::vector<int>* out) {
  ++p->alloc_calls;
  if (p->fail_after >= 0 && p->alloc_calls > p->fail_after) return false;
  if (static_cast<int>(p->free_list.size()) < n) return false;
  for (int i = 0; i < n; ++i) {
    const int pg = p->free_list.back();
    p->free_list.pop_back();
    p->refcnt[pg] = 1;
    out->push_back(pg);
  }
  const long long used = static_cast<long long>(p->refcnt.size()) - static_cast<long long>(p->free_list.size());
  p->high_water = std::max(p->high_water, used);
  return true;
}

void drop_page(Pool* p, int pg) {
  if (pg < 0 || pg >= static_cast<int>(p->refcnt.size()) || p->refcnt[pg] <= 0) return;
  if (--p->refcnt[pg] == 0) p->free_list.push_back(pg);
}

}  // namespace

SLLM_HOST_EXPORT int sllm_kv_pool_create(int num_pages, int page_size) {
  if (num_pages <= 0 || page_size <= 0) return -SLLM_HOST_INVALID;
  Pool* p = new Pool();
  p->page_size = page_size;
  p->refcnt.assign(num_pages, 0);
  p->free_list.reserve(num_pages);
  for (int i = num_pages - 1; i >= 0; --i) p->free_list.push_back(i);  // page 0 is handed out first
  std::lock_guard<std::mutex> g(g_mu);
  const int h = g_next_pool++;
  g_pools[h] = p;
  return h;
}

SLLM_HOST_EXPORT int sllm_kv_pool_destroy(int h) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_pools.find(h);
  if (it == g_pools.end()) return SLLM_HOST_NOT_FOUND;
  delete it->second;
  g_pools.erase(it);
  return SLLM_HOST_OK;
}

SLLM_HOST_EXPORT int sllm_kv_pool_stats(int h, long long* out4) {
  Pool* p = find_pool(h);
  if (!p || !out4) return SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  out4[0] = static_cast<long long>(p->refcnt.size());
  out4[1] = static_cast<long long>(p->free_list.size());
  out4[2] = p->high_water;
  out4[3] = static_cast<long long>(p->seqs.size());
  return SLLM_HOST_OK;
}

SLLM_HOST_EXPORT int sllm_kv_pool_inject_alloc_failure(int h, int fail_after_calls) {
  Pool* p = find_pool(h);
  if (!p) return SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  p->fail_after = fail_after_calls < 0 ? -1 : static_cast<int>(p->alloc_calls) + fail_after_calls;
  return SLLM_HOST_OK;
}

SLLM_HOST_EXPORT int sllm_kv_page_refcount(int h, int page) {
  Pool* p = find_pool(h);
  if (!p) return -SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  if (page < 0 || page >= static_cast<int>(p->refcnt.size())) return -SLLM_HOST_INVALID;
  return p->refcnt[page];
}

SLLM_HOST_EXPORT int sllm_kv_seq_new(int h) {
  Pool* p = find_pool(h);
  if (!p) return -SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  const int id = p->next_seq++;
  p->seqs[id] = Seq();
  return id;
}

SLLM_HOST_EXPORT int sllm_kv_seq_free(int h, int seq) {
  Pool* p = find_pool(h);
  if (!p) return SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return SLLM_HOST_NOT_FOUND;
  for (int pg : it->second.pages) drop_page(p, pg);
  p->seqs.erase(it);
  return SLLM_HOST_OK;
}

// Make sure storage exists for `new_len` tokens.  All-or-nothing: on failure nothing changes.
SLLM_HOST_EXPORT int sllm_kv_seq_reserve(int h, int seq, long long new_len) {
  Pool* p = find_pool(h);
  if (!p) return SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return SLLM_HOST_NOT_FOUND;
  Seq& s = it->second;
  if (new_len < s.published) return SLLM_HOST_INVALID;
  const long long need = (new_len + p->page_size - 1) / p->page_size;
  const long long have = static_cast<long long>(s.pages.size());
  if (need > have) {
    std::vector<int> got;
    if (!take_pages(p, static_cast<int>(need - have), &got)) {
      for (int pg : got) drop_page(p, pg);
      return SLLM_HOST_OUT_OF_PAGES;
    }
    s.pages.insert(s.pages.end(), got.begin(), got.end());
  }
  s.reserved = std::max(s.reserved, new_len);
  return SLLM_HOST_OK;
}

// Publish a length after the step that wrote the tokens has completed.
SLLM_HOST_EXPORT int sllm_kv_seq_commit(int h, int seq, long long new_len) {
  Pool* p = find_pool(h);
  if (!p) return SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return SLLM_HOST_NOT_FOUND;
  Seq& s = it->second;
  if (new_len > static_cast<long long>(s.pages.size()) * p->page_size || new_len < 0) return SLLM_HOST_INVALID;
  s.published = new_len;
  if (s.reserved < new_len) s.reserved = new_len;
  return SLLM_HOST_OK;
}

// Drop tokens beyond `len` (speculative rollback, cancelled append) and free pages no longer needed.
SLLM_HOST_EXPORT int sllm_kv_seq_truncate(int h, int seq, long long len) {
  Pool* p = find_pool(h);
  if (!p) return SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return SLLM_HOST_NOT_FOUND;
  Seq& s = it->second;
  if (len < 0) return SLLM_HOST_INVALID;
  const long long keep = (len + p->page_size - 1) / p->page_size;
  while (static_cast<long long>(s.pages.size()) > keep) {
    drop_page(p, s.pages.back());
    s.pages.pop_back();
  }
  s.published = std::min(s.published, len);
  s.reserved = std::min(s.reserved, len);
  return SLLM_HOST_OK;
}

SLLM_HOST_EXPORT long long sllm_kv_seq_length(int h, int seq) {
  Pool* p = find_pool(h);
  if (!p) return -SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  return it == p->seqs.end() ? -SLLM_HOST_NOT_FOUND : it->second.published;
}

SLLM_HOST_EXPORT int sllm_kv_seq_pages(int h, int seq, int* out, int cap) {
  Pool* p = find_pool(h);
  if (!p) return -SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return -SLLM_HOST_NOT_FOUND;
  const int n = static_cast<int>(it->second.pages.size());
  for (int i = 0; i < n && i < cap; ++i) out[i] = it->second.pages[i];
  return n;
}

// New sequence that shares the first `prefix_len` tokens of `seq`.  Full pages are shared (ref-count
// bump, read-only by convention); a partially filled last page is replaced by a private page and the
// caller is told to copy it: copy_pair[0] = source page, copy_pair[1] = destination page, or -1/-1.
SLLM_HOST_EXPORT int sllm_kv_seq_fork(int h, int seq, long long prefix_len, int* copy_pair) {
  Pool* p = find_pool(h);
  if (!p) return -SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return -SLLM_HOST_NOT_FOUND;
  const Seq& src = it->second;
  if (prefix_len < 0 || prefix_len > src.published) return -SLLM_HOST_INVALID;
  const long long full = prefix_len / p->page_size;
  const bool tail = (prefix_len % p->page_size) != 0;
  Seq child;
  std::vector<int> got;
  if (tail && !take_pages(p, 1, &got)) return -SLLM_HOST_OUT_OF_PAGES;
  for (long long i = 0; i < full; ++i) {
    ++p->refcnt[src.pages[i]];
    child.pages.push_back(src.pages[i]);
  }
  if (copy_pair) {
    copy_pair[0] = -1;
    copy_pair[1] = -1;
  }
  if (tail) {
    child.pages.push_back(got[0]);
    if (copy_pair) {
      copy_pair[0] = src.pages[full];
      copy_pair[1] = got[0];
    }
  }
  child.published = prefix_len;
  child.reserved = prefix_len;
  const int id = p->next_seq++;
  p->seqs[id] = child;
  return id;
}

// Before appending into a page shared with another sequence, give this sequence a private copy.
// Returns 1 and fills copy_pair when a device copy is required, 0 when the tail is already private.
SLLM_HOST_EXPORT int sllm_kv_seq_make_tail_private(int h, int seq, int* copy_pair) {
  Pool* p = find_pool(h);
  if (!p) return -SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->seqs.find(seq);
  if (it == p->seqs.end()) return -SLLM_HOST_NOT_FOUND;
  Seq& s = it->second;
  if (s.pages.empty() || (s.published % p->page_size) == 0) return 0;
  const long long idx = s.published / p->page_size;
  const int pg = s.pages[idx];
  if (p->refcnt[pg] <= 1) return 0;
  std::vector<int> got;
  if (!take_pages(p, 1, &got)) return -SLLM_HOST_OUT_OF_PAGES;
  --p->refcnt[pg];
  s.pages[idx] = got[0];
  if (copy_pair) {
    copy_pair[0] = pg;
    copy_pair[1] = got[0];
  }
  return 1;
}

// Rows of the block table for `n` sequences; unused entries are set to 0 (a valid page index, never
// read because kv_lens bounds every access).
SLLM_HOST_EXPORT int sllm_kv_fill_block_table(int h, const int* seqs, int n, int* table, int max_blocks) {
  Pool* p = find_pool(h);
  if (!p) return SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> g(p->mu);
  for (int i = 0; i < n; ++i) {
    auto it = p->seqs.find(seqs[i]);
    if (it == p->seqs.end()) return SLLM_HOST_NOT_FOUND;
    const std::vector<int>& pg = it->second.pages;
    if (static_cast<int>(pg.size()) > max_blocks) return SLLM_HOST_LIMIT;
    int* row = table + static_cast<long long>(i) * max_blocks;
    std::copy(pg.begin(), pg.end(), row);
    std::fill(row + pg.size(), row + max_blocks, 0);
  }
  return SLLM_HOST_OK;
}
