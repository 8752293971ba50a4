// The host-side books of the paged cache and the builder of a step's index arrays, in C++
// behind a C interface (no device code: the file goes through the same build as the kernels).
//
// What the books hold: per group of layers a pool of reference-counted pages with a LIFO free
// stack (a page that was just given back is the next one handed out; the reference reuses
// returned pages first, crates/sglang-srt/src/cache.rs:464-466); per live request its length,
// its state slot and one block table per group (logical page -> page id, -1 once a window has
// passed the page and it was given back).  An allocation that cannot be met consumes nothing
// (cache.rs:417-422).  State slots are a free list of ids (crates/sglang-srt/src/recurrent_state.rs:23-101).
//
// Every function returns 0 or a positive result, or a negative code: -1 bad argument, -2 out of
// pages (nothing was taken), -3 out of request or state slots, -4 misuse (double free, a request
// that has ended, ...).  srb_last_error() gives the text of the last failure of the calling thread.
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <algorithm>
#include <map>
#include <memory>
#include <vector>

namespace {

thread_local char error_text[256] = "";

int fail(int code, const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(error_text, sizeof(error_text), format, args);
  va_end(args);
  return code;
}

struct Group {
  int window = 0;                  // 0: every key is kept
  int num_pages = 0;
  std::vector<int> refs;
  std::vector<int> free_stack;     // back() is handed out next
};

struct Request {
  bool live = false;
  int length = 0;
  int state_slot = -1;
  std::vector<std::vector<int>> tables;   // one per group
};

struct Core {
  int page_size = 1;
  std::vector<Group> groups;
  std::vector<Request> requests;
  std::vector<int> free_requests;
  std::vector<int> free_states;
  std::vector<char> state_used;
  int live_count = 0;
};

bool good_request(const Core* core, int r) { return core && r >= 0 && r < (int)core->requests.size() && core->requests[r].live; }
bool good_group(const Core* core, int g) { return core && g >= 0 && g < (int)core->groups.size(); }

int release_page(Group& group, int page) {
  if (page < 0 || page >= group.num_pages || group.refs[page] <= 0)
    return fail(-4, "page %d is freed twice or was never handed out", page);
  if (--group.refs[page] == 0) {
    group.free_stack.push_back(page);
    return 1;
  }
  return 0;
}

int pages_for(const Core* core, int tokens) { return (tokens + core->page_size - 1) / core->page_size; }

}  // namespace

extern "C" {

const char* srb_last_error() { return error_text; }

// windows[g] = 0 for a group that keeps every key; num_pages[g] pages per group
void* hc_create(int page_size, int num_groups, const int* windows, const int* num_pages, int max_requests) {
  if (page_size <= 0 || num_groups < 0 || max_requests <= 0) return nullptr;
  Core* core = new Core();
  core->page_size = page_size;
  core->groups.resize(num_groups);
  for (int g = 0; g < num_groups; ++g) {
    Group& group = core->groups[g];
    if (num_pages[g] <= 0) {
      delete core;
      return nullptr;
    }
    group.window = windows[g];
    group.num_pages = num_pages[g];
    group.refs.assign(num_pages[g], 0);
    group.free_stack.resize(num_pages[g]);
    for (int p = 0; p < num_pages[g]; ++p) group.free_stack[p] = num_pages[g] - 1 - p;   // 0, 1, 2, ... come out in turn
  }
  core->requests.resize(max_requests);
  core->state_used.assign(max_requests, 0);
  for (int r = max_requests - 1; r >= 0; --r) {
    core->free_requests.push_back(r);
    core->free_states.push_back(r);
  }
  return core;
}

void hc_destroy(void* handle) { delete static_cast<Core*>(handle); }

// ---- pages of a group (also used by the prefix tree, which holds references of its own)
int hc_free_count(void* handle, int g) {
  Core* core = static_cast<Core*>(handle);
  if (!good_group(core, g)) return fail(-1, "no such group %d", g);
  return (int)core->groups[g].free_stack.size();
}

int hc_allocate(void* handle, int g, int count, int* out) {
  Core* core = static_cast<Core*>(handle);
  if (!good_group(core, g) || count < 0) return fail(-1, "no such group %d, or a negative count", g);
  Group& group = core->groups[g];
  if (count > (int)group.free_stack.size())
    return fail(-2, "%d pages requested, %d free", count, (int)group.free_stack.size());
  for (int i = 0; i < count; ++i) {
    out[i] = group.free_stack.back();
    group.free_stack.pop_back();
    group.refs[out[i]] = 1;
  }
  return count;
}

int hc_retain(void* handle, int g, int page) {
  Core* core = static_cast<Core*>(handle);
  if (!good_group(core, g)) return fail(-1, "no such group %d", g);
  Group& group = core->groups[g];
  if (page < 0 || page >= group.num_pages || group.refs[page] <= 0)
    return fail(-4, "page %d is free and cannot be shared", page);
  return ++group.refs[page];
}

int hc_release(void* handle, int g, int page) {   // 1 if the page went back to the free stack
  Core* core = static_cast<Core*>(handle);
  if (!good_group(core, g)) return fail(-1, "no such group %d", g);
  return release_page(core->groups[g], page);
}

int hc_refcount(void* handle, int g, int page) {
  Core* core = static_cast<Core*>(handle);
  if (!good_group(core, g) || page < 0 || page >= core->groups[g].num_pages) return fail(-1, "no such page %d", page);
  return core->groups[g].refs[page];
}

int hc_free_list(void* handle, int g, int* out, int capacity) {
  Core* core = static_cast<Core*>(handle);
  if (!good_group(core, g)) return fail(-1, "no such group %d", g);
  const std::vector<int>& stack = core->groups[g].free_stack;
  for (int i = 0; i < (int)stack.size() && i < capacity; ++i) out[i] = stack[i];
  return (int)stack.size();
}

// ---- requests
int hc_open(void* handle) {
  Core* core = static_cast<Core*>(handle);
  if (!core) return fail(-1, "no core");
  if (core->free_requests.empty() || core->free_states.empty())
    return fail(-3, "%d requests are live already", core->live_count);
  const int r = core->free_requests.back();
  core->free_requests.pop_back();
  Request& request = core->requests[r];
  request.live = true;
  request.length = 0;
  request.state_slot = core->free_states.back();
  core->free_states.pop_back();
  core->state_used[request.state_slot] = 1;
  request.tables.assign(core->groups.size(), std::vector<int>());
  ++core->live_count;
  return r;
}

int hc_close(void* handle, int r) {
  Core* core = static_cast<Core*>(handle);
  if (!good_request(core, r)) return fail(-4, "request %d is ended twice or was never opened", r);
  Request& request = core->requests[r];
  for (size_t g = 0; g < core->groups.size(); ++g)
    for (int page : request.tables[g])
      if (page >= 0 && release_page(core->groups[g], page) < 0) return -4;
  request.tables.clear();
  core->state_used[request.state_slot] = 0;
  core->free_states.push_back(request.state_slot);
  request.live = false;
  core->free_requests.push_back(r);
  --core->live_count;
  return 0;
}

int hc_live_count(void* handle) { return handle ? static_cast<Core*>(handle)->live_count : fail(-1, "no core"); }

int hc_free_state_count(void* handle) {
  return handle ? (int)static_cast<Core*>(handle)->free_states.size() : fail(-1, "no core");
}

int hc_length(void* handle, int r) {
  Core* core = static_cast<Core*>(handle);
  return good_request(core, r) ? core->requests[r].length : fail(-4, "request %d has ended", r);
}

int hc_state_slot(void* handle, int r) {
  Core* core = static_cast<Core*>(handle);
  return good_request(core, r) ? core->requests[r].state_slot : fail(-4, "request %d has ended", r);
}

int hc_table_length(void* handle, int r, int g) {
  Core* core = static_cast<Core*>(handle);
  if (!good_request(core, r) || !good_group(core, g)) return fail(-4, "request %d has ended, or no group %d", r, g);
  return (int)core->requests[r].tables[g].size();
}

int hc_table(void* handle, int r, int g, int* out, int capacity) {
  Core* core = static_cast<Core*>(handle);
  if (!good_request(core, r) || !good_group(core, g)) return fail(-4, "request %d has ended, or no group %d", r, g);
  const std::vector<int>& table = core->requests[r].tables[g];
  for (int i = 0; i < (int)table.size() && i < capacity; ++i) out[i] = table[i];
  return (int)table.size();
}

// pages that `tokens` more tokens would need per group beyond those the request holds
int hc_pages_needed(void* handle, int r, int tokens, int* out) {
  Core* core = static_cast<Core*>(handle);
  if (!good_request(core, r)) return fail(-4, "request %d has ended", r);
  const Request& request = core->requests[r];
  const int need = pages_for(core, request.length + tokens);
  for (size_t g = 0; g < core->groups.size(); ++g) out[g] = std::max(0, need - (int)request.tables[g].size());
  return 0;
}

// Room for `tokens` more tokens in every group, or nothing changes: -2 with the group that is short
// and by how many pages in short_group / shortfall.
int hc_reserve(void* handle, int r, int tokens, int* short_group, int* shortfall) {
  Core* core = static_cast<Core*>(handle);
  if (!good_request(core, r)) return fail(-4, "request %d has ended", r);
  Request& request = core->requests[r];
  const int need = pages_for(core, request.length + tokens);
  for (size_t g = 0; g < core->groups.size(); ++g) {
    const int count = std::max(0, need - (int)request.tables[g].size());
    const int free_pages = (int)core->groups[g].free_stack.size();
    if (count > free_pages) {
      if (short_group) *short_group = (int)g;
      if (shortfall) *shortfall = count - free_pages;
      return fail(-2, "group %d: %d pages requested, %d free", (int)g, count, free_pages);
    }
  }
  for (size_t g = 0; g < core->groups.size(); ++g) {
    Group& group = core->groups[g];
    std::vector<int>& table = request.tables[g];
    while ((int)table.size() < need) {
      const int page = group.free_stack.back();
      group.free_stack.pop_back();
      group.refs[page] = 1;
      table.push_back(page);
    }
  }
  return 0;
}

// gives back pages that were reserved beyond what the stored tokens need
int hc_trim(void* handle, int r) {
  Core* core = static_cast<Core*>(handle);
  if (!good_request(core, r)) return fail(-4, "request %d has ended", r);
  Request& request = core->requests[r];
  const int keep = pages_for(core, request.length);
  for (size_t g = 0; g < core->groups.size(); ++g) {
    std::vector<int>& table = request.tables[g];
    while ((int)table.size() > keep) {
      const int page = table.back();
      table.pop_back();
      if (page >= 0 && release_page(core->groups[g], page) < 0) return -4;
    }
  }
  return 0;
}

int hc_capacity(void* handle, int r) {
  Core* core = static_cast<Core*>(handle);
  if (!good_request(core, r)) return fail(-4, "request %d has ended", r);
  long long least = 1ll << 30;
  for (const std::vector<int>& table : core->requests[r].tables)
    least = std::min(least, (long long)table.size() * core->page_size);
  return (int)least;
}

// `tokens` more tokens are stored; pages a window has passed are given back
int hc_commit(void* handle, int r, int tokens) {
  Core* core = static_cast<Core*>(handle);
  if (!good_request(core, r) || tokens < 0) return fail(-4, "request %d has ended", r);
  Request& request = core->requests[r];
  if (request.length + tokens > hc_capacity(handle, r))
    return fail(-4, "more tokens were stored than pages were reserved for");
  request.length += tokens;
  for (size_t g = 0; g < core->groups.size(); ++g) {
    Group& group = core->groups[g];
    if (group.window <= 0) continue;
    const int first_kept = std::max(0, request.length - group.window + 1);
    std::vector<int>& table = request.tables[g];
    const int passed = std::min((int)table.size(), first_kept / core->page_size);
    for (int logical = passed - 1; logical >= 0 && table[logical] >= 0; --logical) {   // earlier ones went before
      if (release_page(group, table[logical]) < 0) return -4;
      table[logical] = -1;
    }
  }
  return request.length;
}

// a new request starts on full pages that another owner holds
int hc_adopt_prefix(void* handle, int r, int g, const int* pages, int count) {
  Core* core = static_cast<Core*>(handle);
  if (!good_request(core, r) || !good_group(core, g)) return fail(-4, "request %d has ended, or no group %d", r, g);
  Request& request = core->requests[r];
  if (request.length != 0 || !request.tables[g].empty())
    return fail(-4, "a prefix can only be adopted by a request that holds nothing yet");
  Group& group = core->groups[g];
  for (int i = 0; i < count; ++i)
    if (pages[i] < 0 || pages[i] >= group.num_pages || group.refs[pages[i]] <= 0)
      return fail(-4, "page %d is free and cannot be shared", pages[i]);
  for (int i = 0; i < count; ++i) {
    ++group.refs[pages[i]];
    request.tables[g].push_back(pages[i]);
  }
  request.length = count * core->page_size;
  return request.length;
}

// No page lost, none held more often than counted, none both free and held.  `extra` lists pages
// that holders outside the requests have (the prefix tree): group, page pairs.
int hc_check(void* handle, const int* extra, int extra_pairs) {
  Core* core = static_cast<Core*>(handle);
  if (!core) return fail(-1, "no core");
  for (size_t g = 0; g < core->groups.size(); ++g) {
    const Group& group = core->groups[g];
    std::vector<int> held(group.num_pages, 0), on_stack(group.num_pages, 0);
    for (const Request& request : core->requests)
      if (request.live)
        for (int page : request.tables[g])
          if (page >= 0) ++held[page];
    for (int i = 0; i < extra_pairs; ++i)
      if (extra[2 * i] == (int)g) {
        const int page = extra[2 * i + 1];
        if (page < 0 || page >= group.num_pages) return fail(-4, "group %d: a holder names page %d", (int)g, page);
        ++held[page];
      }
    for (int page : group.free_stack) {
      if (++on_stack[page] > 1) return fail(-4, "group %d: page %d is on the free list twice", (int)g, page);
      if (held[page]) return fail(-4, "group %d: page %d is free and held", (int)g, page);
      if (group.refs[page] != 0) return fail(-4, "group %d: free page %d has references", (int)g, page);
    }
    int held_pages = 0;
    for (int page = 0; page < group.num_pages; ++page) {
      if (!held[page]) continue;
      ++held_pages;
      if (group.refs[page] != held[page])
        return fail(-4, "group %d: page %d held %d times, counted %d", (int)g, page, held[page], group.refs[page]);
    }
    if ((int)group.free_stack.size() + held_pages != group.num_pages)
      return fail(-4, "group %d: %d pages are lost", (int)g, group.num_pages - (int)group.free_stack.size() - held_pages);
  }
  std::vector<int> slot_holders(core->state_used.size(), 0);
  int live = 0;
  for (const Request& request : core->requests)
    if (request.live) {
      ++live;
      if (++slot_holders[request.state_slot] > 1) return fail(-4, "a state slot is held by two requests");
    }
  if (live + (int)core->free_states.size() != (int)core->state_used.size()) return fail(-4, "a state slot is lost");
  return 0;
}

// ---- index arrays of a step
// Block tables and write slots of one group for a step's requests, in the order given: request i
// brings counts[i] rows at positions length .. length + counts[i].  table is [n, stride] (filled with
// -1 beyond a request's pages), slots has one entry per row.
int hc_fill_group(void* handle, int g, const int* requests, const int* counts, int n, int stride, int* table,
                  int* slots) {
  Core* core = static_cast<Core*>(handle);
  if (!good_group(core, g) || n < 0 || stride <= 0) return fail(-1, "no such group %d, or bad sizes", g);
  int row = 0;
  for (int i = 0; i < n; ++i) {
    if (!good_request(core, requests[i])) return fail(-4, "request %d has ended", requests[i]);
    const Request& request = core->requests[requests[i]];
    const std::vector<int>& pages = request.tables[g];
    if ((int)pages.size() > stride) return fail(-1, "a table of %d pages does not fit %d columns", (int)pages.size(), stride);
    int* line = table + (size_t)i * stride;
    std::copy(pages.begin(), pages.end(), line);
    std::fill(line + pages.size(), line + stride, -1);
    for (int j = 0; j < counts[i]; ++j, ++row) {
      const int position = request.length + j;
      const int logical = position / core->page_size;
      if (logical >= (int)pages.size()) return fail(-4, "request %d: no page is reserved for position %d", requests[i], position);
      slots[row] = pages[logical] * core->page_size + position % core->page_size;
    }
  }
  return row;
}

// The whole static buffer of a captured decode step (one row per request, padded to `bucket` rows).
// offsets: tokens, positions, row_request, cu_rows, state_slots, logit_rows, token_from, then per group
// table and slots.  Padding rows: token 0 at position 0, writing to the pool's spare page.
int hc_fill_decode(void* handle, const int* requests, const int* tokens, const int* token_from, int rows, int bucket,
                   int stride, const int* spare_pages, const int* offsets, int* buffer) {
  Core* core = static_cast<Core*>(handle);
  if (!core || rows < 0 || rows > bucket || stride <= 0) return fail(-1, "bad sizes of a decode step");
  int* out_tokens = buffer + offsets[0];
  int* positions = buffer + offsets[1];
  int* row_request = buffer + offsets[2];
  int* cu_rows = buffer + offsets[3];
  int* state_slots = buffer + offsets[4];
  int* logit_rows = buffer + offsets[5];
  int* from = buffer + offsets[6];
  for (int i = 0; i < bucket; ++i) {
    const bool live = i < rows;
    if (live && !good_request(core, requests[i])) return fail(-4, "request %d has ended", requests[i]);
    out_tokens[i] = live ? tokens[i] : 0;
    positions[i] = live ? core->requests[requests[i]].length : 0;
    row_request[i] = i;
    cu_rows[i] = i;
    state_slots[i] = live ? core->requests[requests[i]].state_slot : 0;
    logit_rows[i] = i;
    from[i] = live ? token_from[i] : -1;
  }
  cu_rows[bucket] = bucket;
  for (size_t g = 0; g < core->groups.size(); ++g) {
    int* table = buffer + offsets[7 + 2 * g];
    int* slots = buffer + offsets[8 + 2 * g];
    const int spare = spare_pages[g];
    for (int i = 0; i < bucket; ++i) {
      int* line = table + (size_t)i * stride;
      if (i >= rows) {
        std::fill(line, line + stride, -1);
        line[0] = spare;
        slots[i] = spare * core->page_size;
        continue;
      }
      const Request& request = core->requests[requests[i]];
      const std::vector<int>& pages = request.tables[g];
      if ((int)pages.size() > stride) return fail(-1, "a table of %d pages does not fit %d columns", (int)pages.size(), stride);
      std::copy(pages.begin(), pages.end(), line);
      std::fill(line + pages.size(), line + stride, -1);
      const int logical = request.length / core->page_size;
      if (logical >= (int)pages.size()) return fail(-4, "request %d: no page is reserved for its next token", requests[i]);
      slots[i] = pages[logical] * core->page_size + request.length % core->page_size;
    }
  }
  return 0;
}

}  // extern "C"

// ---- prefix tree over full pages of tokens -------------------------------------------------------
// An edge is one page of tokens, a node holds the page id; the tree holds one reference on every page
// it knows, so a finished request's prompt pages stay until they are evicted: least recently used
// leaves that nobody else holds go first (the reference keeps a per-token trie, floors a match to whole
// pages and never evicts, crates/sglang-srt/src/cache.rs:475-547).  A match never covers the whole
// sequence: at most (len - 1) / page_size pages, so at least one token is computed.
namespace {

struct TreeNode {
  std::vector<int> key;
  int page = -1;
  TreeNode* parent = nullptr;
  long long stamp = 0;
  std::map<std::vector<int>, std::unique_ptr<TreeNode>> children;
};

struct Tree {
  Core* core = nullptr;
  int group = 0;
  int page_size = 1;
  TreeNode root;
  long long clock = 0;
  int pages_held = 0;
};

void collect_leaves(TreeNode* node, std::vector<TreeNode*>& out) {
  for (auto& entry : node->children) {
    if (entry.second->children.empty()) out.push_back(entry.second.get());
    else collect_leaves(entry.second.get(), out);
  }
}

// pages below `node` that only the tree holds and that eviction could reach; `free_out`: the node itself is one
int count_evictable(const Tree* tree, const TreeNode* node, bool is_root, bool* free_out) {
  int total = 0;
  bool all_free = true;
  for (const auto& entry : node->children) {
    bool child_free = false;
    total += count_evictable(tree, entry.second.get(), false, &child_free);
    all_free = all_free && child_free;
  }
  if (is_root) {
    *free_out = false;
    return total;
  }
  const bool mine = all_free && tree->core->groups[tree->group].refs[node->page] == 1;
  *free_out = mine;
  return total + (mine ? 1 : 0);
}

void collect_pages(const TreeNode* node, std::vector<int>& out) {
  for (const auto& entry : node->children) {
    out.push_back(entry.second->page);
    collect_pages(entry.second.get(), out);
  }
}

}  // namespace

extern "C" {

void* hc_tree_create(void* handle, int g, int page_size) {
  Core* core = static_cast<Core*>(handle);
  if (!good_group(core, g) || page_size <= 0) return nullptr;
  Tree* tree = new Tree();
  tree->core = core;
  tree->group = g;
  tree->page_size = page_size;
  return tree;
}

void hc_tree_destroy(void* handle) { delete static_cast<Tree*>(handle); }

// page ids of the longest known prefix of tokens[0..count), leaving at least one token out
int hc_tree_match(void* handle, const int* tokens, int count, int* pages_out) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree || count < 0) return fail(-1, "no tree");
  const int page_size = tree->page_size;
  const int most = count > 0 ? (count - 1) / page_size : 0;
  TreeNode* node = &tree->root;
  const long long stamp = ++tree->clock;
  int found = 0;
  std::vector<int> key(page_size);
  for (int i = 0; i < most; ++i) {
    key.assign(tokens + (size_t)i * page_size, tokens + (size_t)(i + 1) * page_size);
    auto it = node->children.find(key);
    if (it == node->children.end()) break;
    node = it->second.get();
    node->stamp = stamp;
    pages_out[found++] = node->page;
  }
  return found;
}

// Makes the full pages pages[i] holding tokens[i*P..(i+1)*P) known.  Pages new to the tree get one more
// reference; a page whose tokens are known already under another page id is left to its request.
int hc_tree_insert(void* handle, const int* tokens, int token_count, const int* pages, int page_count) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return fail(-1, "no tree");
  const int page_size = tree->page_size;
  Group& group = tree->core->groups[tree->group];
  const int count = std::min(page_count, token_count / page_size);
  TreeNode* node = &tree->root;
  const long long stamp = ++tree->clock;
  int adopted = 0;
  std::vector<int> key(page_size);
  for (int i = 0; i < count; ++i) {
    key.assign(tokens + (size_t)i * page_size, tokens + (size_t)(i + 1) * page_size);
    auto it = node->children.find(key);
    TreeNode* child;
    if (it == node->children.end()) {
      if (pages[i] < 0) break;
      if (pages[i] >= group.num_pages || group.refs[pages[i]] <= 0)
        return fail(-4, "page %d is free and cannot be shared", pages[i]);
      std::unique_ptr<TreeNode> fresh(new TreeNode());
      fresh->key = key;
      fresh->page = pages[i];
      fresh->parent = node;
      child = fresh.get();
      node->children.emplace(key, std::move(fresh));
      ++group.refs[pages[i]];
      ++tree->pages_held;
      ++adopted;
    } else {
      child = it->second.get();
    }
    child->stamp = stamp;
    node = child;
  }
  return adopted;
}

int hc_tree_evictable(void* handle) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return fail(-1, "no tree");
  bool unused = false;
  return count_evictable(tree, &tree->root, true, &unused);
}

// frees up to `pages` pages that nobody but the tree holds, least recently used leaves first
int hc_tree_evict(void* handle, int pages) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return fail(-1, "no tree");
  Group& group = tree->core->groups[tree->group];
  int freed = 0;
  while (freed < pages) {
    std::vector<TreeNode*> leaves;
    collect_leaves(&tree->root, leaves);
    leaves.erase(std::remove_if(leaves.begin(), leaves.end(), [&](TreeNode* n) { return group.refs[n->page] != 1; }),
                 leaves.end());
    if (leaves.empty()) break;
    std::stable_sort(leaves.begin(), leaves.end(), [](TreeNode* a, TreeNode* b) { return a->stamp < b->stamp; });
    for (TreeNode* leaf : leaves) {
      if (release_page(group, leaf->page) < 0) return -4;
      --tree->pages_held;
      ++freed;
      const std::vector<int> key = leaf->key;        // the node, and its key with it, goes with the erase
      leaf->parent->children.erase(key);
      if (freed >= pages) break;
    }
  }
  return freed;
}

int hc_tree_pages_held(void* handle) { return handle ? static_cast<Tree*>(handle)->pages_held : fail(-1, "no tree"); }

int hc_tree_pages(void* handle, int* out, int capacity) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return fail(-1, "no tree");
  std::vector<int> pages;
  collect_pages(&tree->root, pages);
  for (int i = 0; i < (int)pages.size() && i < capacity; ++i) out[i] = pages[i];
  return (int)pages.size();
}

int hc_tree_clear(void* handle) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return fail(-1, "no tree");
  std::vector<int> pages;
  collect_pages(&tree->root, pages);
  for (int page : pages)
    if (release_page(tree->core->groups[tree->group], page) < 0) return -4;
  tree->root.children.clear();
  tree->pages_held = 0;
  return (int)pages.size();
}

}  // extern "C"
