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
  // The prefix tree over this group's pages, if there is one, hears when a page goes from one holder
  // to two or back: it keeps count of the pages that nobody but itself holds.
  void* watcher = nullptr;
  void (*shared_changed)(void* watcher, int page, bool shared) = nullptr;
};

inline void note_holders(Group& group, int page, int before, int after) {
  if (group.shared_changed && ((before == 1 && after == 2) || (before == 2 && after == 1)))
    group.shared_changed(group.watcher, page, after == 2);
}

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
  const int after = --group.refs[page];
  if (after == 0) {
    group.free_stack.push_back(page);
    return 1;
  }
  note_holders(group, page, after + 1, after);
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
  const int after = ++group.refs[page];
  note_holders(group, page, after - 1, after);
  return after;
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
    const int after = ++group.refs[pages[i]];
    note_holders(group, pages[i], after - 1, after);
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
// table and slots.  Padding rows: token 0 at position 0, writing to the pool's spare page; their state slot is
// the spare one behind the slots that requests can hold (index = number of state slots).
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
    state_slots[i] = live ? core->requests[requests[i]].state_slot : (int)core->state_used.size();
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
  int busy = 0;                    // nodes of this subtree, itself included, whose page someone else holds too
  long long serial = 0;            // order of creation: decides between equal stamps
  bool listed = false;             // among the tree's idle leaves, under `listed_stamp`
  long long listed_stamp = 0;
  std::map<std::vector<int>, std::unique_ptr<TreeNode>> children;
};

struct Tree {
  Core* core = nullptr;
  int group = 0;
  int page_size = 1;
  TreeNode root;
  long long clock = 0;
  int pages_held = 0;
  long long lookups = 0, hits = 0;
  // Pages that eviction could free: nodes with nothing busy below them.  Kept up to date as holders
  // come and go (a walk from the node to the root each time), so asking costs nothing.
  int evictable = 0;
  std::vector<TreeNode*> node_of_page;
  // Leaves that only the tree holds, least recently used first: what eviction takes next, without a
  // search.  A node enters when it is a leaf and idle, and leaves when it gets a child, a second holder
  // or a new stamp (it enters again under the new one).
  std::map<std::pair<long long, long long>, TreeNode*> idle_leaves;
  long long serials = 0;
};

void unlist(Tree* tree, TreeNode* node) {
  if (!node->listed) return;
  tree->idle_leaves.erase(std::make_pair(node->listed_stamp, node->serial));
  node->listed = false;
}

void list_if_idle_leaf(Tree* tree, TreeNode* node) {
  if (node == &tree->root || node->listed || node->busy != 0 || !node->children.empty()) return;
  node->listed_stamp = node->stamp;
  node->listed = true;
  tree->idle_leaves[std::make_pair(node->stamp, node->serial)] = node;
}

void touch(Tree* tree, TreeNode* node, long long stamp) {
  const bool was = node->listed;
  unlist(tree, node);
  node->stamp = stamp;
  if (was) list_if_idle_leaf(tree, node);
}

// a page of the tree got a second holder, or lost it
void tree_shared_changed(void* watcher, int page, bool shared) {
  Tree* tree = static_cast<Tree*>(watcher);
  if (page < 0 || page >= (int)tree->node_of_page.size()) return;
  for (TreeNode* node = tree->node_of_page[page]; node && node != &tree->root; node = node->parent) {
    if (shared) {
      if (node->busy++ == 0) {
        --tree->evictable;
        unlist(tree, node);
      }
    } else {
      if (--node->busy == 0) {
        ++tree->evictable;
        list_if_idle_leaf(tree, node);
      }
    }
  }
}

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

// frees up to `pages` pages that nobody but the tree holds, least recently used leaves first
int evict_pages(Tree* tree, int pages) {
  Group& group = tree->core->groups[tree->group];
  int freed = 0;
  while (freed < pages && !tree->idle_leaves.empty()) {
    TreeNode* leaf = tree->idle_leaves.begin()->second;
    unlist(tree, leaf);
    tree->node_of_page[leaf->page] = nullptr;
    --tree->evictable;
    if (release_page(group, leaf->page) < 0) return -4;
    --tree->pages_held;
    ++freed;
    TreeNode* parent = leaf->parent;
    const std::vector<int> key = leaf->key;          // the node, and its key with it, goes with the erase
    parent->children.erase(key);
    list_if_idle_leaf(tree, parent);                 // it may be a leaf now, and the next to go
  }
  return freed;
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
  tree->node_of_page.assign(core->groups[g].num_pages, nullptr);
  core->groups[g].watcher = tree;
  core->groups[g].shared_changed = tree_shared_changed;
  return tree;
}

void hc_tree_destroy(void* handle) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return;
  Group& group = tree->core->groups[tree->group];
  if (group.watcher == tree) {
    group.watcher = nullptr;
    group.shared_changed = nullptr;
  }
  delete tree;
}

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
    touch(tree, node, stamp);
    pages_out[found++] = node->page;
  }
  ++tree->lookups;
  tree->hits += found > 0 ? 1 : 0;
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
      if (tree->node_of_page[pages[i]]) return fail(-4, "page %d is in the tree already", pages[i]);
      std::unique_ptr<TreeNode> fresh(new TreeNode());
      fresh->key = key;
      fresh->page = pages[i];
      fresh->parent = node;
      fresh->serial = ++tree->serials;
      child = fresh.get();
      if (node != &tree->root) unlist(tree, node);   // no leaf any more
      node->children.emplace(key, std::move(fresh));
      ++group.refs[pages[i]];                         // the tree's own hold; who gave the page holds it too
      ++tree->pages_held;
      ++adopted;
      tree->node_of_page[pages[i]] = child;
      ++tree->evictable;                              // as if nobody else held it, then corrected
      if (group.refs[pages[i]] > 1) tree_shared_changed(tree, pages[i], true);
      else list_if_idle_leaf(tree, child);
    } else {
      child = it->second.get();
    }
    touch(tree, child, stamp);
    node = child;
  }
  return adopted;
}

int hc_tree_evictable(void* handle) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return fail(-1, "no tree");
  return tree->evictable;
}

int hc_tree_evict(void* handle, int pages) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return fail(-1, "no tree");
  return evict_pages(tree, pages);
}

// the count that is kept up to date against a walk over the whole tree
int hc_tree_check(void* handle) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return fail(-1, "no tree");
  bool unused = false;
  const int walked = count_evictable(tree, &tree->root, true, &unused);
  if (walked != tree->evictable)
    return fail(-4, "the tree counts %d pages that eviction could free, a walk finds %d", tree->evictable, walked);
  std::vector<int> pages;
  collect_pages(&tree->root, pages);
  if ((int)pages.size() != tree->pages_held) return fail(-4, "the tree holds %d pages, counted %d", (int)pages.size(), tree->pages_held);
  for (int page : pages)
    if (!tree->node_of_page[page] || tree->node_of_page[page]->page != page)
      return fail(-4, "page %d of the tree has no node", page);
  // the list of idle leaves against a walk
  std::vector<TreeNode*> leaves;
  collect_leaves(&tree->root, leaves);
  size_t idle = 0;
  for (TreeNode* leaf : leaves) {
    const bool wanted = tree->core->groups[tree->group].refs[leaf->page] == 1;
    if (wanted != leaf->listed) return fail(-4, "the leaf of page %d is %s the list of idle leaves", leaf->page, leaf->listed ? "wrongly in" : "missing from");
    if (leaf->listed && leaf->listed_stamp != leaf->stamp) return fail(-4, "the leaf of page %d is listed under an old stamp", leaf->page);
    idle += wanted ? 1 : 0;
  }
  if (idle != tree->idle_leaves.size()) return fail(-4, "%d idle leaves are listed, a walk finds %d", (int)tree->idle_leaves.size(), (int)idle);
  return 0;
}

// look-ups of prefixes so far (by the scheduler or through the Python face) and how many found something
int hc_tree_counters(void* handle, long long* out) {
  Tree* tree = static_cast<Tree*>(handle);
  if (!tree) return fail(-1, "no tree");
  out[0] = tree->lookups;
  out[1] = tree->hits;
  return 0;
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
  for (int page : pages) tree->node_of_page[page] = nullptr;      // no node hears of the releases below
  tree->evictable = 0;
  tree->idle_leaves.clear();
  for (int page : pages)
    if (release_page(tree->core->groups[tree->group], page) < 0) return -4;
  tree->root.children.clear();
  tree->pages_held = 0;
  return (int)pages.size();
}

}  // extern "C"

// ---- the scheduler -------------------------------------------------------------------------------
// Decisions only: which rows the next step holds.  First come, first served admission under a limit
// of running requests and a token budget per step that counts only tokens still to be computed (the
// reference: crates/sglang-srt/src/scheduler.rs:463-525); a request finishes on a stop token, which
// stays in its output, unless it ignores them (crates/sglang-srt/src/model_executor.rs:763-769), or
// when its new tokens are out (scheduler.rs:195-197).  Beyond the reference: every step gives each
// decoding request its one row first and fills the rest of the budget with prompt portions, the last
// one cut to fit; when pages run out a portion is cut to the free pages, then the request admitted
// last is preempted (pages freed, tokens kept, recomputed later), and a request that could not fit
// even alone finishes with "cache_full".  A request may have one token that is still on the device
// (`pending`): it counts as a token, its value is not known here.
#include <deque>

namespace {

enum Reason { REASON_NONE = 0, REASON_STOP = 1, REASON_LENGTH = 2, REASON_CONTEXT = 3, REASON_CACHE_FULL = 4, REASON_ABORT = 5 };

struct SchedRequest {
  bool used = false;
  std::vector<int> prompt, output, stops;
  int max_new_tokens = 0;
  bool ignore_eos = false;
  int handle = -1;                 // request of the cache books, -1 while it holds nothing
  bool finished = false;
  int reason = REASON_NONE;
  int cached_tokens = 0, preemptions = 0, published_pages = 0, pending = 0;
  long long admitted_at = -1;
};

struct Entry {
  int request, start, count, samples, from_device;
};

struct Output {
  int request, token, cached_tokens, finished, reason;
};

struct Sched {
  Core* core = nullptr;
  Tree* tree = nullptr;
  int max_running = 1, budget = 1, max_positions = 1, evict_ahead = 32;
  std::vector<int> default_stops;
  std::vector<SchedRequest> requests;
  std::vector<int> free_slots;
  std::deque<int> waiting;
  std::vector<int> running;
  std::vector<Output> unreported;
  std::vector<int> events;                  // cache requests opened (1, handle, request) and closed (0, handle, -1), in order
  std::vector<int> touched;                 // requests whose record changed in a way their entries do not show
  long long clock = 0;
  long long steps = 0, preemptions = 0, failed_cache_full = 0, scheduled_tokens = 0;
  std::vector<Entry> entries;               // of the last schedule call
};

int num_tokens(const SchedRequest& r) { return (int)r.prompt.size() + (int)r.output.size() + r.pending; }
int computed(const Sched* s, const SchedRequest& r) { return r.handle >= 0 ? s->core->requests[r.handle].length : 0; }

bool is_decoding(const Sched* s, const SchedRequest& r) {
  return r.handle >= 0 && (!r.output.empty() || r.pending > 0) && computed(s, r) == num_tokens(r) - 1;
}

bool ends_whatever_comes(const Sched* s, const SchedRequest& r) {
  return r.pending > 0 && ((int)r.output.size() + r.pending >= r.max_new_tokens || num_tokens(r) >= s->max_positions);
}

int token_at(const SchedRequest& r, int position) {
  const int n = (int)r.prompt.size();
  if (position < n) return r.prompt[position];
  if (position - n < (int)r.output.size()) return r.output[position - n];
  return -1;                                   // still on the device
}

int reclaimable(const Sched* s, int g) { return s->tree && s->tree->group == g ? s->tree->evictable : 0; }

int evict(Sched* s, int pages) { return evict_pages(s->tree, pages); }

// room for `tokens` more tokens, evicting cached prefixes if that helps; false: nothing changed
bool reserve(Sched* s, int handle, int tokens) {
  int short_group = 0, shortfall = 0;
  int status = hc_reserve(s->core, handle, tokens, &short_group, &shortfall);
  if (status == -2 && s->tree && s->tree->group == short_group) {
    evict(s, std::max(shortfall, s->evict_ahead));
    status = hc_reserve(s->core, handle, tokens, &short_group, &shortfall);
  }
  return status == 0;
}

bool can_reserve(const Sched* s, int handle, int tokens) {
  const Request& request = s->core->requests[handle];
  const int need = pages_for(s->core, request.length + tokens);
  for (size_t g = 0; g < s->core->groups.size(); ++g) {
    const int count = std::max(0, need - (int)request.tables[g].size());
    const int free_pages = (int)s->core->groups[g].free_stack.size();
    if (count > free_pages && count > free_pages + reclaimable(s, (int)g)) return false;
  }
  return true;
}

void close_handle(Sched* s, SchedRequest& r) {
  if (r.handle >= 0) {
    hc_close(s->core, r.handle);
    s->events.insert(s->events.end(), {0, r.handle, -1});
    r.handle = -1;
  }
}

void finish(Sched* s, int slot, int reason, bool report) {
  SchedRequest& r = s->requests[slot];
  s->touched.push_back(slot);
  close_handle(s, r);
  r.finished = true;
  r.reason = reason;
  if (report) s->unreported.push_back(Output{slot, -1, r.cached_tokens, 1, reason});
}

void remove_running(Sched* s, int slot) {
  s->running.erase(std::remove(s->running.begin(), s->running.end(), slot), s->running.end());
}

bool is_running(const Sched* s, int slot) { return std::find(s->running.begin(), s->running.end(), slot) != s->running.end(); }

int youngest_running(const Sched* s) {
  int best = s->running.front();
  for (int slot : s->running)
    if (s->requests[slot].admitted_at > s->requests[best].admitted_at) best = slot;
  return best;
}

void preempt(Sched* s, int victim) {
  s->entries.erase(std::remove_if(s->entries.begin(), s->entries.end(), [&](const Entry& e) { return e.request == victim; }),
                   s->entries.end());
  remove_running(s, victim);
  SchedRequest& r = s->requests[victim];
  s->touched.push_back(victim);
  close_handle(s, r);
  r.published_pages = 0;
  ++r.preemptions;
  ++s->preemptions;
  s->waiting.push_front(victim);
}

int schedule_portion(Sched* s, int slot, int budget) {
  SchedRequest& r = s->requests[slot];
  const int total = num_tokens(r);
  const int start = computed(s, r);
  int count = std::min(budget, total - start);
  // cut the portion down to the pages that are free
  while (count > 0 && !can_reserve(s, r.handle, count)) {
    int free_pages = 1 << 30;
    for (size_t g = 0; g < s->core->groups.size(); ++g)
      free_pages = std::min(free_pages, (int)s->core->groups[g].free_stack.size() + reclaimable(s, (int)g));
    if (s->core->groups.empty()) free_pages = 0;
    const int room = hc_capacity(s->core, r.handle) - start + free_pages * s->core->page_size;
    count = std::min(count - 1, std::max(room, 0));
  }
  if (count <= 0) return 0;
  if (!reserve(s, r.handle, count)) return 0;
  s->entries.push_back(Entry{slot, start, count, start + count == total ? 1 : 0, 0});
  return count;
}

bool can_never_fit(const Sched* s, const SchedRequest& r) {
  // prompt (and what was generated before a preemption) plus the token to be sampled next
  const int need = pages_for(s->core, num_tokens(r) + 1);
  for (const Group& group : s->core->groups)
    if (group.window <= 0 && need > group.num_pages) return true;
  return false;
}

void schedule_once(Sched* s) {
  int budget = s->budget;
  s->entries.clear();
  const long long preempted_before = s->preemptions;
  // 1. every decoding request gets its one row; make room by preemption if needed
  std::vector<int> decoding;
  for (int slot : s->running)
    if (is_decoding(s, s->requests[slot])) decoding.push_back(slot);
  for (int slot : decoding) {
    if (!is_running(s, slot)) continue;                       // preempted below, earlier in this loop
    SchedRequest& r = s->requests[slot];
    if (ends_whatever_comes(s, r)) continue;                  // it finishes when its token arrives
    while (true) {
      if (reserve(s, r.handle, 1)) break;
      const int victim = youngest_running(s);
      if (victim == slot && s->running.size() == 1) {
        // alone and the pool is full of its own tokens: it can never go on
        remove_running(s, slot);
        finish(s, slot, REASON_CACHE_FULL, true);
        ++s->failed_cache_full;
        break;
      }
      preempt(s, victim);
      if (victim == slot) break;
    }
    if (is_running(s, slot) && !r.finished) {
      s->entries.push_back(Entry{slot, computed(s, r), 1, 1, r.pending > 0 ? 1 : 0});
      --budget;
    }
  }
  // 2. prompts in progress go on, oldest first; 3. then new requests are admitted
  std::vector<int> in_progress;
  for (int slot : s->running)
    if (!is_decoding(s, s->requests[slot])) in_progress.push_back(slot);
  for (int slot : in_progress) {
    if (budget <= 0) break;
    if (s->requests[slot].pending) continue;
    bool scheduled = false;
    for (const Entry& e : s->entries) scheduled = scheduled || e.request == slot;
    if (scheduled) continue;
    budget -= schedule_portion(s, slot, budget);
  }
  while (!s->waiting.empty() && budget > 0 && (int)s->running.size() < s->max_running) {
    if (s->preemptions != preempted_before && !s->running.empty()) break;   // pages were just taken away: admit nobody
    const int slot = s->waiting.front();
    SchedRequest& r = s->requests[slot];
    if (can_never_fit(s, r)) {
      s->waiting.pop_front();
      finish(s, slot, REASON_CACHE_FULL, true);
      ++s->failed_cache_full;
      continue;
    }
    const int handle = hc_open(s->core);
    if (handle < 0) break;
    r.handle = handle;
    s->touched.push_back(slot);
    s->events.insert(s->events.end(), {1, handle, slot});
    if (s->tree) {
      std::vector<int> tokens(r.prompt);
      tokens.insert(tokens.end(), r.output.begin(), r.output.end());
      std::vector<int> shared(tokens.size() / s->tree->page_size + 1);
      const int found = hc_tree_match(s->tree, tokens.data(), (int)tokens.size(), shared.data());
      if (found > 0) {
        hc_adopt_prefix(s->core, handle, s->tree->group, shared.data(), found);
        r.published_pages = found;
        if (!r.preemptions) r.cached_tokens = std::min(s->core->requests[handle].length, (int)r.prompt.size());
      }
    }
    const int taken = schedule_portion(s, slot, budget);
    if (taken == 0) {
      close_handle(s, r);                                     // no page free: it stays at the head
      break;
    }
    s->waiting.pop_front();
    r.admitted_at = s->clock++;
    s->running.push_back(slot);
    budget -= taken;
  }
}

}  // namespace

extern "C" {

void* hs_create(void* core, void* tree, int max_running, int budget, int max_positions, const int* stops, int num_stops) {
  if (!core || max_running <= 0 || budget <= 0) return nullptr;
  Sched* s = new Sched();
  s->core = static_cast<Core*>(core);
  s->tree = static_cast<Tree*>(tree);
  s->max_running = max_running;
  s->budget = budget;
  s->max_positions = max_positions;
  s->default_stops.assign(stops, stops + num_stops);
  return s;
}

void hs_destroy(void* handle) { delete static_cast<Sched*>(handle); }

void hs_set_tree(void* handle, void* tree) { static_cast<Sched*>(handle)->tree = static_cast<Tree*>(tree); }

int hs_add(void* handle, const int* prompt, int prompt_len, int max_new_tokens, const int* stops, int num_stops,
           int ignore_eos) {
  Sched* s = static_cast<Sched*>(handle);
  if (!s || prompt_len <= 0) return fail(-1, "a request needs a prompt");
  int slot;
  if (!s->free_slots.empty()) {
    slot = s->free_slots.back();
    s->free_slots.pop_back();
  } else {
    slot = (int)s->requests.size();
    s->requests.emplace_back();
  }
  SchedRequest& r = s->requests[slot];
  r = SchedRequest();
  r.used = true;
  r.prompt.assign(prompt, prompt + prompt_len);
  r.max_new_tokens = max_new_tokens;
  r.stops.assign(stops, stops + num_stops);
  r.ignore_eos = ignore_eos != 0;
  s->waiting.push_back(slot);
  return slot;
}

// a finished request's record may be used again
int hs_forget(void* handle, int slot) {
  Sched* s = static_cast<Sched*>(handle);
  if (!s || slot < 0 || slot >= (int)s->requests.size() || !s->requests[slot].used) return fail(-1, "no such request");
  if (!s->requests[slot].finished) return fail(-4, "the request is not finished");
  s->requests[slot] = SchedRequest();
  s->free_slots.push_back(slot);
  return 0;
}

int hs_has_work(void* handle) {
  Sched* s = static_cast<Sched*>(handle);
  return s && (!s->waiting.empty() || !s->running.empty());
}

// Chooses the rows of the next step and reserves their pages.  Returns the number of entries; the entries
// are read with hs_entries, the tokens of all entries, one after another, with hs_entry_tokens.
int hs_schedule(void* handle, int ahead) {
  Sched* s = static_cast<Sched*>(handle);
  if (!s) return fail(-1, "no scheduler");
  while (true) {
    schedule_once(s);
    if (!s->entries.empty() || s->running.empty() || ahead) break;
    // Nothing could move although requests are running: prompts in progress hold all pages between
    // them.  The one admitted last gives its pages up.
    preempt(s, youngest_running(s));
  }
  ++s->steps;
  for (const Entry& e : s->entries) s->scheduled_tokens += e.count;
  return (int)s->entries.size();
}

int hs_entries(void* handle, int* out /* [n][5]: request, start, count, samples, from_device */) {
  Sched* s = static_cast<Sched*>(handle);
  for (size_t i = 0; i < s->entries.size(); ++i) {
    const Entry& e = s->entries[i];
    out[5 * i] = e.request; out[5 * i + 1] = e.start; out[5 * i + 2] = e.count; out[5 * i + 3] = e.samples;
    out[5 * i + 4] = e.from_device;
  }
  return (int)s->entries.size();
}

int hs_entry_tokens(void* handle, int* out, int capacity) {
  Sched* s = static_cast<Sched*>(handle);
  int written = 0;
  for (const Entry& e : s->entries)
    for (int j = 0; j < e.count; ++j) {
      if (written >= capacity) return fail(-1, "the token buffer is too small");
      out[written++] = token_at(s->requests[e.request], e.start + j);
    }
  return written;
}

// After the step: entries [n][5] as given by hs_entries, one sampled token per entry with `samples` set, in
// order.  Outputs [m][5]: request, token (-1: none), cached tokens, finished, reason; returns m.
int hs_process(void* handle, const int* entries, int num_entries, const int* sampled, int num_sampled, int* out,
               int capacity) {
  Sched* s = static_cast<Sched*>(handle);
  if (!s) return fail(-1, "no scheduler");
  std::vector<Output> outputs(s->unreported);
  s->unreported.clear();
  int next_pick = 0;
  for (int i = 0; i < num_entries; ++i) {
    const int slot = entries[5 * i];
    const bool samples = entries[5 * i + 3] != 0;
    SchedRequest& r = s->requests[slot];
    if (s->tree && r.handle >= 0) {
      // full pages of prompt tokens become known as soon as they are computed
      const int full = std::min(s->core->requests[r.handle].length, (int)r.prompt.size()) / s->core->page_size;
      if (full > r.published_pages) {
        const std::vector<int>& table = s->core->requests[r.handle].tables[s->tree->group];
        hc_tree_insert(s->tree, r.prompt.data(), full * s->core->page_size, table.data(), std::min(full, (int)table.size()));
        r.published_pages = full;
      }
    }
    if (!samples) continue;
    if (next_pick >= num_sampled) return fail(-1, "fewer tokens than entries that sample");
    const int token = sampled[next_pick++];
    r.pending = std::max(0, r.pending - 1);
    if (r.finished) continue;                  // it ended (stop token, abort) while this step was already running
    r.output.push_back(token);
    bool is_stop = std::find(r.stops.begin(), r.stops.end(), token) != r.stops.end() ||
                   std::find(s->default_stops.begin(), s->default_stops.end(), token) != s->default_stops.end();
    int reason = REASON_NONE;
    if (is_stop && !r.ignore_eos) reason = REASON_STOP;
    else if ((int)r.output.size() >= r.max_new_tokens) reason = REASON_LENGTH;
    else if (num_tokens(r) >= s->max_positions) reason = REASON_CONTEXT;
    if (reason != REASON_NONE) {
      remove_running(s, slot);
      finish(s, slot, reason, false);
    }
    outputs.push_back(Output{slot, token, r.cached_tokens, r.finished ? 1 : 0, reason});
  }
  if ((int)outputs.size() > capacity) return fail(-1, "the output buffer is too small");
  for (size_t i = 0; i < outputs.size(); ++i) {
    out[5 * i] = outputs[i].request; out[5 * i + 1] = outputs[i].token; out[5 * i + 2] = outputs[i].cached_tokens;
    out[5 * i + 3] = outputs[i].finished; out[5 * i + 4] = outputs[i].reason;
  }
  return (int)outputs.size();
}

// the step raised: every request of the batch is failed and gives its pages back
int hs_step_failed(void* handle, const int* entries, int num_entries) {
  Sched* s = static_cast<Sched*>(handle);
  for (int i = 0; i < num_entries; ++i) {
    const int slot = entries[5 * i];
    if (is_running(s, slot)) {
      remove_running(s, slot);
      finish(s, slot, REASON_ABORT, true);
    }
  }
  return 0;
}

int hs_abort(void* handle, int slot) {
  Sched* s = static_cast<Sched*>(handle);
  if (!s || slot < 0 || slot >= (int)s->requests.size() || !s->requests[slot].used) return 0;
  auto in_waiting = std::find(s->waiting.begin(), s->waiting.end(), slot);
  if (in_waiting != s->waiting.end()) {
    s->waiting.erase(in_waiting);
  } else if (is_running(s, slot)) {
    remove_running(s, slot);
  } else {
    return 0;
  }
  finish(s, slot, REASON_ABORT, true);
  return 1;
}

// the caller takes a running request out of the scheduler's hands (it keeps its pages)
int hs_release(void* handle, int slot) {
  Sched* s = static_cast<Sched*>(handle);
  if (!s || !is_running(s, slot)) return fail(-4, "the request is not running");
  remove_running(s, slot);
  return 0;
}

int hs_mark_pending(void* handle, int slot, int delta) {
  Sched* s = static_cast<Sched*>(handle);
  s->requests[slot].pending += delta;
  return s->requests[slot].pending;
}

// what a request's record holds: out[0..8] = handle, finished, reason, cached tokens, preemptions, published pages,
// pending, outputs so far, decoding; out[9] admitted_at (low 31 bits)
int hs_state(void* handle, int slot, int* out) {
  Sched* s = static_cast<Sched*>(handle);
  if (!s || slot < 0 || slot >= (int)s->requests.size() || !s->requests[slot].used) return fail(-1, "no such request");
  const SchedRequest& r = s->requests[slot];
  out[0] = r.handle; out[1] = r.finished; out[2] = r.reason; out[3] = r.cached_tokens; out[4] = r.preemptions;
  out[5] = r.published_pages; out[6] = r.pending; out[7] = (int)r.output.size(); out[8] = is_decoding(s, r) ? 1 : 0;
  out[9] = (int)(r.admitted_at & 0x7fffffff) * (r.admitted_at < 0 ? -1 : 1);
  return 0;
}

int hs_outputs(void* handle, int slot, int from, int* out, int capacity) {
  Sched* s = static_cast<Sched*>(handle);
  const SchedRequest& r = s->requests[slot];
  int written = 0;
  for (int i = from; i < (int)r.output.size() && written < capacity; ++i) out[written++] = r.output[i];
  return written;
}

int hs_queue(void* handle, int which /* 0 waiting, 1 running */, int* out, int capacity) {
  Sched* s = static_cast<Sched*>(handle);
  int written = 0;
  if (which == 0) {
    for (int slot : s->waiting)
      if (written < capacity) out[written++] = slot;
    return (int)s->waiting.size();
  }
  for (int slot : s->running)
    if (written < capacity) out[written++] = slot;
  return (int)s->running.size();
}

// cache requests opened (1, handle, request) and closed (0, handle, -1) since the last call, in order
int hs_handle_events(void* handle, int* out, int capacity) {
  Sched* s = static_cast<Sched*>(handle);
  const int count = (int)s->events.size();
  if (count > capacity) return fail(-1, "the event buffer is too small");
  std::copy(s->events.begin(), s->events.end(), out);
  s->events.clear();
  return count / 3;
}

// requests that were admitted, preempted or finished since the last call
int hs_touched(void* handle, int* out, int capacity) {
  Sched* s = static_cast<Sched*>(handle);
  std::sort(s->touched.begin(), s->touched.end());
  s->touched.erase(std::unique(s->touched.begin(), s->touched.end()), s->touched.end());
  const int count = (int)s->touched.size();
  if (count > capacity) return fail(-1, "the buffer is too small");
  std::copy(s->touched.begin(), s->touched.end(), out);
  s->touched.clear();
  return count;
}

// for tests that build a state by hand: a waiting request becomes a running one on a cache request
int hs_force_running(void* handle, int slot, int cache_request, int admitted_at) {
  Sched* s = static_cast<Sched*>(handle);
  auto in_waiting = std::find(s->waiting.begin(), s->waiting.end(), slot);
  if (in_waiting == s->waiting.end()) return fail(-4, "the request is not waiting");
  s->waiting.erase(in_waiting);
  s->requests[slot].handle = cache_request;
  s->requests[slot].admitted_at = admitted_at;
  s->running.push_back(slot);
  return 0;
}

int hs_stats(void* handle, long long* out /* steps, preemptions, failed_cache_full, scheduled_tokens */) {
  Sched* s = static_cast<Sched*>(handle);
  out[0] = s->steps; out[1] = s->preemptions; out[2] = s->failed_cache_full; out[3] = s->scheduled_tokens;
  return 0;
}

}  // extern "C"
