// Paged-KV block allocator and continuous-batching decode scheduler (host side, no CUDA).
//
// BlockManager follows the behaviour of the reference's allocator
// (crates/wukong_codegen_gpu/src/paged_kv.rs:428-628): a LIFO free list that hands out pages in
// ascending order on a fresh pool, per-slot logical->physical tables, `append` allocating only on a
// page boundary, bulk `reserve`, `free` returning a slot's pages, a `layout_epoch` that moves
// whenever any table changes, and a padded row-major flat table (zeros past each slot's pages).
// Running out of pages is reported (-1), never fatal, and leaves the allocator unchanged.
//
// Scheduler follows crates/wukong_codegen_gpu/src/serving.rs:1346-1595: fixed `bcap` slots,
// first-fit admission with a look-ahead window of 64 waiting requests, one step = admit -> advance
// every active slot -> run the model -> retire finished sequences and free their pages.  Unlike
// the reference's (which carries lengths only and runs no embedding, LM head or sampling), requests
// here carry token ids: a slot first consumes its prompt in chunks ("prefill rows"), then feeds back
// its own sampled token one row per step.  The model side sees a flat batch of rows
// (token, position, slot, visible keys) and the index of the row to sample for each slot.
#include "../../include/wukong_b200.h"
#include <algorithm>
#include <cstring>
#include <deque>
#include <vector>

namespace {

struct BlockManager {
  int64_t block_size, num_blocks, mbps;
  std::vector<uint32_t> free_list;
  std::vector<std::vector<uint32_t>> tables;
  std::vector<int64_t> ctx;
  uint64_t epoch = 0;

  BlockManager(int64_t nb, int64_t bs, int64_t slots, int64_t m) : block_size(bs), num_blocks(nb), mbps(m) {
    free_list.resize((size_t)nb);
    for (int64_t i = 0; i < nb; ++i) free_list[(size_t)i] = (uint32_t)(nb - 1 - i);  // pop() yields 0, 1, 2, ...
    tables.resize((size_t)slots);
    ctx.assign((size_t)slots, 0);
  }
  int64_t blocks_for(int64_t tokens) const { return (tokens + block_size - 1) / block_size; }
  bool can_grow(int64_t slot, int64_t tokens) const {
    int64_t have = (int64_t)tables[(size_t)slot].size() * block_size;
    int64_t need = ctx[(size_t)slot] + tokens;
    if (need > have) {
      int64_t nb = blocks_for(need) - (int64_t)tables[(size_t)slot].size();
      if (nb > (int64_t)free_list.size()) return false;
      if ((int64_t)tables[(size_t)slot].size() + nb > mbps) return false;
    }
    return true;
  }
  bool push_block(int64_t slot) {
    auto& t = tables[(size_t)slot];
    if ((int64_t)t.size() >= mbps || free_list.empty()) return false;
    t.push_back(free_list.back());
    free_list.pop_back();
    ++epoch;
    return true;
  }
  int64_t append(int64_t slot, uint32_t* phys, int64_t* off) {
    int64_t pos = ctx[(size_t)slot], logical = pos / block_size;
    if (logical >= (int64_t)tables[(size_t)slot].size() && !push_block(slot)) return -1;
    if (phys) *phys = tables[(size_t)slot][(size_t)logical];
    if (off) *off = pos % block_size;
    ctx[(size_t)slot] = pos + 1;
    return 0;
  }
  int64_t reserve(int64_t slot, int64_t tokens) {
    if (!can_grow(slot, tokens)) return -1;
    int64_t start = ctx[(size_t)slot], need = start + tokens;
    while ((int64_t)tables[(size_t)slot].size() * block_size < need) push_block(slot);
    ctx[(size_t)slot] = need;
    return start;
  }
  // Pages for `tokens` more positions without advancing the context (admission-time reservation).
  bool ensure_capacity(int64_t slot, int64_t tokens) {
    if (!can_grow(slot, tokens)) return false;
    int64_t need = ctx[(size_t)slot] + tokens;
    while ((int64_t)tables[(size_t)slot].size() * block_size < need) push_block(slot);
    return true;
  }
  void release(int64_t slot) {
    auto& t = tables[(size_t)slot];
    if (!t.empty()) ++epoch;
    for (uint32_t b : t) free_list.push_back(b);
    t.clear();
    ctx[(size_t)slot] = 0;
  }
};

struct Request {
  int64_t id;
  std::vector<int32_t> prompt;
  int64_t gen_len;
};

struct Inflight {
  int64_t id = -1;
  std::vector<int32_t> prompt;
  int64_t fed = 0;        // prompt tokens already sent through the model
  int64_t remaining = 0;  // tokens still to emit
  int32_t last = 0;       // last sampled token (the next decode input)
  int64_t planned = 0;    // rows planned for this slot in the open step
  bool samples = false;   // the open step samples a token for this slot
};

struct Scheduler {
  BlockManager mgr;
  int64_t bcap, max_rows, prefill_chunk;
  std::vector<Inflight> slots;
  std::deque<Request> waiting;
  std::vector<std::vector<int32_t>> outputs;  // per request id
  int64_t emitted = 0, admitted = 0, completed = 0, next_id = 0;
  bool step_open = false;
  static constexpr int64_t LOOKAHEAD = 64;

  Scheduler(int64_t bcap_, int64_t nblocks, int64_t bs, int64_t mbps, int64_t max_rows_, int64_t chunk)
      : mgr(nblocks, bs, bcap_, mbps), bcap(bcap_), max_rows(max_rows_), prefill_chunk(chunk), slots((size_t)bcap_) {}

  int64_t num_active() const {
    int64_t n = 0;
    for (auto& s : slots) n += s.id >= 0;
    return n;
  }

  int64_t admit() {
    int64_t n = 0;
    for (int64_t slot = 0; slot < bcap; ++slot) {
      if (slots[(size_t)slot].id >= 0) continue;
      if (waiting.empty()) break;
      int64_t pick = -1, lim = std::min<int64_t>(LOOKAHEAD, (int64_t)waiting.size());
      for (int64_t i = 0; i < lim; ++i) {
        int64_t need = std::max<int64_t>(1, (int64_t)waiting[(size_t)i].prompt.size());
        if (mgr.can_grow(slot, need)) { pick = i; break; }
      }
      if (pick < 0) break;  // nothing in the window fits: leave the queue intact
      Request r = std::move(waiting[(size_t)pick]);
      waiting.erase(waiting.begin() + pick);
      mgr.ensure_capacity(slot, std::max<int64_t>(1, (int64_t)r.prompt.size()));  // as the reference reserves
      Inflight& f = slots[(size_t)slot];
      f = Inflight();
      f.id = r.id;
      f.prompt = std::move(r.prompt);
      f.remaining = std::max<int64_t>(1, r.gen_len);
      ++admitted;
      ++n;
    }
    return n;
  }
};

}  // namespace

extern "C" {

// ---- block manager -----------------------------------------------------------------------------
void* wkb_blockmgr_new(int64_t num_blocks, int64_t block_size, int64_t num_slots, int64_t max_blocks_per_seq) {
  if (num_blocks <= 0 || block_size <= 0 || num_slots <= 0 || max_blocks_per_seq <= 0) return nullptr;
  return new BlockManager(num_blocks, block_size, num_slots, max_blocks_per_seq);
}
void wkb_blockmgr_delete(void* h) { delete (BlockManager*)h; }
int64_t wkb_blockmgr_append(void* h, int64_t slot, uint32_t* phys, int64_t* off) { return ((BlockManager*)h)->append(slot, phys, off); }
int64_t wkb_blockmgr_reserve(void* h, int64_t slot, int64_t tokens) { return ((BlockManager*)h)->reserve(slot, tokens); }
void wkb_blockmgr_release(void* h, int64_t slot) { ((BlockManager*)h)->release(slot); }
int64_t wkb_blockmgr_can_grow(void* h, int64_t slot, int64_t tokens) { return ((BlockManager*)h)->can_grow(slot, tokens) ? 1 : 0; }
int64_t wkb_blockmgr_free_blocks(void* h) { return (int64_t)((BlockManager*)h)->free_list.size(); }
int64_t wkb_blockmgr_used_blocks(void* h) { auto* m = (BlockManager*)h; return m->num_blocks - (int64_t)m->free_list.size(); }
int64_t wkb_blockmgr_context_len(void* h, int64_t slot) { return ((BlockManager*)h)->ctx[(size_t)slot]; }
int64_t wkb_blockmgr_layout_epoch(void* h) { return (int64_t)((BlockManager*)h)->epoch; }
int64_t wkb_blockmgr_locate(void* h, int64_t slot, int64_t pos, uint32_t* phys, int64_t* off) {
  auto* m = (BlockManager*)h;
  int64_t logical = pos / m->block_size;
  if (pos < 0 || logical >= (int64_t)m->tables[(size_t)slot].size()) return -1;
  *phys = m->tables[(size_t)slot][(size_t)logical];
  *off = pos % m->block_size;
  return 0;
}
void wkb_blockmgr_flat_table(void* h, uint32_t* out) {
  auto* m = (BlockManager*)h;
  size_t w = (size_t)m->mbps;
  std::memset(out, 0, m->tables.size() * w * sizeof(uint32_t));
  for (size_t s = 0; s < m->tables.size(); ++s)
    std::copy(m->tables[s].begin(), m->tables[s].end(), out + s * w);
}
void wkb_blockmgr_ctx_lens(void* h, int32_t* out) {
  auto* m = (BlockManager*)h;
  for (size_t s = 0; s < m->ctx.size(); ++s) out[s] = (int32_t)m->ctx[s];
}

// ---- scheduler -----------------------------------------------------------------------------------
void* wkb_sched_new(int64_t bcap, int64_t num_blocks, int64_t block_size, int64_t max_blocks_per_seq,
                    int64_t max_rows, int64_t prefill_chunk) {
  if (bcap <= 0 || num_blocks <= 0 || block_size <= 0 || max_blocks_per_seq <= 0 || max_rows < bcap || prefill_chunk <= 0)
    return nullptr;
  return new Scheduler(bcap, num_blocks, block_size, max_blocks_per_seq, max_rows, prefill_chunk);
}
void wkb_sched_delete(void* h) { delete (Scheduler*)h; }

int64_t wkb_sched_enqueue(void* h, const int32_t* prompt, int64_t prompt_len, int64_t gen_len) {
  auto* s = (Scheduler*)h;
  if (prompt_len <= 0 || gen_len <= 0) return -1;
  if (s->mgr.blocks_for(prompt_len + gen_len) > s->mgr.mbps) return -2;  // can never fit a table row
  Request r;
  r.id = s->next_id++;
  r.prompt.assign(prompt, prompt + prompt_len);
  r.gen_len = gen_len;
  s->outputs.emplace_back();
  s->waiting.push_back(std::move(r));
  return r.id;
}

// Admit, then lay out this step's rows.  Outputs (caller-owned, capacities max_rows / bcap):
//   row_token, row_pos, row_slot, row_ctx  per row;  sample_row[slot] = row to sample or -1.
// Admission (slot assignment and the prompt's page reservation) happens first and is kept whatever follows.
// Slots whose rows need more pages than are free are left out of this step, decode rows being served before
// prompt chunks; they run again once other sequences retire and release pages.  Returns the number of rows
// (0: idle), or -1 when sequences are resident but not one row can get a page: no step was planned, and the
// state can only move on if the caller releases a slot (the reference returns Err(OutOfBlocks) here too).
int64_t wkb_sched_plan_step(void* h, int32_t* row_token, int32_t* row_pos, int32_t* row_slot, int32_t* row_ctx,
                            int32_t* sample_row) {
  auto* s = (Scheduler*)h;
  if (s->step_open) return -3;
  s->admit();
  // pass 1: decide row counts (decode rows first, the rest of the budget to prefill chunks)
  int64_t budget = s->max_rows, rows = 0;
  for (auto& f : s->slots) { f.planned = 0; f.samples = false; }
  for (auto& f : s->slots)
    if (f.id >= 0 && f.fed >= (int64_t)f.prompt.size()) { f.planned = 1; f.samples = true; --budget; }
  for (auto& f : s->slots)
    if (f.id >= 0 && f.fed < (int64_t)f.prompt.size() && budget > 0) {
      int64_t left = (int64_t)f.prompt.size() - f.fed;
      f.planned = std::min<int64_t>({left, s->prefill_chunk, budget});
      f.samples = f.planned == left;
      budget -= f.planned;
    }
  // pass 2: hand the free pages out, decode rows first; a slot that cannot get its pages sits this step out
  {
    int64_t free_left = (int64_t)s->mgr.free_list.size(), planned_rows = 0, wanted_rows = 0;
    for (int pass = 0; pass < 2; ++pass)
      for (int64_t slot = 0; slot < s->bcap; ++slot) {
        auto& f = s->slots[(size_t)slot];
        const bool decode = f.id >= 0 && f.fed >= (int64_t)f.prompt.size();
        if (f.planned == 0 || decode != (pass == 0)) continue;
        wanted_rows += f.planned;
        int64_t have = (int64_t)s->mgr.tables[(size_t)slot].size();
        int64_t want = s->mgr.blocks_for(s->mgr.ctx[(size_t)slot] + f.planned);
        int64_t extra = std::max<int64_t>(0, want - have);
        if (want > s->mgr.mbps || extra > free_left) { f.planned = 0; f.samples = false; continue; }
        free_left -= extra;
        planned_rows += f.planned;
      }
    if (wanted_rows > 0 && planned_rows == 0) {
      for (auto& f : s->slots) { f.planned = 0; f.samples = false; }
      return -1;
    }
  }
  // pass 3: lay the rows out
  for (int64_t slot = 0; slot < s->bcap; ++slot) {
    auto& f = s->slots[(size_t)slot];
    sample_row[slot] = -1;
    if (f.planned == 0) continue;
    for (int64_t i = 0; i < f.planned; ++i) {
      int64_t pos = s->mgr.ctx[(size_t)slot];
      s->mgr.append(slot, nullptr, nullptr);
      bool prefill = f.fed < (int64_t)f.prompt.size();
      row_token[rows] = prefill ? f.prompt[(size_t)f.fed] : f.last;
      if (prefill) ++f.fed;
      row_pos[rows] = (int32_t)pos;
      row_slot[rows] = (int32_t)slot;
      row_ctx[rows] = (int32_t)(pos + 1);
      ++rows;
    }
    if (f.samples) sample_row[slot] = (int32_t)(rows - 1);
  }
  s->step_open = rows > 0;
  return rows;
}

// Close the step: sampled[slot] is the token drawn from sample_row[slot] (ignored elsewhere).
// Returns the number of tokens emitted.
int64_t wkb_sched_commit_step(void* h, const int32_t* sampled) {
  auto* s = (Scheduler*)h;
  if (!s->step_open) return 0;
  int64_t n = 0;
  for (int64_t slot = 0; slot < s->bcap; ++slot) {
    auto& f = s->slots[(size_t)slot];
    if (f.id < 0 || !f.samples) continue;
    f.last = sampled[slot];
    s->outputs[(size_t)f.id].push_back(f.last);
    ++s->emitted;
    ++n;
    if (--f.remaining == 0) {
      s->mgr.release(slot);
      f = Inflight();
      ++s->completed;
    }
  }
  s->step_open = false;
  return n;
}

void* wkb_sched_blockmgr(void* h) { return &((Scheduler*)h)->mgr; }
int64_t wkb_sched_num_active(void* h) { return ((Scheduler*)h)->num_active(); }
int64_t wkb_sched_pending(void* h) { return (int64_t)((Scheduler*)h)->waiting.size(); }
int64_t wkb_sched_emitted(void* h) { return ((Scheduler*)h)->emitted; }
int64_t wkb_sched_admitted(void* h) { return ((Scheduler*)h)->admitted; }
int64_t wkb_sched_completed(void* h) { return ((Scheduler*)h)->completed; }
int64_t wkb_sched_is_idle(void* h) { auto* s = (Scheduler*)h; return (s->waiting.empty() && s->num_active() == 0) ? 1 : 0; }
int64_t wkb_sched_output_len(void* h, int64_t request) {
  auto* s = (Scheduler*)h;
  return request < 0 || request >= (int64_t)s->outputs.size() ? -1 : (int64_t)s->outputs[(size_t)request].size();
}
int64_t wkb_sched_output(void* h, int64_t request, int32_t* out, int64_t cap) {
  auto* s = (Scheduler*)h;
  if (request < 0 || request >= (int64_t)s->outputs.size()) return -1;
  auto& o = s->outputs[(size_t)request];
  int64_t n = std::min<int64_t>(cap, (int64_t)o.size());
  std::copy(o.begin(), o.begin() + n, out);
  return n;
}
}
