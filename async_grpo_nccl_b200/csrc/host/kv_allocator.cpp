#include "kv_allocator.h"

#include <algorithm>
#include <stdexcept>

namespace agrpo {

BlockAllocator::BlockAllocator(int num_blocks) : ref_(num_blocks, 0) {
  free_.reserve(num_blocks);
  for (int i = num_blocks - 1; i >= 0; --i) free_.push_back(i);
}
int BlockAllocator::alloc() {
  if (free_.empty()) return -1;
  const int b = free_.back();
  free_.pop_back();
  ref_[b] = 1;
  return b;
}
void BlockAllocator::incref(int block) {
  if (block < 0 || block >= (int)ref_.size() || ref_[block] <= 0) throw std::runtime_error("incref of a free block");
  ++ref_[block];
}
void BlockAllocator::release(int block) {
  if (block < 0 || block >= (int)ref_.size() || ref_[block] <= 0) throw std::runtime_error("release of a free block");
  if (--ref_[block] == 0) free_.push_back(block);
}

Scheduler::Scheduler(int num_blocks, int block_size, int max_seqs, int max_blocks_per_seq, int max_prefill_tokens)
    : alloc_(num_blocks), block_size_(block_size), max_seqs_(max_seqs), max_blocks_per_seq_(max_blocks_per_seq),
      max_prefill_tokens_(max_prefill_tokens), slot_owner_(max_seqs, -1) {
  for (int s = max_seqs - 1; s >= 0; --s) free_slots_.push_back(s);
}

void Scheduler::add_group(const GroupRequest& req) {
  if (req.n <= 0 || req.prompt_len <= 0) throw std::runtime_error("add_group: empty request");
  if (!req.forced_new_tokens.empty() && (int)req.forced_new_tokens.size() != req.n)
    throw std::runtime_error("add_group: forced_new_tokens needs one entry per sample");
  const int max_total = req.prompt_len + req.max_new_tokens;
  if ((max_total + block_size_ - 1) / block_size_ > max_blocks_per_seq_)
    throw std::runtime_error("add_group: sequence would exceed max_blocks_per_seq");
  if (req.n > max_seqs_) throw std::runtime_error("add_group: n exceeds max_seqs");
  waiting_.push_back(req);
}

PrefillPlan Scheduler::plan_prefill() {
  PrefillPlan plan;
  int tokens = 0;
  while (!waiting_.empty()) {
    const GroupRequest& g = waiting_.front();
    const int full = g.prompt_len / block_size_;
    const int rem = g.prompt_len % block_size_;
    // blocks: shared full blocks + one private block per child for the partial tail (or the first new token)
    const int need_blocks = full + g.n;
    // keep one spare block per running sequence so that the next decode steps do not immediately preempt
    const int reserve = num_running_ + g.n;
    if ((int)free_slots_.size() < g.n) break;
    if (alloc_.num_free() < need_blocks + reserve) break;
    if (!plan.group_ids.empty() && tokens + g.prompt_len > max_prefill_tokens_) break;
    // shared prompt blocks
    std::vector<int> shared(full);
    for (int b = 0; b < full; ++b) shared[b] = alloc_.alloc();
    std::vector<int> tails(g.n);
    for (int c = 0; c < g.n; ++c) tails[c] = alloc_.alloc();
    // slot mapping for the prompt tokens: full blocks, then child 0's tail block
    for (int p = 0; p < g.prompt_len; ++p) {
      const int bi = p / block_size_;
      const int blk = bi < full ? shared[bi] : tails[0];
      plan.slot_mapping.push_back(blk * block_size_ + p % block_size_);
    }
    for (int c = 0; c < g.n; ++c) {
      SeqState s;
      s.seq_id = next_seq_id_++;
      s.group_id = g.group_id;
      s.child = c;
      s.slot = free_slots_.back();
      free_slots_.pop_back();
      slot_owner_[s.slot] = s.seq_id;
      s.prompt_len = g.prompt_len;
      s.len = g.prompt_len;
      s.max_len = g.prompt_len + g.max_new_tokens;
      s.forced_len = g.forced_new_tokens.empty() ? -1 : g.prompt_len + g.forced_new_tokens[c];
      s.blocks = shared;
      if (c > 0)
        for (int b : shared) alloc_.incref(b);
      s.blocks.push_back(tails[c]);
      if (c > 0 && rem > 0) {
        plan.copy_src.push_back(tails[0]);
        plan.copy_dst.push_back(tails[c]);
      }
      for (int b = 0; b < (int)s.blocks.size(); ++b) plan.updates.push_back({s.slot, b, s.blocks[b]});
      plan.seq_ids.push_back(s.seq_id);
      plan.seq_slots.push_back(s.slot);
      seqs_.emplace(s.seq_id, std::move(s));
      ++num_running_;
    }
    plan.group_ids.push_back(g.group_id);
    plan.prompt_lens.push_back(g.prompt_len);
    tokens += g.prompt_len;
    waiting_.pop_front();
  }
  return plan;
}

DecodePlan Scheduler::plan_decode() {
  DecodePlan plan;
  // The token produced by the previous step (or by prefill) is written at position `len`; make sure its block exists.
  std::vector<SeqState*> order;
  for (int slot = 0; slot < max_seqs_; ++slot) {
    if (slot_owner_[slot] < 0) continue;
    auto it = seqs_.find(slot_owner_[slot]);
    if (it == seqs_.end() || it->second.finished) continue;
    order.push_back(&it->second);
  }
  for (SeqState* s : order) {
    if (s->slot < 0) continue;  // preempted earlier in this loop
    const int need_index = s->len / block_size_;
    while ((int)s->blocks.size() <= need_index) {
      int b = alloc_.alloc();
      if (b < 0) {
        // Pool exhausted: evict the youngest running sequence (highest seq id) other than this one.
        SeqState* victim = nullptr;
        for (SeqState* o : order)
          if (o != s && o->slot >= 0 && (victim == nullptr || o->seq_id > victim->seq_id)) victim = o;
        if (victim == nullptr) throw std::runtime_error("KV cache too small for a single sequence");
        plan.preempted.push_back(victim->seq_id);
        release_seq(*victim);
        continue;
      }
      s->blocks.push_back(b);
      plan.updates.push_back({s->slot, (int)s->blocks.size() - 1, b});
    }
  }
  for (SeqState* s : order) {
    if (s->slot < 0) continue;
    s->len += 1;
    plan.active_slots.push_back(s->slot);
    plan.batch_rows = std::max(plan.batch_rows, s->slot + 1);
  }
  plan.num_active = (int)plan.active_slots.size();
  // drop table updates that belong to sequences evicted later in the same pass
  plan.updates.erase(std::remove_if(plan.updates.begin(), plan.updates.end(),
                                    [&](const TableUpdate& u) { return slot_owner_[u.slot] < 0; }),
                     plan.updates.end());
  return plan;
}

void Scheduler::release_seq(SeqState& s) {
  for (int b : s.blocks) alloc_.release(b);
  s.blocks.clear();
  if (s.slot >= 0) {
    slot_owner_[s.slot] = -1;
    free_slots_.push_back(s.slot);
    s.slot = -1;
    --num_running_;
  }
  s.finished = true;
}

int Scheduler::highest_slot() const {
  for (int s = max_seqs_ - 1; s >= 0; --s)
    if (slot_owner_[s] >= 0) return s;
  return -1;
}

std::vector<std::pair<int, int>> Scheduler::compact_slots() {
  std::vector<std::pair<int, int>> moves;
  int lo = 0, hi = max_seqs_ - 1;
  while (true) {
    while (lo < max_seqs_ && slot_owner_[lo] >= 0) ++lo;  // lowest free slot
    while (hi >= 0 && slot_owner_[hi] < 0) --hi;           // highest occupied slot
    if (lo >= hi || hi < 0) break;
    const long long id = slot_owner_[hi];
    auto it = seqs_.find(id);
    if (it == seqs_.end()) {  // stale owner entry: just drop it
      slot_owner_[hi] = -1;
      continue;
    }
    it->second.slot = lo;
    slot_owner_[lo] = id;
    slot_owner_[hi] = -1;
    moves.emplace_back(hi, lo);
  }
  // free list ordered so that the next admission takes the lowest free slot
  free_slots_.clear();
  for (int s = max_seqs_ - 1; s >= 0; --s)
    if (slot_owner_[s] < 0) free_slots_.push_back(s);
  return moves;
}

void Scheduler::finish(long long seq_id) {
  auto it = seqs_.find(seq_id);
  if (it == seqs_.end()) return;
  if (!it->second.finished || it->second.slot >= 0) release_seq(it->second);
  seqs_.erase(it);
}

const SeqState* Scheduler::seq(long long seq_id) const {
  auto it = seqs_.find(seq_id);
  return it == seqs_.end() ? nullptr : &it->second;
}
const SeqState* Scheduler::seq_at_slot(int slot) const {
  if (slot < 0 || slot >= max_seqs_ || slot_owner_[slot] < 0) return nullptr;
  return seq(slot_owner_[slot]);
}
int Scheduler::seq_len_at_slot(int slot) const {
  const SeqState* s = seq_at_slot(slot);
  return s ? s->len : 0;
}

}  // namespace agrpo
