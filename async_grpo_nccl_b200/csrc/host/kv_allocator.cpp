#include "kv_allocator.h"

#include <algorithm>
#include <stdexcept>

namespace agrpo {

BlockAllocator::BlockAllocator(int num_blocks)
    : ref_(num_blocks, 0), hash_(num_blocks, 0ull), gen_(num_blocks, 0u), evict_stamp_(num_blocks, 0u) {
  free_.reserve(num_blocks);
  for (int i = num_blocks - 1; i >= 0; --i) free_.push_back(i);
}
int BlockAllocator::alloc() {
  int b = -1;
  if (!free_.empty()) {
    b = free_.back();
    free_.pop_back();
  } else {
    while (!evictable_.empty()) {  // oldest cached block without users
      const auto e = evictable_.front();
      evictable_.pop_front();
      if (evict_stamp_[e.first] != e.second || ref_[e.first] != 0) continue;  // stale entry
      b = e.first;
      evict_stamp_[b] = 0;
      --n_evictable_;
      cached_.erase(hash_[b]);
      hash_[b] = 0;
      break;
    }
    if (b < 0) return -1;
  }
  ref_[b] = 1;
  ++gen_[b];
  return b;
}
void BlockAllocator::incref(int block) {
  if (block < 0 || block >= (int)ref_.size() || ref_[block] <= 0) throw std::runtime_error("incref of a free block");
  ++ref_[block];
}
void BlockAllocator::push_evictable(int block) {
  evict_stamp_[block] = next_stamp_++;
  if (next_stamp_ == 0) next_stamp_ = 1;
  evictable_.emplace_back(block, evict_stamp_[block]);
  ++n_evictable_;
}
void BlockAllocator::release(int block) {
  if (block < 0 || block >= (int)ref_.size() || ref_[block] <= 0) throw std::runtime_error("release of a free block");
  if (--ref_[block] == 0) {
    if (hash_[block] != 0) push_evictable(block);
    else free_.push_back(block);
  }
}
int BlockAllocator::lookup(unsigned long long hash) const {
  if (hash == 0) return -1;
  auto it = cached_.find(hash);
  return it == cached_.end() ? -1 : it->second;
}
void BlockAllocator::acquire(int block) {
  if (block < 0 || block >= (int)ref_.size() || hash_[block] == 0) throw std::runtime_error("acquire of a block that is not cached");
  if (ref_[block] == 0) {
    evict_stamp_[block] = 0;  // its queue entry is now stale
    --n_evictable_;
  }
  ++ref_[block];
}
void BlockAllocator::set_hash(int block, unsigned long long hash, unsigned int generation) {
  if (hash == 0 || block < 0 || block >= (int)ref_.size()) return;
  if (gen_[block] != generation || ref_[block] <= 0 || hash_[block] != 0) return;  // handed out again, or already known
  if (cached_.count(hash)) return;  // another block already holds this chain
  cached_[hash] = block;
  hash_[block] = hash;
}
void BlockAllocator::clear_cache() {
  for (const auto& kv : cached_) {
    const int b = kv.second;
    hash_[b] = 0;
    if (ref_[b] == 0) {
      evict_stamp_[b] = 0;
      free_.push_back(b);
    }
  }
  cached_.clear();
  evictable_.clear();
  n_evictable_ = 0;
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
  commit_pending_hashes();
  int tokens = 0;
  while (!waiting_.empty()) {
    const GroupRequest& g = waiting_.front();
    const int full = g.prompt_len / block_size_;
    const int rem = g.prompt_len % block_size_;
    // leading full blocks that the prefix cache already holds (at least one prompt token is always computed: its
    // hidden state is what the first sampled token comes from)
    std::vector<int> hit_blocks;
    int hit_unused = 0;
    {
      const int lim = std::min(full, (int)g.block_hashes.size());
      while ((int)hit_blocks.size() < lim) {
        const int b = alloc_.lookup(g.block_hashes[hit_blocks.size()]);
        if (b < 0) break;
        hit_blocks.push_back(b);
      }
      if (!hit_blocks.empty() && (int)hit_blocks.size() * block_size_ == g.prompt_len) hit_blocks.pop_back();
      for (int b : hit_blocks) hit_unused += alloc_.refcount(b) == 0 ? 1 : 0;
    }
    const int hit = (int)hit_blocks.size();
    const int cached = hit * block_size_;
    // blocks: shared full blocks + one private block per child for the partial tail (or the first new token)
    const int need_blocks = (full - hit) + g.n;
    // keep one spare block per running sequence so that the next decode steps do not immediately preempt
    const int reserve = num_running_ + g.n;
    if ((int)free_slots_.size() < g.n) break;
    if (alloc_.num_free() - hit_unused < need_blocks + reserve) break;  // hit blocks without users count as free today
    if (!plan.group_ids.empty() && tokens + (g.prompt_len - cached) > max_prefill_tokens_) break;
    // shared prompt blocks: the cached ones, then new ones
    std::vector<int> shared(full);
    for (int b = 0; b < hit; ++b) {
      alloc_.acquire(hit_blocks[b]);
      shared[b] = hit_blocks[b];
    }
    for (int b = hit; b < full; ++b) {
      shared[b] = alloc_.alloc();
      if (b < (int)g.block_hashes.size())
        pending_hashes_.push_back({shared[b], g.block_hashes[b], alloc_.generation(shared[b])});
    }
    std::vector<int> tails(g.n);
    for (int c = 0; c < g.n; ++c) tails[c] = alloc_.alloc();
    // slot mapping for the prompt tokens: full blocks, then child 0's tail block
    for (int p = 0; p < g.prompt_len; ++p) {
      const int bi = p / block_size_;
      const int blk = bi < full ? shared[bi] : tails[0];
      (p < cached ? plan.prefix_slots : plan.slot_mapping).push_back(blk * block_size_ + p % block_size_);
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
    plan.cached_lens.push_back(cached);
    tokens += g.prompt_len - cached;
    waiting_.pop_front();
  }
  return plan;
}

// What the last planned prefill computes is in the cache by the time the scheduler is called again: from then on other
// prompts may find those blocks (and they stay findable after their sequences finish).
void Scheduler::commit_pending_hashes() {
  for (const PendingHash& ph : pending_hashes_) alloc_.set_hash(ph.block, ph.hash, ph.generation);
  pending_hashes_.clear();
}

DecodePlan Scheduler::plan_decode() {
  DecodePlan plan;
  commit_pending_hashes();
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
  commit_pending_hashes();
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
