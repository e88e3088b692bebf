// Paged KV-cache block allocator and continuous-batching scheduler for the native rollout engine
// (host side, no CUDA). They take over the parts of vLLM's engine core that the reference relies on
// for generation (vllm_worker.py:203-284): block accounting with reference counts so that the n
// samples of one prompt share the prompt's blocks, admission control, slot assignment, preemption
// when the pool runs dry, and per-step block-table updates. Prefix caching across requests (vllm_worker.py:224,
// enable_prefix_caching): a full prompt block carries the hash of the token chain up to and including it; a block whose
// last user has gone stays findable under that hash until the pool needs it back (least recently released first), and a
// later prompt that starts with the same chain takes those blocks instead of recomputing them.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace agrpo {

class BlockAllocator {
 public:
  explicit BlockAllocator(int num_blocks);
  int num_blocks() const { return (int)ref_.size(); }
  // blocks that alloc() can hand out: never-hashed free blocks plus cached blocks nobody uses
  int num_free() const { return (int)free_.size() + n_evictable_; }
  // Returns a block id with refcount 1, or -1 when the pool is empty. Takes a plain free block when there is one,
  // otherwise evicts the cached block that has been unused for the longest time.
  int alloc();
  void incref(int block);
  // Drops one reference; at zero the block returns to the pool (it stays findable by its hash until it is evicted).
  void release(int block);
  int refcount(int block) const { return ref_[block]; }
  // ---- prefix cache ----
  int lookup(unsigned long long hash) const;          // block holding this chain, or -1
  void acquire(int block);                            // one more user of a cached block (it may have had none)
  // The block now holds the chain `hash`. `generation` must be the value generation(block) had when the caller
  // allocated it: a block that was released and handed out again in the meantime is not registered.
  void set_hash(int block, unsigned long long hash, unsigned int generation);
  unsigned int generation(int block) const { return gen_[block]; }
  int num_cached() const { return (int)cached_.size(); }
  void clear_cache();                                 // forget every hash (the weights changed)

 private:
  void push_evictable(int block);
  std::vector<int> ref_;
  std::vector<int> free_;
  std::vector<unsigned long long> hash_;              // 0 = none
  std::vector<unsigned int> gen_;                     // bumped by every alloc()
  std::vector<unsigned int> evict_stamp_;             // stamp of the block's live entry in evictable_, 0 = not in it
  std::deque<std::pair<int, unsigned int>> evictable_;  // (block, stamp), oldest first; stale entries are skipped
  std::unordered_map<unsigned long long, int> cached_;
  int n_evictable_ = 0;
  unsigned int next_stamp_ = 1;
};

struct SeqState {
  long long seq_id = -1;
  long long group_id = -1;     // request (prompt) this sequence belongs to
  int child = 0;               // index within the group
  int slot = -1;               // row in the decode batch, -1 while waiting
  int prompt_len = 0;
  int len = 0;                 // tokens whose KV is (or is about to be) in the cache
  int max_len = 0;             // prompt_len + max new tokens
  int forced_len = -1;         // total length at which generation is cut (EOS forced), -1 = none
  bool finished = false;
  std::vector<int> blocks;
};

struct TableUpdate { int slot, index, block; };

struct GroupRequest {
  long long group_id;
  int prompt_len;
  int n;
  int max_new_tokens;
  std::vector<int> forced_new_tokens;  // per child, empty = none
  // Hash of the token chain up to and including each full prompt block (prompt_len / block_size entries); empty = this
  // request takes no part in prefix caching. 0 is reserved.
  std::vector<unsigned long long> block_hashes;
};

struct PrefillPlan {
  std::vector<long long> group_ids;     // prompts to prefill this step
  std::vector<int> prompt_lens;
  std::vector<int> cached_lens;         // leading tokens of each prompt whose blocks came from the prefix cache
  std::vector<int> slot_mapping;        // cache slot of every prompt token that has to be computed, prompts concatenated
  std::vector<int> prefix_slots;        // cache slot of every cached prompt token, prompts concatenated
  std::vector<long long> seq_ids;       // children created, n per group in order
  std::vector<int> seq_slots;           // decode-batch row of each child
  std::vector<int> copy_src, copy_dst;  // partial last prompt block: copy src -> dst for children 1..n-1
  std::vector<TableUpdate> updates;     // block-table entries to write on the device
};

struct DecodePlan {
  int batch_rows = 0;                   // highest active slot + 1
  int num_active = 0;
  std::vector<TableUpdate> updates;     // new blocks for sequences crossing a block boundary
  std::vector<int> active_slots;
  std::vector<long long> preempted;     // sequences evicted to make room (caller re-queues their groups)
};

class Scheduler {
 public:
  Scheduler(int num_blocks, int block_size, int max_seqs, int max_blocks_per_seq, int max_prefill_tokens);

  void add_group(const GroupRequest& req);
  int num_waiting() const { return (int)waiting_.size(); }
  int num_running() const { return num_running_; }
  int num_free_blocks() const { return alloc_.num_free(); }
  int num_free_slots() const { return (int)free_slots_.size(); }
  int num_cached_blocks() const { return alloc_.num_cached(); }
  void clear_prefix_cache() { pending_hashes_.clear(); alloc_.clear_cache(); }

  // Admits as many waiting groups as fit (slots, blocks, prefill-token budget). Empty plan = nothing admitted.
  PrefillPlan plan_prefill();
  // Accounts for one more token per running sequence and allocates blocks where a boundary is crossed.
  DecodePlan plan_decode();
  // Marks a sequence finished and frees its slot and blocks.
  void finish(long long seq_id);
  // Moves the sequences in the highest slots into the lowest free slots so that the running sequences occupy a dense
  // prefix of the slot range (the decode batch is as many rows as the highest occupied slot). Returns (from, to) pairs;
  // the caller moves its per-slot state the same way. Blocks stay with their sequences.
  std::vector<std::pair<int, int>> compact_slots();
  int highest_slot() const;
  const SeqState* seq(long long seq_id) const;
  const SeqState* seq_at_slot(int slot) const;
  int seq_len_at_slot(int slot) const;

 private:
  void release_seq(SeqState& s);
  void commit_pending_hashes();
  BlockAllocator alloc_;
  int block_size_, max_seqs_, max_blocks_per_seq_, max_prefill_tokens_;
  std::deque<GroupRequest> waiting_;
  std::unordered_map<long long, SeqState> seqs_;
  std::vector<long long> slot_owner_;
  std::vector<int> free_slots_;
  int num_running_ = 0;
  long long next_seq_id_ = 0;
  // blocks whose content the prefill planned last will have written by the next planning call: only then may another
  // prompt find them (block, hash, generation at allocation)
  struct PendingHash { int block; unsigned long long hash; unsigned int generation; };
  std::vector<PendingHash> pending_hashes_;
};

}  // namespace agrpo
