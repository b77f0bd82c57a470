// ca_host::Attention — the C++ object behind chunk_attn.Attention.
//
// Same constructor arguments, methods, row-order contract and error messages as the reference's
// GPT::Attention (cpp/chunk_attn/attention.h:16-75, cpp/chunk_attn/attention.cpp), so that the
// reference's llama_hf model and ModelHost drive it unchanged.  Differences in substance:
// K/V live in ONE device allocation in the library's private tile layout and every data-path
// operation (prefill scatter, token append, copy-on-write, attention) is a CUDA kernel behind
// the C ABI of include/chunk_attn_b200.h, launched on torch's current stream.  There is no CPU
// implementation: constructing it on a non-CUDA device throws.
#pragma once
#include <torch/torch.h>

#include <condition_variable>
#include <deque>
#include <functional>
#include <future>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "../../../include/chunk_attn_b200.h"
#include "prefix_tree.h"

namespace ca_host {

class Attention {
  public:
    Attention(int n_heads, int d_head, int chunk_size, int memory_mb = 2048, bool share_prefix = true,
              int tpp_threshold = 1, torch::Dtype dtype = torch::kFloat16,
              torch::Device device = torch::Device(torch::kCUDA));
    // same configuration, fresh empty cache (one per transformer layer in the reference's model)
    Attention(Attention& other);
    ~Attention();
    Attention& operator=(const Attention&) = delete;

    int add_seq(const std::vector<int>& tokens, torch::Tensor k, torch::Tensor v);
    // add_seq on a worker thread of this object; the kernels go to the stream that is current on the
    // calling thread now.  Insertions run in the order they were queued.  Until the future is ready
    // no other method of this object may be called (the tree is not locked).
    std::shared_ptr<std::future<int>> add_seq_async(const std::vector<int>& tokens, torch::Tensor k, torch::Tensor v);
    void remove_seq(int seq_idx);
    std::vector<Chunk*> append_token(const std::vector<int>& tokens, torch::Tensor k, torch::Tensor v, bool fused = true);
    void refresh_kernel_context(bool force = false);
    std::vector<Chunk*> reserve();
    void clear();
    int64_t peak_memory_allocated() const { return tree_->pool().peak_memory_allocated(); }
    void duplicate(int seq_idx, int copies);
    // One beam-search step for row seq_idx: it forks into tokens.size() rows (seq_idx, seq_idx + 1, ...),
    // row seq_idx + i continuing with tokens[i] whose K/V are k[i], v[i] ([n_tokens, n_heads, d_head]).
    // Returns seq_idx.
    int append_completion(int seq_idx, const std::vector<int>& tokens, torch::Tensor k, torch::Tensor v);
    torch::Tensor forward(torch::Tensor q, int partition = 0);
    // forward for queries in host memory: returns a CPU tensor (written into `out` when given).  Pinned
    // tensors are used in place, the result rows are stored into host memory by the last kernel, and
    // the call returns when they are there.
    torch::Tensor forward_host(torch::Tensor q, c10::optional<torch::Tensor> out, int partition = 0);
    // head-sharded forward: rows are written into every rank's full-width output buffer (device
    // addresses this GPU can reach), this cache's heads landing at head_offset of total_heads
    // multicast_ptr != 0: a multicast address mapping the same buffer on every rank; rows are then written with one
    // multimem.st each instead of one store per rank
    void forward_to_peers(torch::Tensor q, const std::vector<int64_t>& peer_out_ptrs, int total_heads, int head_offset,
                          int64_t multicast_ptr = 0);

    Chunk* get_trie() { return tree_->root(); }
    std::vector<Chunk*> tails() { return tree_->tails(); }
    void print(Chunk* root = nullptr, int level = 0);
    std::vector<ca_chunk_info> get_chunks() { return tree_->get_chunks(); }

    // introspection used by the benchmark and the tests
    ca_plan_stats plan_stats();
    void set_option(int option, int64_t value);
    int device_status();
    // (plans built, plans reused) by this cache and the caches it shares its work lists with
    std::pair<int64_t, int64_t> plan_sharing() const { return {shared_plan_->builds, shared_plan_->reuses}; }
    // host time spent bringing the work lists up to date since the object was made: the tree walk (get_chunks),
    // planning (or finding the shared plan current) and the upload, in nanoseconds, and how many refreshes
    struct HostTimes { int64_t refreshes = 0, walk_ns = 0, plan_ns = 0, upload_ns = 0; };
    HostTimes host_times() const { return host_times_; }
    // the two launches of forward(), separately (per-kernel timing)
    void attn_partials(torch::Tensor q, int phases);
    void attn_merge(torch::Tensor out);

  private:
    void init();
    void* stream() const;
    torch::Tensor to_cache(torch::Tensor t) const;  // dtype/device of the cache, last dim contiguous

    int n_heads_, d_head_, chunk_size_, memory_mb_, tpp_threshold_;
    bool share_prefix_;
    torch::TensorOptions options_;
    int ca_dtype_ = 0;
    int64_t max_chunks_ = 0;
    int64_t chunk_bytes_ = 0;
    torch::Tensor pool_;  // one uint8 tensor: [max_chunks][n_heads][K|V][chunk_size][d_head]
    std::unique_ptr<PrefixTree> tree_;
    ca_context* ctx_ = nullptr;
    bool valid_ = false;
    HostTimes host_times_;

    // The work list of the current tree, shared by the caches made from one another with
    // Attention(other) (a model's layers): whoever refreshes first after a tree change plans, the
    // others find their chunk list identical and only upload.
    struct SharedPlan {
        std::vector<ca_chunk_info> infos;
        int n_seqs = -1;
        ca_plan* plan = nullptr;
        int64_t builds = 0, reuses = 0;
        ~SharedPlan();
    };
    std::shared_ptr<SharedPlan> shared_plan_;

    // add_seq_async: one worker thread, started on first use, runs the queued insertions in order
    void worker_loop();
    std::thread worker_;
    std::mutex worker_mutex_;
    std::condition_variable worker_cv_;
    std::deque<std::function<void()>> worker_queue_;
    bool worker_stop_ = false;
};

}  // namespace ca_host
