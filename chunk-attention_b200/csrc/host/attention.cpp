#include "attention.h"

#include <chrono>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cstring>
#include <iostream>
#include <stdexcept>

namespace ca_host {
namespace {

void check_rc(int rc, const char* what) {
    if (rc != CA_OK) throw std::runtime_error(std::string(what) + ": " + ca_last_error());
}

}  // namespace

Attention::Attention(int n_heads, int d_head, int chunk_size, int memory_mb, bool share_prefix, int tpp_threshold,
                     torch::Dtype dtype, torch::Device device)
  : n_heads_(n_heads), d_head_(d_head), chunk_size_(chunk_size), memory_mb_(memory_mb),
    tpp_threshold_(tpp_threshold), share_prefix_(share_prefix),
    options_(torch::TensorOptions().dtype(dtype).layout(torch::kStrided).device(device).requires_grad(false)) {
    init();
}

Attention::Attention(Attention& other)
  : n_heads_(other.n_heads_), d_head_(other.d_head_), chunk_size_(other.chunk_size_), memory_mb_(other.memory_mb_),
    tpp_threshold_(other.tpp_threshold_), share_prefix_(other.share_prefix_), options_(other.options_) {
    init();
    shared_plan_ = other.shared_plan_;  // same configuration, same sequence of tree operations: same work lists
}

void Attention::init() {
    if (!options_.device().is_cuda())
        throw std::runtime_error(
            "chunk_attn (B200 build) computes on CUDA devices only and has no CPU path: got device " +
            options_.device().str());
    if (n_heads_ <= 0 || d_head_ <= 0 || chunk_size_ <= 0 || memory_mb_ < 0)
        throw std::runtime_error("n_heads, d_head, chunk_size must be positive");
    const auto st = c10::typeMetaToScalarType(options_.dtype());
    if (st == torch::kFloat16) {
        ca_dtype_ = CA_DTYPE_F16;
    } else if (st == torch::kFloat32) {
        ca_dtype_ = CA_DTYPE_F32;
    } else {
        throw std::runtime_error(std::string("unsupported dtype ") + c10::toString(st));
    }
    if (!options_.device().has_index())
        options_ = options_.device(torch::Device(torch::kCUDA, c10::cuda::current_device()));
    chunk_bytes_ = ca_chunk_bytes(n_heads_, d_head_, chunk_size_, ca_dtype_);
    // same sizing rule as the reference's allocator: as many whole chunks as memory_mb holds
    max_chunks_ = (int64_t)((double)memory_mb_ * 1024.0 * 1024.0 / (double)chunk_bytes_);
    c10::cuda::CUDAGuard guard(options_.device());
    pool_ = torch::empty({std::max<int64_t>(max_chunks_, 1) * chunk_bytes_}, options_.dtype(torch::kUInt8));
    tree_.reset(new PrefixTree(chunk_size_, max_chunks_, chunk_bytes_, share_prefix_));
    check_rc(ca_context_create(&ctx_, options_.device().index(), n_heads_, d_head_, chunk_size_, ca_dtype_,
                               pool_.data_ptr(), max_chunks_, tpp_threshold_),
             "chunk_attn: context");
    valid_ = false;
    shared_plan_ = std::make_shared<SharedPlan>();
}

Attention::SharedPlan::~SharedPlan() {
    if (plan) ca_plan_destroy(plan);
}

Attention::~Attention() {
    if (worker_.joinable()) {
        {
            std::lock_guard<std::mutex> lock(worker_mutex_);
            worker_stop_ = true;
        }
        worker_cv_.notify_all();
        worker_.join();
    }
    if (ctx_) ca_context_destroy(ctx_);
}

void Attention::worker_loop() {
    for (;;) {
        std::function<void()> task;
        {
            std::unique_lock<std::mutex> lock(worker_mutex_);
            worker_cv_.wait(lock, [this] { return worker_stop_ || !worker_queue_.empty(); });
            if (worker_queue_.empty()) return;  // stop requested and nothing left to run
            task = std::move(worker_queue_.front());
            worker_queue_.pop_front();
        }
        task();
    }
}

void* Attention::stream() const {
    return c10::cuda::getCurrentCUDAStream(options_.device().index()).stream();
}

torch::Tensor Attention::to_cache(torch::Tensor t) const {
    if (t.device() != options_.device() || t.scalar_type() != c10::typeMetaToScalarType(options_.dtype()))
        t = t.to(options_);
    if (t.dim() > 0 && t.stride(t.dim() - 1) != 1) t = t.contiguous();
    return t;
}

int Attention::add_seq(const std::vector<int>& tokens, torch::Tensor k, torch::Tensor v) {
    if (k.dim() != 3 || v.dim() != 3 || k.size(0) != v.size(0) || k.size(1) != n_heads_ || v.size(1) != n_heads_ ||
        k.size(2) != d_head_ || v.size(2) != d_head_)
        throw std::runtime_error("add_seq: k and v must be [n_tokens, n_heads, d_head]");
    // rows past the last token (a right-padded prompt) are ignored, as the reference's slices do
    if (k.size(0) < (int64_t)tokens.size()) throw std::runtime_error("add_seq: one K/V row per token is required");
    std::vector<NewChunk> created;
    const int seq_idx = tree_->add_seq(tokens, created);
    valid_ = false;
    if (!created.empty()) {
        // the new chunks hold one contiguous token range: a single scatter fills them all.  K/V of
        // the matched prefix are not read (the first sequence that brought a chunk wrote it).
        k = to_cache(k);
        v = to_cache(v);
        if (k.strides() != v.strides()) {
            k = k.contiguous();
            v = v.contiguous();
        }
        std::vector<int32_t> ids;
        ids.reserve(created.size());
        int n_tokens = 0;
        for (const NewChunk& nc : created) {
            ids.push_back(nc.chunk->id);
            n_tokens += nc.n_tokens;
        }
        c10::cuda::CUDAGuard guard(options_.device());
        check_rc(ca_scatter_prefill(ctx_, k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), created.front().token_start,
                                    n_tokens, ids.data(), stream()),
                 "add_seq");
    }
    return seq_idx;
}

std::shared_ptr<std::future<int>> Attention::add_seq_async(const std::vector<int>& tokens, torch::Tensor k,
                                                           torch::Tensor v) {
    // The reference declares this and throws (cpp/chunk_attn/attention.cpp:195-208).  Here the
    // insertion runs on this object's worker thread; the tensors are held by value until it is done.
    auto promise = std::make_shared<std::promise<int>>();
    auto future = std::make_shared<std::future<int>>(promise->get_future());
    const c10::cuda::CUDAStream caller_stream = c10::cuda::getCurrentCUDAStream(options_.device().index());
    {
        std::lock_guard<std::mutex> lock(worker_mutex_);
        if (!worker_.joinable()) worker_ = std::thread([this] { worker_loop(); });
        worker_queue_.emplace_back([this, promise, tokens, k, v, caller_stream]() mutable {
            try {
                c10::cuda::CUDAStreamGuard guard(caller_stream);  // the current stream is per thread
                promise->set_value(add_seq(tokens, k, v));
            } catch (...) {
                promise->set_exception(std::current_exception());
            }
            k.reset();
            v.reset();
        });
    }
    worker_cv_.notify_one();
    return future;
}

int Attention::append_completion(int seq_idx, const std::vector<int>& tokens, torch::Tensor k, torch::Tensor v) {
    const int64_t n = (int64_t)tokens.size();
    if (k.dim() != 3 || v.dim() != 3 || k.size(0) != n || v.size(0) != n || k.size(1) != n_heads_ || v.size(1) != n_heads_ ||
        k.size(2) != d_head_ || v.size(2) != d_head_)
        throw std::runtime_error("append_completion: k and v must be [n_tokens, n_heads, d_head]");
    std::vector<std::pair<Chunk*, Chunk*>> pairs;
    std::vector<std::pair<Chunk*, int>> slots;
    tree_->append_completion(seq_idx, tokens, pairs, slots);
    valid_ = false;
    k = to_cache(k);
    v = to_cache(v);
    if (k.strides() != v.strides()) {
        k = k.contiguous();
        v = v.contiguous();
    }
    c10::cuda::CUDAGuard guard(options_.device());
    if (!pairs.empty()) {  // copy-on-write of the forked leaf, before the beams diverge
        std::vector<int32_t> src, dst;
        for (auto& p : pairs) {
            src.push_back(p.first->id);
            dst.push_back(p.second->id);
        }
        check_rc(ca_copy_chunks(ctx_, src.data(), dst.data(), (int)src.size(), stream()), "append_completion");
    }
    std::vector<int32_t> ids, rows;
    for (auto& s : slots) {
        ids.push_back(s.first->id);
        rows.push_back(s.second);
    }
    check_rc(ca_scatter_rows(ctx_, k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), (int)ids.size(), ids.data(),
                             rows.data(), stream()),
             "append_completion");
    return seq_idx;
}

void Attention::remove_seq(int seq_idx) {
    tree_->remove_seq(seq_idx);
    valid_ = false;
}

std::vector<Chunk*> Attention::reserve() {
    std::vector<Chunk*> fresh = tree_->reserve();
    if (!fresh.empty()) valid_ = false;
    return fresh;
}

namespace {
inline int64_t now_ns() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

void Attention::refresh_kernel_context(bool force) {
    if (!force && valid_) return;
    const int64_t t0 = now_ns();
    std::vector<ca_chunk_info> infos = tree_->get_chunks();
    const int64_t t1 = now_ns();
    c10::cuda::CUDAGuard guard(options_.device());
    SharedPlan& sp = *shared_plan_;
    const bool same = sp.plan != nullptr && sp.n_seqs == tree_->n_seqs() && sp.infos.size() == infos.size() &&
                      (infos.empty() || std::memcmp(sp.infos.data(), infos.data(), infos.size() * sizeof(ca_chunk_info)) == 0);
    if (!same) {
        sp.n_seqs = -1;  // nothing to reuse if the rebuild below is refused
        check_rc(ca_plan_build_for_context(ctx_, &sp.plan, infos.data(), (int)infos.size(), tree_->n_seqs()),
                 "refresh_kernel_context");
        sp.infos.swap(infos);
        sp.n_seqs = tree_->n_seqs();
        sp.builds++;
    } else {
        sp.reuses++;
    }
    const int64_t t2 = now_ns();
    check_rc(ca_refresh_from_plan(ctx_, sp.plan, stream()), "refresh_kernel_context");
    valid_ = true;
    const int64_t t3 = now_ns();
    host_times_.refreshes++;
    host_times_.walk_ns += t1 - t0;
    host_times_.plan_ns += t2 - t1;
    host_times_.upload_ns += t3 - t2;
}

std::vector<Chunk*> Attention::append_token(const std::vector<int>& tokens, torch::Tensor k, torch::Tensor v, bool) {
    if (tree_->tails().size() != tokens.size()) throw std::runtime_error("num of seqs is not equal to num of tokens");
    const int64_t n = (int64_t)tokens.size();
    if (k.dim() != 3 || v.dim() != 3 || k.size(0) != n || v.size(0) != n || k.size(1) != n_heads_ ||
        v.size(1) != n_heads_ || k.size(2) != d_head_ || v.size(2) != d_head_)
        throw std::runtime_error("append_token: k and v must be [n_seqs, n_heads, d_head]");
    std::vector<Chunk*> fresh = reserve();
    refresh_kernel_context(false);
    k = to_cache(k).contiguous();
    v = to_cache(v).contiguous();
    c10::cuda::CUDAGuard guard(options_.device());
    check_rc(ca_append_kv(ctx_, k.data_ptr(), v.data_ptr(), (int)n, stream()), "append_token");
    tree_->append_token_ids(tokens);
    return fresh;
}

void Attention::clear() {
    tree_->clear();
    valid_ = false;
}

void Attention::duplicate(int seq_idx, int copies) {
    std::vector<std::pair<Chunk*, Chunk*>> pairs;
    tree_->duplicate(seq_idx, copies, pairs);
    if (pairs.empty()) return;
    valid_ = false;
    std::vector<int32_t> src, dst;
    for (auto& p : pairs) {
        src.push_back(p.first->id);
        dst.push_back(p.second->id);
    }
    c10::cuda::CUDAGuard guard(options_.device());
    check_rc(ca_copy_chunks(ctx_, src.data(), dst.data(), (int)src.size(), stream()), "duplicate");
}

torch::Tensor Attention::forward(torch::Tensor q, int partition) {
    if (!q.is_contiguous()) throw std::runtime_error("q is not contiguous");
    if (q.dim() != 3 || q.size(1) != n_heads_ || q.size(2) != d_head_)
        throw std::runtime_error("forward: q must be [n_seqs, n_heads, d_head]");
    if (q.size(0) != (int64_t)tree_->n_seqs()) throw std::runtime_error("forward: one query row per live sequence is required");
    if (q.device() != options_.device() || q.scalar_type() != c10::typeMetaToScalarType(options_.dtype()))
        throw std::runtime_error("forward: q must have the dtype and device of the cache");
    if (partition < 0 || partition > 2) throw std::runtime_error("Unsupported partition type");
    c10::cuda::CUDAGuard guard(options_.device());
    torch::Tensor output = torch::empty({q.size(0), n_heads_, d_head_}, options_);
    refresh_kernel_context(false);
    check_rc(ca_attention(ctx_, q.data_ptr(), output.data_ptr(), (int)q.size(0), partition, stream()), "forward");
    return output;
}

torch::Tensor Attention::forward_host(torch::Tensor q, c10::optional<torch::Tensor> out, int partition) {
    const auto st = c10::typeMetaToScalarType(options_.dtype());
    if (q.is_cuda()) throw std::runtime_error("forward_host: q must be a CPU tensor (use forward for device tensors)");
    if (!q.is_contiguous()) throw std::runtime_error("q is not contiguous");
    if (q.dim() != 3 || q.size(1) != n_heads_ || q.size(2) != d_head_ || q.scalar_type() != st)
        throw std::runtime_error("forward_host: q must be [n_seqs, n_heads, d_head] with the dtype of the cache");
    if (q.size(0) != (int64_t)tree_->n_seqs()) throw std::runtime_error("forward: one query row per live sequence is required");
    if (partition < 0 || partition > 2) throw std::runtime_error("Unsupported partition type");
    torch::Tensor result;
    if (out.has_value()) {
        result = *out;
        if (result.is_cuda() || !result.is_contiguous() || result.sizes() != q.sizes() || result.scalar_type() != st)
            throw std::runtime_error("forward_host: out must be a contiguous CPU tensor shaped and typed like q");
    } else {
        result = torch::empty(q.sizes(), torch::TensorOptions().dtype(st).device(torch::kCPU).pinned_memory(true));
    }
    c10::cuda::CUDAGuard guard(options_.device());
    refresh_kernel_context(false);
    check_rc(ca_attention_host(ctx_, q.data_ptr(), result.data_ptr(), (int)q.size(0), partition, stream()), "forward_host");
    return result;
}

void Attention::forward_to_peers(torch::Tensor q, const std::vector<int64_t>& peer_out_ptrs, int total_heads,
                                 int head_offset, int64_t multicast_ptr) {
    if (!q.is_contiguous()) throw std::runtime_error("q is not contiguous");
    if (q.dim() != 3 || q.size(0) != (int64_t)tree_->n_seqs() || q.size(1) != n_heads_ || q.size(2) != d_head_ ||
        q.device() != options_.device() || q.scalar_type() != c10::typeMetaToScalarType(options_.dtype()))
        throw std::runtime_error("forward_to_peers: q must be [n_seqs, n_heads, d_head] with the dtype and device of the cache");
    std::vector<void*> ptrs;
    for (int64_t p : peer_out_ptrs) ptrs.push_back(reinterpret_cast<void*>(p));
    c10::cuda::CUDAGuard guard(options_.device());
    refresh_kernel_context(false);
    check_rc(ca_attention_to_peers(ctx_, q.data_ptr(), ptrs.data(), (int)ptrs.size(), reinterpret_cast<void*>(multicast_ptr),
                                   total_heads, head_offset, (int)q.size(0), stream()),
             "forward_to_peers");
}

void Attention::print(Chunk* root, int level) {
    if (root == nullptr) root = tree_->root();
    std::string indent(4 * level, ' ');
    std::cout << indent << root->to_string(true) << std::endl;
    for (Chunk* child : root->children) print(child, level + 1);
}

ca_plan_stats Attention::plan_stats() {
    refresh_kernel_context(false);
    ca_plan_stats st;
    check_rc(ca_context_stats(ctx_, &st), "plan_stats");
    return st;
}

void Attention::set_option(int option, int64_t value) {
    check_rc(ca_context_set_option(ctx_, option, value), "set_option");
    valid_ = false;
    shared_plan_ = std::make_shared<SharedPlan>();  // its work lists now differ from its siblings'
}

void Attention::attn_partials(torch::Tensor q, int phases) {
    if (!q.is_contiguous() || q.dim() != 3 || q.size(0) != (int64_t)tree_->n_seqs() || q.size(1) != n_heads_ ||
        q.size(2) != d_head_ || q.device() != options_.device() ||
        q.scalar_type() != c10::typeMetaToScalarType(options_.dtype()))
        throw std::runtime_error("attn_partials: q must be a contiguous [n_seqs, n_heads, d_head] tensor of the cache's dtype and device");
    c10::cuda::CUDAGuard guard(options_.device());
    refresh_kernel_context(false);
    check_rc(ca_attn_partials(ctx_, q.data_ptr(), (int)q.size(0), phases, stream()), "attn_partials");
}

void Attention::attn_merge(torch::Tensor out) {
    if (!out.is_contiguous() || out.dim() != 3 || out.size(0) != (int64_t)tree_->n_seqs() || out.size(1) != n_heads_ ||
        out.size(2) != d_head_ || out.device() != options_.device() ||
        out.scalar_type() != c10::typeMetaToScalarType(options_.dtype()))
        throw std::runtime_error("attn_merge: out must be a contiguous [n_seqs, n_heads, d_head] tensor of the cache's dtype and device");
    c10::cuda::CUDAGuard guard(options_.device());
    check_rc(ca_attn_merge(ctx_, out.data_ptr(), (int)out.size(0), stream()), "attn_merge");
}

int Attention::device_status() {
    int32_t st = 0;
    c10::cuda::CUDAGuard guard(options_.device());
    const int rc = ca_status_read(ctx_, stream(), &st);
    if (rc != CA_OK && rc != CA_ERR_DEVICE_STATUS) check_rc(rc, "device_status");
    return st;
}

}  // namespace ca_host
