// C ABI of the library (declared in include/chunk_attn_b200.h): argument checking, the context
// that owns the device work lists and the partial-result scratch, and the launch sequence of one
// decode step.  No torch, no exceptions across the boundary.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <new>
#include <string>

#include "../../include/chunk_attn_b200.h"
#include "ca_kernels.h"
#include "ca_plan.h"

namespace {

thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}
int fail_cuda(cudaError_t e, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    return CA_ERR_CUDA;
}
#define CA_CUDA(call)                                        \
    do {                                                     \
        cudaError_t e__ = (call);                            \
        if (e__ != cudaSuccess) return fail_cuda(e__, #call); \
    } while (0)

// Make the context's device current for the duration of a call and put the caller's back after.
struct DeviceGuard {
    int prev = -1;
    bool changed = false;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) {
            err = cudaSetDevice(device);
            changed = (err == cudaSuccess);
        }
    }
    ~DeviceGuard() {
        if (changed) cudaSetDevice(prev);
    }
};

int esize_of(int dtype) { return dtype == CA_DTYPE_F16 ? 2 : (dtype == CA_DTYPE_F32 ? 4 : 0); }

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

namespace ca {
// lets the other translation units of the library leave a message for ca_last_error()
void set_last_error(const std::string& msg) { g_last_error = msg; }
}  // namespace ca

struct ca_plan {
    ca::Plan plan;
    // what the plan was built for (checked when it is uploaded into a context)
    int64_t max_chunks = INT64_MAX;
    bool fast = true;
    int wide_mode = 1;
    int d_head = ca::FAST_D;
    int esize = 2;
};

namespace {
constexpr int kTraceCtas = 4096;
}

struct ca_context {
    int device = 0;
    int dtype = 0;
    ca::Geometry geo{};
    void* pool = nullptr;
    int64_t max_chunks = 0;
    int tpp_threshold = 1;
    bool fast = false;
    int num_sms = 1;
    bool opt_split = false;
    int opt_ctas = 0;
    bool opt_sf_tensor = true;
    int opt_pdl = 3;
    int opt_wide = 1;
    bool opt_overlap = false;
    cudaStream_t side_stream = nullptr;   // the short-tails kernel runs here beside the wide-runs kernel
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    long long opt_wait_limit = ca::DEFAULT_WAIT_LIMIT_CYCLES;
    int opt_withhold_item = -1;
    unsigned long long* trace = nullptr;  // [kTraceCtas][4], allocated when tracing is switched on
    int trace_ctas = 0;                   // CTAs of the last traced launch
    int trace_cycles = 0;                 // CA_OPT_TRACE = 2: the tcgen05 kernel accounts for cycles per role instead
    int opt_finish_in_tails = 1;          // CA_OPT_FINISH_IN_TAILS: the short-tails kernel finishes the rows when it can
    bool out_is_host = false;             // set by ca_attention_host around its launches: the rows go to host memory

    ca::Plan plan;  // scratch of ca_refresh_kernel_context (vectors keep their capacity)
    // what the launches need to know about the work list that is on the device
    struct {
        int n_seqs = 0, n_items = 0, n_items_cf = 0, n_items_short = 0, n_items_wide = 0, n_wide_chunks = 0, n_ctas = 1;
        bool short_all_empty = false;  // the short tails were all empty at the refresh and their (max, sum) rows are zeroed
        int64_t n_merge_slots = 0;  // entries of merge_slots
        int max_merge_len = 0;
        bool split_phases = false;
        ca_plan_stats stats{};
    } meta;
    bool valid = false;
    int delta_tokens = 0;
    int max_tail_tokens = 0;

    // work lists: one pinned staging buffer, one device buffer, one upload per refresh
    char* host_blob = nullptr;
    size_t host_cap = 0;
    char* dev_blob = nullptr;
    size_t dev_cap = 0;
    cudaEvent_t upload_done = nullptr;
    bool upload_pending = false;
    // device views into dev_blob
    const int4* d_items = nullptr;
    const int32_t *d_merge_off = nullptr, *d_merge_slots = nullptr;
    const int32_t *d_path_off = nullptr, *d_path_chunks = nullptr, *d_path_tokens = nullptr;
    const int32_t *d_tail_chunk = nullptr, *d_tail_tokens = nullptr;
    const int32_t* d_wide_chunks = nullptr;
    // The per-row path lists are read by the any-geometry kernel only: a context of the tensor-core geometry
    // builds and uploads them on the first partition = 2 request after a refresh, from this copy of the input.
    bool paths_on_device = false;
    ca::Plan path_plan;           // infos + path_* of the current tree
    char* paths_host = nullptr;
    char* paths_dev = nullptr;
    size_t paths_cap = 0;
    cudaEvent_t paths_done = nullptr;
    bool paths_pending = false;

    // partial results of the current step (scratch)
    float* part_o = nullptr;
    float2* part_ml = nullptr;
    size_t part_cap = 0;  // slots
    int* status = nullptr;
    int* counters = nullptr;  // two item counters: a launch draws from one and zeroes the other
    int launch_parity = 0;

    // ca_attention_host: device copy of the queries, pinned stand-ins for pageable caller buffers
    void* q_stage = nullptr;
    void* host_q_stage = nullptr;
    void* host_out_stage = nullptr;
    size_t q_stage_cap = 0, host_q_cap = 0, host_out_cap = 0;
};

extern "C" {

const char* ca_last_error(void) { return g_last_error.c_str(); }
int ca_version(void) { return 100; }

int64_t ca_chunk_bytes(int n_heads, int d_head, int chunk_size, int dtype) {
    const int es = esize_of(dtype);
    if (es == 0 || n_heads <= 0 || d_head <= 0 || chunk_size <= 0) return -1;
    return (int64_t)n_heads * 2 * chunk_size * d_head * es;
}

int64_t ca_tile_elem_offset(int d_head, int chunk_size, int dtype, int token, int elem) {
    const int es = esize_of(dtype);
    if (es == 0 || d_head <= 0 || chunk_size <= 0 || token < 0 || token >= chunk_size || elem < 0 || elem >= d_head) return -1;
    const ca::Geometry g = ca::make_geometry(1, d_head, chunk_size, es);
    return ca::tile_elem_offset(g, token, elem);
}

int ca_context_create(ca_context** out, int device, int n_heads, int d_head, int chunk_size, int dtype,
                      void* pool, int64_t max_chunks, int tpp_threshold) {
    if (!out) return fail(CA_ERR_INVALID, "out is null");
    *out = nullptr;
    const int es = esize_of(dtype);
    if (es == 0) return fail(CA_ERR_INVALID, "unsupported dtype (fp16 and fp32 only)");
    if (n_heads <= 0 || d_head <= 0 || chunk_size <= 0) return fail(CA_ERR_INVALID, "n_heads, d_head, chunk_size must be positive");
    if (d_head > 256) return fail(CA_ERR_INVALID, "d_head above 256 is not supported");
    if (max_chunks < 0 || (max_chunks > 0 && !pool)) return fail(CA_ERR_INVALID, "pool is null");
    if (reinterpret_cast<uintptr_t>(pool) % 256 != 0) return fail(CA_ERR_INVALID, "pool must be 256-byte aligned");
    int n_dev = 0;
    CA_CUDA(cudaGetDeviceCount(&n_dev));
    if (device < 0 || device >= n_dev) return fail(CA_ERR_INVALID, "no such CUDA device");
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    cudaDeviceProp prop;
    CA_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(CA_ERR_CUDA, "this library carries sm_100a code only; device is sm_" + std::to_string(prop.major * 10 + prop.minor));

    ca_context* c = new (std::nothrow) ca_context();
    if (!c) return fail(CA_ERR_INVALID, "out of host memory");
    c->device = device;
    c->dtype = dtype;
    c->geo = ca::make_geometry(n_heads, d_head, chunk_size, es);
    c->pool = pool;
    c->max_chunks = max_chunks;
    c->tpp_threshold = tpp_threshold < 1 ? 1 : tpp_threshold;
    c->fast = (dtype == CA_DTYPE_F16 && d_head == ca::FAST_D && chunk_size == ca::FAST_C);
    c->num_sms = prop.multiProcessorCount;
    cudaError_t e = cudaEventCreateWithFlags(&c->upload_done, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->paths_done, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&c->status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&c->counters, 2 * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->counters, 0, 2 * sizeof(int));
    if (e == cudaSuccess && c->fast) e = ca::configure_fast_kernels();
    if (e == cudaSuccess && c->fast) e = ca::configure_wide_kernel();
    if (e != cudaSuccess) {
        ca_context_destroy(c);
        return fail_cuda(e, "context set-up");
    }
    *out = c;
    return CA_OK;
}

void ca_context_destroy(ca_context* c) {
    if (!c) return;
    DeviceGuard guard(c->device);
    if (c->upload_done) {
        if (c->upload_pending) cudaEventSynchronize(c->upload_done);
        cudaEventDestroy(c->upload_done);
    }
    if (c->side_stream) {
        cudaStreamSynchronize(c->side_stream);
        cudaStreamDestroy(c->side_stream);
    }
    if (c->ev_fork) cudaEventDestroy(c->ev_fork);
    if (c->ev_join) cudaEventDestroy(c->ev_join);
    if (c->paths_done) {
        if (c->paths_pending) cudaEventSynchronize(c->paths_done);
        cudaEventDestroy(c->paths_done);
    }
    if (c->paths_host) cudaFreeHost(c->paths_host);
    if (c->paths_dev) cudaFree(c->paths_dev);
    if (c->host_blob) cudaFreeHost(c->host_blob);
    if (c->dev_blob) cudaFree(c->dev_blob);
    if (c->part_o) cudaFree(c->part_o);
    if (c->part_ml) cudaFree(c->part_ml);
    if (c->trace) cudaFree(c->trace);
    if (c->status) cudaFree(c->status);
    if (c->counters) cudaFree(c->counters);
    if (c->q_stage) cudaFree(c->q_stage);
    if (c->host_q_stage) cudaFreeHost(c->host_q_stage);
    if (c->host_out_stage) cudaFreeHost(c->host_out_stage);
    delete c;
}

int ca_context_set_option(ca_context* c, int option, int64_t value) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    if (option == CA_OPT_SPLIT_PHASES) {
        c->opt_split = value != 0;
    } else if (option == CA_OPT_NUM_CTAS) {
        if (value < 0 || value > 4096) return fail(CA_ERR_INVALID, "CTA count out of range");
        c->opt_ctas = (int)value;
    } else if (option == CA_OPT_SEQ_FIRST_TENSOR) {
        c->opt_sf_tensor = value != 0;
    } else if (option == CA_OPT_WIDE_RUNS) {
        if (value < 0 || value > 2) return fail(CA_ERR_INVALID, "wide-runs mode must be 0, 1 or 2");
        c->opt_wide = (int)value;
    } else if (option == CA_OPT_OVERLAP_KERNELS) {
        c->opt_overlap = value != 0;
        return CA_OK;
    } else if (option == CA_OPT_DEPENDENT_LAUNCH) {
        if (value < 0 || value > 3) return fail(CA_ERR_INVALID, "dependent-launch mask out of range");
        c->opt_pdl = (int)value;
        return CA_OK;
    } else if (option == CA_OPT_WAIT_LIMIT_CYCLES) {
        if (value < 1000) return fail(CA_ERR_INVALID, "wait limit below 1000 cycles");
        c->opt_wait_limit = value;
        return CA_OK;
    } else if (option == CA_OPT_TEST_WITHHOLD_ITEM) {
        c->opt_withhold_item = value < 0 ? -1 : (int)value;
        return CA_OK;
    } else if (option == CA_OPT_FINISH_IN_TAILS) {
        if (value != 0 && value != 1) return fail(CA_ERR_INVALID, "CA_OPT_FINISH_IN_TAILS takes 0 or 1");
        c->opt_finish_in_tails = (int)value;
        return CA_OK;
    } else if (option == CA_OPT_TRACE) {
        DeviceGuard guard(c->device);
        if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
        if (value < 0 || value > 2) return fail(CA_ERR_INVALID, "CA_OPT_TRACE takes 0, 1 or 2");
        c->trace_cycles = value == 2 ? 1 : 0;
        if (value && !c->trace) {
            CA_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->trace), (size_t)kTraceCtas * 8 * sizeof(unsigned long long)));
            CA_CUDA(cudaMemset(c->trace, 0, (size_t)kTraceCtas * 8 * sizeof(unsigned long long)));
        } else if (!value && c->trace) {
            CA_CUDA(cudaFree(c->trace));
            c->trace = nullptr;
        }
        return CA_OK;
    } else {
        return fail(CA_ERR_INVALID, "unknown option");
    }
    c->valid = false;  // schedules depend on the options
    return CA_OK;
}

static int upload_plan(ca_context* c, const ca::Plan& pl, cudaStream_t stream);

int ca_refresh_kernel_context(ca_context* c, const ca_chunk_info* infos, int n_infos, int n_seqs, ca_stream stream_) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    c->valid = false;
    const int n_ctas = c->opt_ctas > 0 ? c->opt_ctas : c->num_sms * ca::FAST_CTAS_PER_SM;
    std::string err = ca::build_plan(c->plan, infos, n_infos, n_seqs, c->geo.n_heads, c->geo.chunk_size,
                                     c->tpp_threshold, n_ctas, c->max_chunks, c->opt_split, c->geo.d_head,
                                     c->geo.esize, c->fast, c->opt_sf_tensor, c->opt_wide, /*want_paths=*/!c->fast);
    if (!err.empty()) return fail(CA_ERR_INVALID, "work list rejected: " + err);
    return upload_plan(c, c->plan, stream);
}

int ca_plan_build_for_context(const ca_context* c, ca_plan** out, const ca_chunk_info* infos, int n_infos, int n_seqs) {
    if (!c || !out) return fail(CA_ERR_INVALID, "null argument");
    ca_plan* p = *out;  // an existing plan is rebuilt in place and keeps its buffers
    if (!p) p = new (std::nothrow) ca_plan();
    if (!p) return fail(CA_ERR_INVALID, "out of host memory");
    const int n_ctas = c->opt_ctas > 0 ? c->opt_ctas : c->num_sms * ca::FAST_CTAS_PER_SM;
    std::string err = ca::build_plan(p->plan, infos, n_infos, n_seqs, c->geo.n_heads, c->geo.chunk_size, c->tpp_threshold,
                                     n_ctas, c->max_chunks, c->opt_split, c->geo.d_head, c->geo.esize, c->fast,
                                     c->opt_sf_tensor, c->opt_wide, /*want_paths=*/!c->fast);
    if (!err.empty()) {
        if (!*out) delete p;  // a caller-owned plan is left to the caller (its contents are unspecified now)
        return fail(CA_ERR_INVALID, "work list rejected: " + err);
    }
    p->max_chunks = c->max_chunks;
    p->wide_mode = c->opt_wide;
    p->fast = c->fast;
    p->d_head = c->geo.d_head;
    p->esize = c->geo.esize;
    *out = p;
    return CA_OK;
}

int ca_refresh_from_plan(ca_context* c, const ca_plan* plan, ca_stream stream_) {
    if (!c || !plan) return fail(CA_ERR_INVALID, "null argument");
    const ca::Plan& pl = plan->plan;
    const int n_ctas = c->opt_ctas > 0 ? c->opt_ctas : c->num_sms * ca::FAST_CTAS_PER_SM;
    if (pl.n_heads != c->geo.n_heads || pl.chunk_size != c->geo.chunk_size || plan->d_head != c->geo.d_head ||
        plan->esize != c->geo.esize || plan->fast != c->fast || plan->max_chunks > c->max_chunks ||
        pl.split_phases != c->opt_split || pl.tpp_threshold != c->tpp_threshold || (c->fast && pl.n_ctas > n_ctas) ||
        plan->wide_mode != c->opt_wide)
        return fail(CA_ERR_INVALID, "the plan was built for a different geometry, pool size or set of options");
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    c->valid = false;
    return upload_plan(c, pl, static_cast<cudaStream_t>(stream_));
}

static int upload_plan(ca_context* c, const ca::Plan& pl, cudaStream_t stream) {

    // pack every table into one staging buffer
    struct Part { const void* src; size_t bytes; size_t off; };
    Part parts[9] = {
        {pl.items.data(), pl.items.size() * sizeof(ca::PlanItem), 0},
        {pl.merge_off.data(), pl.merge_off.size() * 4, 0},
        {pl.merge_slots.data(), pl.merge_slots.size() * 4, 0},
        {pl.path_off.data(), pl.has_paths ? pl.path_off.size() * 4 : 0, 0},
        {pl.path_chunks.data(), pl.has_paths ? pl.path_chunks.size() * 4 : 0, 0},
        {pl.path_tokens.data(), pl.has_paths ? pl.path_tokens.size() * 4 : 0, 0},
        {pl.tail_chunk.data(), pl.tail_chunk.size() * 4, 0},
        {pl.tail_tokens.data(), pl.tail_tokens.size() * 4, 0},
        {pl.wide_chunks.data(), pl.wide_chunks.size() * 4, 0},
    };
    size_t total = 0;
    for (Part& p : parts) {
        p.off = total;
        total += align_up(p.bytes, 256);
    }
    total = align_up(total + 256, 256);
    if (c->upload_pending) {  // the previous upload may still be reading the staging buffer
        CA_CUDA(cudaEventSynchronize(c->upload_done));
        c->upload_pending = false;
    }
    if (total > c->host_cap) {
        if (c->host_blob) CA_CUDA(cudaFreeHost(c->host_blob));
        c->host_blob = nullptr;
        c->host_cap = 0;
        const size_t cap = align_up(total * 3 / 2, 4096);
        CA_CUDA(cudaMallocHost(reinterpret_cast<void**>(&c->host_blob), cap));
        c->host_cap = cap;
    }
    if (total > c->dev_cap) {
        if (c->dev_blob) CA_CUDA(cudaFree(c->dev_blob));  // synchronises with work that still reads it
        c->dev_blob = nullptr;
        c->dev_cap = 0;
        const size_t cap = align_up(total * 3 / 2, 4096);
        CA_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->dev_blob), cap));
        c->dev_cap = cap;
    }
    for (const Part& p : parts)
        if (p.bytes) std::memcpy(c->host_blob + p.off, p.src, p.bytes);
    CA_CUDA(cudaMemcpyAsync(c->dev_blob, c->host_blob, total, cudaMemcpyHostToDevice, stream));
    CA_CUDA(cudaEventRecord(c->upload_done, stream));
    c->upload_pending = true;
    c->d_items = reinterpret_cast<const int4*>(c->dev_blob + parts[0].off);
    c->d_merge_off = reinterpret_cast<const int32_t*>(c->dev_blob + parts[1].off);
    c->d_merge_slots = reinterpret_cast<const int32_t*>(c->dev_blob + parts[2].off);
    c->d_path_off = reinterpret_cast<const int32_t*>(c->dev_blob + parts[3].off);
    c->d_path_chunks = reinterpret_cast<const int32_t*>(c->dev_blob + parts[4].off);
    c->d_path_tokens = reinterpret_cast<const int32_t*>(c->dev_blob + parts[5].off);
    c->d_tail_chunk = reinterpret_cast<const int32_t*>(c->dev_blob + parts[6].off);
    c->d_tail_tokens = reinterpret_cast<const int32_t*>(c->dev_blob + parts[7].off);
    c->d_wide_chunks = reinterpret_cast<const int32_t*>(c->dev_blob + parts[8].off);
    c->paths_on_device = pl.has_paths;
    if (!pl.has_paths) {  // keep what a later partition = 2 request needs to build them
        c->path_plan.infos = pl.infos;
        c->path_plan.n_seqs = pl.n_seqs;
        c->path_plan.has_paths = false;
    }

    // partial-result scratch, grow-only
    const size_t slots = (size_t)pl.stats.n_slots;
    if (slots > c->part_cap) {
        if (c->part_o) CA_CUDA(cudaFree(c->part_o));
        if (c->part_ml) CA_CUDA(cudaFree(c->part_ml));
        c->part_o = nullptr;
        c->part_ml = nullptr;
        c->part_cap = 0;
        const size_t cap = slots * 3 / 2 + 64;
        CA_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->part_o), cap * ca::FAST_D * sizeof(float)));
        CA_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->part_ml), cap * sizeof(float2)));
        c->part_cap = cap;
    }
    // Short tails that are all empty (freshly reserved ones under a fully shared prefix) have nothing to compute until a
    // token is appended: their (max, sum) rows are zeroed here -- a sum of zero marks a piece without tokens -- and the
    // launch of their kernel is left out while delta_tokens is 0.
    c->meta.short_all_empty = false;
    if (pl.n_items_short > 0 && pl.short_all_empty) {
        CA_CUDA(cudaMemsetAsync(c->part_ml + (size_t)pl.short_slot_base * pl.n_heads, 0,
                                (size_t)pl.n_items_short * pl.n_heads * sizeof(float2), stream));
        c->meta.short_all_empty = true;
    }
    c->max_tail_tokens = 0;
    for (int32_t t : pl.tail_tokens) c->max_tail_tokens = t > c->max_tail_tokens ? t : c->max_tail_tokens;
    c->delta_tokens = 0;
    c->meta.n_seqs = pl.n_seqs;
    c->meta.n_items = (int)pl.items.size();
    c->meta.n_items_cf = pl.n_items_cf;
    c->meta.n_items_short = pl.n_items_short;
    c->meta.n_items_wide = pl.n_items_wide;
    c->meta.n_wide_chunks = (int)pl.wide_chunks.size();
    c->meta.n_ctas = pl.n_ctas;
    c->meta.n_merge_slots = (int64_t)pl.merge_slots.size();
    c->meta.max_merge_len = pl.max_merge_len;
    c->meta.split_phases = pl.split_phases;
    c->meta.stats = pl.stats;
    c->valid = true;
    return CA_OK;
}

int ca_context_delta_tokens(const ca_context* c) { return c ? c->delta_tokens : -1; }

int ca_append_kv(ca_context* c, const void* k, const void* v, int n_seqs, ca_stream stream_) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    if (!c->valid) return fail(CA_ERR_STATE, "work list is stale: call ca_refresh_kernel_context first");
    if (n_seqs != c->meta.n_seqs) return fail(CA_ERR_INVALID, "n_seqs differs from the refreshed work list");
    if (n_seqs == 0) return CA_OK;
    if (!k || !v) return fail(CA_ERR_INVALID, "k or v is null");
    if (c->max_tail_tokens + c->delta_tokens >= c->geo.chunk_size)
        return fail(CA_ERR_STATE, "a tail chunk is full: reserve a new tail and refresh before appending");
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    ca::AppendParams p;
    p.pool = c->pool;
    p.geo = c->geo;
    p.k = k;
    p.v = v;
    p.tail_chunk = c->d_tail_chunk;
    p.tail_tokens = c->d_tail_tokens;
    p.n_seqs = n_seqs;
    p.delta_tokens = c->delta_tokens;
    const bool vec16 = c->geo.epg > 1 && reinterpret_cast<uintptr_t>(k) % 16 == 0 && reinterpret_cast<uintptr_t>(v) % 16 == 0;
    CA_CUDA(ca::launch_append_kv(p, vec16, static_cast<cudaStream_t>(stream_)));
    c->delta_tokens += 1;
    return CA_OK;
}

static int check_attention_args(ca_context* c, const void* q, int n_seqs) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    if (!c->valid) return fail(CA_ERR_STATE, "work list is stale: call ca_refresh_kernel_context first");
    if (n_seqs != c->meta.n_seqs) return fail(CA_ERR_INVALID, "n_seqs differs from the refreshed work list");
    if (n_seqs > 0 && !q) return fail(CA_ERR_INVALID, "q is null");
    if (reinterpret_cast<uintptr_t>(q) % 16 != 0 && c->fast) return fail(CA_ERR_INVALID, "q must be 16-byte aligned");
    return CA_OK;
}

// True when the short-tails kernel finishes the step's rows itself: every row has a short tail item, and the batch is
// one where that pays.  Measured on B200: 6-8 % of the step at 256 rows x 32 heads (a launch less), nothing at 1024
// rows, -3 % at 2048 rows (the kernel is bound by the latency of its lookups, and the merge kernel hides that better
// at its higher occupancy); with the output rows going to HOST memory it is 15-35 % of the end-to-end time at every size
// (whole 256-byte rows per half-warp cross the bus better than the merge kernel's stores).
static bool tails_can_finish(const ca_context* c) {
    return c->fast && c->opt_finish_in_tails && !c->opt_overlap && !c->meta.split_phases && c->meta.n_items_short > 0 &&
           c->meta.n_items_short == c->meta.n_seqs &&
           (c->out_is_host || ((long long)c->meta.n_seqs * c->geo.n_heads <= 32768 &&
                               // tails that are all empty cost no launch of their own: nothing to save (a fully shared
                               // batch of 64 x 32 pairs with nine pieces each: 16.8 us with the merge kernel, 18.0 without)
                               !(c->meta.short_all_empty && c->delta_tokens == 0)));
}

// The partial results of a step.  finish != null and tails_can_finish(): the short-tails kernel goes LAST and stores the
// output rows described by *finish; *finished tells the caller that no merge is needed.
static int run_partials(ca_context* c, const void* q, int n_seqs, int phases, ca_stream stream_, const ca::MergeParams* finish,
                        bool* finished) {
    if (finished) *finished = false;
    int rc = check_attention_args(c, q, n_seqs);
    if (rc != CA_OK) return rc;
    if (!c->fast) return fail(CA_ERR_INVALID, "partials exist only for fp16 / d_head 128 / chunk_size 64");
    if (phases < 1 || phases > 3) return fail(CA_ERR_INVALID, "phases must be 1, 2 or 3");
    if (phases != 3 && !c->meta.split_phases) return fail(CA_ERR_STATE, "single phases need CA_OPT_SPLIT_PHASES");
    if (n_seqs == 0) return CA_OK;
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    ca::PartialParams p;
    p.pool = static_cast<const uint8_t*>(c->pool);
    p.n_heads = c->geo.n_heads;
    p.q = q;
    p.items = c->d_items;
    p.part_o = c->part_o;
    p.part_ml = c->part_ml;
    p.delta_tokens = c->delta_tokens;
    p.scale_log2 = 1.4426950408889634f / std::sqrt((float)c->geo.d_head);
    p.status = c->status;
    p.trace = c->trace;
    p.n_slots = c->meta.stats.n_slots;
    p.n_seqs = n_seqs;
    p.max_chunks = (int)(c->max_chunks < INT32_MAX ? c->max_chunks : INT32_MAX);
    p.wait_limit = c->opt_wait_limit;
    p.withhold_item = c->opt_withhold_item;
    // The work list holds every item once for all heads; a launch is given a range of (item, head) pieces.
    // One launch per range; every launch draws from the counter the previous launch zeroed.
    const int H = c->geo.n_heads;
    auto launch = [&](int lo, int hi) -> cudaError_t {
        lo *= H;
        hi *= H;
        if (hi <= lo) return cudaSuccess;
        p.item_lo = lo;
        p.item_hi = hi;
        p.counter = c->counters + c->launch_parity;
        p.counter_next = c->counters + (c->launch_parity ^ 1);
        const int n_ctas = c->meta.n_ctas < hi - lo ? c->meta.n_ctas : hi - lo;
        c->trace_ctas = n_ctas;
        const cudaError_t e = ca::launch_attn_partials(p, n_ctas, stream, (c->opt_pdl & 2) != 0);
        // the counters change roles only once the launch that zeroes the other one is really in the stream
        if (e == cudaSuccess) c->launch_parity ^= 1;
        return e;
    };
    // Items are laid out [persistent kernel][short private tails][wide shared runs]; the two other kernels go
    // first (the short tails before the wide runs, whose set-up then overlaps them) so that the persistent kernel's
    // tail leads straight into the merge.
    const int n_items = c->meta.n_items - c->meta.n_items_short - c->meta.n_items_wide;
    const bool finish_in_tails = finish && finished && phases == 3 && tails_can_finish(c);
    const bool run_short = !finish_in_tails && c->meta.n_items_short > 0 && (phases & 2) &&
                           !(c->meta.short_all_empty && c->delta_tokens == 0);
    const bool run_wide = c->meta.n_items_wide > 0 && (phases & 1);
    // The short tails are bound by memory, the wide runs by the tensor and special-function pipes, and they touch
    // disjoint partial rows: optionally (CA_OPT_OVERLAP_KERNELS) the short-tails kernel runs on a second stream
    // BESIDE the wide kernel (forked and joined with events) instead of before it.  Off by default: measured, the
    // wide kernel's CTAs leave too little of an SM for the other kernel to make headway beside them.
    const bool beside = run_short && run_wide && c->opt_overlap;
    if (run_short) {
        p.item_lo = n_items * H;
        p.item_hi = (n_items + c->meta.n_items_short) * H;
        if (beside) {
            CA_CUDA(cudaEventRecord(c->ev_fork, stream));
            CA_CUDA(cudaStreamWaitEvent(c->side_stream, c->ev_fork, 0));
            CA_CUDA(ca::launch_attn_short_tails(p, c->side_stream, false));
            CA_CUDA(cudaEventRecord(c->ev_join, c->side_stream));
        } else {
            CA_CUDA(ca::launch_attn_short_tails(p, stream, (c->opt_pdl & 2) != 0));
        }
    }
    if (run_wide) {
        ca::WideParams w;
        w.pool = p.pool;
        w.n_heads = p.n_heads;
        w.q = q;
        w.items = c->d_items;
        w.item_lo = (c->meta.n_items - c->meta.n_items_wide) * H;
        w.item_hi = c->meta.n_items * H;
        w.wide_chunks = c->d_wide_chunks;
        w.n_wide_chunks = c->meta.n_wide_chunks;
        w.part_o = c->part_o;
        w.part_ml = c->part_ml;
        w.scale_log2 = p.scale_log2;
        w.status = c->status;
        w.n_slots = p.n_slots;
        w.n_seqs = p.n_seqs;
        w.max_chunks = p.max_chunks;
        w.wait_limit = p.wait_limit;
        w.trace = c->trace;
        w.trace_cycles = c->trace_cycles;
        c->trace_ctas = (w.item_hi - w.item_lo) < kTraceCtas ? (w.item_hi - w.item_lo) : 0;
        if (c->trace_ctas == 0) w.trace = nullptr;
        CA_CUDA(ca::launch_attn_wide(w, stream, (c->opt_pdl & 2) != 0));
    }
    if (beside) CA_CUDA(cudaStreamWaitEvent(stream, c->ev_join, 0));
    if (!c->meta.split_phases) {
        CA_CUDA(launch(0, n_items));
    } else {
        if (phases & 1) CA_CUDA(launch(0, c->meta.n_items_cf));
        if (phases & 2) CA_CUDA(launch(c->meta.n_items_cf, n_items));
    }
    if (finish_in_tails) {
        p.item_lo = n_items * H;
        p.item_hi = (n_items + c->meta.n_items_short) * H;
        CA_CUDA(ca::launch_attn_short_tails(p, stream, (c->opt_pdl & 2) != 0, finish));
        *finished = true;
    }
    return CA_OK;
}

int ca_attn_partials(ca_context* c, const void* q, int n_seqs, int phases, ca_stream stream_) {
    return run_partials(c, q, n_seqs, phases, stream_, nullptr, nullptr);
}

static ca::MergeParams merge_params_of(const ca_context* c, void* out, int n_seqs) {
    ca::MergeParams m;
    m.part_o = c->part_o;
    m.part_ml = c->part_ml;
    m.merge_off = c->d_merge_off;
    m.merge_slots = c->d_merge_slots;
    m.out = out;
    m.n_pairs = n_seqs * c->geo.n_heads;
    m.n_merge_entries = (long long)c->meta.n_merge_slots;
    m.max_list = c->meta.max_merge_len;
    m.n_slots = c->meta.stats.n_slots;
    m.status = c->status;
    m.n_heads = c->geo.n_heads;
    return m;
}

namespace {
// true when the device can read / write the host range directly (page-locked and mapped);
// *dev_ptr receives the address to use on the device
bool device_view_of_host(const void* host_ptr, void** dev_ptr) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, host_ptr) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (attr.type != cudaMemoryTypeHost || attr.devicePointer == nullptr) return false;
    *dev_ptr = attr.devicePointer;
    return true;
}
}  // namespace

int ca_attention_host(ca_context* c, const void* q_host, void* out_host, int n_seqs, int partition, ca_stream stream_) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    if (!c->valid) return fail(CA_ERR_STATE, "work list is stale: call ca_refresh_kernel_context first");
    if (n_seqs != c->meta.n_seqs) return fail(CA_ERR_INVALID, "n_seqs differs from the refreshed work list");
    if (partition < 0 || partition > 2) return fail(CA_ERR_INVALID, "Unsupported partition type");
    if (n_seqs == 0) return CA_OK;
    if (!q_host || !out_host) return fail(CA_ERR_INVALID, "q or out is null");
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const size_t bytes = (size_t)n_seqs * c->geo.n_heads * c->geo.d_head * c->geo.esize;
    if (bytes > c->q_stage_cap) {
        if (c->q_stage) CA_CUDA(cudaFree(c->q_stage));
        c->q_stage = nullptr;
        c->q_stage_cap = 0;
        CA_CUDA(cudaMalloc(&c->q_stage, align_up(bytes * 2, 4096)));
        c->q_stage_cap = align_up(bytes * 2, 4096);
    }
    auto grow_host = [&](void*& buf, size_t& cap) -> cudaError_t {
        if (bytes <= cap) return cudaSuccess;
        if (buf) cudaFreeHost(buf);
        buf = nullptr;
        cap = 0;
        cudaError_t e = cudaMallocHost(&buf, align_up(bytes * 2, 4096));
        if (e == cudaSuccess) cap = align_up(bytes * 2, 4096);
        return e;
    };
    // queries: one copy into device memory (every item re-reads its rows, so they must not stay
    // behind the bus); a pageable source goes through a pinned stand-in first
    void* unused = nullptr;
    const void* q_src = q_host;
    if (!device_view_of_host(q_host, &unused)) {
        CA_CUDA(grow_host(c->host_q_stage, c->host_q_cap));
        std::memcpy(c->host_q_stage, q_host, bytes);
        q_src = c->host_q_stage;
    }
    CA_CUDA(cudaMemcpyAsync(c->q_stage, q_src, bytes, cudaMemcpyHostToDevice, stream));
    // output: the last kernel stores its rows straight into the caller's page-locked buffer
    void* out_dev = nullptr;
    const bool direct = device_view_of_host(out_host, &out_dev) && reinterpret_cast<uintptr_t>(out_dev) % 16 == 0;
    if (!direct) {
        CA_CUDA(grow_host(c->host_out_stage, c->host_out_cap));
        if (!device_view_of_host(c->host_out_stage, &out_dev)) return fail(CA_ERR_CUDA, "pinned staging buffer is not mapped");
    }
    c->out_is_host = true;
    int rc = ca_attention(c, c->q_stage, out_dev, n_seqs, partition, stream_);
    c->out_is_host = false;
    if (rc != CA_OK) return rc;
    CA_CUDA(cudaStreamSynchronize(stream));
    if (!direct) std::memcpy(out_host, c->host_out_stage, bytes);
    return CA_OK;
}

int ca_attn_merge(ca_context* c, void* out, int n_seqs, ca_stream stream_) {
    int rc = check_attention_args(c, out, n_seqs);
    if (rc != CA_OK) return rc;
    if (!c->fast) return fail(CA_ERR_INVALID, "partials exist only for fp16 / d_head 128 / chunk_size 64");
    if (n_seqs == 0) return CA_OK;
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    const ca::MergeParams m = merge_params_of(c, out, n_seqs);
    CA_CUDA(ca::launch_attn_merge(m, static_cast<cudaStream_t>(stream_), (c->opt_pdl & 1) != 0));
    return CA_OK;
}

int ca_peer_barrier(void* const* flag_arrays, int n_peers, int rank, uint32_t epoch, int64_t timeout_ns, int32_t* status,
                    ca_stream stream_) {
    if (n_peers < 1 || n_peers > ca::MERGE_MAX_PEERS || !flag_arrays) return fail(CA_ERR_INVALID, "1 to 8 flag arrays are required");
    if (rank < 0 || rank >= n_peers) return fail(CA_ERR_INVALID, "rank outside the group");
    if (timeout_ns <= 0) return fail(CA_ERR_INVALID, "the barrier needs a time limit");
    ca::PeerBarrierParams p{};
    for (int i = 0; i < n_peers; i++) {
        if (!flag_arrays[i] || reinterpret_cast<uintptr_t>(flag_arrays[i]) % 4) return fail(CA_ERR_INVALID, "null or misaligned flag array");
        p.flags[i] = static_cast<uint32_t*>(flag_arrays[i]);
    }
    p.n_peers = n_peers;
    p.rank = rank;
    p.epoch = epoch;
    p.timeout_ns = timeout_ns;
    p.status = status;
    CA_CUDA(ca::launch_peer_barrier(p, static_cast<cudaStream_t>(stream_)));
    return CA_OK;
}

int ca_attention_to_peers(ca_context* c, const void* q, void* const* peer_out, int n_peers, void* multicast_out,
                          int total_heads, int head_offset, int n_seqs, ca_stream stream_) {
    int rc = check_attention_args(c, q, n_seqs);
    if (rc != CA_OK) return rc;
    if (!c->fast) return fail(CA_ERR_INVALID, "writing into peers' outputs exists only for fp16 / d_head 128 / chunk_size 64");
    if (n_peers < 1 || n_peers > ca::MERGE_MAX_PEERS || !peer_out) return fail(CA_ERR_INVALID, "1 to 8 peer outputs are required");
    if (head_offset < 0 || total_heads < head_offset + c->geo.n_heads) return fail(CA_ERR_INVALID, "head slice outside the full width");
    for (int i = 0; i < n_peers; i++)
        if (!peer_out[i] || reinterpret_cast<uintptr_t>(peer_out[i]) % 16) return fail(CA_ERR_INVALID, "null or misaligned peer output");
    if (reinterpret_cast<uintptr_t>(multicast_out) % 16) return fail(CA_ERR_INVALID, "misaligned multicast output");
    if (n_seqs == 0) return CA_OK;
    ca::MergeParams m = merge_params_of(c, nullptr, n_seqs);
    m.n_peers = n_peers;
    m.total_heads = total_heads;
    m.head_offset = head_offset;
    for (int i = 0; i < n_peers; i++) m.peer_out[i] = peer_out[i];
    m.mc_out = multicast_out;
    bool finished = false;
    rc = run_partials(c, q, n_seqs, 3, stream_, &m, &finished);
    if (rc != CA_OK) return rc;
    if (finished) return CA_OK;
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    CA_CUDA(ca::launch_attn_merge(m, static_cast<cudaStream_t>(stream_), (c->opt_pdl & 1) != 0));
    return CA_OK;
}

// The any-geometry kernel's path lists for a context that planned without them (one build and one upload per
// tree change, on the first request that needs them).
static int ensure_paths(ca_context* c, cudaStream_t stream) {
    if (c->paths_on_device) return CA_OK;
    ca::Plan& pp = c->path_plan;
    ca::build_paths(pp);
    const size_t b0 = align_up(pp.path_off.size() * 4, 256), b1 = align_up(pp.path_chunks.size() * 4, 256),
                 b2 = align_up(pp.path_tokens.size() * 4, 256);
    const size_t total = b0 + b1 + b2 + 256;
    if (c->paths_pending) {
        CA_CUDA(cudaEventSynchronize(c->paths_done));
        c->paths_pending = false;
    }
    if (total > c->paths_cap) {
        if (c->paths_host) CA_CUDA(cudaFreeHost(c->paths_host));
        if (c->paths_dev) CA_CUDA(cudaFree(c->paths_dev));
        c->paths_host = c->paths_dev = nullptr;
        c->paths_cap = 0;
        const size_t cap = align_up(total * 3 / 2, 4096);
        CA_CUDA(cudaMallocHost(reinterpret_cast<void**>(&c->paths_host), cap));
        CA_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->paths_dev), cap));
        c->paths_cap = cap;
    }
    std::memcpy(c->paths_host, pp.path_off.data(), pp.path_off.size() * 4);
    if (!pp.path_chunks.empty()) std::memcpy(c->paths_host + b0, pp.path_chunks.data(), pp.path_chunks.size() * 4);
    if (!pp.path_tokens.empty()) std::memcpy(c->paths_host + b0 + b1, pp.path_tokens.data(), pp.path_tokens.size() * 4);
    CA_CUDA(cudaMemcpyAsync(c->paths_dev, c->paths_host, total - 256, cudaMemcpyHostToDevice, stream));
    CA_CUDA(cudaEventRecord(c->paths_done, stream));
    c->paths_pending = true;
    c->d_path_off = reinterpret_cast<const int32_t*>(c->paths_dev);
    c->d_path_chunks = reinterpret_cast<const int32_t*>(c->paths_dev + b0);
    c->d_path_tokens = reinterpret_cast<const int32_t*>(c->paths_dev + b0 + b1);
    c->paths_on_device = true;
    return CA_OK;
}

int ca_attention(ca_context* c, const void* q, void* out, int n_seqs, int partition, ca_stream stream_) {
    int rc = check_attention_args(c, q, n_seqs);
    if (rc != CA_OK) return rc;
    if (partition < 0 || partition > 2) return fail(CA_ERR_INVALID, "Unsupported partition type");
    if (n_seqs == 0) return CA_OK;
    if (!out) return fail(CA_ERR_INVALID, "out is null");
    if (c->fast && partition != CA_PARTITION_SEQ_FIRST) {
        const ca::MergeParams m = merge_params_of(c, out, n_seqs);
        bool finished = false;
        rc = run_partials(c, q, n_seqs, 3, stream_, &m, &finished);
        if (rc != CA_OK || finished) return rc;
        return ca_attn_merge(c, out, n_seqs, stream_);
    }
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    rc = ensure_paths(c, static_cast<cudaStream_t>(stream_));
    if (rc != CA_OK) return rc;
    ca::GenericParams g;
    g.pool = c->pool;
    g.geo = c->geo;
    g.q = q;
    g.out = out;
    g.path_off = c->d_path_off;
    g.path_chunks = c->d_path_chunks;
    g.path_tokens = c->d_path_tokens;
    g.n_seqs = n_seqs;
    g.delta_tokens = c->delta_tokens;
    g.scale = 1.0f / std::sqrt((float)c->geo.d_head);
    CA_CUDA(ca::launch_attn_seq_generic(g, c->dtype, static_cast<cudaStream_t>(stream_)));
    return CA_OK;
}

int ca_scatter_prefill(ca_context* c, const void* k, const void* v, int64_t stride_token, int64_t stride_head,
                       int first_token, int n_tokens, const int32_t* chunk_ids, ca_stream stream_) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    if (n_tokens < 0 || first_token < 0) return fail(CA_ERR_INVALID, "negative token range");
    if (n_tokens == 0) return CA_OK;
    if (!k || !v || !chunk_ids) return fail(CA_ERR_INVALID, "k, v or chunk_ids is null");
    const int C = c->geo.chunk_size;
    const int n_chunks = (n_tokens + C - 1) / C;
    for (int i = 0; i < n_chunks; i++)
        if (chunk_ids[i] < 0 || chunk_ids[i] >= c->max_chunks) return fail(CA_ERR_INVALID, "chunk id outside the pool");
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    const int es = c->geo.esize;
    const char* kb = static_cast<const char*>(k) + (int64_t)first_token * stride_token * es;
    const char* vb = static_cast<const char*>(v) + (int64_t)first_token * stride_token * es;
    // 16-byte moves need every source row to start on a 16-byte boundary
    const bool vec16 = c->geo.epg > 1 && reinterpret_cast<uintptr_t>(kb) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(vb) % 16 == 0 && (stride_token * es) % 16 == 0 &&
                       (stride_head * es) % 16 == 0;
    for (int c0 = 0; c0 < n_chunks; c0 += ca::SCATTER_MAX_CHUNKS) {
        const int nc = n_chunks - c0 < ca::SCATTER_MAX_CHUNKS ? n_chunks - c0 : ca::SCATTER_MAX_CHUNKS;
        ca::ScatterParams p;
        p.pool = c->pool;
        p.geo = c->geo;
        p.k = kb + (int64_t)c0 * C * stride_token * es;
        p.v = vb + (int64_t)c0 * C * stride_token * es;
        p.stride_token = stride_token;
        p.stride_head = stride_head;
        const int tok_end = (c0 + nc) * C < n_tokens ? (c0 + nc) * C : n_tokens;
        p.n_tokens = tok_end - c0 * C;
        std::memcpy(p.chunk_ids, chunk_ids + c0, nc * sizeof(int32_t));
        CA_CUDA(ca::launch_scatter_prefill(p, vec16, static_cast<cudaStream_t>(stream_)));
    }
    return CA_OK;
}

int ca_scatter_rows(ca_context* c, const void* k, const void* v, int64_t stride_token, int64_t stride_head,
                    int n_tokens, const int32_t* chunk_ids, const int32_t* rows, ca_stream stream_) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    if (n_tokens < 0) return fail(CA_ERR_INVALID, "negative token count");
    if (n_tokens == 0) return CA_OK;
    if (!k || !v || !chunk_ids || !rows) return fail(CA_ERR_INVALID, "k, v, chunk_ids or rows is null");
    for (int i = 0; i < n_tokens; i++) {
        if (chunk_ids[i] < 0 || chunk_ids[i] >= c->max_chunks) return fail(CA_ERR_INVALID, "chunk id outside the pool");
        if (rows[i] < 0 || rows[i] >= c->geo.chunk_size) return fail(CA_ERR_INVALID, "row outside the chunk");
    }
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    const int es = c->geo.esize;
    const bool vec16 = c->geo.epg > 1 && reinterpret_cast<uintptr_t>(k) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(v) % 16 == 0 && (stride_token * es) % 16 == 0 &&
                       (stride_head * es) % 16 == 0;
    // the plan's tail fill counts no longer describe the pool: the next step needs a fresh work list
    c->valid = false;
    for (int t0 = 0; t0 < n_tokens; t0 += ca::SCATTER_MAX_ROWS) {
        const int nt = n_tokens - t0 < ca::SCATTER_MAX_ROWS ? n_tokens - t0 : ca::SCATTER_MAX_ROWS;
        ca::ScatterRowsParams p;
        p.pool = c->pool;
        p.geo = c->geo;
        p.k = static_cast<const char*>(k) + (int64_t)t0 * stride_token * es;
        p.v = static_cast<const char*>(v) + (int64_t)t0 * stride_token * es;
        p.stride_token = stride_token;
        p.stride_head = stride_head;
        p.n_tokens = nt;
        std::memcpy(p.chunk_ids, chunk_ids + t0, nt * sizeof(int32_t));
        std::memcpy(p.rows, rows + t0, nt * sizeof(int32_t));
        CA_CUDA(ca::launch_scatter_rows(p, vec16, static_cast<cudaStream_t>(stream_)));
    }
    return CA_OK;
}

int ca_copy_chunks(ca_context* c, const int32_t* src_ids, const int32_t* dst_ids, int n, ca_stream stream_) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    if (n < 0) return fail(CA_ERR_INVALID, "negative count");
    if (n == 0) return CA_OK;
    if (!src_ids || !dst_ids) return fail(CA_ERR_INVALID, "id array is null");
    for (int i = 0; i < n; i++) {
        if (src_ids[i] < 0 || src_ids[i] >= c->max_chunks || dst_ids[i] < 0 || dst_ids[i] >= c->max_chunks)
            return fail(CA_ERR_INVALID, "chunk id outside the pool");
        if (src_ids[i] == dst_ids[i]) return fail(CA_ERR_INVALID, "source and destination chunk are the same");
    }
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    for (int i0 = 0; i0 < n; i0 += ca::COPY_MAX_PAIRS) {
        ca::CopyParams p;
        p.pool = c->pool;
        p.chunk_bytes = c->geo.chunk_elems * c->geo.esize;
        p.n = n - i0 < ca::COPY_MAX_PAIRS ? n - i0 : ca::COPY_MAX_PAIRS;
        std::memcpy(p.src, src_ids + i0, p.n * sizeof(int32_t));
        std::memcpy(p.dst, dst_ids + i0, p.n * sizeof(int32_t));
        CA_CUDA(ca::launch_copy_chunks(p, static_cast<cudaStream_t>(stream_)));
    }
    return CA_OK;
}

int ca_read_chunk(ca_context* c, int chunk_id, int n_tokens, void* k_out, void* v_out, ca_stream stream_) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    if (chunk_id < 0 || chunk_id >= c->max_chunks) return fail(CA_ERR_INVALID, "chunk id outside the pool");
    if (n_tokens < 0 || n_tokens > c->geo.chunk_size) return fail(CA_ERR_INVALID, "n_tokens outside the chunk");
    if (n_tokens == 0) return CA_OK;
    if (!k_out || !v_out) return fail(CA_ERR_INVALID, "output is null");
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    ca::ReadChunkParams p;
    p.pool = c->pool;
    p.geo = c->geo;
    p.chunk_id = chunk_id;
    p.n_tokens = n_tokens;
    p.k_out = k_out;
    p.v_out = v_out;
    CA_CUDA(ca::launch_read_chunk(p, static_cast<cudaStream_t>(stream_)));
    return CA_OK;
}

int ca_status_read(ca_context* c, ca_stream stream_, int32_t* status) {
    if (!c || !status) return fail(CA_ERR_INVALID, "null argument");
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int32_t host = 0;
    CA_CUDA(cudaMemcpyAsync(&host, c->status, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    CA_CUDA(cudaStreamSynchronize(stream));
    *status = host;
    if (host != 0) return fail(CA_ERR_DEVICE_STATUS, "a kernel gave up a bounded wait, status " + std::to_string(host));
    return CA_OK;
}

int ca_status_clear(ca_context* c, ca_stream stream_) {
    if (!c) return fail(CA_ERR_INVALID, "context is null");
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    CA_CUDA(cudaMemsetAsync(c->status, 0, sizeof(int), static_cast<cudaStream_t>(stream_)));
    return CA_OK;
}

int ca_context_read_trace(ca_context* c, uint64_t* out, int max_ctas, int* n_ctas, ca_stream stream_) {
    if (!c || !out || !n_ctas || max_ctas < 0) return fail(CA_ERR_INVALID, "null argument");
    if (!c->trace) return fail(CA_ERR_STATE, "tracing is off: set CA_OPT_TRACE first");
    DeviceGuard guard(c->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int n = c->trace_ctas < max_ctas ? c->trace_ctas : max_ctas;
    CA_CUDA(cudaStreamSynchronize(stream));
    if (n > 0) CA_CUDA(cudaMemcpy(out, c->trace, (size_t)n * 8 * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    *n_ctas = n;
    return CA_OK;
}

int ca_context_stats(const ca_context* c, ca_plan_stats* out) {
    if (!c || !out) return fail(CA_ERR_INVALID, "null argument");
    if (!c->valid) return fail(CA_ERR_STATE, "work list is stale");
    *out = c->meta.stats;
    if (tails_can_finish(c)) out->kernels_per_step -= 1;  // the short-tails kernel stores the rows: no merge launch
    else if (c->meta.short_all_empty && c->delta_tokens == 0) out->kernels_per_step -= 1;  // nothing to do for empty tails
    return CA_OK;
}

// ---- host-only planner ---------------------------------------------------------------------------------
int ca_plan_build(ca_plan** out, const ca_chunk_info* infos, int n_infos, int n_seqs, int n_heads,
                  int chunk_size, int tpp_threshold, int n_ctas, int64_t max_chunks, int split_phases,
                  int seq_first_tensor, int wide_runs) {
    if (!out) return fail(CA_ERR_INVALID, "out is null");
    *out = nullptr;
    ca_plan* p = new (std::nothrow) ca_plan();
    if (!p) return fail(CA_ERR_INVALID, "out of host memory");
    std::string err = ca::build_plan(p->plan, infos, n_infos, n_seqs, n_heads, chunk_size, tpp_threshold, n_ctas,
                                     max_chunks, split_phases != 0, ca::FAST_D, 2, true, seq_first_tensor != 0, wide_runs);
    p->wide_mode = wide_runs;
    if (!err.empty()) {
        delete p;
        return fail(CA_ERR_INVALID, "work list rejected: " + err);
    }
    *out = p;
    return CA_OK;
}

int ca_plan_array(const ca_plan* plan, int which, const int32_t** data, int64_t* count) {
    if (!plan || !data || !count) return fail(CA_ERR_INVALID, "null argument");
    const ca::Plan& pl = plan->plan;
    if (!pl.has_paths && (which == CA_PLAN_PATH_OFF || which == CA_PLAN_PATH_CHUNKS || which == CA_PLAN_PATH_TOKENS))
        ca::build_paths(const_cast<ca::Plan&>(pl));   // built on first use
    const std::vector<int32_t>* v = nullptr;
    switch (which) {
        case CA_PLAN_ITEMS:
            *data = reinterpret_cast<const int32_t*>(pl.items.data());
            *count = (int64_t)pl.items.size() * 16;
            return CA_OK;
        case CA_PLAN_MERGE_OFF: v = &pl.merge_off; break;
        case CA_PLAN_MERGE_SLOTS: v = &pl.merge_slots; break;
        case CA_PLAN_PATH_OFF: v = &pl.path_off; break;
        case CA_PLAN_PATH_CHUNKS: v = &pl.path_chunks; break;
        case CA_PLAN_PATH_TOKENS: v = &pl.path_tokens; break;
        case CA_PLAN_TAIL_CHUNK: v = &pl.tail_chunk; break;
        case CA_PLAN_TAIL_TOKENS: v = &pl.tail_tokens; break;
        case CA_PLAN_WIDE_CHUNKS: v = &pl.wide_chunks; break;
        default: return fail(CA_ERR_INVALID, "unknown plan array");
    }
    *data = v->data();
    *count = (int64_t)v->size();
    return CA_OK;
}

int ca_plan_stats_get(const ca_plan* plan, ca_plan_stats* out) {
    if (!plan || !out) return fail(CA_ERR_INVALID, "null argument");
    *out = plan->plan.stats;
    return CA_OK;
}

void ca_plan_destroy(ca_plan* plan) { delete plan; }

}  // extern "C"
