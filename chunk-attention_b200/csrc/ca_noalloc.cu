// ca_attention_static: the decode step for callers that must not allocate device memory.
//
// Who that is: a plugin running inside a serving process whose framework has taken the whole GPU
// for its own arena at start-up (a raw cudaMalloc then fails, or is forbidden by policy), and a
// latency-critical decode loop that cannot afford the device-wide synchronisation cudaMalloc and
// cudaFree imply.  The ordinary entry point, ca_attention, keeps its partial results in scratch
// that ca_refresh_kernel_context grows with cudaMalloc; this one keeps them in a fixed array that
// is part of the library image, and takes every table it reads as a caller-owned device pointer.
//
// The scratch is one file-scope __device__ array, CA_STATIC_MAX_SLOTS partial rows
// (CA_STATIC_MAX_SLOTS * 520 bytes, about 8.1 MiB).  Every GPU that loads the library carries it
// until the process exits, which is why it is kept modest.  A work list that needs more partial
// rows is refused with CA_ERR_INVALID.
#include <cuda_runtime.h>

#include <cmath>
#include <mutex>
#include <string>

#include "../../include/chunk_attn_b200.h"
#include "ca_kernels.h"

namespace {

constexpr int kMaxSlots = CA_STATIC_MAX_SLOTS;
constexpr size_t kPartOBytes = (size_t)kMaxSlots * ca::FAST_D * sizeof(float);
constexpr size_t kPartMlBytes = (size_t)kMaxSlots * sizeof(float2);
constexpr int kMaxDevices = 64;

// Partial outputs [kMaxSlots][128] fp32, then (max, sum) pairs [kMaxSlots].  In HOST code this name
// is only a handle for cudaGetSymbolAddress, never an address a kernel can use.
static __device__ __align__(256) unsigned char g_static_scratch[kPartOBytes + kPartMlBytes];
// Kernel status word used when the caller passes none; cleared at the start of every call and readable with
// ca_attention_static_status.
static __device__ int g_static_status;
// The item counter the self-scheduling kernel draws from, and a spare word the kernel zeroes for "the
// launch after it" (the ordinary entry point alternates two counters that way; here every call zeroes its
// own counter on the stream, so a call does not depend on how the one before it ended).
static __device__ int g_static_counters[2];

struct DeviceSetup {
    bool done = false;
    unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
    int* status = nullptr;             // device address of g_static_status on this device
    int* counters = nullptr;           // device address of g_static_counters on this device
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

int fail(int code, const std::string& msg) {
    ca::set_last_error(msg);  // read back with ca_last_error()
    return code;
}

}  // namespace

extern "C" {

int ca_attention_static(const void* pool, int n_heads, const void* q, void* out, int n_seqs,
                        const int32_t* items, int n_items, int n_ctas, const int32_t* merge_off,
                        const int32_t* merge_slots, int n_slots, int delta_tokens, int32_t* status,
                        ca_stream stream_) {
    if (n_seqs < 0 || n_heads <= 0 || n_items < 0 || n_ctas < 0 || n_slots < 0 || delta_tokens < 0)
        return fail(CA_ERR_INVALID, "negative size");
    if (n_slots > kMaxSlots)
        return fail(CA_ERR_INVALID, "work list needs " + std::to_string(n_slots) + " partial rows; the static scratch holds " +
                                        std::to_string(kMaxSlots) + " (CA_STATIC_MAX_SLOTS): use ca_attention, or plan fewer, larger pieces");
    if (n_ctas > 4096) return fail(CA_ERR_INVALID, "more than 4096 CTAs");
    if (n_slots % n_heads != 0) return fail(CA_ERR_INVALID, "n_slots must be a multiple of n_heads (ca_plan_stats.n_slots is)");
    if ((long long)n_items * n_heads > INT32_MAX) return fail(CA_ERR_INVALID, "too many items");
    if (n_seqs == 0) return CA_OK;
    if (!pool || !q || !out || !items || !merge_off || !merge_slots) return fail(CA_ERR_INVALID, "null pointer");
    if (n_ctas < 1 || n_items < 1) return fail(CA_ERR_INVALID, "a non-empty batch needs at least one item and one CTA");
    if (reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(out) % 8 ||
        reinterpret_cast<uintptr_t>(pool) % 256 || reinterpret_cast<uintptr_t>(items) % 16)
        return fail(CA_ERR_INVALID, "misaligned pointer (pool 256, q and items 16, out 8 bytes)");

    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices) return fail(CA_ERR_INVALID, "device index out of range");
    DeviceSetup& su = g_setup[device];
    {
        // First call on this device: look up where this device keeps the two symbols and opt the
        // kernel in to its shared-memory size.  Neither allocates.
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!su.done) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
            su.scratch = static_cast<unsigned char*>(p);
            e = cudaGetSymbolAddress(&p, g_static_status);
            if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("cudaGetSymbolAddress(status): ") + cudaGetErrorString(e));
            su.status = static_cast<int*>(p);
            e = cudaGetSymbolAddress(&p, g_static_counters);
            if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("cudaGetSymbolAddress(counters): ") + cudaGetErrorString(e));
            su.counters = static_cast<int*>(p);
            e = ca::configure_fast_kernels();
            if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
            su.done = true;
        }
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int* status_word = status ? status : su.status;
    // The scratch keeps whatever the previous call left in it.  No partial row has to start at
    // zero: every row a merge list names is written by this call before it is read.  Two words do
    // have to start at zero and are cleared here, on the stream, by every call: the status word
    // (kernels only ever set it) and the item counter the launch draws from (a call therefore
    // does not depend on how the previous one ended: a failed launch, or the same call replayed).
    e = cudaMemsetAsync(status_word, 0, sizeof(int), stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(su.counters, 0, 2 * sizeof(int), stream);
    if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));

    ca::PartialParams p;
    p.pool = static_cast<const uint8_t*>(pool);
    p.n_heads = n_heads;
    p.q = q;
    p.items = reinterpret_cast<const int4*>(items);
    p.item_lo = 0;
    p.item_hi = n_items * n_heads;  // every item stands for one piece of work per head
    p.counter = su.counters;
    p.counter_next = su.counters + 1;
    p.part_o = reinterpret_cast<float*>(su.scratch);
    p.part_ml = reinterpret_cast<float2*>(su.scratch + kPartOBytes);
    p.delta_tokens = delta_tokens;
    p.scale_log2 = 1.4426950408889634f / std::sqrt((float)ca::FAST_D);
    p.status = status_word;
    // The work list lives in device memory the host never saw: the kernels check every slot, row and head
    // it names against these sizes, skip what falls outside and report STATUS_BAD_WORK_LIST (4).  The pool's
    // size is not known here, so chunk numbers are taken as they come (max_chunks = 0).
    p.n_slots = n_slots;
    p.n_seqs = n_seqs;
    e = ca::launch_attn_partials(p, n_ctas < p.item_hi ? n_ctas : p.item_hi, stream);
    if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("partial kernel launch: ") + cudaGetErrorString(e));
    ca::MergeParams m;
    m.part_o = p.part_o;
    m.part_ml = p.part_ml;
    m.merge_off = merge_off;
    m.merge_slots = merge_slots;
    m.out = out;
    m.n_pairs = n_seqs * n_heads;
    m.n_merge_entries = n_slots / n_heads;  // every partial row is named once, per item, for all heads
    m.n_slots = n_slots;
    m.status = status_word;
    m.n_heads = n_heads;
    e = ca::launch_attn_merge(m, stream, true);
    if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("merge kernel launch: ") + cudaGetErrorString(e));
    return CA_OK;
}

int ca_attention_static_status(int32_t* status, ca_stream stream_) {
    if (!status) return fail(CA_ERR_INVALID, "status is null");
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices || !g_setup[device].done) {
        *status = 0;  // no call has run on this device yet
        return CA_OK;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int32_t host = 0;
    e = cudaMemcpyAsync(&host, g_setup[device].status, sizeof(int32_t), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(CA_ERR_CUDA, std::string("reading the status word: ") + cudaGetErrorString(e));
    *status = host;
    return host == 0 ? CA_OK : fail(CA_ERR_DEVICE_STATUS, "a kernel of ca_attention_static reported status " + std::to_string(host));
}

}  // extern "C"
