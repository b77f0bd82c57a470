// chunk_attn_c.ops — the three functions the reference's model code imports from the extension module
// (`from chunk_attn import ops`, src/chunk_attn/models/llama_hf/layernorm_vllm.py:7,
// rotary_embedding_vllm.py:30), with the reference's argument lists
// (cpp/chunk_attn/layernorm_kernels.h:8-16, pos_encoding_kernels.h:13-19).  They unwrap the
// tensors and call the C ABI on torch's current stream.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <stdexcept>

#include "../../../include/chunk_attn_b200.h"

namespace ca_host {
namespace {

int dtype_of(const torch::Tensor& t, const char* what) {
    if (t.scalar_type() == torch::kFloat16) return CA_DTYPE_F16;
    if (t.scalar_type() == torch::kFloat32) return CA_DTYPE_F32;
    throw std::runtime_error(std::string(what) + ": fp16 and fp32 tensors only");
}
void need(bool ok, const char* msg) {
    if (!ok) throw std::runtime_error(msg);
}
void check_rc(int rc, const char* what) {
    if (rc != CA_OK) throw std::runtime_error(std::string(what) + ": " + ca_last_error());
}
void* stream_of(const torch::Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

void rms_norm(torch::Tensor& out, torch::Tensor& input, torch::Tensor& weight, float epsilon) {
    need(input.is_cuda() && out.is_cuda() && weight.is_cuda(), "rms_norm: CUDA tensors are required (there is no CPU path)");
    need(input.is_contiguous() && out.is_contiguous() && weight.is_contiguous(), "rms_norm: tensors must be contiguous");
    need(out.sizes() == input.sizes() && out.scalar_type() == input.scalar_type() &&
           weight.scalar_type() == input.scalar_type() && weight.numel() == input.size(-1),
         "rms_norm: out/input/weight shapes or dtypes disagree");
    const int hidden = (int)input.size(-1);
    c10::cuda::CUDAGuard guard(input.device());
    check_rc(ca_rms_norm(out.data_ptr(), input.data_ptr(), weight.data_ptr(), epsilon, input.numel() / hidden, hidden,
                         dtype_of(input, "rms_norm"), stream_of(input)),
             "rms_norm");
}

void fused_add_rms_norm(torch::Tensor& input, torch::Tensor& residual, torch::Tensor& weight, float epsilon) {
    need(input.is_cuda() && residual.is_cuda() && weight.is_cuda(), "fused_add_rms_norm: CUDA tensors are required (there is no CPU path)");
    need(input.is_contiguous() && residual.is_contiguous() && weight.is_contiguous(), "fused_add_rms_norm: tensors must be contiguous");
    need(residual.sizes() == input.sizes() && residual.scalar_type() == input.scalar_type() &&
           weight.scalar_type() == input.scalar_type() && weight.numel() == input.size(-1),
         "fused_add_rms_norm: input/residual/weight shapes or dtypes disagree");
    const int hidden = (int)input.size(-1);
    c10::cuda::CUDAGuard guard(input.device());
    check_rc(ca_fused_add_rms_norm(input.data_ptr(), residual.data_ptr(), weight.data_ptr(), epsilon, input.numel() / hidden,
                                   hidden, dtype_of(input, "fused_add_rms_norm"), stream_of(input)),
             "fused_add_rms_norm");
}

// One int32 status word per device, made on first use: rotary_embedding skips tokens whose position lies
// outside the cos/sin table (the reference reads past the table) and records it here.
torch::Tensor status_tensor(torch::Device device) {
    static std::mutex mu;
    static std::map<int, torch::Tensor> words;
    std::lock_guard<std::mutex> lock(mu);
    auto it = words.find(device.index());
    if (it == words.end())
        it = words.emplace(device.index(), torch::zeros({1}, torch::TensorOptions().dtype(torch::kInt32).device(device))).first;
    return it->second;
}
int32_t* rotary_status_word(torch::Device device) { return status_tensor(device).data_ptr<int32_t>(); }

void rotary_embedding(torch::Tensor& positions, torch::Tensor& query, torch::Tensor& key, int head_size,
                      torch::Tensor& cos_sin_cache, bool is_neox) {
    need(query.is_cuda() && key.is_cuda() && positions.is_cuda() && cos_sin_cache.is_cuda(),
         "rotary_embedding: CUDA tensors are required (there is no CPU path)");
    need(positions.scalar_type() == torch::kInt64 && positions.is_contiguous(), "rotary_embedding: positions must be contiguous int64");
    need(query.dim() >= 2 && key.dim() >= 2 && query.stride(-1) == 1 && key.stride(-1) == 1 && cos_sin_cache.dim() == 2 &&
           cos_sin_cache.is_contiguous(),
         "rotary_embedding: query/key need a contiguous last dimension, cos_sin_cache must be [max_position, rot_dim]");
    need(key.scalar_type() == query.scalar_type() && cos_sin_cache.scalar_type() == query.scalar_type(),
         "rotary_embedding: query, key and cos_sin_cache must share a dtype");
    need(head_size > 0 && query.size(-1) % head_size == 0 && key.size(-1) % head_size == 0, "rotary_embedding: bad head_size");
    // tokens are addressed as token * stride(-2): the leading dimensions must collapse into one
    auto collapses = [](const torch::Tensor& t) {
        for (int64_t i = 0; i + 2 < t.dim(); i++)
            if (t.size(i) != 1 && t.stride(i) != t.stride(i + 1) * t.size(i + 1)) return false;
        return true;
    };
    need(collapses(query) && collapses(key), "rotary_embedding: the leading dimensions of query/key must be collapsible into one token axis");
    const int64_t num_tokens = query.numel() / query.size(-1);
    need(positions.numel() == num_tokens && key.numel() / key.size(-1) == num_tokens, "rotary_embedding: one position per token is required");
    c10::cuda::CUDAGuard guard(query.device());
    check_rc(ca_rotary_embedding(positions.data_ptr<int64_t>(), query.data_ptr(), key.data_ptr(), cos_sin_cache.data_ptr(),
                                 (int)cos_sin_cache.size(1), query.stride(-2), key.stride(-2), (int)(query.size(-1) / head_size),
                                 (int)(key.size(-1) / head_size), head_size, num_tokens, is_neox ? 1 : 0,
                                 dtype_of(query, "rotary_embedding"), cos_sin_cache.size(0),
                                 rotary_status_word(query.device()), stream_of(query)),
             "rotary_embedding");
}

// 0 when every position seen since the last call lay inside its cos/sin table, else 5; clears the word.
// Synchronises the current stream.
int rotary_embedding_status(torch::Device device) {
    torch::Tensor word = status_tensor(device);
    const int v = word.item<int>();
    if (v != 0) word.zero_();
    return v;
}

}  // namespace

void init_ops(pybind11::module& m) {
    m.def("rotary_embedding", &rotary_embedding, "Apply GPT-NeoX or GPT-J style rotary embedding to query and key");
    m.def("rotary_embedding_status", [](pybind11::object device) {
              return rotary_embedding_status(torch::python::detail::py_object_to_device(device));
          }, pybind11::arg("device"),
          "0, or 5 when rotary_embedding skipped a token whose position lay outside cos_sin_cache since the last call");
    m.def("rms_norm", &rms_norm, "Apply Root Mean Square (RMS) Normalization to the input tensor.");
    m.def("fused_add_rms_norm", &fused_add_rms_norm, "In-place fused Add and RMS Normalization");
}

}  // namespace ca_host
