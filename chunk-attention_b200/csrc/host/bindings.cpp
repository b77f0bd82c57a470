// pybind11 module chunk_attn_c: the Python surface of the reference's module of the same name
// (cpp/chunk_attn/python_exports.cpp:11-87) — classes Attention, Chunk, IntFuture with the same
// constructor keywords, defaults, method names and return-value policies — plus PrefixTree, the
// host-only tree, for checks that need no device.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "attention.h"

namespace py = pybind11;
using ca_host::Attention;
using ca_host::Chunk;
using ca_host::PrefixTree;

namespace ca_host {
void init_ops(py::module& m);
}

namespace {

py::dict stats_to_dict(const ca_plan_stats& st) {
    py::dict d;
    d["unique_kv_bytes"] = st.unique_kv_bytes;
    d["n_chunks"] = st.n_chunks;
    d["n_shared_chunks"] = st.n_shared_chunks;
    d["n_runs"] = st.n_runs;
    d["n_items"] = st.n_items;
    d["n_slots"] = st.n_slots;
    d["n_ctas"] = st.n_ctas;
    d["fast_path"] = st.fast_path;
    d["kernels_per_step"] = st.kernels_per_step;
    d["n_items_cf"] = st.n_items_cf;
    d["n_items_short"] = st.n_items_short;
    d["n_items_wide"] = st.n_items_wide;
    return d;
}

}  // namespace

// module_local: the reference's own extension registers types with the same names; keeping these
// local lets both be imported into one interpreter (the parity tests do that).
PYBIND11_MODULE(chunk_attn_c, m) {
    py::class_<std::future<int>, std::shared_ptr<std::future<int>>>(m, "IntFuture", py::module_local())
      .def(py::init<>())
      // the GIL is released while waiting: the worker may need it to drop a tensor reference
      .def("get", &std::future<int>::get, py::call_guard<py::gil_scoped_release>());

    py::class_<Chunk>(m, "Chunk", py::module_local())
      .def_readonly("children", &Chunk::children, py::return_value_policy::reference)
      .def_readonly("tokens", &Chunk::tokens)
      .def_property_readonly("capacity", &Chunk::capacity)
      .def_readonly("n_seqs", &Chunk::n_seqs)
      .def_property_readonly("n_tokens", &Chunk::n_tokens)
      .def_readonly("id", &Chunk::id);

    py::class_<Attention, std::shared_ptr<Attention>>(m, "Attention", py::module_local())
      .def(py::init([](int n_heads, int d_head, int chunk_size, int memory_mb, bool share_prefix, int tpp_threshold,
                       py::object dtype, py::object device) {
               torch::Dtype dtype_c = torch::get_default_dtype_as_scalartype();
               if (!dtype.is_none()) dtype_c = torch::python::detail::py_object_to_dtype(dtype);
               // the default device is wherever a fresh tensor lands; asking Python (not libtorch)
               // honours `with torch.device(...)` and torch.set_default_device, which live there
               if (device.is_none()) device = py::module_::import("torch").attr("empty")(0).attr("device");
               // a device given by name ("cuda:0"), as the reference's llama_hf passes its config.torch_device
               if (py::isinstance<py::str>(device)) device = py::module_::import("torch").attr("device")(device);
               if (py::isinstance<py::str>(dtype)) dtype = py::module_::import("torch").attr(dtype);
               torch::Device device_c = torch::python::detail::py_object_to_device(device);
               return new Attention(n_heads, d_head, chunk_size, memory_mb, share_prefix, tpp_threshold, dtype_c,
                                    device_c);
           }),
           py::arg("n_heads") = 12, py::arg("d_head") = 64, py::arg("chunk_size") = 64, py::arg("memory_mb") = 1024,
           py::arg("share_prefix") = true, py::arg("tpp_threshold") = 1, py::arg("dtype") = py::none(),
           py::arg("device") = py::none())
      .def(py::init<Attention&>())
      .def("forward", &Attention::forward, py::arg("q"), py::arg("partition") = 0)
      .def("add_seq", &Attention::add_seq, py::arg("tokens"), py::arg("k"), py::arg("v"))
      .def("add_seq_async", &Attention::add_seq_async, py::arg("tokens"), py::arg("k"), py::arg("v"))
      .def("append_token", &Attention::append_token, py::arg("tokens"), py::arg("k"), py::arg("v"),
           py::arg("fused") = true, py::return_value_policy::reference)
      .def("refresh_kernel_context", &Attention::refresh_kernel_context, py::arg("force") = false)
      .def("reserve", &Attention::reserve, py::return_value_policy::reference)
      .def("duplicate", &Attention::duplicate, py::arg("seq_idx"), py::arg("copies"))
      .def("append_completion", &Attention::append_completion, py::arg("seq_idx"), py::arg("tokens"), py::arg("k"),
           py::arg("v"))
      .def("remove_seq", &Attention::remove_seq, py::arg("seq_idx"))
      .def("clear", &Attention::clear)
      .def("get_trie", &Attention::get_trie, py::return_value_policy::reference)
      .def_property_readonly("tails", &Attention::tails, py::return_value_policy::reference)
      .def("print", &Attention::print, py::arg("root") = nullptr, py::arg("level") = 0)
      .def("peak_memory_allocated", &Attention::peak_memory_allocated)
      // additions (not in the reference): counters of the current work list, tuning, kernel status
      .def("plan_stats", [](Attention& a) { return stats_to_dict(a.plan_stats()); })
      .def("set_option", &Attention::set_option, py::arg("option"), py::arg("value"))
      .def("device_status", &Attention::device_status)
      .def("plan_sharing", &Attention::plan_sharing)
      .def("host_times", [](Attention& a) {
          const auto t = a.host_times();
          py::dict d;
          d["refreshes"] = t.refreshes;
          d["walk_us"] = t.walk_ns * 1e-3;
          d["plan_us"] = t.plan_ns * 1e-3;
          d["upload_us"] = t.upload_ns * 1e-3;
          return d;
      })
      // blocks until the result is in host memory: other Python threads run meanwhile
      .def("forward_host", &Attention::forward_host, py::arg("q"), py::arg("out") = py::none(), py::arg("partition") = 0,
           py::call_guard<py::gil_scoped_release>())
      .def("forward_to_peers", &Attention::forward_to_peers, py::arg("q"), py::arg("peer_out_ptrs"),
           py::arg("total_heads"), py::arg("head_offset"), py::arg("multicast_ptr") = 0)
      .def("attn_partials", &Attention::attn_partials, py::arg("q"), py::arg("phases") = 3)
      .def("attn_merge", &Attention::attn_merge, py::arg("out"));

    // the reference carries this submodule whenever it is built for CUDA (python_exports.cpp:83-86)
    py::module ops = m.def_submodule("ops");
    ca_host::init_ops(ops);

    py::class_<PrefixTree>(m, "PrefixTree", py::module_local())
      .def(py::init([](int chunk_size, int64_t max_chunks, bool share_prefix) {
               return new PrefixTree(chunk_size, max_chunks, 1, share_prefix);
           }),
           py::arg("chunk_size"), py::arg("max_chunks"), py::arg("share_prefix") = true)
      .def("add_seq",
           [](PrefixTree& t, const std::vector<int>& tokens) {
               std::vector<ca_host::NewChunk> created;
               return t.add_seq(tokens, created);
           },
           py::arg("tokens"))
      .def("add_seq_detailed",
           [](PrefixTree& t, const std::vector<int>& tokens) {
               // (row index, [(chunk id, first token position, token count)] of the chunks to fill)
               std::vector<ca_host::NewChunk> created;
               const int idx = t.add_seq(tokens, created);
               std::vector<std::tuple<int, int, int>> out;
               for (const auto& nc : created) out.emplace_back(nc.chunk->id, nc.token_start, nc.n_tokens);
               return std::make_pair(idx, out);
           },
           py::arg("tokens"))
      .def("remove_seq", &PrefixTree::remove_seq, py::arg("seq_idx"))
      .def("reserve", &PrefixTree::reserve, py::return_value_policy::reference)
      .def("append_token",
           [](PrefixTree& t, const std::vector<int>& tokens) {
               if (t.tails().size() != tokens.size())
                   throw std::runtime_error("num of seqs is not equal to num of tokens");
               t.reserve();
               t.append_token_ids(tokens);
           },
           py::arg("tokens"))
      .def("duplicate",
           [](PrefixTree& t, int seq_idx, int copies) {
               std::vector<std::pair<Chunk*, Chunk*>> pairs;
               t.duplicate(seq_idx, copies, pairs);
               std::vector<std::pair<int, int>> ids;
               for (auto& p : pairs) ids.emplace_back(p.first->id, p.second->id);
               return ids;
           },
           py::arg("seq_idx"), py::arg("copies"))
      .def("append_completion",
           [](PrefixTree& t, int seq_idx, const std::vector<int>& tokens) {
               // ([(source chunk id, clone chunk id)], [(chunk id, row) of token i])
               std::vector<std::pair<Chunk*, Chunk*>> pairs;
               std::vector<std::pair<Chunk*, int>> slots;
               t.append_completion(seq_idx, tokens, pairs, slots);
               std::vector<std::pair<int, int>> p, s;
               for (auto& x : pairs) p.emplace_back(x.first->id, x.second->id);
               for (auto& x : slots) s.emplace_back(x.first->id, x.second);
               return std::make_pair(p, s);
           },
           py::arg("seq_idx"), py::arg("tokens"))
      .def("clear", &PrefixTree::clear)
      .def("get_trie", &PrefixTree::root, py::return_value_policy::reference)
      .def_property_readonly("tails", &PrefixTree::tails, py::return_value_policy::reference)
      .def("get_chunks",
           [](PrefixTree& t) {
               std::vector<std::tuple<int, int, int, int>> out;
               for (const ca_chunk_info& ci : t.get_chunks())
                   out.emplace_back(ci.chunk_id, ci.n_tokens, ci.seq_begin, ci.seq_end);
               return out;
           })
      .def("chunks_in_use", [](PrefixTree& t) { return t.pool().in_use(); });
}
