// Test-side shim (not product code, not reference code), force-included when the reference's
// CUDA build is compiled for the parity comparator. The reference logs tensor.dtype() through
// spdlog/fmt (cpp/chunk_attn/kernel_cuda.cu:1189,1267,1314); fmt >= 10 needs an explicit
// formatter for a type that only has operator<<.
#pragma once
#include <spdlog/spdlog.h>
#include <spdlog/fmt/ostr.h>
#include <c10/util/typeid.h>
template <>
struct fmt::formatter<caffe2::TypeMeta> : fmt::ostream_formatter {};
