// Test-side shim (not product code, not reference code).
//
// The reference includes oneMKL's <mkl_vml_functions.h> for vsExp
// (cpp/chunk_attn/kernel_cpu_mkl.cpp:3,69,99,100,180). libtorch_cpu.so exports vsExp from
// the oneMKL it embeds; this header only declares it.
#pragma once

extern "C" void vsExp(const int n, const float* a, float* r);
