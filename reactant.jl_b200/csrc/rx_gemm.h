// dot_general launcher (src/Ops.jl:1075-1200): bf16/f32 operands, fp32 accumulate.
#pragma once
#include <string>

#include "rx_runtime.h"

namespace rx {
// `epilogue`: the step's program with operand / result pointers bound, when the step carries a fused epilogue
// (st.gemm.has_epilogue); col_partial / full_partial: the partial-sum buffers of its reductions.
struct GemmEpilogueArgs {
  const VmProgram* prog = nullptr;
  float* col_partial[2] = {nullptr, nullptr};
  float* full_partial[2] = {nullptr, nullptr};
};
// for compile-only checks of a fused step (no device needed)
std::string gemm_epilogue_members(const GemmDesc& g);
const char* gemm_epilogue_family(bool wide);
cudaError_t run_gemm(RxDevice* d, const Step& st, const void* a, const void* b, void* out, const GemmEpilogueArgs* epilogue = nullptr);
}
