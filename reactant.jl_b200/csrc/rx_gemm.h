// dot_general launcher (src/Ops.jl:1075-1200): bf16/f32 operands, fp32 accumulate.
#pragma once
#include "rx_runtime.h"

namespace rx {
cudaError_t run_gemm(RxDevice* d, const Step& st, const void* a, const void* b, void* out);
}
