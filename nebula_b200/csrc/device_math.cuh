// Scalar device helpers shared by every kernel: the reference's activation
// functions and TF32 rounding.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nebula_b200.h"

namespace nb {

// Round-to-nearest conversion of an fp32 value to TF32 (10-bit mantissa), kept
// in fp32 storage with the low 13 mantissa bits cleared.  The tensor core reads
// only the upper 19 bits of each operand, so pre-rounded data makes its result
// independent of how it treats the dropped bits.
__device__ __forceinline__ float round_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// The reference's CPU activations (common/activations.cc:6-91).  Its constants
// are doubles, so each formula is evaluated in double and stored back as float,
// which reproduces the CPU results including tanh's NaN for large inputs
// ((inf-1)/(inf+1)) and the non-textbook elu/hardtan/lhtan definitions.
__device__ __forceinline__ float apply_activation(float x, int act) {
    switch (act) {
        case NB_ACT_LINEAR: return x;
        case NB_ACT_RELU: return x > 0.0f ? x : 0.0f;
        case NB_ACT_LEAKY: return x > 0.0f ? x : (float)(0.1 * (double)x);
        case NB_ACT_RELIE: return x > 0.0f ? x : (float)(0.01 * (double)x);
        case NB_ACT_LOGISTIC: return (float)(1.0 / (1.0 + exp(0.0 - (double)x)));
        case NB_ACT_LOGGY: return (float)(2.0 / (1.0 + exp(0.0 - (double)x)) - 1.0);
        case NB_ACT_TANH: {
            const double e = exp(2.0 * (double)x);
            return (float)((e - 1.0) / (e + 1.0));
        }
        case NB_ACT_ELU: return x > 0.0f ? x * x : (float)((double)x * (exp((double)x) - 1.0));
        case NB_ACT_HARDTAN: return (x < 1.0f && x > -1.0f) ? 1.0f : 0.0f;
        case NB_ACT_LHTAN: return (x > 0.0f && x < 1.0f) ? 1.0f : 0.0f;
        case NB_ACT_PLSE:
            if (x < -4.0f) return (float)(0.01 * ((double)x + 4.0));
            if (x > 4.0f) return (float)(0.01 * ((double)x - 4.0) + 1.0);
            return (float)(0.125 * (double)x + 0.5);
        case NB_ACT_RAMP: return x > 0.0f ? (float)((double)x * ((double)x + 0.01)) : (float)(0.01 * (double)x);
        case NB_ACT_STAIR: {
            const int n = (int)x;
            if (n % 2) return x - (float)n + (float)(int)((double)x / 2.0);
            return (float)(int)((double)x / 2.0);
        }
        default: return x;
    }
}

// Out-of-line copy for unrolled epilogues: keeps the (large) switch out of the
// instruction stream of loops that almost always run relu / leaky / linear.
static __device__ __noinline__ float apply_activation_call(float x, int act) { return apply_activation(x, act); }

// One LSTM cell update (lstm_layer.cc:286-311) from the four gate pre-activations of a hidden unit: out of line to
// keep the GEMM epilogue small, with the four gate activations inline so that their exp chains overlap. The
// products and the sum round to fp32 separately, as the CPU path's loops do.
static __device__ __noinline__ float2 lstm_cell_unit(float zi, float zf, float zg, float zo, float c_prev) {
    const float ig = apply_activation(zi, NB_ACT_LOGISTIC);
    const float fg = apply_activation(zf, NB_ACT_LOGISTIC);
    const float gg = apply_activation(zg, NB_ACT_TANH);
    const float og = apply_activation(zo, NB_ACT_LOGISTIC);
    const float c = __fadd_rn(__fmul_rn(c_prev, fg), __fmul_rn(ig, gg));
    return make_float2(c, __fmul_rn(apply_activation(c, NB_ACT_TANH), og));
}

// The same update with the gate activations evaluated in fp32 (expf/tanhf, a few ulp from the double formulas):
// used by the TF32 GEMM epilogue, where the pre-activations already carry ~1e-3 of operand rounding and the few
// epilogue threads of a small-batch step cannot hide double-precision latency.
__device__ __forceinline__ float2 lstm_cell_unit_f32_inline(float zi, float zf, float zg, float zo, float c_prev) {
    const float ig = 1.0f / (1.0f + expf(-zi));
    const float fg = 1.0f / (1.0f + expf(-zf));
    const float gg = tanhf(zg);
    const float og = 1.0f / (1.0f + expf(-zo));
    const float c = __fadd_rn(__fmul_rn(c_prev, fg), __fmul_rn(ig, gg));
    return make_float2(c, __fmul_rn(tanhf(c), og));
}
// (out of line for the GEMM epilogue, which has no registers to spare; the same operations in the same order)
static __device__ __noinline__ float2 lstm_cell_unit_f32(float zi, float zf, float zg, float zo, float c_prev) {
    const float ig = 1.0f / (1.0f + expf(-zi));
    const float fg = 1.0f / (1.0f + expf(-zf));
    const float gg = tanhf(zg);
    const float og = 1.0f / (1.0f + expf(-zo));
    const float c = __fadd_rn(__fmul_rn(c_prev, fg), __fmul_rn(ig, gg));
    return make_float2(c, __fmul_rn(tanhf(c), og));
}

// relu, leaky and linear inline; everything else through the out-of-line copy
__device__ __forceinline__ float apply_activation_fast(float x, int act) {
    if (act == NB_ACT_RELU) return x > 0.0f ? x : 0.0f;
    if (act == NB_ACT_LINEAR) return x;
    if (act == NB_ACT_LEAKY) return x > 0.0f ? x : (float)(0.1 * (double)x);
    return apply_activation_call(x, act);
}

}  // namespace nb
