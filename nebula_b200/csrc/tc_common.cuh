// Shared device code of the tcgen05 kernels: PTX wrappers (mbarrier, TMA, tcgen05),
// descriptor builders, and the fused epilogue that both the generic GEMM kernel and
// the 3x3 halo convolution kernel run on every 128-row x 32-column slab.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_math.cuh"
#include "nb_internal.h"

namespace nb {
namespace tc {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 32;                  // fp32 elements = one 128-byte swizzle row
constexpr int UMMA_K = 8;                    // tf32
constexpr int A_STAGE_BYTES = BLOCK_M * BLOCK_K * 4;   // 16 KiB
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;  // ~2 s at 2 GHz


// What the epilogue needs to know, common to both kernels.
struct EpiParams {
    const float *scale, *shift, *addend;    // scale/shift readable up to the next multiple of 32 columns
    long ld_addend;
    int addend_vec;             // addend rows are 16-byte aligned
    int addend_cols;            // columns the addend covers (a residual may have fewer channels than the output)
    int addend_post;            // add the addend AFTER the activation (the sum of two activated gate layers) instead of before
    // residual mode (res_stride > 0): the addend is an NHWC tensor [NB][res_h][res_w][ld_addend] and output
    // pixel (n,oh,ow) takes pixel (n, oh*res_stride, ow*res_stride) of it -- the reference's shortcut
    // (common/utils.cc:28-60) with sample == 1; otherwise the addend has the output's own row indexing
    int res_stride, res_h, res_w;
    int act, round_out;
    float *y;
    long ldy;
    int tma_store;              // y meets TMA's rules: slabs leave through a tensor map; else plain stores
    int pool;                   // fuse the following 2x2 stride-2 max-pool: only the pooled tensor is written
    int N;                      // valid output columns
    // LSTM mode (lstm_H > 0): columns are gate pre-activations laid out [hidden unit][i,f,g,o]; instead of
    // storing them the epilogue runs the cell update (lstm_layer.cc:286-311) and writes c_t, h_t [rows][H]
    int lstm_H;
    int lstm_vec;               // H % 8 == 0 and 16-byte aligned state tensors: 128-bit loads and stores
    int lstm_f32;               // gate activations in fp32 (TF32 mode) instead of the double formulas
    const float *lstm_c_prev;   // may be null (c_{t-1} = 0)
    float *lstm_c, *lstm_h, *lstm_h_round;      // lstm_h_round may be null
};
// Per thread: its row of the staging slab (-1: this accumulator row is not an output pixel), the
// output pixel index for plain stores / addend reads, and whether that pixel exists.
struct EpiRow { int srow; long grow; bool row_ok; const float *arow; };

// This pixel's addend row (nullptr: nothing to add).
__device__ __forceinline__ const float *addend_row(const EpiParams &e, bool row_ok, long grow, int n, int oh, int ow) {
    if (!e.addend || !row_ok) return nullptr;
    if (e.res_stride == 0) return e.addend + grow * e.ld_addend;
    const int ih = oh * e.res_stride, iw = ow * e.res_stride;
    if (oh >= e.res_h || ow >= e.res_w || ih >= e.res_h || iw >= e.res_w) return nullptr;
    return e.addend + (((long)n * e.res_h + ih) * e.res_w + iw) * e.ld_addend;
}
// The pixel box one slab covers and its origin in output coordinates.
struct EpiBox { int bw, bh, bn, ow0, oh0, n0; };

// ------------------------------------------------------------------ PTX glue
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// try_wait that lets the hardware park the thread (up to `ns`) until the phase completes, so a
// waiting role does not take issue slots from the warps that share its scheduler
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t *bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait or another ran out).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; i++)
            if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            atomicExch(status, (int)DEV_TIMEOUT);
            return false;
        }
    }
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *tm, uint64_t *bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(void *dst, const CUtensorMap *tm, uint64_t *bar, int c0, int c1, int c2, int c3,
                                            int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *tm, uint64_t *bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *tm, uint64_t *bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap *tm, const void *src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(tm), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Named barrier `id` over the 128 threads of one epilogue group.  The form without `.aligned` counts threads, not
// warps, so a warp whose lanes arrive from different sides of a branch is still counted once per lane; the warp is
// re-converged first because the instructions that follow (tcgen05.ld, the next barrier) want it whole.
__device__ __forceinline__ void epilogue_bar_sync(int id) {
    __syncwarp();
    asm volatile("barrier.cta.sync %0, 128;" ::"r"(id) : "memory");
}
// AND-vote across the 128 threads of an epilogue group (named barrier `id`), so that leaving
// the tile loop is a uniform decision and no thread is left alone at a later bar.sync.
__device__ __forceinline__ bool epilogue_all(bool pred, int id) {
    uint32_t r;
    __syncwarp();       // the waits before this vote end lane by lane
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %1, 0;\n\t"
        "barrier.cta.red.and.pred q, %2, 128, p;\n\t"
        "selp.b32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)pred), "r"(id)
        : "memory");
    return r != 0;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 B
// apart, 8-row groups 1024 B apart (bits: start>>4 [0,14), LBO>>4 [16,30),
// SBO>>4 [32,46), version=1 [46,48), layout=SWIZZLE_128B(2) [61,64)).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// The same descriptor split in halves, for the MMA issue loop: the upper word is a constant, the lower
// word is (start >> 4) | LBO, so stepping the start address by b bytes is `lo += b >> 4` (shared-memory
// addresses stay below 2^18, so the 14-bit field never carries).
constexpr uint32_t SMEM_DESC_HI = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFF) | (1u << 16); }
__device__ __forceinline__ uint64_t smem_desc(uint32_t lo) { return ((uint64_t)SMEM_DESC_HI << 32) | lo; }
// (An operand read at a row offset -- a start address off the pattern's 1024-byte repeat -- keeps base offset 0 as
// long as the data was laid down by TMA: both sides derive the swizzle phase from the absolute shared-memory address.
// Measured: a non-zero base offset on such a descriptor garbles the product.)

// Instruction descriptor for kind::tf32: D=f32 (bits 4-5 = 1), A=B=tf32 (bits
// 7-9, 10-12 = 2), both K-major (bits 15,16 = 0), N>>3 at bit 17, M>>4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ float4 lds128(const float *p) {
    float4 r;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(smem_u32(p)));
    return r;
}

// Warp-wide (.sync.aligned): the warp is re-converged first, whatever branch its lanes came from.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
    __syncwarp();
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    __syncwarp();
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}


// One 128-row x 32-column slab of accumulators (already in registers): folded batch-norm
// scale/shift + bias, optional addend, activation, optional TF32 rounding, then either a swizzled
// staging slab that leaves by TMA (optionally 2x2/2 max-pooled first) or plain global stores.
// Called by the 128 threads of one epilogue group; `t` is the thread's index in the group.
// F64_CELL: the LSTM cell's activations by the reference's double formulas (the 3xTF32 kernels) instead of fp32 ones;
// a compile-time choice because the double path's registers would otherwise be charged to every epilogue mode.
// `stores_in_flight`: bulk stores of this group that may still be reading their staging buffer when this slab's
// buffer is written (1 when the group alternates between two buffers, else 0).  `staged()` is called once the
// accumulators have left the registers (staged in shared memory): the caller starts the next `tcgen05.ld` there, so
// that its latency passes behind the fence, the barrier and the store; it is not called in the modes that keep
// the values in registers to the end (plain stores, the LSTM cell).
template <bool F64_CELL, class Staged>
__device__ __forceinline__ void epilogue_chunk(const EpiParams &e, const CUtensorMap *tm_y, const CUtensorMap *tm_yp,
                                               uint32_t (&v)[32], int col0, const EpiRow &rw, const EpiBox &bx,
                                               float4 *slab, int bar_id, bool store_thread, int t, int stores_in_flight,
                                               Staged &&staged, const float *aff = nullptr, int aff_shift = 0) {
    const bool full_cols = col0 + 32 <= e.N;
    // affine part: folded batch-norm scale/shift + bias (vectors padded to a multiple of 32).  `aff`: this slab's 32
    // scale values in shared memory and its 32 shift values `aff_shift` floats further (the caller stages them once per
    // tile column: read from global memory here, 8-16 loads sit on every slab's critical path)
    if (aff) {
        if (e.scale) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 sc = lds128(aff + j), sh = lds128(aff + aff_shift + j);
                v[j] = __float_as_uint(fmaf(__uint_as_float(v[j]), sc.x, sh.x));
                v[j + 1] = __float_as_uint(fmaf(__uint_as_float(v[j + 1]), sc.y, sh.y));
                v[j + 2] = __float_as_uint(fmaf(__uint_as_float(v[j + 2]), sc.z, sh.z));
                v[j + 3] = __float_as_uint(fmaf(__uint_as_float(v[j + 3]), sc.w, sh.w));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 sh = lds128(aff + aff_shift + j);
                v[j] = __float_as_uint(__uint_as_float(v[j]) + sh.x);
                v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + sh.y);
                v[j + 2] = __float_as_uint(__uint_as_float(v[j + 2]) + sh.z);
                v[j + 3] = __float_as_uint(__uint_as_float(v[j + 3]) + sh.w);
            }
        }
    } else if (e.scale) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 sc = __ldg(reinterpret_cast<const float4 *>(e.scale + col0 + j));
            const float4 sh = __ldg(reinterpret_cast<const float4 *>(e.shift + col0 + j));
            v[j] = __float_as_uint(fmaf(__uint_as_float(v[j]), sc.x, sh.x));
            v[j + 1] = __float_as_uint(fmaf(__uint_as_float(v[j + 1]), sc.y, sh.y));
            v[j + 2] = __float_as_uint(fmaf(__uint_as_float(v[j + 2]), sc.z, sh.z));
            v[j + 3] = __float_as_uint(fmaf(__uint_as_float(v[j + 3]), sc.w, sh.w));
        }
    } else if (e.shift) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 sh = __ldg(reinterpret_cast<const float4 *>(e.shift + col0 + j));
            v[j] = __float_as_uint(__uint_as_float(v[j]) + sh.x);
            v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + sh.y);
            v[j + 2] = __float_as_uint(__uint_as_float(v[j + 2]) + sh.z);
            v[j + 3] = __float_as_uint(__uint_as_float(v[j + 3]) + sh.w);
        }
    }
    auto add_addend = [&]() {
        const float *arow = rw.arow + col0;
        if (col0 + 32 <= e.addend_cols && e.addend_vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 ad = *reinterpret_cast<const float4 *>(arow + j);
                v[j] = __float_as_uint(__uint_as_float(v[j]) + ad.x);
                v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + ad.y);
                v[j + 2] = __float_as_uint(__uint_as_float(v[j + 2]) + ad.z);
                v[j + 3] = __float_as_uint(__uint_as_float(v[j + 3]) + ad.w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (col0 + j < e.addend_cols) v[j] = __float_as_uint(__uint_as_float(v[j]) + arow[j]);
        }
    };
    auto activate = [&]() {
        // the common ones inline, the rest through one out-of-line call per value
        if (e.act == NB_ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __float_as_uint(fmaxf(__uint_as_float(v[j]), 0.0f));   // NaN and -0 give +0, as x > 0 ? x : 0 does
        } else if (e.act == NB_ACT_LEAKY) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float x = __uint_as_float(v[j]);
                v[j] = __float_as_uint(x > 0.0f ? x : (float)(0.1 * (double)x));
            }
        } else if (e.act != NB_ACT_LINEAR) {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __float_as_uint(apply_activation_call(__uint_as_float(v[j]), e.act));
        }
    };
    const bool has_addend = rw.arow && col0 < e.addend_cols;
    if (has_addend && !e.addend_post) add_addend();
    if (e.addend_post) {        // act(acc*scale + shift) + addend: two activated layers summed (lstm_layer.cc:252-282)
        activate();
        if (has_addend) add_addend();
    }
    if (e.lstm_H > 0) {
        // 32 columns = 8 hidden units x (i, f, g, o): the cell update of this row's units, with the CPU
        // path's separate fp32 roundings (no fused multiply-add)
        const int j0 = col0 >> 2;
        if (rw.row_ok && j0 < e.lstm_H) {
            const long idx0 = rw.grow * e.lstm_H + j0;
            // four units at a time (the 32 accumulators plus the states of all eight at once cost the other epilogue
            // modes registers); within a half the loads of c_{t-1} overlap
#pragma unroll
            for (int q = 0; q < 2; q++) {
                float cp[4], cn[4], hn[4];
                const long idx = idx0 + 4 * q;
                if (!e.lstm_c_prev) {
#pragma unroll
                    for (int u = 0; u < 4; u++) cp[u] = 0.0f;
                } else if (e.lstm_vec) {
                    const float4 c4 = *reinterpret_cast<const float4 *>(e.lstm_c_prev + idx);
                    cp[0] = c4.x; cp[1] = c4.y; cp[2] = c4.z; cp[3] = c4.w;
                } else {
#pragma unroll
                    for (int u = 0; u < 4; u++) cp[u] = j0 + 4 * q + u < e.lstm_H ? e.lstm_c_prev[idx + u] : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int c = 4 * (4 * q + u);
                    const float zi = __uint_as_float(v[c]), zf = __uint_as_float(v[c + 1]);
                    const float zg = __uint_as_float(v[c + 2]), zo = __uint_as_float(v[c + 3]);
                    const float2 ch = F64_CELL ? lstm_cell_unit(zi, zf, zg, zo, cp[u]) : lstm_cell_unit_f32(zi, zf, zg, zo, cp[u]);
                    cn[u] = ch.x; hn[u] = ch.y;
                }
                if (e.lstm_vec) {
                    *reinterpret_cast<float4 *>(e.lstm_c + idx) = make_float4(cn[0], cn[1], cn[2], cn[3]);
                    *reinterpret_cast<float4 *>(e.lstm_h + idx) = make_float4(hn[0], hn[1], hn[2], hn[3]);
                    if (e.lstm_h_round)
                        *reinterpret_cast<float4 *>(e.lstm_h_round + idx) =
                            make_float4(round_tf32(hn[0]), round_tf32(hn[1]), round_tf32(hn[2]), round_tf32(hn[3]));
                } else {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        if (j0 + 4 * q + u < e.lstm_H) {
                            e.lstm_c[idx + u] = cn[u];
                            e.lstm_h[idx + u] = hn[u];
                            if (e.lstm_h_round) e.lstm_h_round[idx + u] = round_tf32(hn[u]);
                        }
                    }
                }
            }
        }
        return;
    }
    if (!e.addend_post) activate();
    if (e.round_out) {
        // (cvt.rna.tf32.f32 runs at 32 per cycle per SM; (bits + 0x1000) & 0xFFFFE000 gives the same bits for every
        // input that is not a NaN, but sending half of the values through the integer pipe instead measured no faster)
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = __float_as_uint(round_tf32(__uint_as_float(v[j])));
    }
    if (e.pool || e.tma_store) {
        // the group's previous store must have finished reading the staging buffer
        if (store_thread) {
            if (stores_in_flight) tma_store_wait_read<1>();
            else tma_store_wait_read<0>();
        }
        epilogue_bar_sync(bar_id);
        if (rw.srow >= 0) {
#pragma unroll
        for (int j = 0; j < 8; j++)     // 16-byte chunk j of row r lives at chunk j ^ (r % 8)
            slab[rw.srow * 8 + (j ^ (rw.srow & 7))] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                     __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
        }
        staged();
        if (!e.pool) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            epilogue_bar_sync(bar_id);
            if (store_thread) {
                tma_store_4d(tm_y, slab, col0, bx.ow0, bx.oh0, bx.n0);
                tma_store_commit();
            }
        } else {
            // conv + 2x2/2 max-pool (pooling_layer.cc:117-146): each thread reduces two 16-byte
            // chunks of one pooled pixel from the full-resolution slab, then the pooled rows
            // overwrite the head of the same buffer and leave by TMA.
            epilogue_bar_sync(bar_id);
            const int pr = t >> 2, hw = bx.bw >> 1, hh = bx.bh >> 1;
            const int pw = pr % hw, ph = (pr / hw) % hh, pn = pr / (hw * hh);
            float4 m[2];
            if (pn < bx.bn) {
                const int r00 = (pn * bx.bh + 2 * ph) * bx.bw + 2 * pw;
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int c = (t & 3) * 2 + e;
                    m[e] = make_float4(-1e8f, -1e8f, -1e8f, -1e8f);     // the reference's identity
#pragma unroll
                    for (int w4 = 0; w4 < 4; w4++) {
                        const int rr = r00 + (w4 >> 1) * bx.bw + (w4 & 1);
                        const float4 x4 = slab[rr * 8 + (c ^ (rr & 7))];
                        m[e].x = x4.x > m[e].x ? x4.x : m[e].x; m[e].y = x4.y > m[e].y ? x4.y : m[e].y;
                        m[e].z = x4.z > m[e].z ? x4.z : m[e].z; m[e].w = x4.w > m[e].w ? x4.w : m[e].w;
                    }
                }
            }
            epilogue_bar_sync(bar_id);      // every source row has been read
            if (pn < bx.bn) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int c = (t & 3) * 2 + e;
                    slab[pr * 8 + (c ^ (pr & 7))] = m[e];
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            epilogue_bar_sync(bar_id);
            if (store_thread) {
                tma_store_4d(tm_yp, slab, col0, bx.ow0 >> 1, bx.oh0 >> 1, bx.n0);
                tma_store_commit();
            }
        }
    } else if (rw.row_ok) {
        float *yrow = e.y + rw.grow * e.ldy + col0;
#pragma unroll
        for (int j = 0; j < 32; j++)
            if (full_cols || col0 + j < e.N) yrow[j] = __uint_as_float(v[j]);
    }
}

}  // namespace tc
}  // namespace nb
