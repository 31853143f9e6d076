// Tensor-core GEMM / implicit-GEMM convolution for sm_100a.
//
//   D[M,N] = A[M,K] * B[N,K]^T   (both operands K-major, fp32 storage, TF32 math,
//                                 fp32 accumulation in tensor memory)
//
// Replaces the reference's per-image im2col + SGEMM pair
// (models/layers/convolutional_layer.cu:47-70, common/utils.cu:34-74) and its
// fully-connected SGEMM (models/layers/connected_layer.cu:21-38) with ONE
// persistent kernel over the whole batch:
//   * rows of A are output pixels (image, oh, ow); the im2col matrix is never
//     materialised -- for every filter tap (kh,kw) and 32-channel slice a TMA
//     box load fetches the shifted NHWC window, out-of-bounds coordinates give
//     the zero padding;
//   * columns of D are filters; B is the weight tensor re-laid out once as
//     [tap][filter][channel];
//   * tcgen05.mma (kind::tf32, M=128, N=BLOCK_N, K=8) accumulates into TMEM,
//     double-buffered so the epilogue of tile i overlaps the main loop of i+1;
//   * the epilogue applies folded batch-norm scale/shift + bias, an optional
//     addend (residual / LSTM input projection), the activation, and optional
//     TF32 rounding for the next contraction, and stores NHWC rows directly.
// A plain row-major matrix is the special case "image of height 1, 1x1 filter".
//
// Warp roles (320 threads; 448 with the extra operand warps):
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (one elected lane)
//   warps 2-9   epilogue, two groups of four (TMEM -> registers -> shared-memory slab -> TMA store)
//   warps 10-13 three-pass mode: split each A tile into hi/lo TF32 terms; gather mode: build the
//               A tile in shared memory from a strided tensor (3-channel input layers)
//
// Every wait is bounded: a wait that runs out sets the CTA's abort flag and the
// device status word, all roles drain, TMEM is freed and the kernel returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstring>

#include "tc_common.cuh"

namespace nb {

using namespace tc;

namespace {

constexpr int GATHER_MAX_K = 384;      // largest k*k*C (rounded up to 32) the gather table in the kernel parameters holds

struct TcParams {
    CUtensorMap tm_a;
    CUtensorMap tm_b;
    CUtensorMap tm_b_lo;
    CUtensorMap tm_y;
    CUtensorMap tm_yp;          // 2x2/2 max-pooled output (pool mode)
    // tiling of the M dimension into (bw x bh x bn) boxes of output pixels
    int bw, bh, bn;
    int tiles_w, tiles_h, tiles_n;
    int OW, OH, NB;
    int ksize_w, stride, pad_w, pad_h;      // filter columns (the tap index is kh*ksize_w + kw) and paddings
    int c_blocks;               // 32-channel slices per tap
    int num_k_blocks;           // ksize*ksize*c_blocks
    int m_tiles, n_tiles;
    // tile order: consecutive tiles share the A tile (n fastest) or, when the weights are what streams from HBM
    // (connected layers wider than L2), the B tile (m fastest), so that the second reader finds it in L2
    int m_fastest;
    int tx_bytes_a;             // bytes one A box load delivers
    // split-K: a tile is (m_tile, n_tile, split); split s runs K blocks [s*kb_per_split, (s+1)*kb_per_split)
    // and stores into slab s of y (batch coordinate n + s*NB): y then holds k_splits partial tensors
    int k_splits, kb_per_split;
    // The tensor core's fp32 accumulator rounds toward zero at every K=8 step (a bias that grows with K).
    // After every kb_per_part K blocks the partial sums are promoted to registers (round-to-nearest adds)
    // and the TMEM accumulator restarts; parts = number of such partial sums per tile (1: no promotion).
    int kb_per_part, parts;
    // Ring stages of `cbs` K blocks (1 or 2).  One TMA request costs its issuing thread a few hundred cycles whatever
    // its size, and a narrow tile's K block is only 180-350 cycles of MMAs, so convolutions with 64-128 input
    // channels fetch two 32-channel slices of a tap per request: the A map then has the slice index as a fifth
    // dimension (tm_a is 5-D, tm_b 4-D), a stage is [A0 | A1 | B0 | B1], `stages` of them fit the ring.
    int cbs, stages;
    // Filter-column stages (col3 = 1): 3x3 stride-1 convolutions with few input channels are bound by the L2 -> shared
    // memory traffic of re-loading the activation tile once per tap.  Here a stage is one filter COLUMN kw of one channel
    // slice: ONE activation box of bh + 2 image rows (a_box_bytes) and the three weight tiles kh = 0..2.  Tap (kh, kw)
    // reads the box from image row kh on: a start address kh * bw * 128 bytes further, which for bw = 16 stays on the
    // 1024-byte repeat of the swizzle pattern.  Three activation loads per slice instead of nine.
    int col3, a_box_bytes, stage_bytes;
    // col3 only: a tile of `halves` (1 or 2) vertically adjacent 16 x 8 boxes.  Both read the same activation box
    // (bh * halves + 2 image rows, the second half 8 image rows further down) and the same three weight tiles, which
    // halves the weight traffic per pixel; each half has its own accumulator columns.
    int halves;
    // Byte offset (from the ring's start) of a second staging buffer per epilogue group, or 0.  A bulk store takes over
    // a thousand cycles to read its 16 KB out of shared memory; where the ring leaves room, a group alternates between
    // two buffers and lets one store read while the next slab is staged.
    int slab2_offset;
    EpiParams e;                // fused epilogue
    // gather mode: warps 6-9 build the A tile in shared memory from a strided activation tensor
    // (channel counts TMA cannot address, e.g. the 3-channel input layer); rows are output pixels
    int gather;
    const float *gx;
    long gsn, gsh, gsw;         // element strides of the gathered tensor
    int gks, gpad, gK;          // filter size, padding, k*k*C: column kk = (kh, kw, c), c fastest
    int gH, gW, gOH, gOW, gstride, gM, ground;
    // per column: {element offset of (c, kh-pad, kw-pad) from the pixel's origin, (kh-pad) & 0xffff | (kw-pad) << 16}
    int2 gtab[GATHER_MAX_K];
    int *status;
};

// The digits (split, n_tile, tw, th, tn) of a CTA's current tile.  Decoding a tile index costs seven integer
// divisions (over a thousand cycles of dependent instructions on a role's critical path), so the index is decoded
// once and then advanced by the digits of the grid stride, with carries.
struct TileIter {
    int split, n_tile, tw, th, tn;      // current tile
    int ds, dn, dw, dh, dt;             // the grid stride

    __device__ __forceinline__ static void decode(const TcParams &p, int tile, int &s, int &n, int &w, int &h, int &t) {
        s = tile % p.k_splits;
        const int mn = tile / p.k_splits;
        const int m_tile = p.m_fastest ? mn % p.m_tiles : mn / p.n_tiles;
        n = p.m_fastest ? mn / p.m_tiles : mn % p.n_tiles;
        w = m_tile % p.tiles_w;
        h = (m_tile / p.tiles_w) % p.tiles_h;
        t = m_tile / (p.tiles_w * p.tiles_h);
    }
    __device__ __forceinline__ TileIter(const TcParams &p, int first, int step) {
        decode(p, first, split, n_tile, tw, th, tn);
        decode(p, step, ds, dn, dw, dh, dt);
    }
    // digit + stride digit + carry < 2 * radix: one conditional subtraction per digit
    __device__ __forceinline__ static int add(int &digit, int inc, int radix) {
        digit += inc;
        const int carry = digit >= radix ? 1 : 0;
        if (carry) digit -= radix;
        return carry;
    }
    __device__ __forceinline__ void next(const TcParams &p) {
        int c = add(split, ds, p.k_splits);
        if (p.m_fastest) {
            c = add(tw, dw + c, p.tiles_w);
            c = add(th, dh + c, p.tiles_h);
            c = add(tn, dt + c, p.tiles_n);
            n_tile += dn + c;
        } else {
            c = add(n_tile, dn + c, p.n_tiles);
            c = add(tw, dw + c, p.tiles_w);
            c = add(th, dh + c, p.tiles_h);
            tn += dt + c;
        }
    }
};

template <int BLOCK_N, bool THREE>
struct Cfg {
    static constexpr int B_STAGE_BYTES = BLOCK_N * BLOCK_K * 4;
    static constexpr int STAGE_BYTES = (A_STAGE_BYTES + B_STAGE_BYTES) * (THREE ? 2 : 1);
    static constexpr int STAGES = (196 * 1024) / STAGE_BYTES < 8 ? (196 * 1024) / STAGE_BYTES : 8;
    static constexpr int TMEM_COLS = 2 * BLOCK_N;
    static constexpr int OUT_STAGE_BYTES = BLOCK_M * 32 * 4;     // one 128 x 32 output slab
    static constexpr int LAYOUT_BYTES = STAGES * STAGE_BYTES + 2 * OUT_STAGE_BYTES + 256 /*barriers*/;
    // all of the 227 KB a CTA may have: what the layout and its alignment leave over holds the epilogue's scale/shift values
    static constexpr int SMEM_BYTES = 227 * 1024;
    static_assert(LAYOUT_BYTES + 1024 <= SMEM_BYTES, "ring, staging buffers and barriers must fit");
};

// ------------------------------------------------------------------- kernel
// GATHER: warps 10-13 build the A tile (compiled apart so that the common variants, which launch ten warps, are not
// held to the register budget of fourteen).
template <int BLOCK_N, bool THREE, bool PROMOTE, bool GATHER>
__global__ void __launch_bounds__((THREE || GATHER) ? 448 : 320, 1)
gemm_tf32_tcgen05_kernel(const __grid_constant__ TcParams p) {
    using C = Cfg<BLOCK_N, THREE>;
    constexpr int STAGES = C::STAGES;                   // barrier slots; the ring uses the first p.stages of them
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // per stage: [A | B | (A_lo | B_lo)], or [A0 | A1 | B0 | B1] with two K blocks per stage
    const int cbs = THREE ? 1 : p.cbs;
    const int stages = p.stages;
    const int stage_bytes = p.stage_bytes;
    const int halves = (THREE || PROMOTE || BLOCK_N > 128) ? 1 : p.halves;
    const int acc_cols = halves * BLOCK_N;              // TMEM columns of one accumulator set
    // 3xTF32 with several partial sums per tile: the two small cross terms (a_lo*b_hi + a_hi*b_lo) accumulate in a set of
    // columns of their own for the whole tile (their magnitude is 2^-11 of the product's, so what the tensor core's
    // truncating accumulation loses on them is nothing), one set per tile parity behind the two product accumulators.
    // Only the hi*hi chain is then promoted, and a K block adds 4 MMAs to it instead of 12: a third of the promotions
    // for the same chain length.
    const bool cross_cols = THREE && p.parts > 1;
    const uint32_t tmem_cols = (uint32_t)(C::TMEM_COLS * (THREE ? 2 : halves));
    uint8_t *out_stage = smem + STAGES * C::STAGE_BYTES;      // 2 x [128 rows][32 floats], 128B-swizzled
    uint64_t *bars = (uint64_t *)(out_stage + 2 * C::OUT_STAGE_BYTES);
    uint64_t *full = bars;                    // TMA -> (splitter or MMA)
    uint64_t *empty = bars + STAGES;          // MMA -> TMA
    uint64_t *split = bars + 2 * STAGES;      // splitter -> MMA (three-pass only)
    uint64_t *acc_full = bars + 3 * STAGES;   // MMA -> epilogue   [2]
    uint64_t *acc_empty = acc_full + 2;       // epilogue -> MMA   [2]
    uint32_t *tmem_slot = (uint32_t *)(acc_empty + 2);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    // per epilogue group: scale [BLOCK_N / 2] then shift [BLOCK_N / 2] of the columns of its slabs, if the alignment of
    // the dynamic shared memory left room behind the barriers (it does when the base is 1024-byte aligned already)
    float *aff_base = (float *)((uint8_t *)bars + 256);
    const bool aff_smem = !THREE && !PROMOTE && p.e.shift != nullptr && p.e.lstm_H == 0 &&
                          smem_raw + C::SMEM_BYTES >= (uint8_t *)(aff_base + 2 * BLOCK_N);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles * p.k_splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], GATHER ? 129 : 1);
            mbar_init(&empty[s], 1);
            mbar_init(&split[s], 128);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 256);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // A pixel box of fewer than 128 rows leaves the tail rows of every A stage unwritten by TMA, and the MMA reads
    // all 128: those rows only feed accumulator rows that are never stored, but they are given a defined value
    // (zero) once, here; no copy touches them afterwards.
    {
        const int box_rows = (GATHER || p.col3) ? BLOCK_M : p.bw * p.bh * p.bn;
        if (box_rows < BLOCK_M) {
            const int tail16 = (BLOCK_M - box_rows) * 8;          // 16-byte chunks per stage tail
            for (int i = threadIdx.x; i < stages * tail16; i += blockDim.x) {      // (two-block stages only take full boxes)
                const int s = i / tail16, c = i - s * tail16;
                reinterpret_cast<float4 *>(smem + s * stage_bytes + box_rows * 128)[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        // One elected lane runs the loop and issues every copy.  (Measured: running the loop and the waits in all 32 lanes
        // with only the copies elected -- uniform control flow -- changes nothing for narrow tiles and costs 256-wide
        // tiles 2 %.)
        const bool leader = elect_one();
        if (leader) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        TileIter ti(p, blockIdx.x, gridDim.x);
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ti.next(p)) {
            const int split = ti.split, n_tile = ti.n_tile, tw = ti.tw, th = ti.th, tn = ti.tn;
            const int w0 = tw * p.bw * p.stride - p.pad_w;
            const int h0 = th * p.bh * halves * p.stride - p.pad_h;
            const int n0 = tn * p.bn;
            const int kb0 = split * p.kb_per_split;
            const int kb_end = min(kb0 + p.kb_per_split, p.num_k_blocks);      // the last split may be shorter
            if (!THREE && p.col3) {
                // two requests per stage: the activation box and the three weight tiles of this filter column
                // (tm_b is 4-D here, {C, N, kw, kh}: a box of one kw and all three kh)
                const uint32_t tx3 = (uint32_t)(p.a_box_bytes + 3 * C::B_STAGE_BYTES);
                for (int cb3 = 0; cb3 < p.c_blocks && ok; cb3++) {       // kw fastest, then the channel slice
                    for (int kw3 = 0; kw3 < p.ksize_w; kw3++) {
                        if (!(ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status))) break;
                        uint8_t *sa = smem + stage * stage_bytes;
                        if (leader) {
                            mbar_expect_tx(&full[stage], tx3);
                            tma_load_4d(sa, &p.tm_a, &full[stage], cb3 * BLOCK_K, w0 + kw3, h0, n0);
                            tma_load_4d(sa + p.a_box_bytes, &p.tm_b, &full[stage], cb3 * BLOCK_K, n_tile * BLOCK_N, kw3, 0);
                        }
                        if (++stage == stages) { stage = 0; phase ^= 1; }
                    }
                }
                continue;
            }
            int tap = 0, cb = 0, kh = 0, kw = 0;
            if (kb0) {
                tap = kb0 / p.c_blocks; cb = kb0 - tap * p.c_blocks;
                kh = tap / p.ksize_w; kw = tap - kh * p.ksize_w;
            }
            const uint32_t tx_bytes = (uint32_t)(((GATHER ? 0 : p.tx_bytes_a) + C::B_STAGE_BYTES * (THREE ? 2 : 1)) * cbs);
            for (int kb = kb0; kb < kb_end; kb += cbs) {
                if (!(ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status))) break;
                uint8_t *sa = smem + stage * stage_bytes;
                uint8_t *sb = sa + A_STAGE_BYTES * cbs;
                if (leader) {
                    mbar_expect_tx(&full[stage], tx_bytes);
                    if (cbs == 2) {
                        tma_load_5d(sa, &p.tm_a, &full[stage], 0, w0 + kw, h0 + kh, n0, cb);
                        tma_load_4d(sb, &p.tm_b, &full[stage], 0, n_tile * BLOCK_N, cb, tap);
                    } else {
                        if (!GATHER) tma_load_4d(sa, &p.tm_a, &full[stage], cb * BLOCK_K, w0 + kw, h0 + kh, n0);
                        tma_load_3d(sb, &p.tm_b, &full[stage], cb * BLOCK_K, n_tile * BLOCK_N, tap);
                        if (THREE)
                            tma_load_3d(sb + C::B_STAGE_BYTES + A_STAGE_BYTES, &p.tm_b_lo, &full[stage], cb * BLOCK_K,
                                        n_tile * BLOCK_N, tap);
                    }
                }
                if ((cb += cbs) == p.c_blocks) {
                    cb = 0; tap++;
                    if (++kw == p.ksize_w) { kw = 0; kh++; }
                }
                if (++stage == stages) { stage = 0; phase ^= 1; }
            }
        }
        // Tail: the MMA warp's last release of every stage (an mbarrier arrive that the tensor core performs
        // when those MMAs retire) must have landed in this CTA's shared memory before the CTA may exit.
        for (int i = 0; i < stages && ok; i++) {
            ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status);
            if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        }
        __syncwarp();
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        // One elected lane.  Its time per MMA is the tensor core's: about 65 cycles for a 128 x 64 x 8 TF32 MMA, 75 for
        // 128 x 128 x 8 and 138 for 128 x 256 x 8 (the issue blocks while the queue is full), so 64-filter tiles run the
        // tensor core at about half rate whatever the pipeline around it does.
        const bool leader = elect_one();
        if (leader) {
        constexpr uint32_t idesc = make_idesc(BLOCK_M, BLOCK_N);
        int stage = 0;
        uint32_t phase = 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        int tile_parity = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            if (!(ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status))) break;
            tc_fence_after();
            uint32_t d_tmem = tmem_base + (uint32_t)(acc * acc_cols);
            int kb_in_part = 0;
            if (!THREE && p.col3) {
                for (int it = 0; it < p.ksize_w * p.c_blocks; it++) {
                    if (!(ok = mbar_wait(&full[stage], phase, abort_flag, p.status))) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * stage_bytes);
                    if (leader) {
#pragma unroll
                        for (int kh3 = 0; kh3 < 3; kh3++) {
                            const uint32_t b_lo = smem_desc_lo(sa + (uint32_t)p.a_box_bytes + kh3 * C::B_STAGE_BYTES);
                            for (int hf = 0; hf < halves; hf++) {       // image row kh3 (+ bh for the second half) of the box
                                const uint32_t a_lo = smem_desc_lo(sa + (uint32_t)((hf * p.bh + kh3) * p.bw * 128));
#pragma unroll
                                for (int k = 0; k < BLOCK_K / UMMA_K; k++)
                                    umma_tf32(d_tmem + (uint32_t)(hf * BLOCK_N), smem_desc(a_lo + 2 * k), smem_desc(b_lo + 2 * k),
                                              idesc, (it | kh3 | k) != 0);
                            }
                        }
                        umma_commit(&empty[stage]);
                    }
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
                if (ok && leader) umma_commit(&acc_full[acc]);
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                continue;
            }
            const int ksplit = p.k_splits > 1 ? tile % p.k_splits : 0;
            const int tile_kb = min(p.kb_per_split, p.num_k_blocks - ksplit * p.kb_per_split);
            const uint32_t x_tmem = tmem_base + (uint32_t)(2 * BLOCK_N + tile_parity * BLOCK_N);    // cross terms of this tile
            tile_parity ^= 1;
            for (int kb = 0; kb < tile_kb; kb += cbs, kb_in_part += cbs) {
                if (kb_in_part == p.kb_per_part) {
                    // hand this partial sum to the epilogue warps and restart in the other accumulator
                    if (leader) umma_commit(&acc_full[acc]);
                    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                    if (!(ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status))) break;
                    tc_fence_after();
                    d_tmem = tmem_base + (uint32_t)(acc * acc_cols);
                    kb_in_part = 0;
                }
                uint64_t *ready = (THREE && !GATHER) ? &split[stage] : &full[stage];
                if (!(ok = mbar_wait(ready, phase, abort_flag, p.status))) break;
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + stage * stage_bytes);
                if (leader) {
                    for (int c = 0; c < cbs; c++) {
                        const uint32_t a_lo = smem_desc_lo(sa + c * A_STAGE_BYTES);
                        const uint32_t b_lo = smem_desc_lo(sa + cbs * A_STAGE_BYTES + c * C::B_STAGE_BYTES);
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; k++) {        // +32 bytes per K step = +2 in the descriptor
                            const uint64_t da = smem_desc(a_lo + 2 * k), db = smem_desc(b_lo + 2 * k);
                            if (THREE) {
                                const uint64_t da_lo = smem_desc(b_lo + (C::B_STAGE_BYTES >> 4) + 2 * k);
                                const uint64_t db_lo = smem_desc(b_lo + ((C::B_STAGE_BYTES + A_STAGE_BYTES) >> 4) + 2 * k);
                                if (cross_cols) {
                                    umma_tf32(x_tmem, da_lo, db, idesc, (kb | k) != 0);
                                    umma_tf32(x_tmem, da, db_lo, idesc, 1);
                                    umma_tf32(d_tmem, da, db, idesc, (kb_in_part | k) != 0);
                                } else {
                                    umma_tf32(d_tmem, da_lo, db, idesc, (kb_in_part | k) != 0);
                                    umma_tf32(d_tmem, da, db_lo, idesc, 1);
                                    umma_tf32(d_tmem, da, db, idesc, 1);
                                }
                            } else {
                                umma_tf32(d_tmem, da, db, idesc, (kb_in_part | c | k) != 0);
                            }
                        }
                    }
                    umma_commit(&empty[stage]);     // frees the stage once these MMAs have read it
                }
                if (++stage == stages) { stage = 0; phase ^= 1; }
            }
            if (ok && leader) umma_commit(&acc_full[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ---------------------------------------------------------- epilogue
        // Two groups of four warps; group g owns the 32-column slabs of parity g, its own staging
        // buffer, named barrier and TMA-store thread, so two slabs are in flight per tile and every
        // scheduler has two epilogue warps to alternate between.
        const int ew = warp - 2;                // 0..7
        const int grp = ew >> 2;
        const int bar_id = 1 + grp;
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int r = q * 32 + lane;            // row inside the tile
        const int t = (ew & 3) * 32 + lane;     // index inside the group
        const int rw = r % p.bw, rh = (r / p.bw) % p.bh, rn = r / (p.bw * p.bh);
        const bool store_thread = t == 0;
        constexpr int CH = BLOCK_N >= 64 ? BLOCK_N / 64 : 1;    // 32-column slabs per group
        float4 *slab0 = reinterpret_cast<float4 *>(out_stage + grp * C::OUT_STAGE_BYTES);
        float4 *slab1 = p.slab2_offset ? reinterpret_cast<float4 *>(smem + p.slab2_offset + grp * C::OUT_STAGE_BYTES) : slab0;
        const int stores_in_flight = p.slab2_offset ? 1 : 0;
        float4 *slab = slab0;
        int aff_tile = -1;
        int epi_tile_parity = 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        TileIter ti(p, blockIdx.x, gridDim.x);
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ti.next(p)) {
            const int split = ti.split, n_tile = ti.n_tile, tw = ti.tw, th = ti.th, tn = ti.tn;
            const int ow = tw * p.bw + rw, oh = th * p.bh * halves + rh, n = tn * p.bn + rn;
            const bool row_ok = (rn < p.bn) && ow < p.OW && oh < p.OH && n < p.NB;
            const long row = ((long)n * p.OH + oh) * p.OW + ow;
            const EpiRow erow{r, row, row_ok, addend_row(p.e, row_ok, row, n, oh, ow)};
            const EpiBox ebox{p.bw, p.bh, p.bn, tw * p.bw, th * p.bh * halves, tn * p.bn + split * p.NB};
            if (aff_smem && n_tile != aff_tile) {
                // this group's scale/shift values for the tile column (its slabs are chunks grp, grp + 2, ...)
                float *ga = aff_base + grp * BLOCK_N;
                epilogue_bar_sync(bar_id);          // the previous column's values are no longer read
                if (t < BLOCK_N / 2) {
                    const int col = n_tile * BLOCK_N + (grp + 2 * (t >> 5)) * 32 + (t & 31);
                    const bool in = col < ((p.e.N + 31) & ~31);     // the vectors are padded to a multiple of 32
                    ga[t] = (in && p.e.scale) ? p.e.scale[col] : 1.0f;
                    ga[BLOCK_N / 2 + t] = in ? p.e.shift[col] : 0.0f;
                }
                epilogue_bar_sync(bar_id);
                aff_tile = n_tile;
            }
            if (erow.arow) {
                // The addend (a residual tensor, the LSTM's input-side projection) comes from DRAM and each slab's
                // 128 bytes of it are needed only once the accumulators are in registers: start this group's lines
                // towards L2 now, while the tile's MMAs still run.
#pragma unroll 1
                for (int chunk = grp; chunk < BLOCK_N / 32; chunk += 2) {
                    const int col0 = n_tile * BLOCK_N + chunk * 32;
                    if (col0 >= p.e.addend_cols) break;
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(erow.arow + col0));
                }
            }
            if (!PROMOTE || p.parts == 1) {
                if (!(ok = epilogue_all(mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status), bar_id))) break;
                tc_fence_after();
                uint32_t v[32];
                bool loaded = false;            // v holds a tcgen05.ld issued while the previous slab was being stored
#pragma unroll 1
                for (int hf = 0; hf < halves; hf++) {
                    // the second half of a two-box tile: the same raster p.bh image rows further down
                    EpiRow hrow = erow;
                    EpiBox hbox = ebox;
                    if (hf) {
                        const int oh2 = oh + p.bh;
                        hrow.row_ok = (rn < p.bn) && ow < p.OW && oh2 < p.OH && n < p.NB;
                        hrow.grow = ((long)n * p.OH + oh2) * p.OW + ow;
                        hrow.arow = addend_row(p.e, hrow.row_ok, hrow.grow, n, oh2, ow);
                        hbox.oh0 += p.bh;
                    }
#pragma unroll 1
                    for (int chunk = grp; chunk < BLOCK_N / 32; chunk += 2) {
                        const int col0 = n_tile * BLOCK_N + chunk * 32;
                        if (col0 >= p.e.N) break;         // uniform across the group
                        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * acc_cols + hf * BLOCK_N + chunk * 32);
                        if (!loaded) tmem_ld_32x32(taddr, v);
                        tmem_ld_wait();
                        loaded = false;
                        // this group's next slab of the tile: the next pair of columns, else the first of the other half
                        uint32_t next = 0;
                        if (PROMOTE) {}         // (those variants have no registers to spare for it)
                        else if (chunk + 2 < BLOCK_N / 32 && col0 + 64 < p.e.N) next = taddr + 64;
                        else if (hf + 1 < halves) next = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * acc_cols + (hf + 1) * BLOCK_N + grp * 32);
                        epilogue_chunk<THREE>(p.e, &p.tm_y, &p.tm_yp, v, col0, hrow, hbox, slab, bar_id, store_thread, t, stores_in_flight,
                                              [&] { if (next) { tmem_ld_32x32(next, v); loaded = true; } },
                                              aff_smem ? aff_base + grp * BLOCK_N + (chunk >> 1) * 32 : nullptr, BLOCK_N / 2);
                        slab = slab == slab0 ? slab1 : slab0;
                    }
                }
                tc_fence_before();
                mbar_arrive(&acc_empty[acc]);
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            } else if constexpr (PROMOTE) {
                // promoted accumulation: this group's slabs of every partial sum are added in registers
                uint32_t sum[CH][32];
                const int tile_kb = min(p.kb_per_split, p.num_k_blocks - split * p.kb_per_split);
                const int parts = (tile_kb + p.kb_per_part - 1) / p.kb_per_part;
                const uint32_t x_cols = (uint32_t)(2 * BLOCK_N + epi_tile_parity * BLOCK_N);
                epi_tile_parity ^= 1;
                for (int part = 0; part < parts && ok; part++) {
                    if (!(ok = epilogue_all(mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status), bar_id))) break;
                    tc_fence_after();
#pragma unroll
                    for (int ci = 0; ci < CH; ci++) {
                        const int chunk = grp + 2 * ci;
                        if (chunk * 32 < BLOCK_N && n_tile * BLOCK_N + chunk * 32 < p.e.N) {
                            uint32_t v[32];
                            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BLOCK_N + chunk * 32), v);
                            tmem_ld_wait();
                            if (part == 0) {
#pragma unroll
                                for (int j = 0; j < 32; j++) sum[ci][j] = v[j];
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    sum[ci][j] = __float_as_uint(__uint_as_float(sum[ci][j]) + __uint_as_float(v[j]));
                            }
                            if (cross_cols && part == parts - 1) {      // the tile's cross terms: complete with its last MMAs
                                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + x_cols + (uint32_t)(chunk * 32), v);
                                tmem_ld_wait();
#pragma unroll
                                for (int j = 0; j < 32; j++)
                                    sum[ci][j] = __float_as_uint(__uint_as_float(sum[ci][j]) + __uint_as_float(v[j]));
                            }
                        }
                    }
                    tc_fence_before();
                    mbar_arrive(&acc_empty[acc]);
                    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                }
                if (!ok) break;
#pragma unroll
                for (int ci = 0; ci < CH; ci++) {
                    const int chunk = grp + 2 * ci;
                    const int col0 = n_tile * BLOCK_N + chunk * 32;
                    if (chunk * 32 < BLOCK_N && col0 < p.e.N)
                        epilogue_chunk<THREE>(p.e, &p.tm_y, &p.tm_yp, sum[ci], col0, erow, ebox, slab0, bar_id, store_thread, t, 0, [] {});
                }
            }
        }
        if (store_thread) tma_store_wait_all();     // staged tiles must have left shared memory
    } else if (GATHER) {
        // ------------------------------------------------- in-kernel patch gather
        // One thread per tile row (output pixel): 32 columns (kh,kw,c) of this K block are read
        // through the cache (neighbouring threads read neighbouring pixels) and written as one
        // 128-byte swizzled row, TF32-rounded (or split into hi/lo for the three-pass kernel).
        const int t = threadIdx.x - 320;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int m_tile = tile / p.k_splits / p.n_tiles;
            const long m = (long)m_tile * BLOCK_M + t;
            const bool valid = m < p.gM;
            int ih0 = 0, iw0 = 0;
            const float *base = p.gx;
            if (valid) {
                const int per = p.gOH * p.gOW;
                const int n = (int)(m / per), rem = (int)(m - (long)n * per);
                const int oh = rem / p.gOW, ow = rem - oh * p.gOW;
                ih0 = oh * p.gstride; iw0 = ow * p.gstride;
                base = p.gx + (long)n * p.gsn + (long)ih0 * p.gsh + (long)iw0 * p.gsw;
            }
            // does every tap of this pixel fall inside the image?  (true for all but border pixels)
            const int ihf = ih0 - p.gpad, iwf = iw0 - p.gpad;
            const bool interior = valid && ihf >= 0 && iwf >= 0 && ihf + p.gks <= p.gH && iwf + p.gks <= p.gW;
            for (int kb = 0; kb < p.kb_per_split; kb++) {        // gather mode never splits K
                if (!(ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status))) break;
                float4 *a_row = reinterpret_cast<float4 *>(smem + stage * C::STAGE_BYTES + t * 128);
                float4 *a_lo_row = reinterpret_cast<float4 *>(smem + stage * C::STAGE_BYTES + A_STAGE_BYTES + C::B_STAGE_BYTES + t * 128);
                const int2 *tab = p.gtab + kb * BLOCK_K;        // kernel-parameter (constant bank) table
                float x[32];
                if (interior) {
#pragma unroll
                    for (int i = 0; i < 32; i++)                // 32 independent loads in flight
                        x[i] = (kb * BLOCK_K + i < p.gK) ? __ldg(base + tab[i].x) : 0.0f;
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int ih = ih0 + (int)(short)(tab[i].y & 0xffff), iw = iw0 + (tab[i].y >> 16);
                        const bool inb = valid && kb * BLOCK_K + i < p.gK && ih >= 0 && ih < p.gH && iw >= 0 && iw < p.gW;
                        x[i] = inb ? __ldg(base + tab[i].x) : 0.0f;
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float v[4], lo[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        if (THREE) {
                            v[e] = round_tf32(x[4 * j + e]);
                            lo[e] = round_tf32(x[4 * j + e] - v[e]);
                        } else {
                            v[e] = p.ground ? round_tf32(x[4 * j + e]) : x[4 * j + e];
                        }
                    }
                    a_row[j ^ (t & 7)] = make_float4(v[0], v[1], v[2], v[3]);
                    if (THREE) a_lo_row[j ^ (t & 7)] = make_float4(lo[0], lo[1], lo[2], lo[3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&full[stage]);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (THREE) {
        // ---------------------------------------------- hi/lo operand splitter
        // hi = RN_tf32(x), lo = RN_tf32(x - hi), the same split the weights get at load: both terms are exact TF32
        // values, so the tensor core's truncation of its operands changes nothing and the split has no bias.
        // Element positions are kept, so the swizzled tile layout written by TMA is preserved.
        const int t = threadIdx.x - 320;        // 0..127
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < p.kb_per_split; kb++) {
                if (!(ok = mbar_wait(&full[stage], phase, abort_flag, p.status))) break;
                float4 *a = reinterpret_cast<float4 *>(smem + stage * C::STAGE_BYTES);
                float4 *a_lo = reinterpret_cast<float4 *>(smem + stage * C::STAGE_BYTES + A_STAGE_BYTES + C::B_STAGE_BYTES);
#pragma unroll
                for (int i = 0; i < A_STAGE_BYTES / 16 / 128; i++) {
                    float4 x = a[i * 128 + t], h, l;
                    h.x = round_tf32(x.x); l.x = round_tf32(x.x - h.x);
                    h.y = round_tf32(x.y); l.y = round_tf32(x.y - h.y);
                    h.z = round_tf32(x.z); l.z = round_tf32(x.z - h.z);
                    h.w = round_tf32(x.w); l.w = round_tf32(x.w - h.w);
                    a[i * 128 + t] = h;
                    a_lo[i * 128 + t] = l;
                }
                // make the generic-proxy writes visible to the tensor core (async proxy)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&split[stage]);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    }

    // ------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give copies and MMAs still in flight time to land before TMEM is released
        for (int i = 0; i < 64; i++) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------- host side
struct Box { int bw, bh, bn; };

// Chooses the (bw x bh x bn) pixel box (<= 128 rows) that wastes the fewest MMA rows.  Among equally full boxes the
// one that spans the fewest images wins (its rows are the longest contiguous runs in memory), then the widest.
// bn_divides: the images of a box must not run past the batch (split-K slabs follow each other in y)
// image_bytes: size of one image of the A tensor -- a box that runs past the batch makes the load unit read that many
// bytes per missing image behind the tensor, so such boxes are only taken while that stays small
Box choose_box(int OW, int OH, int NB, int stride, bool even, bool bn_divides, double image_bytes) {
    Box best{1, 1, 1};
    double best_eff = -1;
    const int max_dim = 256 / std::max(1, stride);     // TMA box extent limit (elements traversed)
    for (int bw = 1; bw <= std::min({OW, 128, max_dim}); bw++) {
        const int rem = 128 / bw;
        for (int bh = 1; bh <= std::min({OH, rem, max_dim}); bh++) {
            int bn = std::min({NB, 128 / (bw * bh), 256});
            if (bn < 1) continue;
            while ((bn_divides || (double)(((NB + bn - 1) / bn) * bn - NB) * image_bytes > 4e6) && NB % bn) bn--;
            if (even && ((bw | bh) & 1)) continue;      // 2x2 pooling windows must not straddle tiles
            auto eff1 = [](int ext, int b) { return (double)ext / ((double)((ext + b - 1) / b) * b); };
            double eff = eff1(OW, bw) * eff1(OH, bh) * eff1(NB, bn) * (double)(bw * bh * bn) / 128.0;
            eff += 1e-6 * bw + 1e-4 / bn;
            if (eff > best_eff) { best_eff = eff; best = Box{bw, bh, bn}; }
        }
    }
    return best;
}

void encode(nb_handle_s *h, CUtensorMap *tm, const void *base, int rank, const cuuint64_t *dims,
            const cuuint64_t *strides_bytes, const cuuint32_t *box, const cuuint32_t *elem_strides) {
    encode_tensor_map(h, tm, base, rank, dims, strides_bytes, box, elem_strides);
}

typedef void (*TcKernel)(const TcParams);

struct Variant { TcKernel kernel; int smem; };

template <int BLOCK_N, bool THREE, bool PROMOTE, bool GATHER>
Variant variant() { return {gemm_tf32_tcgen05_kernel<BLOCK_N, THREE, PROMOTE, GATHER>, Cfg<BLOCK_N, THREE>::SMEM_BYTES}; }

// index: [gather][three][promote][block_n: 0 = 64, 1 = 128, 2 = 256]; absent combinations are null
const Variant VARIANTS[2][2][2][3] = {
    {{{variant<64, false, false, false>(), variant<128, false, false, false>(), variant<256, false, false, false>()},
      {variant<64, false, true, false>(), variant<128, false, true, false>(), {nullptr, 0}}},
     {{{nullptr, 0}, {nullptr, 0}, {nullptr, 0}},
      {variant<64, true, true, false>(), variant<128, true, true, false>(), {nullptr, 0}}}},
    {{{variant<64, false, false, true>(), variant<128, false, false, true>(), {nullptr, 0}},
      {{nullptr, 0}, {nullptr, 0}, {nullptr, 0}}},
     {{{nullptr, 0}, {nullptr, 0}, {nullptr, 0}},
      {variant<64, true, true, true>(), variant<128, true, true, true>(), {nullptr, 0}}}},
};

// One worked-out launch: kernel parameters (tile geometry, tensor maps), kernel variant, grid.
struct TcLaunch : LaunchRecord {
    TcParams p;
    Variant v;
    int grid = 1, threads = 320;
    double flops = 0;
    std::string desc;       // names the launch in error messages
};

inline bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

void gemm_tc_prepare_device() {
    for (auto &g : VARIANTS)
        for (auto &t : g)
            for (auto &pr : t)
                for (auto &v : pr)
                    if (v.kernel) NB_CHECK_CUDA(cudaFuncSetAttribute(v.kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, v.smem));
}

void encode_tensor_map(nb_handle_s *h, CUtensorMap *tm, const void *base, int rank, const cuuint64_t *dims,
                       const cuuint64_t *strides_bytes, const cuuint32_t *box, const cuuint32_t *elem_strides) {
    CUresult r = h->encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void *>(base), dims,
                                 strides_bytes, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw Error(NB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}

std::string gemm_args_key(const GemmArgs &a, char tag, int extra) {
    std::string k;
    k.reserve(320);
    k.push_back(tag);
    key_add(k, extra);
    key_add(k, a.a); key_add(k, a.a_is_conv); key_add(k, a.lda);
    const ConvGeom &g = a.g;
    key_add(k, g.batch); key_add(k, g.C); key_add(k, g.H); key_add(k, g.W); key_add(k, g.OH); key_add(k, g.OW);
    key_add(k, g.ksize); key_add(k, g.stride); key_add(k, g.pad); key_add(k, g.ksize_w); key_add(k, g.pad_w);
    key_add(k, g.sn); key_add(k, g.sc); key_add(k, g.sh); key_add(k, g.sw);
    key_add(k, a.a_gather); key_add(k, a.b); key_add(k, a.b_lo); key_add(k, a.ldb);
    key_add(k, a.M); key_add(k, a.N); key_add(k, a.Kc);
    key_add(k, a.scale); key_add(k, a.shift); key_add(k, a.addend); key_add(k, a.ld_addend); key_add(k, a.addend_after_act);
    key_add(k, a.res_stride); key_add(k, a.res_c); key_add(k, a.res_h); key_add(k, a.res_w);
    key_add(k, a.act); key_add(k, a.round_out_tf32); key_add(k, a.y); key_add(k, a.ldy); key_add(k, a.y_pool);
    key_add(k, a.lstm_H); key_add(k, a.lstm_c_prev); key_add(k, a.lstm_c); key_add(k, a.lstm_h); key_add(k, a.lstm_h_round);
    key_add(k, a.split_k); key_add(k, a.block_n_hint); key_add(k, a.algo_flops);
    return k;
}

bool gemm_tc_supported(const nb_handle_s *h, const GemmArgs &a) {
    if (!h->encode_tiled || h->cc_major != 10) return false;
    if (a.a_gather) return (a.Kc % 32) == 0 && a.Kc <= GATHER_MAX_K && (a.ldb % 4) == 0 && aligned16(a.b);
    if (a.Kc < 32 || (a.Kc % 4) != 0 || (a.ldb % 4) != 0 || !aligned16(a.b) || !aligned16(a.a)) return false;
    if (a.a_is_conv) {
        const ConvGeom &g = a.g;
        // NHWC only: channel stride 1 and every other stride a multiple of 4 elements
        if (g.sc != 1 || (g.sw % 4) || (g.sh % 4) || (g.sn % 4)) return false;
        if (g.stride > 8) return false;
    } else {
        if ((a.lda % 4) != 0) return false;
    }
    return true;
}

namespace {

// Works out one launch: tiling, kernel variant, tensor maps; checks that every operand's extent lies inside the
// device allocation its pointer belongs to.
std::unique_ptr<TcLaunch> build_launch(nb_handle_s *h, const GemmArgs &a, bool three_pass) {
    if (!gemm_tc_supported(h, a)) throw Error(NB_ERR_UNSUPPORTED, "operands do not satisfy the TMA layout rules");
    if (a.y_pool && a.a_gather) throw Error(NB_ERR_UNSUPPORTED, "fused pooling is not available with the gathered A operand");
    if (three_pass && !a.b_lo) throw Error(NB_ERR_INVALID_ARG, "three-pass GEMM needs the low-order weight split");
    std::unique_ptr<TcLaunch> L(new TcLaunch());
    TcParams &p = L->p;
    std::memset(&p, 0, sizeof p);

    ConvGeom g;
    const bool gather = a.a_gather;
    if (a.a_is_conv && !gather) {
        g = a.g;
    } else {
        // plain matrix = one image of height 1 and width M with Kc channels, 1x1 filter
        g.batch = 1; g.C = a.Kc; g.H = 1; g.W = a.M; g.OH = 1; g.OW = a.M;
        g.ksize = 1; g.stride = 1; g.pad = 0;
        g.sc = 1; g.sw = a.lda; g.sh = (long)a.lda * a.M; g.sn = (long)a.lda * a.M;
    }
    // Split-K: the K blocks (taps x channel slices) are divided among `split_k` tiles that each write their
    // own slab of y ([split][batch][OH][OW][N]); the caller adds the slabs and applies the epilogue.
    const int S = (!gather && a.split_k > 1) ? a.split_k : 1;
    const int kc = a.Kc;
    const int ksize_w = g.ksize_w > 0 ? g.ksize_w : g.ksize;
    const int taps = g.ksize * ksize_w;
    const bool pool = a.y_pool != nullptr;
    Box box = choose_box(g.OW, g.OH, g.batch, g.stride, pool, S > 1, (double)g.sn * 4.0);
    // filter-column stages: 3x3 / stride 1, at most 128 input channels and filters (the layers that are bound by
    // re-loading activations from L2), a fixed 16 x 8 pixel box; not worth it when the box wastes much of the plane
    // (the row-window layout of a layer with <= 4 input channels has the filter columns folded into its "channels":
    // three filter rows, one column, no padding in w)
    const bool col3 = a.a_is_conv && !gather && !three_pass && S == 1 && g.ksize == 3 && g.stride == 1 && g.pad <= 1 &&
                      ((ksize_w == 3 && (g.pad_w < 0 || g.pad_w == g.pad)) || (ksize_w == 1 && g.pad_w == 0)) &&
                      kc <= 128 && a.N <= 128 && g.OW >= 16 && g.OH >= 8 &&
                      ((double)g.OW / ((g.OW + 15) / 16 * 16)) * ((double)g.OH / ((g.OH + 7) / 8 * 8)) >= 0.8;
    if (col3) box = Box{16, 8, 1};
    // two boxes per tile when the plane is tall enough for 16-row tiles not to waste much of it
    const int halves = (col3 && g.OH >= 16 && ((double)g.OW / ((g.OW + 15) / 16 * 16)) * ((double)g.OH / ((g.OH + 15) / 16 * 16)) >= 0.8)
                           ? 2 : 1;
    p.bw = box.bw; p.bh = box.bh; p.bn = box.bn;
    p.tiles_w = (g.OW + box.bw - 1) / box.bw;
    p.tiles_h = (g.OH + box.bh * halves - 1) / (box.bh * halves);
    p.tiles_n = (g.batch + box.bn - 1) / box.bn;
    p.OW = g.OW; p.OH = g.OH; p.NB = g.batch;
    p.ksize_w = ksize_w; p.stride = g.stride; p.pad_h = g.pad; p.pad_w = g.pad_w >= 0 ? g.pad_w : g.pad;
    p.c_blocks = (kc + BLOCK_K - 1) / BLOCK_K;
    p.num_k_blocks = taps * p.c_blocks;
    p.kb_per_split = (p.num_k_blocks + S - 1) / S;
    if (S > 1 && ((long)(S - 1) * p.kb_per_split >= p.num_k_blocks || a.y_pool || a.addend || three_pass || a.scale || a.shift || a.act != NB_ACT_LINEAR))
        throw Error(NB_ERR_INVALID_ARG, "split-K needs non-empty splits of ceil(K blocks / splits) blocks and a plain epilogue");
    p.k_splits = S;
    p.m_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
    p.e.N = a.N;
    p.tx_bytes_a = BLOCK_K * 4 * box.bw * box.bh * box.bn;
    p.e.scale = a.scale; p.e.shift = a.shift; p.e.addend = a.addend; p.e.ld_addend = a.ld_addend;
    p.e.act = a.act; p.e.round_out = a.round_out_tf32 ? 1 : 0;
    p.e.addend_vec = a.addend && aligned16(a.addend) && (a.ld_addend % 4) == 0;
    p.e.addend_cols = a.addend ? (a.res_stride > 0 ? a.res_c : a.N) : 0;
    p.e.res_stride = a.addend ? a.res_stride : 0; p.e.res_h = a.res_h; p.e.res_w = a.res_w;
    p.e.addend_post = (a.addend && a.addend_after_act) ? 1 : 0;
    if (a.lstm_H > 0 && a.act != NB_ACT_LINEAR && !p.e.addend_post)
        throw Error(NB_ERR_INVALID_ARG, "LSTM epilogue: a non-linear gate activation needs the addend added after it");
    p.e.y = a.y; p.e.ldy = a.ldy;
    p.e.tma_store = a.y && aligned16(a.y) && (a.ldy % 4) == 0;
    if (S > 1 && !p.e.tma_store) throw Error(NB_ERR_INVALID_ARG, "split-K needs a 16-byte aligned output with ldy % 4 == 0");
    p.e.pool = pool ? 1 : 0;
    if (pool) {
        if (!a.a_is_conv || (g.OW & 1) || (g.OH & 1) || (a.N % 4) || !aligned16(a.y_pool) || a.addend)
            throw Error(NB_ERR_UNSUPPORTED, "fused 2x2 pooling needs even output extents and a 16-byte aligned NHWC tensor");
        p.e.tma_store = 0;
    } else if (a.lstm_H > 0) {
        if (a.a_is_conv || S > 1 || a.N != 4 * a.lstm_H || !a.lstm_c || !a.lstm_h)
            throw Error(NB_ERR_INVALID_ARG, "LSTM epilogue needs a plain [M,4H] product and c/h outputs");
        p.e.tma_store = 0;
        p.e.lstm_H = a.lstm_H; p.e.lstm_c_prev = a.lstm_c_prev; p.e.lstm_c = a.lstm_c; p.e.lstm_h = a.lstm_h;
        p.e.lstm_h_round = a.lstm_h_round;
        p.e.lstm_f32 = three_pass ? 0 : 1;
        p.e.lstm_vec = (a.lstm_H % 8) == 0 && aligned16(a.lstm_c) && aligned16(a.lstm_h) &&
                       (!a.lstm_c_prev || aligned16(a.lstm_c_prev)) && (!a.lstm_h_round || aligned16(a.lstm_h_round));
    } else if (!a.y) {
        throw Error(NB_ERR_INVALID_ARG, "GEMM without an output tensor");
    }
    p.status = h->d_status;

    // tile width in filters: widest tile that still gives every SM work
    // Promoted accumulation: always for 3xTF32 (its point is fp32-level agreement); in TF32 mode only for
    // very long contractions, where the accumulator's round-toward-zero bias (~K * 7.5e-9) nears TF32's own error.
    const bool promote = three_pass || (long)p.kb_per_split * BLOCK_K >= 8192;   // per split when K is split
    int block_n = 256;
    if (three_pass || gather || promote) block_n = 128;
    if (a.block_n_hint) block_n = std::min(block_n, a.block_n_hint);
    if (!a.block_n_hint) {
        // Cost of a K block of a 128 x bn tile: its MMAs (128 / 64 / 48 cycles per K = 8 step at bn = 256 / 128 / 64) or
        // the operand bytes it needs at the ~71 B/cycle/SM that L2 delivers to 148 SMs loading at once, whichever is
        // larger; times the number of waves of tiles.  Wider tiles move fewer bytes per FLOP, so a single wave of
        // 256-wide tiles on two thirds of the SMs beats two waves of 128-wide ones (conv5_x at 32 images per GPU).
        const int widest = block_n;
        long best_cost = 0;
        for (int bn = widest; bn >= 64; bn /= 2) {
            if (bn > 64 && a.N <= bn / 2) continue;         // more than half of the tile would be padding
            const long tiles = (long)p.m_tiles * S * ((a.N + bn - 1) / bn);
            const long waves = (tiles + h->sm_count - 1) / h->sm_count;
            const long mma = bn == 256 ? 512 : (bn == 128 ? 256 : 192);
            const long supply = (long)(BLOCK_M + bn) * BLOCK_K * 4 / 71;
            const long cost = waves * std::max(mma, supply);
            if (best_cost == 0 || cost < best_cost) { best_cost = cost; block_n = bn; }
        }
    }
    p.n_tiles = (a.N + block_n - 1) / block_n;
    p.m_fastest = (!a.a_is_conv && !gather && (size_t)a.N * a.Kc * 4 > ((size_t)48 << 20)) ? 1 : 0;
    // accumulation chains of at most 512 K elements (TF32) / 12 MMAs (3xTF32) in the tensor core: every accumulating MMA
    // truncates the running sum (a shrink of about 6e-8 per step that adds up layer after layer).  A 3xTF32 K block is
    // 12 MMAs, of which only the 4 hi*hi ones go into the promoted chain (the cross terms have columns of their own)
    p.kb_per_part = !promote ? p.kb_per_split : (three_pass ? 3 : 16);
    p.parts = (p.kb_per_split + p.kb_per_part - 1) / p.kb_per_part;

    // two K blocks per ring stage: narrow tiles (<= 128 filters) of a convolution whose channel slices pair up, a
    // full 128-row pixel box (the second slice's tile must start on a swizzle-pattern boundary), one K split
    p.col3 = (col3 && !promote && block_n <= 128) ? 1 : 0;
    p.halves = p.col3 ? halves : 1;
    if (halves == 2 && !p.col3) throw Error(NB_ERR_UNSUPPORTED, "two-box tiles need the filter-column mode");
    p.cbs = (!p.col3 && !three_pass && !gather && !promote && S == 1 && a.a_is_conv && block_n <= 128 &&
             (kc % (2 * BLOCK_K)) == 0 && box.bw * box.bh * box.bn == BLOCK_M) ? 2 : 1;
    {
        const int b_stage = block_n * BLOCK_K * 4;
        const int stage1 = (A_STAGE_BYTES + b_stage) * (three_pass ? 2 : 1);
        const int ring = std::min(8, (196 * 1024) / stage1) * stage1;       // bytes the variant's ring holds
        p.a_box_bytes = BLOCK_K * 4 * box.bw * (box.bh * halves + 2);
        p.stage_bytes = p.col3 ? p.a_box_bytes + 3 * b_stage : stage1 * p.cbs;
        p.stages = std::min(8, ring / p.stage_bytes);
        // a second staging buffer per epilogue group in what the ring leaves unused; a one-column filter (row windows:
        // one stage per tile, bound by its epilogue) gives up its third stage for it
        if (p.col3 && ksize_w == 1 && p.stages > 2) p.stages = 2;
        const int ring_cap = std::min(8, (196 * 1024) / stage1) * stage1;
        const int used = p.stages * p.stage_bytes;
        p.slab2_offset = (!three_pass && !promote && !gather && ring_cap - used >= 2 * BLOCK_M * 32 * 4) ? used : 0;
    }
    p.gather = gather ? 1 : 0;
    if (gather) {
        p.gx = a.a;
        p.gsn = a.g.sn; p.gsh = a.g.sh; p.gsw = a.g.sw;
        p.gks = a.g.ksize; p.gpad = a.g.pad; p.gK = a.g.C * a.g.ksize * a.g.ksize;
        for (int kk = 0; kk < a.Kc; kk++) {
            int off = 0, dh = 30000, dw = 0;        // padding columns: a row offset that is never inside an image
            if (kk < p.gK) {
                const int tap = kk / a.g.C, c = kk - tap * a.g.C;
                dh = tap / a.g.ksize - a.g.pad; dw = tap % a.g.ksize - a.g.pad;
                off = (int)(c * a.g.sc + dh * a.g.sh + dw * a.g.sw);
            }
            p.gtab[kk] = make_int2(off, (dh & 0xffff) | (dw << 16));
        }
        p.gH = a.g.H; p.gW = a.g.W; p.gOH = a.g.OH; p.gOW = a.g.OW; p.gstride = a.g.stride; p.gM = a.M;
        p.ground = three_pass ? 0 : 1;
    }

    // ---- every operand must lie inside the allocation its pointer belongs to.  For the operands TMA loads, that
    // includes what the boxes at out-of-bounds coordinates cover: such elements arrive as zeros, but the load unit
    // still reads the addresses they map to (rows above the first image, past the last one, past the last filter).
    const long long F4 = 4;
    const long long n32 = ((long long)a.N + 31) / 32 * 32;
    const long long cmax = (long long)p.c_blocks * BLOCK_K - 1;
    if (gather) {
        const long long last = (long long)(a.g.batch - 1) * a.g.sn + (long long)(a.g.H - 1) * a.g.sh +
                               (long long)(a.g.W - 1) * a.g.sw + (long long)(a.g.C - 1) * a.g.sc;
        check_extent(h, a.a, 0, (last + 1) * F4, "gathered input tensor");
    } else {
        const long long wmin = -(long long)p.pad_w, hmin = -(long long)p.pad_h;
        const long long wmax = (long long)(p.tiles_w - 1) * box.bw * g.stride + wmin + (ksize_w - 1) + (long long)box.bw * g.stride - 1;
        const long long bh_tile = (long long)box.bh * halves;
        const long long hmax = (long long)(p.tiles_h - 1) * bh_tile * g.stride + hmin + (g.ksize - 1) + bh_tile * g.stride - 1;
        const long long nmax = (long long)p.tiles_n * box.bn - 1;
        const long long lo = std::min(wmin, 0LL) * g.sw + std::min(hmin, 0LL) * g.sh;
        const long long hi = wmax * g.sw + hmax * g.sh + nmax * g.sn + cmax + 1;
        check_extent(h, a.a, lo * F4, hi * F4, "A operand (with the out-of-bounds elements its boxes cover)");
    }
    {
        const long long rows = (long long)(taps - 1) * a.N + (long long)p.n_tiles * block_n;
        const long long b_floats = (rows - 1) * a.ldb + cmax + 1;
        check_extent(h, a.b, 0, b_floats * F4, "B operand (with the rows past the last filter its boxes cover)");
        if (three_pass) check_extent(h, a.b_lo, 0, b_floats * F4, "low-order B operand");
    }
    if (a.scale) check_extent(h, a.scale, 0, n32 * F4, "epilogue scale vector (padded to 32 columns)");
    if (a.shift) check_extent(h, a.shift, 0, n32 * F4, "epilogue shift vector (padded to 32 columns)");
    if (a.addend) {
        const long long fl = a.res_stride > 0
            ? ((long long)g.batch * a.res_h * a.res_w - 1) * a.ld_addend + a.res_c
            : ((long long)a.M - 1) * a.ld_addend + a.N;
        check_extent(h, a.addend, 0, fl * F4, "addend");
    }
    if (a.y && !pool && !a.lstm_H)
        check_extent(h, a.y, 0, (((long long)S * a.M - 1) * a.ldy + a.N) * F4, "output");
    if (pool) check_extent(h, a.y_pool, 0, (long long)g.batch * (g.OH / 2) * (g.OW / 2) * a.N * F4, "pooled output");
    if (a.lstm_H > 0) {
        const long long fl = (long long)a.M * a.lstm_H * F4;
        if (a.lstm_c_prev) check_extent(h, a.lstm_c_prev, 0, fl, "previous cell state");
        check_extent(h, a.lstm_c, 0, fl, "cell state");
        check_extent(h, a.lstm_h, 0, fl, "hidden state");
        if (a.lstm_h_round) check_extent(h, a.lstm_h_round, 0, fl, "rounded hidden state");
    }

    if (p.cbs == 2) {   // A: dims {32, W, H, N, C/32}; B: dims {32, N, C/32, taps}: the channel slice is a dimension of its own
        cuuint64_t dims[5] = {(cuuint64_t)BLOCK_K, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.batch, (cuuint64_t)p.c_blocks};
        cuuint64_t strides[4] = {(cuuint64_t)g.sw * 4, (cuuint64_t)g.sh * 4, (cuuint64_t)g.sn * 4, (cuuint64_t)BLOCK_K * 4};
        cuuint32_t bx[5] = {(cuuint32_t)BLOCK_K, (cuuint32_t)(box.bw * g.stride), (cuuint32_t)(box.bh * g.stride),
                            (cuuint32_t)box.bn, 2};
        cuuint32_t es[5] = {1, (cuuint32_t)g.stride, (cuuint32_t)g.stride, 1, 1};
        encode(h, &p.tm_a, a.a, 5, dims, strides, bx, es);
        cuuint64_t bdims[4] = {(cuuint64_t)BLOCK_K, (cuuint64_t)a.N, (cuuint64_t)p.c_blocks, (cuuint64_t)taps};
        cuuint64_t bstrides[3] = {(cuuint64_t)a.ldb * 4, (cuuint64_t)BLOCK_K * 4, (cuuint64_t)a.ldb * 4 * (cuuint64_t)a.N};
        cuuint32_t bbx[4] = {(cuuint32_t)BLOCK_K, (cuuint32_t)block_n, 2, 1};
        cuuint32_t bes[4] = {1, 1, 1, 1};
        encode(h, &p.tm_b, a.b, 4, bdims, bstrides, bbx, bes);
    }
    if (!gather && p.cbs == 1) {   // A: dims {C, W, H, N}
        cuuint64_t dims[4] = {(cuuint64_t)kc, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.batch};
        cuuint64_t strides[3] = {(cuuint64_t)g.sw * 4, (cuuint64_t)g.sh * 4, (cuuint64_t)g.sn * 4};
        cuuint32_t bx[4] = {(cuuint32_t)BLOCK_K, (cuuint32_t)(box.bw * g.stride),
                            (cuuint32_t)(p.col3 ? box.bh * halves + 2 : box.bh * g.stride), (cuuint32_t)box.bn};
        cuuint32_t es[4] = {1, (cuuint32_t)g.stride, (cuuint32_t)g.stride, 1};
        encode(h, &p.tm_a, a.a, 4, dims, strides, bx, es);
    }
    if (p.col3) {       // B: dims {Kc, N, kw, kh}; a box is one filter column: kw fixed, kh = 0..2
        cuuint64_t dims[4] = {(cuuint64_t)kc, (cuuint64_t)a.N, (cuuint64_t)ksize_w, 3};
        cuuint64_t strides[3] = {(cuuint64_t)a.ldb * 4, (cuuint64_t)a.ldb * 4 * (cuuint64_t)a.N,
                                 (cuuint64_t)a.ldb * 4 * (cuuint64_t)a.N * (cuuint64_t)ksize_w};
        cuuint32_t bx[4] = {(cuuint32_t)BLOCK_K, (cuuint32_t)block_n, 1, 3};
        cuuint32_t es[4] = {1, 1, 1, 1};
        encode(h, &p.tm_b, a.b, 4, dims, strides, bx, es);
    } else if (p.cbs == 1) {   // B: dims {Kc, N, taps}
        cuuint64_t dims[3] = {(cuuint64_t)kc, (cuuint64_t)a.N, (cuuint64_t)taps};
        cuuint64_t strides[2] = {(cuuint64_t)a.ldb * 4, (cuuint64_t)a.ldb * 4 * (cuuint64_t)a.N};
        cuuint32_t bx[3] = {(cuuint32_t)BLOCK_K, (cuuint32_t)block_n, 1};
        cuuint32_t es[3] = {1, 1, 1};
        encode(h, &p.tm_b, a.b, 3, dims, strides, bx, es);
        if (three_pass) encode(h, &p.tm_b_lo, a.b_lo, 3, dims, strides, bx, es);
    }

    if (p.e.tma_store) {   // Y: dims {N, OW, OH, NB}; the same pixel box as A, 32 columns wide
        cuuint64_t dims[4] = {(cuuint64_t)a.N, (cuuint64_t)g.OW, (cuuint64_t)g.OH, (cuuint64_t)g.batch * (cuuint64_t)S};
        cuuint64_t strides[3] = {(cuuint64_t)a.ldy * 4, (cuuint64_t)a.ldy * 4 * (cuuint64_t)g.OW,
                                 (cuuint64_t)a.ldy * 4 * (cuuint64_t)g.OW * (cuuint64_t)g.OH};
        cuuint32_t bx[4] = {32, (cuuint32_t)box.bw, (cuuint32_t)box.bh, (cuuint32_t)box.bn};
        cuuint32_t es[4] = {1, 1, 1, 1};
        encode(h, &p.tm_y, a.y, 4, dims, strides, bx, es);
    }

    if (pool) {          // pooled Y: dims {N, OW/2, OH/2, NB}
        cuuint64_t dims[4] = {(cuuint64_t)a.N, (cuuint64_t)(g.OW / 2), (cuuint64_t)(g.OH / 2), (cuuint64_t)g.batch};
        cuuint64_t strides[3] = {(cuuint64_t)a.N * 4, (cuuint64_t)a.N * 4 * (cuuint64_t)(g.OW / 2),
                                 (cuuint64_t)a.N * 4 * (cuuint64_t)(g.OW / 2) * (cuuint64_t)(g.OH / 2)};
        cuuint32_t bx[4] = {32, (cuuint32_t)(box.bw / 2), (cuuint32_t)(box.bh / 2), (cuuint32_t)box.bn};
        cuuint32_t es[4] = {1, 1, 1, 1};
        encode(h, &p.tm_yp, a.y_pool, 4, dims, strides, bx, es);
    }

    L->v = VARIANTS[gather ? 1 : 0][three_pass ? 1 : 0][promote ? 1 : 0][block_n == 256 ? 2 : (block_n == 128 ? 1 : 0)];
    if (!L->v.kernel) throw Error(NB_ERR_UNSUPPORTED, "no tensor-core kernel variant for this tile width");
    const int tiles = p.m_tiles * p.n_tiles * p.k_splits;
    L->grid = std::max(1, std::min(tiles, h->sm_count));
    L->threads = (three_pass || gather) ? 448 : 320;
    L->flops = a.algo_flops > 0 ? a.algo_flops : 2.0 * (double)a.M * a.N * a.Kc * taps;
    L->desc = " [M=" + std::to_string(a.M) + " N=" + std::to_string(a.N) + " K=" + std::to_string(a.Kc) + " taps=" +
              std::to_string(taps) + " stride=" + std::to_string(g.stride) + " out=" + std::to_string(g.OW) + "x" +
              std::to_string(g.OH) + "x" + std::to_string(g.batch) + " box=" + std::to_string(box.bw) + "x" +
              std::to_string(box.bh) + "x" + std::to_string(box.bn) + " block_n=" + std::to_string(block_n) +
              " splits=" + std::to_string(S) + (p.col3 ? (p.halves == 2 ? " col3x2" : " col3") : "") + (p.cbs == 2 ? " cbs2" : "") + (gather ? " gather" : "") +
              (three_pass ? " 3xtf32" : "") +
              (pool ? " pool" : "") + (a.addend ? " addend" : "") + (a.lstm_H ? " lstm" : "") + "]";
    return L;
}

}  // namespace

void gemm_tc(nb_handle_s *h, const GemmArgs &a, bool three_pass) {
    std::string key = gemm_args_key(a, 'G', three_pass ? 1 : 0);
    auto it = h->launch_cache.find(key);
    if (it == h->launch_cache.end()) {
        if (h->launch_cache.size() > 4096) h->launch_cache.clear();
        it = h->launch_cache.emplace(std::move(key), build_launch(h, a, three_pass)).first;
    }
    const TcLaunch &L = static_cast<const TcLaunch &>(*it->second);
    ProfileScope prof(h, 0, L.flops);
    L.v.kernel<<<L.grid, L.threads, L.v.smem, h->stream>>>(L.p);
    try {
        check_launch("gemm_tf32_tcgen05_kernel");
    } catch (const Error &err) {
        throw Error(err.code, std::string(err.what()) + L.desc);    // an asynchronous fault is otherwise hard to place
    }
    count_launch(h);
    if (h->trace_host && !h->trace_names.empty()) h->trace_names.back() += L.desc;
    prof.finish();
}

}  // namespace nb
