// 3x3 stride-1 convolution for layers with few input channels (C <= 128), where the
// generic implicit-GEMM kernel is bound by L2 -> shared-memory traffic: it re-loads
// the activation tile once per filter tap (9x the input bytes).
//
// Here every 32-channel slice of the input is loaded ONCE per tile as a halo box
// {32 ch, bw+2, bh+2} and all nine taps read it in place: tap (kh,kw) is the same
// shared-memory tile with the operand descriptor's start address advanced by
// (kh*(bw+2) + kw) rows of 128 bytes (the 128-byte swizzle is a function of the
// shared-memory address, so a row-shifted start stays consistent with what TMA
// wrote).  The accumulator rows therefore run over a (bw+2)-wide raster: two
// columns per image row are junk and are dropped by the epilogue when it compacts
// rows into the staging slab.  A tile is 1 or 2 such 128-row halves (two MMAs per
// K step share one weight tile, halving the weight traffic per pixel); weights are
// streamed per tap through their own ring.
//
// Replaces the same reference code as the generic kernel
// (models/layers/convolutional_layer.cu:47-70, common/utils.cu:34-74) for these
// layers; same fused epilogue (batch-norm/bias/activation/TF32 rounding, optional
// 2x2/2 max-pool).  Warp roles: 0 TMA producer, 1 MMA issuer, 2-9 epilogue.
// Every wait is bounded, as in the generic kernel.
#include <algorithm>
#include <cstring>

#include "tc_common.cuh"

namespace nb {

using namespace tc;

namespace {

constexpr int A_RING = 3;
constexpr int A_BYTES = 37 * 1024;          // up to 296 rows of 128 B: halo box + slack for the last tap's overrun
constexpr int OUT_BYTES = BLOCK_M * 32 * 4;

struct HaloParams {
    CUtensorMap tm_a, tm_b, tm_y, tm_yp;
    int bw, bh, wt;             // valid tile width/height in pixels, raster width wt = bw + 2
    int halves;                 // 128-row accumulator halves per tile (1 or 2)
    int rows_half;              // image rows per half (128 / wt when halves == 2, else bh)
    int tiles_w, tiles_h, NB, OW, OH;
    int pad;
    int c_blocks;
    int m_tiles, n_tiles;
    int halo_bytes;
    EpiParams e;
    int *status;
};

template <int BLOCK_N>
struct HCfg {
    static constexpr int B_BYTES = BLOCK_N * BLOCK_K * 4;
    static constexpr int B_RING = 64 * 1024 / B_BYTES;                // 8 (N=64) or 4 (N=128)
    static constexpr int SMEM_BYTES = A_RING * A_BYTES + B_RING * B_BYTES + 2 * OUT_BYTES + 1024 + 256;
};

template <int BLOCK_N>
__global__ void __launch_bounds__(320, 1) conv3x3_halo_tcgen05_kernel(const __grid_constant__ HaloParams p) {
    using C = HCfg<BLOCK_N>;
    constexpr int B_RING = C::B_RING;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *a_ring = smem;
    uint8_t *b_ring = a_ring + A_RING * A_BYTES;
    uint8_t *out_stage = b_ring + B_RING * C::B_BYTES;
    uint64_t *bars = (uint64_t *)(out_stage + 2 * OUT_BYTES);
    uint64_t *a_full = bars, *a_empty = a_full + A_RING;
    uint64_t *b_full = a_empty + A_RING, *b_empty = b_full + B_RING;
    uint64_t *acc_full = b_empty + B_RING, *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = (uint32_t *)(acc_empty + 2);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int acc_cols = p.halves * BLOCK_N;            // TMEM columns of one accumulator set
    // power of two >= 2 * acc_cols
    const uint32_t tmem_cols = (2 * acc_cols <= 128) ? 128 : (2 * acc_cols <= 256 ? 256 : 512);

    if (threadIdx.x == 0) {
        for (int s = 0; s < A_RING; s++) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
        for (int s = 0; s < B_RING; s++) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        for (int a = 0; a < 2; a++) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 256); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // The last tap of a half reads up to two rows past the halo box (raster rows wt*(bh+2) and +1): they only feed
    // junk accumulator rows, but they get a defined value (zero) once, here; no copy touches them afterwards.
    {
        const int box_rows = p.wt * (p.bh + 2);
        constexpr int TAIL16 = 8 * 8;                   // eight rows of 128 bytes in 16-byte chunks
        for (int i = threadIdx.x; i < A_RING * TAIL16; i += blockDim.x) {
            const int s = i / TAIL16, c = i - s * TAIL16;
            reinterpret_cast<float4 *>(a_ring + s * A_BYTES + box_rows * 128)[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (elect_one()) {
            int sa = 0, sb = 0;
            uint32_t pa = 0, pb = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m_tile = tile / p.n_tiles, n_tile = tile % p.n_tiles;
                const int tw = m_tile % p.tiles_w;
                const int th = (m_tile / p.tiles_w) % p.tiles_h;
                const int n = m_tile / (p.tiles_w * p.tiles_h);
                for (int cb = 0; cb < p.c_blocks && ok; cb++) {
                    if (!(ok = mbar_wait(&a_empty[sa], pa ^ 1, abort_flag, p.status))) break;
                    mbar_expect_tx(&a_full[sa], (uint32_t)p.halo_bytes);
                    tma_load_4d(a_ring + sa * A_BYTES, &p.tm_a, &a_full[sa], cb * BLOCK_K, tw * p.bw - p.pad,
                                th * p.bh - p.pad, n);
                    if (++sa == A_RING) { sa = 0; pa ^= 1; }
                    for (int tap = 0; tap < 9; tap++) {
                        if (!(ok = mbar_wait(&b_empty[sb], pb ^ 1, abort_flag, p.status))) break;
                        mbar_expect_tx(&b_full[sb], (uint32_t)C::B_BYTES);
                        tma_load_3d(b_ring + sb * C::B_BYTES, &p.tm_b, &b_full[sb], cb * BLOCK_K, n_tile * BLOCK_N, tap);
                        if (++sb == B_RING) { sb = 0; pb ^= 1; }
                    }
                }
            }
            // Tail: the issuers' last releases of every ring slot (mbarrier arrives that the tensor core performs when
            // those MMAs retire) must have landed in this CTA's shared memory before the CTA may exit.
            for (int i = 0; i < A_RING && ok; i++) {
                ok = mbar_wait(&a_empty[sa], pa ^ 1, abort_flag, p.status);
                if (++sa == A_RING) { sa = 0; pa ^= 1; }
            }
            for (int i = 0; i < B_RING && ok; i++) {
                ok = mbar_wait(&b_empty[sb], pb ^ 1, abort_flag, p.status);
                if (++sb == B_RING) { sb = 0; pb ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        // One thread issues the MMAs of both 128-row halves: per tap, the two halves share the weight tile.
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc(BLOCK_M, BLOCK_N);
            int sa = 0, sb = 0, acc = 0;
            uint32_t pa = 0, pb = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!(ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * acc_cols);
                for (int cb = 0; cb < p.c_blocks && ok; cb++) {
                    if (!(ok = mbar_wait(&a_full[sa], pa, abort_flag, p.status))) break;
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(a_ring + sa * A_BYTES);
                    for (int tap = 0; tap < 9; tap++) {
                        if (!(ok = mbar_wait(&b_full[sb], pb, abort_flag, p.status))) break;
                        tc_fence_after();
                        const uint32_t b_lo = smem_desc_lo(smem_u32(b_ring + sb * C::B_BYTES));
                        const int kh = tap / 3, kw = tap - kh * 3;
                        const uint32_t a_lo = smem_desc_lo(a_base + (uint32_t)((kh * p.wt + kw) * 128));
                        for (int hf = 0; hf < p.halves; hf++) {
#pragma unroll
                            for (int k = 0; k < BLOCK_K / UMMA_K; k++)      // +32 bytes per K step = +2 in the descriptor;
                                umma_tf32(d_tmem + (uint32_t)(hf * BLOCK_N),    // the second half starts 128 rows = 16 KiB further on
                                          smem_desc(a_lo + hf * (BLOCK_M * 128 >> 4) + 2 * k), smem_desc(b_lo + 2 * k), idesc,
                                          (cb | tap | k) != 0);
                        }
                        umma_commit(&b_empty[sb]);
                        if (++sb == B_RING) { sb = 0; pb ^= 1; }
                    }
                    if (ok) umma_commit(&a_empty[sa]);
                    if (++sa == A_RING) { sa = 0; pa ^= 1; }
                }
                if (ok) umma_commit(&acc_full[acc]);
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ---------------------------------------------------------- epilogue
        const int ew = warp - 2, grp = ew >> 2, bar_id = 1 + grp;
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const int t = (ew & 3) * 32 + lane;
        const bool store_thread = t == 0;
        float4 *slab = reinterpret_cast<float4 *>(out_stage + grp * OUT_BYTES);
        const int chunks_n = BLOCK_N / 32;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int m_tile = tile / p.n_tiles, n_tile = tile % p.n_tiles;
            const int tw = m_tile % p.tiles_w;
            const int th = (m_tile / p.tiles_w) % p.tiles_h;
            const int n = m_tile / (p.tiles_w * p.tiles_h);
            if (!(ok = epilogue_all(mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status), bar_id))) break;
            tc_fence_after();
#pragma unroll 1
            for (int item = grp; item < p.halves * chunks_n; item += 2) {
                const int hf = item / chunks_n, chunk = item - hf * chunks_n;
                const int col0 = n_tile * BLOCK_N + chunk * 32;
                if (col0 >= p.e.N) continue;        // uniform across the group
                // accumulator row -> raster position -> pixel of this half's box
                const int m = hf * BLOCK_M + r;
                const int jh = m / p.wt, jw = m - jh * p.wt;
                const int lh = jh - hf * p.rows_half;                  // row inside the half's box
                const bool in_box = jw < p.bw && jh < p.bh && lh >= 0 && lh < p.rows_half;
                const int ow = tw * p.bw + jw, oh = th * p.bh + jh;
                EpiRow rw;
                rw.srow = in_box ? lh * p.bw + jw : -1;
                rw.row_ok = in_box && ow < p.OW && oh < p.OH;
                rw.grow = ((long)n * p.OH + oh) * p.OW + ow;
                rw.arow = addend_row(p.e, rw.row_ok, rw.grow, n, oh, ow);
                const EpiBox bx{p.bw, p.rows_half, 1, tw * p.bw, th * p.bh + hf * p.rows_half, n};
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * acc_cols + hf * BLOCK_N + chunk * 32), v);
                tmem_ld_wait();
                epilogue_chunk<false>(p.e, &p.tm_y, &p.tm_yp, v, col0, rw, bx, slab, bar_id, store_thread, t, 0, [] {});
            }
            tc_fence_before();
            mbar_arrive(&acc_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        if (store_thread) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

void encode(nb_handle_s *h, CUtensorMap *tm, const void *base, int rank, const cuuint64_t *dims,
            const cuuint64_t *strides_bytes, const cuuint32_t *box) {
    const cuuint32_t es[5] = {1, 1, 1, 1, 1};
    encode_tensor_map(h, tm, base, rank, dims, strides_bytes, box, es);
}

typedef void (*HaloKernel)(const HaloParams);

struct HaloLaunch : LaunchRecord {
    HaloParams p;
    HaloKernel kernel = nullptr;
    int smem = 0, grid = 1;
    double flops = 0;
    std::string desc;
};

inline bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

void conv_halo_prepare_device() {
    NB_CHECK_CUDA(cudaFuncSetAttribute(conv3x3_halo_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       HCfg<64>::SMEM_BYTES));
    NB_CHECK_CUDA(cudaFuncSetAttribute(conv3x3_halo_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       HCfg<128>::SMEM_BYTES));
}

// Shapes this kernel takes: 3x3, stride 1, NHWC input with 32 <= C <= 128 and C % 4 == 0, TF32 mode,
// output (or pooled output) addressable by TMA.
bool conv_halo_supported(const nb_handle_s *h, const GemmArgs &a) {
    if (!h->encode_tiled || h->cc_major != 10 || !a.a_is_conv || a.a_gather) return false;
    const ConvGeom &g = a.g;
    if (g.ksize != 3 || g.stride != 1 || g.pad > 1 || g.sc != 1) return false;
    if (a.Kc < 32 || a.Kc > 128 || (a.Kc % 4) || (a.ldb % 4) || (a.N % 4)) return false;
    if ((g.sw % 4) || (g.sh % 4) || (g.sn % 4) || !aligned16(a.a) || !aligned16(a.b)) return false;
    if (g.OW < 14 || g.OH < 8) return false;
    if (a.addend && (a.res_stride <= 0 || (a.ld_addend % 4) || !aligned16(a.addend) || a.addend_after_act)) return false;
    if (a.y_pool ? ((g.OW | g.OH) & 1) || !aligned16(a.y_pool) : (!a.y || !aligned16(a.y) || (a.ldy % 4))) return false;
    return true;
}

namespace {

std::unique_ptr<HaloLaunch> build_launch(nb_handle_s *h, const GemmArgs &a) {
    if (!conv_halo_supported(h, a)) throw Error(NB_ERR_UNSUPPORTED, "shape not supported by the 3x3 halo kernel");
    const ConvGeom &g = a.g;
    std::unique_ptr<HaloLaunch> L(new HaloLaunch());
    HaloParams &p = L->p;
    std::memset(&p, 0, sizeof p);
    p.bw = 14; p.wt = 16;
    p.halves = g.OH >= 16 ? 2 : 1;
    p.rows_half = 8;
    p.bh = 8 * p.halves;
    p.tiles_w = (g.OW + p.bw - 1) / p.bw;
    p.tiles_h = (g.OH + p.bh - 1) / p.bh;
    p.NB = g.batch; p.OW = g.OW; p.OH = g.OH;
    p.pad = g.pad;
    p.c_blocks = (a.Kc + BLOCK_K - 1) / BLOCK_K;
    p.m_tiles = p.tiles_w * p.tiles_h * g.batch;
    const int block_n = a.N > 64 ? 128 : 64;
    p.n_tiles = (a.N + block_n - 1) / block_n;
    p.halo_bytes = BLOCK_K * 4 * p.wt * (p.bh + 2);
    p.e.scale = a.scale; p.e.shift = a.shift; p.e.addend = a.addend; p.e.ld_addend = a.ld_addend;
    p.e.addend_vec = a.addend ? 1 : 0; p.e.addend_cols = a.addend ? a.res_c : 0;
    p.e.res_stride = a.addend ? a.res_stride : 0; p.e.res_h = a.res_h; p.e.res_w = a.res_w;
    p.e.act = a.act; p.e.round_out = a.round_out_tf32 ? 1 : 0;
    p.e.y = a.y; p.e.ldy = a.ldy; p.e.tma_store = a.y_pool ? 0 : 1; p.e.pool = a.y_pool ? 1 : 0; p.e.N = a.N;
    p.status = h->d_status;

    // every operand must lie inside the allocation its pointer belongs to
    const long long F4 = 4, n32 = ((long long)a.N + 31) / 32 * 32;
    // (TMA loads read the addresses of out-of-bounds box elements too, although those arrive as zeros)
    {
        const long long cmax = (long long)p.c_blocks * BLOCK_K - 1;
        const long long wmax = (long long)(p.tiles_w - 1) * p.bw - p.pad + p.wt - 1;
        const long long hmax = (long long)(p.tiles_h - 1) * p.bh - p.pad + p.bh + 1;
        const long long lo = -(long long)p.pad * (g.sw + g.sh);
        const long long hi = wmax * g.sw + hmax * g.sh + (long long)(g.batch - 1) * g.sn + cmax + 1;
        check_extent(h, a.a, lo * F4, hi * F4, "A operand (with the out-of-bounds elements its halo boxes cover)");
        const long long rows = 8LL * a.N + (long long)p.n_tiles * block_n;
        check_extent(h, a.b, 0, ((rows - 1) * a.ldb + cmax + 1) * F4, "B operand (with the rows past the last filter its boxes cover)");
    }
    if (a.scale) check_extent(h, a.scale, 0, n32 * F4, "epilogue scale vector (padded to 32 columns)");
    if (a.shift) check_extent(h, a.shift, 0, n32 * F4, "epilogue shift vector (padded to 32 columns)");
    if (a.addend)
        check_extent(h, a.addend, 0, (((long long)g.batch * a.res_h * a.res_w - 1) * a.ld_addend + a.res_c) * F4, "addend");
    if (a.y_pool) check_extent(h, a.y_pool, 0, (long long)g.batch * (g.OH / 2) * (g.OW / 2) * a.N * F4, "pooled output");
    else check_extent(h, a.y, 0, (((long long)g.batch * g.OH * g.OW - 1) * a.ldy + a.N) * F4, "output");

    {   // A halo: dims {C, W, H, N}, box {32, bw+2, bh+2, 1}
        cuuint64_t dims[4] = {(cuuint64_t)a.Kc, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.batch};
        cuuint64_t strides[3] = {(cuuint64_t)g.sw * 4, (cuuint64_t)g.sh * 4, (cuuint64_t)g.sn * 4};
        cuuint32_t bx[4] = {(cuuint32_t)BLOCK_K, (cuuint32_t)p.wt, (cuuint32_t)(p.bh + 2), 1};
        encode(h, &p.tm_a, a.a, 4, dims, strides, bx);
    }
    {   // B: dims {C, N, 9}
        cuuint64_t dims[3] = {(cuuint64_t)a.Kc, (cuuint64_t)a.N, 9};
        cuuint64_t strides[2] = {(cuuint64_t)a.ldb * 4, (cuuint64_t)a.ldb * 4 * (cuuint64_t)a.N};
        cuuint32_t bx[3] = {(cuuint32_t)BLOCK_K, (cuuint32_t)block_n, 1};
        encode(h, &p.tm_b, a.b, 3, dims, strides, bx);
    }
    if (a.y_pool) {
        cuuint64_t dims[4] = {(cuuint64_t)a.N, (cuuint64_t)(g.OW / 2), (cuuint64_t)(g.OH / 2), (cuuint64_t)g.batch};
        cuuint64_t strides[3] = {(cuuint64_t)a.N * 4, (cuuint64_t)a.N * 4 * (cuuint64_t)(g.OW / 2),
                                 (cuuint64_t)a.N * 4 * (cuuint64_t)(g.OW / 2) * (cuuint64_t)(g.OH / 2)};
        cuuint32_t bx[4] = {32, (cuuint32_t)(p.bw / 2), (cuuint32_t)(p.rows_half / 2), 1};
        encode(h, &p.tm_yp, a.y_pool, 4, dims, strides, bx);
    } else {
        cuuint64_t dims[4] = {(cuuint64_t)a.N, (cuuint64_t)g.OW, (cuuint64_t)g.OH, (cuuint64_t)g.batch};
        cuuint64_t strides[3] = {(cuuint64_t)a.ldy * 4, (cuuint64_t)a.ldy * 4 * (cuuint64_t)g.OW,
                                 (cuuint64_t)a.ldy * 4 * (cuuint64_t)g.OW * (cuuint64_t)g.OH};
        cuuint32_t bx[4] = {32, (cuuint32_t)p.bw, (cuuint32_t)p.rows_half, 1};
        encode(h, &p.tm_y, a.y, 4, dims, strides, bx);
    }
    const int tiles = p.m_tiles * p.n_tiles;
    L->grid = std::max(1, std::min(tiles, h->sm_count));
    if (block_n == 128) { L->kernel = conv3x3_halo_tcgen05_kernel<128>; L->smem = HCfg<128>::SMEM_BYTES; }
    else { L->kernel = conv3x3_halo_tcgen05_kernel<64>; L->smem = HCfg<64>::SMEM_BYTES; }
    L->flops = a.algo_flops > 0 ? a.algo_flops : 2.0 * (double)a.M * a.N * a.Kc * 9;
    L->desc = " [3x3 halo C=" + std::to_string(a.Kc) + " N=" + std::to_string(a.N) + " out=" + std::to_string(g.OW) + "x" +
              std::to_string(g.OH) + "x" + std::to_string(g.batch) + " block_n=" + std::to_string(block_n) +
              (a.y_pool ? " pool" : "") + (a.addend ? " addend" : "") + "]";
    return L;
}

}  // namespace

void conv_halo_tc(nb_handle_s *h, const GemmArgs &a) {
    std::string key = gemm_args_key(a, 'H', 0);
    auto it = h->launch_cache.find(key);
    if (it == h->launch_cache.end()) {
        if (h->launch_cache.size() > 4096) h->launch_cache.clear();
        it = h->launch_cache.emplace(std::move(key), build_launch(h, a)).first;
    }
    const HaloLaunch &L = static_cast<const HaloLaunch &>(*it->second);
    ProfileScope prof(h, 2, L.flops);
    L.kernel<<<L.grid, 320, L.smem, h->stream>>>(L.p);
    try {
        check_launch("conv3x3_halo_tcgen05_kernel");
    } catch (const Error &err) {
        throw Error(err.code, std::string(err.what()) + L.desc);
    }
    count_launch(h);
    if (h->trace_host && !h->trace_names.empty()) h->trace_names.back() += L.desc;
    prof.finish();
}

}  // namespace nb
