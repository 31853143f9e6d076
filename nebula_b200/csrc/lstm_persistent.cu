// The recurrence of one LSTM layer as ONE cooperative kernel over all time steps (lstm_layer.cc:262-311 per step).
//
// A launch per time step costs about 20 us on this part for a 64 x 4096 x 1024 product that needs 3: pipeline fill,
// 32 small K blocks issued by single lanes, launch gaps.  Here every CTA owns 32 gate columns (8 hidden units x
// i,f,g,o), keeps its 32 x H slice of the recurrent weights in shared memory for the whole sequence (128 KB at
// H = 1024, loaded once by TMA) and the cell state of its units in registers.  Per step it streams h_{t-1} (rounded
// to TF32, [B x H]) from L2 into a ring of 128-byte-swizzled K blocks with plain loads, multiplies on the tensor core
// (tcgen05.mma kind::tf32, M = 128, N = 32, accumulator in TMEM), adds the input-side pre-activations, runs the cell
// update and writes c_t, h_t and the rounded h_t.  A grid-wide barrier (one atomic counter, bounded spin) separates
// the steps: step t + 1 of every CTA reads what all CTAs wrote in step t.
//
// h_{t-1} was written by other SMs' ordinary stores earlier in this same kernel and is read here by TMA, i.e. through
// the async proxy: the writers release (fence + release-add on the barrier counter), the reader acquires the counter and
// then issues fence.proxy.async before its first copy of the step.  (A first version read h with ld.global.cg from
// 128 threads: correct, but 63 us per step, three times slower than a launch per step.)  The results are bit-identical
// to the per-step path (same K order, same fp32 cell arithmetic).
#include <cstring>

#include "tc_common.cuh"

namespace nb {

using namespace tc;

namespace {

constexpr int LP_N = 32;                    // gate columns per CTA
constexpr int LP_STAGES = 4;                // most ring stages (barrier slots)
constexpr int LP_THREADS = 192;             // warps 0-3: epilogue and grid barrier; warp 4: MMA issue; warp 5: TMA
constexpr int LP_W_TILE = LP_N * 128;       // one K block of the weight slice: 32 rows x 128 bytes

struct LstmPParams {
    CUtensorMap tm_w;           // recurrent weights [4H rows][H], box {32, 32}
    CUtensorMap tm_h;           // rounded hidden states as {32, T*B rows, H/32}, box {32, B, cbs}
    int cbs;                    // K blocks per ring stage and TMA request (2 when B % 8 == 0 and H % 64 == 0)
    int stages, stage_bytes;    // ring geometry: a stage holds cbs slices of B rows and the 128-row window of the last
    const float *pre;           // [T][B][4H] input-side pre-activations (biases included), columns [unit][i,f,g,o]
    float *hr_w;                // [T][B][H] rounded hidden states: step t writes [t]; step t + 1 reads it through tm_h
    float *cell, *out;          // [T][B][H]
    int T, B, H;
    int t_first;                // first step this kernel runs (the steps before it are in cell/out/hr already)
    unsigned int *sync;         // grid barrier counter, zero at launch
    int *status;
};

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned int *p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(LP_THREADS, 1) lstm_persistent_kernel(const __grid_constant__ LstmPParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int KB = p.H / BLOCK_K;                           // K blocks per step
    uint8_t *w_smem = smem;                                  // [KB][32 rows][128 B], swizzled by TMA
    uint8_t *a_ring = smem + (size_t)KB * LP_W_TILE;         // [LP_STAGES][128 rows][128 B]
    const int stages = p.stages, stage_bytes = p.stage_bytes, cbs = p.cbs;
    uint64_t *bars = (uint64_t *)(a_ring + stages * stage_bytes);
    uint64_t *full = bars;                  // loaders -> MMA   [LP_STAGES]
    uint64_t *empty = bars + LP_STAGES;     // MMA -> loaders   [LP_STAGES]
    uint64_t *w_full = bars + 2 * LP_STAGES;
    uint64_t *acc_full = w_full + 1;
    uint64_t *step_go = acc_full + 1;       // grid barrier passed: h of the previous step is complete
    uint32_t *tmem_slot = (uint32_t *)(step_go + 1);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < LP_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(w_full, 1);
        mbar_init(acc_full, 1);
        mbar_init(step_go, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(32u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // rows of the A tiles that no batch row fills: the MMA reads all 128, give them a defined value once
    for (int i = threadIdx.x; i < stages * stage_bytes / 16; i += blockDim.x)
        reinterpret_cast<float4 *>(a_ring)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int n0 = blockIdx.x * LP_N;                       // first gate column of this CTA
    const unsigned int ctas = gridDim.x;
    bool ok = true;

    if (warp == 4) {
        // ------------------------------------------------ weights (once), then the MMAs of every step
        if (elect_one()) {
            mbar_expect_tx(w_full, (uint32_t)(KB * LP_W_TILE));
            for (int kb = 0; kb < KB; kb++) tma_load_3d(w_smem + kb * LP_W_TILE, &p.tm_w, w_full, kb * BLOCK_K, n0, 0);
            ok = mbar_wait(w_full, 0, abort_flag, p.status);
            const uint32_t idesc = p.B <= 64 ? make_idesc(64, LP_N) : make_idesc(BLOCK_M, LP_N);     // 64-row MMAs for small batches
            int stage = 0;
            uint32_t phase = 0;
            for (int t = p.t_first; t < p.T && ok; t++) {
                for (int kb = 0; kb < KB; kb += cbs) {
                    if (!(ok = mbar_wait(&full[stage], phase, abort_flag, p.status))) break;
                    tc_fence_after();
                    for (int c = 0; c < cbs; c++) {
                        const uint32_t a_lo = smem_desc_lo(smem_u32(a_ring + stage * stage_bytes + c * p.B * 128));
                        const uint32_t b_lo = smem_desc_lo(smem_u32(w_smem + (kb + c) * LP_W_TILE));
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; k++)
                            umma_tf32(tmem_base, smem_desc(a_lo + 2 * k), smem_desc(b_lo + 2 * k), idesc, (kb | c | k) != 0);
                    }
                    umma_commit(&empty[stage]);
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(acc_full);
            }
            // the last releases of the ring must have landed before the CTA may exit
            for (int i = 0; i < stages && ok; i++) {
                ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status);
                if (++stage == stages) { stage = 0; phase ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        // ------------------------------------------------ h_{t-1} of every step, one K block per ring stage
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0, go_phase = 0;
            const uint32_t tx = (uint32_t)(p.B * BLOCK_K * 4 * cbs);
            for (int t = p.t_first; t < p.T && ok; t++) {
                if (t > p.t_first) {
                    // the other CTAs' stores of h_{t-1} (generic proxy) are ordered before the acquire that opened the
                    // barrier; this fence orders the copies below (async proxy) behind it
                    if (!(ok = mbar_wait(step_go, go_phase, abort_flag, p.status))) break;
                    go_phase ^= 1;
                    asm volatile("fence.proxy.async;" ::: "memory");
                }
                for (int kb = 0; kb < KB; kb += cbs) {
                    if (!(ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status))) break;
                    mbar_expect_tx(&full[stage], tx);
                    tma_load_3d(a_ring + stage * stage_bytes, &p.tm_h, &full[stage], 0, (t - 1) * p.B, kb);
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------ epilogue of every step, then the grid barrier
        const int tid = threadIdx.x;                        // 0..127
        // the batch row whose accumulators this thread's TMEM lane holds: lane = row for a 128-row MMA; a 64-row MMA
        // puts 16 rows into the first 16 lanes of each 32-lane quarter
        const int lane = tid & 31;
        const int brow = p.B <= 64 ? (lane < 16 ? 16 * warp + lane : 1 << 20) : tid;
        const bool row_ok = brow < p.B;
        const int unit0 = n0 >> 2;                          // first hidden unit of this CTA (8 of them)
        float c[8];
#pragma unroll
        for (int u = 0; u < 8; u++) c[u] = 0.0f;
        if (row_ok && p.t_first > 0) {
            const float *cp = p.cell + ((size_t)(p.t_first - 1) * p.B + brow) * p.H + unit0;
            const float4 lo = *reinterpret_cast<const float4 *>(cp), hi = *reinterpret_cast<const float4 *>(cp + 4);
            c[0] = lo.x; c[1] = lo.y; c[2] = lo.z; c[3] = lo.w; c[4] = hi.x; c[5] = hi.y; c[6] = hi.z; c[7] = hi.w;
        }
        uint32_t acc_phase = 0;
        for (int t = p.t_first; t < p.T && ok; t++) {
            // gates of this CTA's 8 units for row `tid`; threads only leave the loop together, at the votes, so that
            // none is left alone at a barrier
            // the input-side pre-activations of this step come from DRAM: fetched while the MMAs run
            const size_t row = (size_t)t * p.B + brow;
            float4 z4[8];
            if (row_ok) {
                const float4 *zin = reinterpret_cast<const float4 *>(p.pre + row * 4 * p.H + n0);
#pragma unroll
                for (int u = 0; u < 8; u++) z4[u] = __ldg(zin + u);
            }
            ok = epilogue_all(mbar_wait(acc_full, acc_phase, abort_flag, p.status), 1);
            if (!ok) break;
            acc_phase ^= 1;
            tc_fence_after();
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16), v);
            tmem_ld_wait();
            tc_fence_before();
            if (row_ok) {
                float hn[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const float zi = __uint_as_float(v[4 * u]) + z4[u].x, zf = __uint_as_float(v[4 * u + 1]) + z4[u].y;
                    const float zg = __uint_as_float(v[4 * u + 2]) + z4[u].z, zo = __uint_as_float(v[4 * u + 3]) + z4[u].w;
                    const float2 ch = lstm_cell_unit_f32_inline(zi, zf, zg, zo, c[u]);
                    c[u] = ch.x; hn[u] = ch.y;
                }
                const size_t o = row * p.H + unit0;
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    *reinterpret_cast<float4 *>(p.cell + o + 4 * q) = make_float4(c[4 * q], c[4 * q + 1], c[4 * q + 2], c[4 * q + 3]);
                    *reinterpret_cast<float4 *>(p.out + o + 4 * q) = make_float4(hn[4 * q], hn[4 * q + 1], hn[4 * q + 2], hn[4 * q + 3]);
                    *reinterpret_cast<float4 *>(p.hr_w + o + 4 * q) = make_float4(round_tf32(hn[4 * q]), round_tf32(hn[4 * q + 1]),
                                                                                   round_tf32(hn[4 * q + 2]), round_tf32(hn[4 * q + 3]));
                }
            }
            // ---- grid barrier: every CTA's h_t is written before any CTA reads it
            if (t + 1 < p.T) {
                __threadfence();
                epilogue_bar_sync(1);
                bool arrived = true;
                if (tid == 0) {
                    red_release_add(p.sync, 1u);
                    const unsigned int target = ctas * (unsigned int)(t - p.t_first + 1);
                    const long long t0 = clock64();
                    while (ld_acquire_u32(p.sync) < target) {
                        if (*abort_flag || clock64() - t0 > WAIT_LIMIT_CYCLES) {
                            *abort_flag = 1;
                            atomicExch(p.status, (int)DEV_TIMEOUT);
                            arrived = false;
                            break;
                        }
                    }
                    __threadfence();
                    if (arrived) mbar_arrive(step_go);
                }
                ok = epilogue_all(arrived, 1);
            }
        }
        if (!ok) *abort_flag = 1;
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(2000);     // let copies and MMAs in flight land before TMEM goes
        __syncthreads();
    }
    if (warp == 4) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u) : "memory");
    }
}

struct LstmPLaunch : LaunchRecord {
    LstmPParams p;
    int grid, smem;
    double flops;
};

}  // namespace

void lstm_persistent_prepare_device() {
    NB_CHECK_CUDA(cudaFuncSetAttribute(lstm_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
}

// Whether the recurrence of an LSTM layer can run as the persistent kernel: TF32 mode on the tensor-core path, gate
// layers without an activation of their own, H a multiple of 32 whose weight slice and ring fit in shared memory,
// one CTA per 32 gate columns with all of them resident at once, a batch of at most 128 rows.
bool lstm_persistent_supported(const nb_handle_s *h, int T, int B, int H) {
    if (!h->encode_tiled || h->cc_major != 10 || !h->cooperative_launch) return false;
    if (T < 2 || B < 1 || B > 128 || (H % 32) != 0) return false;      // (a box of B rows: any B up to 128)
    const int ctas = 4 * H / LP_N;
    const size_t smem = (size_t)(H / BLOCK_K) * LP_W_TILE + 2 * (A_STAGE_BYTES + (size_t)B * 128) + 1024 + 256;   // two stages at least
    return ctas <= h->sm_count && smem <= 227 * 1024;
}

// Steps t_first .. T-1 of the recurrence (t_first >= 1: c, h and the rounded h of step t_first - 1 are in place).
void lstm_persistent(nb_handle_s *h, const float *w_hi, const float *pre, float *cell, float *out, float *hr, int T, int B,
                     int H, int t_first) {
    std::string key;
    key.push_back('P');
    key_add(key, w_hi); key_add(key, pre); key_add(key, cell); key_add(key, out); key_add(key, hr);
    key_add(key, T); key_add(key, B); key_add(key, H); key_add(key, t_first);
    auto it = h->launch_cache.find(key);
    if (it == h->launch_cache.end()) {
        std::unique_ptr<LstmPLaunch> L(new LstmPLaunch());
        std::memset(&L->p, 0, sizeof L->p);
        const long long F4 = 4;
        check_extent(h, w_hi, 0, (long long)4 * H * H * F4, "recurrent weights");
        check_extent(h, pre, 0, (long long)T * B * 4 * H * F4, "input-side pre-activations");
        check_extent(h, cell, 0, (long long)T * B * H * F4, "cell states");
        check_extent(h, out, 0, (long long)T * B * H * F4, "hidden states");
        check_extent(h, hr, 0, (long long)T * B * H * F4, "rounded hidden states");
        cuuint64_t dims[3] = {(cuuint64_t)H, (cuuint64_t)(4 * H), 1};
        cuuint64_t strides[2] = {(cuuint64_t)H * 4, (cuuint64_t)H * 4 * (cuuint64_t)(4 * H)};
        cuuint32_t bx[3] = {(cuuint32_t)BLOCK_K, (cuuint32_t)LP_N, 1};
        cuuint32_t es[3] = {1, 1, 1};
        encode_tensor_map(h, &L->p.tm_w, w_hi, 3, dims, strides, bx, es);
        // two K blocks per request when the second slice starts on the swizzle pattern's 1024-byte repeat
        const int cbs = ((B % 8) == 0 && (H % (2 * BLOCK_K)) == 0) ? 2 : 1;
        const int stage_bytes = (cbs - 1) * B * 128 + A_STAGE_BYTES;
        const int w_bytes = (H / BLOCK_K) * LP_W_TILE;
        const int stages = std::min(LP_STAGES, (227 * 1024 - 1024 - 256 - w_bytes) / stage_bytes);
        cuuint64_t hdims[3] = {(cuuint64_t)BLOCK_K, (cuuint64_t)T * (cuuint64_t)B, (cuuint64_t)(H / BLOCK_K)};
        cuuint64_t hstrides[2] = {(cuuint64_t)H * 4, (cuuint64_t)BLOCK_K * 4};
        cuuint32_t hbx[3] = {(cuuint32_t)BLOCK_K, (cuuint32_t)B, (cuuint32_t)cbs};
        cuuint32_t hes[3] = {1, 1, 1};
        encode_tensor_map(h, &L->p.tm_h, hr, 3, hdims, hstrides, hbx, hes);
        L->p.cbs = cbs; L->p.stages = stages; L->p.stage_bytes = stage_bytes;
        L->p.pre = pre; L->p.hr_w = hr; L->p.cell = cell; L->p.out = out;
        L->p.T = T; L->p.B = B; L->p.H = H; L->p.t_first = t_first;
        L->p.sync = h->d_grid_sync; L->p.status = h->d_status;
        L->grid = 4 * H / LP_N;
        L->smem = w_bytes + stages * stage_bytes + 1024 + 256;
        L->flops = 2.0 * (double)(T - t_first) * B * 4.0 * H * H;
        if (h->launch_cache.size() > 4096) h->launch_cache.clear();
        it = h->launch_cache.emplace(std::move(key), std::move(L)).first;
    }
    const LstmPLaunch &L = static_cast<const LstmPLaunch &>(*it->second);
    NB_CHECK_CUDA(cudaMemsetAsync(h->d_grid_sync, 0, sizeof(unsigned int), h->stream));
    ProfileScope prof(h, 0, L.flops);
    void *args[1] = {const_cast<LstmPParams *>(&L.p)};
    NB_CHECK_CUDA(cudaLaunchCooperativeKernel((const void *)lstm_persistent_kernel, dim3(L.grid), dim3(LP_THREADS), args, (size_t)L.smem,
                                              h->stream));
    check_launch("lstm_persistent_kernel");
    count_launch(h);
    prof.finish();
}

}  // namespace nb
