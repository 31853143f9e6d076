// Internal declarations shared by the kernels and the C-ABI layer.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/nebula_b200.h"

namespace nb {

// ----------------------------------------------------------------- errors
struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string &m) : std::runtime_error(m), code(c) {}
};

#define NB_CHECK_CUDA(expr)                                                                     \
    do {                                                                                        \
        cudaError_t _e = (expr);                                                                \
        if (_e != cudaSuccess)                                                                  \
            throw nb::Error(NB_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e));   \
    } while (0)

#define NB_REQUIRE(cond, msg)                                                  \
    do {                                                                       \
        if (!(cond)) throw nb::Error(NB_ERR_INVALID_ARG, std::string(msg));    \
    } while (0)

// device status word written by kernels whose bounded waits give up
enum : int { DEV_OK = 0, DEV_TIMEOUT = 1 };

}  // namespace nb

typedef CUresult (*nb_encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                       const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                       CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                       CUtensorMapFloatOOBfill);

typedef CUresult (*nb_get_address_range_fn)(CUdeviceptr *, size_t *, CUdeviceptr);

namespace nb {
struct Arena;
// A launch whose parameters (tile geometry, tensor maps, grid) were worked out before: kept per handle under a key
// made of every argument that went into them, so that a layer's second and later forward passes only launch.
struct LaunchRecord { virtual ~LaunchRecord() {} };
}  // namespace nb

struct nb_handle_s {
    int device = 0;
    cudaStream_t stream = 0;
    int math_mode = NB_MATH_TF32;
    int sm_count = 0;
    int cc_major = 0;
    std::string last_error;
    int *d_status = nullptr;            // device status word (nb::DEV_*)
    unsigned int *d_grid_sync = nullptr; // arrival counter of the persistent LSTM kernel's grid barrier
    bool cooperative_launch = false;    // the device co-schedules the CTAs of a cooperative launch
    nb_encode_tiled_fn encode_tiled = nullptr;
    nb_get_address_range_fn get_address_range = nullptr;   // cuMemGetAddressRange: the allocation a pointer lies in
    unsigned long long launches = 0;
    // optional per-launch event timing of the contraction kernels
    struct Timed { cudaEvent_t start, stop; double flops; int kind; };
    bool profiling = false;
    std::vector<Timed> timed;
    std::vector<cudaEvent_t> event_pool;    // events are re-used across profiling windows
    std::unordered_map<std::string, std::unique_ptr<nb::LaunchRecord>> launch_cache;
    std::shared_ptr<nb::Arena> arena;
    // Opt-in launch trace (NEBULA_B200_TRACE=1 when the handle is created): after every kernel the stream writes that
    // launch's ordinal into page-locked host memory, so that after an asynchronous device error the message can
    // name the last launch that finished and the one that did not.
    typedef CUresult (*write_value_fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    write_value_fn write_value = nullptr;
    volatile unsigned *trace_host = nullptr;
    CUdeviceptr trace_dev = 0;
    std::vector<std::string> trace_names;
    // device allocations seen by check_extent: [base, end) by base address
    std::map<uintptr_t, uintptr_t> known_ranges;
};

namespace nb {

// ------------------------------------------------------------ device memory
// Every device buffer of the library comes out of a per-handle arena: a few large cudaMalloc'd chunks, carved first-fit.
// Why not one cudaMalloc per buffer: a TMA tiled load whose box lies partly (or wholly) at out-of-bounds coordinates
// delivers the fill value for those elements but still READS the addresses the coordinates map to (measured: the L2
// read-sector count of a box load does not depend on how much of the box is in bounds).  The zero padding of a
// convolution is made of exactly such loads, so they read the row above a tensor's first image, below its last
// one, and the rows past a weight matrix's last filter.  Those addresses must be mapped.  Inside a chunk they
// are: a buffer's neighbours are other buffers of the library, and END_GUARD bytes at both ends of every chunk
// are never handed out.  Launches check the range they can reach against the chunk (check_extent).
struct Arena {
    static constexpr size_t END_GUARD = (size_t)16 << 20;
    static constexpr size_t MIN_CHUNK = (size_t)256 << 20;
    struct Chunk {
        char *base = nullptr;
        size_t size = 0;
        std::map<size_t, size_t> free;      // offset -> length of the free runs
    };
    std::vector<Chunk> chunks;
    std::unordered_map<void *, std::pair<char *, size_t>> live;     // pointer -> (its chunk's base, length)
    size_t in_use = 0;
    ~Arena();
    void *alloc(size_t bytes);
    void release(void *p);
    // the arena of the handle whose call is running on this thread (set by the C-ABI entry points)
    static std::shared_ptr<Arena> &current();
};

struct DeviceBuffer {
    float *p = nullptr;
    size_t n = 0;
    size_t guard = 0;                       // floats after the n-th that belong to the buffer too (never read back)
    std::shared_ptr<Arena> owner;
    DeviceBuffer() {}
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    ~DeviceBuffer() { release(); }
    // guard_floats: extra floats behind the tensor that TMA boxes running past its last row may read
    void alloc(size_t count, size_t guard_floats = 0) {
        release();
        if (count) {
            owner = Arena::current();
            if (!owner) throw Error(NB_ERR_INVALID_ARG, "device allocation outside a library call");
            p = (float *)owner->alloc((count + guard_floats) * sizeof(float));
        }
        n = count;
        guard = guard_floats;
    }
    // true when the buffer had to grow (the caller may want to know that an allocation happened)
    bool reserve(size_t count, size_t guard_floats = 0) {
        if (n >= count && guard >= guard_floats) return false;
        alloc(count, guard_floats);
        return true;
    }
    void release() {
        if (p && owner) owner->release(p);
        p = nullptr;
        n = 0;
        guard = 0;
        owner.reset();
    }
};

// -------------------------------------------------------------- GEMM core
// D[M,N] = A[M,K] * B[N,K]^T, both operands K-major, with a fused epilogue
//   v = acc * scale[n] + shift[n] (+ addend[m,n]);  y[m,n] = act(v)
// A is either a plain row-major matrix or an implicit im2col view of an NHWC
// (or arbitrarily strided) activation tensor: row m = (image, oh, ow), column
// k = (kh, kw, c) with c fastest.
struct ConvGeom {
    int batch = 1, C = 1, H = 1, W = 1;     // input extents
    int OH = 1, OW = 1;                     // output extents
    int ksize = 1, stride = 1, pad = 0;
    // tensor-core TMA path only: a filter of ksize rows x ksize_w columns (0: square) with its own horizontal padding
    // (-1: same as pad).  Used by the row-window route, where each filter row is one run of `C` contiguous floats.
    int ksize_w = 0, pad_w = -1;
    // element strides of the input tensor (for the CUDA-core gather path)
    long sn = 0, sc = 1, sh = 0, sw = 0;
};

struct GemmArgs {
    // A operand
    const float *a = nullptr;
    bool a_is_conv = false;     // false: plain [M,K] with row stride lda
    long lda = 0;
    ConvGeom g;                 // used when a_is_conv
    // tensor-core path only: build A in shared memory from the strided tensor described by g (any
    // channel count, any strides) instead of loading it by TMA.  Column kk of A is (kh, kw, c) with c
    // fastest, Kc = k*k*C rounded up to a multiple of 32; B is then a plain [N][Kc] matrix.
    bool a_gather = false;
    // B operand: [taps][N][Kc] (taps = ksize*ksize, Kc = channels per tap, row stride ldb)
    const float *b = nullptr;       // operand used by the TF32 / FP32 paths
    const float *b_lo = nullptr;    // low-order split of B for the 3xTF32 path
    long ldb = 0;
    int M = 0, N = 0;           // logical output extents
    int Kc = 0;                 // contraction length per tap (channels or FC inputs)
    // epilogue
    const float *scale = nullptr;   // may be null (=1)
    const float *shift = nullptr;   // may be null (=0)
    const float *addend = nullptr;  // may be null; same indexing as y unless res_stride > 0
    long ld_addend = 0;
    bool addend_after_act = false;  // y = act(acc*scale + shift) + addend instead of act(acc*scale + shift + addend)
    // residual form of the addend (tensor-core conv kernels): NHWC tensor [batch][res_h][res_w][ld_addend] of
    // which output pixel (n,oh,ow) takes channels [0,res_c) of pixel (n, oh*res_stride, ow*res_stride)
    int res_stride = 0, res_c = 0, res_h = 0, res_w = 0;
    int act = NB_ACT_LINEAR;
    bool round_out_tf32 = false;    // store RN(TF32) values (the consumer is a TF32 contraction)
    float *y = nullptr;
    long ldy = 0;
    // tensor-core conv only: write the 2x2 stride-2 max-pooled output [B][OH/2][OW/2][N] here INSTEAD of y
    float *y_pool = nullptr;
    // tensor-core kernel, plain matrices: the N = 4*lstm_H columns are gate pre-activations laid out
    // [hidden unit][i,f,g,o]; the epilogue runs the LSTM cell update and writes c_t, h_t (and a TF32-rounded
    // copy of h_t) [M][lstm_H] instead of y
    int lstm_H = 0;
    const float *lstm_c_prev = nullptr;
    float *lstm_c = nullptr, *lstm_h = nullptr, *lstm_h_round = nullptr;
    // plain matrices only: contract K in `split_k` slices of ceil(K blocks / split_k) 32-wide blocks (the last may be
    // shorter, none empty); slice s writes y + s*M*ldy
    // (y must hold split_k * M * ldy floats; the caller reduces the slices and applies the epilogue)
    int split_k = 1;
    // tensor-core kernel: tile width in output columns (64, 128 or 256) instead of the built-in choice; 0 = automatic
    int block_n_hint = 0;
    double algo_flops = 0;          // algorithmic FLOPs of this launch for profiling (0: 2*M*N*Kc*taps)
};

// Tensor-core path (tcgen05 + TMA).  Throws nb::Error(NB_ERR_UNSUPPORTED) when the
// operands do not meet TMA's layout rules; callers then use gemm_simt.
bool gemm_tc_supported(const nb_handle_s *h, const GemmArgs &a);
void gemm_tc(nb_handle_s *h, const GemmArgs &a, bool three_pass);
// 3x3 stride-1 convolutions with 32..128 input channels: one halo load per channel slice serves all nine taps.
bool conv_halo_supported(const nb_handle_s *h, const GemmArgs &a);
void conv_halo_tc(nb_handle_s *h, const GemmArgs &a);
// CUDA-core fp32 path: any extents, strides and alignments.
void gemm_simt(nb_handle_s *h, const GemmArgs &a);
// Dispatch on the handle's math mode.
void gemm(nb_handle_s *h, const GemmArgs &a);

// ------------------------------------------------------- elementwise et al.
void launch_activation(nb_handle_s *h, int act, float *data, size_t n);
void launch_bias(nb_handle_s *h, float *out, const float *bias, unsigned channel, unsigned size, unsigned batch);
void launch_bn_normalize(nb_handle_s *h, float *out, const float *mean, const float *var, unsigned channel,
                         unsigned size, unsigned batch);
void launch_bn_scale(nb_handle_s *h, float *out, const float *scale, unsigned channel, unsigned size,
                     unsigned batch);
void launch_softmax(nb_handle_s *h, const float *x, float *y, int rows, int classes);
// src NCHW -> dst NHWC (to_nhwc) or back; optional TF32 rounding of the copy
void launch_layout(nb_handle_s *h, const float *src, float *dst, int B, int C, int H, int W, bool to_nhwc,
                   bool round_tf32);
void launch_round_tf32(nb_handle_s *h, const float *src, float *dst, size_t n);
void launch_split_tf32(nb_handle_s *h, const float *src, float *hi, float *lo, size_t n);
void launch_pool(nb_handle_s *h, const nb_pool_desc_t &d, const float *x, float *y, bool round_tf32);
void launch_shortcut(nb_handle_s *h, const nb_shortcut_desc_t &d, const float *prev, const float *conn, float *y,
                     bool round_tf32);
// weights OIHW [F,C,k,k] -> [k*k][F][Cp] (Cp >= C, zero padded), optionally permuting FC columns
// first-layer row windows: [F][C][k][k] -> [kh][F][inner], column = kw*4 + c (zero elsewhere)
void launch_weight_rowwin(nb_handle_s *h, const float *w, float *dst, int F, int C, int k, int inner);
// NCHW or NHWC [N][C][H][W] -> [N][H][Wp][4] with `pad` zero pixels on the left, zeros on the right and in channels >= C
void launch_rowwin_input(nb_handle_s *h, const float *x, float *dst, int N, int C, int H, int W, int Wp, int pad, bool nhwc_in,
                         bool round);
// decoded 8-bit images [N][H][W][C] -> fp32 NCHW batch, or (rowwin) the first convolution's [N][H][Wp][4] tensor
void launch_u8_pack(nb_handle_s *h, const unsigned char *img, float *dst, int N, int C, int H, int W, bool rowwin, int Wp,
                    int pad, bool round);
void launch_weight_relayout(nb_handle_s *h, const float *w_oihw, float *dst, int F, int C, int k, int Cp);
// weights OIHW -> [F][Kpad] with column (kh,kw,c), zero padded: the B operand of the gathered-A convolution
void launch_weight_pack(nb_handle_s *h, const float *w_oihw, float *dst, int F, int C, int k, int Kpad);
// FC weights whose columns index (c,h,w) -> columns indexing (h,w,c)
void launch_fc_permute(nb_handle_s *h, const float *w, float *dst, int out, int C, int H, int W);
// sum of S slices [S][M][N] + folded scale/shift + activation (+ TF32 rounding) -> y [M][N]
void launch_splitk_reduce(nb_handle_s *h, const float *ws, int S, int M, int N, const float *scale, const float *shift,
                          int act, bool round_tf32, float *y);
// LSTM cell: z [B,4H] laid out [hidden unit][i,f,g,o] -> c_t, h_t (+ TF32-rounded copy of h_t)
void launch_lstm_cell(nb_handle_s *h, const float *z, const float *c_prev, float *c_out, float *h_out,
                      float *h_round, int B, int H);

// _gemm_ of the operator library: row-major C = alpha*op(A)*op(B) + beta*C
void launch_sgemm(nb_handle_s *h, bool ta, bool tb, int M, int N, int K, float alpha, const float *A, int lda,
                  const float *B, int ldb, float beta, float *C, int ldc);

// Brackets one contraction launch with events while profiling is on
// (kind 0 = generic tensor-core kernel, 1 = CUDA-core kernel, 2 = 3x3 halo tensor-core kernel).
struct ProfileScope {
    nb_handle_s *h;
    nb_handle_s::Timed t;
    bool on;
    ProfileScope(nb_handle_s *hh, int kind, double flops) : h(hh), on(hh->profiling) {
        if (!on) return;
        t.kind = kind; t.flops = flops;
        t.start = t.stop = nullptr;
        auto take = [&](cudaEvent_t &e) {
            if (h->event_pool.empty()) NB_CHECK_CUDA(cudaEventCreate(&e));
            else { e = h->event_pool.back(); h->event_pool.pop_back(); }
        };
        take(t.start); take(t.stop);
        NB_CHECK_CUDA(cudaEventRecord(t.start, h->stream));
    }
    // call after the launch; a scope that is abandoned (the launch threw) returns its events to the pool
    void finish() {
        if (!on) return;
        on = false;
        NB_CHECK_CUDA(cudaEventRecord(t.stop, h->stream));
        h->timed.push_back(t);
    }
    ~ProfileScope() {
        if (!on) return;
        if (t.start) h->event_pool.push_back(t.start);
        if (t.stop) h->event_pool.push_back(t.stop);
    }
};

// fp32, 128-byte swizzle, zero fill: the one kind of tensor map the kernels use (cached per handle)
void encode_tensor_map(nb_handle_s *h, CUtensorMap *tm, const void *base, int rank, const cuuint64_t *dims,
                       const cuuint64_t *strides_bytes, const cuuint32_t *box, const cuuint32_t *elem_strides);

void trace_launch(nb_handle_s *h);
inline void count_launch(nb_handle_s *h, int n = 1) {
    h->launches += (unsigned long long)n;
    if (h->trace_host) trace_launch(h);
}
void check_launch(const char *what);
// what the launch trace knows about where the stream got to (empty when tracing is off)
std::string trace_report(nb_handle_s *h);

// Fails with NB_ERR_INVALID_ARG when [p + lo_bytes, p + hi_bytes) is not inside ONE device allocation (as the driver
// reports it for p).  Pointers the driver does not know as an allocation (module globals, host memory) pass.
void check_extent(nb_handle_s *h, const void *p, long long lo_bytes, long long hi_bytes, const char *what);

// Appends the raw bytes of a value to a cache key.
template <class T>
inline void key_add(std::string &k, const T &v) { k.append(reinterpret_cast<const char *>(&v), sizeof v); }
// Every field of a GemmArgs that decides a launch's parameters.
std::string gemm_args_key(const GemmArgs &a, char tag, int extra);

// Per-device set-up of the tensor-core kernels (shared-memory limits; also loads their code), once per handle.
void gemm_tc_prepare_device();
void lstm_persistent_prepare_device();
bool lstm_persistent_supported(const nb_handle_s *h, int T, int B, int H);
void lstm_persistent(nb_handle_s *h, const float *w_hi, const float *pre, float *cell, float *out, float *hr, int T, int B,
                     int H, int t_first);
void conv_halo_prepare_device();
void elementwise_prepare_device();

}  // namespace nb
