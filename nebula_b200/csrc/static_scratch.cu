// nb_fc_forward_static: a connected-layer forward that allocates nothing.
//
// Who needs it: callers that are not allowed to allocate device memory while they
// run -- a serving loop whose whole device-memory budget was handed to another
// allocator (a framework's caching pool, a fixed arena carved up at start-up), or
// a latency-critical phase where cudaMalloc's device-wide synchronisation, or its
// failing under memory pressure, is not acceptable.  The plan-based entry points
// allocate lazily (rounded operand copies, weight splits); this one keeps its
// working copies in a fixed array that is part of the library image instead.
//
// The scratch is the file-scope array below: NB_STATIC_SCRATCH_FLOATS floats
// (16 MiB), present on every GPU that loads the library until the process exits.
// Its name is only a host-side stand-in; the device address is looked up once per
// device with cudaGetSymbolAddress (with that device current) on the first call
// for that device, and that pointer is what the kernels receive.  Make that first
// call before starting any stream capture.
//
// All calls share the one array and it keeps whatever the last call left there.
// Nothing in it has to start at zero: every call overwrites exactly the regions it
// reads afterwards.  Two calls that overlap on the GPU (different streams, or
// different host threads) race on it; serialise them.
#include <mutex>

#include "nb_internal.h"

#define NB_STATIC_SCRATCH_FLOATS (4u * 1024u * 1024u)

static __device__ __align__(256) float nb_static_scratch[NB_STATIC_SCRATCH_FLOATS];

namespace {

constexpr int kMaxDevices = 64;
float *g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of the scratch array on `device` (which must be current).
float *scratch_for_device(int device) {
    if (device < 0 || device >= kMaxDevices) throw nb::Error(NB_ERR_INVALID_ARG, "device index beyond the scratch table");
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[device]) {
        float *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&p, nb_static_scratch);
        if (e != cudaSuccess || !p)
            throw nb::Error(NB_ERR_CUDA, std::string("cudaGetSymbolAddress(nb_static_scratch): ") + cudaGetErrorString(e));
        g_scratch_ptr[device] = p;
    }
    return g_scratch_ptr[device];
}

inline size_t round_up64(size_t n) { return (n + 63) / 64 * 64; }     // keeps every region 256-byte aligned
inline bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

extern "C" int nb_fc_forward_static(nb_handle_t h, const float *x, const float *weight, const float *bias, int batch,
                                    int inputs, int outputs, int activation, float *y) {
    if (!h) return NB_ERR_INVALID_ARG;
    try {
        NB_REQUIRE(x && weight && bias && y, "connected (static): null pointer");
        NB_REQUIRE(batch > 0 && inputs > 0 && outputs > 0, "connected (static): non-positive extent");
        NB_REQUIRE(activation > NB_ACT_UNDEFINED && activation < NB_ACT_COUNT, "connected (static): undefined activation");
        int prev = -1;
        NB_CHECK_CUDA(cudaGetDevice(&prev));
        if (prev != h->device) NB_CHECK_CUDA(cudaSetDevice(h->device));
        struct Restore { int prev, cur; ~Restore() { if (prev != cur) cudaSetDevice(prev); } } restore{prev, h->device};

        const size_t xn = (size_t)batch * inputs, wn = (size_t)outputs * inputs;
        const bool tensor_core = h->math_mode != NB_MATH_FP32 && h->encode_tiled && (inputs % 4) == 0 && inputs >= 32 &&
                                 aligned16(x) && aligned16(weight) && aligned16(y);
        const bool three = h->math_mode == NB_MATH_TF32X3;
        // working copies: TF32 -> rounded x and rounded W; 3xTF32 -> hi and lo parts of W; plus the bias,
        // which the kernel reads 32 columns at a time (the copy is padded to a multiple of 64)
        // Both operands are read by TMA from the array (never from the caller's tensors: a box that runs past a
        // matrix's last row is delivered as zeros, but the load unit still reads the addresses behind the matrix,
        // so those must lie inside the array as well).  Layout: bias | x | W (| W low part) | headroom, the headroom
        // being the rows the widest weight tile can run past the last output: 256 * inputs + 32 floats.
        const size_t bn = round_up64((size_t)outputs);
        const size_t headroom = 256 * (size_t)inputs + 32;
        const size_t need = !tensor_core ? 0 : bn + round_up64(xn) + (three ? 2 : 1) * round_up64(wn) + headroom;
        if (need > NB_STATIC_SCRATCH_FLOATS)
            throw nb::Error(NB_ERR_INVALID_ARG,
                            "connected (static): needs " + std::to_string(need) + " scratch floats (operand copies plus " +
                                std::to_string(headroom) + " of headroom), the built-in array holds " +
                                std::to_string((size_t)NB_STATIC_SCRATCH_FLOATS) + " (16 MiB); use the plan-based nb_fc_forward");
        nb::GemmArgs a;
        a.lda = inputs; a.ldb = inputs;
        a.M = batch; a.N = outputs; a.Kc = inputs;
        a.shift = bias;
        a.act = activation;
        a.y = y; a.ldy = outputs;
        if (!tensor_core) {
            a.a = x; a.b = weight;
            nb::gemm_simt(h, a);
        } else {
            float *scratch = scratch_for_device(h->device);
            NB_CHECK_CUDA(cudaMemcpyAsync(scratch, bias, (size_t)outputs * sizeof(float), cudaMemcpyDeviceToDevice, h->stream));
            a.shift = scratch;          // columns beyond `outputs` hold stale values that only masked lanes see
            scratch += bn;
            if (three) {
                float *x_c = scratch, *w_hi = scratch + round_up64(xn), *w_lo = w_hi + round_up64(wn);
                NB_CHECK_CUDA(cudaMemcpyAsync(x_c, x, xn * sizeof(float), cudaMemcpyDeviceToDevice, h->stream));
                nb::launch_split_tf32(h, weight, w_hi, w_lo, wn);
                a.a = x_c; a.b = w_hi; a.b_lo = w_lo;
            } else {
                float *x_r = scratch, *w_r = scratch + round_up64(xn);
                nb::launch_round_tf32(h, x, x_r, xn);
                nb::launch_round_tf32(h, weight, w_r, wn);
                a.a = x_r; a.b = w_r;
            }
            nb::gemm_tc(h, a, three);
        }
        return NB_OK;
    } catch (const nb::Error &e) {
        h->last_error = e.what();
        return e.code;
    } catch (const std::exception &e) {
        h->last_error = e.what();
        return NB_ERR_INVALID_ARG;
    }
}
