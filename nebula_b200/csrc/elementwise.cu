// Memory-bound kernels of the forward path: activations, bias, inference
// batch-norm passes, pooling, shortcut, softmax, layout changes, TF32
// rounding/splitting of operands, weight re-layouts and the LSTM cell.
// All are grid-stride, bounds-checked, and use 128-bit accesses where the
// innermost extent allows.
#include <algorithm>
#include <cstdlib>

#include "device_math.cuh"
#include "nb_internal.h"

namespace nb {

// NEBULA_B200_SYNC_LAUNCHES=1 in the environment waits for every kernel before returning, so that an asynchronous
// device error is reported against the launch that caused it (debugging aid; off by default).
namespace { thread_local const char *t_last_launch = ""; }

void trace_launch(nb_handle_s *h) {
    if (h->trace_names.size() > (1u << 20)) return;
    h->trace_names.push_back(t_last_launch);
    h->write_value((CUstream)h->stream, h->trace_dev, (cuuint32_t)h->trace_names.size(), 0);
}
std::string trace_report(nb_handle_s *h) {
    if (!h->trace_host) return "";
    const unsigned done = *h->trace_host;
    std::string r = " [launch trace: " + std::to_string(done) + " of " + std::to_string(h->trace_names.size()) + " launches finished";
    if (done > 0 && done <= h->trace_names.size()) r += "; last finished: #" + std::to_string(done) + " " + h->trace_names[done - 1];
    for (unsigned i = done; i < h->trace_names.size() && i < done + 3; i++)
        r += "; then #" + std::to_string(i + 1) + " " + h->trace_names[i];
    return r + "]";
}

void check_launch(const char *what) {
    t_last_launch = what;
    static const bool sync_launches = [] {
        const char *v = std::getenv("NEBULA_B200_SYNC_LAUNCHES");
        return v && *v && *v != '0';
    }();
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && sync_launches) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) throw Error(NB_ERR_CUDA, std::string(what) + " launch: " + cudaGetErrorString(e));
}

void check_extent(nb_handle_s *h, const void *p, long long lo_bytes, long long hi_bytes, const char *what) {
    if (!h->get_address_range || !p || hi_bytes <= lo_bytes) return;
    const uintptr_t q = (uintptr_t)p, a = q + lo_bytes, b = q + hi_bytes;
    auto it = h->known_ranges.upper_bound(q);
    if (it != h->known_ranges.begin()) {
        --it;
        if (q < it->second && a >= it->first && b <= it->second) return;
    }
    // not covered by what was seen before (or that allocation has been replaced since): ask the driver
    CUdeviceptr base = 0;
    size_t size = 0;
    if (h->get_address_range(&base, &size, (CUdeviceptr)q) != CUDA_SUCCESS || !size) return;   // not an allocation
    const uintptr_t lo = (uintptr_t)base, hi = lo + size;
    for (auto k = h->known_ranges.begin(); k != h->known_ranges.end();)     // forget stale overlapping entries
        k = (k->first < hi && k->second > lo) ? h->known_ranges.erase(k) : std::next(k);
    if (h->known_ranges.size() > 4096) h->known_ranges.clear();
    h->known_ranges[lo] = hi;
    if (a < lo || b > hi)
        throw Error(NB_ERR_INVALID_ARG, std::string(what) + ": the launch would touch bytes [" + std::to_string(lo_bytes) + ", " +
                                            std::to_string(hi_bytes) + ") from its pointer, but the allocation it lies in holds [" +
                                            std::to_string((long long)lo - (long long)q) + ", " +
                                            std::to_string((long long)hi - (long long)q) + ")");
}

namespace {

constexpr int TPB = 256;

inline unsigned grid_for(size_t n, const nb_handle_s *h, int per_thread = 1) {
    size_t blocks = (n + (size_t)TPB * per_thread - 1) / ((size_t)TPB * per_thread);
    size_t cap = (size_t)std::max(1, h->sm_count) * 32;       // grid-stride beyond this
    return (unsigned)std::max<size_t>(1, std::min(blocks, cap));
}

// ------------------------------------------------------------- activations
// _<name>_activation_ (common/activations.cu:8-141) with the CPU formulas.
__global__ void activation_kernel(float *data, size_t n, int act) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if ((((uintptr_t)data) & 15) == 0) {
        const size_t n4 = n / 4;
        float4 *d4 = reinterpret_cast<float4 *>(data);
        for (size_t j = i; j < n4; j += stride) {
            float4 v = d4[j];
            v.x = apply_activation(v.x, act); v.y = apply_activation(v.y, act);
            v.z = apply_activation(v.z, act); v.w = apply_activation(v.w, act);
            d4[j] = v;
        }
        for (size_t j = n4 * 4 + i; j < n; j += stride) data[j] = apply_activation(data[j], act);
    } else {
        for (; i < n; i += stride) data[i] = apply_activation(data[i], act);
    }
}

// _add_bias_ (common/utils.cu:118-134): y[b,c,s] += bias[c]
__global__ void bias_kernel(float *out, const float *bias, unsigned channel, unsigned size, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
        out[i] += bias[(i / size) % channel];
}
// _normalize_ (common/batchnorm.cu:77-84) with the CPU formula (batchnorm.cc:70):
// float subtraction, double divisor sqrt(var)+0.00001, stored as float.
__global__ void bn_normalize_kernel(float *out, const float *mean, const float *var, unsigned channel, unsigned size,
                                    size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const unsigned c = (i / size) % channel;
        out[i] = (float)((double)(out[i] - mean[c]) / (sqrt((double)var[c]) + 0.00001));
    }
}
// _scale_ (common/batchnorm.cu:86-104)
__global__ void bn_scale_kernel(float *out, const float *scale, unsigned channel, unsigned size, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
        out[i] *= scale[(i / size) % channel];
}

// ----------------------------------------------------------------- softmax
// softmax_layer_t::softmax (softmax_layer.cc:85-106): one block per row; warp
// shuffles reduce the max and the sum.  exp is evaluated in double on the float
// difference, as the CPU path does.
__device__ __forceinline__ float warp_max(float v) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__global__ void softmax_kernel(const float *x, float *y, int rows, int classes) {
    __shared__ float red[32];
    __shared__ float bcast;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float *in = x + (size_t)row * classes;
        float *out = y + (size_t)row * classes;
        float m = -3.402823466e+38f;
        for (int j = threadIdx.x; j < classes; j += blockDim.x) m = fmaxf(m, in[j]);
        m = warp_max(m);
        if (lane == 0) red[warp] = m;
        __syncthreads();
        if (warp == 0) {
            float v = lane < nw ? red[lane] : -3.402823466e+38f;
            v = warp_max(v);
            if (lane == 0) bcast = v;
        }
        __syncthreads();
        m = bcast;
        float s = 0.0f;
        for (int j = threadIdx.x; j < classes; j += blockDim.x) {
            const float e = (float)exp((double)(in[j] - m));
            out[j] = e;
            s += e;
        }
        s = warp_sum(s);
        __syncthreads();
        if (lane == 0) red[warp] = s;
        __syncthreads();
        if (warp == 0) {
            float v = lane < nw ? red[lane] : 0.0f;
            v = warp_sum(v);
            if (lane == 0) bcast = v;
        }
        __syncthreads();
        s = bcast;
        for (int j = threadIdx.x; j < classes; j += blockDim.x) out[j] = out[j] / s;
        __syncthreads();
    }
}

// ------------------------------------------------------------------ layouts
// [B][C][HW] <-> [B][HW][C] through a 32x32 shared-memory tile.
__global__ void transpose_kernel(const float *src, float *dst, int rows, int cols, int round) {
    // src is [batch][rows][cols], dst is [batch][cols][rows]
    __shared__ float tile[32][33];
    const size_t img = (size_t)blockIdx.z * rows * cols;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[j][threadIdx.x] = src[img + (size_t)r * cols + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int c = c0 + j, r = r0 + threadIdx.x;
        if (r < rows && c < cols) {
            const float v = tile[threadIdx.x][j];
            dst[img + (size_t)c * rows + r] = round ? round_tf32(v) : v;
        }
    }
}

// 128-bit accesses when both pointers are 16-byte aligned (every buffer of the library is); scalar tail / fallback.
__global__ void round_tf32_kernel(const float *src, float *dst, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t done = 0;
    if (((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {
        const size_t n4 = n / 4;
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        float4 *d4 = reinterpret_cast<float4 *>(dst);
        for (size_t i = tid; i < n4; i += stride) {
            float4 v = s4[i];
            v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w);
            d4[i] = v;
        }
        done = n4 * 4;
    }
    for (size_t i = done + tid; i < n; i += stride) dst[i] = round_tf32(src[i]);
}
// hi = RN_tf32(x), lo = RN_tf32(x - hi): the two terms of the 3xTF32 product.
__global__ void split_tf32_kernel(const float *src, float *hi, float *lo, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t done = 0;
    if (((((uintptr_t)src) | ((uintptr_t)hi) | ((uintptr_t)lo)) & 15) == 0) {
        const size_t n4 = n / 4;
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        float4 *h4 = reinterpret_cast<float4 *>(hi), *l4 = reinterpret_cast<float4 *>(lo);
        for (size_t i = tid; i < n4; i += stride) {
            const float4 x = s4[i];
            float4 h, l;
            h.x = round_tf32(x.x); h.y = round_tf32(x.y); h.z = round_tf32(x.z); h.w = round_tf32(x.w);
            l.x = round_tf32(x.x - h.x); l.y = round_tf32(x.y - h.y); l.z = round_tf32(x.z - h.z); l.w = round_tf32(x.w - h.w);
            h4[i] = h;
            l4[i] = l;
        }
        done = n4 * 4;
    }
    for (size_t i = done + tid; i < n; i += stride) {
        const float x = src[i], h = round_tf32(x);
        hi[i] = h;
        lo[i] = round_tf32(x - h);
    }
}

// ------------------------------------------------------------------ pooling
// pooling_layer_t::forward (pooling_layer.cc:109-182): window origin oh*s-p,
// max identity -1e8, average divisor k*k (padding included).
template <bool NHWC>
__global__ void pool_kernel(const float *x, float *y, int B, int C, int H, int W, int OH, int OW, int k, int s, int p,
                            int is_max, int round, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int c, ow, oh, b;
        size_t t = i;
        if (NHWC) { c = t % C; t /= C; ow = t % OW; t /= OW; oh = t % OH; b = (int)(t / OH); }
        else { ow = t % OW; t /= OW; oh = t % OH; t /= OH; c = t % C; b = (int)(t / C); }
        float mx = -1e8f, sum = 0.0f;
        for (int di = 0; di < k; di++) {
            const int r = oh * s + di - p;
            for (int dj = 0; dj < k; dj++) {
                const int q = ow * s + dj - p;
                const bool valid = r >= 0 && r < H && q >= 0 && q < W;
                float v = 0.0f;
                if (valid) v = NHWC ? x[(((size_t)b * H + r) * W + q) * C + c] : x[(((size_t)b * C + c) * H + r) * W + q];
                if (is_max) { v = valid ? v : -1e8f; mx = v > mx ? v : mx; }
                else sum += v;
            }
        }
        float o = is_max ? mx : sum / (float)(k * k);
        y[i] = round ? round_tf32(o) : o;
    }
}
// NHWC with C % 4 == 0: one thread per 4 channels
__global__ void pool_nhwc4_kernel(const float4 *x, float4 *y, int B, int C4, int H, int W, int OH, int OW, int k, int s,
                                  int p, int is_max, int round, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t t = i;
        const int c = t % C4; t /= C4;
        const int ow = t % OW; t /= OW;
        const int oh = t % OH;
        const int b = (int)(t / OH);
        float4 mx = make_float4(-1e8f, -1e8f, -1e8f, -1e8f), sum = make_float4(0, 0, 0, 0);
        for (int di = 0; di < k; di++) {
            const int r = oh * s + di - p;
            for (int dj = 0; dj < k; dj++) {
                const int q = ow * s + dj - p;
                const bool valid = r >= 0 && r < H && q >= 0 && q < W;
                if (valid) {
                    const float4 v = x[(((size_t)b * H + r) * W + q) * C4 + c];
                    mx.x = v.x > mx.x ? v.x : mx.x; mx.y = v.y > mx.y ? v.y : mx.y;
                    mx.z = v.z > mx.z ? v.z : mx.z; mx.w = v.w > mx.w ? v.w : mx.w;
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
            }
        }
        const float d = (float)(k * k);
        float4 o = is_max ? mx : make_float4(sum.x / d, sum.y / d, sum.z / d, sum.w / d);
        if (round) { o.x = round_tf32(o.x); o.y = round_tf32(o.y); o.z = round_tf32(o.z); o.w = round_tf32(o.w); }
        y[i] = o;
    }
}

// ----------------------------------------------------------------- shortcut
// shortcut() (common/utils.cc:28-60) + activation, as one pass over the output.
template <bool NHWC>
__global__ void shortcut_kernel(const float *prev, const float *conn, float *y, int B, int Ci, int Hi, int Wi, int Co,
                                int Ho, int Wo, int stride, int sample, int act, int round, size_t total) {
    const int mw = Wi < Wo ? Wi : Wo, mh = Hi < Ho ? Hi : Ho, mc = Ci < Co ? Ci : Co;
    const size_t gstride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
        int c, w, h, b;
        size_t t = i;
        if (NHWC) { c = t % Co; t /= Co; w = t % Wo; t /= Wo; h = t % Ho; b = (int)(t / Ho); }
        else { w = t % Wo; t /= Wo; h = t % Ho; t /= Ho; c = t % Co; b = (int)(t / Co); }
        float v = prev[i];
        if (c < mc && (h % sample) == 0 && (w % sample) == 0) {
            const int hh = h / sample, ww = w / sample;
            const int ih = hh * stride, iw = ww * stride;
            if (hh < mh && ww < mw && ih < Hi && iw < Wi) {
                v += NHWC ? conn[(((size_t)b * Hi + ih) * Wi + iw) * Ci + c] : conn[(((size_t)b * Ci + c) * Hi + ih) * Wi + iw];
            }
        }
        v = apply_activation(v, act);
        y[i] = round ? round_tf32(v) : v;
    }
}

// NHWC with both channel counts divisible by 4: one thread per 4 channels, 128-bit accesses
__global__ void shortcut_nhwc4_kernel(const float4 *prev, const float4 *conn, float4 *y, int B, int Ci4, int Hi, int Wi, int Co4,
                                      int Ho, int Wo, int stride, int sample, int act, int round, size_t total) {
    const int mw = Wi < Wo ? Wi : Wo, mh = Hi < Ho ? Hi : Ho, mc = Ci4 < Co4 ? Ci4 : Co4;
    const size_t gstride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
        size_t t = i;
        const int c = (int)(t % Co4); t /= Co4;
        const int w = (int)(t % Wo); t /= Wo;
        const int h = (int)(t % Ho);
        const int b = (int)(t / Ho);
        float4 v = prev[i];
        if (c < mc && (h % sample) == 0 && (w % sample) == 0) {
            const int hh = h / sample, ww = w / sample;
            const int ih = hh * stride, iw = ww * stride;
            if (hh < mh && ww < mw && ih < Hi && iw < Wi) {
                const float4 r = conn[(((size_t)b * Hi + ih) * Wi + iw) * Ci4 + c];
                v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
            }
        }
        v.x = apply_activation_fast(v.x, act); v.y = apply_activation_fast(v.y, act);
        v.z = apply_activation_fast(v.z, act); v.w = apply_activation_fast(v.w, act);
        if (round) { v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w); }
        y[i] = v;
    }
}

// ---------------------------------------------------- gathered-A weight layout
// OIHW [F][C][k][k] -> [F][Kpad] with column (tap*C + c), zero padded
__global__ void weight_pack_kernel(const float *w, float *dst, int F, int C, int k, int Kpad, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int taps = k * k, K = taps * C;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int kk = (int)(i % Kpad);
        const size_t f = i / Kpad;
        float v = 0.0f;
        if (kk < K) {
            const int tap = kk / C, c = kk - tap * C;
            v = w[(f * C + c) * taps + tap];
        }
        dst[i] = v;
    }
}

// ------------------------------------------------------ first-layer row windows
// A layer with at most 4 input channels is fed to the tensor cores one filter ROW at a time: in a pixel-major
// tensor with 4 floats per pixel, the k taps of a filter row are one contiguous run of 4*k floats, which a TMA box
// can fetch for a whole tile of output pixels (overlapping windows, 16-byte stride).  The horizontal padding is
// physical (zero pixels), the vertical padding is TMA's out-of-bounds fill.
__global__ void weight_rowwin_kernel(const float *w, float *dst, int F, int C, int k, int inner, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int j = (int)(i % inner);
        const size_t f = (i / inner) % F;
        const int kh = (int)(i / ((size_t)inner * F));
        const int kw = j >> 2, c = j & 3;
        dst[i] = (kw < k && c < C) ? w[((f * C + c) * k + kh) * k + kw] : 0.0f;
    }
}
__global__ void rowwin_input_kernel(const float *x, float4 *dst, int N, int C, int H, int W, int Wp, int pad, int nhwc_in,
                                    int round, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int pcol = (int)(i % Wp);
        const size_t nh = i / Wp;
        const int hrow = (int)(nh % H);
        const size_t n = nh / H;
        const int iw = pcol - pad;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (iw >= 0 && iw < W) {
            for (int c = 0; c < C; c++) {
                const float t = nhwc_in ? x[((n * H + hrow) * W + iw) * C + c] : x[((n * C + c) * H + hrow) * W + iw];
                v[c] = round ? round_tf32(t) : t;
            }
        }
        dst[i] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// Decoded 8-bit images [N][H][W][C] (C = 3: BGR as OpenCV holds them, or 1) -> the network input, with the reference's
// conversion (models/networks/convolutional.cc:386-398): value / 255.0 evaluated in double and stored as float, planes 0
// and 2 swapped for three channels.  Two destinations: the reference's own fp32 NCHW batch, or (rowwin != 0) the
// first convolution's row-window tensor [N][H][Wp][4] directly (zero pixels left and right, zero in channels >= C).
__global__ void u8_pack_kernel(const unsigned char *img, float *dst, int N, int C, int H, int W, int rowwin, int Wp, int pad,
                               int round, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        if (rowwin) {       // one thread per padded pixel
            const int pcol = (int)(i % Wp);
            const size_t nh = i / Wp;
            const int iw = pcol - pad;
            float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (iw >= 0 && iw < W) {
                const unsigned char *px = img + (nh * W + iw) * C;
                for (int c = 0; c < C; c++) {
                    const float t = (float)((double)px[C == 3 ? 2 - c : c] / 255.0);
                    v[c] = round ? round_tf32(t) : t;
                }
            }
            reinterpret_cast<float4 *>(dst)[i] = make_float4(v[0], v[1], v[2], v[3]);
        } else {            // one thread per output element of [N][C][H][W]
            size_t t = i;
            const int w = (int)(t % W); t /= W;
            const int hh = (int)(t % H); t /= H;
            const int c = (int)(t % C);
            const size_t n = t / C;
            dst[i] = (float)((double)img[((n * H + hh) * W + w) * C + (C == 3 ? 2 - c : c)] / 255.0);
        }
    }
}

// ---------------------------------------------------------- weight layouts
// OIHW [F][C][k][k] -> [tap][F][Cp], zero for c >= C
__global__ void weight_relayout_kernel(const float *w, float *dst, int F, int C, int k, int Cp, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int taps = k * k;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t t = i;
        const int c = t % Cp; t /= Cp;
        const int f = t % F;
        const int tap = (int)(t / F);
        dst[i] = c < C ? w[((size_t)f * C + c) * taps + tap] : 0.0f;
    }
}
// FC weight columns (c,h,w) -> (h,w,c)
__global__ void fc_permute_kernel(const float *w, float *dst, int out, int C, int HW, size_t total) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t in = (size_t)C * HW;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t o = i / in, rem = i - o * in;
        const int c = rem % C;
        const size_t hw = rem / C;
        dst[i] = w[o * in + (size_t)c * HW + hw];
    }
}

// -------------------------------------------------------------- split-K tail
// y[m][n] = act(scale[n] * sum_s ws[s][m][n] + shift[n]): the epilogue of a split-K contraction
// (slices are added in a fixed order, so the result does not depend on scheduling).
// N % 4 == 0 (what the split-K path requires) and 16-byte aligned tensors: four columns per thread, 128-bit accesses
__global__ void splitk_reduce4_kernel(const float4 *ws, int S, size_t MN4, int N4, const float4 *scale, const float4 *shift,
                                      int act, int round, float4 *y) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < MN4; i += stride) {
        float4 acc = ws[i];
        for (int s = 1; s < S; s++) {       // slices in a fixed order: the sum does not depend on scheduling
            const float4 v = ws[(size_t)s * MN4 + i];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const int n = (int)(i % N4);
        if (scale) {
            const float4 sc = scale[n], sh = shift[n];
            acc.x = fmaf(acc.x, sc.x, sh.x); acc.y = fmaf(acc.y, sc.y, sh.y);
            acc.z = fmaf(acc.z, sc.z, sh.z); acc.w = fmaf(acc.w, sc.w, sh.w);
        } else if (shift) {
            const float4 sh = shift[n];
            acc.x += sh.x; acc.y += sh.y; acc.z += sh.z; acc.w += sh.w;
        }
        acc.x = apply_activation_fast(acc.x, act); acc.y = apply_activation_fast(acc.y, act);
        acc.z = apply_activation_fast(acc.z, act); acc.w = apply_activation_fast(acc.w, act);
        if (round) { acc.x = round_tf32(acc.x); acc.y = round_tf32(acc.y); acc.z = round_tf32(acc.z); acc.w = round_tf32(acc.w); }
        y[i] = acc;
    }
}
__global__ void splitk_reduce_kernel(const float *ws, int S, size_t MN, int N, const float *scale, const float *shift,
                                     int act, int round, float *y) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < MN; i += stride) {
        float acc = ws[i];
        for (int s = 1; s < S; s++) acc += ws[(size_t)s * MN + i];
        const int n = (int)(i % N);
        if (scale) acc = fmaf(acc, scale[n], shift[n]);
        else if (shift) acc += shift[n];
        acc = apply_activation_fast(acc, act);
        y[i] = round ? round_tf32(acc) : acc;
    }
}

// ---------------------------------------------------------------- LSTM cell
// lstm_layer_t::forward (lstm_layer.cc:286-311): i,f,o = logistic(z), g = tanh(z),
// c_t = c_{t-1}*f + i*g, h_t = tanh(c_t)*o.  Products and the sum are separate
// fp32 roundings as on the CPU path (no fused multiply-add).
__global__ void lstm_cell_kernel(const float *z, const float *c_prev, float *c_out, float *h_out, float *h_round,
                                 int B, int H) {
    const size_t total = (size_t)B * H;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t b = idx / H, j = idx - b * H;
        const float4 zr = *reinterpret_cast<const float4 *>(z + (b * (size_t)H + j) * 4);     // [unit][i,f,g,o]
        const float ig = apply_activation(zr.x, NB_ACT_LOGISTIC);
        const float fg = apply_activation(zr.y, NB_ACT_LOGISTIC);
        const float gg = apply_activation(zr.z, NB_ACT_TANH);
        const float og = apply_activation(zr.w, NB_ACT_LOGISTIC);
        const float cp = c_prev ? c_prev[idx] : 0.0f;
        const float c = __fadd_rn(__fmul_rn(cp, fg), __fmul_rn(ig, gg));
        const float hv = __fmul_rn(apply_activation(c, NB_ACT_TANH), og);
        if (c_out) c_out[idx] = c;
        h_out[idx] = hv;
        if (h_round) h_round[idx] = round_tf32(hv);
    }
}

// ------------------------------------------------------------ generic SGEMM
// _gemm_ (common/gemm.h:21-25) with the CPU path's meaning of every argument
// (row-major, leading dimensions honoured, all four transpose cases), unlike the
// reference's CUDA stand-in (common/gemm.cu:38-153) which ignores lda/ldb/ldc.
__global__ void sgemm_kernel(int ta, int tb, int M, int N, int K, float alpha, const float *A, int lda, const float *B,
                             int ldb, float beta, float *C, int ldc) {
    __shared__ float As[16][17], Bs[16][17];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int row = blockIdx.y * 16 + ty, col = blockIdx.x * 16 + tx;
    float acc = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 16) {
        const int ka = k0 + tx, kb = k0 + ty;
        As[ty][tx] = (row < M && ka < K) ? (ta ? A[(size_t)ka * lda + row] : A[(size_t)row * lda + ka]) : 0.0f;
        Bs[ty][tx] = (col < N && kb < K) ? (tb ? B[(size_t)col * ldb + kb] : B[(size_t)kb * ldb + col]) : 0.0f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; k++) acc = fmaf(As[ty][k], Bs[k][tx], acc);
        __syncthreads();
    }
    if (row < M && col < N) {
        float *c = C + (size_t)row * ldc + col;
        *c = alpha * acc + (beta == 0.0f ? 0.0f : beta * *c);
    }
}

}  // namespace

// Loads the code of every kernel of this file on the current device (a kernel's code is otherwise loaded by its
// first launch, in the middle of the first forward pass).
void elementwise_prepare_device() {
    cudaFuncAttributes fa;
    const void *kernels[] = {
        (const void *)activation_kernel, (const void *)bias_kernel, (const void *)bn_normalize_kernel,
        (const void *)bn_scale_kernel, (const void *)softmax_kernel, (const void *)transpose_kernel,
        (const void *)round_tf32_kernel, (const void *)split_tf32_kernel, (const void *)pool_kernel<true>,
        (const void *)pool_kernel<false>, (const void *)pool_nhwc4_kernel, (const void *)shortcut_kernel<true>,
        (const void *)shortcut_kernel<false>, (const void *)weight_pack_kernel, (const void *)weight_rowwin_kernel,
        (const void *)rowwin_input_kernel, (const void *)weight_relayout_kernel, (const void *)fc_permute_kernel,
        (const void *)splitk_reduce_kernel, (const void *)lstm_cell_kernel, (const void *)sgemm_kernel,
        (const void *)u8_pack_kernel, (const void *)splitk_reduce4_kernel, (const void *)shortcut_nhwc4_kernel};
    for (const void *k : kernels) NB_CHECK_CUDA(cudaFuncGetAttributes(&fa, k));
}

// ---------------------------------------------------------------- launchers
void launch_sgemm(nb_handle_s *h, bool ta, bool tb, int M, int N, int K, float alpha, const float *A, int lda,
                  const float *B, int ldb, float beta, float *C, int ldc) {
    dim3 grid((N + 15) / 16, (M + 15) / 16), block(16, 16);
    if (grid.y > 65535) throw Error(NB_ERR_UNSUPPORTED, "gemm: M too large for this operator");
    sgemm_kernel<<<grid, block, 0, h->stream>>>(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
    check_launch("sgemm_kernel");
    count_launch(h);
}
void launch_activation(nb_handle_s *h, int act, float *data, size_t n) {
    if (act == NB_ACT_LINEAR || n == 0) return;
    activation_kernel<<<grid_for(n, h, 4), TPB, 0, h->stream>>>(data, n, act);
    check_launch("activation_kernel");
    count_launch(h);
}
void launch_bias(nb_handle_s *h, float *out, const float *bias, unsigned channel, unsigned size, unsigned batch) {
    const size_t total = (size_t)channel * size * batch;
    if (!total) return;
    bias_kernel<<<grid_for(total, h), TPB, 0, h->stream>>>(out, bias, channel, size, total);
    check_launch("bias_kernel");
    count_launch(h);
}
void launch_bn_normalize(nb_handle_s *h, float *out, const float *mean, const float *var, unsigned channel,
                         unsigned size, unsigned batch) {
    const size_t total = (size_t)channel * size * batch;
    if (!total) return;
    bn_normalize_kernel<<<grid_for(total, h), TPB, 0, h->stream>>>(out, mean, var, channel, size, total);
    check_launch("bn_normalize_kernel");
    count_launch(h);
}
void launch_bn_scale(nb_handle_s *h, float *out, const float *scale, unsigned channel, unsigned size, unsigned batch) {
    const size_t total = (size_t)channel * size * batch;
    if (!total) return;
    bn_scale_kernel<<<grid_for(total, h), TPB, 0, h->stream>>>(out, scale, channel, size, total);
    check_launch("bn_scale_kernel");
    count_launch(h);
}
void launch_softmax(nb_handle_s *h, const float *x, float *y, int rows, int classes) {
    if (rows <= 0 || classes <= 0) return;
    const int threads = classes >= 1024 ? 256 : (classes >= 128 ? 128 : 32);
    softmax_kernel<<<std::min(rows, h->sm_count * 16), threads, 0, h->stream>>>(x, y, rows, classes);
    check_launch("softmax_kernel");
    count_launch(h);
}
void launch_layout(nb_handle_s *h, const float *src, float *dst, int B, int C, int H, int W, bool to_nhwc,
                   bool round) {
    if (!B || !C || !H || !W) return;
    const int HW = H * W;
    const int rows = to_nhwc ? C : HW, cols = to_nhwc ? HW : C;
    for (int b0 = 0; b0 < B; b0 += 65535) {
        const int nb_ = std::min(65535, B - b0);
        dim3 grid((cols + 31) / 32, (rows + 31) / 32, nb_), block(32, 8);
        if (grid.y > 65535) throw Error(NB_ERR_UNSUPPORTED, "layout conversion: extent too large");
        transpose_kernel<<<grid, block, 0, h->stream>>>(src + (size_t)b0 * C * HW, dst + (size_t)b0 * C * HW, rows, cols,
                                                       round ? 1 : 0);
        check_launch("transpose_kernel");
        count_launch(h);
    }
}
void launch_round_tf32(nb_handle_s *h, const float *src, float *dst, size_t n) {
    if (!n) return;
    round_tf32_kernel<<<grid_for(n, h), TPB, 0, h->stream>>>(src, dst, n);
    check_launch("round_tf32_kernel");
    count_launch(h);
}
void launch_split_tf32(nb_handle_s *h, const float *src, float *hi, float *lo, size_t n) {
    if (!n) return;
    split_tf32_kernel<<<grid_for(n, h), TPB, 0, h->stream>>>(src, hi, lo, n);
    check_launch("split_tf32_kernel");
    count_launch(h);
}
void launch_pool(nb_handle_s *h, const nb_pool_desc_t &d, const float *x, float *y, bool round) {
    const int OH = (d.height + 2 * d.padding) / d.stride, OW = (d.width + 2 * d.padding) / d.stride;
    const size_t total = (size_t)d.batch * d.channels * OH * OW;
    if (!total) return;
    const int is_max = d.mode == NB_POOL_MAX;
    if (d.layout == NB_LAYOUT_NHWC && (d.channels % 4) == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0) {
        const size_t t4 = total / 4;
        pool_nhwc4_kernel<<<grid_for(t4, h), TPB, 0, h->stream>>>((const float4 *)x, (float4 *)y, d.batch, d.channels / 4,
                                                                   d.height, d.width, OH, OW, d.size, d.stride, d.padding,
                                                                   is_max, round ? 1 : 0, t4);
    } else if (d.layout == NB_LAYOUT_NHWC) {
        pool_kernel<true><<<grid_for(total, h), TPB, 0, h->stream>>>(x, y, d.batch, d.channels, d.height, d.width, OH, OW,
                                                                      d.size, d.stride, d.padding, is_max, round ? 1 : 0,
                                                                      total);
    } else {
        pool_kernel<false><<<grid_for(total, h), TPB, 0, h->stream>>>(x, y, d.batch, d.channels, d.height, d.width, OH,
                                                                       OW, d.size, d.stride, d.padding, is_max,
                                                                       round ? 1 : 0, total);
    }
    check_launch("pool_kernel");
    count_launch(h);
}
void launch_shortcut(nb_handle_s *h, const nb_shortcut_desc_t &d, const float *prev, const float *conn, float *y,
                     bool round) {
    const size_t total = (size_t)d.batch * d.out_channels * d.out_height * d.out_width;
    if (!total) return;
    const int stride = d.conn_width / d.out_width > 1 ? d.conn_width / d.out_width : 1;
    const int sample = d.out_width / d.conn_width > 1 ? d.out_width / d.conn_width : 1;
    if (d.layout == NB_LAYOUT_NHWC && (d.conn_channels % 4) == 0 && (d.out_channels % 4) == 0 &&
        ((((uintptr_t)prev) | ((uintptr_t)conn) | ((uintptr_t)y)) & 15) == 0)
        shortcut_nhwc4_kernel<<<grid_for(total / 4, h), TPB, 0, h->stream>>>(
            (const float4 *)prev, (const float4 *)conn, (float4 *)y, d.batch, d.conn_channels / 4, d.conn_height, d.conn_width,
            d.out_channels / 4, d.out_height, d.out_width, stride, sample, d.activation, round ? 1 : 0, total / 4);
    else if (d.layout == NB_LAYOUT_NHWC)
        shortcut_kernel<true><<<grid_for(total, h), TPB, 0, h->stream>>>(
            prev, conn, y, d.batch, d.conn_channels, d.conn_height, d.conn_width, d.out_channels, d.out_height,
            d.out_width, stride, sample, d.activation, round ? 1 : 0, total);
    else
        shortcut_kernel<false><<<grid_for(total, h), TPB, 0, h->stream>>>(
            prev, conn, y, d.batch, d.conn_channels, d.conn_height, d.conn_width, d.out_channels, d.out_height,
            d.out_width, stride, sample, d.activation, round ? 1 : 0, total);
    check_launch("shortcut_kernel");
    count_launch(h);
}
void launch_weight_pack(nb_handle_s *h, const float *w, float *dst, int F, int C, int k, int Kpad) {
    const size_t total = (size_t)F * Kpad;
    weight_pack_kernel<<<grid_for(total, h), TPB, 0, h->stream>>>(w, dst, F, C, k, Kpad, total);
    check_launch("weight_pack_kernel");
    count_launch(h);
}
void launch_weight_rowwin(nb_handle_s *h, const float *w, float *dst, int F, int C, int k, int inner) {
    const size_t total = (size_t)k * F * inner;
    weight_rowwin_kernel<<<grid_for(total, h), TPB, 0, h->stream>>>(w, dst, F, C, k, inner, total);
    check_launch("weight_rowwin_kernel");
    count_launch(h);
}
void launch_rowwin_input(nb_handle_s *h, const float *x, float *dst, int N, int C, int H, int W, int Wp, int pad, bool nhwc_in,
                         bool round) {
    const size_t total = (size_t)N * H * Wp;
    rowwin_input_kernel<<<grid_for(total, h), TPB, 0, h->stream>>>(x, reinterpret_cast<float4 *>(dst), N, C, H, W, Wp, pad,
                                                                  nhwc_in ? 1 : 0, round ? 1 : 0, total);
    check_launch("rowwin_input_kernel");
    count_launch(h);
}
void launch_u8_pack(nb_handle_s *h, const unsigned char *img, float *dst, int N, int C, int H, int W, bool rowwin, int Wp,
                    int pad, bool round) {
    const size_t total = rowwin ? (size_t)N * H * Wp : (size_t)N * C * H * W;
    if (!total) return;
    u8_pack_kernel<<<grid_for(total, h), TPB, 0, h->stream>>>(img, dst, N, C, H, W, rowwin ? 1 : 0, Wp, pad, round ? 1 : 0, total);
    check_launch("u8_pack_kernel");
    count_launch(h);
}
void launch_weight_relayout(nb_handle_s *h, const float *w, float *dst, int F, int C, int k, int Cp) {
    const size_t total = (size_t)k * k * F * Cp;
    weight_relayout_kernel<<<grid_for(total, h), TPB, 0, h->stream>>>(w, dst, F, C, k, Cp, total);
    check_launch("weight_relayout_kernel");
    count_launch(h);
}
void launch_fc_permute(nb_handle_s *h, const float *w, float *dst, int out, int C, int H, int W) {
    const size_t total = (size_t)out * C * H * W;
    fc_permute_kernel<<<grid_for(total, h), TPB, 0, h->stream>>>(w, dst, out, C, H * W, total);
    check_launch("fc_permute_kernel");
    count_launch(h);
}
void launch_splitk_reduce(nb_handle_s *h, const float *ws, int S, int M, int N, const float *scale, const float *shift,
                          int act, bool round, float *y) {
    const size_t MN = (size_t)M * N;
    const bool vec = (N % 4) == 0 && ((((uintptr_t)ws) | ((uintptr_t)y) | ((uintptr_t)scale) | ((uintptr_t)shift)) & 15) == 0;
    if (vec)
        splitk_reduce4_kernel<<<grid_for(MN / 4, h), TPB, 0, h->stream>>>((const float4 *)ws, S, MN / 4, N / 4, (const float4 *)scale,
                                                                         (const float4 *)shift, act, round ? 1 : 0, (float4 *)y);
    else
        splitk_reduce_kernel<<<grid_for(MN, h), TPB, 0, h->stream>>>(ws, S, MN, N, scale, shift, act, round ? 1 : 0, y);
    check_launch("splitk_reduce_kernel");
    count_launch(h);
}
void launch_lstm_cell(nb_handle_s *h, const float *z, const float *c_prev, float *c_out, float *h_out, float *h_round,
                      int B, int H) {
    lstm_cell_kernel<<<grid_for((size_t)B * H, h), TPB, 0, h->stream>>>(z, c_prev, c_out, h_out, h_round, B, H);
    check_launch("lstm_cell_kernel");
    count_launch(h);
}

}  // namespace nb
