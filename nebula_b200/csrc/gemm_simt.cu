// CUDA-core fp32 GEMM / implicit-GEMM convolution (NB_MATH_FP32, and the path for
// operands the tensor-core kernel cannot take: channel counts that are not a
// multiple of 4 such as the 3-channel input layer, unaligned pointers).
//
// Same contract as the tensor-core kernel: D[M,N] = A[M,K] * B[N,K]^T with A an
// implicit im2col view (row = output pixel, column = (kh,kw,c)) gathered through
// arbitrary element strides, so an NCHW network input is read in place.  Exact
// fp32 products, fp32 FMA accumulation.  Replaces the same reference code as the
// tensor-core kernel (models/layers/convolutional_layer.cu:47-70,
// models/layers/connected_layer.cu:21-38).
#include "device_math.cuh"
#include "nb_internal.h"

namespace nb {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct SimtParams {
    const float *a, *b;
    ConvGeom g;
    long ldb;
    int M, N, Kc, taps;
    const float *scale, *shift, *addend;
    long ld_addend;
    int act, round_out, addend_post;
    float *y;
    long ldy;
};

__global__ void __launch_bounds__(256) gemm_fp32_simt_kernel(const SimtParams p) {
    __shared__ float As[TK][TM + 1];
    __shared__ float Bs[TK][TN + 1];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const long m0 = (long)blockIdx.x * TM;
    const int n0 = blockIdx.y * TN;

    // the A/B element this thread stages: row (tid/4), four consecutive k
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    const long am = m0 + lrow;
    const bool a_row_ok = am < p.M;
    int an = 0, aoh = 0, aow = 0;
    if (a_row_ok) {
        const long per = (long)p.g.OH * p.g.OW;
        an = (int)(am / per);
        const int rem = (int)(am - (long)an * per);
        aoh = rem / p.g.OW;
        aow = rem - aoh * p.g.OW;
    }
    const int bn_ = n0 + lrow;
    const bool b_row_ok = bn_ < p.N;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (int tap = 0; tap < p.taps; tap++) {
        const int kh = tap / p.g.ksize, kw = tap - kh * p.g.ksize;
        const int ih = aoh * p.g.stride + kh - p.g.pad, iw = aow * p.g.stride + kw - p.g.pad;
        const bool pix_ok = a_row_ok && ih >= 0 && ih < p.g.H && iw >= 0 && iw < p.g.W;
        const float *ap = p.a + (long)an * p.g.sn + (long)ih * p.g.sh + (long)iw * p.g.sw;
        const float *bp = p.b + ((long)tap * p.N + bn_) * p.ldb;
        for (int c0 = 0; c0 < p.Kc; c0 += TK) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int c = c0 + lk + e;
                As[lk + e][lrow] = (pix_ok && c < p.Kc) ? ap[(long)c * p.g.sc] : 0.0f;
                Bs[lk + e][lrow] = (b_row_ok && c < p.Kc) ? bp[c] : 0.0f;
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < TK; k++) {
                float av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) av[i] = As[k][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; j++) bv[j] = Bs[k][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
            }
            __syncthreads();
        }
    }

#pragma unroll
    for (int i = 0; i < 4; i++) {
        const long m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            float x = acc[i][j];
            if (p.scale) x *= p.scale[n];
            if (p.shift) x += p.shift[n];
            if (p.addend && !p.addend_post) x += p.addend[m * p.ld_addend + n];
            x = apply_activation_fast(x, p.act);
            if (p.addend && p.addend_post) x += p.addend[m * p.ld_addend + n];
            p.y[m * p.ldy + n] = p.round_out ? round_tf32(x) : x;
        }
    }
}

}  // namespace

void gemm_simt(nb_handle_s *h, const GemmArgs &a) {
    if (a.addend && a.res_stride > 0) throw Error(NB_ERR_UNSUPPORTED, "the CUDA-core path takes no fused residual");
    SimtParams p;
    p.a = a.a; p.b = a.b;
    if (a.a_is_conv) {
        p.g = a.g;
    } else {
        p.g = ConvGeom();
        p.g.batch = 1; p.g.C = a.Kc; p.g.H = 1; p.g.W = a.M; p.g.OH = 1; p.g.OW = a.M;
        p.g.sc = 1; p.g.sw = a.lda; p.g.sh = 0; p.g.sn = 0;
    }
    p.ldb = a.ldb; p.M = a.M; p.N = a.N; p.Kc = a.Kc; p.taps = p.g.ksize * p.g.ksize;
    p.scale = a.scale; p.shift = a.shift; p.addend = a.addend; p.ld_addend = a.ld_addend;
    p.act = a.act; p.round_out = a.round_out_tf32 ? 1 : 0; p.addend_post = a.addend_after_act ? 1 : 0;
    p.y = a.y; p.ldy = a.ldy;
    ProfileScope prof(h, 1, 2.0 * (double)a.M * a.N * a.Kc * p.taps);
    dim3 grid((unsigned)((a.M + TM - 1) / TM), (unsigned)((a.N + TN - 1) / TN));
    gemm_fp32_simt_kernel<<<grid, 256, 0, h->stream>>>(p);
    check_launch("gemm_fp32_simt_kernel");
    count_launch(h);
    prof.finish();
}

void gemm(nb_handle_s *h, const GemmArgs &a) {
    if (h->math_mode != NB_MATH_FP32 && gemm_tc_supported(h, a)) {
        gemm_tc(h, a, h->math_mode == NB_MATH_TF32X3);
    } else {
        gemm_simt(h, a);
    }
}

}  // namespace nb
