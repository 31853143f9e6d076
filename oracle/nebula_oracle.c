/* CPU restatement of the reference's forward-inference operators, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker's arithmetic: the
 * tests, the smoke check and the bench's CPU-baseline leg may load it; the
 * product library must never link, load or call it.
 *
 * Every function restates one operator of the reference's CPU path (tensors are
 * NCHW fp32, weights OIHW) and cites the file:line it follows.  Loop orders and
 * float/double promotion follow the reference so that results agree with the
 * reference built with its in-tree GEMM (-DCUSTOM_BLAS) to the last bit where
 * the order of additions is the same, and to fp32 rounding noise against the
 * OpenBLAS build.  Pinned against the compiled reference by
 * tests/test_oracle_pin.py and by the vectors under tests/golden/.
 *
 * Threading: images (or rows) are split over pthreads; the split never changes
 * the order of additions inside one output element.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* activation codes = the reference's activation_type_t (common/def.h:59-75) */
enum {
    NBO_ACT_UNDEFINED = 0, NBO_ACT_ELU, NBO_ACT_HARDTAN, NBO_ACT_LEAKY, NBO_ACT_LHTAN,
    NBO_ACT_LINEAR, NBO_ACT_LOGGY, NBO_ACT_LOGISTIC, NBO_ACT_PLSE, NBO_ACT_RAMP,
    NBO_ACT_RELIE, NBO_ACT_RELU, NBO_ACT_STAIR, NBO_ACT_TANH
};

/* ------------------------------------------------------------------ threads */
typedef void (*nbo_range_fn)(void *ctx, long begin, long end);
typedef struct { nbo_range_fn fn; void *ctx; long begin, end; } nbo_job;
static void *nbo_job_main(void *p) { nbo_job *j = (nbo_job *)p; j->fn(j->ctx, j->begin, j->end); return NULL; }

static int g_threads = 1;
void nbo_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }

/* Splits [0,n) like the reference's fork-join helpers (tid*n/T .. (tid+1)*n/T,
 * common/utils.cc:88-118). */
static void nbo_parallel_for(long n, nbo_range_fn fn, void *ctx) {
    int t = g_threads;
    if (t > n) t = (int)(n > 0 ? n : 1);
    if (t <= 1) { fn(ctx, 0, n); return; }
    pthread_t th[256]; nbo_job jobs[256];
    for (int i = 0; i < t; i++) {
        jobs[i].fn = fn; jobs[i].ctx = ctx;
        jobs[i].begin = (long)i * n / t; jobs[i].end = (long)(i + 1) * n / t;
        pthread_create(&th[i], NULL, nbo_job_main, &jobs[i]);
    }
    for (int i = 0; i < t; i++) pthread_join(th[i], NULL);
}

/* -------------------------------------------------------------- activations */
/* common/activations.cc:6-91.  Constants are doubles in the reference, so the
 * arithmetic is done in double and stored back as float. */
void nbo_activate(float *y, long n, int act) {
    long i;
    switch (act) {
    case NBO_ACT_LINEAR: break;                                   /* activations.cc:32-33 */
    case NBO_ACT_RELU:   for (i = 0; i < n; i++) y[i] = y[i] > 0.0 ? y[i] : 0.0; break;       /* :70-74 */
    case NBO_ACT_LEAKY:  for (i = 0; i < n; i++) y[i] = y[i] > 0.0 ? y[i] : 0.1 * y[i]; break; /* :21-25 */
    case NBO_ACT_RELIE:  for (i = 0; i < n; i++) y[i] = y[i] > 0.0 ? y[i] : 0.01 * y[i]; break; /* :65-69 */
    case NBO_ACT_LOGISTIC: for (i = 0; i < n; i++) y[i] = 1.0 / (1.0 + exp(0.0 - y[i])); break; /* :40-44 */
    case NBO_ACT_LOGGY:  for (i = 0; i < n; i++) y[i] = 2.0 / (1.0 + exp(0.0 - y[i])) - 1.0; break; /* :35-39 */
    case NBO_ACT_TANH:                                            /* :84-89 (NaN for x >~ 355) */
        for (i = 0; i < n; i++) y[i] = (exp(2.0 * y[i]) - 1.0) / (exp(2.0 * y[i]) + 1.0);
        break;
    case NBO_ACT_ELU:                                             /* :6-12 (x*x for x>0, as written) */
        for (i = 0; i < n; i++) y[i] = y[i] > 0.0 ? y[i] * y[i] : y[i] * (exp(y[i]) - 1.0);
        break;
    case NBO_ACT_HARDTAN:                                         /* :14-19 (0/1 indicator) */
        for (i = 0; i < n; i++) y[i] = (y[i] < 1.0 && y[i] > -1.0) ? 1.0f : 0.0f;
        break;
    case NBO_ACT_LHTAN:                                           /* :26-31 */
        for (i = 0; i < n; i++) y[i] = (y[i] > 0.0 && y[i] < 1.0) ? 1.0f : 0.0f;
        break;
    case NBO_ACT_PLSE:                                            /* :45-57 */
        for (i = 0; i < n; i++) {
            if (y[i] < -4.0) y[i] = 0.01 * (y[i] + 4.0);
            else if (y[i] > 4.0) y[i] = 0.01 * (y[i] - 4.0) + 1.0;
            else y[i] = 0.125 * y[i] + 0.5;
        }
        break;
    case NBO_ACT_RAMP:                                            /* :58-64 */
        for (i = 0; i < n; i++) y[i] = y[i] > 0.0 ? y[i] * (y[i] + 0.01) : 0.01 * y[i];
        break;
    case NBO_ACT_STAIR:                                           /* :75-83 */
        for (i = 0; i < n; i++) {
            if ((int)y[i] % 2) y[i] = y[i] - (float)(int)y[i] + (float)(int)(y[i] / 2.0);
            else y[i] = (float)(int)(y[i] / 2.0);
        }
        break;
    default: break;
    }
}

/* -------------------------------------------------------------------- GEMM */
/* common/gemm.h:51-61 (gemm_nn): C[i,j] += (alpha*A[i,k]) * B[k,j], k outer, j inner. */
static void gemm_nn_rows(long r0, long r1, int N, int K, const float *A, int lda,
                         const float *B, int ldb, float *C, int ldc) {
    for (long i = r0; i < r1; i++)
        for (int k = 0; k < K; k++) {
            float a = 1.0f * A[i * lda + k];
            for (int j = 0; j < N; j++) C[i * ldc + j] += a * B[(long)k * ldb + j];
        }
}
/* common/gemm.h:77-89 (gemm_nt): sum over k into a float, then C[i,j] += sum. */
static void gemm_nt_rows(long r0, long r1, int N, int K, const float *A, int lda,
                         const float *B, int ldb, float *C, int ldc) {
    for (long i = r0; i < r1; i++)
        for (int j = 0; j < N; j++) {
            float sum = 0;
            for (int k = 0; k < K; k++) sum += 1.0f * A[i * lda + k] * B[(long)j * ldb + k];
            C[i * ldc + j] += sum;
        }
}

/* ------------------------------------------------------------------ im2col */
/* common/utils.cc:81-119: row i=(c,kh,kw) with kw fastest, column (oh,ow);
 * zero outside the image (the reference tests the wrapped unsigned index). */
static void im2col_image(const float *im, int C, int H, int W, int k, int s, int p, float *col) {
    int OH = (H + 2 * p - k) / s + 1, OW = (W + 2 * p - k) / s + 1;
    int rows = C * k * k;
    for (int i = 0; i < rows; i++) {
        int ow_off = i % k, oh_off = (i / k) % k, c = i / k / k;
        for (int h = 0; h < OH; h++)
            for (int w = 0; w < OW; w++) {
                int r = oh_off + h * s - p, q = ow_off + w * s - p;
                long ci = ((long)i * OH + h) * OW + w;
                col[ci] = (r < 0 || q < 0 || r >= H || q >= W) ? 0.0f : im[q + (long)W * (r + (long)H * c)];
            }
    }
}

/* -------------------------------------------------- bias / batchnorm passes */
/* common/batchnorm.cc:58-97 (normalize with the ROLLING statistics, then
 * scale) and common/utils.cc:162-179 (bias, applied after batchnorm).
 * normalize: (y - mean) is a float subtraction; the divisor sqrt(var)+0.00001
 * is a double; the quotient is stored as float. */
static void bn_bias_image(float *y, int channels, long size, const float *scale,
                          const float *mean, const float *var, const float *bias) {
    if (scale) {
        for (int c = 0; c < channels; c++)
            for (long s = 0; s < size; s++) {
                long idx = (long)c * size + s;
                y[idx] = (y[idx] - mean[c]) / (sqrt(var[c]) + 0.00001);
            }
        for (int c = 0; c < channels; c++)
            for (long s = 0; s < size; s++) y[(long)c * size + s] *= scale[c];
    }
    for (int c = 0; c < channels; c++)
        for (long s = 0; s < size; s++) y[(long)c * size + s] += bias[c];
}

/* ------------------------------------------------------------- convolution */
typedef struct {
    const float *x, *w, *bias, *scale, *mean, *var; float *y;
    int B, C, H, W, F, k, s, p, act;
} conv_ctx;

static void conv_range(void *vp, long b0, long b1) {
    conv_ctx *c = (conv_ctx *)vp;
    int OH = (c->H + 2 * c->p - c->k) / c->s + 1, OW = (c->W + 2 * c->p - c->k) / c->s + 1;
    int K = c->C * c->k * c->k; long N = (long)OH * OW;
    float *col = (float *)malloc(sizeof(float) * (size_t)K * N);
    for (long b = b0; b < b1; b++) {
        float *yb = c->y + b * c->F * N;
        memset(yb, 0, sizeof(float) * c->F * N);
        im2col_image(c->x + b * (long)c->C * c->H * c->W, c->C, c->H, c->W, c->k, c->s, c->p, col);
        gemm_nn_rows(0, c->F, (int)N, K, c->w, K, col, (int)N, yb, (int)N);
        bn_bias_image(yb, c->F, N, c->scale, c->mean, c->var, c->bias);
        nbo_activate(yb, c->F * N, c->act);
    }
    free(col);
}

/* models/layers/convolutional_layer.cc:365-409: per image im2col + SGEMM
 * (M=F, N=OH*OW, K=C*k*k, beta=1 onto zeroed output), then inference batchnorm
 * (:502-536, only if scale != NULL), bias, activation.  Output extents follow
 * :150-153. */
void nbo_conv_forward(const float *x, int B, int C, int H, int W, int F, int k, int s, int p,
                      const float *w, const float *bias, const float *scale, const float *mean,
                      const float *var, int act, float *y) {
    conv_ctx c = { x, w, bias, scale, mean, var, y, B, C, H, W, F, k, s, p, act };
    nbo_parallel_for(B, conv_range, &c);
}

/* --------------------------------------------------------- connected layer */
typedef struct {
    const float *x, *w, *bias, *scale, *mean, *var; float *y; int B, in, out, act;
} fc_ctx;
static void fc_range(void *vp, long b0, long b1) {
    fc_ctx *c = (fc_ctx *)vp;
    memset(c->y + b0 * c->out, 0, sizeof(float) * (b1 - b0) * c->out);
    gemm_nt_rows(b0, b1, c->out, c->in, c->x, c->in, c->w, c->in, c->y, c->out);
    for (long b = b0; b < b1; b++) {
        /* batchnorm/bias with channel=out, size=1 (connected_layer.cc:273, :462-492) */
        bn_bias_image(c->y + b * c->out, c->out, 1, c->scale, c->mean, c->var, c->bias);
        nbo_activate(c->y + b * c->out, c->out, c->act);
    }
}
/* models/layers/connected_layer.cc:245-277: Y[B,out] = act(BN?(X[B,in] * W[out,in]^T) + bias). */
void nbo_connected_forward(const float *x, int B, int in, int out, const float *w, const float *bias,
                           const float *scale, const float *mean, const float *var, int act, float *y) {
    fc_ctx c = { x, w, bias, scale, mean, var, y, B, in, out, act };
    nbo_parallel_for(B, fc_range, &c);
}

/* ------------------------------------------------------------------ pooling */
/* models/layers/pooling_layer.cc:40-63 output rule: OH = (H + 2p) / stride. */
typedef struct { const float *x; float *y; int B, C, H, W, k, s, p, is_max; } pool_ctx;
static void pool_range(void *vp, long b0, long b1) {
    pool_ctx *c = (pool_ctx *)vp;
    int OH = (c->H + 2 * c->p) / c->s, OW = (c->W + 2 * c->p) / c->s;
    for (long b = b0; b < b1; b++)
        for (int ch = 0; ch < c->C; ch++)
            for (int h = 0; h < OH; h++)
                for (int w = 0; w < OW; w++) {
                    const float *xp = c->x + (b * c->C + ch) * (long)c->H * c->W;
                    float mx = -1e8; float sum = 0.0;
                    for (int i = 0; i < c->k; i++)
                        for (int j = 0; j < c->k; j++) {
                            int r = h * c->s + i - c->p, q = w * c->s + j - c->p;
                            int valid = r >= 0 && r < c->H && q >= 0 && q < c->W;
                            if (c->is_max) {            /* pooling_layer.cc:117-146, identity -1e8 */
                                float v = valid ? xp[(long)r * c->W + q] : -1e8;
                                mx = v > mx ? v : mx;
                            } else {                    /* :150-176, divisor k*k incl. padding */
                                sum += valid ? xp[(long)r * c->W + q] : 0.0;
                            }
                        }
                    long oi = w + (long)OW * (h + (long)OH * (ch + (long)c->C * b));
                    c->y[oi] = c->is_max ? mx : sum / (c->k * c->k);
                }
}
void nbo_pool_forward(const float *x, int B, int C, int H, int W, int k, int s, int p, int is_max, float *y) {
    pool_ctx c = { x, y, B, C, H, W, k, s, p, is_max };
    nbo_parallel_for(B, pool_range, &c);
}

/* ----------------------------------------------------------------- shortcut */
/* models/layers/shortcut_layer.cc:68-79 + common/utils.cc:28-60: out = prev;
 * out[b,c,h*sample,w*sample] += conn[b,c,h*stride,w*stride] over the min
 * extents; then the activation.  "in" is the connection (hops back), "out"
 * has the previous layer's shape. */
void nbo_shortcut_forward(const float *prev, const float *conn, int B, int Cin, int Hin, int Win,
                          int Cout, int Hout, int Wout, int act, float *y) {
    long on = (long)B * Cout * Hout * Wout;
    memcpy(y, prev, sizeof(float) * on);
    int stride = Win / Wout > 1 ? Win / Wout : 1;
    int sample = Wout / Win > 1 ? Wout / Win : 1;
    int W = Win < Wout ? Win : Wout, H = Hin < Hout ? Hin : Hout, C = Cin < Cout ? Cin : Cout;
    for (int b = 0; b < B; b++)
        for (int c = 0; c < C; c++)
            for (int h = 0; h < H; h++)
                for (int w = 0; w < W; w++) {
                    long oi = w * sample + (long)Wout * (h * sample + (long)Hout * (c + (long)Cout * b));
                    long ii = w * stride + (long)Win * (h * stride + (long)Hin * (c + (long)Cin * b));
                    y[oi] += conn[ii];
                }
    nbo_activate(y, on, act);
}

/* ------------------------------------------------------------------ softmax */
/* models/layers/softmax_layer.cc:85-106: row max, exp(x-max) (double exp of a
 * float difference, stored as float), float sum, divide. */
void nbo_softmax_forward(const float *x, int B, int n, float *y) {
    for (int b = 0; b < B; b++) {
        const float *in = x + (long)b * n; float *out = y + (long)b * n;
        float sum = 0.0, mx = -3.402823466e+38F;
        for (int j = 0; j < n; j++) if (in[j] > mx) mx = in[j];
        for (int j = 0; j < n; j++) { float e = exp(in[j] - mx); sum += e; out[j] = e; }
        for (int j = 0; j < n; j++) out[j] /= sum;
    }
}

/* --------------------------------------------------------------------- LSTM */
/* models/layers/lstm_layer.cc:233-346.  x is time-major [T,B,in]; out and
 * cell are [T,B,H]; h0 = c0 = 0 (first call on a fresh layer).  Each gate is
 * the sum of two connected layers, W on h_{t-1} and U on x_t, each applying its
 * own (optional) batchnorm, bias and the section's activation
 * (connected_layer.cc:279-313).  Weight blobs come in the weight-file order
 * iW,fW,oW,cW,iU,fU,oU,cU (lstm_layer.cc:194-206); each blob is
 * {bias[H], weight[H*in_g], and iff bn: scale[H], mean[H], var[H]}.
 * Gate maths (:286-311): i,f,o = logistic, g = tanh, c_t = f*c_{t-1} + i*g,
 * h_t = o*tanh(c_t); products follow the reference's axmy (common/gemm.h:28-34,
 * Y *= alpha*X with alpha a float 1.0). */
typedef struct { const float *bias, *w, *scale, *mean, *var; } nbo_fc_blob;

void nbo_lstm_forward(const float *x, int T, int B, int in, int H, const nbo_fc_blob *blobs /*8*/,
                      int has_bn, int act, float *out, float *cell) {
    long n = (long)B * H;
    float *hid = (float *)calloc(n, sizeof(float));
    float *gw[4], *gu[4];
    for (int g = 0; g < 4; g++) { gw[g] = (float *)malloc(sizeof(float) * n); gu[g] = (float *)malloc(sizeof(float) * n); }
    /* forward order of gates: i, f, c(g), o; blob order: i, f, o, c */
    static const int blob_of_gate[4] = { 0, 1, 3, 2 };
    for (int t = 0; t < T; t++) {
        for (int g = 0; g < 4; g++) {
            const nbo_fc_blob *bw = &blobs[blob_of_gate[g]], *bu = &blobs[4 + blob_of_gate[g]];
            nbo_connected_forward(hid, B, H, H, bw->w, bw->bias, has_bn ? bw->scale : NULL, bw->mean, bw->var, act, gw[g]);
            nbo_connected_forward(x + (long)t * B * in, B, in, H, bu->w, bu->bias, has_bn ? bu->scale : NULL, bu->mean, bu->var, act, gu[g]);
            for (long i = 0; i < n; i++) gu[g][i] += 1.0f * gw[g][i];          /* saxpy, :279-282 */
        }
        float *ig = gu[0], *fg = gu[1], *cg = gu[2], *og = gu[3];
        nbo_activate(ig, n, NBO_ACT_LOGISTIC);
        nbo_activate(fg, n, NBO_ACT_LOGISTIC);
        nbo_activate(og, n, NBO_ACT_LOGISTIC);
        nbo_activate(cg, n, NBO_ACT_TANH);
        float *ct = cell + (long)t * n;
        for (long i = 0; i < n; i++) ig[i] *= 1.0f * cg[i];                     /* :291 */
        if (t) memcpy(ct, ct - n, sizeof(float) * n); else memset(ct, 0, sizeof(float) * n);
        for (long i = 0; i < n; i++) ct[i] *= 1.0f * fg[i];                     /* :298 */
        for (long i = 0; i < n; i++) ct[i] += 1.0f * ig[i];                     /* :300-303 */
        memcpy(hid, ct, sizeof(float) * n);
        nbo_activate(hid, n, NBO_ACT_TANH);
        for (long i = 0; i < n; i++) hid[i] *= 1.0f * og[i];                    /* :308 */
        memcpy(out + (long)t * n, hid, sizeof(float) * n);
    }
    for (int g = 0; g < 4; g++) { free(gw[g]); free(gu[g]); }
    free(hid);
}

/* ------------------------------------------------------------------- RNN
 * rnn_layer_t::forward (rnn_layer.cc:91-141).  Three connected layers built from
 * one section: input gate (on x_t), hidden gate (on the state), output gate.
 * state_t = in(x_t) + hid(.) by two saxpys onto a zeroed buffer (:107-115).  At
 * step 0 the gates run forward() without an argument, i.e. on their predecessor's
 * output (:100-101,116-117): the hidden gate reads the input gate's output and
 * the output gate reads the hidden gate's output; from step 1 on both read the
 * state.  blobs: input, hidden, output gate.  x [T,B,in], out [T,B,H]. */
void nbo_rnn_forward(const float *x, int T, int B, int in, int H, const nbo_fc_blob *blobs /*3*/, int has_bn, int act,
                     float *out) {
    long n = (long)B * H;
    float *a = (float *)malloc(sizeof(float) * n), *hd = (float *)malloc(sizeof(float) * n);
    float *state = (float *)calloc(n, sizeof(float));
    const nbo_fc_blob *bi = &blobs[0], *bh = &blobs[1], *bo = &blobs[2];
    for (int t = 0; t < T; t++) {
        nbo_connected_forward(x + (long)t * B * in, B, in, H, bi->w, bi->bias, has_bn ? bi->scale : NULL, bi->mean, bi->var, act, a);
        nbo_connected_forward(t ? state : a, B, H, H, bh->w, bh->bias, has_bn ? bh->scale : NULL, bh->mean, bh->var, act, hd);
        memset(state, 0, sizeof(float) * n);
        for (long i = 0; i < n; i++) state[i] += 1.0f * a[i];
        for (long i = 0; i < n; i++) state[i] += 1.0f * hd[i];
        nbo_connected_forward(t ? state : hd, B, H, H, bo->w, bo->bias, has_bn ? bo->scale : NULL, bo->mean, bo->var, act,
                              out + (long)t * n);
    }
    free(a); free(hd); free(state);
}

/* ------------------------------------------------------------------ GEMM
 * gemm<T> of the operator library (common/gemm.h:51-147), row-major with leading
 * dimensions: C *= beta, then one of four loop nests by transpose flags -- nn and
 * tn accumulate a_p * B[k][j] into C directly (a_p = alpha * A), nt and tt form
 * sum += alpha * A * B in a float and add it to C once.  The reference splits the
 * rows of C over threads; rows are independent, so one thread gives the same bits. */
void nbo_gemm(int TA, int TB, int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb,
              float beta, float *C, int ldc) {
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) C[(long)i * ldc + j] *= beta;
    for (int i = 0; i < M; i++) {
        if (!TB) {
            for (int k = 0; k < K; k++) {
                float a_p = alpha * (TA ? A[(long)k * lda + i] : A[(long)i * lda + k]);
                for (int j = 0; j < N; j++) C[(long)i * ldc + j] += a_p * B[(long)k * ldb + j];
            }
        } else {
            for (int j = 0; j < N; j++) {
                float sum = 0;
                for (int k = 0; k < K; k++)
                    sum += alpha * (TA ? A[(long)k * lda + i] : A[(long)i * lda + k]) * B[(long)j * ldb + k];
                C[(long)i * ldc + j] += sum;
            }
        }
    }
}
