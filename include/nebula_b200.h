/* nebula_b200 -- C ABI of the B200 (sm_100a) forward-inference backend for Nebula.
 *
 * Every entry point replaces one piece of the reference's GPU path behind the
 * reference's own layer contract (models/layers/layer.h:11-85): a layer's
 * init() creates a plan, init_weight() uploads weights in weight-file layout,
 * _forward_() calls nb_*_forward with the layer's own device buffers.  Tensors
 * are fp32; activations are NCHW (the reference's layout) unless a descriptor
 * says NB_LAYOUT_NHWC, which the network executor uses internally.
 *
 * Conventions: all functions return an nb_status; nothing throws or exits;
 * nb_last_error() returns a message for the most recent failure on a handle.
 * One handle per host thread and GPU; calls on a handle are not concurrent.
 * Kernels are launched on the handle's stream (default: the legacy default
 * stream, as the reference does, models/networks/network.cc:44-47).
 */
#ifndef NEBULA_B200_H
#define NEBULA_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nb_handle_s *nb_handle_t;
typedef struct nb_plan_s *nb_plan_t;
typedef struct nb_network_s *nb_network_t;

typedef enum {
    NB_OK = 0,
    NB_ERR_INVALID_ARG = 1,     /* bad pointer, extent, alignment or enum */
    NB_ERR_CUDA = 2,            /* a CUDA runtime/driver call failed */
    NB_ERR_UNSUPPORTED = 3,     /* valid request this backend does not implement */
    NB_ERR_WEIGHTS = 4,         /* weight stream shorter/longer than the network needs */
    NB_ERR_CONFIG = 5,          /* network.cfg text could not be interpreted */
    NB_ERR_DEVICE_TIMEOUT = 6,  /* a bounded device-side wait gave up */
    NB_ERR_NO_WEIGHTS = 7       /* forward called before weights were set */
} nb_status;

/* Arithmetic of the dense contractions.  TF32: operands rounded to TF32
 * (round-to-nearest), fp32 accumulate, on tcgen05 tensor cores.  TF32X3: each
 * operand split into two TF32 terms, three tensor-core products, fp32-level
 * agreement.  FP32: CUDA-core fp32 FMA kernel (exact fp32 products). */
typedef enum { NB_MATH_TF32 = 0, NB_MATH_TF32X3 = 1, NB_MATH_FP32 = 2 } nb_math_mode;

/* Same codes as the reference's activation_type_t (common/def.h:59-75). */
typedef enum {
    NB_ACT_UNDEFINED = 0, NB_ACT_ELU, NB_ACT_HARDTAN, NB_ACT_LEAKY, NB_ACT_LHTAN, NB_ACT_LINEAR,
    NB_ACT_LOGGY, NB_ACT_LOGISTIC, NB_ACT_PLSE, NB_ACT_RAMP, NB_ACT_RELIE, NB_ACT_RELU,
    NB_ACT_STAIR, NB_ACT_TANH, NB_ACT_COUNT
} nb_activation;

typedef enum { NB_LAYOUT_NCHW = 0, NB_LAYOUT_NHWC = 1 } nb_layout;
typedef enum { NB_POOL_MAX = 0, NB_POOL_AVG = 1 } nb_pool_mode;
typedef enum { NB_MEM_HOST = 0, NB_MEM_DEVICE = 1 } nb_mem;

/* ------------------------------------------------------------------ handle */
/* Replaces network_t's constructor-time device set-up (cudaSetDevice(0) +
 * cublasCreate, models/networks/network.cc:44-51); device_id makes it rank-aware. */
int nb_create(int device_id, nb_handle_t *handle);
int nb_destroy(nb_handle_t handle);
const char *nb_last_error(nb_handle_t handle);
/* stream is a cudaStream_t; NULL selects the legacy default stream. */
int nb_set_stream(nb_handle_t handle, void *stream);
int nb_set_math_mode(nb_handle_t handle, int mode);
int nb_get_math_mode(nb_handle_t handle, int *mode);
/* Synchronises the handle's stream and reports NB_ERR_DEVICE_TIMEOUT if any
 * kernel's bounded wait gave up since the last call (no reference counterpart:
 * the reference never reads a CUDA status). */
int nb_synchronize(nb_handle_t handle);
/* Number of kernels this library has launched on the handle so far. */
int nb_launch_count(nb_handle_t handle, unsigned long long *count);

/* Per-kernel timing of the contraction kernels with CUDA events on the handle's
 * stream (no reference counterpart: the reference times whole iterations with
 * gettimeofday, common/stopwatch.cc:15-28).  Between begin and end every launch
 * of the tensor-core kernel and of the CUDA-core contraction kernel is bracketed
 * by an event pair; end synchronises and returns the summed device time and the
 * algorithmic FLOPs (2*M*N*K) of those launches. */
typedef struct {
    double tc_ms, tc_flops;
    unsigned long long tc_launches;
    double simt_ms, simt_flops;
    unsigned long long simt_launches;
    double halo_ms, halo_flops;             /* the 3x3 halo convolution kernel (few input channels) */
    unsigned long long halo_launches;
} nb_profile_t;
int nb_profile_begin(nb_handle_t handle);
int nb_profile_end(nb_handle_t handle, nb_profile_t *result);

/* ------------------------------------------------------------- convolution */
/* Extents as read from a [convolutional] section (convolutional_layer.cc:119-153). */
typedef struct {
    int batch, channels, height, width;     /* input [B,C,H,W] */
    int filters, size, stride, padding;
    int batch_normalize;                    /* 0/1: weights carry scale, rolling mean/variance */
    int activation;                         /* nb_activation */
    int layout;                             /* nb_layout of x and y */
} nb_conv2d_desc_t;

/* init(): replaces the buffer set-up of convolutional_layer_t::init (convolutional_layer.cc:119-254). */
int nb_conv2d_plan_create(nb_handle_t handle, const nb_conv2d_desc_t *desc, nb_plan_t *plan);
/* init_weight(): replaces the cudaMemcpy block of convolutional_layer_t::init_weight
 * (convolutional_layer.cc:257-332).  weight is OIHW [F,C,k,k]; bias [F]; the three
 * batch-norm vectors [F] are read only when batch_normalize=1. */
int nb_conv2d_set_weights(nb_plan_t plan, const float *weight, const float *bias, const float *bn_scale,
                          const float *bn_rolling_mean, const float *bn_rolling_variance, int mem);
/* _forward_(): replaces convolutional_layer_t::_forward_ (convolutional_layer.cu:11-84):
 * y = act(BN(W * x) + bias) with the CPU path's batch-norm formula
 * (common/batchnorm.cc:58-97).  x, y are device pointers. */
int nb_conv2d_forward(nb_plan_t plan, const float *x, float *y);
/* The same forward with the layers that follow it folded into its epilogue (NB_LAYOUT_NHWC plans on the
 * tensor-core paths only; anything else returns NB_ERR_UNSUPPORTED):
 *   residual != NULL: the [shortcut] layer that follows (shortcut_layer.cu:27-52, sampling rule of
 *     common/utils.cc:28-60 with sample == 1): y = res_activation(conv(x) + residual), residual being the NHWC tensor
 *     [B, res_height, res_width, res_channels] of the connected layer; the plan's own activation must be linear;
 *   pool_out != NULL: the 2x2 stride-2 [maxpool] that follows (pooling_layer.cu:150-175): only the pooled NHWC
 *     tensor [B, OH/2, OW/2, F] is written, y is ignored and may be NULL.
 * One of the two at most. */
typedef struct {
    const float *residual;
    int res_channels, res_height, res_width, res_activation;
    float *pool_out;
} nb_conv2d_fusion_t;
int nb_conv2d_forward_fused(nb_plan_t plan, const float *x, float *y, const nb_conv2d_fusion_t *fusion);
/* Output extents {C,H,W} of any plan. */
int nb_plan_output_dims(nb_plan_t plan, int dims[3]);
/* Scratch memory (the reference's per-layer `workspace`, convolutional_layer.cc:152-153,187): a plan's forward
 * needs device scratch for layout changes, TF32-rounded operand copies and split-K partial sums.
 * nb_plan_prepare allocates it now, for the handle's current math mode, so that the forward calls that follow
 * allocate nothing; nb_workspace_size returns the bytes of scratch the plan holds (after prepare or a forward:
 * what this plan needs). */
int nb_plan_prepare(nb_plan_t plan);
size_t nb_workspace_size(nb_plan_t plan);
int nb_plan_destroy(nb_plan_t plan);

/* --------------------------------------------------------- connected layer */
typedef struct {
    int batch, inputs, outputs;
    int batch_normalize, activation;
} nb_fc_desc_t;
/* connected_layer_t::init / init_weight / _forward_ (connected_layer.cc:98-199,
 * connected_layer.cu:10-48).  weight [out,in] row-major, bias [out] added per
 * output as on the CPU path (connected_layer.cc:273). */
int nb_fc_plan_create(nb_handle_t handle, const nb_fc_desc_t *desc, nb_plan_t *plan);
int nb_fc_set_weights(nb_plan_t plan, const float *weight, const float *bias, const float *bn_scale,
                      const float *bn_rolling_mean, const float *bn_rolling_variance, int mem);
/* x [B,in] (the previous layer's buffer read flat), y [B,out]; device pointers.
 * Also serves connected_layer_t::_forward_(float*) (connected_layer.cu:50-88). */
int nb_fc_forward(nb_plan_t plan, const float *x, float *y);

/* Connected-layer forward that allocates nothing (no counterpart in the
 * reference).  For callers that must not allocate device memory while running:
 * a serving loop whose device memory all belongs to another allocator, or a phase
 * where cudaMalloc's device-wide synchronisation (or its failure) is unacceptable.
 * y[batch,outputs] = act(x[batch,inputs] * weight[outputs,inputs]^T + bias); all
 * pointers are device pointers, no batch-norm.  Working copies (TF32-rounded
 * operands, or the 3xTF32 weight split) live in a 16 MiB array built into the
 * library: batch*inputs + outputs*inputs + outputs floats (batch*inputs + 2*outputs*inputs
 * + outputs for 3xTF32) plus 256*inputs + 32 floats of headroom behind the weights must fit
 * in 4 Mi floats, else NB_ERR_INVALID_ARG.  The first call on a device looks
 * the array's device address up and should be made before any stream capture
 * begins.  All calls share the array: calls that overlap on the GPU race. */
int nb_fc_forward_static(nb_handle_t handle, const float *x, const float *weight, const float *bias, int batch,
                         int inputs, int outputs, int activation, float *y);

/* ------------------------------------------------------------------ pooling */
/* pooling_layer_t::init / _forward_ (pooling_layer.cc:40-63, pooling_layer.cu:150-175),
 * output extent (H+2p)/stride, max identity -1e8, average divisor size*size. */
typedef struct {
    int batch, channels, height, width;
    int size, stride, padding;
    int mode;                               /* nb_pool_mode */
    int layout;
} nb_pool_desc_t;
int nb_pool_forward(nb_handle_t handle, const nb_pool_desc_t *desc, const float *x, float *y);

/* ----------------------------------------------------------------- shortcut */
/* shortcut_layer_t::_forward_ (shortcut_layer.cu:27-52) with the CPU path's
 * sampling rule (common/utils.cc:28-60): y = prev; y[b,c,h*sample,w*sample] +=
 * conn[b,c,h*stride,w*stride] over the min extents; then the activation. */
typedef struct {
    int batch;
    int conn_channels, conn_height, conn_width;     /* the layer `hops` back */
    int out_channels, out_height, out_width;        /* the previous layer */
    int activation, layout;
} nb_shortcut_desc_t;
int nb_shortcut_forward(nb_handle_t handle, const nb_shortcut_desc_t *desc, const float *prev,
                        const float *conn, float *y);

/* --------------------------------------------------------------------- LSTM */
/* lstm_layer_t::init / init_weight / forward (lstm_layer.cc:84-142,194-206,233-346;
 * the CPU path is canonical).  x [T,B,in] and out [T,B,H] are time-major; h0=c0=0.
 * weights: the eight connected blobs in weight-file order iW,fW,oW,cW,iU,fU,oU,cU,
 * each {bias[H], weight[H*in_g], (scale,mean,var)[H] iff batch_normalize}. */
typedef struct {
    int time_steps, batch, inputs, hidden;
    int batch_normalize, activation;        /* section activation of the eight gate layers (shipped cfgs: linear) */
} nb_lstm_desc_t;
int nb_lstm_plan_create(nb_handle_t handle, const nb_lstm_desc_t *desc, nb_plan_t *plan);
int nb_lstm_set_weights(nb_plan_t plan, const float *blob_stream, size_t count, int mem);
/* cell may be NULL; otherwise it receives c_t for every step, [T,B,H]. */
int nb_lstm_forward(nb_plan_t plan, const float *x, float *out, float *cell);

/* ---------------------------------------------------------------------- RNN */
/* rnn_layer_t::init / init_weight / forward (rnn_layer.cc:34-141): input, hidden and output gate are three
 * connected layers built from one section.  Per step: a_t = in(x_t); h_t = hid(t ? s_{t-1} : a_0);
 * s_t = a_t + h_t; out_t = outg(t ? s_t : h_0).  x [T,B,in], out [T,B,H] time-major.  weights: the three
 * connected blobs in weight-file order input, hidden, output gate. */
typedef struct {
    int time_steps, batch, inputs, hidden;
    int batch_normalize, activation;
} nb_rnn_desc_t;
int nb_rnn_plan_create(nb_handle_t handle, const nb_rnn_desc_t *desc, nb_plan_t *plan);
int nb_rnn_set_weights(nb_plan_t plan, const float *blob_stream, size_t count, int mem);
int nb_rnn_forward(nb_plan_t plan, const float *x, float *out);

/* ------------------------------------------------------- operator library */
/* _<name>_activation_(out, n) (common/activations.h:38-50), in place. */
int nb_activation_forward(nb_handle_t handle, int activation, float *data, size_t n);
/* _forward_bias_ (common/utils.h:55-56): y[b,c,s] += bias[c]. */
int nb_forward_bias(nb_handle_t handle, float *out, const float *bias, unsigned channel, unsigned size,
                    unsigned batch);
/* _batchnorm_normalize_ / _batchnorm_scale_down_ (common/batchnorm.h:31-33), CPU formula. */
int nb_batchnorm_normalize(nb_handle_t handle, float *out, const float *mean, const float *variance,
                           unsigned channel, unsigned size, unsigned batch);
int nb_batchnorm_scale_down(nb_handle_t handle, float *out, const float *scale, unsigned channel,
                            unsigned size, unsigned batch);
/* softmax_layer_t::_forward_ (softmax_layer.cu:30-40): per-row softmax of x [rows,classes]. */
int nb_softmax_forward(nb_handle_t handle, const float *x, float *y, int rows, int classes);
/* _gemm_(TA,TB,M,N,K,alpha,A,lda,B,ldb,beta,C,ldc) (common/gemm.h:21-25), row-major. */
int nb_gemm(nb_handle_t handle, int TA, int TB, int M, int N, int K, float alpha, const float *A, int lda,
            const float *B, int ldb, float beta, float *C, int ldc);
/* NCHW <-> NHWC copies of a [B,C,H,W] tensor (no reference counterpart). */
int nb_layout_convert(nb_handle_t handle, const float *src, float *dst, int batch, int channels, int height,
                      int width, int src_layout);

/* ------------------------------------------------------------------ network */
/* network_t::init / forward (models/networks/network.cc:57-63,82-122) for the
 * cfg files the reference's convolutional_t, recurrent_t and fully_connected_t accept
 * (convolutional.cc:52-122, recurrent.cc:116-176, fully_connected.cc:52-120; an [rbm] section runs
 * rbm_layer_t::forward, rbm_layer.cc:345-374).  cfg_text is the content of a
 * network.cfg; batch_override > 0 replaces [net] batch (the per-GPU shard).
 * `cost` sections are parsed and skipped at inference. */
int nb_network_create(nb_handle_t handle, const char *cfg_text, int batch_override, nb_network_t *net);
/* network_t::init_weight (network.cc:99-122): a headerless fp32 stream in layer
 * order.  Unlike the reference the length is checked (NB_ERR_WEIGHTS). */
int nb_network_load_weights(nb_network_t net, const float *stream, size_t count, int mem);
int nb_network_load_weight_file(nb_network_t net, const char *path);
size_t nb_network_weight_count(nb_network_t net);
/* One pass of network_t::forward over a device-resident batch: NCHW
 * [B,C,H,W], or time-major [T,B,in] for a recurrent cfg. */
int nb_network_forward(nb_network_t net, const float *input);
/* Same pass from a host batch: copies it in, runs, and copies the network
 * output (see nb_network_output) back; the call returns with `output` filled. */
int nb_network_forward_host(nb_network_t net, const float *input_host, float *output_host);

/* The hand-off the reference does in load_data (models/networks/convolutional.cc:263-423) and print_results:
 * a batch of decoded images goes to the device and the probabilities come back.  Pipelined: submit returns once the
 * work is queued; the copy of batch i+1 (on a copy stream of the network's own, into the second of two device input
 * buffers) overlaps the forward pass of batch i.  At most two submissions may be outstanding: the third waits for
 * the first.  input_host and output_host must stay valid (and should be page-locked) until nb_network_wait returns.
 *   nb_network_submit_host: an fp32 batch as nb_network_forward takes it.
 *   nb_network_submit_u8:   decoded 8-bit images [B,H,W,C] with C = 3 (BGR, as OpenCV holds them) or 1; the
 *     device does the reference's conversion: value/255.0 in double stored as float, planes swapped to RGB
 *     (convolutional.cc:386-398), straight into the first layer's input layout.
 * nb_network_wait blocks until every submitted batch is done and its output is in host memory. */
int nb_network_submit_host(nb_network_t net, const float *input_host, float *output_host);
int nb_network_submit_u8(nb_network_t net, const unsigned char *images_host, float *output_host);
int nb_network_wait(nb_network_t net);
/* One pass over decoded 8-bit images that are already on the device (same conversion). */
int nb_network_forward_u8(nb_network_t net, const unsigned char *images_dev);
/* Replays a forward pass as one CUDA graph once it has run with the same input pointer before (default off;
 * no reference counterpart: the reference launches every kernel from the host).  Profiling windows
 * (nb_profile_begin) always run the kernels one by one. */
int nb_network_set_graph(nb_network_t net, int enable);
/* Bytes of device memory the network holds besides weights and layer outputs (scratch of all its layers). */
size_t nb_network_workspace_size(nb_network_t net);

/* Layer fusion (default on): a 2x2 stride-2 max-pool that follows a convolution is
 * computed in that convolution's epilogue, so the convolution's own output_data is
 * never written and nb_network_layer_output refuses it.  Turn fusion off to
 * materialise every layer's output as the reference does (no reference counterpart). */
int nb_network_set_fusion(nb_network_t net, int enable);

typedef struct {
    int type;                   /* the reference's layer_type_t code (common/def.h:28-42) */
    int channels, height, width;
    size_t size;                /* output elements per sample = the layer's output_size */
    int activation;
} nb_layer_info_t;
int nb_network_num_layers(nb_network_t net);
int nb_network_layer_info(nb_network_t net, int index, nb_layer_info_t *info);
/* Copies layer `index`'s output_data in the reference's layout ([rows,C,H,W]
 * NCHW, rows = batch or T*B) to dst (host or device).  Negative index counts
 * from the end. */
int nb_network_layer_output(nb_network_t net, int index, float *dst, int mem);
/* The last layer's output (softmax probabilities when the cfg ends in
 * [softmax]) and the logits (output of the last [connected] layer). */
int nb_network_output(nb_network_t net, float *dst, int mem);
int nb_network_logits(nb_network_t net, float *dst, int mem);
size_t nb_network_output_size(nb_network_t net);     /* elements of nb_network_output */
size_t nb_network_logits_size(nb_network_t net);
size_t nb_network_input_size(nb_network_t net);      /* elements of one input batch */
int nb_network_destroy(nb_network_t net);

#ifdef __cplusplus
}
#endif
#endif /* NEBULA_B200_H */
