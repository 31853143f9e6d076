// The C ABI (include/nebula_b200.h): argument validation, error translation and
// dispatch into plans, kernels and the network executor.  Nothing here computes
// on the host; a missing or non-sm_100 device is an error, not a fallback.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>

#include "network.h"

using namespace nb;

namespace {

// While a call runs, its handle's arena is the one device buffers are allocated from.
struct ArenaScope {
    std::shared_ptr<Arena> prev;
    explicit ArenaScope(nb_handle_s *h) : prev(Arena::current()) { if (h) Arena::current() = h->arena; }
    ~ArenaScope() { Arena::current() = prev; }
};

template <class F>
int guarded(nb_handle_s *h, F &&f) {
    try {
        ArenaScope scope(h);
        f();
        return NB_OK;
    } catch (const Error &e) {
        if (h) h->last_error = e.code == NB_ERR_CUDA ? e.what() + trace_report(h) : std::string(e.what());
        return e.code;
    } catch (const std::bad_alloc &) {
        if (h) h->last_error = "host allocation failed";
        return NB_ERR_CUDA;
    } catch (const std::exception &e) {
        if (h) h->last_error = e.what();
        return NB_ERR_INVALID_ARG;
    }
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) NB_CHECK_CUDA(cudaSetDevice(dev));
        else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

thread_local std::string g_create_error;

}  // namespace

extern "C" {

int nb_create(int device_id, nb_handle_t *handle) {
    if (!handle) return NB_ERR_INVALID_ARG;
    *handle = nullptr;
    nb_handle_s *h = new (std::nothrow) nb_handle_s();
    if (!h) return NB_ERR_CUDA;
    int rc = guarded(h, [&] {
        int count = 0;
        NB_CHECK_CUDA(cudaGetDeviceCount(&count));
        NB_REQUIRE(device_id >= 0 && device_id < count, "device id out of range");
        DeviceGuard g(device_id);       // the caller's current device is put back on return
        h->device = device_id;
        h->arena = std::make_shared<Arena>();
        cudaDeviceProp prop;
        NB_CHECK_CUDA(cudaGetDeviceProperties(&prop, device_id));
        h->sm_count = prop.multiProcessorCount;
        h->cc_major = prop.major;
        if (prop.major != 10)
            throw Error(NB_ERR_UNSUPPORTED, std::string("this library is built for sm_100a only; device is sm_") +
                                                std::to_string(prop.major) + std::to_string(prop.minor));
        NB_CHECK_CUDA(cudaMalloc((void **)&h->d_status, sizeof(int)));
        NB_CHECK_CUDA(cudaMemset(h->d_status, 0, sizeof(int)));
        NB_CHECK_CUDA(cudaMalloc((void **)&h->d_grid_sync, sizeof(unsigned int)));
        NB_CHECK_CUDA(cudaMemset(h->d_grid_sync, 0, sizeof(unsigned int)));
        int coop = 0;
        NB_CHECK_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device_id));
        h->cooperative_launch = coop != 0;
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        NB_CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !fn) throw Error(NB_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
        h->encode_tiled = (nb_encode_tiled_fn)fn;
        fn = nullptr;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            h->get_address_range = (nb_get_address_range_fn)fn;     // optional: without it operand extents go unchecked
        // Shared-memory limits of the tensor-core kernels are a per-device setting; setting them here, with this
        // handle's device current, also loads every kernel's code before the first forward pass.
        const char *tr = std::getenv("NEBULA_B200_TRACE");
        if (tr && *tr && *tr != '0') {
            fn = nullptr;
            if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
                qres == cudaDriverEntryPointSuccess && fn) {
                unsigned *hp = nullptr;
                NB_CHECK_CUDA(cudaHostAlloc((void **)&hp, sizeof(unsigned), cudaHostAllocMapped));
                *hp = 0;
                void *dp = nullptr;
                NB_CHECK_CUDA(cudaHostGetDevicePointer(&dp, hp, 0));
                h->write_value = (nb_handle_s::write_value_fn)fn;
                h->trace_host = hp;
                h->trace_dev = (CUdeviceptr)dp;
            }
        }
        gemm_tc_prepare_device();
        lstm_persistent_prepare_device();
        conv_halo_prepare_device();
        elementwise_prepare_device();
    });
    if (rc != NB_OK) {
        g_create_error = h->last_error;
        if (h->d_status) cudaFree(h->d_status);
        if (h->d_grid_sync) cudaFree(h->d_grid_sync);
        delete h;
        return rc;
    }
    *handle = h;
    return NB_OK;
}

int nb_destroy(nb_handle_t h) {
    if (!h) return NB_ERR_INVALID_ARG;
    cudaSetDevice(h->device);
    cudaStreamSynchronize(h->stream);
    if (h->d_status) cudaFree(h->d_status);
    if (h->d_grid_sync) cudaFree(h->d_grid_sync);
    for (auto e : h->event_pool) cudaEventDestroy(e);
    for (auto &t : h->timed) { cudaEventDestroy(t.start); cudaEventDestroy(t.stop); }
    delete h;
    return NB_OK;
}

const char *nb_last_error(nb_handle_t h) { return h ? h->last_error.c_str() : g_create_error.c_str(); }

int nb_set_stream(nb_handle_t h, void *stream) {
    if (!h) return NB_ERR_INVALID_ARG;
    h->stream = (cudaStream_t)stream;
    return NB_OK;
}

int nb_set_math_mode(nb_handle_t h, int mode) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(mode == NB_MATH_TF32 || mode == NB_MATH_TF32X3 || mode == NB_MATH_FP32, "unknown math mode");
        h->math_mode = mode;
    });
}
int nb_get_math_mode(nb_handle_t h, int *mode) {
    if (!h || !mode) return NB_ERR_INVALID_ARG;
    *mode = h->math_mode;
    return NB_OK;
}

int nb_synchronize(nb_handle_t h) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        DeviceGuard g(h->device);
        NB_CHECK_CUDA(cudaStreamSynchronize(h->stream));
        int st = 0;
        NB_CHECK_CUDA(cudaMemcpy(&st, h->d_status, sizeof(int), cudaMemcpyDeviceToHost));
        if (st != DEV_OK) {
            NB_CHECK_CUDA(cudaMemset(h->d_status, 0, sizeof(int)));
            throw Error(NB_ERR_DEVICE_TIMEOUT, "a kernel's bounded wait ran out (pipeline barrier never completed)");
        }
    });
}

int nb_launch_count(nb_handle_t h, unsigned long long *count) {
    if (!h || !count) return NB_ERR_INVALID_ARG;
    *count = h->launches;
    return NB_OK;
}

int nb_profile_begin(nb_handle_t h) {
    if (!h) return NB_ERR_INVALID_ARG;
    for (auto &t : h->timed) { h->event_pool.push_back(t.start); h->event_pool.push_back(t.stop); }
    h->timed.clear();
    h->profiling = true;
    return NB_OK;
}
int nb_profile_end(nb_handle_t h, nb_profile_t *r) {
    if (!h || !r) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        DeviceGuard g(h->device);
        h->profiling = false;
        NB_CHECK_CUDA(cudaStreamSynchronize(h->stream));
        std::memset(r, 0, sizeof *r);
        for (auto &t : h->timed) {
            float ms = 0;
            NB_CHECK_CUDA(cudaEventElapsedTime(&ms, t.start, t.stop));
            if (t.kind == 0) { r->tc_ms += ms; r->tc_flops += t.flops; r->tc_launches++; }
            else if (t.kind == 2) { r->halo_ms += ms; r->halo_flops += t.flops; r->halo_launches++; }
            else { r->simt_ms += ms; r->simt_flops += t.flops; r->simt_launches++; }
            h->event_pool.push_back(t.start); h->event_pool.push_back(t.stop);
        }
        h->timed.clear();
    });
}

// ----------------------------------------------------------------- plans
int nb_conv2d_plan_create(nb_handle_t h, const nb_conv2d_desc_t *desc, nb_plan_t *plan) {
    if (!h || !plan) return NB_ERR_INVALID_ARG;
    *plan = nullptr;
    return guarded(h, [&] {
        NB_REQUIRE(desc != nullptr, "null descriptor");
        DeviceGuard g(h->device);
        *plan = new ConvPlan(h, *desc);
    });
}
int nb_conv2d_set_weights(nb_plan_t plan, const float *weight, const float *bias, const float *s, const float *m,
                          const float *v, int mem) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        NB_REQUIRE(plan->kind == NB_PLAN_CONV, "not a convolution plan");
        NB_REQUIRE(mem == NB_MEM_HOST || mem == NB_MEM_DEVICE, "bad memory kind");
        DeviceGuard g(plan->h->device);
        static_cast<ConvPlan *>(plan)->set_weights(weight, bias, s, m, v, mem);
    });
}
int nb_conv2d_forward(nb_plan_t plan, const float *x, float *y) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        NB_REQUIRE(plan->kind == NB_PLAN_CONV, "not a convolution plan");
        DeviceGuard g(plan->h->device);
        ConvPlan *p = static_cast<ConvPlan *>(plan);
        ForwardOpts o;
        o.x_nhwc = o.y_nhwc = p->d.layout == NB_LAYOUT_NHWC;
        o.x_foreign = true;
        p->forward(x, y, o);
    });
}
int nb_conv2d_forward_fused(nb_plan_t plan, const float *x, float *y, const nb_conv2d_fusion_t *f) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        NB_REQUIRE(plan->kind == NB_PLAN_CONV, "not a convolution plan");
        NB_REQUIRE(f != nullptr, "null fusion descriptor");
        NB_REQUIRE(!(f->residual && f->pool_out), "a convolution folds in a shortcut or a pooling layer, not both");
        DeviceGuard g(plan->h->device);
        ConvPlan *p = static_cast<ConvPlan *>(plan);
        if (p->d.layout != NB_LAYOUT_NHWC) throw Error(NB_ERR_UNSUPPORTED, "fused layers need an NB_LAYOUT_NHWC plan");
        ForwardOpts o;
        o.x_nhwc = o.y_nhwc = true;
        o.x_foreign = true;
        if (f->residual) {
            NB_REQUIRE(f->res_channels > 0 && f->res_height > 0 && f->res_width > 0, "residual: non-positive extent");
            NB_REQUIRE(f->res_activation > NB_ACT_UNDEFINED && f->res_activation < NB_ACT_COUNT, "residual: undefined activation");
            if (!p->can_fuse_shortcut(f->res_channels, f->res_height, f->res_width))
                throw Error(NB_ERR_UNSUPPORTED, "this convolution cannot fold the shortcut in (it needs a tensor-core path, a "
                                                "linear activation, channel counts divisible by 4 and a connection at "
                                                "least as large as the output)");
            o.residual = f->residual;
            o.res_c = f->res_channels; o.res_h = f->res_height; o.res_w = f->res_width; o.res_act = f->res_activation;
        }
        if (f->pool_out) {
            if (!p->can_fuse_pool())
                throw Error(NB_ERR_UNSUPPORTED, "this convolution cannot fold the pooling in (it needs a tensor-core path, "
                                                "even output extents and a filter count divisible by 4)");
            o.pool_out = f->pool_out;
        }
        p->forward(x, f->pool_out ? nullptr : y, o);
    });
}
int nb_plan_prepare(nb_plan_t plan) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        DeviceGuard g(plan->h->device);
        switch (plan->kind) {
            case NB_PLAN_CONV: {
                ConvPlan *p = static_cast<ConvPlan *>(plan);
                ForwardOpts o;
                o.x_nhwc = o.y_nhwc = p->d.layout == NB_LAYOUT_NHWC;
                o.x_foreign = true;
                p->reserve(o);
                break;
            }
            case NB_PLAN_FC: {
                ForwardOpts o;
                o.x_foreign = true;
                static_cast<FcPlan *>(plan)->reserve(o);
                break;
            }
            case NB_PLAN_LSTM: static_cast<LstmPlan *>(plan)->reserve(true, false, false); break;
            case NB_PLAN_RNN: static_cast<RnnPlan *>(plan)->reserve(false); break;
            default: throw Error(NB_ERR_INVALID_ARG, "unknown plan kind");
        }
        NB_CHECK_CUDA(cudaStreamSynchronize(plan->h->stream));
    });
}
size_t nb_workspace_size(nb_plan_t plan) { return plan ? plan->workspace_bytes() : 0; }
int nb_plan_output_dims(nb_plan_t plan, int dims[3]) {
    if (!plan || !dims) return NB_ERR_INVALID_ARG;
    plan->output_dims(dims);
    return NB_OK;
}
int nb_plan_destroy(nb_plan_t plan) {
    if (!plan) return NB_ERR_INVALID_ARG;
    cudaSetDevice(plan->h->device);
    cudaStreamSynchronize(plan->h->stream);
    delete plan;
    return NB_OK;
}

int nb_fc_plan_create(nb_handle_t h, const nb_fc_desc_t *desc, nb_plan_t *plan) {
    if (!h || !plan) return NB_ERR_INVALID_ARG;
    *plan = nullptr;
    return guarded(h, [&] {
        NB_REQUIRE(desc != nullptr, "null descriptor");
        DeviceGuard g(h->device);
        *plan = new FcPlan(h, *desc);
    });
}
int nb_fc_set_weights(nb_plan_t plan, const float *weight, const float *bias, const float *s, const float *m,
                      const float *v, int mem) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        NB_REQUIRE(plan->kind == NB_PLAN_FC, "not a connected-layer plan");
        NB_REQUIRE(mem == NB_MEM_HOST || mem == NB_MEM_DEVICE, "bad memory kind");
        DeviceGuard g(plan->h->device);
        static_cast<FcPlan *>(plan)->set_weights(weight, bias, s, m, v, mem);
    });
}
int nb_fc_forward(nb_plan_t plan, const float *x, float *y) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        NB_REQUIRE(plan->kind == NB_PLAN_FC, "not a connected-layer plan");
        DeviceGuard g(plan->h->device);
        ForwardOpts o;
        o.x_foreign = true;
        static_cast<FcPlan *>(plan)->forward(x, y, o);
    });
}

int nb_lstm_plan_create(nb_handle_t h, const nb_lstm_desc_t *desc, nb_plan_t *plan) {
    if (!h || !plan) return NB_ERR_INVALID_ARG;
    *plan = nullptr;
    return guarded(h, [&] {
        NB_REQUIRE(desc != nullptr, "null descriptor");
        DeviceGuard g(h->device);
        *plan = new LstmPlan(h, *desc);
    });
}
int nb_lstm_set_weights(nb_plan_t plan, const float *stream, size_t count, int mem) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        NB_REQUIRE(plan->kind == NB_PLAN_LSTM, "not an LSTM plan");
        NB_REQUIRE(mem == NB_MEM_HOST || mem == NB_MEM_DEVICE, "bad memory kind");
        DeviceGuard g(plan->h->device);
        static_cast<LstmPlan *>(plan)->set_weights(stream, count, mem);
    });
}
int nb_lstm_forward(nb_plan_t plan, const float *x, float *out, float *cell) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        NB_REQUIRE(plan->kind == NB_PLAN_LSTM, "not an LSTM plan");
        DeviceGuard g(plan->h->device);
        static_cast<LstmPlan *>(plan)->forward(x, out, cell, false, nullptr);
    });
}

int nb_rnn_plan_create(nb_handle_t h, const nb_rnn_desc_t *desc, nb_plan_t *plan) {
    if (!h || !plan) return NB_ERR_INVALID_ARG;
    *plan = nullptr;
    return guarded(h, [&] {
        NB_REQUIRE(desc != nullptr, "null descriptor");
        DeviceGuard g(h->device);
        *plan = new RnnPlan(h, *desc);
    });
}
int nb_rnn_set_weights(nb_plan_t plan, const float *stream, size_t count, int mem) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        NB_REQUIRE(plan->kind == NB_PLAN_RNN, "not an RNN plan");
        NB_REQUIRE(mem == NB_MEM_HOST || mem == NB_MEM_DEVICE, "bad memory kind");
        NB_REQUIRE(stream != nullptr, "null weight stream");
        DeviceGuard g(plan->h->device);
        static_cast<RnnPlan *>(plan)->set_weights(stream, count, mem);
    });
}
int nb_rnn_forward(nb_plan_t plan, const float *x, float *out) {
    if (!plan) return NB_ERR_INVALID_ARG;
    return guarded(plan->h, [&] {
        NB_REQUIRE(plan->kind == NB_PLAN_RNN, "not an RNN plan");
        DeviceGuard g(plan->h->device);
        static_cast<RnnPlan *>(plan)->forward(x, out, false, false);
    });
}

// ------------------------------------------------------- stateless operators
int nb_pool_forward(nb_handle_t h, const nb_pool_desc_t *d, const float *x, float *y) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(d && x && y, "null argument");
        NB_REQUIRE(d->batch > 0 && d->channels > 0 && d->height > 0 && d->width > 0, "pool: non-positive extent");
        NB_REQUIRE(d->size > 0 && d->stride > 0 && d->padding >= 0, "pool: bad window");
        NB_REQUIRE(d->mode == NB_POOL_MAX || d->mode == NB_POOL_AVG, "pool: bad mode");
        NB_REQUIRE(d->layout == NB_LAYOUT_NCHW || d->layout == NB_LAYOUT_NHWC, "pool: bad layout");
        DeviceGuard g(h->device);
        launch_pool(h, *d, x, y, false);
    });
}
int nb_shortcut_forward(nb_handle_t h, const nb_shortcut_desc_t *d, const float *prev, const float *conn, float *y) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(d && prev && conn && y, "null argument");
        NB_REQUIRE(d->batch > 0 && d->conn_channels > 0 && d->conn_height > 0 && d->conn_width > 0 &&
                       d->out_channels > 0 && d->out_height > 0 && d->out_width > 0, "shortcut: non-positive extent");
        NB_REQUIRE(d->activation > NB_ACT_UNDEFINED && d->activation < NB_ACT_COUNT, "shortcut: undefined activation");
        NB_REQUIRE(d->layout == NB_LAYOUT_NCHW || d->layout == NB_LAYOUT_NHWC, "shortcut: bad layout");
        DeviceGuard g(h->device);
        launch_shortcut(h, *d, prev, conn, y, false);
    });
}
int nb_activation_forward(nb_handle_t h, int activation, float *data, size_t n) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(data || !n, "null data");
        NB_REQUIRE(activation > NB_ACT_UNDEFINED && activation < NB_ACT_COUNT, "undefined activation");
        DeviceGuard g(h->device);
        launch_activation(h, activation, data, n);
    });
}
int nb_forward_bias(nb_handle_t h, float *out, const float *bias, unsigned channel, unsigned size, unsigned batch) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(out && bias, "null argument");
        DeviceGuard g(h->device);
        launch_bias(h, out, bias, channel, size, batch);
    });
}
int nb_batchnorm_normalize(nb_handle_t h, float *out, const float *mean, const float *var, unsigned channel,
                           unsigned size, unsigned batch) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(out && mean && var, "null argument");
        DeviceGuard g(h->device);
        launch_bn_normalize(h, out, mean, var, channel, size, batch);
    });
}
int nb_batchnorm_scale_down(nb_handle_t h, float *out, const float *scale, unsigned channel, unsigned size,
                            unsigned batch) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(out && scale, "null argument");
        DeviceGuard g(h->device);
        launch_bn_scale(h, out, scale, channel, size, batch);
    });
}
int nb_softmax_forward(nb_handle_t h, const float *x, float *y, int rows, int classes) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(x && y && rows > 0 && classes > 0, "softmax: bad argument");
        DeviceGuard g(h->device);
        launch_softmax(h, x, y, rows, classes);
    });
}
int nb_layout_convert(nb_handle_t h, const float *src, float *dst, int batch, int channels, int height, int width,
                      int src_layout) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(src && dst && src != dst, "layout: bad pointers");
        NB_REQUIRE(batch > 0 && channels > 0 && height > 0 && width > 0, "layout: non-positive extent");
        NB_REQUIRE(src_layout == NB_LAYOUT_NCHW || src_layout == NB_LAYOUT_NHWC, "layout: bad layout");
        DeviceGuard g(h->device);
        launch_layout(h, src, dst, batch, channels, height, width, src_layout == NB_LAYOUT_NCHW, false);
    });
}
int nb_gemm(nb_handle_t h, int TA, int TB, int M, int N, int K, float alpha, const float *A, int lda, const float *B,
            int ldb, float beta, float *C, int ldc) {
    if (!h) return NB_ERR_INVALID_ARG;
    return guarded(h, [&] {
        NB_REQUIRE(A && B && C, "gemm: null matrix");
        NB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: non-positive extent");
        NB_REQUIRE(lda >= (TA ? M : K) && ldb >= (TB ? K : N) && ldc >= N, "gemm: leading dimension too small");
        DeviceGuard g(h->device);
        launch_sgemm(h, TA != 0, TB != 0, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
    });
}

// ---------------------------------------------------------------- network
int nb_network_create(nb_handle_t h, const char *cfg_text, int batch_override, nb_network_t *net) {
    if (!h || !net) return NB_ERR_INVALID_ARG;
    *net = nullptr;
    return guarded(h, [&] {
        NB_REQUIRE(cfg_text != nullptr, "null cfg text");
        DeviceGuard g(h->device);
        std::unique_ptr<nb_network_s> n(new nb_network_s());
        n->h = h;
        n->build(cfg_text, batch_override);
        *net = n.release();
    });
}
int nb_network_load_weights(nb_network_t net, const float *stream, size_t count, int mem) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        NB_REQUIRE(mem == NB_MEM_HOST || mem == NB_MEM_DEVICE, "bad memory kind");
        DeviceGuard g(net->h->device);
        net->load_weights(stream, count, mem);
    });
}
int nb_network_load_weight_file(nb_network_t net, const char *path) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        NB_REQUIRE(path != nullptr, "null path");
        std::ifstream f(path, std::ios::binary | std::ios::ate);
        if (!f.is_open()) throw Error(NB_ERR_WEIGHTS, std::string("failed to open ") + path);
        const std::streamoff bytes = f.tellg();
        if (bytes % 4) throw Error(NB_ERR_WEIGHTS, "weight file size is not a multiple of 4 bytes");
        std::vector<float> buf((size_t)bytes / 4);
        f.seekg(0);
        f.read((char *)buf.data(), bytes);
        DeviceGuard g(net->h->device);
        net->load_weights(buf.data(), buf.size(), NB_MEM_HOST);
    });
}
size_t nb_network_weight_count(nb_network_t net) { return net ? net->weight_count() : 0; }

int nb_network_forward(nb_network_t net, const float *input) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        DeviceGuard g(net->h->device);
        net->forward(input);
    });
}
int nb_network_forward_host(nb_network_t net, const float *input_host, float *output_host) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        DeviceGuard g(net->h->device);
        net->submit(input_host, false, output_host);
        net->wait();
    });
}
int nb_network_submit_host(nb_network_t net, const float *input_host, float *output_host) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        DeviceGuard g(net->h->device);
        net->submit(input_host, false, output_host);
    });
}
int nb_network_submit_u8(nb_network_t net, const unsigned char *images_host, float *output_host) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        DeviceGuard g(net->h->device);
        net->submit(images_host, true, output_host);
    });
}
int nb_network_wait(nb_network_t net) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        DeviceGuard g(net->h->device);
        net->wait();
    });
}
int nb_network_forward_u8(nb_network_t net, const unsigned char *images_dev) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        DeviceGuard g(net->h->device);
        if (!net->weights_loaded && net->weight_count() > 0)
            throw Error(NB_ERR_NO_WEIGHTS, "network forward before weights were loaded");
        net->forward_u8(images_dev);
    });
}
int nb_network_set_graph(nb_network_t net, int enable) {
    if (!net) return NB_ERR_INVALID_ARG;
    net->use_graph = enable != 0;
    return NB_OK;
}
size_t nb_network_workspace_size(nb_network_t net) { return net ? net->workspace_bytes() : 0; }
int nb_network_set_fusion(nb_network_t net, int enable) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        DeviceGuard g(net->h->device);
        net->fuse = enable != 0;
        if (net->weights_loaded) net->prepare();
    });
}
int nb_network_num_layers(nb_network_t net) { return net ? (int)net->layers.size() : -1; }
int nb_network_layer_info(nb_network_t net, int index, nb_layer_info_t *info) {
    if (!net || !info) return NB_ERR_INVALID_ARG;
    const int n = (int)net->layers.size();
    if (index < 0) index += n;
    if (index < 0 || index >= n) return NB_ERR_INVALID_ARG;
    const NetLayer &l = *net->layers[index];
    info->type = l.type; info->channels = l.C; info->height = l.H; info->width = l.W;
    info->size = l.size; info->activation = l.activation;
    return NB_OK;
}
int nb_network_layer_output(nb_network_t net, int index, float *dst, int mem) {
    if (!net) return NB_ERR_INVALID_ARG;
    return guarded(net->h, [&] {
        NB_REQUIRE(mem == NB_MEM_HOST || mem == NB_MEM_DEVICE, "bad memory kind");
        DeviceGuard g(net->h->device);
        net->layer_output(index, dst, mem);
    });
}
int nb_network_output(nb_network_t net, float *dst, int mem) { return nb_network_layer_output(net, -1, dst, mem); }
int nb_network_logits(nb_network_t net, float *dst, int mem) {
    if (!net) return NB_ERR_INVALID_ARG;
    if (net->logits_layer < 0) {
        net->h->last_error = "the network has no [connected] layer";
        return NB_ERR_UNSUPPORTED;
    }
    return nb_network_layer_output(net, net->logits_layer, dst, mem);
}
size_t nb_network_output_size(nb_network_t net) { return net ? net->layers.back()->size * net->rows : 0; }
size_t nb_network_logits_size(nb_network_t net) {
    return (net && net->logits_layer >= 0) ? net->layers[net->logits_layer]->size * net->rows : 0;
}
size_t nb_network_input_size(nb_network_t net) { return net ? net->input_size * net->rows : 0; }
int nb_network_destroy(nb_network_t net) {
    if (!net) return NB_ERR_INVALID_ARG;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(net->h->device);
    cudaStreamSynchronize(net->h->stream);
    if (net->copy_stream) cudaStreamSynchronize(net->copy_stream);
    delete net;
    if (prev >= 0) cudaSetDevice(prev);
    return NB_OK;
}

}  // extern "C"
