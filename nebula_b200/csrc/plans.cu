// Per-layer plans: weight upload/re-layout and the forward bodies that a Nebula
// layer's _forward_() would call.
#include "plans.h"

#include <algorithm>
#include <cstdlib>
#include <cmath>
#include <cstring>

namespace nb {

void upload(nb_handle_s *h, DeviceBuffer &dst, const float *src, size_t n, int mem, size_t guard) {
    dst.alloc(n, guard);
    if (!n) return;
    NB_REQUIRE(src != nullptr, "null source pointer");
    NB_CHECK_CUDA(cudaMemcpyAsync(dst.p, src, n * sizeof(float),
                                  mem == NB_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, h->stream));
    if (mem == NB_MEM_HOST) NB_CHECK_CUDA(cudaStreamSynchronize(h->stream));   // the host buffer may go away
}
void upload_vec(nb_handle_s *h, DeviceBuffer &dst, const std::vector<float> &v, size_t guard) {
    upload(h, dst, v.data(), v.size(), NB_MEM_HOST, guard);
}
// Per-column epilogue vectors are read 32 columns at a time: pad them to a multiple of 32.
void upload_padded(nb_handle_s *h, DeviceBuffer &dst, std::vector<float> v, float fill) {
    v.resize((v.size() + 31) / 32 * 32, fill);
    upload_vec(h, dst, v);
}
std::vector<float> to_host(nb_handle_s *h, const float *src, size_t n, int mem) {
    std::vector<float> v(n);
    if (!n) return v;
    NB_REQUIRE(src != nullptr, "null source pointer");
    if (mem == NB_MEM_DEVICE) {
        NB_CHECK_CUDA(cudaMemcpyAsync(v.data(), src, n * sizeof(float), cudaMemcpyDeviceToHost, h->stream));
        NB_CHECK_CUDA(cudaStreamSynchronize(h->stream));
    } else {
        std::memcpy(v.data(), src, n * sizeof(float));
    }
    return v;
}

void fold_bn(int n, const float *bias, const float *gamma, const float *mean, const float *var, bool has_bn,
             std::vector<float> &scale, std::vector<float> &shift) {
    scale.clear();
    shift.resize(n);
    if (!has_bn) {
        for (int i = 0; i < n; i++) shift[i] = bias[i];
        return;
    }
    scale.resize(n);
    for (int i = 0; i < n; i++) {
        const double s = (double)gamma[i] / (std::sqrt((double)var[i]) + 0.00001);
        scale[i] = (float)s;
        shift[i] = (float)((double)bias[i] - (double)mean[i] * s);
    }
}

// -------------------------------------------------------------------- conv
ConvPlan::ConvPlan(nb_handle_s *hh, const nb_conv2d_desc_t &desc) : nb_plan_s(NB_PLAN_CONV, hh), d(desc) {
    NB_REQUIRE(d.batch > 0 && d.channels > 0 && d.height > 0 && d.width > 0, "conv: non-positive input extent");
    NB_REQUIRE(d.filters > 0 && d.size > 0 && d.stride > 0 && d.padding >= 0, "conv: bad filter geometry");
    NB_REQUIRE(d.height + 2 * d.padding >= d.size && d.width + 2 * d.padding >= d.size, "conv: filter larger than padded input");
    NB_REQUIRE(d.activation > NB_ACT_UNDEFINED && d.activation < NB_ACT_COUNT, "conv: undefined activation");
    NB_REQUIRE(d.layout == NB_LAYOUT_NCHW || d.layout == NB_LAYOUT_NHWC, "conv: bad layout");
    // convolutional_layer.cc:150-151
    OH = (d.height + 2 * d.padding - d.size) / d.stride + 1;
    OW = (d.width + 2 * d.padding - d.size) / d.stride + 1;
    Cp = (d.channels + 3) / 4 * 4;
    const int K = d.channels * d.size * d.size;
    Kpad = (K + 31) / 32 * 32;
    pack_ok = (Cp != d.channels || d.channels < 32) && Kpad <= 384;    // the gather table lives in the kernel parameters
    // row windows: 4 floats per pixel, a filter row of k taps is 4k floats, rounded up to whole 32-float K blocks
    rw_inner = (4 * d.size + 31) / 32 * 32;
    rw_wp = std::max((OW - 1) * d.stride + rw_inner / 4, d.width + 2 * d.padding);
    // NEBULA_B200_ROW_WINDOWS=0 (read when the plan is created) sends these layers through the in-kernel gather instead
    const char *rw_env = std::getenv("NEBULA_B200_ROW_WINDOWS");
    rowwin_ok = !(rw_env && *rw_env == '0') && d.channels <= 4 && rw_inner <= 256 && d.stride <= 8 && h->encode_tiled &&
                h->cc_major == 10;
}

void ConvPlan::set_weights(const float *weight, const float *bias, const float *g, const float *m, const float *v,
                           int mem) {
    NB_REQUIRE(weight && bias, "conv: null weight or bias");
    NB_REQUIRE(!d.batch_normalize || (g && m && v), "conv: batch_normalize=1 needs scale, mean and variance");
    const size_t wn = (size_t)d.filters * d.channels * d.size * d.size;
    DeviceBuffer raw;
    upload(h, raw, weight, wn, mem);
    w.exact.alloc((size_t)d.size * d.size * d.filters * Cp, weight_guard(Cp));
    w.split_ready = false;
    launch_weight_relayout(h, raw.p, w.exact.p, d.filters, d.channels, d.size, Cp);
    const bool tensor_cores = h->encode_tiled && h->cc_major == 10;
    if (tensor_cores) w.ensure_split(h);
    if (rowwin_ok) {
        wr.exact.alloc((size_t)d.size * d.filters * rw_inner, weight_guard(rw_inner));
        wr.split_ready = false;
        launch_weight_rowwin(h, raw.p, wr.exact.p, d.filters, d.channels, d.size, rw_inner);
        wr.ensure_split(h);
    }
    if (pack_ok) {
        wp.exact.alloc((size_t)d.filters * Kpad, weight_guard(Kpad));
        wp.split_ready = false;
        launch_weight_pack(h, raw.p, wp.exact.p, d.filters, d.channels, d.size, Kpad);
        if (tensor_cores) wp.ensure_split(h);
    }
    NB_CHECK_CUDA(cudaStreamSynchronize(h->stream));
    std::vector<float> hb = to_host(h, bias, d.filters, mem), hg, hm, hv, sc, sh;
    if (d.batch_normalize) {
        hg = to_host(h, g, d.filters, mem);
        hm = to_host(h, m, d.filters, mem);
        hv = to_host(h, v, d.filters, mem);
    }
    fold_bn(d.filters, hb.data(), hg.data(), hm.data(), hv.data(), d.batch_normalize != 0, sc, sh);
    has_scale = !sc.empty();
    if (has_scale) upload_padded(h, scale, sc, 1.0f);
    upload_padded(h, shift, sh, 0.0f);
    ready = true;
}

GemmPath ConvPlan::path(const ForwardOpts &) const {
    if (h->math_mode == NB_MATH_FP32) return PATH_SIMT;
    const bool tc_ok = h->encode_tiled && h->cc_major == 10 && Cp == d.channels && d.channels >= 32 && d.stride <= 8;
    if (!tc_ok) return PATH_SIMT;
    return h->math_mode == NB_MATH_TF32X3 ? PATH_TC3 : PATH_TC;
}

bool ConvPlan::can_fuse_pool() const {
    const GemmPath pth = path(ForwardOpts());
    return (pth == PATH_TC || pth == PATH_TC3) && !(OH & 1) && !(OW & 1) && (d.filters % 4) == 0 && OH >= 2 && OW >= 2;
}

bool ConvPlan::can_fuse_shortcut(int conn_c, int conn_h, int conn_w) const {
    const GemmPath pth = path(ForwardOpts());
    // sample == 1 (the connection is not smaller than this layer's output), linear conv, aligned channel rows
    return (pth == PATH_TC || pth == PATH_TC3) && d.activation == NB_ACT_LINEAR && conn_w >= OW && conn_h >= OH &&
           (conn_c % 4) == 0 && (d.filters % 4) == 0;
}

// Which of the three routes forward() takes, and the scratch each needs.
size_t ConvPlan::reserve(const ForwardOpts &o) {
    const GemmPath pth = path(o);
    const size_t xin = (size_t)d.batch * d.channels * d.height * d.width;
    const size_t yout = (size_t)d.batch * d.filters * OH * OW;
    const bool tc_mode = h->math_mode != NB_MATH_FP32;
    if (!o.y_nhwc) y_scratch.reserve(yout);
    if (pth == PATH_SIMT && rowwin_ok && tc_mode) {
        x_rowwin.reserve((size_t)d.batch * d.height * rw_wp * 4);
    } else if (pth == PATH_SIMT && pack_ok && tc_mode && h->encode_tiled) {
        // the kernel gathers x in place
    } else if (pth != PATH_SIMT) {
        const bool need_round = (pth == PATH_TC) && !o.x_rounded;
        if (!o.x_nhwc || need_round || o.x_foreign) x_scratch.reserve(xin);
    }
    return workspace_bytes();
}

void ConvPlan::forward(const float *x, float *y, const ForwardOpts &o) {
    if (!ready) throw Error(NB_ERR_NO_WEIGHTS, "conv: forward before set_weights");
    NB_REQUIRE(x && (y || o.pool_out), "conv: null tensor pointer");
    const GemmPath pth = path(o);
    const size_t xin = (size_t)d.batch * d.channels * d.height * d.width;
    reserve(o);

    GemmArgs a;
    a.a_is_conv = true;
    ConvGeom &g = a.g;
    g.batch = d.batch; g.C = d.channels; g.H = d.height; g.W = d.width; g.OH = OH; g.OW = OW;
    g.ksize = d.size; g.stride = d.stride; g.pad = d.padding;

    if (pth == PATH_SIMT && rowwin_ok && h->math_mode != NB_MATH_FP32) {
        // tensor-core route for 1-4 input channels: one TMA-fetched K slice per filter row
        const bool three = h->math_mode == NB_MATH_TF32X3;
        float *xw = x_rowwin.p;
        if (o.x_rowwin) xw = const_cast<float *>(x);       // the caller already holds the input in this layout
        else launch_rowwin_input(h, x, xw, d.batch, d.channels, d.height, d.width, rw_wp, d.padding, o.x_nhwc, !three);
        GemmArgs ra;
        ra.a = xw; ra.a_is_conv = true;
        ConvGeom &rg = ra.g;
        rg.batch = d.batch; rg.C = rw_inner; rg.H = d.height; rg.W = rw_wp - rw_inner / 4 + 1; rg.OH = OH; rg.OW = OW;
        rg.ksize = d.size; rg.ksize_w = 1; rg.stride = d.stride; rg.pad = d.padding; rg.pad_w = 0;
        rg.sc = 1; rg.sw = 4; rg.sh = (long)rw_wp * 4; rg.sn = (long)d.height * rw_wp * 4;
        ra.ldb = rw_inner; ra.M = d.batch * OH * OW; ra.N = d.filters; ra.Kc = rw_inner;
        ra.scale = has_scale ? scale.p : nullptr; ra.shift = shift.p; ra.act = d.activation;
        ra.round_out_tf32 = o.round_out; ra.addend = o.addend; ra.ld_addend = d.filters;
        float *yo = y;
        if (!o.y_nhwc) {
            NB_REQUIRE(o.addend == nullptr, "conv: addend needs NHWC output");
            yo = y_scratch.p;
        }
        ra.y = yo; ra.ldy = d.filters;
        ra.algo_flops = 2.0 * (double)ra.M * d.filters * d.channels * d.size * d.size;
        ra.b = wr.hi.p; ra.b_lo = wr.lo.p;
        if (gemm_tc_supported(h, ra)) {
            gemm_tc(h, ra, three);
            if (!o.y_nhwc) launch_layout(h, yo, y, d.batch, d.filters, OH, OW, false, false);
            return;
        }
    }
    if (pth == PATH_SIMT && pack_ok && h->math_mode != NB_MATH_FP32 && h->encode_tiled) {
        // tensor-core route for small channel counts: the kernel gathers the patches itself
        const bool three = h->math_mode == NB_MATH_TF32X3;
        const size_t M = (size_t)d.batch * OH * OW;
        if (o.x_nhwc) {
            g.sc = 1; g.sw = d.channels; g.sh = (long)d.width * d.channels; g.sn = (long)d.height * d.width * d.channels;
        } else {
            g.sw = 1; g.sh = d.width; g.sc = (long)d.height * d.width; g.sn = (long)d.channels * d.height * d.width;
        }
        GemmArgs pa;
        pa.a = x; pa.a_is_conv = true; pa.g = g; pa.a_gather = true;
        pa.ldb = Kpad; pa.M = (int)M; pa.N = d.filters; pa.Kc = Kpad;
        pa.scale = has_scale ? scale.p : nullptr; pa.shift = shift.p; pa.act = d.activation;
        pa.round_out_tf32 = o.round_out; pa.addend = o.addend; pa.ld_addend = d.filters;
        float *yo = y;
        if (!o.y_nhwc) {
            NB_REQUIRE(o.addend == nullptr, "conv: addend needs NHWC output");
            yo = y_scratch.p;
        }
        pa.y = yo; pa.ldy = d.filters;
        pa.algo_flops = 2.0 * (double)M * d.filters * d.channels * d.size * d.size;
        wp.ensure_split(h);
        pa.b = wp.hi.p; pa.b_lo = wp.lo.p;
        gemm_tc(h, pa, three);
        if (!o.y_nhwc) launch_layout(h, yo, y, d.batch, d.filters, OH, OW, false, false);
        return;
    }

    const float *xa = x;
    bool nhwc = o.x_nhwc;
    if (pth != PATH_SIMT) {
        const bool need_round = (pth == PATH_TC) && !o.x_rounded;
        if (!nhwc) {
            launch_layout(h, x, x_scratch.p, d.batch, d.channels, d.height, d.width, true, need_round);
            xa = x_scratch.p;
            nhwc = true;
        } else if (need_round) {
            launch_round_tf32(h, x, x_scratch.p, xin);
            xa = x_scratch.p;
        } else if (o.x_foreign) {
            NB_CHECK_CUDA(cudaMemcpyAsync(x_scratch.p, x, xin * sizeof(float), cudaMemcpyDeviceToDevice, h->stream));
            xa = x_scratch.p;
        }
    }
    if (nhwc) {
        g.sc = 1; g.sw = d.channels; g.sh = (long)d.width * d.channels; g.sn = (long)d.height * d.width * d.channels;
    } else {
        g.sw = 1; g.sh = d.width; g.sc = (long)d.height * d.width; g.sn = (long)d.channels * d.height * d.width;
    }
    a.a = xa;
    a.ldb = Cp;
    a.M = d.batch * OH * OW;
    a.N = d.filters;
    a.Kc = d.channels;
    a.scale = has_scale ? scale.p : nullptr;
    a.shift = shift.p;
    a.act = d.activation;
    a.round_out_tf32 = o.round_out;
    a.addend = o.addend;
    a.ld_addend = d.filters;
    float *yo = y;
    if (!o.y_nhwc) {
        NB_REQUIRE(o.addend == nullptr, "conv: addend needs NHWC output");
        yo = y_scratch.p;
    }
    a.y = yo;
    a.ldy = d.filters;
    if (o.residual) {
        NB_REQUIRE(o.y_nhwc && pth != PATH_SIMT && !o.addend && !o.pool_out, "conv: fused shortcut needs the tensor-core path and NHWC output");
        a.addend = o.residual;
        a.ld_addend = o.res_c;
        a.res_stride = std::max(1, o.res_w / OW);       // common/utils.cc:31
        a.res_c = std::min(o.res_c, d.filters);
        a.res_h = o.res_h; a.res_w = o.res_w;
        a.act = o.res_act;
    }
    if (o.pool_out) {
        NB_REQUIRE(o.y_nhwc && pth != PATH_SIMT, "conv: fused pooling needs the tensor-core path and NHWC output");
        a.y = nullptr;
        a.y_pool = o.pool_out;
    }
    if (pth == PATH_SIMT) {
        a.b = w.exact.p;
        gemm_simt(h, a);
    } else {
        w.ensure_split(h);
        a.b = w.hi.p;
        a.b_lo = w.lo.p;
        // few input channels: the generic kernel would re-load the activations once per tap from L2
        // The halo kernel is routed off: a kernel launched right behind it has faulted (illegal address) in a few
        // runs out of many and the cause is not known.  NEBULA_B200_HALO=1 turns it on for investigation only.
        static const bool halo_on = [] {
            const char *v = std::getenv("NEBULA_B200_HALO");
            return v && *v == '1';
        }();
        bool halo = halo_on && pth == PATH_TC && (d.channels <= 64 || (d.channels <= 128 && d.filters <= 128)) &&
                    conv_halo_supported(h, a);
        if (halo) {
            const int bh = OH >= 16 ? 16 : 8;
            const double eff = ((double)OW / ((OW + 13) / 14 * 14)) * ((double)OH / ((OH + bh - 1) / bh * bh));
            halo = eff >= 0.6;
        }
        if (halo) conv_halo_tc(h, a);
        else gemm_tc(h, a, pth == PATH_TC3);
    }
    if (!o.y_nhwc) launch_layout(h, yo, y, d.batch, d.filters, OH, OW, false, false);
}

// ---------------------------------------------------------------------- fc
FcPlan::FcPlan(nb_handle_s *hh, const nb_fc_desc_t &desc) : nb_plan_s(NB_PLAN_FC, hh), d(desc) {
    NB_REQUIRE(d.batch > 0 && d.inputs > 0 && d.outputs > 0, "connected: non-positive extent");
    NB_REQUIRE(d.activation > NB_ACT_UNDEFINED && d.activation < NB_ACT_COUNT, "connected: undefined activation");
}

void FcPlan::set_weights(const float *weight, const float *bias, const float *g, const float *m, const float *v,
                         int mem) {
    NB_REQUIRE(weight && bias, "connected: null weight or bias");
    NB_REQUIRE(!d.batch_normalize || (g && m && v), "connected: batch_normalize=1 needs scale, mean and variance");
    const size_t wn = (size_t)d.outputs * d.inputs;
    w.split_ready = false;
    if (perm_c > 0 && perm_h * perm_w > 1) {
        NB_REQUIRE((size_t)perm_c * perm_h * perm_w == (size_t)d.inputs, "connected: permutation does not match inputs");
        DeviceBuffer raw;
        upload(h, raw, weight, wn, mem);
        w.exact.alloc(wn, weight_guard(d.inputs));
        launch_fc_permute(h, raw.p, w.exact.p, d.outputs, perm_c, perm_h, perm_w);
        NB_CHECK_CUDA(cudaStreamSynchronize(h->stream));
    } else {
        upload(h, w.exact, weight, wn, mem, weight_guard(d.inputs));
    }
    if (h->encode_tiled && h->cc_major == 10 && (d.inputs % 4) == 0 && d.inputs >= 32) w.ensure_split(h);
    std::vector<float> hb = to_host(h, bias, d.outputs, mem), hg, hm, hv, sc, sh;
    if (d.batch_normalize) {
        hg = to_host(h, g, d.outputs, mem);
        hm = to_host(h, m, d.outputs, mem);
        hv = to_host(h, v, d.outputs, mem);
    }
    fold_bn(d.outputs, hb.data(), hg.data(), hm.data(), hv.data(), d.batch_normalize != 0, sc, sh);
    has_scale = !sc.empty();
    if (has_scale) upload_padded(h, scale, sc, 1.0f);
    upload_padded(h, shift, sh, 0.0f);
    ready = true;
}

GemmPath FcPlan::path() const {
    if (h->math_mode == NB_MATH_FP32) return PATH_SIMT;
    const bool tc_ok = h->encode_tiled && h->cc_major == 10 && (d.inputs % 4) == 0 && d.inputs >= 32;
    if (!tc_ok) return PATH_SIMT;
    return h->math_mode == NB_MATH_TF32X3 ? PATH_TC3 : PATH_TC;
}

// Few rows and a long contraction (weight streaming): split K so that every SM pulls weights.  Chosen from K, N
// and the SM count only, never from the batch: a batch and its slices add in the same order.  Wide tiles keep the
// most weight bytes in flight per SM; the split count then fills the SMs, and of the three tile widths the one
// that leaves the fewest SMs idle in the last wave wins.
void FcPlan::split_choice(bool tc, bool has_addend, int *S_out, int *block_n_out) const {
    int S = 1, block_n = 0;
    if (tc && !has_addend && (d.outputs % 4) == 0 && d.inputs >= 2048) {
        const int kblocks = (d.inputs + 31) / 32;
        double best = 0.0;
        for (int bn = 256; bn >= 64; bn /= 2) {
            const int nt = (d.outputs + bn - 1) / bn;
            int s = std::max(1, std::min({32, h->sm_count / nt, kblocks / 8}));
            const int per = (kblocks + s - 1) / s;
            s = (kblocks + per - 1) / per;
            const long tiles = (long)nt * s;
            const double fill = (double)tiles / (double)(((tiles + h->sm_count - 1) / h->sm_count) * h->sm_count);
            if (fill > best + 0.05) { best = fill; S = s; block_n = bn; }
        }
        if (S == 1) block_n = 0;
    }
    *S_out = S; *block_n_out = block_n;
}

size_t FcPlan::reserve(const ForwardOpts &o, int rows) {
    const int M = rows > 0 ? rows : d.batch;
    const GemmPath pth = path();
    if ((pth == PATH_TC && !o.x_rounded) || (pth == PATH_TC3 && o.x_foreign)) x_scratch.reserve((size_t)M * d.inputs);
    int S, bn;
    split_choice(pth == PATH_TC, o.addend != nullptr, &S, &bn);
    if (S > 1) split_ws.reserve((size_t)S * M * d.outputs);
    return workspace_bytes();
}

void FcPlan::forward(const float *x, float *y, const ForwardOpts &o, int rows) {
    if (!ready) throw Error(NB_ERR_NO_WEIGHTS, "connected: forward before set_weights");
    NB_REQUIRE(x && y, "connected: null tensor pointer");
    const int M = rows > 0 ? rows : d.batch;
    GemmPath pth = path();
    reserve(o, rows);
    if (pth != PATH_SIMT && (((uintptr_t)x) & 15)) pth = PATH_SIMT;
    GemmArgs a;
    const float *xa = x;
    if (pth == PATH_TC && !o.x_rounded) {
        launch_round_tf32(h, x, x_scratch.p, (size_t)M * d.inputs);
        xa = x_scratch.p;
    } else if (pth == PATH_TC3 && o.x_foreign) {
        NB_CHECK_CUDA(cudaMemcpyAsync(x_scratch.p, x, (size_t)M * d.inputs * sizeof(float), cudaMemcpyDeviceToDevice, h->stream));
        xa = x_scratch.p;
    }
    a.a = xa; a.lda = d.inputs;
    a.ldb = d.inputs;
    a.M = M; a.N = d.outputs; a.Kc = d.inputs;
    a.scale = has_scale ? scale.p : nullptr;
    a.shift = shift.p;
    a.act = d.activation;
    a.round_out_tf32 = o.round_out;
    a.addend = o.addend; a.ld_addend = d.outputs; a.addend_after_act = o.addend != nullptr && o.addend_post;
    a.y = y; a.ldy = d.outputs;
    if (pth == PATH_SIMT) {
        a.b = w.exact.p;
        gemm_simt(h, a);
        return;
    }
    w.ensure_split(h);
    a.b = w.hi.p; a.b_lo = w.lo.p;
    int S, block_n;
    split_choice(pth == PATH_TC, o.addend != nullptr, &S, &block_n);
    if (S > 1) {
        GemmArgs sa = a;
        sa.split_k = S; sa.block_n_hint = block_n;
        sa.scale = nullptr; sa.shift = nullptr; sa.act = NB_ACT_LINEAR; sa.round_out_tf32 = false;
        sa.y = split_ws.p; sa.ldy = d.outputs;
        sa.algo_flops = 2.0 * (double)M * d.outputs * d.inputs;
        gemm_tc(h, sa, false);
        launch_splitk_reduce(h, split_ws.p, S, M, d.outputs, a.scale, a.shift, d.activation, o.round_out, y);
    } else {
        gemm_tc(h, a, pth == PATH_TC3);
    }
}

// -------------------------------------------------------------------- lstm
LstmPlan::LstmPlan(nb_handle_s *hh, const nb_lstm_desc_t &desc) : nb_plan_s(NB_PLAN_LSTM, hh), d(desc) {
    NB_REQUIRE(d.time_steps > 0 && d.batch > 0 && d.inputs > 0 && d.hidden > 0, "lstm: non-positive extent");
    NB_REQUIRE(d.activation > NB_ACT_UNDEFINED && d.activation < NB_ACT_COUNT, "lstm: undefined activation");
}

size_t LstmPlan::weight_count() const {
    size_t n = 0;
    for (int gidx = 0; gidx < 8; gidx++) {
        const size_t gin = gidx < 4 ? d.hidden : d.inputs;
        n += (size_t)d.hidden + (size_t)d.hidden * gin + (d.batch_normalize ? 3 * (size_t)d.hidden : 0);
    }
    return n;
}

void LstmPlan::set_weights(const float *stream, size_t count, int mem) {
    if (count != weight_count())
        throw Error(NB_ERR_WEIGHTS, "lstm: weight stream has " + std::to_string(count) + " floats, layer needs " +
                                        std::to_string(weight_count()));
    std::vector<float> hs = to_host(h, stream, count, mem);
    const int H = d.hidden, in = d.inputs;
    struct Blob { const float *bias, *w, *g, *m, *v; };
    Blob blob[8];
    size_t pos = 0;
    for (int gidx = 0; gidx < 8; gidx++) {     // file order iW,fW,oW,cW,iU,fU,oU,cU (lstm_layer.cc:194-206)
        const size_t gin = gidx < 4 ? H : in;
        blob[gidx].bias = hs.data() + pos; pos += H;
        blob[gidx].w = hs.data() + pos; pos += (size_t)H * gin;
        blob[gidx].g = blob[gidx].m = blob[gidx].v = nullptr;
        if (d.batch_normalize) {
            blob[gidx].g = hs.data() + pos; pos += H;
            blob[gidx].m = hs.data() + pos; pos += H;
            blob[gidx].v = hs.data() + pos; pos += H;
        }
    }
    // gate rows in the order i, f, g(cell), o; file indices of those gates:
    const int file_of_gate[4] = {0, 1, 3, 2};
    const bool linear = d.activation == NB_ACT_LINEAR;
    std::vector<float> u((size_t)4 * H * in), wr((size_t)4 * H * H), sh_u((size_t)4 * H, 0.0f), sh_w((size_t)4 * H, 0.0f);
    for (int gate = 0; gate < 4; gate++) {
        for (int side = 0; side < 2; side++) {      // 0: W (recurrent), 1: U (input)
            const Blob &b = blob[file_of_gate[gate] + (side ? 4 : 0)];
            const size_t gin = side ? in : H;
            std::vector<float> sc, s1;
            fold_bn(H, b.bias, b.g, b.m, b.v, d.batch_normalize != 0, sc, s1);
            // output row of hidden unit r, gate `gate`: 4*r + gate (a thread of the GEMM epilogue then holds all
            // four gates of a unit in neighbouring columns); a batch-norm scale is folded into the weight row
            float *dst = side ? u.data() : wr.data();
            for (int r = 0; r < H; r++) {
                const float s = sc.empty() ? 1.0f : sc[r];
                const size_t row = (size_t)4 * r + gate;
                for (size_t c = 0; c < gin; c++) dst[row * gin + c] = b.w[(size_t)r * gin + c] * s;
                // linear gate layers: both sides' shifts are one vector, applied once by the input-side GEMM
                ((side || linear) ? sh_u : sh_w)[row] += s1[r];
            }
        }
    }
    upload_vec(h, wu.exact, u, weight_guard(in));
    upload_vec(h, ww.exact, wr, weight_guard(H));
    wu.split_ready = ww.split_ready = false;
    if (h->encode_tiled && h->cc_major == 10) {
        if ((in % 4) == 0 && in >= 32) wu.ensure_split(h);
        if ((H % 4) == 0 && H >= 32) ww.ensure_split(h);
    }
    upload_padded(h, shift, sh_u, 0.0f);
    upload_padded(h, shift_w, sh_w, 0.0f);
    NB_CHECK_CUDA(cudaStreamSynchronize(h->stream));
    ready = true;
}

size_t LstmPlan::reserve(bool own_cell, bool x_rounded, bool have_out_round, bool x_foreign) {
    const int T = d.time_steps, B = d.batch, H = d.hidden, in = d.inputs;
    const size_t rows = (size_t)T * B;
    const bool tcm = h->math_mode != NB_MATH_FP32 && h->encode_tiled && h->cc_major == 10;
    const bool tc_u = tcm && (in % 4) == 0 && in >= 32;
    const bool tc_w = tcm && (H % 4) == 0 && H >= 32;
    const bool three = h->math_mode == NB_MATH_TF32X3;
    pre.reserve(rows * 4 * H);
    if (!tc_w) z.reserve((size_t)B * 4 * H);
    if (own_cell) cell_own.reserve(rows * H);
    if (!have_out_round && tc_w && !three) h_round.reserve(rows * H);
    if (tc_u && ((!three && !x_rounded) || (three && x_foreign))) x_round.reserve(rows * in);
    if (d.activation != NB_ACT_LINEAR && h_zero.reserve((size_t)B * H))
        NB_CHECK_CUDA(cudaMemsetAsync(h_zero.p, 0, (size_t)B * H * sizeof(float), h->stream));
    return workspace_bytes();
}

void LstmPlan::forward(const float *x, float *out, float *cell, bool x_rounded, float *out_round, bool x_foreign) {
    if (!ready) throw Error(NB_ERR_NO_WEIGHTS, "lstm: forward before set_weights");
    NB_REQUIRE(x && out, "lstm: null tensor pointer");
    const int T = d.time_steps, B = d.batch, H = d.hidden, in = d.inputs;
    const size_t rows = (size_t)T * B;
    const bool tcm = h->math_mode != NB_MATH_FP32 && h->encode_tiled && h->cc_major == 10;
    const bool tc_u = tcm && (in % 4) == 0 && in >= 32 && !(((uintptr_t)x) & 15);
    const bool tc_w = tcm && (H % 4) == 0 && H >= 32;
    const bool three = h->math_mode == NB_MATH_TF32X3;
    const bool linear = d.activation == NB_ACT_LINEAR;
    reserve(cell == nullptr, x_rounded, out_round != nullptr, x_foreign);
    if (!cell) cell = cell_own.p;
    float *hr = out_round;
    if (!hr && tc_w && !three) hr = h_round.p;
    // 1. input-side gate layers of every time step in one GEMM: pre = act(X * U^T + bU) (linear: + bW as well)
    {
        const float *xa = x;
        if (tc_u && !three && !x_rounded) {
            launch_round_tf32(h, x, x_round.p, rows * in);
            xa = x_round.p;
        } else if (tc_u && three && x_foreign) {
            NB_CHECK_CUDA(cudaMemcpyAsync(x_round.p, x, rows * in * sizeof(float), cudaMemcpyDeviceToDevice, h->stream));
            xa = x_round.p;
        }
        GemmArgs a;
        a.a = xa; a.lda = in; a.ldb = in; a.M = (int)rows; a.N = 4 * H; a.Kc = in;
        a.shift = shift.p; a.act = d.activation; a.y = pre.p; a.ldy = 4 * H;
        if (tc_u) {
            wu.ensure_split(h);
            a.b = wu.hi.p; a.b_lo = wu.lo.p;
            gemm_tc(h, a, three);
        } else {
            a.b = wu.exact.p;
            gemm_simt(h, a);
        }
    }
    // 2. the recurrence: z_t = pre_t + act(h_{t-1} * W^T + bW), then the cell update.  With linear gate layers
    //    step 0 has nothing to multiply (h_{-1} = 0 and bW is already in pre); otherwise act(bW) is not zero and
    //    step 0 runs the recurrent layer on a zero state like every other step.
    // With linear gate layers on the TF32 tensor-core path, steps 1 .. T-1 run as one cooperative kernel that keeps
    // the recurrent weights in shared memory (lstm_persistent.cu); step 0 is the cell update alone.
    const char *lp_env = std::getenv("NEBULA_B200_LSTM_PERSISTENT");
    bool persistent = tc_w && !three && linear && hr && (H % 8) == 0 && lstm_persistent_supported(h, T, B, H) &&
                      !(lp_env && *lp_env == '0');
    if (persistent) {
        launch_lstm_cell(h, pre.p, nullptr, cell, out, hr, B, H);
        ww.ensure_split(h);
        lstm_persistent(h, ww.hi.p, pre.p, cell, out, hr, T, B, H, 1);
        return;
    }
    for (int t = 0; t < T; t++) {
        const float *zt = pre.p + (size_t)t * B * 4 * H;
        float *ct = cell + (size_t)t * B * H, *ht = out + (size_t)t * B * H, *hrt = hr ? hr + (size_t)t * B * H : nullptr;
        const float *c_prev = t ? cell + (size_t)(t - 1) * B * H : nullptr;
        if (t > 0 || !linear) {
            GemmArgs a;
            const float *hprev = t == 0 ? h_zero.p
                                        : ((tc_w && !three) ? hr + (size_t)(t - 1) * B * H : out + (size_t)(t - 1) * B * H);
            a.a = hprev; a.lda = H; a.ldb = H; a.M = B; a.N = 4 * H; a.Kc = H;
            a.addend = zt; a.ld_addend = 4 * H; a.act = d.activation;
            if (!linear) { a.shift = shift_w.p; a.addend_after_act = true; }
            if (tc_w) {
                // the cell update runs in the GEMM epilogue: one launch per time step
                ww.ensure_split(h);
                a.b = ww.hi.p; a.b_lo = ww.lo.p;
                a.lstm_H = H; a.lstm_c_prev = c_prev; a.lstm_c = ct; a.lstm_h = ht; a.lstm_h_round = hrt;
                gemm_tc(h, a, three);
                continue;
            }
            a.y = z.p; a.ldy = 4 * H;
            a.b = ww.exact.p;
            gemm_simt(h, a);
            zt = z.p;
        }
        launch_lstm_cell(h, zt, c_prev, ct, ht, hrt, B, H);
    }
}

// --------------------------------------------------------------------- rnn
RnnPlan::RnnPlan(nb_handle_s *hh, const nb_rnn_desc_t &desc) : nb_plan_s(NB_PLAN_RNN, hh), d(desc) {
    NB_REQUIRE(d.time_steps > 0 && d.batch > 0 && d.inputs > 0 && d.hidden > 0, "rnn: non-positive extent");
    NB_REQUIRE(d.activation > NB_ACT_UNDEFINED && d.activation < NB_ACT_COUNT, "rnn: undefined activation");
    // the three gates are connected layers built from the same section (rnn_layer.cc:47-54)
    nb_fc_desc_t g{};
    g.batch = d.batch; g.outputs = d.hidden; g.batch_normalize = d.batch_normalize; g.activation = d.activation;
    g.inputs = d.inputs;
    in_gate.reset(new FcPlan(h, g));
    g.inputs = d.hidden;
    hid_gate.reset(new FcPlan(h, g));
    out_gate.reset(new FcPlan(h, g));
}

size_t RnnPlan::weight_count() const {
    const size_t H = d.hidden, bn = d.batch_normalize ? 3 * H : 0;
    return (H + H * d.inputs + bn) + 2 * (H + H * H + bn);
}

void RnnPlan::set_weights(const float *stream, size_t count, int mem) {
    if (count != weight_count())
        throw Error(NB_ERR_WEIGHTS, "rnn: weight stream has " + std::to_string(count) + " floats, layer needs " +
                                        std::to_string(weight_count()));
    // blobs in the order input gate, hidden gate, output gate (rnn_layer.cc:69-73), each a connected-layer blob
    const size_t H = d.hidden;
    size_t pos = 0;
    FcPlan *gates[3] = {in_gate.get(), hid_gate.get(), out_gate.get()};
    for (FcPlan *g : gates) {
        const float *p = stream + pos;
        const size_t wn = H * g->d.inputs;
        g->set_weights(p + H, p, d.batch_normalize ? p + H + wn : nullptr, d.batch_normalize ? p + 2 * H + wn : nullptr,
                       d.batch_normalize ? p + 3 * H + wn : nullptr, mem);
        pos += H + wn + (d.batch_normalize ? 3 * H : 0);
    }
    ready = true;
}

size_t RnnPlan::reserve(bool x_rounded, bool x_foreign) {
    const size_t T = d.time_steps, B = d.batch, H = d.hidden;
    a_all.reserve(T * B * H);
    state.reserve(T * B * H);
    h0.reserve(B * H);
    const bool tf32 = h->math_mode == NB_MATH_TF32;
    ForwardOpts o;
    o.x_rounded = x_rounded; o.x_foreign = x_foreign;
    in_gate->reserve(o, (int)(T * B));
    o.x_rounded = false; o.x_foreign = false;
    hid_gate->reserve(o, (int)B);                   // step 0 reads the (unrounded) input-gate output
    o.x_rounded = tf32;
    out_gate->reserve(o, (int)((T > 1 ? T - 1 : 1) * B));
    return workspace_bytes();
}

void RnnPlan::forward(const float *x, float *out, bool x_rounded, bool round_out, bool x_foreign) {
    if (!ready) throw Error(NB_ERR_NO_WEIGHTS, "rnn: forward before set_weights");
    NB_REQUIRE(x && out, "rnn: null tensor pointer");
    const int T = d.time_steps, B = d.batch;
    const size_t BH = (size_t)B * d.hidden;
    const bool tf32 = h->math_mode == NB_MATH_TF32;     // stored states are then TF32 values, ready to be operands
    reserve(x_rounded, x_foreign);
    ForwardOpts o;
    // a_t for every step at once: the input gate does not depend on the state
    o.x_rounded = x_rounded; o.x_foreign = x_foreign;
    in_gate->forward(x, a_all.p, o, T * B);
    // step 0: the hidden gate reads the input gate's output, the output gate reads the hidden gate's
    o = ForwardOpts();
    o.round_out = tf32;
    hid_gate->forward(a_all.p, h0.p, o, B);
    o.addend = a_all.p; o.addend_post = true;
    hid_gate->forward(a_all.p, state.p, o, B);          // s_0 = a_0 + h_0 (same product, then the sum)
    // steps 1..T-1: h_t = hid(s_{t-1}), s_t = a_t + h_t
    for (int t = 1; t < T; t++) {
        ForwardOpts s;
        s.x_rounded = tf32; s.round_out = tf32;
        s.addend = a_all.p + t * BH; s.addend_post = true;
        hid_gate->forward(state.p + (t - 1) * BH, state.p + t * BH, s, B);
    }
    // outputs: step 0 from h_0, the others from their states in one product
    ForwardOpts q;
    q.x_rounded = tf32; q.round_out = round_out;
    out_gate->forward(h0.p, out, q, B);
    if (T > 1) out_gate->forward(state.p + BH, out + BH, q, (T - 1) * B);
}

}  // namespace nb
