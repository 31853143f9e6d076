// Plan objects behind the C ABI: per-layer state that a Nebula layer would own
// (re-laid-out weights, folded batch-norm vectors, scratch for layout changes).
#pragma once

#include <memory>

#include "nb_internal.h"

enum nb_plan_kind { NB_PLAN_CONV = 1, NB_PLAN_FC = 2, NB_PLAN_LSTM = 3, NB_PLAN_RNN = 4 };

struct nb_plan_s {
    int kind;
    nb_handle_s *h;
    nb_plan_s(int k, nb_handle_s *hh) : kind(k), h(hh) {}
    virtual ~nb_plan_s() {}
    virtual void output_dims(int dims[3]) const = 0;
    virtual size_t workspace_bytes() const = 0;     // scratch tensors the plan holds right now
};

namespace nb {

enum GemmPath { PATH_TC = 0, PATH_TC3 = 1, PATH_SIMT = 2 };

// Weights of one contraction in the three forms the math modes need.
struct WeightSet {
    DeviceBuffer exact;     // fp32 as loaded (re-laid out)
    DeviceBuffer hi, lo;    // TF32 split, built on first use
    bool split_ready = false;
    // hi = RN_tf32(w), lo = RN_tf32(w - hi); done when the weights are set, so that a forward pass allocates nothing
    void ensure_split(nb_handle_s *h) {
        if (split_ready) return;
        hi.alloc(exact.n, exact.guard);
        lo.alloc(exact.n, exact.guard);
        launch_split_tf32(h, exact.p, hi.p, lo.p, exact.n);
        split_ready = true;
    }
    size_t bytes() const { return (exact.n + hi.n + lo.n) * sizeof(float); }
};

// Folds the reference's inference batch-norm + bias into y = acc*scale + shift:
// (acc - mean) / (sqrt(var) + 1e-5) * gamma + bias  (common/batchnorm.cc:58-97,
// common/utils.cc:162-179).  Without batch-norm scale is absent and shift = bias.
void fold_bn(int n, const float *bias, const float *gamma, const float *mean, const float *var, bool has_bn,
             std::vector<float> &scale, std::vector<float> &shift);

struct ForwardOpts {
    bool x_nhwc = false;            // conv: x already NHWC (else NCHW, the reference layout)
    bool y_nhwc = false;            // conv: write y as NHWC
    bool x_rounded = false;         // x already holds TF32-rounded values
    bool x_rowwin = false;          // conv with at most 4 input channels: x already is this plan's row-window tensor
    // x is memory the library did not allocate: TMA loads never read it (their boxes also read what lies around a
    // tensor, which is only known to be mapped inside the library's arena), it is copied to scratch first
    bool x_foreign = false;
    bool round_out = false;         // store TF32-rounded outputs (consumer is a TF32 contraction)
    const float *addend = nullptr;  // optional tensor added before the activation (same layout as y)
    bool addend_post = false;       // ... or after it: y = act(...) + addend
    float *pool_out = nullptr;      // conv: write only the 2x2/2 max-pooled NHWC output here (y is not written)
    // conv (tensor-core path, NHWC): fuse the following shortcut layer -- add channels [0,min(C)) of this NHWC
    // tensor (sub-sampled when it is spatially larger) and apply `res_act` instead of the conv's own (linear) activation
    const float *residual = nullptr;
    int res_c = 0, res_h = 0, res_w = 0, res_act = 0;
};

struct ConvPlan : nb_plan_s {
    nb_conv2d_desc_t d;
    int OH, OW, Cp;
    WeightSet w;                    // [tap][F][Cp]
    // Small channel counts (3-channel input layers) cannot be addressed by TMA boxes:
    // the kernel's gather warps build those A tiles in shared memory instead.
    bool pack_ok = false;
    int Kpad = 0;
    WeightSet wp;                   // [F][Kpad], column = (kh,kw,c)
    // At most 4 input channels on the tensor-core path: the input is re-laid as [N][H][Wp][4] (zero pixels left and
    // right) and every filter ROW becomes one K slice of `rw_inner` floats that TMA fetches as overlapping windows.
    bool rowwin_ok = false;
    int rw_inner = 0, rw_wp = 0;
    WeightSet wr;                   // [kh][F][rw_inner], column = kw*4 + c
    DeviceBuffer x_rowwin;
    DeviceBuffer scale, shift;
    bool has_scale = false, ready = false;
    DeviceBuffer x_scratch, y_scratch;
    ConvPlan(nb_handle_s *h, const nb_conv2d_desc_t &desc);
    void set_weights(const float *weight, const float *bias, const float *g, const float *m, const float *v, int mem);
    void forward(const float *x, float *y, const ForwardOpts &o);
    // allocates the scratch tensors forward() would need with these options in the handle's current math mode
    // (forward() calls it too: a pass that was prepared allocates nothing); returns their total size in bytes
    size_t reserve(const ForwardOpts &o);
    size_t workspace_bytes() const override { return (x_rowwin.n + x_scratch.n + y_scratch.n) * sizeof(float); }
    void output_dims(int dims[3]) const override { dims[0] = d.filters; dims[1] = OH; dims[2] = OW; }
    GemmPath path(const ForwardOpts &o) const;
    // can the following 2x2 stride-2 max-pool be done in this layer's epilogue?
    bool can_fuse_pool() const;
    bool can_fuse_shortcut(int conn_c, int conn_h, int conn_w) const;
};

struct FcPlan : nb_plan_s {
    nb_fc_desc_t d;
    WeightSet w;                    // [out][in]
    DeviceBuffer scale, shift;
    bool has_scale = false, ready = false;
    DeviceBuffer x_scratch, split_ws;
    // when the input is an NHWC activation, columns are permuted (c,h,w) -> (h,w,c)
    int perm_c = 0, perm_h = 0, perm_w = 0;
    FcPlan(nb_handle_s *h, const nb_fc_desc_t &desc);
    void set_weights(const float *weight, const float *bias, const float *g, const float *m, const float *v, int mem);
    void forward(const float *x, float *y, const ForwardOpts &o, int rows = -1);
    size_t reserve(const ForwardOpts &o, int rows = -1);
    size_t workspace_bytes() const override { return (x_scratch.n + split_ws.n) * sizeof(float); }
    // split-K choice for `rows` input rows: number of K slices (1: none) and the tile width that goes with it
    void split_choice(bool tc, bool has_addend, int *S, int *block_n) const;
    void output_dims(int dims[3]) const override { dims[0] = d.outputs; dims[1] = 1; dims[2] = 1; }
    GemmPath path() const;
};

struct LstmPlan : nb_plan_s {
    nb_lstm_desc_t d;
    WeightSet wu;                   // [4H][in]  input-side gates, rows i,f,g,o
    WeightSet ww;                   // [4H][H]   recurrent gates
    // linear gate layers: one vector [4H] of summed biases (+ folded batch-norm shifts), applied by the input-side
    // GEMM.  Any other section activation is applied to each gate layer on its own (lstm_layer.cc:252-260), so the
    // two sides keep their own vectors: shift = input side, shift_w = recurrent side.
    DeviceBuffer shift, shift_w;
    DeviceBuffer h_zero;            // [B][H] zeros: h_{-1} when step 0 has to run the recurrent layer too
    DeviceBuffer pre;               // [T*B][4H] input-side projection for all steps
    DeviceBuffer z;                 // [B][4H]   gate pre-activations of one step
    DeviceBuffer cell_own;          // [T*B][H]  when the caller passes no cell buffer
    DeviceBuffer h_round;           // [T*B][H]  TF32-rounded hidden states
    DeviceBuffer x_round;           // [T*B][in]
    bool ready = false;
    LstmPlan(nb_handle_s *h, const nb_lstm_desc_t &desc);
    void set_weights(const float *stream, size_t count, int mem);
    size_t weight_count() const;
    // out_round (optional): receives a TF32-rounded copy of out
    void forward(const float *x, float *out, float *cell, bool x_rounded, float *out_round, bool x_foreign = true);
    size_t reserve(bool own_cell, bool x_rounded, bool have_out_round, bool x_foreign = true);
    size_t workspace_bytes() const override {
        return (pre.n + z.n + cell_own.n + h_round.n + x_round.n + h_zero.n) * sizeof(float);
    }
    void output_dims(int dims[3]) const override { dims[0] = d.hidden; dims[1] = 1; dims[2] = 1; }
};

// rnn_layer_t (rnn_layer.cc:34-141): three connected layers sharing one section (output, batch_normalize,
// activation).  Per time step t: a_t = in(x_t); h_t = hid(t ? s_{t-1} : a_0); s_t = a_t + h_t;
// out_t = outg(t ? s_t : h_0) -- step 0 feeds each gate its predecessor's output, as the reference's
// forward() without an argument does.
struct RnnPlan : nb_plan_s {
    nb_rnn_desc_t d;
    std::unique_ptr<FcPlan> in_gate, hid_gate, out_gate;
    DeviceBuffer a_all;             // [T*B][H] input-gate outputs of every step
    DeviceBuffer state;             // [T*B][H] s_t
    DeviceBuffer h0;                // [B][H]   hidden-gate output of step 0
    bool ready = false;
    RnnPlan(nb_handle_s *h, const nb_rnn_desc_t &desc);
    size_t weight_count() const;
    void set_weights(const float *stream, size_t count, int mem);
    void forward(const float *x, float *out, bool x_rounded, bool round_out, bool x_foreign = true);
    size_t reserve(bool x_rounded, bool x_foreign = true);
    size_t workspace_bytes() const override {
        return (a_all.n + state.n + h0.n) * sizeof(float) + in_gate->workspace_bytes() + hid_gate->workspace_bytes() +
               out_gate->workspace_bytes();
    }
    void output_dims(int dims[3]) const override { dims[0] = d.hidden; dims[1] = 1; dims[2] = 1; }
};

// host or device source -> freshly filled device buffer
// guard: floats behind the tensor that belong to the buffer (weight matrices: the rows past the last filter that
// the last tile's box covers)
void upload(nb_handle_s *h, DeviceBuffer &dst, const float *src, size_t n, int mem, size_t guard = 0);
void upload_vec(nb_handle_s *h, DeviceBuffer &dst, const std::vector<float> &v, size_t guard = 0);
// rows a weight tile may run past the last filter (the widest tile), plus a K block
inline size_t weight_guard(size_t row_floats) { return 256 * row_floats + 32; }
void upload_padded(nb_handle_s *h, DeviceBuffer &dst, std::vector<float> v, float fill);
std::vector<float> to_host(nb_handle_s *h, const float *src, size_t n, int mem);

}  // namespace nb
