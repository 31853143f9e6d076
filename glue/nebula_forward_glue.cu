// Replacement bodies of the reference's GPU forward methods on top of libnebula_b200.so.
//
// Written against the reference's own headers; nothing of the reference is changed or copied.  Each body
// replaces the method of the same name in models/layers/<layer>.cu (cited per method).  The reference's
// classes have no member to keep a plan in, so plans live in a table keyed by the layer object; they are
// created on the layer's first forward call -- by then init() has fixed every extent and init_weight() has
// filled the host-side weight arrays, which is all a plan needs.  One library handle per network_t.
//
// Training (_backward_, _update_) stays on the reference's own code.
#ifdef NEBULA_B200
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <map>
#include <vector>

#include "nebula_b200.h"

#include "connected_layer.h"
#include "convolutional_layer.h"
#include "lstm_layer.h"
#include "network.h"
#include "pooling_layer.h"
#include "rbm_layer.h"
#include "rnn_layer.h"
#include "shortcut_layer.h"
#include "softmax_layer.h"

namespace nebula {
namespace nb_glue {

// The reference's convention on errors is a message and exit(1) (e.g. layer.cc:103-107).
inline void check(int status, nb_handle_t h, const char *what) {
    if (status == NB_OK) return;
    std::cerr << "Error: " << what << ": " << nb_last_error(h) << std::endl;
    exit(1);
}

// One handle per network (replaces cudaSetDevice(0) + cublasCreate, models/networks/network.cc:44-51).
inline nb_handle_t handle_of(network_t *network) {
    static std::map<network_t *, nb_handle_t> handles;
    nb_handle_t &h = handles[network];
    if (!h) {
        const char *dev = getenv("NEBULA_B200_DEVICE");         // rank-aware where the launcher sets it
        check(nb_create(dev ? atoi(dev) : 0, &h), NULL, "nb_create");
        const char *math = getenv("NEBULA_B200_MATH");          // tf32 (default) | tf32x3 | fp32
        std::string m = math ? math : "tf32";
        check(nb_set_math_mode(h, m == "fp32" ? NB_MATH_FP32 : (m == "tf32x3" ? NB_MATH_TF32X3 : NB_MATH_TF32)), h, "math mode");
    }
    return h;
}

inline nb_plan_t &plan_slot(const layer_t *layer) {
    static std::map<const layer_t *, nb_plan_t> plans;
    return plans[layer];
}

}  // namespace nb_glue

// ---- convolutional_layer_t::_forward_ (models/layers/convolutional_layer.cu:11-84)
void convolutional_layer_t::_forward_() {
    nb_handle_t h = nb_glue::handle_of(network);
    nb_plan_t &plan = nb_glue::plan_slot(this);
    if (!plan) {
        nb_conv2d_desc_t d = {(int)network->batch_size, (int)input_channel, (int)input_height, (int)input_width,
                              (int)num_filters, (int)filter_size, (int)stride, (int)padding,
                              (int)batch_normalize, (int)activation_type, NB_LAYOUT_NCHW};
        nb_glue::check(nb_conv2d_plan_create(h, &d, &plan), h, "convolutional plan");
        nb_glue::check(nb_conv2d_set_weights(plan, weight, bias, scale, rolling_mean, rolling_variance, NB_MEM_HOST), h,
                       "convolutional weights");
    }
    float *input_data_dev = prev_layer ? prev_layer->output_data_dev : network->input_data_dev;
    nb_glue::check(nb_conv2d_forward(plan, input_data_dev, output_data_dev), h, "convolutional forward");
}

// ---- connected_layer_t::_forward_ / _forward_(float*) (models/layers/connected_layer.cu:10-88)
static void connected_forward(connected_layer_t *l, network_t *network, nb_plan_t &plan, const nb_fc_desc_t &d,
                              const float *w, const float *b, const float *s, const float *m, const float *v,
                              const float *x_dev, float *y_dev) {
    nb_handle_t h = nb_glue::handle_of(network);
    if (!plan) {
        nb_glue::check(nb_fc_plan_create(h, &d, &plan), h, "connected plan");
        nb_glue::check(nb_fc_set_weights(plan, w, b, s, m, v, NB_MEM_HOST), h, "connected weights");
    }
    nb_glue::check(nb_fc_forward(plan, x_dev, y_dev), h, "connected forward");
    (void)l;
}
void connected_layer_t::_forward_() {
    nb_fc_desc_t d = {(int)network->batch_size, (int)input_size, (int)output_size, (int)batch_normalize, (int)activation_type};
    float *input_data_dev = prev_layer ? prev_layer->output_data_dev : network->input_data_dev;
    connected_forward(this, network, nb_glue::plan_slot(this), d, weight, bias, scale, rolling_mean, rolling_variance,
                      input_data_dev, output_data_dev);
}
void connected_layer_t::_forward_(float *m_input_data_dev) {
    nb_fc_desc_t d = {(int)network->batch_size, (int)input_size, (int)output_size, (int)batch_normalize, (int)activation_type};
    float *input_data_dev = m_input_data_dev ? m_input_data_dev
                                             : (prev_layer ? prev_layer->output_data_dev : network->input_data_dev);
    connected_forward(this, network, nb_glue::plan_slot(this), d, weight, bias, scale, rolling_mean, rolling_variance,
                      input_data_dev, output_data_dev);
}

// ---- pooling_layer_t::_forward_ (models/layers/pooling_layer.cu:150-175)
void pooling_layer_t::_forward_() {
    nb_handle_t h = nb_glue::handle_of(network);
    nb_pool_desc_t d = {(int)network->batch_size, (int)input_channel, (int)input_height, (int)input_width,
                        (int)filter_size, (int)stride, (int)padding,
                        layer_type == MAXPOOL_LAYER ? NB_POOL_MAX : NB_POOL_AVG, NB_LAYOUT_NCHW};
    float *input_data_dev = prev_layer ? prev_layer->output_data_dev : network->input_data_dev;
    nb_glue::check(nb_pool_forward(h, &d, input_data_dev, output_data_dev), h, "pooling forward");
}

// ---- shortcut_layer_t::_forward_ (models/layers/shortcut_layer.cu:27-52); input_* are the connection's extents
// (shortcut_layer.cc:43-50), output_* the previous layer's
void shortcut_layer_t::_forward_() {
    nb_handle_t h = nb_glue::handle_of(network);
    nb_shortcut_desc_t d = {(int)network->batch_size, (int)input_channel, (int)input_height, (int)input_width,
                            (int)output_channel, (int)output_height, (int)output_width, (int)activation_type, NB_LAYOUT_NCHW};
    float *input_data_dev = prev_layer ? prev_layer->output_data_dev : network->input_data_dev;
    nb_glue::check(nb_shortcut_forward(h, &d, input_data_dev, connection->output_data_dev, output_data_dev), h,
                   "shortcut forward");
}

// ---- softmax_layer_t::_forward_ (models/layers/softmax_layer.cu:30-40); the copy to the host array stays
void softmax_layer_t::_forward_() {
    nb_handle_t h = nb_glue::handle_of(network);
    float *input_data_dev = prev_layer ? prev_layer->output_data_dev : network->input_data_dev;
    nb_glue::check(nb_softmax_forward(h, input_data_dev, output_data_dev, (int)network->batch_size, (int)input_size), h,
                   "softmax forward");
    nb_glue::check(nb_synchronize(h), h, "softmax forward");
    cudaMemcpy(output_data, output_data_dev, output_size * network->batch_size * sizeof(float), cudaMemcpyDeviceToHost);
}

// The weight arrays of a recurrent layer's connected sub-layers are private to connected_layer_t, but the layer's own
// store_weight() writes them in weight-file order (lstm_layer.cc:214-227, rnn_layer.cc:75-79): that stream, read
// back from a scratch file, is exactly what nb_lstm_set_weights / nb_rnn_set_weights take.
template <class Layer>
static std::vector<float> weight_stream_of(Layer *layer) {
    char path[] = "/tmp/nebula_b200_weights_XXXXXX";
    int fd = mkstemp(path);
    if (fd < 0) { std::cerr << "Error: cannot create a scratch file for the recurrent layer's weights" << std::endl; exit(1); }
    close(fd);
    std::fstream f(path, std::ios::in | std::ios::out | std::ios::binary | std::ios::trunc);
    layer->store_weight(f);
    f.flush();
    const std::streamoff bytes = f.tellp();
    std::vector<float> stream((size_t)bytes / sizeof(float));
    f.seekg(0);
    f.read((char *)stream.data(), bytes);
    f.close();
    remove(path);
    return stream;
}

// ---- lstm_layer_t::_forward_ (models/layers/lstm_layer.cu:20-140): the eight sub-layers, the pointer bumping and
// the per-step launches collapse into one call over all time steps
void lstm_layer_t::_forward_() {
    nb_handle_t h = nb_glue::handle_of(network);
    nb_plan_t &plan = nb_glue::plan_slot(this);
    const int T = (int)network->time_step, B = (int)(network->batch_size / network->time_step);
    if (!plan) {
        nb_lstm_desc_t d = {T, B, (int)input_size, (int)output_size, (int)batch_normalize, (int)activation_type};
        nb_glue::check(nb_lstm_plan_create(h, &d, &plan), h, "lstm plan");
        std::vector<float> stream = weight_stream_of(this);     // iW,fW,oW,cW,iU,fU,oU,cU (lstm_layer.cc:194-206)
        nb_glue::check(nb_lstm_set_weights(plan, stream.data(), stream.size(), NB_MEM_HOST), h, "lstm weights");
    }
    float *input_data_dev = prev_layer ? prev_layer->output_data_dev : network->input_data_dev;
    nb_glue::check(nb_lstm_forward(plan, input_data_dev, output_data_dev, cell_state_dev), h, "lstm forward");
}

// ---- rnn_layer_t::_forward_ (models/layers/rnn_layer.cu; CPU semantics of rnn_layer.cc:91-141)
void rnn_layer_t::_forward_() {
    nb_handle_t h = nb_glue::handle_of(network);
    nb_plan_t &plan = nb_glue::plan_slot(this);
    const int T = (int)network->time_step, B = (int)(network->batch_size / network->time_step);
    if (!plan) {
        nb_rnn_desc_t d = {T, B, (int)input_size, (int)output_size, (int)batch_normalize, (int)activation_type};
        nb_glue::check(nb_rnn_plan_create(h, &d, &plan), h, "rnn plan");
        std::vector<float> stream = weight_stream_of(this);     // input, hidden, output gate (rnn_layer.cc:69-73)
        nb_glue::check(nb_rnn_set_weights(plan, stream.data(), stream.size(), NB_MEM_HOST), h, "rnn weights");
    }
    float *input_data_dev = prev_layer ? prev_layer->output_data_dev : network->input_data_dev;
    nb_glue::check(nb_rnn_forward(plan, input_data_dev, output_data_dev), h, "rnn forward");
}

// ---- rbm_layer_t::_forward_ (models/layers/rbm_layer.cu; rbm_layer.cc:345-374): a connected layer on the hidden bias
void rbm_layer_t::_forward_() {
    nb_handle_t h = nb_glue::handle_of(network);
    nb_plan_t &plan = nb_glue::plan_slot(this);
    if (!plan) {
        nb_fc_desc_t d = {(int)network->batch_size, (int)input_size, (int)output_size, 0, (int)activation_type};
        nb_glue::check(nb_fc_plan_create(h, &d, &plan), h, "rbm plan");
        nb_glue::check(nb_fc_set_weights(plan, weight, hidden_bias, NULL, NULL, NULL, NB_MEM_HOST), h, "rbm weights");
    }
    float *input_data_dev = prev_layer ? prev_layer->output_data_dev : network->input_data_dev;
    nb_glue::check(nb_fc_forward(plan, input_data_dev, output_data_dev), h, "rbm forward");
}

}  // namespace nebula
#endif  // NEBULA_B200
