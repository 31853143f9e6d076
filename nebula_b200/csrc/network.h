// Host-side mirror of the reference's network object: parses a network.cfg,
// builds the layer list with the reference's shape rules, loads a weight stream
// in weight-file order and runs the forward pass layer by layer
// (models/networks/network.cc:57-63,82-122; convolutional.cc:52-122;
// recurrent.cc:116-176).
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "plans.h"

namespace nb {

// The reference's layer_type_t codes (common/def.h:28-42).
enum LayerType {
    LT_UNDEFINED = 0, LT_CONNECTED, LT_CONVOLUTIONAL, LT_COST, LT_DROPOUT, LT_AVGPOOL, LT_MAXPOOL, LT_SHORTCUT,
    LT_SOFTMAX, LT_RNN, LT_LSTM, LT_RBM
};

struct Section {
    std::string name;
    std::map<std::string, std::string> settings;
    bool get(const std::string &key, int *v) const;
    bool get(const std::string &key, std::string *v) const;
};

// common/config.cc:44-75
std::vector<Section> parse_cfg(const std::string &text);
int activation_from_string(const std::string &s);

struct NetLayer {
    int type = LT_UNDEFINED;
    int C = 1, H = 1, W = 1;            // output extents per sample
    size_t size = 0;                    // output elements per sample (the layer's output_size)
    int activation = NB_ACT_UNDEFINED;
    bool nhwc = false;                  // buffer holds [rows][H][W][C] instead of NCHW
    DeviceBuffer out, out_round;
    float *out_ptr = nullptr;           // may alias another layer's buffer (dropout)
    float *out_round_ptr = nullptr;
    bool out_is_rounded = false;        // set per forward
    std::unique_ptr<ConvPlan> conv;
    std::unique_ptr<FcPlan> fc;
    std::unique_ptr<LstmPlan> lstm;
    nb_pool_desc_t pool;
    nb_shortcut_desc_t shortcut;
    int conn = -1;                      // shortcut: index of the connected layer
    size_t weight_floats = 0;
    bool materialised = true;           // false while this layer's own buffer is skipped by a fusion
};

}  // namespace nb

struct nb_network_s {
    nb_handle_s *h = nullptr;
    bool recurrent = false;
    int batch = 1, time_steps = 1;
    int in_c = 1, in_h = 1, in_w = 1;
    size_t input_size = 0;              // elements per row (sample or time step)
    int rows = 1;                       // batch * time_steps
    std::vector<std::unique_ptr<nb::NetLayer>> layers;
    nb::DeviceBuffer input_dev, input_nhwc, convert_tmp;
    int logits_layer = -1;
    bool weights_loaded = false;
    bool fuse = true;                   // fold 2x2/2 max-pools into the preceding convolution's epilogue

    size_t weight_count() const;
    void build(const std::string &cfg_text, int batch_override);
    void load_weights(const float *stream, size_t count, int mem);
    void forward(const float *input);
    void layer_output(int index, float *dst, int mem);
};
