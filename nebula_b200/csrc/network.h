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
    std::unique_ptr<RnnPlan> rnn;
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
    nb::DeviceBuffer input_nhwc, convert_tmp;
    int logits_layer = -1;
    bool weights_loaded = false;
    bool fuse = true;                   // fold 2x2/2 max-pools and shortcuts into the preceding convolution's epilogue

    // What a pass starts from: the reference's fp32 batch, or the first convolution's row-window tensor already
    // filled by the image-packing kernel.
    enum InputKind { IN_F32 = 0, IN_ROWWIN = 1 };

    // scratch of every layer is allocated for (math mode, fusion) before the first pass, so that passes allocate nothing
    int prepared_mode = -1;
    bool prepared_fuse = false;

    // pipelined host hand-off: two device input slots, a copy stream, events
    struct Slot {
        nb::DeviceBuffer f32;           // fp32 batch
        unsigned char *u8 = nullptr;    // decoded 8-bit batch
        cudaEvent_t copied = nullptr, done = nullptr;
        bool busy = false;
    } slot[2];
    int next_slot = 0;
    cudaStream_t copy_stream = nullptr;

    // CUDA-graph replay of a pass, per (input pointer, kind, math mode, fusion)
    bool use_graph = false;
    struct Graph { const void *input; int kind, mode; bool fuse; cudaGraphExec_t exec; unsigned long long launches; };
    std::vector<Graph> graphs;
    std::vector<const void *> seen_inputs;
    cudaStream_t capture_stream = nullptr;

    ~nb_network_s();
    size_t weight_count() const;
    size_t workspace_bytes() const;
    void build(const std::string &cfg_text, int batch_override);
    void load_weights(const float *stream, size_t count, int mem);
    void prepare();
    // one pass; dry: only size and allocate every layer's scratch
    void walk(const float *input, int kind, bool dry);
    void run(const float *input, int kind);
    void forward(const float *input) { run(input, IN_F32); }
    void forward_u8(const unsigned char *images_dev);
    bool first_layer_takes_rowwin() const;
    void submit(const void *input_host, bool u8, float *output_host);
    void wait();
    void drop_graphs();
    void layer_output(int index, float *dst, int mem, bool sync = true);
};
