// Driver that runs the UNMODIFIED reference CPU path as the parity checker and
// as the timed CPU baseline.  It is compiled against the reference's own
// sources (common/*.cc, models/layers/*.cc, models/networks/network.cc; see the
// Makefile beside this file) and contains none of them.
//
// TEST INFRASTRUCTURE ONLY.  The product library never links, loads or runs
// this program; only the tests, the smoke check and the bench's CPU-baseline
// leg execute it.
//
// What it does: subclasses the reference's abstract network_t
// (models/networks/network.h:17-98), builds the layer list from a network.cfg
// the way the reference's network classes do (section name -> layer class ->
// layer->init(section)), fills input_data from a raw fp32 file, loads a
// reference-format weight file through network_t::init (network.cc:82-122),
// calls network_t::forward() (network.cc:57-63) and writes layers' output_data
// as raw fp32.  `cost` sections are skipped (they need labels and are not part
// of inference); everything else is the reference's code.
//
// Usage:
//   nebula_ref --cfg net.cfg --input in.bin --weights w.wgh [--out out.bin]
//              [--out-layer i] [--dump-dir dir] [--recurrent] [--threads n]
//              [--batch b] [--reps r]
// Prints one JSON line with the forward() wall times in milliseconds.
#ifndef CUSTOM_BLAS
#include <cblas.h>
#endif
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>
#include <unistd.h>

#include "config.h"
#include "layer.h"
#include "network.h"
#include "connected_layer.h"
#include "convolutional_layer.h"
#include "dropout_layer.h"
#include "lstm_layer.h"
#include "pooling_layer.h"
#include "rbm_layer.h"
#include "rnn_layer.h"
#include "shortcut_layer.h"
#include "softmax_layer.h"

namespace {

struct options_t {
    std::string cfg, input, weights, out, dump_dir;
    int out_layer = -1;
    bool recurrent = false;
    int threads = 0;
    int batch = 0;
    int reps = 1;
};

class ref_network_t : public nebula::network_t {
public:
    explicit ref_network_t(const options_t &o) : opt(o) {}
    // Layers are deliberately never deleted: the reference's dropout layer
    // aliases its neighbour's buffers (dropout_layer.cc:37-46) and a used LSTM
    // holds advanced pointers, so running their destructors is not safe.
    ~ref_network_t() {}
    void run(const std::string) {}

    size_t layer_count() const { return layers.size(); }
    nebula::layer_t *layer(size_t i) { return layers[i]; }
    size_t input_elems() const { return (size_t)input_size * batch_size; }

protected:
    void init_network(const std::string cfg_path) {
        nebula::config_t config;
        config.parse(cfg_path);
        for (size_t s = 0; s < config.sections.size(); s++) {
            nebula::section_config_t sec = config.sections[s];
            if (sec.name == "net") {
                sec.get_setting("num_threads", &num_threads);
                if (opt.threads > 0) num_threads = opt.threads;
                sec.get_setting("batch", &batch_size);
                if (opt.batch > 0) batch_size = opt.batch;
                if (opt.recurrent) {
                    sec.get_setting("input_size", &input_size);
                    sec.get_setting("time_steps", &time_step);
                    batch_size *= time_step;
                } else {
                    sec.get_setting("height", &input_height);
                    sec.get_setting("width", &input_width);
                    sec.get_setting("channels", &input_channel);
                    input_size = input_height * input_width * input_channel;
                }
                continue;
            }
            if (sec.name == "cost") continue;
            nebula::layer_t *prev = layers.size() ? layers.back() : NULL;
            nebula::layer_t *l = NULL;
            if (sec.name == "convolutional") l = new nebula::convolutional_layer_t(this, prev, nebula::CONVOLUTIONAL_LAYER);
            else if (sec.name == "connected") l = new nebula::connected_layer_t(this, prev, nebula::CONNECTED_LAYER);
            else if (sec.name == "dropout") l = new nebula::dropout_layer_t(this, prev, nebula::DROPOUT_LAYER);
            else if (sec.name == "maxpool") l = new nebula::pooling_layer_t(this, prev, nebula::MAXPOOL_LAYER);
            else if (sec.name == "avgpool") l = new nebula::pooling_layer_t(this, prev, nebula::AVGPOOL_LAYER);
            else if (sec.name == "shortcut") l = new nebula::shortcut_layer_t(this, prev, nebula::SHORTCUT_LAYER);
            else if (sec.name == "softmax") l = new nebula::softmax_layer_t(this, prev, nebula::SOFTMAX_LAYER);
            else if (sec.name == "lstm") l = new nebula::lstm_layer_t(this, prev, nebula::LSTM_LAYER);
            else if (sec.name == "rnn") l = new nebula::rnn_layer_t(this, prev, nebula::RNN_LAYER);
            else if (sec.name == "rbm") l = new nebula::rbm_layer_t(this, prev, nebula::RBM_LAYER);
            else {
                std::cerr << "ref_driver: unknown section " << sec.name << std::endl;
                exit(2);
            }
            if (!layers.size()) input_layer = l;
            l->init(sec);
            layers.push_back(l);
        }
        num_layers = layers.size();
#ifndef CUSTOM_BLAS
        openblas_set_num_threads(num_threads);
#endif
    }
    void init_data(const std::string) {
        input_data = new float[input_elems()]();
        std::ifstream f(opt.input.c_str(), std::ios::binary);
        if (!f.is_open()) { std::cerr << "ref_driver: cannot open " << opt.input << std::endl; exit(2); }
        f.read((char *)input_data, input_elems() * sizeof(float));
        if ((size_t)f.gcount() != input_elems() * sizeof(float)) {
            std::cerr << "ref_driver: short input file (" << f.gcount() << " bytes)" << std::endl;
            exit(2);
        }
    }
    void load_data(const unsigned) {}
    void print_results() {}

private:
    options_t opt;
};

void write_floats(const std::string &path, const float *p, size_t n) {
    std::ofstream f(path.c_str(), std::ios::binary);
    f.write((const char *)p, n * sizeof(float));
}

}  // namespace

int main(int argc, char **argv) {
    options_t o;
    for (int i = 1; i < argc; i++) {
        std::string a = argv[i];
        auto next = [&]() -> std::string {
            if (i + 1 >= argc) { std::cerr << "missing value for " << a << std::endl; exit(2); }
            return argv[++i];
        };
        if (a == "--cfg") o.cfg = next();
        else if (a == "--input") o.input = next();
        else if (a == "--weights") o.weights = next();
        else if (a == "--out") o.out = next();
        else if (a == "--out-layer") o.out_layer = atoi(next().c_str());
        else if (a == "--dump-dir") o.dump_dir = next();
        else if (a == "--recurrent") o.recurrent = true;
        else if (a == "--threads") o.threads = atoi(next().c_str());
        else if (a == "--batch") o.batch = atoi(next().c_str());
        else if (a == "--reps") o.reps = atoi(next().c_str());
        else { std::cerr << "unknown argument " << a << std::endl; return 2; }
    }
    if (o.cfg.empty() || o.input.empty() || o.weights.empty()) {
        std::cerr << "usage: nebula_ref --cfg c --input i --weights w [--out o] ..." << std::endl;
        return 2;
    }

    std::vector<double> ms;
    // The reference prints progress on stdout from init(); keep stdout for the
    // JSON line only by silencing it during the run.
    std::streambuf *saved = std::cout.rdbuf();
    std::ofstream devnull("/dev/null");
    // A recurrent reference network is single-shot: lstm_layer_t::forward()
    // leaves its eight sub-layers' pointers advanced (lstm_layer.cc:334-345),
    // so every repetition builds a fresh network object.
    ref_network_t *net = NULL;
    for (int r = 0; r < std::max(1, o.reps); r++) {
        if (!net || o.recurrent) {
            net = new ref_network_t(o);
            std::cout.rdbuf(devnull.rdbuf());
            net->init("test", o.cfg, "", o.weights);
            std::cout.rdbuf(saved);
        }
        auto t0 = std::chrono::steady_clock::now();
        net->forward();
        auto t1 = std::chrono::steady_clock::now();
        ms.push_back(std::chrono::duration<double, std::milli>(t1 - t0).count());
    }

    int nl = (int)net->layer_count();
    int ol = o.out_layer < 0 ? nl + o.out_layer : o.out_layer;
    if (ol < 0 || ol >= nl) { std::cerr << "bad --out-layer" << std::endl; return 2; }
    if (!o.out.empty()) {
        nebula::layer_t *l = net->layer(ol);
        write_floats(o.out, l->output_data, (size_t)l->output_size * net->batch_size);
    }
    if (!o.dump_dir.empty()) {
        for (int i = 0; i < nl; i++) {
            nebula::layer_t *l = net->layer(i);
            char name[64];
            snprintf(name, sizeof name, "/layer_%03d.bin", i);
            write_floats(o.dump_dir + name, l->output_data, (size_t)l->output_size * net->batch_size);
        }
    }
    printf("{\"layers\": %d, \"batch\": %u, \"threads\": %u, \"forward_ms\": [", nl, net->batch_size, net->num_threads);
    for (size_t i = 0; i < ms.size(); i++) printf("%s%.3f", i ? ", " : "", ms[i]);
    printf("], \"out_layer\": %d, \"out_elems\": %zu}\n", ol,
           (size_t)net->layer(ol)->output_size * net->batch_size);
    fflush(stdout);
    _exit(0);
}
