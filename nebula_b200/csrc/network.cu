// Network executor: cfg -> layer list -> forward.  Activations of spatial layers
// are kept NHWC in HBM (channels innermost) so that every convolution reads its
// input through TMA boxes and writes its output rows contiguously; the
// reference's NCHW view of any layer is materialised on request.
#include "network.h"

#include <algorithm>
#include <cstdlib>
#include <sstream>

namespace nb {

static std::string lower(std::string s) {
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    return s;
}

bool Section::get(const std::string &key, int *v) const {
    auto it = settings.find(lower(key));
    if (it == settings.end()) return false;
    std::stringstream ss(it->second);       // same extraction as the reference's get_setting<T> (common/config.h:23-29)
    int t;
    if (ss >> t) *v = t;
    return true;
}
bool Section::get(const std::string &key, std::string *v) const {
    auto it = settings.find(lower(key));
    if (it == settings.end()) return false;
    *v = it->second;
    return true;
}

std::vector<Section> parse_cfg(const std::string &text) {
    std::vector<Section> sections;
    std::istringstream in(text);
    std::string line;
    while (std::getline(in, line)) {
        line.erase(std::remove(line.begin(), line.end(), ' '), line.end());
        line.erase(std::remove(line.begin(), line.end(), '\r'), line.end());
        if (line.empty() || line[0] == '#') continue;
        if (line[0] == '[') {
            Section s;
            s.name = line.substr(1, line.size() - 2);
            sections.push_back(s);
            continue;
        }
        const size_t eq = line.find('=');
        if (eq == std::string::npos) throw Error(NB_ERR_CONFIG, "invalid config line: " + line);
        if (sections.empty()) throw Error(NB_ERR_CONFIG, "setting before the first [section]: " + line);
        // std::map::insert in the reference keeps the first value of a repeated key
        sections.back().settings.insert({lower(line.substr(0, eq)), lower(line.substr(eq + 1))});
    }
    return sections;
}

int activation_from_string(const std::string &s) {
    static const char *names[] = {"undefined_activation", "elu", "hardtan", "leaky", "lhtan", "linear", "loggy",
                                  "logistic", "plse", "ramp", "relie", "relu", "stair", "tanh"};
    for (int i = 1; i < NB_ACT_COUNT; i++)
        if (s == names[i]) return i;
    return NB_ACT_UNDEFINED;
}

static int section_activation(const Section &s, const char *what) {
    std::string a;
    if (!s.get("activation", &a)) throw Error(NB_ERR_CONFIG, std::string(what) + ": missing activation");
    const int act = activation_from_string(a);
    if (act == NB_ACT_UNDEFINED) throw Error(NB_ERR_CONFIG, std::string(what) + ": unknown activation " + a);
    return act;
}

}  // namespace nb

using namespace nb;

size_t nb_network_s::weight_count() const {
    size_t n = 0;
    for (auto &l : layers) n += l->weight_floats;
    return n;
}

void nb_network_s::build(const std::string &cfg_text, int batch_override) {
    std::vector<Section> secs = parse_cfg(cfg_text);
    if (secs.empty() || secs[0].name != "net") throw Error(NB_ERR_CONFIG, "the first section must be [net]");
    for (auto &s : secs)
        if (s.name == "lstm" || s.name == "rnn") recurrent = true;
    const Section &net = secs[0];
    int isz = 0;
    if (net.get("input_size", &isz)) recurrent = true;
    net.get("batch", &batch);
    if (batch_override > 0) batch = batch_override;
    if (batch <= 0) throw Error(NB_ERR_CONFIG, "[net] batch must be positive");
    if (recurrent) {
        net.get("time_steps", &time_steps);
        if (isz <= 0 || time_steps <= 0) throw Error(NB_ERR_CONFIG, "[net] input_size and time_steps must be positive");
        in_c = isz; in_h = in_w = 1;
        input_size = (size_t)isz;
        rows = batch * time_steps;          // recurrent.cc:139
    } else {
        net.get("height", &in_h);
        net.get("width", &in_w);
        net.get("channels", &in_c);
        if (in_h <= 0 || in_w <= 0 || in_c <= 0) throw Error(NB_ERR_CONFIG, "[net] height/width/channels must be positive");
        input_size = (size_t)in_h * in_w * in_c;
        rows = batch;
    }

    int C = in_c, H = in_h, W = in_w;       // running output extents
    size_t flat = input_size;
    for (size_t si = 1; si < secs.size(); si++) {
        const Section &s = secs[si];
        if (s.name == "net") throw Error(NB_ERR_CONFIG, "more than one [net] section");
        if (s.name == "cost") continue;     // needs labels; not part of inference
        std::unique_ptr<NetLayer> l(new NetLayer());
        if (s.name == "convolutional") {
            if (recurrent) throw Error(NB_ERR_CONFIG, "[convolutional] in a recurrent network");
            nb_conv2d_desc_t d{};
            d.batch = rows; d.channels = C; d.height = H; d.width = W;
            d.filters = 1; d.size = 1; d.stride = 1; d.padding = 0;
            s.get("filters", &d.filters); s.get("size", &d.size); s.get("stride", &d.stride);
            s.get("padding", &d.padding); s.get("batch_normalize", &d.batch_normalize);
            d.activation = section_activation(s, "convolutional");
            d.layout = NB_LAYOUT_NHWC;
            if (flat != (size_t)C * H * W) throw Error(NB_ERR_CONFIG, "[convolutional] after a flat layer");
            l->type = LT_CONVOLUTIONAL;
            l->conv.reset(new ConvPlan(h, d));
            l->C = d.filters; l->H = l->conv->OH; l->W = l->conv->OW;
            l->activation = d.activation;
            l->nhwc = true;
            l->weight_floats = (size_t)d.filters + (size_t)d.filters * C * d.size * d.size +
                               (d.batch_normalize ? 3 * (size_t)d.filters : 0);
        } else if (s.name == "connected") {
            nb_fc_desc_t d{};
            d.batch = rows; d.inputs = (int)flat; d.outputs = 0;
            s.get("output", &d.outputs); s.get("batch_normalize", &d.batch_normalize);
            d.activation = section_activation(s, "connected");
            l->type = LT_CONNECTED;
            l->fc.reset(new FcPlan(h, d));
            // the input buffer is NHWC when it comes from a spatial layer
            if (!layers.empty() && layers.back()->nhwc && H * W > 1) {
                l->fc->perm_c = C; l->fc->perm_h = H; l->fc->perm_w = W;
            }
            l->C = d.outputs; l->H = l->W = 1;
            l->activation = d.activation;
            l->weight_floats = (size_t)d.outputs + (size_t)d.outputs * flat + (d.batch_normalize ? 3 * (size_t)d.outputs : 0);
            logits_layer = (int)layers.size();
        } else if (s.name == "maxpool" || s.name == "avgpool") {
            if (recurrent) throw Error(NB_ERR_CONFIG, "pooling in a recurrent network");
            if (flat != (size_t)C * H * W) throw Error(NB_ERR_CONFIG, "pooling after a flat layer");
            nb_pool_desc_t d{};
            d.batch = rows; d.channels = C; d.height = H; d.width = W;
            d.stride = 1;
            s.get("stride", &d.stride);
            d.size = d.stride;                      // pooling_layer.cc:43-48
            s.get("size", &d.size);
            d.padding = (d.size - 1) / 2;
            s.get("padding", &d.padding);
            if (d.stride <= 0 || d.size <= 0 || d.padding < 0) throw Error(NB_ERR_CONFIG, "pooling: bad geometry");
            d.mode = s.name == "maxpool" ? NB_POOL_MAX : NB_POOL_AVG;
            d.layout = NB_LAYOUT_NHWC;
            l->type = s.name == "maxpool" ? LT_MAXPOOL : LT_AVGPOOL;
            l->pool = d;
            l->C = C; l->H = (H + 2 * d.padding) / d.stride; l->W = (W + 2 * d.padding) / d.stride;
            l->nhwc = true;
        } else if (s.name == "shortcut") {
            if (recurrent) throw Error(NB_ERR_CONFIG, "shortcut in a recurrent network");
            int hops = 0;
            s.get("hops", &hops);
            const int me = (int)layers.size();
            const int conn = me - hops;             // shortcut_layer.cc:39-41 walks prev_layer `hops` times
            if (hops <= 0 || conn < 0) throw Error(NB_ERR_CONFIG, "shortcut: hops reaches before the first layer");
            NetLayer &cl = *layers[conn];
            if (!cl.nhwc || layers.empty() || !layers.back()->nhwc)
                throw Error(NB_ERR_CONFIG, "shortcut: both inputs must be spatial layers");
            nb_shortcut_desc_t d{};
            d.batch = rows;
            d.conn_channels = cl.C; d.conn_height = cl.H; d.conn_width = cl.W;
            d.out_channels = C; d.out_height = H; d.out_width = W;
            d.activation = section_activation(s, "shortcut");
            d.layout = NB_LAYOUT_NHWC;
            l->type = LT_SHORTCUT;
            l->shortcut = d;
            l->conn = conn;
            l->C = C; l->H = H; l->W = W;
            l->activation = d.activation;
            l->nhwc = true;
        } else if (s.name == "dropout") {
            l->type = LT_DROPOUT;                   // aliases the previous layer's buffers (dropout_layer.cc:37-46)
            l->C = C; l->H = H; l->W = W;
            l->nhwc = !layers.empty() && layers.back()->nhwc;
            if (layers.empty()) throw Error(NB_ERR_UNSUPPORTED, "[dropout] as the first layer");
        } else if (s.name == "softmax") {
            l->type = LT_SOFTMAX;
            l->C = (int)flat; l->H = l->W = 1;
            if (!layers.empty() && layers.back()->nhwc && H * W > 1)
                throw Error(NB_ERR_UNSUPPORTED, "[softmax] directly after a spatial layer");
        } else if (s.name == "lstm") {
            nb_lstm_desc_t d{};
            d.time_steps = time_steps; d.batch = batch; d.inputs = (int)flat; d.hidden = 0;
            s.get("output", &d.hidden); s.get("batch_normalize", &d.batch_normalize);
            d.activation = section_activation(s, "lstm");
            l->type = LT_LSTM;
            l->lstm.reset(new LstmPlan(h, d));
            l->C = d.hidden; l->H = l->W = 1;
            l->activation = d.activation;
            l->weight_floats = l->lstm->weight_count();
        } else if (s.name == "rnn") {
            nb_rnn_desc_t d{};
            d.time_steps = time_steps; d.batch = batch; d.inputs = (int)flat; d.hidden = 0;
            s.get("output", &d.hidden); s.get("batch_normalize", &d.batch_normalize);
            d.activation = section_activation(s, "rnn");
            l->type = LT_RNN;
            l->rnn.reset(new RnnPlan(h, d));
            l->C = d.hidden; l->H = l->W = 1;
            l->activation = d.activation;
            l->weight_floats = l->rnn->weight_count();
        } else if (s.name == "rbm") {
            // inference through a pre-trained RBM is a connected layer on the hidden bias
            // (rbm_layer_t::forward, rbm_layer.cc:345-374; weight file: hidden_bias, weight, rbm_layer.cc:150-157)
            nb_fc_desc_t d{};
            d.batch = rows; d.inputs = (int)flat; d.outputs = 0;
            s.get("output", &d.outputs);
            d.activation = section_activation(s, "rbm");
            l->type = LT_RBM;
            l->fc.reset(new FcPlan(h, d));
            if (!layers.empty() && layers.back()->nhwc && H * W > 1) {
                l->fc->perm_c = C; l->fc->perm_h = H; l->fc->perm_w = W;
            }
            l->C = d.outputs; l->H = l->W = 1;
            l->activation = d.activation;
            l->weight_floats = (size_t)d.outputs + (size_t)d.outputs * flat;
        } else {
            throw Error(NB_ERR_CONFIG, "unknown layer type " + s.name);
        }
        C = l->C; H = l->H; W = l->W;
        flat = (size_t)C * H * W;
        l->size = flat;
        if (l->type == LT_DROPOUT) {
            l->out_ptr = layers.back()->out_ptr;
            l->out_round_ptr = layers.back()->out_round_ptr;
        } else {
            l->out.alloc(flat * rows);
            l->out_ptr = l->out.p;
            if (l->type == LT_LSTM) {
                l->out_round.alloc(flat * rows);
                l->out_round_ptr = l->out_round.p;
            }
        }
        layers.push_back(std::move(l));
    }
    if (layers.empty()) throw Error(NB_ERR_CONFIG, "network has no layers");
}

void nb_network_s::load_weights(const float *stream, size_t count, int mem) {
    NB_REQUIRE(stream != nullptr || count == 0, "null weight stream");
    const size_t need = weight_count();
    if (count != need)
        throw Error(NB_ERR_WEIGHTS, "weight stream has " + std::to_string(count) + " floats, the network needs " +
                                        std::to_string(need));
    size_t pos = 0;
    for (auto &lp : layers) {
        NetLayer &l = *lp;
        const float *p = stream + pos;
        if (l.type == LT_CONVOLUTIONAL) {
            const nb_conv2d_desc_t &d = l.conv->d;
            const size_t F = d.filters, wn = F * d.channels * d.size * d.size;
            // bias, weight, then scale / rolling mean / rolling variance (convolutional_layer.cc:257-316)
            l.conv->set_weights(p + F, p, d.batch_normalize ? p + F + wn : nullptr,
                                d.batch_normalize ? p + 2 * F + wn : nullptr, d.batch_normalize ? p + 3 * F + wn : nullptr,
                                mem);
        } else if (l.type == LT_CONNECTED || l.type == LT_RBM) {
            const nb_fc_desc_t &d = l.fc->d;
            const size_t O = d.outputs, wn = O * d.inputs;
            l.fc->set_weights(p + O, p, d.batch_normalize ? p + O + wn : nullptr,
                              d.batch_normalize ? p + 2 * O + wn : nullptr, d.batch_normalize ? p + 3 * O + wn : nullptr,
                              mem);
        } else if (l.type == LT_LSTM) {
            l.lstm->set_weights(p, l.weight_floats, mem);
        } else if (l.type == LT_RNN) {
            l.rnn->set_weights(p, l.weight_floats, mem);
        }
        pos += l.weight_floats;
    }
    weights_loaded = true;
    prepared_mode = -1;
    prepare();
}

nb_network_s::~nb_network_s() {
    drop_graphs();
    for (Slot &sl : slot) {
        if (sl.u8) (void)cudaFree(sl.u8);
        if (sl.copied) (void)cudaEventDestroy(sl.copied);
        if (sl.done) (void)cudaEventDestroy(sl.done);
    }
    if (copy_stream) (void)cudaStreamDestroy(copy_stream);
    if (capture_stream) (void)cudaStreamDestroy(capture_stream);
}

size_t nb_network_s::workspace_bytes() const {
    size_t n = (input_nhwc.n + convert_tmp.n + slot[0].f32.n + slot[1].f32.n) * sizeof(float);
    for (auto &lp : layers) {
        if (lp->conv) n += lp->conv->workspace_bytes();
        if (lp->fc) n += lp->fc->workspace_bytes();
        if (lp->lstm) n += lp->lstm->workspace_bytes();
        if (lp->rnn) n += lp->rnn->workspace_bytes();
    }
    return n;
}

void nb_network_s::prepare() {
    if (prepared_mode == h->math_mode && prepared_fuse == fuse) return;
    drop_graphs();
    walk(nullptr, IN_F32, true);
    NB_CHECK_CUDA(cudaStreamSynchronize(h->stream));
    prepared_mode = h->math_mode;
    prepared_fuse = fuse;
}

bool nb_network_s::first_layer_takes_rowwin() const {
    if (layers.empty() || layers[0]->type != LT_CONVOLUTIONAL) return false;
    const ConvPlan &c = *layers[0]->conv;
    return c.rowwin_ok && h->math_mode != NB_MATH_FP32 && c.path(ForwardOpts()) == PATH_SIMT;
}

// One pass over the layer list.  dry: nothing is launched; every layer sizes and allocates the scratch this pass
// would use, so that real passes allocate nothing.
void nb_network_s::walk(const float *input, int kind, bool dry) {
    const bool tf32 = h->math_mode == NB_MATH_TF32;
    const int n = (int)layers.size();

    // does layer i's direct consumer run a TF32 tensor-core contraction?
    auto consumer_is_tf32 = [&](int i) -> bool {
        if (!tf32) return false;
        int j = i + 1;
        while (j < n && layers[j]->type == LT_DROPOUT) j++;
        if (j >= n) return false;
        NetLayer &c = *layers[j];
        if (c.type == LT_CONVOLUTIONAL) return c.conv->path(ForwardOpts()) == PATH_TC;
        if (c.type == LT_CONNECTED || c.type == LT_RBM) return c.fc->path() == PATH_TC;
        if (c.type == LT_LSTM || c.type == LT_RNN) return true;
        return false;
    };

    const float *cur = input;
    bool cur_nhwc = false, cur_rounded = false;
    const float *cur_round = nullptr;
    for (int i = 0; i < n; i++) {
        NetLayer &l = *layers[i];
        const bool round_out = consumer_is_tf32(i);
        switch (l.type) {
            case LT_CONVOLUTIONAL: {
                ForwardOpts o;
                o.x_nhwc = cur_nhwc; o.y_nhwc = true; o.x_rounded = cur_rounded; o.round_out = round_out;
                if (i == 0 && kind == IN_ROWWIN) o.x_rowwin = true;
                l.materialised = true;
                // conv -> maxpool 2x2/2: the pooled tensor is produced by the conv epilogue
                bool referenced = false;        // a later shortcut reads this layer's own output
                for (int j = i + 2; j < n; j++) referenced |= layers[j]->type == LT_SHORTCUT && layers[j]->conn == i;
                if (fuse && !referenced && i + 1 < n && layers[i + 1]->type == LT_MAXPOOL && l.conv->can_fuse_pool()) {
                    const nb_pool_desc_t &pd = layers[i + 1]->pool;
                    if (pd.size == 2 && pd.stride == 2 && pd.padding == 0) {
                        NetLayer &pl = *layers[i + 1];
                        const bool pool_round = consumer_is_tf32(i + 1);
                        o.round_out = pool_round;
                        o.pool_out = pl.out_ptr;
                        if (dry) l.conv->reserve(o);
                        else l.conv->forward(cur, nullptr, o);
                        l.materialised = false;
                        pl.out_is_rounded = pool_round;
                        cur = pl.out_ptr; cur_nhwc = true; cur_rounded = pool_round; cur_round = nullptr;
                        i++;            // the pooling layer is done
                        continue;
                    }
                }
                // conv (linear) -> shortcut: the residual add and the shortcut's activation run in the conv epilogue
                if (fuse && !referenced && i + 1 < n && layers[i + 1]->type == LT_SHORTCUT) {
                    NetLayer &sl = *layers[i + 1];
                    const nb_shortcut_desc_t &sd = sl.shortcut;
                    NetLayer &cl = *layers[sl.conn];
                    if (cl.materialised && sl.conn != i && l.conv->can_fuse_shortcut(sd.conn_channels, sd.conn_height, sd.conn_width)) {
                        const bool sc_round = consumer_is_tf32(i + 1);
                        o.round_out = sc_round;
                        o.residual = cl.out_ptr;
                        o.res_c = sd.conn_channels; o.res_h = sd.conn_height; o.res_w = sd.conn_width;
                        o.res_act = sd.activation;
                        if (dry) l.conv->reserve(o);
                        else l.conv->forward(cur, sl.out_ptr, o);
                        l.materialised = false;
                        sl.out_is_rounded = sc_round;
                        cur = sl.out_ptr; cur_nhwc = true; cur_rounded = sc_round; cur_round = nullptr;
                        i++;
                        continue;
                    }
                }
                if (dry) l.conv->reserve(o);
                else l.conv->forward(cur, l.out_ptr, o);
                break;
            }
            case LT_CONNECTED:
            case LT_RBM: {
                ForwardOpts o;
                o.round_out = round_out;
                const float *x = cur;
                o.x_rounded = cur_rounded;
                o.x_foreign = i == 0;
                if (tf32 && cur_round) { x = cur_round; o.x_rounded = true; }
                if (dry) l.fc->reserve(o, rows);
                else l.fc->forward(x, l.out_ptr, o, rows);
                break;
            }
            case LT_MAXPOOL:
            case LT_AVGPOOL: {
                nb_pool_desc_t d = l.pool;
                d.layout = cur_nhwc ? NB_LAYOUT_NHWC : NB_LAYOUT_NCHW;
                if (!cur_nhwc) {
                    // only possible for the first layer: bring the NCHW input to NHWC first
                    input_nhwc.reserve(input_size * rows);
                    if (!dry) launch_layout(h, cur, input_nhwc.p, rows, in_c, in_h, in_w, true, false);
                    cur = input_nhwc.p;
                    d.layout = NB_LAYOUT_NHWC;
                }
                if (!dry) launch_pool(h, d, cur, l.out_ptr, round_out);
                break;
            }
            case LT_SHORTCUT: {
                if (!dry) launch_shortcut(h, l.shortcut, cur, layers[l.conn]->out_ptr, l.out_ptr, round_out);
                break;
            }
            case LT_DROPOUT: break;
            case LT_SOFTMAX: {
                if (!dry) launch_softmax(h, cur, l.out_ptr, rows, l.C);
                break;
            }
            case LT_LSTM: {
                const float *x = cur;
                bool xr = cur_rounded;
                if (tf32 && cur_round) { x = cur_round; xr = true; }
                if (dry) l.lstm->reserve(true, xr, true, i == 0);
                else l.lstm->forward(x, l.out_ptr, nullptr, xr, l.out_round_ptr, i == 0);
                break;
            }
            case LT_RNN: {
                if (dry) l.rnn->reserve(cur_rounded, i == 0);
                else l.rnn->forward(cur, l.out_ptr, cur_rounded, round_out, i == 0);
                break;
            }
            default: throw Error(NB_ERR_UNSUPPORTED, "layer type not executable");
        }
        if (l.type != LT_DROPOUT) {
            l.out_is_rounded = round_out && l.type != LT_SOFTMAX && l.type != LT_LSTM;
            cur_rounded = l.out_is_rounded;
            cur_round = l.type == LT_LSTM ? l.out_round_ptr : nullptr;
        }
        cur = l.out_ptr;
        cur_nhwc = l.nhwc;
    }
}

void nb_network_s::drop_graphs() {
    for (Graph &g : graphs) (void)cudaGraphExecDestroy(g.exec);
    graphs.clear();
    seen_inputs.clear();
}

// A pass, eagerly or as a graph replay.  A pass is captured the second time it is asked for with the same input
// pointer: by then every launch of it has run once, so the capture itself makes no driver query and no allocation.
void nb_network_s::run(const float *input, int kind) {
    if (!weights_loaded && weight_count() > 0) throw Error(NB_ERR_NO_WEIGHTS, "network forward before weights were loaded");
    NB_REQUIRE(input != nullptr, "null input pointer");
    prepare();
    static const bool sync_launches = [] {
        const char *v = std::getenv("NEBULA_B200_SYNC_LAUNCHES");
        return v && *v && *v != '0';
    }();
    if (!use_graph || h->profiling || sync_launches) { walk(input, kind, false); return; }
    for (Graph &g : graphs)
        if (g.input == input && g.kind == kind && g.mode == h->math_mode && g.fuse == fuse) {
            NB_CHECK_CUDA(cudaGraphLaunch(g.exec, h->stream));
            h->launches += g.launches;
            return;
        }
    if (std::find(seen_inputs.begin(), seen_inputs.end(), (const void *)input) == seen_inputs.end()) {
        if (seen_inputs.size() > 16) seen_inputs.clear();
        seen_inputs.push_back(input);
        walk(input, kind, false);
        return;
    }
    if (!capture_stream) NB_CHECK_CUDA(cudaStreamCreateWithFlags(&capture_stream, cudaStreamNonBlocking));
    cudaStream_t user = h->stream;
    const unsigned long long before = h->launches;
    cudaGraph_t graph = nullptr;
    h->stream = capture_stream;
    try {
        NB_CHECK_CUDA(cudaStreamBeginCapture(capture_stream, cudaStreamCaptureModeThreadLocal));
        walk(input, kind, false);
        NB_CHECK_CUDA(cudaStreamEndCapture(capture_stream, &graph));
    } catch (...) {
        h->stream = user;
        if (!graph) (void)cudaStreamEndCapture(capture_stream, &graph);
        if (graph) (void)cudaGraphDestroy(graph);
        throw;
    }
    h->stream = user;
    Graph g{input, kind, h->math_mode, fuse, nullptr, h->launches - before};
    h->launches = before;
    cudaError_t e = cudaGraphInstantiate(&g.exec, graph, 0);
    (void)cudaGraphDestroy(graph);
    NB_CHECK_CUDA(e);
    if (graphs.size() >= 8) { (void)cudaGraphExecDestroy(graphs.front().exec); graphs.erase(graphs.begin()); }
    graphs.push_back(g);
    NB_CHECK_CUDA(cudaGraphLaunch(g.exec, h->stream));
    h->launches += g.launches;
}

void nb_network_s::forward_u8(const unsigned char *images_dev) {
    NB_REQUIRE(images_dev != nullptr, "null image pointer");
    if (recurrent) throw Error(NB_ERR_UNSUPPORTED, "8-bit image input for a recurrent network");
    NB_REQUIRE(in_c == 3 || in_c == 1, "8-bit images need 1 or 3 channels (models/networks/convolutional.cc:305-311)");
    prepare();
    if (first_layer_takes_rowwin()) {
        ConvPlan &c = *layers[0]->conv;
        float *xw = c.x_rowwin.p;
        launch_u8_pack(h, images_dev, xw, rows, in_c, in_h, in_w, true, c.rw_wp, c.d.padding, h->math_mode == NB_MATH_TF32);
        run(xw, IN_ROWWIN);
    } else {
        slot[0].f32.reserve(input_size * rows);
        launch_u8_pack(h, images_dev, slot[0].f32.p, rows, in_c, in_h, in_w, false, 0, 0, false);
        run(slot[0].f32.p, IN_F32);
    }
}

void nb_network_s::submit(const void *input_host, bool u8, float *output_host) {
    NB_REQUIRE(input_host && output_host, "null host buffer");
    if (u8 && recurrent) throw Error(NB_ERR_UNSUPPORTED, "8-bit image input for a recurrent network");
    prepare();
    if (!copy_stream) NB_CHECK_CUDA(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
    Slot &s = slot[next_slot];
    next_slot ^= 1;
    if (!s.copied) {
        NB_CHECK_CUDA(cudaEventCreateWithFlags(&s.copied, cudaEventDisableTiming));
        NB_CHECK_CUDA(cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming));
    }
    if (s.busy) {       // the submission before last used this slot: its pass must be over before the buffer is refilled
        NB_CHECK_CUDA(cudaEventSynchronize(s.done));
        s.busy = false;
    }
    const size_t elems = input_size * rows;
    if (u8) {
        if (!s.u8) NB_CHECK_CUDA(cudaMalloc((void **)&s.u8, elems));
        NB_CHECK_CUDA(cudaMemcpyAsync(s.u8, input_host, elems, cudaMemcpyHostToDevice, copy_stream));
    } else {
        s.f32.reserve(elems);
        NB_CHECK_CUDA(cudaMemcpyAsync(s.f32.p, input_host, elems * sizeof(float), cudaMemcpyHostToDevice, copy_stream));
    }
    NB_CHECK_CUDA(cudaEventRecord(s.copied, copy_stream));
    NB_CHECK_CUDA(cudaStreamWaitEvent(h->stream, s.copied, 0));
    if (u8) forward_u8(s.u8);
    else run(s.f32.p, IN_F32);
    layer_output(-1, output_host, NB_MEM_HOST, false);
    NB_CHECK_CUDA(cudaEventRecord(s.done, h->stream));
    s.busy = true;
}

void nb_network_s::wait() {
    for (Slot &s : slot)
        if (s.busy) {
            NB_CHECK_CUDA(cudaEventSynchronize(s.done));
            s.busy = false;
        }
}

void nb_network_s::layer_output(int index, float *dst, int mem, bool sync) {
    const int n = (int)layers.size();
    if (index < 0) index += n;
    NB_REQUIRE(index >= 0 && index < n, "layer index out of range");
    NB_REQUIRE(dst != nullptr, "null destination");
    NetLayer &l = *layers[index];
    if (!l.materialised)
        throw Error(NB_ERR_UNSUPPORTED, "this layer's output was fused into the next layer's; disable fusion "
                                        "(nb_network_set_fusion) to materialise it");
    const size_t total = l.size * rows;
    const float *src = l.out_ptr;
    if (l.nhwc && l.H * l.W > 1 && l.C > 1) {
        if (mem == NB_MEM_DEVICE) {
            launch_layout(h, src, dst, rows, l.C, l.H, l.W, false, false);
            return;
        }
        convert_tmp.reserve(total);
        launch_layout(h, src, convert_tmp.p, rows, l.C, l.H, l.W, false, false);
        src = convert_tmp.p;
    }
    NB_CHECK_CUDA(cudaMemcpyAsync(dst, src, total * sizeof(float),
                                  mem == NB_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, h->stream));
    if (mem == NB_MEM_HOST && sync) NB_CHECK_CUDA(cudaStreamSynchronize(h->stream));
}
