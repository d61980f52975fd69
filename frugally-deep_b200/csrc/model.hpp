// Host-side model description: the converted-JSON file parsed into layers with pre-packed weights.
//
// Mirrors what the reference builds in import_model.hpp (create_model_layer :397-425, create_layer
// :1771-1966 and the per-class creators) but produces plain data for the plan compiler instead of
// layer objects with virtual apply methods.
#pragma once

#include "common.hpp"
#include "json.hpp"

#include <map>
#include <memory>
#include <string>
#include <vector>

namespace fdk {

struct Conn {
    std::string layer;
    int node = 0;
    int tensor = 0;
};

enum PadMode : int { PAD_VALID = 0, PAD_SAME = 1, PAD_CAUSAL = 2 };

struct ModelDef;

// One weight array on the host.  `gemm` marks [N][K] contraction operands, which additionally get
// TF32 high/low halves on the device.
struct HostWeight {
    std::vector<float> data;
    bool gemm = false;
};

struct Layer {
    std::string cls, name;
    std::vector<std::vector<Conn>> nodes;
    bool has_act = false;  // activation attached from config["activation"] (import_model.hpp:1953-1962)
    ActSpec act;
    std::shared_ptr<ModelDef> sub;  // nested Functional/Model
    std::vector<Layer> cells;       // Bidirectional: forward, backward, merge; RNN: the chain of cells
    bool reverse = false;           // recurrent layer that walks the sequence from its last row to its first

    // geometry / hyper-parameters (meaning depends on cls)
    int k[3] = {1, 1, 1};      // kernel or pool size (d4, h, w)
    int s[3] = {1, 1, 1};      // strides
    int dil[3] = {1, 1, 1};    // dilation
    int pad = PAD_VALID;
    int units = 0;             // filters / units / output features
    int in_feat = 0;           // input channels / features
    int kdim = 0, ldw = 0;     // contraction length and padded row stride of w_main
    std::vector<int> axes;
    float eps = 0.f;
    bool flag_a = false, flag_b = false, flag_c = false;  // class-specific booleans
    int pads[6] = {0, 0, 0, 0, 0, 0};  // front, back, top, bottom, left, right
    std::vector<int64_t> target;       // Reshape target (-1 = inferred), Permute dims
    ActSpec act_main, act_rec;          // recurrent activations
    int heads = 0, key_dim = 0, value_dim = 0, out_dim = 0, input_dim = 0;
    int bin_op = 0;

    // weight ids (-1 = absent)
    int w_main = -1, w_bias = -1, w_scale = -1, w_shift = -1;
    int w_rec = -1;                    // recurrent kernel [gU][U]
    int w_rec_bias = -1;               // GRU reset_after recurrent bias
    // LSTM with units % 16 == 0, tanh / sigmoid: input kernel, recurrent kernel and bias once more with the gate columns
    // in the cell order of the fused time-step kernel (column 64 * (u / 16) + 16 * gate + u % 16)
    int w_cell_in = -1, w_cell_rec = -1, w_cell_bias = -1;
    int w_q = -1, w_k = -1, w_v = -1, w_o = -1, b_q = -1, b_k = -1, b_v = -1, b_o = -1;
    int w_gamma = -1, w_beta = -1;
    int w_aux = -1;
    // Transposed convolution with in_feat % 4 == 0: one sub-filter [N][taps_y][taps_x][C] per output phase
    // (index py * s[2] + px), see transposed_phase(); empty when the layer keeps the gathered form
    std::vector<int> w_phases;
    int kv_heads = 0;                  // GroupedQueryAttention: key/value heads (0 = as many as query heads)
    int w_g = -1, b_g = -1;            // GroupedQueryAttention gate projection
    float f_scale = 1.f, f_w2 = 1.f;   // Attention: scale and concat_score_weight
    std::string eq_in, eq_kernel, eq_out, eq_bias;  // EinsumDense: letters of input, kernel, output; bias letters in output order
    std::vector<int64_t> kernel_dims;               // EinsumDense kernel shape
};

// convolve_transposed (convolution.hpp:443-469) dilates the input by the stride, pads it and runs a stride-1
// convolution, so an output position only meets every s-th filter tap, the others fall on inserted zeros.  All
// output positions with the same remainder p modulo s meet the same taps k0, k0 + s, ...: they are a stride-1
// convolution of the UNDILATED input with that sub-filter, reading input index y' + j + shift for tap j of
// output p + s * y'.  `lead` = low padding + the offset of the first sample in the dilated tensor.
struct TransposedPhase { int k0, taps, shift; };
inline int transposed_lead(int k, int s, int pad) {
    const int pad_lo = pad == PAD_SAME ? (k - 1) / 2 : k - 1;
    const int extra = (pad == PAD_SAME && s > 1) ? s - 1 : 0;
    return pad_lo + extra - extra / 2;
}
inline TransposedPhase transposed_phase(int k, int s, int lead, int p) {
    TransposedPhase t;
    t.k0 = (((lead - p) % s) + s) % s;
    t.taps = t.k0 < k ? (k - t.k0 + s - 1) / s : 0;
    t.shift = (p + t.k0 - lead) / s;  // exact: p + k0 - lead is a multiple of s
    return t;
}

struct ModelDef {
    std::string name;
    std::vector<Layer> layers;
    std::map<std::string, int> index;
    std::vector<Conn> inputs, outputs;
    const Layer& find(const std::string& id) const {
        auto it = index.find(id);
        if (it == index.end()) raise("dangling layer reference: " + id);
        return layers[(size_t)it->second];
    }
};

struct TestCase {
    std::vector<TShape> in_shapes, out_shapes;
    std::vector<std::vector<float>> in_values, out_values;
};

struct LoadedModel {
    std::shared_ptr<ModelDef> root;
    std::vector<HostWeight> weights;
    std::vector<VarShape> input_shapes, output_shapes;
    std::vector<TestCase> tests;
    std::string hash;
};

// Parses the text of a converted model file.  Throws fdk::Error with the reference's messages where
// the reference asserts (unknown layer type, channels_first, stateful RNN flags, ...).
// cell_order_copies: also store LSTM kernels and biases in the column order of the fused time-step kernel (Layer::w_cell_*).
LoadedModel load_model_json(const char* text, size_t len, bool cell_order_copies = false);

std::vector<float> decode_floats(const Json& data);
ActSpec make_activation(const std::string& type, const Json& layer_json);

}  // namespace fdk
