// Loader: converted-JSON text -> LoadedModel (layers with pre-packed weights).
// Follows import_model.hpp of the reference; weight layouts are those written by
// keras_export/convert_model.py (:197-236 convolutions, :429-470 normalisation/dense, :600-631 attention/RNN).
#include "model.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <array>
#include <atomic>
#include <exception>
#include <limits>
#include <thread>

namespace fdk {

// ---- float decoding (import_model.hpp:274-297; base64.hpp:76-109) ------------------------------------
namespace {
// Host threads for the two bulk jobs of a load (base64 decoding, weight transposes) on arrays of a megabyte or more.
int load_threads() {
    static const int n = [] {
        const unsigned hc = std::thread::hardware_concurrency();
        return (int)std::min<unsigned>(hc == 0 ? 1u : hc, 16u);
    }();
    return n;
}
// body(begin, end) over [0, n) in contiguous blocks, on up to load_threads() threads; exceptions are rethrown.
template <typename F>
void parallel_blocks(size_t n, size_t min_per_thread, F&& body) {
    const size_t want = std::max<size_t>(1, std::min<size_t>((size_t)load_threads(), n / std::max<size_t>(1, min_per_thread)));
    if (want <= 1) { body((size_t)0, n); return; }
    std::vector<std::thread> pool;
    std::vector<std::exception_ptr> err(want);
    const size_t per = (n + want - 1) / want;
    for (size_t t = 0; t < want; ++t) {
        const size_t lo = std::min(n, t * per), hi = std::min(n, lo + per);
        pool.emplace_back([&, t, lo, hi] {
            try { if (lo < hi) body(lo, hi); } catch (...) { err[t] = std::current_exception(); }
        });
    }
    for (auto& th : pool) th.join();
    for (auto& e : err) if (e) std::rethrow_exception(e);
}
std::atomic<long long> g_decode_ns{0}, g_pack_ns{0};
struct ScopedNs {
    std::atomic<long long>& sink;
    std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
    explicit ScopedNs(std::atomic<long long>& s) : sink(s) {}
    ~ScopedNs() { sink += std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count(); }
};
const int8_t* base64_table() {
    static const std::array<int8_t, 256> lut = [] {
        std::array<int8_t, 256> t;
        t.fill((int8_t)-1);
        const char* a = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
        for (int i = 0; i < 64; ++i) t[(unsigned char)a[i]] = (int8_t)i;
        return t;
    }();
    return lut.data();
}
// Whole groups of four alphabet characters -> three bytes each; returns the number of characters consumed (stops at
// the first group with any other character).
size_t decode_groups(const char* p, size_t n, uint8_t* o) {
    const int8_t* lut = base64_table();
    size_t i = 0;
    for (; i + 4 <= n; i += 4) {
        const int a = lut[(unsigned char)p[i]], b = lut[(unsigned char)p[i + 1]], c = lut[(unsigned char)p[i + 2]], d = lut[(unsigned char)p[i + 3]];
        if ((a | b | c | d) < 0) break;
        const uint32_t v = ((uint32_t)a << 18) | ((uint32_t)b << 12) | ((uint32_t)c << 6) | (uint32_t)d;
        o[0] = (uint8_t)(v >> 16); o[1] = (uint8_t)(v >> 8); o[2] = (uint8_t)v;
        o += 3;
    }
    return i;
}
}  // namespace

// decode_floats (import_model.hpp:136-171): a list of numbers, or base64 text of little-endian fp32 values, whole or in
// the exporter's chunks (keras_export/convert_model.py:64-83).
std::vector<float> decode_floats(const Json& data) {
    ensure(data.is_array() || data.is_string(), "invalid float array format");
    if (data.is_array() && !data.empty() && data[0].is_number()) {
        std::vector<float> r(data.size());
        for (size_t i = 0; i < data.size(); ++i) r[i] = (float)data[i].number();
        return r;
    }
    ScopedNs timer(g_decode_ns);
    const int8_t* lut = base64_table();
    // the pieces of text, in order
    std::vector<std::pair<const char*, size_t>> parts;
    if (data.is_string()) parts.emplace_back(data.sptr, data.slen);
    else for (const auto& s : data.arr) { ensure(s.is_string(), "invalid float array format"); parts.emplace_back(s.sptr, s.slen); }
    size_t total_chars = 0;
    for (const auto& pr : parts) total_chars += pr.second;
    // Fast form: every piece but the last is whole groups of four alphabet characters (the exporter's 1024-character
    // chunks), so piece i starts at a known byte and the pieces decode independently, straight into the result.
    bool regular = true;
    for (size_t i = 0; i + 1 < parts.size(); ++i) regular = regular && parts[i].second % 4 == 0;
    if (regular && !parts.empty()) {
        std::vector<size_t> first(parts.size() + 1, 0);
        for (size_t i = 0; i < parts.size(); ++i) first[i + 1] = first[i] + parts[i].second / 4 * 3;
        std::vector<float> out((first.back() + 3) / 4 + 1);
        uint8_t* bytes = reinterpret_cast<uint8_t*>(out.data());
        std::atomic<bool> clean{true};
        size_t tail_done = 0;  // characters of the last piece that the group decoder took
        parallel_blocks(parts.size(), ((size_t)1 << 20) / 1024, [&](size_t lo, size_t hi) {
            for (size_t i = lo; i < hi; ++i) {
                const size_t used = decode_groups(parts[i].first, parts[i].second, bytes + first[i]);
                if (i + 1 == parts.size()) tail_done = used;
                else if (used != parts[i].second) clean = false;
            }
        });
        if (clean) {
            // the rest of the last piece: padding, or a group cut short
            size_t n_bytes = first[parts.size() - 1] + tail_done / 4 * 3;
            uint32_t acc = 0;
            int bits = 0;
            const char* p = parts.back().first;
            for (size_t i = tail_done; i < parts.back().second; ++i) {
                const unsigned char ch = (unsigned char)p[i];
                if (ch == '=') break;
                const int8_t v = lut[ch];
                if (v < 0) continue;
                acc = (acc << 6) | (uint32_t)v;
                bits += 6;
                if (bits >= 8) { bits -= 8; bytes[n_bytes++] = (uint8_t)((acc >> bits) & 0xff); }
            }
            ensure(n_bytes % 4 == 0, "invalid float vector data");
            out.resize(n_bytes / 4);
            return out;
        }
    }
    // general form: one character at a time across all pieces (stray characters are skipped, '=' ends the data)
    std::vector<uint8_t> bytes;
    bytes.reserve(total_chars / 4 * 3 + 4);
    uint32_t acc = 0;
    int bits = 0;
    bool done = false;
    for (const auto& pr : parts) {
        for (size_t i = 0; i < pr.second && !done; ++i) {
            const unsigned char ch = (unsigned char)pr.first[i];
            if (ch == '=') { done = true; break; }
            const int8_t v = lut[ch];
            if (v < 0) continue;
            acc = (acc << 6) | (uint32_t)v;
            bits += 6;
            if (bits >= 8) { bits -= 8; bytes.push_back((uint8_t)((acc >> bits) & 0xff)); }
        }
    }
    ensure(bytes.size() % 4 == 0, "invalid float vector data");
    std::vector<float> out(bytes.size() / 4);
    if (!out.empty()) std::memcpy(out.data(), bytes.data(), bytes.size());
    return out;
}

static bool has_value(const Json& cfg, const char* key) { return cfg.is_object() && cfg.contains(key) && !cfg[key].is_null(); }

// import_model.hpp:1654-1696 (activation name -> creator) and the creators at :1172-1399.
ActSpec make_activation(const std::string& type, const Json& layer_json) {
    const Json& cfg = layer_json["config"];
    ActSpec a;
    if (type == "linear") a.kind = ACT_NONE;
    else if (type == "relu") {
        a.kind = ACT_RELU;
        if (has_value(cfg, "max_value")) {
            a.kind = ACT_RELU_GEN;
            a.p0 = (float)cfg["max_value"].number();
            a.p1 = (float)cfg["negative_slope"].number();
            a.p2 = (float)cfg["threshold"].number();
        }
    } else if (type == "relu6") { a.kind = ACT_RELU_GEN; a.p0 = 6.f; a.p1 = 0.f; a.p2 = 0.f; }
    else if (type == "softmax") a.kind = ACT_SOFTMAX;
    else if (type == "log_softmax") a.kind = ACT_LOG_SOFTMAX;
    else if (type == "softplus") a.kind = ACT_SOFTPLUS;
    else if (type == "tanh") a.kind = ACT_TANH;
    else if (type == "sigmoid") a.kind = ACT_SIGMOID;
    else if (type == "swish" || type == "silu") a.kind = ACT_SWISH;
    else if (type == "hard_sigmoid") a.kind = ACT_HARD_SIGMOID;
    else if (type == "hard_tanh") a.kind = ACT_HARD_TANH;
    else if (type == "log_sigmoid") a.kind = ACT_LOG_SIGMOID;
    else if (type == "tanh_shrink") a.kind = ACT_TANH_SHRINK;
    else if (type == "leaky_relu") { a.kind = ACT_LEAKY_RELU; a.p0 = cfg.is_object() && cfg.contains("negative_slope") ? (float)cfg["negative_slope"].number() : 0.2f; }
    else if (type == "selu") a.kind = ACT_SELU;
    else if (type == "elu") { a.kind = ACT_ELU; a.p0 = cfg.is_object() && cfg.contains("alpha") ? (float)cfg["alpha"].number() : 1.0f; }
    else if (type == "celu") { a.kind = ACT_CELU; a.p0 = cfg.is_object() && cfg.contains("alpha") ? (float)cfg["alpha"].number() : 1.0f; }
    else if (type == "exponential") a.kind = ACT_EXP;
    else if (type == "gelu") {
        if (has_value(cfg, "approximate")) ensure(cfg["approximate"].boolean() == false, "Gelu with approximate = True is not supported.");
        a.kind = ACT_GELU;
    } else if (type == "softsign") a.kind = ACT_SOFTSIGN;
    else if (type == "hard_shrink") { a.kind = ACT_HARD_SHRINK; a.p0 = (float)cfg["threshold"].number(); }
    else if (type == "soft_shrink") { a.kind = ACT_SOFT_SHRINK; a.p0 = (float)cfg["threshold"].number(); }
    else if (type == "sparse_plus") a.kind = ACT_SPARSE_PLUS;
    else if (type == "squareplus") { a.kind = ACT_SQUARE_PLUS; a.p0 = has_value(cfg, "b") ? (float)cfg["b"].number() : 4.0f; }
    else if (type == "threshold") {
        // a layer only (import_model.hpp:1274-1287); Keras renamed threshold_value -> threshold, value -> default_value
        a.kind = ACT_THRESHOLD;
        a.p0 = (float)(cfg.contains("threshold") ? cfg["threshold"] : cfg["threshold_value"]).number();
        a.p1 = (float)(cfg.contains("default_value") ? cfg["default_value"] : cfg["value"]).number();
    }
    else raise("unknown activation type: " + type);
    return a;
}

static ActSpec recurrent_activation(const std::string& n) {  // recurrent_ops.hpp:88-115
    ActSpec a;
    if (n == "linear") a.kind = ACT_NONE;
    else if (n == "tanh") a.kind = ACT_TANH;
    else if (n == "sigmoid") a.kind = ACT_SIGMOID;
    else if (n == "swish" || n == "silu") a.kind = ACT_SWISH;
    else if (n == "hard_sigmoid") a.kind = ACT_HARD_SIGMOID;
    else if (n == "relu") a.kind = ACT_RELU;
    else if (n == "selu") a.kind = ACT_SELU;
    else if (n == "elu") { a.kind = ACT_ELU; a.p0 = 1.0f; }
    else if (n == "exponential") a.kind = ACT_EXP;
    else if (n == "gelu") a.kind = ACT_GELU;
    else if (n == "softsign") a.kind = ACT_SOFTSIGN;
    else raise("recurrent activation function '" + n + "' not yet implemented");
    return a;
}

namespace {

struct Loader {
    const Json& params;  // trainable_params
    std::vector<HostWeight>& weights;
    bool cell_order_copies = false;  // LSTM: also store the arrays in the fused step kernel's column order

    int add_weight(std::vector<float>&& v, bool gemm = false) {
        weights.push_back(HostWeight{std::move(v), gemm});
        return (int)weights.size() - 1;
    }
    const Json& param(const std::string& prefix, const std::string& layer, const char* key) const {
        const Json& l = params[prefix + layer];
        const Json& p = l[key];
        return p;
    }
    std::vector<float> floats(const std::string& prefix, const std::string& layer, const char* key) const {
        const Json& p = param(prefix, layer, key);
        ensure(!p.is_null(), "missing parameter '" + std::string(key) + "' of layer '" + prefix + layer + "'");
        return decode_floats(p);
    }

    static void shape2(const Json& d, int& h, int& w) {  // create_shape2, import_model.hpp:229-241
        if (d.is_array()) {
            ensure(d.size() == 1 || d.size() == 2, "invalid number of dimensions in shape2");
            if (d.size() == 1) { h = 1; w = (int)d[0].integer(); } else { h = (int)d[0].integer(); w = (int)d[1].integer(); }
        } else { h = 1; w = (int)d.integer(); }
    }
    static void shape3(const Json& d, int (&o)[3]) {  // create_shape3, import_model.hpp:243-259
        if (d.is_array()) {
            ensure(d.size() >= 1 && d.size() <= 3, "invalid number of dimensions in shape3");
            if (d.size() == 1) { o[0] = 1; o[1] = 1; o[2] = (int)d[0].integer(); }
            else if (d.size() == 2) { o[0] = 1; o[1] = (int)d[0].integer(); o[2] = (int)d[1].integer(); }
            else { o[0] = (int)d[0].integer(); o[1] = (int)d[1].integer(); o[2] = (int)d[2].integer(); }
        } else { o[0] = 1; o[1] = 1; o[2] = (int)d.integer(); }
    }
    static int parse_padding(const std::string& s) {
        if (s == "valid") return PAD_VALID;
        if (s == "same") return PAD_SAME;
        if (s == "causal") return PAD_CAUSAL;
        raise("no padding");
    }
    static std::vector<int> int_list(const Json& d) {
        std::vector<int> r;
        if (d.is_array()) for (const auto& x : d.arr) r.push_back((int)x.integer()); else r.push_back((int)d.integer());
        return r;
    }
    static Conn triple(const Json& d) {
        ensure(d.is_array() && d.size() >= 3, "invalid format for inbound node");
        Conn c;
        c.layer = d[0].str();
        ensure(d[1].integer() >= 0 && d[2].integer() >= 0, "invalid size_t value");
        c.node = (int)d[1].integer();
        c.tensor = (int)d[2].integer();
        return c;
    }
    static std::vector<Conn> model_conns(const Json& d) {  // import_model.hpp:343-360
        ensure(d.is_array(), "input_layers/output_layers must be an array");
        if (!d.empty() && !d[0].is_array()) return {triple(d)};
        std::vector<Conn> r;
        for (const auto& x : d.arr) r.push_back(triple(x));
        return r;
    }
    static std::vector<std::vector<Conn>> create_nodes(const Json& layer) {  // import_model.hpp:1722-1740
        std::vector<std::vector<Conn>> nodes;
        const Json& inbound = layer["inbound_nodes"];
        ensure(inbound.is_array(), "no inbound nodes");
        for (const auto& nd : inbound.arr) {
            const Json& args = nd["args"];
            ensure(args.is_array(), "node args need to be an array");
            ensure(!args.empty(), "invalid args format");
            const Json* list = &args;
            if (args[0].is_array()) { ensure(args.size() == 1, "invalid args format"); list = &args[0]; }
            std::vector<Conn> cs;
            for (const auto& a : list->arr) {
                ensure(a.is_object() && a["config"].is_object() && a["config"].contains("keras_history"),
                       "No keras_history on node connection. Constant-value tensors are not supported.");
                cs.push_back(triple(a["config"]["keras_history"]));
            }
            nodes.push_back(std::move(cs));
        }
        return nodes;
    }

    // [N][K] weights with rows padded to a multiple of 4 floats (16-byte rows for vector and TMA loads).
    int add_gemm_weight(const std::vector<float>& w, int N, int K, int& ldw) {
        ldw = (K + 3) / 4 * 4;
        std::vector<float> p((size_t)N * ldw, 0.f);
        for (int n = 0; n < N; ++n) std::memcpy(&p[(size_t)n * ldw], &w[(size_t)n * K], sizeof(float) * (size_t)K);
        return add_weight(std::move(p), true);
    }
    // [K][N] (Keras dense layout) -> [N][K] padded
    int add_gemm_weight_transposed(const float* w, int K, int N, int& ldw) {
        ScopedNs timer(g_pack_ns);
        ldw = (K + 3) / 4 * 4;
        std::vector<float> p((size_t)N * ldw, 0.f);
        // 32 x 32 blocks (both the rows read and the rows written stay in cache), blocks of output rows per thread
        const size_t ld = (size_t)ldw;
        float* dst = p.data();
        parallel_blocks((size_t)(N + 31) / 32, std::max<size_t>(1, ((size_t)1 << 18) / ((size_t)K * 32 + 1)), [&](size_t lo, size_t hi) {
            for (size_t nb = lo; nb < hi; ++nb) {
                const int n0 = (int)nb * 32, n1 = std::min(N, n0 + 32);
                for (int k0 = 0; k0 < K; k0 += 32) {
                    const int k1 = std::min(K, k0 + 32);
                    for (int n = n0; n < n1; ++n)
                        for (int k = k0; k < k1; ++k) dst[(size_t)n * ld + k] = w[(size_t)k * N + n];
                }
            }
        });
        return add_weight(std::move(p), true);
    }
    // Bias vectors are dropped when they are all equal and sum to zero (convolution.hpp:40).
    int add_conv_bias(const std::vector<float>& b) {
        float sum = 0.f;
        bool same = true;
        for (float x : b) { sum += x; if (x != b[0]) same = false; }
        if (sum == 0.f && same) return -1;
        return add_weight(std::vector<float>(b));
    }

    std::shared_ptr<ModelDef> model(const Json& data, const std::string& name, const std::string& prefix) {
        auto m = std::make_shared<ModelDef>();
        m->name = name;
        const Json& layers = data["config"]["layers"];
        ensure(layers.is_array(), "missing layers array");
        for (const auto& l : layers.arr) {
            Layer L = layer(l, prefix);
            ensure(m->index.find(L.name) == m->index.end(), "layer names must be unique");
            m->index[L.name] = (int)m->layers.size();
            m->layers.push_back(std::move(L));
        }
        ensure(data["config"]["input_layers"].is_array(), "no input layers");
        m->inputs = model_conns(data["config"]["input_layers"]);
        m->outputs = model_conns(data["config"]["output_layers"]);
        return m;
    }

    // One LSTM / GRU / SimpleRNN with its weights (import_model.hpp:1491-1566).  `cell_cfg` holds units,
    // activations, use_bias and reset_after; `outer_cfg` holds return_sequences / return_state and the flags
    // that are refused (for a plain layer both are its config; for keras.layers.RNN they are the cell's and
    // the layer's, import_model.hpp:1568-1592).  Parameters are read from `owner` under `key_prefix` + name.
    void recurrent_cell(Layer& L, const std::string& t, const Json& cell_cfg, const Json& outer_cfg, const std::string& prefix,
                        const std::string& owner, const std::string& key_prefix, bool force_sequences) {
        auto fl = [&](const char* key) { return floats(prefix, owner, (key_prefix + key).c_str()); };
        L.cls = t;
        L.units = (int)cell_cfg["units"].integer();
        ensure(L.units > 0, t + " units must be > 0.");
        L.act_main = recurrent_activation(cell_cfg.get_str("activation", "tanh"));
        L.act_rec = recurrent_activation(cell_cfg.get_str("recurrent_activation", "sigmoid"));
        const bool use_bias = cell_cfg.get_bool("use_bias", true);
        L.flag_a = force_sequences || outer_cfg.get_bool("return_sequences", false);
        L.flag_b = outer_cfg.get_bool("return_state", false);
        L.flag_c = cell_cfg.get_bool("reset_after", true);
        // the exporter rejects these (convert_model.py:618-631); a hand-written file is rejected here
        ensure(!outer_cfg.get_bool("go_backwards", false) && !outer_cfg.get_bool("stateful", false), t + ": go_backwards/stateful are not supported.");
        const int g = t == "LSTM" ? 4 : t == "GRU" ? 3 : 1;
        const std::vector<float> W = fl("weights"), U = fl("recurrent_weights");
        const int gu = g * L.units;
        ensure(W.size() % (size_t)gu == 0 && U.size() == (size_t)L.units * gu, "invalid recurrent weights");
        L.in_feat = (int)(W.size() / (size_t)gu);
        L.w_main = add_gemm_weight_transposed(W.data(), L.in_feat, gu, L.ldw);
        int ldu = 0;
        L.w_rec = add_gemm_weight_transposed(U.data(), L.units, gu, ldu);
        L.kdim = ldu;  // row stride of the recurrent kernel
        std::vector<float> bias_copy;
        if (use_bias) {
            std::vector<float> b = fl("bias");
            if (t == "GRU") {
                ensure(b.size() == (size_t)(L.flag_c ? 2 * gu : gu), "GRU bias size does not match reset_after setting.");
                std::vector<float> bx(b.begin(), b.begin() + gu);
                L.w_bias = add_weight(std::move(bx));
                if (L.flag_c) L.w_rec_bias = add_weight(std::vector<float>(b.begin() + gu, b.end()));
            } else {
                ensure(b.size() == (size_t)gu, "invalid recurrent bias");
                if (t == "LSTM") bias_copy = b;
                L.w_bias = add_weight(std::move(b));
            }
        }
        if (cell_order_copies && t == "LSTM" && L.units % 16 == 0 && L.act_main.kind == ACT_TANH && L.act_rec.kind == ACT_SIGMOID) {
            // The same three arrays with the columns regrouped so that 64 consecutive columns hold the four gates of 16
            // units: the recurrent product's epilogue then finishes the cell itself (engine.cpp, recurrent()).
            const int Un = L.units;
            auto cell_col = [&](int col) { const int gate = col / Un, u = col % Un; return 64 * (u / 16) + 16 * gate + u % 16; };
            auto regroup = [&](const std::vector<float>& src, int rows) {
                std::vector<float> dst(src.size());
                for (int r = 0; r < rows; ++r)
                    for (int col = 0; col < gu; ++col) dst[(size_t)r * gu + cell_col(col)] = src[(size_t)r * gu + col];
                return dst;
            };
            int ld = 0;
            const std::vector<float> Wc = regroup(W, L.in_feat), Uc = regroup(U, Un);
            L.w_cell_in = add_gemm_weight_transposed(Wc.data(), L.in_feat, gu, ld);
            L.w_cell_rec = add_gemm_weight_transposed(Uc.data(), Un, gu, ld);
            if (!bias_copy.empty()) L.w_cell_bias = add_weight(regroup(bias_copy, 1));
        }
    }

    // Registers the weights of a 2-D convolution whose geometry (k, s, dil, units) is already in L: kernel in the
    // exporter's (filters, kh, kw, in_c) order, bias of `units` values (convolution.hpp:29-60, filter.hpp:69-103).
    void conv2d_weights(Layer& L, std::vector<float> w, std::vector<float> bias, bool transposed) {
        ensure((int)bias.size() == L.units, "size of bias does not match");
        const int area = L.k[1] * L.k[2];
        ensure(area > 0 && w.size() % (size_t)area == 0, "invalid number of weights");
        L.in_feat = (int)(w.size() / ((size_t)area * L.units));
        ensure((size_t)L.in_feat * area * L.units == w.size(), "invalid weight size");
        if (transposed) {
            // filters are dilated, then flipped in both spatial directions (filter.hpp:88-97)
            const int kh = L.k[1], kw = L.k[2], C = L.in_feat;
            const int ekh = (kh - 1) * L.dil[1] + 1, ekw = (kw - 1) * L.dil[2] + 1;
            std::vector<float> f((size_t)L.units * ekh * ekw * C, 0.f);
            for (int n = 0; n < L.units; ++n) for (int y = 0; y < kh; ++y) for (int x = 0; x < kw; ++x) for (int c = 0; c < C; ++c) {
                const int yd = y * L.dil[1], xd = x * L.dil[2];
                f[(((size_t)n * ekh + (ekh - 1 - yd)) * ekw + (ekw - 1 - xd)) * C + c] = w[(((size_t)n * kh + y) * kw + x) * C + c];
            }
            w.swap(f);
            L.k[1] = ekh; L.k[2] = ekw; L.dil[1] = L.dil[2] = 1;
            L.flag_a = true;  // transposed
        }
        L.kdim = L.k[1] * L.k[2] * L.in_feat;
        L.w_main = add_gemm_weight(w, L.units, L.kdim, L.ldw);
        L.w_bias = add_conv_bias(bias);
        if (transposed && L.in_feat % 4 == 0 && L.s[1] * L.s[2] <= 16) {
            // sub-filters per output phase for the implicit-GEMM form (no gathered patch matrix)
            const int kh = L.k[1], kw = L.k[2], C = L.in_feat, sy = L.s[1], sx = L.s[2];
            const int lead_y = transposed_lead(kh, sy, L.pad), lead_x = transposed_lead(kw, sx, L.pad);
            bool every_phase_has_taps = true;
            for (int py = 0; py < sy; ++py) every_phase_has_taps = every_phase_has_taps && transposed_phase(kh, sy, lead_y, py).taps > 0;
            for (int px = 0; px < sx; ++px) every_phase_has_taps = every_phase_has_taps && transposed_phase(kw, sx, lead_x, px).taps > 0;
            if (every_phase_has_taps) {
                for (int py = 0; py < sy; ++py) for (int px = 0; px < sx; ++px) {
                    const TransposedPhase ty = transposed_phase(kh, sy, lead_y, py), tx = transposed_phase(kw, sx, lead_x, px);
                    std::vector<float> f((size_t)L.units * ty.taps * tx.taps * C);
                    for (int n = 0; n < L.units; ++n) for (int jy = 0; jy < ty.taps; ++jy) for (int jx = 0; jx < tx.taps; ++jx)
                        std::memcpy(&f[(((size_t)n * ty.taps + jy) * tx.taps + jx) * C],
                                    &w[(((size_t)n * kh + ty.k0 + sy * jy) * kw + tx.k0 + sx * jx) * C], sizeof(float) * (size_t)C);
                    int ld = 0;
                    L.w_phases.push_back(add_gemm_weight(f, L.units, ty.taps * tx.taps * C, ld));
                }
            }
        }
        // Few input channels (first layers of vision models): one 32-float k block holds a whole filter ROW
        // (kw taps x channels padded to a multiple of 4).  Second weight layout [N][kh][32] for that form.
        const int cp = (L.in_feat + 3) / 4 * 4;
        if (!transposed && L.dil[1] == 1 && L.dil[2] == 1 && L.k[1] * L.k[2] > 1 && L.k[2] * cp <= 32) {
            const int kh = L.k[1], kw = L.k[2], C = L.in_feat;
            std::vector<float> rw((size_t)L.units * kh * 32, 0.f);
            for (int n = 0; n < L.units; ++n) for (int y = 0; y < kh; ++y) for (int x = 0; x < kw; ++x) for (int c = 0; c < C; ++c)
                rw[((size_t)n * kh + y) * 32 + (size_t)x * cp + c] = w[(((size_t)n * kh + y) * kw + x) * C + c];
            L.w_aux = add_weight(std::move(rw), true);
        }
    }

    Layer layer(const Json& data, const std::string& prefix) {
        Layer L;
        L.name = data["name"].str();
        L.cls = data["class_name"].str();
        const Json& cfg = data["config"];
        const std::string& t = L.cls;
        auto fl = [&](const char* key) { return floats(prefix, L.name, key); };

        if (t == "Model" || t == "Functional") {
            L.sub = model(data, L.name, prefix + L.name + "_");
            L.nodes = create_nodes(data);
            return L;
        }
        if (t == "InputLayer") {
            ensure(data["inbound_nodes"].empty(), "input layer is not allowed to have inbound nodes");
        } else if (t == "Conv1D" || t == "Conv2D" || t == "Conv1DTranspose" || t == "Conv2DTranspose") {
            const bool transposed = t.find("Transpose") != std::string::npos;
            L.pad = parse_padding(cfg["padding"].str());
            shape2(cfg["strides"], L.s[1], L.s[2]);
            shape2(cfg["dilation_rate"], L.dil[1], L.dil[2]);
            shape2(cfg["kernel_size"], L.k[1], L.k[2]);
            L.units = (int)cfg["filters"].integer();
            std::vector<float> bias((size_t)L.units, 0.f);
            if (cfg["use_bias"].boolean()) bias = fl("bias");
            conv2d_weights(L, fl("weights"), std::move(bias), transposed);
        } else if (t == "ConvLSTM1D" || t == "ConvLSTM2D") {  // import_model.hpp:748-785, conv_lstm_2d_layer.hpp:27-52
            // Two convolutions with 4 * filters outputs (gates i, f, c~, o): one over every time step of the input, one
            // (same padding, stride 1, no bias) over the previous hidden state; held as two Conv2D layers.
            const int units = (int)cfg["filters"].integer();
            L.units = units;
            L.bin_op = t == "ConvLSTM1D" ? 1 : 2;   // rank of the spatial part
            L.flag_b = cfg.get_bool("return_sequences", false);
            L.flag_c = cfg.get_bool("return_state", false);
            L.act_main = recurrent_activation(cfg.contains("activation") && cfg["activation"].is_string() ? cfg["activation"].str() : std::string("tanh"));
            L.act_rec = recurrent_activation(cfg.contains("recurrent_activation") && cfg["recurrent_activation"].is_string()
                                                 ? cfg["recurrent_activation"].str() : std::string("sigmoid"));
            L.cells.resize(2);
            Layer& in_conv = L.cells[0];
            Layer& rec_conv = L.cells[1];
            in_conv.cls = rec_conv.cls = "Conv2D";
            in_conv.name = L.name + "_input_conv";
            rec_conv.name = L.name + "_recurrent_conv";
            in_conv.pad = parse_padding(cfg["padding"].str());
            shape2(cfg["strides"], in_conv.s[1], in_conv.s[2]);
            shape2(cfg["dilation_rate"], in_conv.dil[1], in_conv.dil[2]);
            shape2(cfg["kernel_size"], in_conv.k[1], in_conv.k[2]);
            in_conv.units = rec_conv.units = 4 * units;
            std::vector<float> bias((size_t)(4 * units), 0.f);
            if (cfg.get_bool("use_bias", true)) bias = fl("bias");
            conv2d_weights(in_conv, fl("weights"), std::move(bias), false);
            rec_conv.pad = PAD_SAME;
            rec_conv.k[1] = in_conv.k[1];
            rec_conv.k[2] = in_conv.k[2];
            conv2d_weights(rec_conv, fl("recurrent_weights"), std::vector<float>((size_t)(4 * units), 0.f), false);
            ensure(rec_conv.in_feat == units, "ConvLSTM: the recurrent kernel must have `filters` input channels");
            L.has_act = false;
            L.nodes = create_nodes(data);
            return L;   // the layer's own activation entries are consumed above (no attached activation)
        } else if (t == "Conv3D" || t == "Conv3DTranspose") {  // import_model.hpp:468-526
            const bool transposed = t == "Conv3DTranspose";
            L.pad = parse_padding(cfg["padding"].str());
            shape3(cfg["strides"], L.s);
            shape3(cfg["dilation_rate"], L.dil);
            shape3(cfg["kernel_size"], L.k);
            L.units = (int)cfg["filters"].integer();
            ensure(L.units > 0, "needs at least one filter");
            ensure(L.s[0] > 0 && L.s[1] > 0 && L.s[2] > 0, "invalid strides");
            std::vector<float> bias((size_t)L.units, 0.f);
            if (cfg["use_bias"].boolean()) bias = fl("bias");
            ensure((int)bias.size() == L.units, "size of bias does not match");
            const std::vector<float> w = fl("weights");
            const int vol = L.k[0] * L.k[1] * L.k[2];
            ensure(vol > 0 && w.size() % ((size_t)vol * L.units) == 0, "invalid number of weights");
            L.in_feat = (int)(w.size() / ((size_t)vol * L.units));
            // every filter is dilated with zeros and, for the transposed layer, reversed along its three spatial
            // axes (generate_filters_3d, convolution3d.hpp:198-233)
            const int C = L.in_feat;
            const int ek[3] = {(L.k[0] - 1) * L.dil[0] + 1, (L.k[1] - 1) * L.dil[1] + 1, (L.k[2] - 1) * L.dil[2] + 1};
            std::vector<float> f((size_t)L.units * ek[0] * ek[1] * ek[2] * C, 0.f);
            for (int n = 0; n < L.units; ++n) for (int a = 0; a < L.k[0]; ++a) for (int y = 0; y < L.k[1]; ++y) for (int x = 0; x < L.k[2]; ++x) {
                int pa = a * L.dil[0], py = y * L.dil[1], px = x * L.dil[2];
                if (transposed) { pa = ek[0] - 1 - pa; py = ek[1] - 1 - py; px = ek[2] - 1 - px; }
                std::copy_n(&w[((((size_t)n * L.k[0] + a) * L.k[1] + y) * L.k[2] + x) * C], C,
                            &f[((((size_t)n * ek[0] + pa) * ek[1] + py) * ek[2] + px) * C]);
            }
            for (int i = 0; i < 3; ++i) { L.k[i] = ek[i]; L.dil[i] = 1; }
            L.flag_a = transposed;
            L.kdim = ek[0] * ek[1] * ek[2] * C;
            L.w_main = add_gemm_weight(f, L.units, L.kdim, L.ldw);
            L.w_bias = add_conv_bias(bias);
            if (transposed && C % 4 == 0 && L.s[0] * L.s[1] * L.s[2] <= 27) {
                // sub-filters per output phase (pz, py, px) for the form without a patch matrix, as for the 2-D layer
                int lead[3];
                bool every_phase_has_taps = true;
                for (int i = 0; i < 3; ++i) {
                    lead[i] = transposed_lead(L.k[i], L.s[i], L.pad);
                    for (int p = 0; p < L.s[i]; ++p) every_phase_has_taps = every_phase_has_taps && transposed_phase(L.k[i], L.s[i], lead[i], p).taps > 0;
                }
                if (every_phase_has_taps) {
                    for (int pz = 0; pz < L.s[0]; ++pz) for (int py = 0; py < L.s[1]; ++py) for (int px = 0; px < L.s[2]; ++px) {
                        const TransposedPhase tz = transposed_phase(L.k[0], L.s[0], lead[0], pz), ty = transposed_phase(L.k[1], L.s[1], lead[1], py),
                                              tx = transposed_phase(L.k[2], L.s[2], lead[2], px);
                        std::vector<float> sub((size_t)L.units * tz.taps * ty.taps * tx.taps * C);
                        for (int n = 0; n < L.units; ++n) for (int jz = 0; jz < tz.taps; ++jz) for (int jy = 0; jy < ty.taps; ++jy) for (int jx = 0; jx < tx.taps; ++jx)
                            std::copy_n(&f[((((size_t)n * L.k[0] + tz.k0 + L.s[0] * jz) * L.k[1] + ty.k0 + L.s[1] * jy) * L.k[2] + tx.k0 + L.s[2] * jx) * C], C,
                                        &sub[((((size_t)n * tz.taps + jz) * ty.taps + jy) * tx.taps + jx) * C]);
                        int ld = 0;
                        L.w_phases.push_back(add_gemm_weight(sub, L.units, tz.taps * ty.taps * tx.taps * C, ld));
                    }
                }
            }
        } else if (t == "DepthwiseConv1D" || t == "DepthwiseConv2D" || t == "SeparableConv1D" || t == "SeparableConv2D") {
            const bool separable = t[0] == 'S';
            L.pad = parse_padding(cfg["padding"].str());
            shape2(cfg["strides"], L.s[1], L.s[2]);
            shape2(cfg["dilation_rate"], L.dil[1], L.dil[2]);
            shape2(cfg["kernel_size"], L.k[1], L.k[2]);
            const std::vector<float> sw = fl("slice_weights");
            const int area = L.k[1] * L.k[2];
            ensure(area > 0 && sw.size() % (size_t)area == 0, "invalid number of weights");
            const int C = (int)(sw.size() / (size_t)area);
            L.in_feat = C;
            // (C, kh, kw, 1) -> [kh*kw][C]
            std::vector<float> dw((size_t)area * C);
            for (int c = 0; c < C; ++c) for (int a = 0; a < area; ++a) dw[(size_t)a * C + c] = sw[(size_t)c * area + a];
            L.w_aux = add_weight(std::move(dw));
            if (separable) {
                L.units = (int)cfg["filters"].integer();
                std::vector<float> bias((size_t)L.units, 0.f);
                if (cfg["use_bias"].boolean()) bias = fl("bias");
                ensure((int)bias.size() == L.units, "size of bias does not match");
                const std::vector<float> kw_ = fl("stack_weights");
                ensure(kw_.size() == (size_t)C * L.units, "invalid weights sizes");
                L.kdim = C;
                L.w_main = add_gemm_weight(kw_, L.units, C, L.ldw);  // (Cout,1,1,C)
                L.w_bias = add_conv_bias(bias);
            } else {
                L.units = C;
                std::vector<float> bias((size_t)C, 0.f);
                if (cfg["use_bias"].boolean()) bias = fl("bias");
                ensure((int)bias.size() == C, "size of bias does not match");
                L.w_bias = add_conv_bias(bias);
            }
        } else if (t == "Dense") {
            std::vector<float> w = fl("weights");
            L.units = (int)cfg["units"].integer();
            std::vector<float> bias((size_t)L.units, 0.f);
            if (cfg["use_bias"].boolean()) bias = fl("bias");
            ensure((int)bias.size() == L.units, "size of bias does not match");
            ensure(L.units > 0 && w.size() % (size_t)L.units == 0, "invalid weight count");
            L.in_feat = L.kdim = (int)(w.size() / (size_t)L.units);
            L.w_main = add_gemm_weight_transposed(w.data(), L.in_feat, L.units, L.ldw);
            L.w_bias = add_weight(std::move(bias));  // dense always adds its bias row (dense_layer.hpp:85)
        } else if (t == "BatchNormalization") {
            const std::vector<float> mean = fl("moving_mean"), var = fl("moving_variance");
            const auto axes = int_list(cfg["axis"]);
            ensure(axes.size() == 1, "invalid axis configuration");
            L.axes = axes;
            const float eps = (float)cfg["epsilon"].number();
            std::vector<float> gamma, beta;
            if (cfg["scale"].boolean()) gamma = fl("gamma");
            if (cfg["center"].boolean()) beta = fl("beta");
            ensure(var.size() == mean.size(), "invalid sizes");
            ensure(beta.empty() || beta.size() == mean.size(), "invalid sizes");
            ensure(gamma.empty() || gamma.size() == mean.size(), "invalid sizes");
            // inv = 1/sqrt(var + eps) * gamma; shift = beta - mean * inv (tensor.hpp:782-792), in fp32
            std::vector<float> sc(mean.size()), sh(mean.size());
            for (size_t i = 0; i < mean.size(); ++i) {
                const float ve = var[i] + eps;
                const float inv = (1.0f / std::sqrt(ve)) * (gamma.empty() ? 1.0f : gamma[i]);
                const float prod = mean[i] * inv;
                sc[i] = inv;
                sh[i] = (beta.empty() ? 0.0f : beta[i]) - prod;
            }
            L.units = (int)mean.size();
            L.w_scale = add_weight(std::move(sc));
            L.w_shift = add_weight(std::move(sh));
        } else if (t == "LayerNormalization" || t == "RMSNormalization") {
            L.axes = int_list(cfg["axis"]);
            L.eps = (float)cfg["epsilon"].number();
            if (t == "LayerNormalization") {
                if (cfg["scale"].boolean()) L.w_gamma = add_weight(fl("gamma"));
                if (cfg["center"].boolean()) L.w_beta = add_weight(fl("beta"));
            } else {
                L.w_gamma = add_weight(fl("scale"));
                L.flag_a = true;  // rms
            }
        } else if (t == "UnitNormalization") {  // import_model.hpp:868-873
            L.axes = int_list(cfg["axis"]);
        } else if (t == "GroupNormalization") {  // import_model.hpp:850-866
            L.units = (int)cfg["groups"].number();
            L.axes = {(int)cfg["axis"].number()};
            L.eps = (float)cfg["epsilon"].number();
            ensure(L.units > 0, "GroupNormalization groups must be > 0.");
            if (cfg["scale"].boolean()) L.w_gamma = add_weight(fl("gamma"));
            if (cfg["center"].boolean()) L.w_beta = add_weight(fl("beta"));
        } else if (t == "MaxPooling1D" || t == "MaxPooling2D" || t == "MaxPooling3D" || t == "AveragePooling1D" ||
                   t == "AveragePooling2D" || t == "AveragePooling3D") {
            shape3(cfg["pool_size"], L.k);
            shape3(cfg["strides"], L.s);
            L.pad = parse_padding(cfg["padding"].str());
            L.flag_a = t[0] == 'M';
        } else if (t.rfind("GlobalMaxPooling", 0) == 0 || t.rfind("GlobalAveragePooling", 0) == 0) {
            L.flag_a = t.rfind("GlobalMaxPooling", 0) == 0;
            L.flag_b = cfg["keepdims"].boolean();
        } else if (t == "Add" || t == "Subtract" || t == "Multiply" || t == "Average" || t == "Maximum" || t == "Minimum") {
            // merge layers carry no parameters
        } else if (t == "Concatenate") {
            L.axes = {(int)cfg["axis"].integer()};
        } else if (t == "Flatten") {
        } else if (t == "Reshape") {
            for (const auto& d : cfg["target_shape"].arr) L.target.push_back(d.is_null() || d.integer() < 0 ? -1 : d.integer());
            ensure(!L.target.empty() && L.target.size() <= 5, "tensor_shape_variable needs 1, 2, 3, 4 or 5 dimensions");
        } else if (t == "Permute") {
            for (const auto& d : cfg["dims"].arr) L.target.push_back(d.integer());
            std::vector<int64_t> sorted = L.target;
            std::sort(sorted.begin(), sorted.end());
            bool ok = !sorted.empty() && sorted.front() >= 1 && sorted.back() <= 5;
            for (size_t i = 1; ok && i < sorted.size(); ++i) ok = sorted[i] != sorted[i - 1];
            ensure(ok, "Invalid dims for permute_tensor.");
        } else if (t == "ZeroPadding1D" || t == "ZeroPadding2D" || t == "ZeroPadding3D" || t == "Cropping1D" ||
                   t == "Cropping2D" || t == "Cropping3D") {  // import_model.hpp:1031-1113
            L.flag_a = t[0] == 'Z';
            const Json& p = L.flag_a ? cfg["padding"] : cfg["cropping"];
            std::vector<std::vector<int>> v;
            for (const auto& a : p.arr) v.push_back(int_list(a));
            const bool ok = (v.size() == 2 && v[0].size() == v[1].size()) || (v.size() == 3 && v[0].size() == v[1].size() && v[1].size() == v[2].size());
            ensure(ok, L.flag_a ? "invalid padding format" : "invalid cropping format");
            if (v[0].size() == 1) { L.pads[4] = v[0][0]; L.pads[5] = v[1][0]; }
            else if (v.size() == 2) { L.pads[2] = v[0][0]; L.pads[3] = v[0][1]; L.pads[4] = v[1][0]; L.pads[5] = v[1][1]; }
            else { L.pads[0] = v[0][0]; L.pads[1] = v[0][1]; L.pads[2] = v[1][0]; L.pads[3] = v[1][1]; L.pads[4] = v[2][0]; L.pads[5] = v[2][1]; }
        } else if (t == "Embedding") {
            L.input_dim = (int)cfg["input_dim"].integer();
            L.units = (int)cfg["output_dim"].integer();
            std::vector<float> w = fl("weights");
            ensure(w.size() == (size_t)L.input_dim * L.units, "invalid embedding weights");
            L.w_main = add_weight(std::move(w));
        } else if (t == "LSTM" || t == "GRU" || t == "SimpleRNN") {  // import_model.hpp:1491-1566
            recurrent_cell(L, t, cfg, cfg, prefix, L.name, "", false);
        } else if (t == "Bidirectional") {  // import_model.hpp:1627-1659
            const std::string mode = cfg["merge_mode"].str();
            const Json& wrapped = cfg["layer"];
            const std::string wt = wrapped["class_name"].str();
            ensure(wt == "LSTM" || wt == "GRU" || wt == "SimpleRNN", "Bidirectional wrapper around layer '" + wt + "' not supported.");
            ensure(mode == "concat" || mode == "sum" || mode == "mul" || mode == "ave", "Bidirectional merge mode '" + mode + "' not supported.");
            L.cells.resize(3);
            for (int dir = 0; dir < 2; ++dir) {
                Layer& C = L.cells[(size_t)dir];
                C.name = L.name;
                recurrent_cell(C, wt, wrapped["config"], wrapped["config"], prefix, L.name, dir == 0 ? "forward_" : "backward_", false);
                C.flag_b = false;       // the wrapper never returns states (bidirectional_layer.hpp:66-95)
                C.reverse = dir == 1;
            }
            L.flag_a = L.cells[0].flag_a;
            L.units = L.cells[0].units;
            Layer& M = L.cells[2];      // how the two directions are merged, as a merge layer of its own
            M.name = L.name;
            M.cls = mode == "concat" ? "Concatenate" : mode == "sum" ? "Add" : mode == "mul" ? "Multiply" : "Average";
            if (mode == "concat") M.axes = {-1};
        } else if (t == "TimeDistributed") {  // import_model.hpp:1753-1769: the wrapped layer carries the wrapper's name
            Json inner = cfg["layer"];
            ensure(inner.is_object(), "TimeDistributed: missing wrapped layer");
            auto put = [&](const char* key, const Json& v) {
                for (auto& kv : inner.obj)
                    if (kv.first == key) { kv.second = v; return; }
                inner.obj.emplace_back(key, v);
            };
            put("name", data["name"]);
            put("inbound_nodes", data["inbound_nodes"]);
            L.k[0] = (int)fl("td_input_len").at(0);
            L.k[1] = (int)fl("td_output_len").at(0);
            ensure(L.k[1] > 1, "Wrong input dimension");
            L.cells.push_back(layer(inner, prefix));
        } else if (t == "RNN") {  // import_model.hpp:1568-1626: one cell, or a chain of them (stacked_rnn_layer.hpp:21-45)
            const Json& cell = cfg["cell"];
            const std::string cc = cell["class_name"].str();
            auto layer_class = [&](const std::string& c) -> std::string {
                ensure(c == "LSTMCell" || c == "GRUCell" || c == "SimpleRNNCell", "RNN cell '" + c + "' is not supported.");
                return c.substr(0, c.size() - 4);
            };
            if (cc == "StackedRNNCells") {
                const Json& cells = cell["config"]["cells"];
                ensure(cells.is_array() && cells.size() > 0, "StackedRNNCells must contain at least one cell.");
                L.cells.resize(cells.size());
                for (size_t i = 0; i < cells.size(); ++i) {
                    Layer& C = L.cells[i];
                    C.name = L.name + "_cell" + std::to_string(i);
                    recurrent_cell(C, layer_class(cells.arr[i]["class_name"].str()), cells.arr[i]["config"], cfg, prefix, L.name,
                                   "cell" + std::to_string(i) + "_", i + 1 != cells.size());
                }
            } else {
                L.cells.resize(1);
                L.cells[0].name = L.name;
                recurrent_cell(L.cells[0], layer_class(cc), cell["config"], cfg, prefix, L.name, "", false);
            }
        } else if (t == "MultiHeadAttention") {  // import_model.hpp:1467-1489; multi_head_attention_layer.hpp:20-72
            L.heads = (int)cfg["num_heads"].integer();
            L.key_dim = (int)cfg["key_dim"].integer();
            L.value_dim = (int)cfg["value_dim"].integer();
            const bool use_bias = cfg["use_bias"].boolean();
            const Json& wsj = param(prefix, L.name, "weights");
            const Json& shj = param(prefix, L.name, "weight_shapes");
            ensure(wsj.is_array() && shj.is_array() && wsj.size() == shj.size(), "invalid MultiHeadAttention weights");
            std::vector<std::vector<float>> ws;
            std::vector<std::vector<int>> shapes;
            for (const auto& w : wsj.arr) ws.push_back(decode_floats(w));
            for (const auto& s : shj.arr) shapes.push_back(int_list(s));
            const size_t f = use_bias ? 2 : 1;
            ensure(ws.size() == 4 * f, "invalid number of MultiHeadAttention weights");
            const int H = L.heads;
            auto proj = [&](size_t idx, int units, int& w_id, int& b_id) {
                const std::vector<float>& w = ws[f * idx];
                ensure(shapes[f * idx].size() == 3 && shapes[f * idx][1] == H && shapes[f * idx][2] == units,
                       "Invalid weights shape for attention head dimension.");
                const int dim = shapes[f * idx][0];
                ensure(w.size() == (size_t)dim * H * units, "Invalid weights for number of heads.");
                int ldw = 0;
                w_id = add_gemm_weight_transposed(w.data(), dim, H * units, ldw);  // (dim, H*units) -> [H*units][dim]
                L.in_feat = dim;
                L.ldw = ldw;
                if (use_bias) {
                    ensure(ws[f * idx + 1].size() == (size_t)H * units, "Invalid biases shape for attention head dimension.");
                    b_id = add_weight(std::vector<float>(ws[f * idx + 1]));
                }
            };
            proj(0, L.key_dim, L.w_q, L.b_q);
            proj(1, L.key_dim, L.w_k, L.b_k);
            proj(2, L.value_dim, L.w_v, L.b_v);
            const std::vector<float>& wo = ws[f * 3];
            L.out_dim = shapes[f * 3].back();
            const int hv = H * L.value_dim;
            ensure(wo.size() == (size_t)hv * L.out_dim, "invalid MultiHeadAttention output weights");
            int ldo = 0;
            L.w_o = add_gemm_weight_transposed(wo.data(), hv, L.out_dim, ldo);
            L.kdim = ldo;
            if (use_bias) L.b_o = add_weight(std::vector<float>(ws[f * 3 + 1]));
        } else if (t == "Activation") {
            L.act = make_activation(cfg["activation"].str(), data);
            L.flag_a = true;
        } else if (t == "Rescaling") {  // import_model.hpp:1135-1142: an element-wise scale * x + offset
            L.act.kind = ACT_AFFINE;
            L.act.p0 = (float)cfg["scale"].number();
            L.act.p1 = (float)cfg["offset"].number();
            L.flag_a = true;
        } else if (t == "Normalization") {  // import_model.hpp:1392-1404
            L.axes = int_list(cfg["axis"]);
            if (cfg["axis"].is_array() && cfg["axis"].size() == 0) L.axes.clear();
            ensure(L.axes.size() <= 1, "Unsupported number of axes for Normalization layer");
            std::vector<float> mean = fl("mean"), var = fl("variance");
            ensure(mean.size() == var.size(), "Invalid number of variance values in Normalization layer.");
            L.units = (int)var.size();
            L.flag_a = cfg.get_bool("invert", false);
            L.w_scale = add_weight(std::move(mean));
            L.w_shift = add_weight(std::move(var));
        } else if (t == "UpSampling1D" || t == "UpSampling2D") {  // import_model.hpp:921-939
            if (t == "UpSampling1D") { L.k[1] = 1; L.k[2] = (int)cfg["size"].integer(); }
            else shape2(cfg["size"], L.k[1], L.k[2]);
            const std::string interp = t == "UpSampling2D" ? cfg["interpolation"].str() : std::string("nearest");
            ensure(interp == "nearest" || interp == "bilinear", "Invalid interpolation method: " + interp);
            L.flag_a = interp == "bilinear";
            ensure(L.k[1] > 0 && L.k[2] > 0, "invalid upsampling size");
        } else if (t == "UpSampling3D") {  // import_model.hpp:941-948
            shape3(cfg["size"], L.k);
            ensure(L.k[0] > 0 && L.k[1] > 0 && L.k[2] > 0, "invalid upsampling size");
        } else if (t == "RepeatVector") {  // import_model.hpp:1127-1133
            L.k[1] = 1;
            L.k[2] = (int)cfg["n"].integer();
            ensure(L.k[2] > 0, "invalid RepeatVector count");
        } else if (t == "Resizing") {  // import_model.hpp:1152-1161
            L.k[1] = (int)cfg["height"].integer();
            L.k[2] = (int)cfg["width"].integer();
            ensure(L.k[1] > 0 && L.k[2] > 0, "invalid Resizing size");
            const std::string interp = cfg["interpolation"].str();
            ensure(interp == "nearest" || interp == "bilinear" || interp == "area", "Invalid interpolation method: " + interp);
            L.bin_op = interp == "nearest" ? 0 : interp == "bilinear" ? 1 : 2;
            L.flag_a = cfg["crop_to_aspect_ratio"].boolean();
        } else if (t == "Dot") {  // import_model.hpp:995-1002
            L.axes = int_list(cfg["axes"]);
            ensure(L.axes.size() == 1 || L.axes.size() == 2, "axes must have size 1 or 2");
            if (L.axes.size() == 1) L.axes.push_back(L.axes[0]);
            L.flag_a = cfg["normalize"].boolean();
        } else if (t.rfind("AdaptiveAveragePooling", 0) == 0 || t.rfind("AdaptiveMaxPooling", 0) == 0) {  // import_model.hpp:678-710
            std::vector<int> dims = int_list(cfg["output_size"]);
            ensure(!dims.empty(), "AdaptivePooling needs an output size");
            L.k[0] = dims.size() >= 3 ? dims[dims.size() - 3] : 1;
            L.k[1] = dims.size() >= 2 ? dims[dims.size() - 2] : 1;
            L.k[2] = dims.back();
            L.flag_a = t.rfind("AdaptiveMaxPooling", 0) == 0;
            L.cls = "AdaptivePooling";
        } else if (t == "Discretization") {  // import_model.hpp:787-797
            ensure(cfg["output_mode"].str() == "int", "Discretization only supports output_mode='int'.");
            std::vector<float> bounds;
            for (const auto& v : cfg["bin_boundaries"].arr) bounds.push_back((float)v.number());
            L.units = (int)bounds.size();
            L.w_main = add_weight(std::move(bounds));
        } else if (t == "IntegerLookup") {  // import_model.hpp:799-818, integer_lookup_layer.hpp:24-81
            ensure(cfg["output_mode"].str() == "int", "IntegerLookup only supports output_mode='int'.");
            ensure(!cfg.get_bool("invert", false), "IntegerLookup with invert=True is not supported.");
            ensure(cfg["num_oov_indices"].integer() == 1, "IntegerLookup requires num_oov_indices == 1.");
            L.flag_a = !cfg["mask_token"].is_null();
            const int64_t mask = L.flag_a ? cfg["mask_token"].integer() : 0;
            // Inputs are floats cast to integers: a key matters only if some float equals it.  Later duplicates win, as in
            // the reference's map.  Stored sorted by key: keys | positions (as floats) | mask token.
            std::map<int64_t, int64_t> index;
            int64_t pos = 0;
            for (const auto& v : cfg["vocabulary"].arr) {
                const int64_t key = v.integer();
                if ((int64_t)(float)key == key) index[key] = pos;
                ++pos;
            }
            std::vector<float> table;
            for (const auto& kv : index) table.push_back((float)kv.first);
            for (const auto& kv : index) table.push_back((float)(kv.second + (L.flag_a ? 1 : 0) + 1));   // vocab_offset = mask + one OOV bucket
            table.push_back((float)mask);
            L.units = (int)index.size();
            L.w_main = add_weight(std::move(table));
        } else if (t == "CategoryEncoding") {  // import_model.hpp:1406-1413
            L.units = (int)cfg["num_tokens"].integer();
            const std::string mode = cfg["output_mode"].str();
            ensure(mode == "one_hot" || mode == "multi_hot" || mode == "count", "Unsupported output mode (" + mode + ").");
            L.bin_op = mode == "one_hot" ? 0 : mode == "multi_hot" ? 1 : 2;
            ensure(L.units > 0, "CategoryEncoding needs num_tokens > 0");
        } else if (t == "CenterCrop") {  // import_model.hpp:1118-1125
            L.k[1] = (int)cfg["height"].integer();
            L.k[2] = (int)cfg["width"].integer();
            ensure(L.k[1] > 0 && L.k[2] > 0, "invalid CenterCrop size");
        } else if (t == "EinsumDense") {  // import_model.hpp:820-848
            const std::string eq = cfg["equation"].str();
            const size_t comma = eq.find(','), arrow = eq.find("->");
            ensure(comma != std::string::npos && arrow != std::string::npos && comma < arrow, "EinsumDense: invalid equation");
            L.eq_in = eq.substr(0, comma);
            L.eq_kernel = eq.substr(comma + 1, arrow - comma - 1);
            L.eq_out = eq.substr(arrow + 2);
            ensure(L.eq_out.size() >= 2, "EinsumDense output equation must have at least a batch char and one feature char.");
            ensure(L.eq_in.size() <= 6 && L.eq_out.size() <= 8 && L.eq_kernel.size() <= 5, "EinsumDense: too many letters");
            const std::string axes = cfg["bias_axes"].is_null() ? std::string() : cfg["bias_axes"].str();
            for (char ch : L.eq_out) if (axes.find(ch) != std::string::npos) L.eq_bias.push_back(ch);
            L.target.push_back(-1);  // the batch letter, then Keras' output_shape (import_model.hpp:828-833)
            for (const auto& d : cfg["output_shape"].arr) L.target.push_back(d.is_null() ? -1 : d.integer());
            for (int d : int_list(param(prefix, L.name, "kernel_shape"))) L.kernel_dims.push_back(d);
            ensure(L.eq_kernel.size() <= L.kernel_dims.size(), "EinsumDense: kernel chars exceed kernel dimensions.");
            std::vector<float> kernel = fl("kernel");
            int64_t kvol = 1;
            for (int64_t d : L.kernel_dims) kvol *= d;
            ensure((int64_t)kernel.size() == kvol, "EinsumDense: kernel size does not match kernel_shape");
            std::vector<float> bias;
            if (!axes.empty()) bias = fl("bias");
            // Matrix-product form "X S , S O -> X O" (X not in the kernel): rows = X, K = S, N = O.  The kernel is then
            // stored [N][K] like a Dense kernel and the bias, which may cover only some of O's letters, is spread over N.
            auto sizes_of = [&](const std::string& letters) {
                int64_t v = 1;
                for (char ch : letters) v *= L.kernel_dims[L.kernel_dims.size() - L.eq_kernel.size() + L.eq_kernel.find(ch)];
                return v;
            };
            bool distinct = true;
            for (const std::string* e : {&L.eq_in, &L.eq_kernel, &L.eq_out})
                for (size_t i = 0; i < e->size(); ++i) distinct = distinct && e->find((*e)[i], i + 1) == std::string::npos;
            ensure(distinct, "EinsumDense: repeated letters are not supported");
            size_t ns = 0;
            while (ns < L.eq_kernel.size() && L.eq_out.find(L.eq_kernel[ns]) == std::string::npos) ns++;
            const std::string S = L.eq_kernel.substr(0, ns), O = L.eq_kernel.substr(ns);
            bool matrix = ns > 0 && !O.empty() && L.eq_in.size() > ns && L.eq_in.substr(L.eq_in.size() - ns) == S &&
                          L.eq_out.size() > O.size() && L.eq_out.substr(L.eq_out.size() - O.size()) == O &&
                          L.eq_in.substr(0, L.eq_in.size() - ns) == L.eq_out.substr(0, L.eq_out.size() - O.size());
            for (char ch : L.eq_in.substr(0, L.eq_in.size() - std::min(ns, L.eq_in.size()))) matrix = matrix && L.eq_kernel.find(ch) == std::string::npos;
            for (char ch : L.eq_bias) matrix = matrix && O.find(ch) != std::string::npos;
            if (matrix) {
                L.flag_a = true;
                L.kdim = L.in_feat = (int)sizes_of(S);
                L.units = (int)sizes_of(O);
                L.w_main = add_gemm_weight_transposed(kernel.data(), L.in_feat, L.units, L.ldw);
                if (!L.eq_bias.empty()) {
                    std::vector<float> full((size_t)L.units, 0.f);
                    for (int n = 0; n < L.units; ++n) {
                        int64_t r = n, bo = 0, bstride = 1;
                        for (size_t i = O.size(); i-- > 0;) {
                            const int64_t sz = sizes_of(std::string(1, O[i])), cdx = r % sz;
                            r /= sz;
                            if (L.eq_bias.find(O[i]) != std::string::npos) { bo += cdx * bstride; bstride *= sz; }
                        }
                        ensure((size_t)bo < bias.size(), "EinsumDense: bias size does not match bias_axes");
                        full[(size_t)n] = bias[(size_t)bo];
                    }
                    L.w_bias = add_weight(std::move(full));
                }
            } else {
                L.w_main = add_weight(std::move(kernel));
                if (!L.eq_bias.empty()) { L.input_dim = (int)bias.size(); L.w_bias = add_weight(std::move(bias)); }
            }
        } else if (t == "PReLU") {  // import_model.hpp:1368-1379
            if (cfg.is_object() && cfg.contains("shared_axes") && cfg["shared_axes"].is_array())
                for (const auto& a : cfg["shared_axes"].arr) L.axes.push_back((int)a.integer());
            std::vector<float> alpha = fl("alpha");
            L.input_dim = (int)alpha.size();
            L.w_main = add_weight(std::move(alpha));
        } else if (t == "Attention" || t == "AdditiveAttention") {  // import_model.hpp:1415-1442
            const bool additive = t == "AdditiveAttention";
            const bool use_scale = cfg["use_scale"].boolean();
            const std::string mode = additive ? "additive" : cfg["score_mode"].str();
            ensure(additive || mode == "dot" || mode == "concat", "Invalid score_mode for Attention layer.");
            L.bin_op = additive ? 2 : mode == "concat" ? 1 : 0;
            if (use_scale && additive) {
                std::vector<float> sv = fl("scale");
                L.input_dim = (int)sv.size();
                L.w_aux = add_weight(std::move(sv));
            } else if (use_scale) {
                L.f_scale = (float)param(prefix, L.name, "scale").number();
            }
            if (mode == "concat") L.f_w2 = (float)param(prefix, L.name, "concat_score_weight").number();
        } else if (t == "GroupQueryAttention" || t == "GroupedQueryAttention") {  // import_model.hpp:1444-1466
            // weights: Q, K, [gate], V, out, each followed by its bias (group_query_attention_layer.hpp:46-60)
            const int hd = (int)cfg["head_dim"].integer();
            L.heads = (int)cfg["num_query_heads"].integer();
            L.kv_heads = (int)cfg["num_key_value_heads"].integer();
            L.key_dim = L.value_dim = hd;
            const bool use_bias = cfg["use_bias"].boolean();
            const bool use_gate = cfg.get_bool("use_gate", false);
            ensure(L.kv_heads > 0, "num_key_value_heads must be > 0.");
            ensure(L.heads % L.kv_heads == 0, "num_query_heads must be divisible by num_key_value_heads.");
            const Json& wsj = param(prefix, L.name, "weights");
            const Json& shj = param(prefix, L.name, "weight_shapes");
            ensure(wsj.is_array() && shj.is_array() && wsj.size() == shj.size(), "invalid GroupQueryAttention weights");
            std::vector<std::vector<float>> ws;
            std::vector<std::vector<int>> shapes;
            for (const auto& w : wsj.arr) ws.push_back(decode_floats(w));
            for (const auto& sh : shj.arr) shapes.push_back(int_list(sh));
            const size_t f = use_bias ? 2 : 1;
            ensure(ws.size() == (use_gate ? 5u : 4u) * f, "invalid number of GroupQueryAttention weights");
            L.in_feat = shapes[0].empty() ? 0 : shapes[0][0];
            auto proj = [&](size_t idx, int heads, int& w_id, int& b_id) {
                const std::vector<float>& w = ws[f * idx];
                ensure(shapes[f * idx].size() == 3 && shapes[f * idx][0] == L.in_feat && shapes[f * idx][1] == heads && shapes[f * idx][2] == hd &&
                           w.size() == (size_t)L.in_feat * heads * hd,
                       "GroupQueryAttention kernels must have the shape (dim, heads, head_dim) with one dim for query, key and value.");
                int ldw = 0;
                w_id = add_gemm_weight_transposed(w.data(), L.in_feat, heads * hd, ldw);
                L.ldw = ldw;
                if (use_bias) {
                    ensure(ws[f * idx + 1].size() == (size_t)heads * hd, "invalid GroupQueryAttention bias");
                    b_id = add_weight(std::vector<float>(ws[f * idx + 1]));
                }
            };
            proj(0, L.heads, L.w_q, L.b_q);
            proj(1, L.kv_heads, L.w_k, L.b_k);
            if (use_gate) proj(2, L.heads, L.w_g, L.b_g);
            proj(use_gate ? 3 : 2, L.kv_heads, L.w_v, L.b_v);
            const size_t oi = f * (use_gate ? 4 : 3);
            L.out_dim = shapes[oi].back();
            const int hv = L.heads * hd;
            ensure(ws[oi].size() == (size_t)hv * L.out_dim, "invalid GroupQueryAttention output weights");
            int ldo = 0;
            L.w_o = add_gemm_weight_transposed(ws[oi].data(), hv, L.out_dim, ldo);
            L.kdim = ldo;
            if (use_bias) L.b_o = add_weight(std::vector<float>(ws[oi + 1]));
        } else {
            // parameter-free activation layers and identity layers
            static const std::map<std::string, std::string> act_layers = {
                {"ReLU", "relu"}, {"LeakyReLU", "leaky_relu"}, {"ELU", "elu"}, {"Softmax", "softmax"}, {"Relu6", "relu6"},
                {"Gelu", "gelu"}, {"Sigmoid", "sigmoid"}, {"Tanh", "tanh"}, {"Silu", "silu"}, {"Softplus", "softplus"},
                {"Softsign", "softsign"}, {"Selu", "selu"}, {"Elu", "elu"}, {"Exp", "exponential"}, {"HardSigmoid", "hard_sigmoid"},
                {"LeakyRelu", "leaky_relu"}, {"Celu", "celu"}, {"HardTanh", "hard_tanh"}, {"LogSigmoid", "log_sigmoid"},
                {"LogSoftmax", "log_softmax"}, {"TanhShrink", "tanh_shrink"}, {"Threshold", "threshold"}, {"HardShrink", "hard_shrink"},
                {"SoftShrink", "soft_shrink"}, {"SparsePlus", "sparse_plus"}, {"Squareplus", "squareplus"}};
            // layers that pass their input through at inference (import_model.hpp:1790-1838)
            static const char* identity[] = {"Identity", "Dropout", "Masking", "ActivityRegularization", "AlphaDropout", "FixedDropout",
                                             "GaussianDropout", "GaussianNoise", "SpatialDropout1D", "SpatialDropout2D", "SpatialDropout3D",
                                             "AugMix", "CutMix", "Equalization", "MaxNumBoundingBoxes", "MixUp", "Pipeline", "RandAugment",
                                             "Solarization"};
            auto it = act_layers.find(t);
            if (it != act_layers.end()) {
                L.act = make_activation(it->second, data);
                L.cls = "Activation";
                L.flag_a = true;
            } else {
                bool is_identity = false;
                for (const char* n : identity) if (t == n) is_identity = true;
                if (t.rfind("Random", 0) == 0) is_identity = true;  // augmentation layers pass through at inference
                ensure(is_identity, "unknown layer type: " + t);
                L.cls = "Identity";
            }
        }

        // attached activation (import_model.hpp:1953-1962)
        const bool consumes = t == "Activation" || t == "LSTM" || t == "GRU" || t == "SimpleRNN" || t == "Bidirectional";
        if (!consumes && cfg.is_object() && cfg.contains("activation")) {
            ensure(cfg["activation"].is_string(), "Layer activation must be a string.");
            L.has_act = true;
            ensure(cfg["activation"].str() != "threshold", "unknown activation type: threshold");
            L.act = make_activation(cfg["activation"].str(), data);
        }
        L.nodes = create_nodes(data);
        return L;
    }
};

static std::vector<VarShape> var_shapes(const Json& d) {  // import_model.hpp:338-341,148-208
    std::vector<VarShape> r;
    auto one = [](const Json& s) {
        ensure(s.is_array(), "tensor_shape_variable needs to be an array");
        ensure(s.size() > 0, "need at least one dimension");
        ensure(s.size() <= 5, "tensor_shape_variable needs 1, 2, 3, 4 or 5 dimensions");
        VarShape v;
        for (const auto& x : s.arr) v.dims.push_back(x.is_null() || x.integer() < 0 ? -1 : x.integer());
        return v;
    };
    if (d.is_array() && !d.empty() && d[0].is_array()) for (const auto& s : d.arr) r.push_back(one(s));
    else r.push_back(one(d));
    return r;
}

}  // namespace

LoadedModel load_model_json(const char* text, size_t len, bool cell_order_copies) {
    // FDK_LOAD_TIMING=1 prints how long the JSON parse and the layer/weight decoding take
    static const bool timing = getenv("FDK_LOAD_TIMING") != nullptr;
    const auto t_start = std::chrono::steady_clock::now();
    const Json j = Json::parse(text, len);
    const auto t_parsed = std::chrono::steady_clock::now();
    struct Report {
        bool on; std::chrono::steady_clock::time_point a, b; size_t len;
        ~Report() {
            if (!on) return;
            const auto c = std::chrono::steady_clock::now();
            fprintf(stderr, "fdk load: %.1f MB, parse %.0f ms, layers and weights %.0f ms (of which base64 %.0f ms, transposes %.0f ms; totals of this process)\n",
                    (double)len / 1e6, std::chrono::duration<double, std::milli>(b - a).count(),
                    std::chrono::duration<double, std::milli>(c - b).count(), (double)g_decode_ns.load() / 1e6, (double)g_pack_ns.load() / 1e6);
        }
    } report{timing, t_start, t_parsed, len};
    ensure(j["image_data_format"].is_string() && j["image_data_format"].str() == "channels_last",
           "only channels_last data format supported");
    LoadedModel lm;
    Loader loader{j["trainable_params"], lm.weights};
    loader.cell_order_copies = cell_order_copies;
    const Json& arch = j["architecture"];
    lm.root = loader.model(arch, arch["config"]["name"].is_string() ? arch["config"]["name"].str() : std::string("model"), "");
    lm.input_shapes = var_shapes(j["input_shapes"]);
    lm.output_shapes = var_shapes(j["output_shapes"]);
    lm.hash = j.get_str("hash", "");
    const Json& tests = j["tests"];
    if (tests.is_array()) {
        for (const auto& t : tests.arr) {
            ensure(t["inputs"].is_array(), "test needs inputs");
            ensure(t["outputs"].is_array(), "test needs outputs");
            TestCase tc;
            auto load = [](const Json& arr, std::vector<TShape>& shapes, std::vector<std::vector<float>>& vals) {
                for (const auto& x : arr.arr) {
                    std::vector<int64_t> dims;
                    for (const auto& d : x["shape"].arr) dims.push_back(d.integer());
                    shapes.push_back(TShape::from_dims(dims));
                    vals.push_back(decode_floats(x["values"]));
                    ensure((int64_t)vals.back().size() == shapes.back().volume(), "invalid number of values");
                }
            };
            load(t["inputs"], tc.in_shapes, tc.in_values);
            load(t["outputs"], tc.out_shapes, tc.out_values);
            lm.tests.push_back(std::move(tc));
        }
    }
    return lm;
}

}  // namespace fdk
