// Plan compiler: walks the layer graph for one input-shape signature, infers shapes with the
// reference's rules, emits device operations, folds BatchNormalization / activation / residual Add into
// the producing contraction, and assigns arena offsets by liveness.
#include "engine.hpp"
#include "plan_attrs.hpp"

#include <algorithm>
#include <cmath>
#include <functional>
#include <set>

namespace fdk {

namespace {

int ceil_like(int num, int den) {  // fplus::ceil(float(num) / float(den) - 0.001), convolution.hpp:343-352
    return (int)std::ceil((float)num / (float)den - 0.001f);
}
struct Geom1 { int out, pad_lo, pad_hi; };
// One spatial dimension of preprocess_convolution (convolution.hpp:320-396) /
// preprocess_convolution_3d (convolution3d.hpp:35-134).
Geom1 conv_geom(int in, int k, int s, int pad, bool transposed) {
    Geom1 g{0, 0, 0};
    if (pad == PAD_SAME || pad == PAD_CAUSAL) g.out = ceil_like(in, s);
    else g.out = transposed ? ceil_like(in + k - 1, s) : ceil_like(in - k + 1, s);
    if (transposed) { g.pad_lo = k - 1; g.pad_hi = k - 1; }
    if (pad == PAD_SAME) {
        const int along = (in % s == 0) ? std::max(k - s, 0) : std::max(k - (in % s), 0);
        g.pad_lo = along / 2;
        g.pad_hi = along - g.pad_lo;
    } else if (pad == PAD_CAUSAL) {
        g.pad_lo = k - 1;
        g.pad_hi = 0;
    }
    ensure(g.out >= 0, "invalid convolution geometry");
    return g;
}

int abs_axis_pos(int rank, int axis) {  // rank_aligned_axis_to_absolute_axis (tensor.hpp:692-699), 0-based
    ensure(axis >= -1, "invalid axis");
    ensure(axis <= rank, "invalid axis");
    return axis == -1 ? 4 : 5 + axis - rank - 1;
}

int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

struct Compiler {
    const LoadedModel& lm;
    const EngineOptions& opt;
    Plan& p;

    int new_buffer(int64_t elems) {
        BufferInfo b;
        b.elems = elems;
        p.buffers.push_back(b);
        return (int)p.buffers.size() - 1;
    }
    int new_tensor(const TShape& s) {
        TensorInfo t;
        t.shape = s;
        t.buf = new_buffer(s.volume());
        p.tensors.push_back(t);
        return (int)p.tensors.size() - 1;
    }
    int view(int src, const TShape& s) {
        TensorInfo t;
        t.shape = s;
        t.buf = p.tensors[(size_t)src].buf;
        p.tensors.push_back(t);
        return (int)p.tensors.size() - 1;
    }
    // By value: callers keep the shape across new_tensor(), which may reallocate p.tensors.
    TShape shape(int t) const { return p.tensors[(size_t)t].shape; }
    Op& push(int kind, const Layer* L, std::vector<int> in, std::vector<int> out) {
        Op o;
        o.kind = kind;
        o.layer = L;
        o.in = std::move(in);
        o.out = std::move(out);
        p.ops.push_back(std::move(o));
        return p.ops.back();
    }

    // ---- graph walk (model_layer.hpp:51-66, layer.hpp:63-80, node.hpp:66-74) --------------------------
    std::vector<int> emit_model(const ModelDef& m, const std::vector<int>& inputs) {
        ensure(inputs.size() == m.inputs.size(), "invalid number of input tensors for this model: " + std::to_string(m.inputs.size()) +
                                                     " required but " + std::to_string(inputs.size()) + " provided");
        std::map<std::pair<std::string, int>, std::vector<int>> cache;
        for (size_t i = 0; i < inputs.size(); ++i) cache[{m.inputs[i].layer, m.inputs[i].node}] = {inputs[i]};
        std::function<int(const Conn&, int)> get = [&](const Conn& c, int depth) -> int {
            ensure(depth < 100000, "graph too deep");
            const Layer& L = m.find(c.layer);
            int node_idx = c.node;
            if (L.sub && node_idx >= 1) node_idx -= 1;  // model_layer.hpp:42-44
            const auto key = std::make_pair(c.layer, node_idx);
            auto it = cache.find(key);
            if (it == cache.end()) {
                ensure(node_idx >= 0 && node_idx < (int)L.nodes.size(), "invalid node index");
                std::vector<int> ins;
                for (const Conn& ic : L.nodes[(size_t)node_idx]) ins.push_back(get(ic, depth + 1));
                it = cache.emplace(key, emit_layer(L, ins)).first;
            }
            ensure(c.tensor >= 0 && c.tensor < (int)it->second.size(), "invalid tensor index");
            return it->second[(size_t)c.tensor];
        };
        std::vector<int> outs;
        for (const Conn& c : m.outputs) outs.push_back(get(c, 0));
        return outs;
    }

    int emit_activation(const ActSpec& a, int in, const Layer* L) {
        if (a.kind == ACT_NONE) return in;
        const int out = new_tensor(shape(in));
        if (a.kind == ACT_SOFTMAX || a.kind == ACT_LOG_SOFTMAX) {
            Op& o = push(OP_SOFTMAX, L, {in}, {out});
            o.a[0] = a.kind == ACT_LOG_SOFTMAX;
        } else {
            Op& o = push(OP_UNARY, L, {in}, {out});
            o.act = a;
        }
        return out;
    }

    int single(const std::vector<int>& ins) {
        ensure(ins.size() == 1, "invalid number of input tensors");
        return ins[0];
    }

    // resize_tensor_2d / smart_resize_tensor_2d (tensor.hpp:1113-1163): rank <= 3 input -> (height, width, depth); with
    // `crop` the input is first cropped in the middle to the target's aspect ratio.  mode 0 nearest, 1 bilinear, 2 area.
    int emit_resize(const Layer& L, int in, int64_t height, int64_t width, int mode, bool crop) {
        const TShape sh = shape(in);
        ensure(sh.d[0] == 1 && sh.d[1] == 1, "Resizing: the input must have rank <= 3");
        const int64_t H = sh.d[2], W = sh.d[3];
        int64_t ch = H, cw = W, y0 = 0, x0 = 0;
        if (crop) {
            ch = std::min<int64_t>(H, (int64_t)((float)(W * height) / (float)width));
            cw = std::min<int64_t>(W, (int64_t)((float)(H * width) / (float)height));
            y0 = (int64_t)((float)(H - ch) / 2.0f);
            x0 = (int64_t)((float)(W - cw) / 2.0f);
            ensure(ch > 0 && cw > 0, "Resizing: the cropped input is empty");
        }
        const int out = new_tensor(TShape::from_dims({height, width, sh.d[4]}));
        Op& o = push(OP_RESIZE, &L, {in}, {out});
        o.a[0] = H; o.a[1] = W; o.a[2] = sh.d[4]; o.a[3] = height; o.a[4] = width; o.a[5] = mode;
        o.a[6] = y0; o.a[7] = x0; o.a[8] = ch; o.a[9] = cw;
        return out;
    }

    std::vector<int> emit_layer(const Layer& L, const std::vector<int>& ins) {
        std::vector<int> outs = emit_impl(L, ins);
        if (L.has_act)
            for (int& t : outs) t = emit_activation(L.act, t, &L);
        return outs;
    }

    std::vector<int> emit_impl(const Layer& L, const std::vector<int>& ins) {
        const std::string& t = L.cls;
        if (L.sub) return emit_model(*L.sub, ins);
        if (t == "InputLayer" || t == "Identity") return ins;
        if (t == "Conv1D" || t == "Conv2D" || t == "Conv1DTranspose" || t == "Conv2DTranspose") return {emit_conv(L, single(ins))};
        if (t == "DepthwiseConv1D" || t == "DepthwiseConv2D") return {emit_dwconv(L, single(ins), true)};
        if (t == "SeparableConv1D" || t == "SeparableConv2D") {
            // depthwise without bias, then a 1x1 convolution (separable_conv_2d_layer.hpp:47-52)
            const int mid = emit_dwconv(L, single(ins), false);
            const TShape& s = shape(mid);
            TShape os = s;
            os.d[4] = L.units;
            const int out = new_tensor(os);
            Op& o = push(OP_GEMM, &L, {mid}, {out});
            o.a[GEMM_ROWS] = s.volume() / s.d[4];
            o.w_main = L.w_main; o.ldw = L.ldw; o.K = L.kdim; o.N = L.units;
            o.w_bias = L.w_bias;
            p.flops_per_sample += 2.0 * (double)o.a[GEMM_ROWS] * o.K * o.N;
            return {out};
        }
        if (t == "Dense") {
            const int in = single(ins);
            const TShape& s = shape(in);
            ensure(s.d[4] == L.in_feat && s.volume() % s.d[4] == 0, "Invalid input value count.");
            TShape os = s;
            os.d[4] = L.units;
            const int out = new_tensor(os);
            Op& o = push(OP_GEMM, &L, {in}, {out});
            o.a[GEMM_ROWS] = s.volume() / s.d[4];
            o.w_main = L.w_main; o.ldw = L.ldw; o.K = L.kdim; o.N = L.units;
            o.w_bias = L.w_bias;
            p.flops_per_sample += 2.0 * (double)o.a[GEMM_ROWS] * o.K * o.N;
            return {out};
        }
        if (t == "BatchNormalization") {
            const int in = single(ins);
            const TShape& s = shape(in);
            const int pos = abs_axis_pos(s.rank, L.axes[0]);
            ensure(pos >= 0 && pos < 5 && s.d[pos] == L.units, "Invalid shapes for combining tensors.");
            const int out = new_tensor(s);
            Op& o = push(OP_AFFINE, &L, {in}, {out});
            int64_t outer = 1, inner = 1;
            for (int i = 0; i < pos; ++i) outer *= s.d[i];
            for (int i = pos + 1; i < 5; ++i) inner *= s.d[i];
            o.a[AFF_OUTER] = outer; o.a[AFF_NC] = s.d[pos]; o.a[AFF_INNER] = inner;
            o.w_scale = L.w_scale; o.w_shift = L.w_shift;
            return {out};
        }
        if (t == "GroupNormalization") {
            const int in = single(ins);
            const TShape& s = shape(in);
            ensure(abs_axis_pos(s.rank, L.axes[0]) == 4, "GroupNormalization is currently only supported on the last (channel) axis.");
            ensure(s.d[4] % L.units == 0, "Number of channels must be divisible by number of groups.");
            const int out = new_tensor(s);
            Op& o = push(OP_NORM, &L, {in}, {out});
            o.a[NORM_ROWS] = s.volume() / s.d[4]; o.a[NORM_N] = s.d[4]; o.a[NORM_RMS] = 3;
            o.f[0] = L.eps;
            return {out};
        }
        if (t == "LayerNormalization" || t == "RMSNormalization" || t == "UnitNormalization") {
            const int in = single(ins);
            const TShape& s = shape(in);
            std::set<int> pos;
            for (int a : L.axes) pos.insert(abs_axis_pos(s.rank, a));
            // supported: the normalised axes are the trailing contiguous ones
            int64_t n = 1;
            int lo = 5;
            for (int i = 4; i >= 0 && pos.count(i); --i) { n *= s.d[i]; lo = i; }
            ensure((int)pos.size() == 5 - lo, L.cls + ": only trailing normalisation axes are supported by the device engine");
            const int out = new_tensor(s);
            Op& o = push(OP_NORM, &L, {in}, {out});
            o.a[NORM_ROWS] = s.volume() / n; o.a[NORM_N] = n; o.a[NORM_RMS] = t == "UnitNormalization" ? 2 : L.flag_a ? 1 : 0;
            o.f[0] = L.eps;
            return {out};
        }
        if (t.rfind("MaxPooling", 0) == 0 || t.rfind("AveragePooling", 0) == 0) {
            const int in = single(ins);
            const TShape& s = shape(in);
            ensure(s.d[0] == 1, "pooling: dim5 must be 1");
            const Geom1 g4 = conv_geom((int)s.d[1], L.k[0], L.s[0], L.pad, false);
            const Geom1 gh = conv_geom((int)s.d[2], L.k[1], L.s[1], L.pad, false);
            const Geom1 gw = conv_geom((int)s.d[3], L.k[2], L.s[2], L.pad, false);
            TShape os = s;
            os.d[1] = g4.out; os.d[2] = gh.out; os.d[3] = gw.out;
            const int out = new_tensor(os);
            Op& o = push(OP_POOL, &L, {in}, {out});
            o.a[POOL_PF] = g4.pad_lo; o.a[POOL_PT] = gh.pad_lo; o.a[POOL_PL] = gw.pad_lo; o.a[POOL_MAX] = L.flag_a;
            return {out};
        }
        if (t.rfind("GlobalMaxPooling", 0) == 0 || t.rfind("GlobalAveragePooling", 0) == 0) {
            const int in = single(ins);
            const TShape& s = shape(in);
            ensure(s.d[0] == 1, "global pooling: dim5 must be 1");
            std::vector<int64_t> dims;
            if (L.flag_b) { dims.assign((size_t)s.rank - 1, 1); dims.push_back(s.d[4]); } else dims = {s.d[4]};
            const int out = new_tensor(TShape::from_dims(dims));
            Op& o = push(OP_GPOOL, &L, {in}, {out});
            o.a[0] = L.flag_a;
            return {out};
        }
        if (t == "Add" || t == "Multiply" || t == "Average") {
            ensure(!ins.empty(), "no tensors given");
            const int op = t == "Multiply" ? BINOP_MUL : BINOP_ADD;
            int acc = ins[0];
            for (size_t i = 1; i < ins.size(); ++i) acc = emit_binary(&L, op, acc, ins[i], 1.0f);
            if (t == "Average") {  // sum, then * (1 / n) (tensor.hpp:886-891)
                const int out = new_tensor(shape(acc));
                Op& o = push(OP_AFFINE, &L, {acc}, {out});
                o.a[AFF_OUTER] = shape(acc).volume(); o.a[AFF_NC] = 1; o.a[AFF_INNER] = 1;
                o.a[AFF_CONST] = 1;
                o.f[0] = 1.0f / (float)ins.size();
                return {out};
            }
            if (ins.size() == 1) return {acc};
            return {acc};
        }
        if (t == "Subtract") {
            ensure(ins.size() == 2, "invalid number of input tensors");
            return {emit_binary(&L, BINOP_SUB, ins[0], ins[1], 1.0f)};
        }
        if (t == "Maximum" || t == "Minimum") {
            ensure(!ins.empty(), "no tensors given");
            for (int i : ins) ensure(shape(i) == shape(ins[0]), "all tensors must have the same size");
            int acc = ins[0];
            for (size_t i = 1; i < ins.size(); ++i) acc = emit_binary(&L, t == "Maximum" ? BINOP_MAX : BINOP_MIN, acc, ins[i], 1.0f);
            return {acc};
        }
        if (t == "Concatenate") {
            ensure(!ins.empty(), "no tensors given");
            const int rank = shape(ins[0]).rank;
            int axis = L.axes[0];
            if (axis < 0) axis = axis + rank + 1;
            axis = std::min(5, axis - rank + 5);
            ensure(axis >= 1 && axis <= 5, "Invalid axis (" + std::to_string(axis) + ") for tensor concatenation.");
            const int ax = axis - 1;
            TShape os = shape(ins[0]);
            int64_t total = 0;
            for (int i : ins) {
                for (int k = 0; k < 5; ++k)
                    if (k != ax) ensure(shape(i).d[k] == os.d[k], "Tensor shapes differ on wrong dimension.");
                total += shape(i).d[ax];
            }
            os.d[ax] = total;
            const int out = new_tensor(os);
            Op& o = push(OP_CONCAT, &L, ins, {out});
            o.a[0] = ax;
            return {out};
        }
        if (t == "Flatten") {
            const int in = single(ins);
            return {view(in, TShape::from_dims({shape(in).volume()}))};
        }
        if (t == "Reshape") {  // reshape_layer.hpp:27-33; derive_fixed_tensor_shape
            const int in = single(ins);
            int64_t known = 1;
            for (int64_t d : L.target) if (d >= 0) known *= d;
            ensure(known > 0, "Invalid target shape");
            std::vector<int64_t> dims;
            for (int64_t d : L.target) dims.push_back(d >= 0 ? d : shape(in).volume() / known);
            const TShape os = TShape::from_dims(dims);
            ensure(os.volume() == shape(in).volume(), "invalid number of values");
            return {view(in, os)};
        }
        if (t == "Permute") {  // permute_tensor, tensor.hpp:526-549
            const int in = single(ins);
            const TShape& s = shape(in);
            ensure((int)L.target.size() == s.rank, "Invalid dims for permute_tensor.");
            std::vector<int64_t> dims;
            const auto id = s.dims();
            for (int64_t d : L.target) dims.push_back(id[(size_t)d - 1]);
            const int out = new_tensor(TShape::from_dims(dims));
            Op& o = push(OP_PERMUTE, &L, {in}, {out});
            const int lead = 5 - s.rank;
            for (int i = 0; i < 5; ++i) o.a[i] = i < lead ? i : lead + (int)L.target[(size_t)(i - lead)] - 1;
            return {out};
        }
        if (t.rfind("ZeroPadding", 0) == 0 || t.rfind("Cropping", 0) == 0) {
            const int in = single(ins);
            const TShape& s = shape(in);
            ensure(s.d[0] == 1, "padding/cropping: dim5 must be 1");
            TShape os = s;
            const int sign = L.flag_a ? 1 : -1;
            os.d[1] += sign * (L.pads[0] + L.pads[1]);
            os.d[2] += sign * (L.pads[2] + L.pads[3]);
            os.d[3] += sign * (L.pads[4] + L.pads[5]);
            ensure(os.d[1] > 0 && os.d[2] > 0 && os.d[3] > 0, "invalid cropping");
            const int out = new_tensor(os);
            Op& o = push(OP_WINDOW, &L, {in}, {out});
            o.a[0] = sign * L.pads[0]; o.a[1] = sign * L.pads[2]; o.a[2] = sign * L.pads[4];
            return {out};
        }
        if (t == "Embedding") {  // embedding_layer.hpp:31-57
            ensure(!ins.empty(), "invalid number of input tensors");
            const TShape& f = shape(ins[0]);
            ensure(f.d[0] == 1 && f.d[1] == 1 && f.d[2] == 1 && f.d[3] == 1,
                   "size_dim_5, size_dim_4, height and width dimension must be 1, but shape is '" + f.str() + "'");
            std::vector<int> outs;
            for (int in : ins) {
                const int out = new_tensor(TShape::from_dims({shape(in).d[4], L.units}));
                push(OP_EMBED, &L, {in}, {out});
                outs.push_back(out);
            }
            return outs;
        }
        if (t == "LSTM" || t == "GRU" || t == "SimpleRNN") return emit_recurrent(L, ins);
        if (t == "Bidirectional") {  // bidirectional_layer.hpp:53-111
            ensure(ins.size() == 1, "Invalid number of input tensors.");
            const TShape& s = shape(ins[0]);
            ensure(s.rank == 2, "input tensor must have rank 2, but shape is '" + s.str() + "'");
            // the backward direction reads the rows last to first and, with return_sequences, writes each state
            // at its own row, which is the reference's reverse -> run -> reverse without the two copies
            const int f = emit_recurrent(L.cells[0], ins)[0];
            const int b = emit_recurrent(L.cells[1], ins)[0];
            return emit_impl(L.cells[2], {f, b});
        }
        if (t == "RNN") {  // stacked_rnn_layer.hpp:21-45: every cell is a recurrent layer fed by the one before
            std::vector<int> cur = ins;
            for (const Layer& C : L.cells) cur = emit_recurrent(C, cur);
            return cur;
        }
        if (t == "MultiHeadAttention" || t == "GroupQueryAttention" || t == "GroupedQueryAttention") return {emit_mha(L, ins)};
        if (t == "Attention" || t == "AdditiveAttention") {  // attention_layer.hpp:30-52, additive_attention_layer.hpp:27-45
            ensure(ins.size() == 2 || ins.size() == 3, "Invalid number of inputs for Attention layer.");
            const TShape q = shape(ins[0]), v = shape(ins[1]), k = shape(ins.size() > 2 ? ins[2] : ins[1]);
            ensure(q.rank == 2 && v.rank == 2 && k.rank == 2 && q.d[4] == k.d[4] && v.d[3] == k.d[3], "Invalid shapes for Attention layer.");
            ensure(L.input_dim <= 1 || L.input_dim == q.d[4], "Invalid scale for AdditiveAttention layer.");
            const int out = new_tensor(TShape::from_dims({q.d[3], v.d[4]}));
            Op& o = push(OP_ATTN, &L, ins, {out});
            o.a[MHA_TQ] = q.d[3]; o.a[MHA_TK] = k.d[3];
            p.flops_per_sample += 2.0 * (double)q.d[3] * k.d[3] * (q.d[4] + v.d[4]);
            return {out};
        }
        if (t == "Conv3D" || t == "Conv3DTranspose") {  // convolution3d.hpp:437-506
            const int in = single(ins);
            const TShape sh = shape(in);
            ensure(sh.d[0] == 1, "3-D convolution input must have rank <= 4");
            ensure(sh.d[4] == L.in_feat, "invalid filter depth");
            const bool spread = L.flag_a && !(L.s[0] == 1 && L.s[1] == 1 && L.s[2] == 1);
            ensure(!spread || sh.rank == 4, "Invalid rank for 3d dilation");
            Op o;
            o.kind = OP_CONV3D;
            o.layer = &L;
            o.in = {in};
            TShape os = sh;
            int64_t rows = 1;
            for (int i = 0; i < 3; ++i) {
                const int n = (int)sh.d[1 + i];
                // transposed: the input is spread by the strides (with room for the output to fit under SAME,
                // convolution3d.hpp:144-181), then a stride-1 convolution
                const int extra = (spread && L.pad == PAD_SAME) ? L.s[i] - 1 : 0;
                const int ext = spread ? (n - 1) * L.s[i] + 1 + extra : n;
                const Geom1 g = conv_geom(ext, L.k[i], L.flag_a ? 1 : L.s[i], L.pad, L.flag_a);
                o.a[i] = n; o.a[3 + i] = g.out; o.a[6 + i] = L.flag_a ? 1 : L.s[i]; o.a[9 + i] = g.pad_lo; o.a[12 + i] = ext;
                o.a[15 + i] = extra - extra / 2; o.a[18 + i] = L.flag_a ? L.s[i] : 1;
                os.d[1 + i] = g.out;
                rows *= g.out;
            }
            os.d[4] = L.units;
            const int out = new_tensor(os);
            o.out = {out};
            o.a[21] = rows;
            o.w_main = L.w_main; o.ldw = L.ldw; o.K = L.kdim; o.N = L.units; o.w_bias = L.w_bias;
            // Implicit GEMM (Conv3D with 4 | channels on the tensor-core path): the operand tiles are fetched by TMA per
            // filter tap from the input slices; the transposed layer and other channel counts gather a patch matrix.
            const bool implicit3 = opt.use_tc && !L.flag_a && sh.d[4] % 4 == 0 && L.ldw == L.kdim && L.s[1] <= 8 && L.s[2] <= 8;
            // Transposed: one stride-1 implicit product per output phase (Layer::w_phases).  The output slices of a phase
            // must lie a fixed number of floats apart over all samples, which needs the output depth to be a multiple of
            // the depth stride (always so with SAME padding).
            const bool phases3 = opt.use_tc && L.flag_a && !L.w_phases.empty() && sh.d[4] % 4 == 0 && L.units % 4 == 0 && o.a[3] % L.s[0] == 0;
            o.a[22] = implicit3;
            o.a[23] = phases3;
            if (!implicit3 && !phases3) o.scratch.push_back(new_buffer(rows * L.ldw));
            p.flops_per_sample += 2.0 * (double)rows * L.kdim * L.units;
            p.ops.push_back(std::move(o));
            return {out};
        }
        if (t == "Rescaling") {
            std::vector<int> outs;
            for (int in : ins) outs.push_back(emit_activation(L.act, in, &L));
            return outs;
        }
        if (t == "Normalization") {  // normalization_layer.hpp:37-80
            const int in = single(ins);
            const TShape sh = shape(in);
            int pos = -1;  // statistics along this dimension; -1: one for the whole tensor
            if (!L.axes.empty()) {
                const int axis_dim = L.axes[0] == -1 ? 0 : sh.rank - L.axes[0];
                ensure(axis_dim >= 0 && axis_dim <= 4, "Invalid axis for Normalization layer");
                pos = 4 - axis_dim;
            }
            const int64_t n = pos < 0 ? 1 : sh.d[pos];
            ensure(L.units == n, "Invalid number of variance values in Normalization layer.");
            int64_t inner = 1;
            for (int i = pos + 1; i < 5 && pos >= 0; ++i) inner *= sh.d[i];
            if (pos < 0) inner = sh.volume();
            const int out = new_tensor(sh);
            Op& o = push(OP_NORMALIZE, &L, {in}, {out});
            o.a[0] = sh.volume() / (n * inner); o.a[1] = n; o.a[2] = inner;
            return {out};
        }
        if (t == "UpSampling1D" || t == "UpSampling2D") {  // upsampling_1d_layer.hpp:31-54, upsampling_2d_layer.hpp:33-48
            const int in = single(ins);
            const TShape sh = shape(in);
            ensure(sh.d[0] == 1 && sh.d[1] == 1, "upsampling input must have rank <= 3");
            if (t == "UpSampling1D") ensure(sh.rank == 2, "invalid input shape for Upsampling1D");
            const int out = new_tensor(t == "UpSampling1D" ? TShape::from_dims({sh.d[3] * L.k[2], sh.d[4]})
                                                           : TShape::from_dims({sh.d[2] * L.k[1], sh.d[3] * L.k[2], sh.d[4]}));
            Op& o = push(OP_UPSAMPLE, &L, {in}, {out});
            o.a[0] = sh.d[2]; o.a[1] = sh.d[3]; o.a[2] = sh.d[4]; o.a[3] = 1; o.a[4] = L.k[1]; o.a[5] = L.k[2];  // H, W, C, images per sample, factors
            return {out};
        }
        if (t == "TimeDistributed") {  // time_distributed_layer.hpp:33-91
            // the wrapped layer runs on every slice along the first axis; the results are stacked along a new first axis
            const int in = single(ins);
            const TShape sh = shape(in);
            const int tin = L.k[0], tout = L.k[1];
            ensure(tin >= 2 && tin <= 5, "invalid input dim for TimeDistributed");
            ensure(tout >= 2 && tout <= 5, "invalid output dim for TimeDistributed");
            ensure(tin <= 4 && sh.rank == tin, "TimeDistributed: the series must be the first axis of a tensor of rank 2 to 4");
            const int ax = 5 - tin;            // 2: width, 3: height, 4: dim4
            const int ax_out = 5 - tout;
            const int64_t len = sh.d[ax];
            std::vector<int64_t> slice_dims(sh.d + ax + 1, sh.d + 5);
            std::vector<int> results;
            for (int64_t i = 0; i < len; ++i) {
                TShape ss = sh;
                ss.d[ax] = 1;
                const int cut = new_tensor(ss);
                Op& o = push(OP_WINDOW, &L, {in}, {cut});
                o.a[ax - 1] = -i;
                const std::vector<int> r = emit_layer(L.cells[0], {view(cut, TShape::from_dims(slice_dims))});
                ensure(!r.empty(), "TimeDistributed: the wrapped layer gave no output");
                ensure(shape(r[0]).rank < tout && shape(r[0]).d[ax_out] == 1, "TimeDistributed: rank of the wrapped layer's output does not fit");
                results.push_back(r[0]);
            }
            TShape os = shape(results[0]);
            for (int r : results) ensure(shape(r).same_dims(os), "Tensor shapes differ on wrong dimension.");
            os.d[ax_out] = len;
            os.rank = tout;
            const int out = new_tensor(os);
            Op& o = push(OP_CONCAT, &L, results, {out});
            o.a[0] = ax_out;
            return {out};
        }
        if (t == "RepeatVector") {  // repeat_vector_layer.hpp:31-38: (D) -> (n, D), the vector n times
            const int in = single(ins);
            const TShape sh = shape(in);
            ensure(sh.rank == 1, "Invalid input shape for RepeatVector");
            const int out = new_tensor(TShape::from_dims({(int64_t)L.k[2], sh.d[4]}));
            Op& o = push(OP_UPSAMPLE, &L, {in}, {out});  // nearest upsampling of a width-1 row by n
            o.a[0] = 1; o.a[1] = 1; o.a[2] = sh.d[4]; o.a[3] = 1; o.a[4] = 1; o.a[5] = L.k[2];
            return {out};
        }
        if (t == "UpSampling3D") {  // upsampling_3d_layer.hpp:31-41 -> resize3d_nearest, tensor.hpp:976-995
            // the nearest source index is chosen per axis, so two passes of the 2-D kernel do it: height and width with
            // dim4 as part of the batch, then dim4 with everything behind it as the "depth"
            const int in = single(ins);
            const TShape sh = shape(in);
            ensure(sh.d[0] == 1, "upsampling input must have rank <= 4");
            const int mid = new_tensor(TShape::from_dims({sh.d[1], sh.d[2] * L.k[1], sh.d[3] * L.k[2], sh.d[4]}));
            Op& o1 = push(OP_UPSAMPLE, &L, {in}, {mid});
            o1.a[0] = sh.d[2]; o1.a[1] = sh.d[3]; o1.a[2] = sh.d[4]; o1.a[3] = sh.d[1]; o1.a[4] = L.k[1]; o1.a[5] = L.k[2];
            const int out = new_tensor(TShape::from_dims({sh.d[1] * L.k[0], sh.d[2] * L.k[1], sh.d[3] * L.k[2], sh.d[4]}));
            Op& o2 = push(OP_UPSAMPLE, &L, {mid}, {out});
            o2.a[0] = sh.d[1]; o2.a[1] = 1; o2.a[2] = sh.d[2] * L.k[1] * sh.d[3] * L.k[2] * sh.d[4]; o2.a[3] = 1; o2.a[4] = L.k[0]; o2.a[5] = 1;
            return {out};
        }
        if (t == "ConvLSTM1D" || t == "ConvLSTM2D") {  // conv_lstm_2d_layer.hpp:54-175
            // Per time step: the input convolution of that step's slice, the recurrent convolution of the previous hidden
            // state (skipped at the first step, where the state is zero and the recurrent bias is zero), and one gate kernel.
            const int in = single(ins);
            const TShape sh = shape(in);
            const int rank = L.bin_op;   // 1: (T, W, C); 2: (T, H, W, C)
            ensure(sh.rank == rank + 2, "ConvLSTM: invalid input rank");
            const int ax = rank == 1 ? 2 : 1;
            const int64_t T = sh.d[ax];
            ensure(T >= 1, "ConvLSTM needs at least one timestep");
            const int64_t U = L.units;
            int h_prev = -1, c_prev = -1;
            std::vector<int> hs;
            TShape hshape;
            for (int64_t step = 0; step < T; ++step) {
                TShape ss = sh;
                ss.d[ax] = 1;
                const int cut = new_tensor(ss);
                Op& w = push(OP_WINDOW, &L, {in}, {cut});
                w.a[ax - 1] = -step;
                // rank 1: the slice is a (1, W, C) image; rank 2: (H, W, C)
                const int slice = view(cut, TShape::from_dims({rank == 1 ? (int64_t)1 : sh.d[2], sh.d[3], sh.d[4]}));
                const int x_t = emit_layer(L.cells[0], {slice})[0];
                const TShape xs = shape(x_t);
                hshape = TShape::from_dims({xs.d[2], xs.d[3], U});
                int u_t = -1;
                if (h_prev >= 0) u_t = emit_layer(L.cells[1], {h_prev})[0];
                const int h_t = new_tensor(hshape), c_t = new_tensor(hshape);
                std::vector<int> cell_in = {x_t};
                if (u_t >= 0) { cell_in.push_back(u_t); cell_in.push_back(c_prev); }
                Op& o = push(OP_CONVLSTM_CELL, &L, cell_in, {h_t, c_t});
                o.a[0] = hshape.volume() / U;
                o.a[1] = U;
                h_prev = h_t;
                c_prev = c_t;
                if (L.flag_b) hs.push_back(view(h_t, rank == 1 ? TShape::from_dims({1, xs.d[3], U}) : TShape::from_dims({1, xs.d[2], xs.d[3], U})));
            }
            const TShape state_shape = rank == 1 ? TShape::from_dims({hshape.d[3], U}) : hshape;
            std::vector<int> result;
            if (L.flag_b) {
                TShape os = shape(hs[0]);
                os.d[5 - os.rank] = T;
                const int out = new_tensor(os);
                Op& o = push(OP_CONCAT, &L, hs, {out});
                o.a[0] = 5 - os.rank;
                result.push_back(out);
            } else {
                result.push_back(view(h_prev, state_shape));
            }
            if (L.flag_c) {
                result.push_back(view(h_prev, state_shape));
                result.push_back(view(c_prev, state_shape));
            }
            return result;
        }
        if (t == "Resizing") {  // resizing_layer.hpp:33-42; resize_tensor_2d / smart_resize_tensor_2d, tensor.hpp:1113-1163
            const int in = single(ins);
            return {emit_resize(L, in, L.k[1], L.k[2], L.bin_op, L.flag_a)};
        }
        if (t == "Dot") {  // dot_layer.hpp:32-38; dot_product_tensors, tensor.hpp:814-884
            ensure(ins.size() == 2, "need exactly 2 input tensors");
            const TShape sa = shape(ins[0]), sb = shape(ins[1]);
            const int ax_a = L.axes[0], ax_b = L.axes[1];
            ensure(ax_a >= 1 && ax_a <= sa.rank && ax_b >= 1 && ax_b <= sb.rank, "Dot: axes must be positive and within the inputs' ranks");
            const int pa = 5 - sa.rank + ax_a - 1, pb = 5 - sb.rank + ax_b - 1;
            ensure(sa.d[pa] == sb.d[pb], "Dot: the contracted dimensions differ");
            std::vector<int64_t> dims;
            int64_t a_outer = 1, a_inner = 1, b_outer = 1, b_inner = 1;
            for (int i = 5 - sa.rank; i < 5; ++i) if (i != pa) { dims.push_back(sa.d[i]); (i < pa ? a_outer : a_inner) *= sa.d[i]; }
            for (int i = 5 - sb.rank; i < 5; ++i) if (i != pb) { dims.push_back(sb.d[i]); (i < pb ? b_outer : b_inner) *= sb.d[i]; }
            if (dims.empty()) dims.push_back(1);
            ensure(dims.size() <= 5, "Invalid tensor-shape dimensions");
            const int out = new_tensor(TShape::from_dims(dims));
            Op& o = push(OP_DOT, &L, {ins[0], ins[1]}, {out});
            o.a[0] = a_outer; o.a[1] = a_inner; o.a[2] = b_outer; o.a[3] = b_inner; o.a[4] = sa.d[pa]; o.a[5] = L.flag_a;
            p.flops_per_sample += 2.0 * (double)a_outer * a_inner * b_outer * b_inner * sa.d[pa];
            return {out};
        }
        if (t == "AdaptivePooling") {  // adaptive_pooling_3d_layer.hpp:40-113
            const int in = single(ins);
            const TShape sh = shape(in);
            ensure(sh.d[0] == 1, "AdaptivePooling: dim5 must be 1");
            const int64_t od = L.k[0] == 0 ? sh.d[1] : L.k[0], oh = L.k[1] == 0 ? sh.d[2] : L.k[1], ow = L.k[2];
            ensure(ow > 0, "AdaptivePooling output_size must be > 0.");
            const TShape os = sh.rank == 2 ? TShape::from_dims({ow, sh.d[4]})
                              : sh.rank == 3 ? TShape::from_dims({oh, ow, sh.d[4]}) : TShape::from_dims({od, oh, ow, sh.d[4]});
            const int out = new_tensor(os);
            Op& o = push(OP_ADAPTIVE_POOL, &L, {in}, {out});
            // the loop bounds of the reference are the layer's sizes even where the output shape has fewer dimensions:
            // rank-2 / rank-3 inputs have height / dim4 of 1, for which every range is [0, 1)
            o.a[0] = sh.d[1]; o.a[1] = sh.d[2]; o.a[2] = sh.d[3]; o.a[3] = sh.d[4];
            o.a[4] = os.d[1]; o.a[5] = os.d[2]; o.a[6] = os.d[3]; o.a[7] = L.flag_a;
            return {out};
        }
        if (t == "Discretization" || t == "IntegerLookup") {  // discretization_layer.hpp:31-42, integer_lookup_layer.hpp:57-80
            const int in = single(ins);
            const int out = new_tensor(shape(in));
            Op& o = push(OP_LOOKUP, &L, {in}, {out});
            o.a[0] = t == "Discretization" ? 0 : 1;
            o.a[1] = L.units;
            o.a[2] = shape(in).volume();
            o.a[3] = L.flag_a;
            return {out};
        }
        if (t == "CategoryEncoding") {  // category_encoding_layer.hpp:34-62
            const int in = single(ins);
            const TShape sh = shape(in);
            ensure(sh.rank == 1, "Tensor of rank 1 required, but shape is '" + sh.str() + "'");
            if (L.bin_op == 0) ensure(sh.d[4] == 1, "Tensor of depth 1 required, but is: " + std::to_string(sh.d[4]));
            const int out = new_tensor(TShape::from_dims({L.units}));
            Op& o = push(OP_LOOKUP, &L, {in}, {out});
            o.a[0] = 2 + L.bin_op;   // 2 one_hot, 3 multi_hot, 4 count
            o.a[1] = L.units;
            o.a[2] = sh.d[4];
            return {out};
        }
        if (t == "CenterCrop") {  // centercrop_layer.hpp:31-45
            const int in = single(ins);
            const TShape& sh = shape(in);
            // smaller inputs are resized first in the reference (smart_resize_tensor_2d, bilinear, centercrop_layer.hpp:36-40)
            if (sh.d[2] < L.k[1] || sh.d[3] < L.k[2]) return {emit_resize(L, in, L.k[1], L.k[2], 1, true)};
            TShape os = sh;
            os.d[2] = L.k[1];
            os.d[3] = L.k[2];
            const int out = new_tensor(os);
            Op& o = push(OP_WINDOW, &L, {in}, {out});
            o.a[0] = 0; o.a[1] = -(int64_t)((sh.d[2] - L.k[1]) / 2); o.a[2] = -(int64_t)((sh.d[3] - L.k[2]) / 2);
            return {out};
        }
        if (t == "EinsumDense") {  // einsum_dense_layer.hpp:120-258
            const int in = single(ins);
            const TShape sh = shape(in);
            std::map<char, int64_t> size;
            for (size_t i = 0; i < L.eq_kernel.size(); ++i) size[L.eq_kernel[i]] = L.kernel_dims[L.kernel_dims.size() - L.eq_kernel.size() + i];
            ensure((int)L.eq_in.size() >= sh.rank, "EinsumDense: input rank exceeds lhs char count.");
            const size_t lead = L.eq_in.size() - (size_t)sh.rank;
            for (size_t i = 0; i < L.eq_in.size(); ++i) {  // letters beyond the input's rank are the batch axis, size 1
                const int64_t sz = i >= lead ? sh.d[5 - sh.rank + (int)(i - lead)] : 1;
                if (size.count(L.eq_in[i])) ensure(size[L.eq_in[i]] == sz, "EinsumDense: inconsistent char size in equation.");
                else size[L.eq_in[i]] = sz;
            }
            for (size_t i = 0; i < L.eq_out.size(); ++i)
                if (!size.count(L.eq_out[i])) {
                    ensure(i < L.target.size() && L.target[i] > 0, "EinsumDense: cannot infer size of output-only char.");
                    size[L.eq_out[i]] = L.target[i];
                }
            std::string summed;
            for (char ch : L.eq_in)
                if (L.eq_out.find(ch) == std::string::npos) {
                    ensure(L.eq_kernel.find(ch) != std::string::npos, "EinsumDense: an input letter is neither kept nor summed");
                    summed.push_back(ch);
                }
            for (char ch : L.eq_kernel) ensure(L.eq_out.find(ch) != std::string::npos || summed.find(ch) != std::string::npos, "EinsumDense: a kernel letter is neither kept nor summed");
            std::vector<int64_t> od;
            int64_t out_volume = 1, sum_volume = 1;
            for (size_t i = 1; i < L.eq_out.size(); ++i) od.push_back(size[L.eq_out[i]]);
            ensure(od.size() <= 5, "EinsumDense: output rank above 5");
            for (char ch : L.eq_out) out_volume *= size[ch];
            for (char ch : summed) sum_volume *= size[ch];
            const int out = new_tensor(TShape::from_dims(od));
            p.flops_per_sample += 2.0 * (double)out_volume * sum_volume;
            if (L.flag_a) {  // matrix-product form
                Op& o = push(OP_GEMM, &L, {in}, {out});
                o.a[GEMM_ROWS] = out_volume / L.units;
                o.w_main = L.w_main; o.ldw = L.ldw; o.K = L.kdim; o.N = L.units;
                o.w_bias = L.w_bias;
                return {out};
            }
            auto stride_in = [&](const std::string& letters, char ch) -> int64_t {
                const size_t pos = letters.find(ch);
                if (pos == std::string::npos) return 0;
                int64_t st = 1;
                for (size_t i = letters.size() - 1; i > pos; --i) st *= size[letters[i]];
                return st;
            };
            int64_t bias_volume = 1;
            for (char ch : L.eq_bias) bias_volume *= size[ch];
            ensure(L.eq_bias.empty() || bias_volume == L.input_dim, "EinsumDense: bias size does not match bias_axes");
            Op& o = push(OP_EINSUM, &L, {in}, {out});
            o.a[0] = (int64_t)L.eq_out.size(); o.a[1] = (int64_t)summed.size(); o.a[2] = sh.volume(); o.a[3] = out_volume; o.a[4] = sum_volume;
            for (char ch : L.eq_out) for (int64_t v : {size[ch], stride_in(L.eq_in, ch), stride_in(L.eq_kernel, ch), stride_in(L.eq_bias, ch)}) o.ext.push_back(v);
            for (char ch : summed) for (int64_t v : {size[ch], stride_in(L.eq_in, ch), stride_in(L.eq_kernel, ch)}) o.ext.push_back(v);
            return {out};
        }
        if (t == "PReLU") {  // prelu_layer.hpp:30-68
            const int in = single(ins);
            const TShape sh = shape(in);
            ensure(sh.d[0] == 1 && sh.d[1] == 1, "PReLU on tensors with more than three axes is not supported by the device engine");
            bool hs = false, ws = false, cs = false;
            int shift = 0;
            for (int a : L.axes) {  // Keras axes move when the tensor had fewer than three axes (prelu_layer.hpp:37-47)
                if ((a == 1 && sh.d[2] == 1) || (a == 2 && sh.d[3] == 1)) shift++;
                const int v = a + shift;
                hs = hs || v == 1; ws = ws || v == 2; cs = cs || v == 3;
            }
            const int64_t need = (hs ? 1 : sh.d[2]) * (ws ? 1 : sh.d[3]) * (cs ? 1 : sh.d[4]);
            ensure(L.input_dim >= need, "invalid PReLU alpha size");
            const int out = new_tensor(sh);
            Op& o = push(OP_PRELU, &L, {in}, {out});
            o.a[0] = hs; o.a[1] = ws; o.a[2] = cs;
            return {out};
        }
        if (t == "Activation") return {emit_activation(L.act, single(ins), &L)};
        raise("unknown layer type: " + t);
    }

    int emit_binary(const Layer* L, int op, int a, int b, float post) {
        const TShape &sa = shape(a), &sb = shape(b);
        TShape os;
        for (int i = 0; i < 5; ++i) {
            ensure(std::min(sa.d[i], sb.d[i]) == 1 || sa.d[i] == sb.d[i], "Invalid shapes for combining tensors.");
            os.d[i] = std::max(sa.d[i], sb.d[i]);
        }
        os.rank = std::max(os.minimal_rank(), std::max(sa.rank, sb.rank));  // tensor.hpp:658
        const int out = new_tensor(os);
        Op& o = push(OP_BINARY, L, {a, b}, {out});
        o.a[0] = op;
        o.f[0] = post;
        return out;
    }

    int emit_conv(const Layer& L, int in) {
        const TShape& s = shape(in);
        ensure(s.d[0] == 1 && s.d[1] == 1, "convolution input must have rank <= 3");
        ensure(s.d[4] == L.in_feat, "invalid filter depth");
        const int H = (int)s.d[2], W = (int)s.d[3], C = (int)s.d[4];
        Op o;
        o.kind = OP_CONV;
        o.layer = &L;
        o.in = {in};
        int Ho, Wo;
        if (!L.flag_a) {
            const int ekh = (L.k[1] - 1) * L.dil[1] + 1, ekw = (L.k[2] - 1) * L.dil[2] + 1;
            const Geom1 gh = conv_geom(H, ekh, L.s[1], L.pad, false), gw = conv_geom(W, ekw, L.s[2], L.pad, false);
            Ho = gh.out; Wo = gw.out;
            // the reference asserts the padded input fits the strided window walk (convolution.hpp:251)
            o.a[CONV_PT] = gh.pad_lo; o.a[CONV_PL] = gw.pad_lo;
            o.a[CONV_SY] = L.s[1]; o.a[CONV_SX] = L.s[2]; o.a[CONV_DY] = L.dil[1]; o.a[CONV_DX] = L.dil[2];
        } else {
            // convolve_transposed (convolution.hpp:443-469): dilate the input by the strides, pad, stride-1 conv
            const int sy = L.s[1], sx = L.s[2];
            const bool fits = L.pad == PAD_SAME;
            const int ey = (fits && sy > 1) ? sy - 1 : 0, ex = (fits && sx > 1) ? sx - 1 : 0;
            const int Hd = (sy == 1 && sx == 1) ? H : (H - 1) * sy + 1 + ey;
            const int Wd = (sy == 1 && sx == 1) ? W : (W - 1) * sx + 1 + ex;
            const Geom1 gh = conv_geom(Hd, L.k[1], 1, L.pad, true), gw = conv_geom(Wd, L.k[2], 1, L.pad, true);
            Ho = gh.out; Wo = gw.out;
            o.a[CONV_PT] = gh.pad_lo; o.a[CONV_PL] = gw.pad_lo;
            o.a[CONV_SY] = sy; o.a[CONV_SX] = sx; o.a[CONV_DY] = 1; o.a[CONV_DX] = 1;
            o.a[CONV_OFFY] = ey - ey / 2; o.a[CONV_OFFX] = ex - ex / 2; o.a[CONV_HD] = Hd; o.a[CONV_WD] = Wd;
            o.a[CONV_TRANSPOSED] = 1;
        }
        o.a[CONV_H] = H; o.a[CONV_W] = W; o.a[CONV_C] = C; o.a[CONV_HO] = Ho; o.a[CONV_WO] = Wo;
        o.a[CONV_KH] = L.k[1]; o.a[CONV_KW] = L.k[2];
        o.w_main = L.w_main; o.ldw = L.ldw; o.K = L.kdim; o.N = L.units; o.w_bias = L.w_bias;
        TShape os = s;
        os.d[2] = Ho; os.d[3] = Wo; os.d[4] = L.units;
        const int out = new_tensor(os);
        o.out = {out};
        const bool direct = !L.flag_a && L.k[1] == 1 && L.k[2] == 1 && L.s[1] == 1 && L.s[2] == 1 && o.a[CONV_PT] == 0 && o.a[CONV_PL] == 0 &&
                            Ho == H && Wo == W && L.ldw == C;
        o.a[CONV_DIRECT] = direct;
        // Implicit GEMM on the tensor-core path: TMA fetches the operand tiles per filter tap straight from the
        // NHWC input (needs 16-byte aligned pixels, i.e. C % 4 == 0, and strides within the tensor map's range);
        // everything else gathers an im2col matrix into a scratch buffer first.
        // Few input channels: the row-window form (one k block per filter row) over a zero-padded copy of the
        // input with the channels padded to a multiple of 4.
        const bool rowwin = opt.use_tc && !direct && L.w_aux >= 0 && L.s[1] <= 8;
        const bool implicit = opt.use_tc && !direct && !rowwin && !L.flag_a && C % 4 == 0 && L.s[1] <= 8 && L.s[2] <= 8 && L.ldw == L.kdim;
        const bool phases = opt.use_tc && L.flag_a && !L.w_phases.empty() && C % 4 == 0 && L.units % 4 == 0;
        o.a[CONV_IMPLICIT] = implicit;
        o.a[CONV_ROWWIN] = rowwin;
        o.a[CONV_PHASES] = phases;
        if (rowwin) {
            const int cp = (C + 3) / 4 * 4;
            const int hp = (Ho - 1) * L.s[1] + L.k[1];
            const int wp = std::max((Wo - 1) * L.s[2] + L.k[2], ((Wo - 1) * L.s[2] * cp + 32 + cp - 1) / cp);
            o.a[CONV_RW_HP] = hp; o.a[CONV_RW_WP] = wp; o.a[CONV_RW_CP] = cp;
            o.scratch.push_back(new_buffer((int64_t)hp * wp * cp));
        } else if (!direct && !implicit && !phases) {
            o.scratch.push_back(new_buffer((int64_t)Ho * Wo * L.ldw));
        }
        p.flops_per_sample += 2.0 * (double)Ho * Wo * L.kdim * L.units;
        p.ops.push_back(std::move(o));
        return out;
    }

    int emit_dwconv(const Layer& L, int in, bool with_bias) {
        const TShape& s = shape(in);
        ensure(s.d[0] == 1 && s.d[1] == 1, "convolution input must have rank <= 3");
        ensure(s.d[4] == L.in_feat, "invalid filter count");
        const int H = (int)s.d[2], W = (int)s.d[3];
        // the reference's depthwise path ignores dilation_rate (depthwise_convolution.hpp:74-99)
        const Geom1 gh = conv_geom(H, L.k[1], L.s[1], L.pad, false), gw = conv_geom(W, L.k[2], L.s[2], L.pad, false);
        TShape os = s;
        os.d[2] = gh.out; os.d[3] = gw.out;
        const int out = new_tensor(os);
        Op& o = push(OP_DWCONV, &L, {in}, {out});
        o.a[CONV_H] = H; o.a[CONV_W] = W; o.a[CONV_C] = s.d[4]; o.a[CONV_HO] = gh.out; o.a[CONV_WO] = gw.out;
        o.a[CONV_KH] = L.k[1]; o.a[CONV_KW] = L.k[2]; o.a[CONV_SY] = L.s[1]; o.a[CONV_SX] = L.s[2];
        o.a[CONV_PT] = gh.pad_lo; o.a[CONV_PL] = gw.pad_lo;
        o.w_main = L.w_aux;
        o.w_bias = with_bias ? L.w_bias : -1;
        p.flops_per_sample += 2.0 * (double)gh.out * gw.out * s.d[4] * L.k[1] * L.k[2];
        return out;
    }

    std::vector<int> emit_recurrent(const Layer& L, const std::vector<int>& ins) {
        ensure(ins.size() == 1, "Invalid number of input tensors.");
        const TShape& s = shape(ins[0]);
        ensure(s.d[0] == 1 && s.d[1] == 1 && s.d[2] == 1, "size_dim_5, size_dim_4 and height dimension must be 1, but shape is '" + s.str() + "'");
        ensure(s.d[4] == L.in_feat, "invalid recurrent input features");
        const int64_t T = s.d[3], U = L.units;
        const int g = L.cls == "LSTM" ? 4 : L.cls == "GRU" ? 3 : 1;
        std::vector<int> outs;
        outs.push_back(new_tensor(L.flag_a ? TShape::from_dims({T, U}) : TShape::from_dims({U})));
        if (L.flag_b) {
            outs.push_back(new_tensor(TShape::from_dims({U})));
            if (L.cls == "LSTM") outs.push_back(new_tensor(TShape::from_dims({U})));
        }
        Op& o = push(L.cls == "LSTM" ? OP_LSTM : L.cls == "GRU" ? OP_GRU : OP_RNN, &L, ins, outs);
        o.a[RNN_T] = T; o.a[RNN_F] = s.d[4]; o.a[RNN_U] = U;
        o.scratch.push_back(new_buffer(T * g * U));  // X = in W + b
        o.scratch.push_back(new_buffer(g * U));      // per-step gate pre-activations
        o.scratch.push_back(new_buffer(U));          // h
        o.scratch.push_back(new_buffer(U));          // c (LSTM) / h double buffer (SimpleRNN)
        p.flops_per_sample += 2.0 * (double)T * g * U * (s.d[4] + U);
        return outs;
    }

    int emit_mha(const Layer& L, const std::vector<int>& ins) {
        ensure(ins.size() == 2 || ins.size() == 3, "Invalid number of inputs for MultiHeadAttention layer.");
        const TShape &q = shape(ins[0]), &v = shape(ins[1]), &k = shape(ins.size() > 2 ? ins[2] : ins[1]);
        ensure(q.rank == 2 && v.rank == 2 && k.rank == 2 && q.d[4] == v.d[4] && q.d[4] == k.d[4] && v.d[3] == k.d[3],
               "Invalid shapes; need a query tensor of shape (B, T, dim) and a value/key tensor of shape (B, S, dim).");
        ensure(q.d[4] == L.in_feat, "Invalid input value count.");
        const int64_t Tq = q.d[3], Tk = k.d[3];
        const int kvh = L.kv_heads ? L.kv_heads : L.heads;
        const int out = new_tensor(TShape::from_dims({Tq, L.out_dim}));
        Op& o = push(OP_MHA, &L, ins, {out});
        o.a[MHA_TQ] = Tq; o.a[MHA_TK] = Tk;
        o.scratch.push_back(new_buffer(Tq * L.heads * L.key_dim));
        o.scratch.push_back(new_buffer(Tk * kvh * L.key_dim));
        o.scratch.push_back(new_buffer(Tk * kvh * L.value_dim));
        o.scratch.push_back(new_buffer(Tq * L.heads * L.value_dim));
        if (L.w_g >= 0) o.scratch.push_back(new_buffer(Tq * L.heads * L.value_dim));  // gate pre-activations
        p.flops_per_sample += 2.0 * ((double)Tq * L.in_feat * L.heads * L.key_dim + (double)Tk * L.in_feat * kvh * (L.key_dim + L.value_dim) +
                                     (double)Tq * Tk * L.heads * (L.key_dim + L.value_dim) + (double)Tq * L.heads * L.value_dim * L.out_dim +
                                     (L.w_g >= 0 ? (double)Tq * L.in_feat * L.heads * L.value_dim : 0.0));
        return out;
    }

    // ---- fusion: fold following BN / activation / Add into a contraction's epilogue ---------------------
    void fuse() {
        const size_t nt = p.tensors.size();
        // buffer-level use counts (views share buffers)
        auto recount = [&](std::vector<int>& uses) {
            uses.assign(p.buffers.size(), 0);
            for (const Op& o : p.ops) {
                if (o.dead) continue;
                for (int t : o.in) uses[(size_t)p.tensors[(size_t)t].buf]++;
                if (o.residual >= 0) uses[(size_t)p.tensors[(size_t)o.residual].buf]++;
            }
            for (int t : p.outputs) uses[(size_t)p.tensors[(size_t)t].buf] += 1000;  // model outputs are never folded away
        };
        (void)nt;
        std::vector<int> uses;
        // ZeroPadding -> pooling: the pooling kernel reads the zero frame itself (pool geometry was inferred
        // on the padded shape already), which saves writing and re-reading the padded tensor
        recount(uses);
        for (size_t i = 0; i < p.ops.size(); ++i) {
            Op& P = p.ops[i];
            if (P.dead || P.kind != OP_WINDOW || !P.layer->flag_a) continue;
            const int buf = p.tensors[(size_t)P.out[0]].buf;
            if (uses[(size_t)buf] != 1) continue;
            for (size_t j = i + 1; j < p.ops.size(); ++j) {
                Op& C = p.ops[j];
                if (C.dead || C.in.empty() || C.in[0] != P.out[0]) continue;
                if (C.kind == OP_POOL && !C.a[POOL_FRAMED]) {
                    C.in[0] = P.in[0];
                    C.a[POOL_FRAMED] = 1;
                    for (int k = 0; k < 6; ++k) C.a[POOL_ZF + k] = P.layer->pads[k];
                    P.dead = true;
                } else if ((C.kind == OP_DWCONV || (C.kind == OP_CONV && !C.a[CONV_DIRECT] && !C.a[CONV_TRANSPOSED])) &&
                           P.layer->pads[0] == 0 && P.layer->pads[1] == 0) {
                    // convolutions bounds-check (or let TMA zero-fill) around the unpadded input instead
                    const TShape& us = shape(P.in[0]);
                    C.in[0] = P.in[0];
                    C.a[CONV_H] = us.d[2];
                    C.a[CONV_W] = us.d[3];
                    C.a[CONV_PT] += P.layer->pads[2];
                    C.a[CONV_PL] += P.layer->pads[4];
                    P.dead = true;
                }
                break;
            }
        }
        bool changed = true;
        while (changed) {
            changed = false;
            recount(uses);
            for (size_t i = 0; i < p.ops.size() && !changed; ++i) {
                Op& P = p.ops[i];
                // an attention operation ends in its output projection, which can take a following Add as residual (only that)
                const bool mha = P.kind == OP_MHA;
                if (P.dead || !(P.kind == OP_CONV || P.kind == OP_GEMM || P.kind == OP_DWCONV || mha)) continue;
                const int t = P.out[0];
                const int buf = p.tensors[(size_t)t].buf;
                if (uses[(size_t)buf] != 1) continue;
                // the single consumer
                size_t j = i + 1;
                for (; j < p.ops.size(); ++j) {
                    const Op& C = p.ops[j];
                    if (C.dead) continue;
                    bool reads = false;
                    for (int x : C.in) if (p.tensors[(size_t)x].buf == buf) reads = true;
                    if (C.residual >= 0 && p.tensors[(size_t)C.residual].buf == buf) reads = true;
                    if (reads) break;
                }
                if (j >= p.ops.size()) continue;
                Op& C = p.ops[j];
                // the consumer must see the tensor with the producer's own shape (no reshape in between)
                if (mha && C.kind != OP_BINARY) continue;
                if (C.kind == OP_UNARY && C.in[0] == t) {
                    if (P.stage < 1) { P.act1 = C.act; P.stage = 1; }
                    else if (P.stage < 4) { P.act2 = C.act; P.stage = 4; }
                    else continue;
                } else if (C.kind == OP_AFFINE && C.in[0] == t && !C.a[AFF_CONST] && C.a[AFF_INNER] == 1 && P.stage < 2 &&
                           C.a[AFF_NC] == shape(t).d[4]) {
                    P.w_scale = C.w_scale; P.w_shift = C.w_shift; P.stage = 2;
                } else if (C.kind == OP_BINARY && C.a[0] == BINOP_ADD && C.f[0] == 1.0f && P.stage < 3 && (C.in[0] == t || C.in[1] == t) &&
                           C.in[0] != C.in[1]) {
                    const int other = C.in[0] == t ? C.in[1] : C.in[0];
                    if (!(shape(other).same_dims(shape(t)) && shape(C.out[0]).same_dims(shape(t)))) continue;
                    P.residual = other; P.stage = 3;
                } else continue;
                // move the producer to the consumer's slot and take over its output
                Op fused = P;
                fused.out = C.out;
                P.dead = true;
                p.ops[j] = fused;
                changed = true;
            }
        }
        std::vector<Op> live;
        for (Op& o : p.ops) if (!o.dead) live.push_back(std::move(o));
        p.ops.swap(live);
    }

    // ---- liveness and arena offsets -------------------------------------------------------------------------
    void allocate() {
        auto touch = [&](int buf, int idx) {
            BufferInfo& b = p.buffers[(size_t)buf];
            if (b.first < 0) b.first = idx;
            b.last = std::max(b.last, idx);
        };
        for (size_t i = 0; i < p.inputs.size(); ++i) p.buffers[(size_t)p.tensors[(size_t)p.inputs[i]].buf].ext_input = (int)i;
        const int n_ops = (int)p.ops.size();
        for (int i = 0; i < n_ops; ++i) {
            const Op& o = p.ops[(size_t)i];
            for (int t : o.in) touch(p.tensors[(size_t)t].buf, i);
            for (int t : o.out) touch(p.tensors[(size_t)t].buf, i);
            if (o.residual >= 0) touch(p.tensors[(size_t)o.residual].buf, i);
            for (int b : o.scratch) touch(b, i);
        }
        for (int t : p.outputs) {
            BufferInfo& b = p.buffers[(size_t)p.tensors[(size_t)t].buf];
            if (b.first < 0) b.first = 0;
            b.last = n_ops;
            b.pinned_to_end = true;
        }
        // greedy first-fit over a free list, in order of first use
        std::vector<int> order;
        for (size_t b = 0; b < p.buffers.size(); ++b)
            if (p.buffers[b].first >= 0 && p.buffers[b].ext_input < 0) order.push_back((int)b);
        std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return p.buffers[(size_t)x].first < p.buffers[(size_t)y].first; });
        struct Block { int64_t off, size; };
        std::vector<Block> free_list;
        std::vector<std::pair<int, int>> active;  // (last, buf)
        int64_t top = 0;
        auto release = [&](int buf) {
            const BufferInfo& b = p.buffers[(size_t)buf];
            Block blk{b.offset, round_up(std::max<int64_t>(b.elems, 1), 64)};
            free_list.push_back(blk);
            std::sort(free_list.begin(), free_list.end(), [](const Block& x, const Block& y) { return x.off < y.off; });
            std::vector<Block> merged;
            for (const Block& f : free_list) {
                if (!merged.empty() && merged.back().off + merged.back().size == f.off) merged.back().size += f.size;
                else merged.push_back(f);
            }
            if (!merged.empty() && merged.back().off + merged.back().size == top) { top = merged.back().off; merged.pop_back(); }
            free_list.swap(merged);
        };
        for (int buf : order) {
            BufferInfo& b = p.buffers[(size_t)buf];
            for (size_t k = 0; k < active.size();) {
                if (active[k].first < b.first) { release(active[k].second); active.erase(active.begin() + (long)k); }
                else ++k;
            }
            const int64_t need = round_up(std::max<int64_t>(b.elems, 1), 64);
            int best = -1;
            for (size_t k = 0; k < free_list.size(); ++k)
                if (free_list[k].size >= need && (best < 0 || free_list[k].size < free_list[(size_t)best].size)) best = (int)k;
            if (best >= 0) {
                b.offset = free_list[(size_t)best].off;
                free_list[(size_t)best].off += need;
                free_list[(size_t)best].size -= need;
                if (free_list[(size_t)best].size == 0) free_list.erase(free_list.begin() + best);
            } else {
                b.offset = top;
                top += need;
            }
            p.arena_elems = std::max(p.arena_elems, top);
            active.emplace_back(b.last, buf);
        }
    }
};

}  // namespace

std::shared_ptr<Plan> compile_plan(const LoadedModel& lm, const EngineOptions& opt, const std::vector<TShape>& in_shapes) {
    auto plan = std::make_shared<Plan>();
    Compiler c{lm, opt, *plan};
    plan->in_shapes = in_shapes;
    // model.hpp:132-139: the input shapes must match the model's (variable) input shapes
    ensure(in_shapes.size() == lm.input_shapes.size(), "Invalid number of input tensors for this model: " +
                                                           std::to_string(lm.input_shapes.size()) + " required but " +
                                                           std::to_string(in_shapes.size()) + " provided");
    for (size_t i = 0; i < in_shapes.size(); ++i) {
        if (!lm.input_shapes[i].matches(in_shapes[i])) {
            std::string have, want;
            for (size_t k = 0; k < in_shapes.size(); ++k) { have += in_shapes[k].str(); want += lm.input_shapes[k].str(); }
            raise("Invalid inputs shape. The model takes " + want + " but you provided: " + have);
        }
        plan->inputs.push_back(c.new_tensor(in_shapes[i]));
    }
    plan->outputs = c.emit_model(*lm.root, plan->inputs);
    for (size_t i = 0; i < plan->outputs.size() && i < lm.output_shapes.size(); ++i)
        if (!lm.output_shapes[i].matches(plan->tensors[(size_t)plan->outputs[i]].shape))
            raise("Invalid outputs shape. The model should return " + lm.output_shapes[i].str() + " but actually returned: " +
                  plan->tensors[(size_t)plan->outputs[i]].shape.str());
    c.fuse();
    c.allocate();
    return plan;
}

std::string describe_plan(const Plan& p) {
    static const char* names[] = {"conv", "gemm", "dwconv", "pool", "gpool", "binary", "unary", "affine", "softmax", "norm",
                                  "window", "concat", "permute", "embed", "lstm", "gru", "rnn", "mha", "copy", "attn", "prelu", "einsum", "conv3d", "normalize", "upsample",
                                  "resize", "dot", "adaptive_pool", "lookup", "convlstm_cell"};
    static_assert(sizeof(names) / sizeof(names[0]) == (size_t)OP_CONVLSTM_CELL + 1, "one name per op kind");
    std::string r;
    r += "arena_elems_per_sample=" + std::to_string(p.arena_elems) + " flops_per_sample=" + std::to_string((long long)p.flops_per_sample) + "\n";
    for (size_t i = 0; i < p.outputs.size(); ++i) r += "output " + std::to_string(i) + " " + p.tensors[(size_t)p.outputs[i]].shape.str() + "\n";
    for (const Op& o : p.ops) {
        r += std::string(names[o.kind]) + " " + (o.layer ? o.layer->name : std::string("?"));
        r += " out=" + p.tensors[(size_t)o.out[0]].shape.str();
        if (o.kind == OP_CONV || o.kind == OP_GEMM || o.kind == OP_DWCONV) {
            r += " epi=";
            if (o.w_bias >= 0) r += "bias,";
            if (!o.act1.none()) r += "act" + std::to_string(o.act1.kind) + ",";
            if (o.w_scale >= 0) r += "affine,";
            if (o.residual >= 0) r += "residual,";
            if (!o.act2.none()) r += "act" + std::to_string(o.act2.kind) + ",";
            if (o.kind == OP_CONV) r += o.a[CONV_DIRECT] ? " direct" : (o.a[CONV_ROWWIN] ? " rowwin" : (o.a[CONV_IMPLICIT] ? " implicit" : (o.a[CONV_PHASES] ? " phases" : " im2col")));
        }
        if (o.kind == OP_CONV3D) r += o.a[22] ? " implicit" : (o.a[23] ? " phases" : " im2col");
        const BufferInfo& b = p.buffers[(size_t)p.tensors[(size_t)o.out[0]].buf];
        r += " off=" + std::to_string(b.offset) + " elems=" + std::to_string(b.elems) + "\n";
    }
    return r;
}

}  // namespace fdk
