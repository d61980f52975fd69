// Drop-in C++ host API of the B200 engine: the public surface of frugally-deep's <fdeep/fdeep.hpp>
// (fdeep::tensor, tensor_shape, tensor_pos, tensor_shape_variable, model, load_model, ...) with the
// same names, argument meaning and error behaviour, implemented over the C ABI in
// include/fdeep_b200.h.  Link with libfdeep_b200.so.  Each declaration names the reference header
// it mirrors (paths relative to the reference's include/fdeep/).
//
// What differs from the reference on purpose:
//   * there is no CPU implementation behind predict: all arithmetic runs in CUDA kernels on sm_100a,
//     and load_model throws when no CUDA device is present;
//   * predict_multi batches the samples and shards them over the model's GPUs instead of starting
//     one CPU thread per sample; results keep the input order either way;
//   * custom layer creators (user-supplied CPU layers) cannot run on the device and are rejected;
//   * float_vec is a plain std::vector<float> (the reference uses Eigen's aligned allocator) and the
//     fplus::maybe / fplus::shared_ref types that leak through the reference's API are provided by
//     small stand-ins below unless FunctionalPlus itself is included first;
//   * a tensor may keep its values on the GPU (an additional state, see class tensor): results of a model that was
//     asked to keep them there (model::keep_results_on_device), or of a prediction on device-resident inputs, reach
//     host memory only when the host first looks at them, so that models chain on the GPU.
#pragma once

#include "../../../include/fdeep_b200.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <fstream>
#include <functional>
#include <iomanip>
#include <iostream>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#ifndef FDEEP_FLOAT_TYPE
#define FDEEP_FLOAT_TYPE float
#endif

// ---- stand-ins for the FunctionalPlus types in the reference's public signatures -------------------
#ifndef FDEEP_B200_HAVE_FPLUS
namespace fplus {
template <typename T>
class maybe {  // fplus::maybe as used by tensor_shape_variable.hpp:97-101
public:
    maybe() : has_(false), v_() {}
    maybe(const T& v) : has_(true), v_(v) {}
    bool is_just() const { return has_; }
    bool is_nothing() const { return !has_; }
    const T& unsafe_get_just() const {
        if (!has_) throw std::runtime_error("maybe is nothing");
        return v_;
    }
    T get_with_default(const T& d) const { return has_ ? v_ : d; }
    bool operator==(const maybe& o) const { return has_ == o.has_ && (!has_ || v_ == o.v_); }
    bool operator!=(const maybe& o) const { return !(*this == o); }

private:
    bool has_;
    T v_;
};
template <typename T> maybe<T> just(const T& v) { return maybe<T>(v); }
template <typename T> maybe<T> nothing() { return maybe<T>(); }
template <typename T> T just_with_default(const T& d, const maybe<T>& m) { return m.get_with_default(d); }

template <typename T>
class shared_ref {  // fplus::shared_ref: a shared_ptr that is never null
public:
    explicit shared_ref(std::shared_ptr<T> p) : p_(std::move(p)) {}
    T* operator->() const { return p_.get(); }
    T& operator*() const { return *p_; }
    T* get() const { return p_.get(); }

private:
    std::shared_ptr<T> p_;
};
template <typename T, typename... Args>
shared_ref<T> make_shared_ref(Args&&... args) { return shared_ref<T>(std::make_shared<T>(std::forward<Args>(args)...)); }
}  // namespace fplus
#endif

namespace fdeep {
namespace internal {

// common.hpp:42-63
inline std::runtime_error error(const std::string& message) { return std::runtime_error(message); }
inline void raise_error(const std::string& msg) { throw error(msg); }
inline void assertion(bool cond, const std::string& error) { if (!cond) raise_error(error); }

typedef FDEEP_FLOAT_TYPE float_type;
static_assert(sizeof(float_type) == 4, "the device engine computes in float32 only");
typedef std::vector<float_type> float_vec;
typedef std::vector<float_type> float_vec_unaligned;
typedef fplus::shared_ref<float_vec> shared_float_vec;

// tensor_pos.hpp:23-114
class tensor_pos {
public:
    explicit tensor_pos(std::size_t d5, std::size_t d4, std::size_t y, std::size_t x, std::size_t z)
        : pos_dim_5_(d5), pos_dim_4_(d4), y_(y), x_(x), z_(z), rank_(5) {}
    explicit tensor_pos(std::size_t d4, std::size_t y, std::size_t x, std::size_t z) : pos_dim_5_(0), pos_dim_4_(d4), y_(y), x_(x), z_(z), rank_(4) {}
    explicit tensor_pos(std::size_t y, std::size_t x, std::size_t z) : pos_dim_5_(0), pos_dim_4_(0), y_(y), x_(x), z_(z), rank_(3) {}
    explicit tensor_pos(std::size_t x, std::size_t z) : pos_dim_5_(0), pos_dim_4_(0), y_(0), x_(x), z_(z), rank_(2) {}
    explicit tensor_pos(std::size_t z) : pos_dim_5_(0), pos_dim_4_(0), y_(0), x_(0), z_(z), rank_(1) {}
    std::size_t rank() const { return rank_; }
    std::vector<std::size_t> dimensions() const {
        const std::size_t all[5] = {pos_dim_5_, pos_dim_4_, y_, x_, z_};
        return std::vector<std::size_t>(all + 5 - rank_, all + 5);
    }
    std::size_t pos_dim_5_, pos_dim_4_, y_, x_, z_;

private:
    std::size_t rank_;
};

// tensor_shape.hpp:23-170
class tensor_shape {
public:
    explicit tensor_shape(std::size_t d5, std::size_t d4, std::size_t h, std::size_t w, std::size_t d)
        : size_dim_5_(d5), size_dim_4_(d4), height_(h), width_(w), depth_(d), rank_(5) {}
    explicit tensor_shape(std::size_t d4, std::size_t h, std::size_t w, std::size_t d) : size_dim_5_(1), size_dim_4_(d4), height_(h), width_(w), depth_(d), rank_(4) {}
    explicit tensor_shape(std::size_t h, std::size_t w, std::size_t d) : size_dim_5_(1), size_dim_4_(1), height_(h), width_(w), depth_(d), rank_(3) {}
    explicit tensor_shape(std::size_t w, std::size_t d) : size_dim_5_(1), size_dim_4_(1), height_(1), width_(w), depth_(d), rank_(2) {}
    explicit tensor_shape(std::size_t d) : size_dim_5_(1), size_dim_4_(1), height_(1), width_(1), depth_(d), rank_(1) {}
    std::size_t volume() const { return size_dim_5_ * size_dim_4_ * height_ * width_ * depth_; }
    std::size_t rank() const {
        assertion(rank_ >= 1 && rank_ <= 5, "Invalid rank");
        return rank_;
    }
    std::size_t minimal_rank() const {
        if (size_dim_5_ > 1) return 5;
        if (size_dim_4_ > 1) return 4;
        if (height_ > 1) return 3;
        if (width_ > 1) return 2;
        return 1;
    }
    void shrink_rank() { rank_ = minimal_rank(); }
    void shrink_rank_with_min(std::size_t min_rank_to_keep) { rank_ = std::max(minimal_rank(), min_rank_to_keep); }
    void maximize_rank() { rank_ = 5; }
    std::vector<std::size_t> dimensions() const {
        const std::size_t all[5] = {size_dim_5_, size_dim_4_, height_, width_, depth_};
        return std::vector<std::size_t>(all + 5 - rank(), all + 5);
    }
    std::size_t size_dim_5_, size_dim_4_, height_, width_, depth_;

private:
    std::size_t rank_;
};
inline bool operator==(const tensor_shape& a, const tensor_shape& b) {
    return a.rank() == b.rank() && a.size_dim_5_ == b.size_dim_5_ && a.size_dim_4_ == b.size_dim_4_ && a.height_ == b.height_ &&
           a.width_ == b.width_ && a.depth_ == b.depth_;
}
inline bool operator!=(const tensor_shape& a, const tensor_shape& b) { return !(a == b); }
inline tensor_shape create_tensor_shape_from_dims(const std::vector<std::size_t>& d) {
    assertion(d.size() >= 1 && d.size() <= 5, "Invalid tensor-shape dimensions");
    if (d.size() == 5) return tensor_shape(d[0], d[1], d[2], d[3], d[4]);
    if (d.size() == 4) return tensor_shape(d[0], d[1], d[2], d[3]);
    if (d.size() == 3) return tensor_shape(d[0], d[1], d[2]);
    if (d.size() == 2) return tensor_shape(d[0], d[1]);
    return tensor_shape(d[0]);
}

// tensor_shape_variable.hpp:20-118
class tensor_shape_variable {
public:
    typedef fplus::maybe<std::size_t> dim;
    explicit tensor_shape_variable(dim d5, dim d4, dim h, dim w, dim d) : size_dim_5_(d5), size_dim_4_(d4), height_(h), width_(w), depth_(d), rank_(5) {}
    explicit tensor_shape_variable(dim d4, dim h, dim w, dim d) : size_dim_5_(1), size_dim_4_(d4), height_(h), width_(w), depth_(d), rank_(4) {}
    explicit tensor_shape_variable(dim h, dim w, dim d) : size_dim_5_(1), size_dim_4_(1), height_(h), width_(w), depth_(d), rank_(3) {}
    explicit tensor_shape_variable(dim w, dim d) : size_dim_5_(1), size_dim_4_(1), height_(1), width_(w), depth_(d), rank_(2) {}
    explicit tensor_shape_variable(dim d) : size_dim_5_(1), size_dim_4_(1), height_(1), width_(1), depth_(d), rank_(1) {}
    std::size_t rank() const { return rank_; }
    dim size_dim_5_, size_dim_4_, height_, width_, depth_;

private:
    std::size_t rank_;
};
inline bool operator==(const tensor_shape_variable& a, const tensor_shape_variable& b) {
    return a.size_dim_5_ == b.size_dim_5_ && a.size_dim_4_ == b.size_dim_4_ && a.height_ == b.height_ && a.width_ == b.width_ && a.depth_ == b.depth_;
}
inline bool operator!=(const tensor_shape_variable& a, const tensor_shape_variable& b) { return !(a == b); }
// tensor_shape.hpp:206-237
inline tensor_shape make_tensor_shape_with(const tensor_shape& def, const tensor_shape_variable& s) {
    std::vector<std::size_t> d;
    if (s.rank() >= 5) d.push_back(s.size_dim_5_.get_with_default(def.size_dim_5_));
    if (s.rank() >= 4) d.push_back(s.size_dim_4_.get_with_default(def.size_dim_4_));
    if (s.rank() >= 3) d.push_back(s.height_.get_with_default(def.height_));
    if (s.rank() >= 2) d.push_back(s.width_.get_with_default(def.width_));
    d.push_back(s.depth_.get_with_default(def.depth_));
    return create_tensor_shape_from_dims(d);
}

inline std::string show_dims(const std::vector<std::string>& parts) {
    std::string r = "(";
    for (std::size_t i = 0; i < parts.size(); ++i) r += parts[i] + (i + 1 < parts.size() ? ", " : "");
    return r + ")";
}

inline std::string c_abi_error() {
    const std::size_t n = fdk_last_error(nullptr, 0);
    std::string s(n + 1, '\0');
    fdk_last_error(&s[0], n + 1);
    s.resize(n);
    return s;
}
inline void check(int rc) { if (rc != 0) raise_error(c_abi_error()); }

// One allocation on a GPU, shared by the tensors whose values lie in it (all results of one predict_multi call share
// one block per model output).  The first tensor that the host looks at fetches the whole block once; the others
// then copy their part from that host image.
struct device_block {
    void* ptr = nullptr;
    int cuda_device = 0;
    std::size_t floats = 0;
    std::mutex mu;
    std::vector<float_type> host_image;   // filled by the first host access to any tensor of the block
    bool fetched = false;
    device_block(int dev, std::size_t n) : cuda_device(dev), floats(n) { check(fdk_device_alloc(dev, n * sizeof(float_type), &ptr)); }
    ~device_block() { fdk_device_free(cuda_device, ptr); }
    device_block(const device_block&) = delete;
    device_block& operator=(const device_block&) = delete;
};
// The device side of one tensor: where its values lie and which copy is current.  Shared by the copies of a tensor,
// like the host vector is.
struct device_values {
    std::shared_ptr<device_block> block;
    std::size_t offset = 0;        // first value, in floats from the start of the block
    std::mutex mu;
    bool host_current = false;     // the host vector holds the values
    bool device_current = true;    // the device buffer holds the values (false once the host copy may have been written)
};

// tensor.hpp:28-168.  A shape plus shared storage, with value semantics as in the reference.  The storage is a host
// vector; a tensor that came out of a prediction kept on the device additionally (or instead) has a device buffer,
// and its host vector is filled on the first access from the host (get, as_vector, to_vector, show_tensor ...).
// Writing through set() or the non-const as_vector() makes the host vector the current copy.
class tensor {
public:
    tensor(const tensor_shape& shape, const shared_float_vec& values);
    tensor(const tensor_shape& shape, float_vec&& values) : tensor(shape, fplus::make_shared_ref<float_vec>(std::move(values))) {}
    tensor(const tensor_shape& shape, const float_vec_unaligned& values) : tensor(shape, fplus::make_shared_ref<float_vec>(values)) {}
    tensor(const tensor_shape& shape, float_type value) : tensor(shape, fplus::make_shared_ref<float_vec>(shape.volume(), value)) {}
    // a tensor whose values lie on the device (built by model::predict / model::to_device)
    tensor(const tensor_shape& shape, const std::shared_ptr<device_block>& block, std::size_t offset)
        : shape_(shape), values_(fplus::make_shared_ref<float_vec>()), dev_(std::make_shared<device_values>()) {
        assertion(block && offset + shape.volume() <= block->floats, "device tensor outside its buffer");
        dev_->block = block;
        dev_->offset = offset;
    }
    float_type get(const tensor_pos& pos) const { fetch(); return (*values_)[idx(pos)]; }
    float_type get_ignore_rank(const tensor_pos& pos) const { fetch(); return (*values_)[idx_ignore_rank(pos)]; }
    void set(const tensor_pos& pos, float_type value) { fetch_for_writing(); (*values_)[idx(pos)] = value; }
    void set_ignore_rank(const tensor_pos& pos, float_type value) { fetch_for_writing(); (*values_)[idx_ignore_rank(pos)] = value; }
    // deprecated five-index forms of the reference (tensor.hpp:88-109)
    float_type get(std::size_t d5, std::size_t d4, std::size_t y, std::size_t x, std::size_t z) const { return get_ignore_rank(tensor_pos(d5, d4, y, x, z)); }
    void set(std::size_t d5, std::size_t d4, std::size_t y, std::size_t x, std::size_t z, float_type v) { set_ignore_rank(tensor_pos(d5, d4, y, x, z), v); }
    const tensor_shape& shape() const { return shape_; }
    void shrink_rank() { shape_.shrink_rank(); }
    void shrink_rank_with_min(std::size_t m) { shape_.shrink_rank_with_min(m); }
    void maximize_rank() { shape_.maximize_rank(); }
    std::size_t rank() const { return shape_.rank(); }
    std::size_t depth() const { return shape_.depth_; }
    std::size_t height() const { return shape_.height_; }
    std::size_t width() const { return shape_.width_; }
    const shared_float_vec& as_vector() const { fetch(); return values_; }
    shared_float_vec& as_vector() { fetch_for_writing(); return values_; }
    float_vec_unaligned to_vector() const { fetch(); return float_vec_unaligned(*values_); }

    // ---- device side (not part of the reference's API) ----
    // True while the values can be read on the GPU without a copy from the host.
    bool on_device() const {
        if (!dev_) return false;
        std::lock_guard<std::mutex> lock(dev_->mu);
        return dev_->device_current;
    }
    int cuda_device() const { return dev_ ? dev_->block->cuda_device : -1; }
    // Device address of the first value (valid while on_device()); the tensor keeps the buffer alive.
    const float_type* device_data() const { return dev_ ? static_cast<const float_type*>(dev_->block->ptr) + dev_->offset : nullptr; }

private:
    // Makes the host vector hold the values (one device-to-host copy per block, the first time any tensor of the
    // block is read on the host).
    void fetch() const {
        if (!dev_) return;
        std::lock_guard<std::mutex> lock(dev_->mu);
        if (dev_->host_current) return;
        device_block& b = *dev_->block;
        {
            std::lock_guard<std::mutex> block_lock(b.mu);
            if (!b.fetched) {
                b.host_image.resize(b.floats);
                check(fdk_device_copy(b.cuda_device, b.host_image.data(), b.ptr, b.floats * sizeof(float_type), 1));
                b.fetched = true;
            }
        }
        values_->assign(b.host_image.begin() + (std::ptrdiff_t)dev_->offset, b.host_image.begin() + (std::ptrdiff_t)(dev_->offset + shape_.volume()));
        dev_->host_current = true;
    }
    void fetch_for_writing() {
        fetch();
        if (dev_) {
            std::lock_guard<std::mutex> lock(dev_->mu);
            dev_->device_current = false;   // the caller may change the host values: the device copy no longer counts
        }
    }
    std::size_t idx_ignore_rank(const tensor_pos& p) const {
        return (((p.pos_dim_5_ * shape_.size_dim_4_ + p.pos_dim_4_) * shape_.height_ + p.y_) * shape_.width_ + p.x_) * shape_.depth_ + p.z_;
    }
    std::size_t idx(const tensor_pos& p) const {
        assertion(p.rank() == shape_.rank(), "Invalid position rank for tensor");
        return idx_ignore_rank(p);
    }
    tensor_shape shape_;
    shared_float_vec values_;
    std::shared_ptr<device_values> dev_;   // null for a tensor that only ever lived on the host
};
typedef std::vector<tensor> tensors;
typedef std::vector<tensors> tensors_vec;

// import_model.hpp:376-381: user-supplied CPU layers; kept for signature compatibility, rejected at load.
class layer;
typedef std::map<std::string, std::function<std::shared_ptr<layer>(const void*, const void*, const std::string&)>> layer_creators;

}  // namespace internal

using float_type = internal::float_type;
using float_vec = internal::float_vec;
using shared_float_vec = internal::shared_float_vec;
using tensor_shape = internal::tensor_shape;
using tensor_shape_variable = internal::tensor_shape_variable;
using tensor_pos = internal::tensor_pos;
using tensor = internal::tensor;
using tensors = internal::tensors;
using tensors_vec = internal::tensors_vec;

inline std::string show_tensor_shape(const tensor_shape& s) {  // tensor_shape.hpp:349-356
    std::vector<std::string> parts;
    for (std::size_t d : s.dimensions()) parts.push_back(std::to_string(d));
    return internal::show_dims(parts);
}
inline std::string show_tensor_shapes(const std::vector<tensor_shape>& shapes) {
    std::string r = "[";
    for (std::size_t i = 0; i < shapes.size(); ++i) r += show_tensor_shape(shapes[i]) + (i + 1 < shapes.size() ? ", " : "");
    return r + "]";
}
inline std::string show_tensor_shape_variable(const tensor_shape_variable& s) {  // tensor_shape_variable.hpp:120-133
    const fplus::maybe<std::size_t> all[5] = {s.size_dim_5_, s.size_dim_4_, s.height_, s.width_, s.depth_};
    std::vector<std::string> parts;
    for (std::size_t i = 5 - s.rank(); i < 5; ++i) parts.push_back(all[i].is_just() ? "Just " + std::to_string(all[i].unsafe_get_just()) : "Nothing");
    return std::to_string(s.rank()) + internal::show_dims(parts);
}
inline std::string show_tensor_shapes_variable(const std::vector<tensor_shape_variable>& shapes) {
    std::string r = "[";
    for (std::size_t i = 0; i < shapes.size(); ++i) r += show_tensor_shape_variable(shapes[i]) + (i + 1 < shapes.size() ? ", " : "");
    return r + "]";
}

inline internal::tensor::tensor(const tensor_shape& shape, const shared_float_vec& values) : shape_(shape), values_(values) {
    assertion(shape.volume() == values->size(), std::string("invalid number of values. shape: ") + show_tensor_shape(shape) +
                                                    "; value count: " + std::to_string(values->size()));
}

// tensor.hpp:1203-1220: nested lists of fixed-precision values, padded to equal width
inline std::string show_tensor(const tensor& t) {
    const float_vec& xs = *t.as_vector();
    auto fmt = [](float_type v, std::size_t width) {
        std::ostringstream ss;
        ss << std::fixed << std::setprecision(4) << v;
        std::string s = ss.str();
        if (s.size() < width) s = std::string(width - s.size(), ' ') + s;
        return s;
    };
    std::size_t max_len = 0;
    for (float_type v : xs) max_len = std::max(max_len, fmt(v, 0).size());
    const tensor_shape& s = t.shape();
    std::string r = "[";
    std::size_t i = 0;
    for (std::size_t d5 = 0; d5 < s.size_dim_5_; ++d5) {
        r += std::string(d5 ? ", " : "") + "[";
        for (std::size_t d4 = 0; d4 < s.size_dim_4_; ++d4) {
            r += std::string(d4 ? ", " : "") + "[";
            for (std::size_t y = 0; y < s.height_; ++y) {
                r += std::string(y ? ", " : "") + "[";
                for (std::size_t x = 0; x < s.width_; ++x) {
                    r += std::string(x ? ", " : "") + "[";
                    for (std::size_t z = 0; z < s.depth_; ++z, ++i) r += std::string(z ? ", " : "") + fmt(xs[i], max_len);
                    r += "]";
                }
                r += "]";
            }
            r += "]";
        }
        r += "]";
    }
    return r + "]";
}
inline std::string show_tensors(const tensors& ts) {
    std::string r = "[";
    for (std::size_t i = 0; i < ts.size(); ++i) r += show_tensor(ts[i]) + (i + 1 < ts.size() ? ", " : "");
    return r + "]";
}

// tensor.hpp:1230-1280: 8-bit images <-> tensors; [0, 255] <-> [low, high]
inline tensor tensor_from_bytes(const std::uint8_t* value_ptr, std::size_t height, std::size_t width, std::size_t channels,
                                float_type low = 0.0f, float_type high = 1.0f) {
    float_vec values(height * width * channels);
    const float_type scale = (high - low) / 255.0f;  // fplus::reference_interval: scale first, then scale * x + low
    for (std::size_t i = 0; i < values.size(); ++i) values[i] = scale * static_cast<float_type>(value_ptr[i]) + low;
    return tensor(tensor_shape(height, width, channels), std::move(values));
}
inline void tensor_into_bytes(const tensor& t, std::uint8_t* value_ptr, std::size_t bytes_available, float_type low = 0.0f, float_type high = 1.0f) {
    const float_vec& values = *t.as_vector();
    internal::assertion(bytes_available == values.size(), "invalid buffer size");
    for (std::size_t i = 0; i < values.size(); ++i) {
        const float_type v = 0.0f + (values[i] - low) * 255.0f / (high - low);
        const float_type c = std::min(255.0f, std::max(0.0f, std::round(v)));
        value_ptr[i] = static_cast<std::uint8_t>(c);
    }
}
inline std::vector<std::uint8_t> tensor_to_bytes(const tensor& t, float_type low = 0.0f, float_type high = 1.0f) {
    std::vector<std::uint8_t> bytes(t.shape().volume(), 0);
    tensor_into_bytes(t, bytes.data(), bytes.size(), low, high);
    return bytes;
}

// model.hpp:184-193
inline void cout_logger(const std::string& str) { std::cout << str << std::flush; }
inline void dev_null_logger(const std::string&) {}

namespace internal {
struct model_handle {
    fdk_model* h = nullptr;
    bool results_on_device = false;   // model::keep_results_on_device
    ~model_handle() { if (h) fdk_model_destroy(h); }
};
inline void dims5_of(const tensor_shape& s, std::int64_t* d) {
    d[0] = (std::int64_t)s.size_dim_5_; d[1] = (std::int64_t)s.size_dim_4_; d[2] = (std::int64_t)s.height_;
    d[3] = (std::int64_t)s.width_; d[4] = (std::int64_t)s.depth_;
}
inline tensor_shape_variable var_shape_from(const std::int64_t* d, int rank) {
    typedef fplus::maybe<std::size_t> M;
    auto m = [&](int i) { return d[i] < 0 ? M() : M((std::size_t)d[i]); };
    if (rank == 5) return tensor_shape_variable(m(0), m(1), m(2), m(3), m(4));
    if (rank == 4) return tensor_shape_variable(m(1), m(2), m(3), m(4));
    if (rank == 3) return tensor_shape_variable(m(2), m(3), m(4));
    if (rank == 2) return tensor_shape_variable(m(3), m(4));
    return tensor_shape_variable(m(4));
}
}  // namespace internal

// model.hpp:19-182
class model {
public:
    // A single forward pass (no batches).  model.hpp:23-26
    tensors predict(const tensors& inputs) const { return predict_multi(std::vector<tensors>{inputs}, false).front(); }

    // Forward pass multiple data.  model.hpp:31-42.  The samples are batched on the GPU and split in
    // contiguous blocks over the model's devices; `parallelly` is accepted for compatibility.
    std::vector<tensors> predict_multi(const std::vector<tensors>& inputs_vec, bool parallelly) const {
        (void)parallelly;
        const std::size_t n_in = input_shapes_.size(), n_out = output_shapes_.size(), ns = inputs_vec.size();
        if (ns == 0) return {};
        // Device path: taken when the model keeps its results on the device, or when an input already lies there.
        bool device_path = h_->results_on_device;
        for (std::size_t s = 0; s < ns && !device_path; ++s)
            for (const tensor& t : inputs_vec[s]) device_path = device_path || t.on_device();
        if (device_path) return predict_multi_on_device(inputs_vec);
        std::vector<const float*> in_ptrs(ns * n_in);
        std::vector<std::int64_t> in_dims(ns * n_in * 5);
        std::vector<int> in_ranks(ns * n_in);
        for (std::size_t s = 0; s < ns; ++s) {
            internal::assertion(inputs_vec[s].size() == n_in, "Invalid number of input tensors for this model: " + std::to_string(n_in) +
                                                                  " required but " + std::to_string(inputs_vec[s].size()) + " provided");
            for (std::size_t i = 0; i < n_in; ++i) {
                const tensor& t = inputs_vec[s][i];
                in_ptrs[s * n_in + i] = t.as_vector()->data();
                internal::dims5_of(t.shape(), &in_dims[(s * n_in + i) * 5]);
                in_ranks[s * n_in + i] = (int)t.rank();
            }
        }
        std::vector<tensors> result(ns);
        std::vector<float*> out_ptrs(ns * n_out);
        std::vector<std::int64_t> od(n_out * 5);
        std::vector<int> orank(n_out);
        for (std::size_t s = 0; s < ns; ++s) {
            internal::check(fdk_model_infer_shapes(h_->h, &in_dims[s * n_in * 5], &in_ranks[s * n_in], od.data(), orank.data()));
            for (std::size_t o = 0; o < n_out; ++o) {
                std::vector<std::size_t> dims;
                for (int k = 5 - orank[o]; k < 5; ++k) dims.push_back((std::size_t)od[o * 5 + (std::size_t)k]);
                result[s].push_back(tensor(internal::create_tensor_shape_from_dims(dims), static_cast<float_type>(0)));
                out_ptrs[s * n_out + o] = result[s].back().as_vector()->data();
            }
        }
        internal::check(fdk_model_predict_multi(h_->h, (std::int64_t)ns, in_ptrs.data(), in_dims.data(), in_ranks.data(), out_ptrs.data()));
        return result;
    }

    // ---- device-resident results (not part of the reference's API) ----
    // With `on` the results of predict / predict_multi stay on the model's first GPU: the returned tensors hold device
    // buffers and reach host memory only when the host first reads them.  Feeding them to another model's predict
    // then needs no copy through host memory.  (The flag belongs to the model and its copies.)
    void keep_results_on_device(bool on = true) const { h_->results_on_device = on; }
    // A copy of a host tensor whose values lie on this model's first GPU.
    tensor to_device(const tensor& t) const {
        const int dev = first_cuda_device();
        auto block = std::make_shared<internal::device_block>(dev, t.shape().volume());
        internal::check(fdk_device_copy(dev, block->ptr, t.as_vector()->data(), t.shape().volume() * sizeof(float_type), 0));
        return tensor(t.shape(), block, 0);
    }

    // model.hpp:48-68
    std::size_t predict_class(const tensors& inputs) const { return predict_class_with_confidence(inputs).first; }
    std::pair<std::size_t, float_type> predict_class_with_confidence(const tensors& inputs) const {
        const tensors outputs = predict(inputs);
        internal::assertion(outputs.size() == 1, std::string("invalid number of outputs.\n") + "Use model::predict instead of model::predict_class.");
        const tensor_shape& s = outputs.front().shape();
        internal::assertion(s.size_dim_5_ == 1 && s.size_dim_4_ == 1 && s.height_ == 1 && s.width_ == 1,
                            std::string("invalid output shape.\n") + "Use model::predict instead of model::predict_class.");
        const float_vec& v = *outputs.front().as_vector();
        const std::size_t pos = (std::size_t)(std::max_element(v.begin(), v.end()) - v.begin());
        return std::make_pair(pos, v[pos]);
    }
    float_type predict_single_output(const tensors& inputs) const {
        const tensors outputs = predict(inputs);
        internal::assertion(outputs.size() == 1, "invalid number of outputs");
        internal::assertion(outputs.front().shape().volume() == 1, "invalid output shape");
        return outputs.front().to_vector().front();
    }

    // model.hpp:70-95
    const std::vector<tensor_shape_variable>& get_input_shapes() const { return input_shapes_; }
    const std::vector<tensor_shape_variable>& get_output_shapes() const { return output_shapes_; }
    const std::vector<tensor_shape> get_dummy_input_shapes() const {
        std::vector<tensor_shape> r;
        for (const auto& s : input_shapes_) r.push_back(internal::make_tensor_shape_with(tensor_shape(42, 42, 42), s));
        return r;
    }
    tensors generate_dummy_inputs() const {
        tensors r;
        for (const auto& s : get_dummy_input_shapes()) r.push_back(tensor(s, 0));
        return r;
    }
    // model.hpp:98-104: seconds for one forward pass on zero-filled dummy inputs
    double test_speed() const {
        const tensors inputs = generate_dummy_inputs();
        const auto t0 = std::chrono::steady_clock::now();
        predict(inputs);
        return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    }
    const std::string& name() const { return name_; }
    const std::string& hash() const { return hash_; }

private:
    model() {}
    int first_cuda_device() const {
        int dev = 0;
        internal::check(fdk_model_cuda_device(h_->h, 0, &dev));
        return dev;
    }
    // predict_multi on the model's first GPU with inputs gathered there (device-resident tensors by a copy on the
    // device, or not at all when a single sample already lies in one piece; host tensors by an upload) and results left
    // there: one block per model output, shared by the returned tensors.  Samples of different shapes go one by one.
    std::vector<tensors> predict_multi_on_device(const std::vector<tensors>& inputs_vec) const {
        const std::size_t n_in = input_shapes_.size(), n_out = output_shapes_.size(), ns = inputs_vec.size();
        for (std::size_t s = 0; s < ns; ++s)
            internal::assertion(inputs_vec[s].size() == n_in, "Invalid number of input tensors for this model: " + std::to_string(n_in) +
                                                                  " required but " + std::to_string(inputs_vec[s].size()) + " provided");
        bool same_shapes = true;
        for (std::size_t s = 1; s < ns && same_shapes; ++s)
            for (std::size_t i = 0; i < n_in; ++i) same_shapes = same_shapes && inputs_vec[s][i].shape() == inputs_vec[0][i].shape();
        if (!same_shapes) {
            std::vector<tensors> result;
            for (std::size_t s = 0; s < ns; ++s) result.push_back(predict_multi_on_device(std::vector<tensors>{inputs_vec[s]}).front());
            return result;
        }
        const int dev = first_cuda_device();
        std::vector<std::int64_t> in_dims(n_in * 5);
        std::vector<int> in_ranks(n_in);
        std::vector<std::shared_ptr<internal::device_block>> gathered(n_in);   // keeps gathered inputs alive until the call is done
        std::vector<const float*> d_in(n_in);
        for (std::size_t i = 0; i < n_in; ++i) {
            const tensor& first = inputs_vec[0][i];
            internal::dims5_of(first.shape(), &in_dims[i * 5]);
            in_ranks[i] = (int)first.rank();
            const std::size_t vol = first.shape().volume();
            if (ns == 1 && first.on_device() && first.cuda_device() == dev) {
                d_in[i] = first.device_data();
                continue;
            }
            gathered[i] = std::make_shared<internal::device_block>(dev, ns * vol);
            float* base = static_cast<float*>(gathered[i]->ptr);
            for (std::size_t s = 0; s < ns; ++s) {
                const tensor& t = inputs_vec[s][i];
                if (t.on_device() && t.cuda_device() == dev)
                    internal::check(fdk_device_copy(dev, base + s * vol, t.device_data(), vol * sizeof(float_type), 2));
                else
                    internal::check(fdk_device_copy(dev, base + s * vol, t.as_vector()->data(), vol * sizeof(float_type), 0));
            }
            d_in[i] = base;
        }
        std::vector<std::int64_t> od(n_out * 5);
        std::vector<int> orank(n_out);
        internal::check(fdk_model_infer_shapes(h_->h, in_dims.data(), in_ranks.data(), od.data(), orank.data()));
        std::vector<tensor_shape> out_shapes;
        std::vector<std::shared_ptr<internal::device_block>> out_blocks;
        std::vector<float*> d_out(n_out);
        for (std::size_t o = 0; o < n_out; ++o) {
            std::vector<std::size_t> dims;
            for (int k = 5 - orank[o]; k < 5; ++k) dims.push_back((std::size_t)od[o * 5 + (std::size_t)k]);
            out_shapes.push_back(internal::create_tensor_shape_from_dims(dims));
            out_blocks.push_back(std::make_shared<internal::device_block>(dev, ns * out_shapes.back().volume()));
            d_out[o] = static_cast<float*>(out_blocks.back()->ptr);
        }
        internal::check(fdk_model_predict_batch_device(h_->h, 0, (std::int64_t)ns, d_in.data(), in_dims.data(), in_ranks.data(), d_out.data(), nullptr));
        internal::check(fdk_model_sync(h_->h, 0));
        std::vector<tensors> result(ns);
        for (std::size_t s = 0; s < ns; ++s)
            for (std::size_t o = 0; o < n_out; ++o) result[s].push_back(tensor(out_shapes[o], out_blocks[o], s * out_shapes[o].volume()));
        return result;
    }
    std::shared_ptr<internal::model_handle> h_;
    std::vector<tensor_shape_variable> input_shapes_, output_shapes_;
    std::string name_, hash_;
    friend model read_model_from_string(const std::string&, bool, const std::function<void(std::string)>&, float_type, const internal::layer_creators&);
};

// model.hpp:272-281.  Devices: all visible CUDA devices unless FDEEP_B200_DEVICES lists indices ("0,1").
inline model read_model_from_string(const std::string& content, bool verify = true,
                                    const std::function<void(std::string)>& logger = cout_logger,
                                    float_type verify_epsilon = static_cast<float_type>(0.0001),
                                    const internal::layer_creators& custom_layer_creators = internal::layer_creators()) {
    internal::assertion(custom_layer_creators.empty(), "custom layer creators are not supported: user-defined CPU layers cannot run on the device");
    const auto t0 = std::chrono::steady_clock::now();
    auto elapsed = [&] {
        std::ostringstream ss;
        ss << std::fixed << std::setprecision(6) << std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        return ss.str();
    };
    if (logger) logger("Loading json and building model ... ");
    std::vector<int> devices;
    if (const char* env = std::getenv("FDEEP_B200_DEVICES")) {
        std::stringstream ss(env);
        std::string item;
        while (std::getline(ss, item, ',')) if (!item.empty()) devices.push_back(std::atoi(item.c_str()));
    } else {
        int n = 0;
        internal::check(fdk_device_count(&n));
        for (int i = 0; i < n; ++i) devices.push_back(i);
    }
    const unsigned flags = std::getenv("FDEEP_B200_NO_TENSOR_CORES") ? 1u : 0u;
    model m;
    m.h_ = std::make_shared<internal::model_handle>();
    internal::check(fdk_model_load_json(content.data(), content.size(), devices.empty() ? nullptr : devices.data(), (int)devices.size(), flags, &m.h_->h));
    if (logger) logger("done. elapsed time: " + elapsed() + " s\n");
    std::int64_t d[5];
    int rank = 0;
    for (int i = 0; i < fdk_model_num_inputs(m.h_->h); ++i) {
        internal::check(fdk_model_input_shape(m.h_->h, i, d, &rank));
        m.input_shapes_.push_back(internal::var_shape_from(d, rank));
    }
    for (int i = 0; i < fdk_model_num_outputs(m.h_->h); ++i) {
        internal::check(fdk_model_output_shape(m.h_->h, i, d, &rank));
        m.output_shapes_.push_back(internal::var_shape_from(d, rank));
    }
    m.name_ = fdk_model_name(m.h_->h);
    m.hash_ = fdk_model_hash(m.h_->h);
    if (verify) {  // model.hpp:254-267
        int n_tests = 0;
        const int rc = fdk_model_run_tests(m.h_->h, verify_epsilon, &n_tests);
        if (logger) logger(n_tests == 0 ? std::string("No test cases available\n") : "Running " + std::to_string(n_tests) + " test(s) ... ");
        internal::check(rc);
        if (logger && n_tests > 0) logger("done. elapsed time: " + elapsed() + " s\n");
    }
    return m;
}

// model.hpp:198-270
inline model read_model(std::istream& model_file_stream, bool verify = true, const std::function<void(std::string)>& logger = cout_logger,
                        float_type verify_epsilon = static_cast<float_type>(0.0001),
                        const internal::layer_creators& custom_layer_creators = internal::layer_creators()) {
    std::ostringstream ss;
    ss << model_file_stream.rdbuf();
    return read_model_from_string(ss.str(), verify, logger, verify_epsilon, custom_layer_creators);
}

// model.hpp:285-301
inline model load_model(const std::string& file_path, bool verify = true, const std::function<void(std::string)>& logger = cout_logger,
                        float_type verify_epsilon = static_cast<float_type>(0.0001),
                        const internal::layer_creators& custom_layer_creators = internal::layer_creators()) {
    const auto t0 = std::chrono::steady_clock::now();
    std::ifstream in_stream(file_path, std::ios::binary);
    internal::assertion(in_stream.good(), "Can not open " + file_path);
    const model m = read_model(in_stream, verify, logger, verify_epsilon, custom_layer_creators);
    if (logger) {
        std::ostringstream ss;
        ss << std::fixed << std::setprecision(6) << std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        logger("Loading, constructing" + std::string(verify ? ", testing" : "") + " of " + file_path + " took " + ss.str() + " s overall.\n");
    }
    return m;
}

}  // namespace fdeep
