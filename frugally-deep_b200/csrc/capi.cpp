// extern "C" boundary (declared in include/fdeep_b200.h).  Translates exceptions into status codes.
#include "../../include/fdeep_b200.h"

#include "engine.hpp"
#include "kernels.cuh"
#include "session.hpp"

#include <cstring>
#include <fstream>
#include <sstream>

using namespace fdk;

struct fdk_model {
    std::unique_ptr<Engine> eng;
    std::string name, hash;
};

struct fdk_session {
    std::unique_ptr<DecodeSession> s;
};

static thread_local std::string g_last_error;

template <typename F>
static int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return 1;
    } catch (...) {
        g_last_error = "unknown error";
        return 2;
    }
}

static std::vector<TShape> shapes_from(const int64_t* dims5, const int* ranks, size_t n) {
    std::vector<TShape> r(n);
    for (size_t i = 0; i < n; ++i) {
        ensure(ranks[i] >= 1 && ranks[i] <= 5, "Invalid rank");
        for (int k = 0; k < 5; ++k) {
            r[i].d[k] = dims5[i * 5 + (size_t)k];
            ensure(r[i].d[k] >= 1, "tensor dimensions must be positive");
            if (k < 5 - ranks[i]) ensure(r[i].d[k] == 1, "dimensions above the rank must be 1");
        }
        r[i].rank = ranks[i];
    }
    return r;
}

extern "C" {

size_t fdk_last_error(char* buf, size_t buf_size) {
    if (buf && buf_size > 0) {
        const size_t n = std::min(buf_size - 1, g_last_error.size());
        std::memcpy(buf, g_last_error.data(), n);
        buf[n] = 0;
    }
    return g_last_error.size();
}

int fdk_device_count(int* count) {
    return guarded([&] {
        ensure(count != nullptr, "null argument");
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); n = 0; }
        *count = n;
    });
}

int fdk_model_load_json(const char* json_text, size_t json_len, const int* devices, int n_devices, unsigned flags, fdk_model** out) {
    return guarded([&] {
        ensure(json_text != nullptr && out != nullptr, "null argument");
        LoadedModel lm = load_model_json(json_text, json_len, (flags & 4u) != 0);
        EngineOptions opt;
        opt.use_tc = (flags & 1u) == 0;
        opt.skinny = (flags & 2u) != 0;
        opt.fuse_cells = (flags & 4u) != 0;
        std::vector<int> devs;
        for (int i = 0; i < n_devices; ++i) devs.push_back(devices[i]);
        auto m = std::make_unique<fdk_model>();
        m->name = lm.root->name;
        m->hash = lm.hash;
        m->eng = std::make_unique<Engine>(std::move(lm), devs, opt);
        *out = m.release();
    });
}

int fdk_model_load_file(const char* path, const int* devices, int n_devices, unsigned flags, fdk_model** out) {
    std::string text;
    const int rc = guarded([&] {
        ensure(path != nullptr, "null argument");
        std::ifstream f(path, std::ios::binary);
        ensure(f.good(), std::string("Can not open ") + path);
        std::ostringstream ss;
        ss << f.rdbuf();
        text = ss.str();
    });
    if (rc != 0) return rc;
    return fdk_model_load_json(text.data(), text.size(), devices, n_devices, flags, out);
}

void fdk_model_destroy(fdk_model* m) { delete m; }

int fdk_model_num_inputs(const fdk_model* m) { return m ? (int)m->eng->model().input_shapes.size() : 0; }
int fdk_model_num_outputs(const fdk_model* m) { return m ? (int)m->eng->model().output_shapes.size() : 0; }
int fdk_model_num_devices(const fdk_model* m) { return m ? m->eng->num_devices() : 0; }
const char* fdk_model_name(const fdk_model* m) { return m ? m->name.c_str() : ""; }
const char* fdk_model_hash(const fdk_model* m) { return m ? m->hash.c_str() : ""; }

static int var_shape_out(const std::vector<VarShape>& v, int index, int64_t dims5[5], int* rank) {
    return guarded([&] {
        ensure(index >= 0 && index < (int)v.size(), "shape index out of range");
        const VarShape& s = v[(size_t)index];
        for (int k = 0; k < 5; ++k) dims5[k] = 1;
        for (size_t i = 0; i < s.dims.size(); ++i) dims5[5 - s.dims.size() + i] = s.dims[i];
        *rank = (int)s.dims.size();
    });
}
int fdk_model_input_shape(const fdk_model* m, int index, int64_t dims5[5], int* rank) {
    if (!m) { g_last_error = "null model"; return 1; }
    return var_shape_out(m->eng->model().input_shapes, index, dims5, rank);
}
int fdk_model_output_shape(const fdk_model* m, int index, int64_t dims5[5], int* rank) {
    if (!m) { g_last_error = "null model"; return 1; }
    return var_shape_out(m->eng->model().output_shapes, index, dims5, rank);
}

int fdk_model_infer_shapes(fdk_model* m, const int64_t* in_dims5, const int* in_ranks, int64_t* out_dims5, int* out_ranks) {
    return guarded([&] {
        ensure(m != nullptr, "null model");
        const size_t n_in = m->eng->model().input_shapes.size();
        const std::vector<TShape> outs = m->eng->infer(shapes_from(in_dims5, in_ranks, n_in));
        for (size_t o = 0; o < outs.size(); ++o) {
            for (int k = 0; k < 5; ++k) out_dims5[o * 5 + (size_t)k] = outs[o].d[k];
            out_ranks[o] = outs[o].rank;
        }
    });
}

int fdk_model_predict_multi(fdk_model* m, int64_t n_samples, const float* const* in_ptrs, const int64_t* in_dims5,
                            const int* in_ranks, float* const* out_ptrs) {
    return guarded([&] {
        ensure(m != nullptr, "null model");
        ensure(n_samples >= 0, "negative sample count");
        if (n_samples == 0) return;
        const size_t n_in = m->eng->model().input_shapes.size();
        const std::vector<TShape> sh = shapes_from(in_dims5, in_ranks, (size_t)n_samples * n_in);
        m->eng->predict_multi(n_samples, in_ptrs, sh.data(), out_ptrs);
    });
}

int fdk_model_predict_multi_u8(fdk_model* m, int64_t n_samples, const uint8_t* const* in_ptrs, const int64_t* in_dims5,
                               const int* in_ranks, float low, float high, float* const* out_ptrs) {
    return guarded([&] {
        ensure(m != nullptr, "null model");
        ensure(n_samples >= 0, "negative sample count");
        if (n_samples == 0) return;
        const size_t n_in = m->eng->model().input_shapes.size();
        const std::vector<TShape> sh = shapes_from(in_dims5, in_ranks, (size_t)n_samples * n_in);
        ByteScale bs;
        bs.low = low; bs.high = high;
        m->eng->predict_multi(n_samples, reinterpret_cast<const float* const*>(in_ptrs), sh.data(), out_ptrs, &bs);
    });
}

int fdk_model_predict_batch_device(fdk_model* m, int device_index, int64_t batch, const float* const* d_in, const int64_t* in_dims5,
                                   const int* in_ranks, float* const* d_out, void* stream) {
    return guarded([&] {
        ensure(m != nullptr, "null model");
        const size_t n_in = m->eng->model().input_shapes.size();
        m->eng->predict_batch_device(device_index, batch, d_in, shapes_from(in_dims5, in_ranks, n_in), d_out, (cudaStream_t)stream);
    });
}

int fdk_model_sync(fdk_model* m, int device_index) {
    return guarded([&] {
        ensure(m != nullptr, "null model");
        ensure(device_index >= 0 && device_index < m->eng->num_devices(), "invalid device index");
        DeviceCtx& c = m->eng->ctx(device_index);
        int prev = 0;
        FDK_CUDA(cudaGetDevice(&prev));
        FDK_CUDA(cudaSetDevice(c.device));
        FDK_CUDA(cudaMemcpyAsync(c.h_err, c.d_err, sizeof(int), cudaMemcpyDeviceToHost, c.stream));
        FDK_CUDA(cudaStreamSynchronize(c.stream));
        const int err = *c.h_err;
        const int st = gemm_tc_take_status(c.stream);
        if (err) FDK_CUDA(cudaMemsetAsync(c.d_err, 0, sizeof(int), c.stream));
        cudaSetDevice(prev);
        if (err) raise(input_error_text(err));
        if (st) raise("tensor-core contraction kernel gave up waiting on a barrier (status " + std::to_string(st) + ")");
    });
}

int fdk_model_cuda_device(const fdk_model* m, int device_index, int* cuda_device) {
    return guarded([&] {
        ensure(m != nullptr && cuda_device != nullptr, "null argument");
        ensure(device_index >= 0 && device_index < m->eng->num_devices(), "invalid device index");
        *cuda_device = const_cast<fdk_model*>(m)->eng->ctx(device_index).device;
    });
}

namespace {
struct CurrentDevice {
    int prev = 0;
    explicit CurrentDevice(int dev) {
        FDK_CUDA(cudaGetDevice(&prev));
        if (prev != dev) FDK_CUDA(cudaSetDevice(dev));
    }
    ~CurrentDevice() { cudaSetDevice(prev); }
};
}  // namespace

int fdk_device_alloc(int cuda_device, size_t bytes, void** d_ptr) {
    return guarded([&] {
        ensure(d_ptr != nullptr, "null argument");
        CurrentDevice g(cuda_device);
        void* p = nullptr;
        const cudaError_t e = cudaMalloc(&p, bytes > 0 ? bytes : 1);
        if (e != cudaSuccess) {
            cudaGetLastError();
            raise("device allocation of " + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e));
        }
        *d_ptr = p;
    });
}

int fdk_device_free(int cuda_device, void* d_ptr) {
    return guarded([&] {
        if (!d_ptr) return;
        CurrentDevice g(cuda_device);
        FDK_CUDA(cudaFree(d_ptr));
    });
}

int fdk_device_copy(int cuda_device, void* dst, const void* src, size_t bytes, int kind) {
    return guarded([&] {
        ensure(kind >= 0 && kind <= 2, "fdk_device_copy: kind must be 0 (host to device), 1 (device to host) or 2 (device to device)");
        if (bytes == 0) return;
        ensure(dst != nullptr && src != nullptr, "null argument");
        CurrentDevice g(cuda_device);
        const cudaMemcpyKind k = kind == 0 ? cudaMemcpyHostToDevice : kind == 1 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
        FDK_CUDA(cudaMemcpy(dst, src, bytes, k));
        if (kind == 0) count_transfer(true, bytes);
        if (kind == 1) count_transfer(false, bytes);
    });
}

int fdk_transfer_bytes(uint64_t* host_to_device, uint64_t* device_to_host) {
    return guarded([&] {
        uint64_t a = 0, b = 0;
        transfer_totals(a, b);
        if (host_to_device) *host_to_device = a;
        if (device_to_host) *device_to_host = b;
    });
}

int fdk_model_run_tests(fdk_model* m, float epsilon, int* n_tests) {
    return guarded([&] {
        ensure(m != nullptr, "null model");
        if (n_tests) *n_tests = (int)m->eng->model().tests.size();
        m->eng->run_tests(epsilon);
    });
}

int64_t fdk_model_launch_count(const fdk_model* m) { return m ? m->eng->launches() : 0; }

int fdk_model_plan_info(fdk_model* m, const int64_t* in_dims5, const int* in_ranks, double* flops_per_sample,
                        int64_t* arena_bytes_per_sample, int64_t* max_batch) {
    return guarded([&] {
        ensure(m != nullptr, "null model");
        const size_t n_in = m->eng->model().input_shapes.size();
        const std::vector<TShape> sh = shapes_from(in_dims5, in_ranks, n_in);
        if (flops_per_sample) *flops_per_sample = m->eng->plan_flops(sh);
        if (arena_bytes_per_sample) *arena_bytes_per_sample = m->eng->plan_arena_bytes(sh);
        if (max_batch) *max_batch = m->eng->max_batch_for(sh, 0);
    });
}

int fdk_model_profile(fdk_model* m, int device_index, int64_t batch, const float* const* d_in, const int64_t* in_dims5,
                      const int* in_ranks, char* buf, size_t buf_size, size_t* needed) {
    return guarded([&] {
        ensure(m != nullptr, "null model");
        const size_t n_in = m->eng->model().input_shapes.size();
        const std::string text = m->eng->profile_batch_device(device_index, batch, d_in, shapes_from(in_dims5, in_ranks, n_in));
        if (needed) *needed = text.size() + 1;
        if (buf && buf_size > 0) {
            const size_t n = std::min(buf_size - 1, text.size());
            std::memcpy(buf, text.data(), n);
            buf[n] = 0;
        }
    });
}

int fdk_plan_describe(const char* json_text, size_t json_len, const int64_t* in_dims5, const int* in_ranks, int n_inputs, char* buf,
                      size_t buf_size, size_t* needed) {
    return guarded([&] {
        ensure(json_text != nullptr, "null argument");
        const LoadedModel lm = load_model_json(json_text, json_len);
        ensure((size_t)n_inputs == lm.input_shapes.size(), "Invalid number of input tensors for this model: " +
                                                               std::to_string(lm.input_shapes.size()) + " required but " +
                                                               std::to_string(n_inputs) + " provided");
        EngineOptions opt;
        const auto plan = compile_plan(lm, opt, shapes_from(in_dims5, in_ranks, (size_t)n_inputs));
        const std::string text = describe_plan(*plan);
        if (needed) *needed = text.size() + 1;
        if (buf && buf_size > 0) {
            const size_t n = std::min(buf_size - 1, text.size());
            std::memcpy(buf, text.data(), n);
            buf[n] = 0;
        }
    });
}

int fdk_gemm(int path, const float* dA, int64_t lda, const float* dW, int64_t ldw, float* dC, int64_t ldc, int64_t M, int N, int K,
             const float* d_bias, int relu, void* stream) {
    return guarded([&] {
        Epilogue e;
        e.bias = d_bias;
        if (relu) e.act2.kind = ACT_RELU;
        cudaStream_t s = (cudaStream_t)stream;
        if (path == 0) {
            launch_gemm_ffma(dA, lda, dW, ldw, dC, ldc, M, N, K, e, s);
        } else if (path == 3) {
            // row products (at most 64 rows) on the tcgen05 tensor cores: cluster split-K, nothing allocated
            ensure(gemm_rows_supported(M, N, K, lda, ldw, dA, dW), "fdk_gemm: shape not supported by the row-product path");
            const float* w1[1] = {dW};
            float* c1[1] = {dC};
            const int64_t l1[1] = {ldc};
            const float* b1[1] = {d_bias};
            launch_gemm_rows(dA, lda, 1, w1, ldw, c1, l1, b1, e, M, N, K, nullptr, s);
            FDK_CUDA(cudaStreamSynchronize(s));
            const int st = gemm_tc_take_status(s);
            if (st != 0) raise("tensor-core contraction kernel gave up waiting on a barrier (status " + std::to_string(st) + ")");
        } else if (path == 2) {
            // the weight-streaming split-K kernel for at most 64 rows, with a temporary (cleared) workspace
            ensure(gemm_skinny_supported(M, N, K, lda, ldw, dA, dW), "fdk_gemm: shape not supported by the skinny path");
            int slices = 1, kps = K;
            int64_t ws = 0;
            gemm_skinny_plan(N, K, slices, kps, ws, M);
            float* work = nullptr;
            if (ws > 0) FDK_CUDA(cudaMalloc(&work, (size_t)ws * sizeof(float)));
            try {
                if (ws > 0) FDK_CUDA(cudaMemsetAsync(work, 0, (size_t)ws * sizeof(float), s));
                launch_gemm_skinny(dA, lda, dW, ldw, dC, ldc, M, N, K, e, work, s);
                FDK_CUDA(cudaStreamSynchronize(s));
            } catch (...) {
                cudaFree(work);
                throw;
            }
            FDK_CUDA(cudaFree(work));
        } else {
            ensure(gemm_tc_supported(M, N, K, lda, ldw, dA, dW), "fdk_gemm: shape not supported by the tensor-core path");
            ensure(K <= ldw && K <= lda, "fdk_gemm: K must not exceed the row strides lda and ldw");
            // split the weights into TF32 halves in a temporary allocation.  Only the floats from the first row's start
            // to the last row's K-th value are read: W may be a block of rows of a larger matrix that ends there.
            float* halves = nullptr;
            const size_t n = (size_t)N * (size_t)ldw;
            const size_t n_read = (size_t)(N - 1) * (size_t)ldw + (size_t)K;
            FDK_CUDA(cudaMalloc(&halves, 2 * n * sizeof(float)));
            try {
                launch_split_tf32(dW, halves, halves + n, (int64_t)n_read, s);
                launch_gemm_tc(dA, lda, halves, halves + n, ldw, dC, ldc, M, N, K, e, s);
                FDK_CUDA(cudaStreamSynchronize(s));
                const int st = gemm_tc_take_status(s);
                if (st != 0) raise("tensor-core contraction kernel gave up waiting on a barrier (status " + std::to_string(st) + ")");
            } catch (...) {
                cudaFree(halves);
                throw;
            }
            FDK_CUDA(cudaFree(halves));
        }
    });
}

int fdk_shard_block(int64_t n_samples, int n_parts, int part, int64_t* begin, int64_t* end) {
    return guarded([&] {
        ensure(begin && end, "null argument");
        ensure(n_samples >= 0 && n_parts >= 1 && part >= 0 && part < n_parts, "fdk_shard_block: invalid argument");
        shard_block(n_samples, n_parts, part, *begin, *end);
    });
}

int fdk_split_tf32(const float* dW, float* d_big, float* d_small, int64_t n, void* stream) {
    return guarded([&] {
        ensure(dW && d_big && d_small && n >= 0, "fdk_split_tf32: invalid argument");
        launch_split_tf32(dW, d_big, d_small, n, (cudaStream_t)stream);
    });
}

int fdk_gemm_presplit(const float* dA, int64_t lda, const float* dW_big, const float* dW_small, int64_t ldw, float* dC, int64_t ldc,
                      int64_t M, int N, int K, const float* d_bias, const float* d_residual, int relu, void* stream) {
    return guarded([&] {
        Epilogue e;
        e.bias = d_bias;
        e.residual = d_residual;
        e.ldr = ldc;
        if (relu) e.act2.kind = ACT_RELU;
        ensure(gemm_tc_supported(M, N, K, lda, ldw, dA, dW_big), "fdk_gemm_presplit: shape not supported by the tensor-core path");
        launch_gemm_tc(dA, lda, dW_big, dW_small, ldw, dC, ldc, M, N, K, e, (cudaStream_t)stream);
    });
}

int fdk_gemm_static(const float* dA, int64_t lda, const float* dW, int64_t ldw, float* dC, int64_t ldc, int64_t M, int N, int K,
                    const float* d_bias, int relu, void* stream) {
    return guarded([&] {
        Epilogue e;
        e.bias = d_bias;
        if (relu) e.act2.kind = ACT_RELU;
        launch_gemm_tc_static(dA, lda, dW, ldw, dC, ldc, M, N, K, e, (cudaStream_t)stream);
    });
}

int64_t fdk_gemm_static_max_weight_floats(void) { return gemm_static_max_weight_floats(); }

int fdk_session_create(fdk_model* first, fdk_model* step, int64_t batch, int64_t max_len, fdk_session** out) {
    return guarded([&] {
        ensure(first && step && out, "null argument");
        std::unique_ptr<fdk_session> h(new fdk_session());
        h->s.reset(new DecodeSession(*first->eng, *step->eng, batch, max_len));
        *out = h.release();
    });
}

int fdk_session_step(fdk_session* s, const float* tokens, float* next_tokens, float* logits) {
    return guarded([&] {
        ensure(s != nullptr, "null session");
        s->s->step(tokens, next_tokens, logits);
    });
}

int fdk_session_info(const fdk_session* s, int64_t* length, int64_t* batch, int64_t* vocab) {
    return guarded([&] {
        ensure(s != nullptr, "null session");
        if (length) *length = s->s->length();
        if (batch) *batch = s->s->batch();
        if (vocab) *vocab = s->s->vocab();
    });
}

int fdk_session_reset(fdk_session* s) {
    return guarded([&] {
        ensure(s != nullptr, "null session");
        s->s->reset();
    });
}

void fdk_session_destroy(fdk_session* s) { delete s; }

int fdk_tc_status(void* stream, int* status) {
    return guarded([&] {
        ensure(status != nullptr, "null argument");
        *status = gemm_tc_take_status((cudaStream_t)stream);
    });
}

}  // extern "C"
