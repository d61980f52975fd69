#include "session.hpp"

#include "kernels.cuh"

#include <chrono>
#include <cstdio>
#include <cstring>
#include <cstdlib>

namespace fdk {

namespace {
struct DeviceSwitch {
    int prev = 0;
    explicit DeviceSwitch(int dev) { FDK_CUDA(cudaGetDevice(&prev)); FDK_CUDA(cudaSetDevice(dev)); }
    ~DeviceSwitch() { cudaSetDevice(prev); }
};
int64_t last_dim(const VarShape& s) { return s.dims.empty() ? -1 : s.dims.back(); }
// FDK_SESSION_TIMING=1: every session prints, when it is destroyed, how the host time of its steps divides into
// plan look-up (compilation at a new length included), queueing of the launches and waiting for the device.
bool timing_enabled() {
    static const bool on = [] { const char* v = getenv("FDK_SESSION_TIMING"); return v && *v && *v != '0'; }();
    return on;
}
bool env_flag(const char* name, bool dflt) {
    const char* v = getenv(name);
    return v && *v ? *v != '0' : dflt;
}
double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
}  // namespace

DecodeSession::DecodeSession(Engine& first, Engine& step, int64_t batch, int64_t max_len)
    : first_(first), step_(step), batch_(batch), max_len_(max_len) {
    ensure(batch >= 1 && max_len >= 1, "decode session: batch and max_len must be positive");
    const LoadedModel& mf = first.model();
    const LoadedModel& ms = step.model();
    ensure(mf.input_shapes.size() == 2, "decode session: the first-position model must have two inputs (token id, position)");
    ensure(mf.output_shapes.size() >= 2, "decode session: the first-position model must emit logits and one row per block");
    layers_ = (int)mf.output_shapes.size() - 1;
    ensure(ms.input_shapes.size() == (size_t)(2 + layers_), "decode session: the step model needs token id, position and one past tensor per block");
    ensure(ms.output_shapes.size() == mf.output_shapes.size(), "decode session: the two models must have the same outputs");
    vocab_ = last_dim(mf.output_shapes[0]);
    dim_ = last_dim(mf.output_shapes[1]);
    ensure(vocab_ > 0 && dim_ > 0, "decode session: logits and rows need a fixed last dimension");
    for (int l = 0; l < layers_; ++l) {
        ensure(last_dim(mf.output_shapes[(size_t)(1 + l)]) == dim_ && last_dim(ms.output_shapes[(size_t)(1 + l)]) == dim_ &&
                   last_dim(ms.input_shapes[(size_t)(2 + l)]) == dim_,
               "decode session: all rows and past tensors must have the same width");
    }
    device_ = first.ctx(0).device;
    ensure(step.ctx(0).device == device_, "decode session: both models must live on the same device");
    DeviceSwitch g(device_);
    FDK_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    const size_t B = (size_t)batch_, L = (size_t)layers_, D = (size_t)dim_, T = (size_t)max_len_;
    FDK_CUDA(cudaMalloc(&d_tokens_, B * sizeof(float)));
    FDK_CUDA(cudaMalloc(&d_next_, B * sizeof(float)));
    FDK_CUDA(cudaMalloc(&d_pos_, B * sizeof(float)));
    FDK_CUDA(cudaMalloc(&d_logits_, B * (size_t)vocab_ * sizeof(float)));
    FDK_CUDA(cudaMalloc(&d_rows_, L * B * D * sizeof(float)));
    FDK_CUDA(cudaMalloc(&d_len_, sizeof(int)));
    FDK_CUDA(cudaMemset(d_len_, 0, sizeof(int)));
    FDK_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&h_pub_), (B + 2) * sizeof(float), cudaHostAllocMapped));
    FDK_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&d_pub_), h_pub_, 0));
    std::memset(h_pub_, 0, (B + 2) * sizeof(float));
    status_a_ = gemm_tc_status_address();
    status_b_ = gemm_rows_status_address();
    // FDK_SESSION_DEVICE_LEN=0: every position is queued with its length known on the host (one plan per length);
    // FDK_SESSION_GRAPH=0: positions are queued launch by launch instead of being replayed from a recorded graph.
    device_len_ = env_flag("FDK_SESSION_DEVICE_LEN", true);
    use_graph_ = env_flag("FDK_SESSION_GRAPH", true);
    // can every attention block work on a key/value cache?
    std::vector<TShape> sf = {TShape::from_dims({1}), TShape::from_dims({1})};
    std::vector<TShape> ss = sf;
    for (int l = 0; l < layers_; ++l) ss.push_back(TShape::from_dims({1, dim_}));
    const auto bf = first.attention_blocks(sf), bs = step.attention_blocks(ss);
    cached_ = !bf.empty() && bf.size() == bs.size();
    int kw = 0, vw = 0;
    for (size_t i = 0; cached_ && i < bf.size(); ++i) {
        cached_ = bf[i].cacheable && bs[i].cacheable && bf[i].key_width == bs[i].key_width && bf[i].value_width == bs[i].value_width;
        kw = std::max(kw, bf[i].key_width);
        vw = std::max(vw, bf[i].value_width);
    }
    if (cached_) {
        kv_.max_len = max_len_;
        kv_.k_block_stride = (int64_t)(B * T) * kw;
        kv_.v_block_stride = (int64_t)(B * T) * vw;
        FDK_CUDA(cudaMalloc(&kv_.k, bf.size() * (size_t)kv_.k_block_stride * sizeof(float)));
        FDK_CUDA(cudaMalloc(&kv_.v, bf.size() * (size_t)kv_.v_block_stride * sizeof(float)));
    } else {
        FDK_CUDA(cudaMalloc(&d_past_[0], L * B * T * D * sizeof(float)));
        FDK_CUDA(cudaMalloc(&d_past_[1], L * B * T * D * sizeof(float)));
    }
}

void DecodeSession::reset() {
    DeviceSwitch g(device_);
    FDK_CUDA(cudaStreamSynchronize(stream_));
    FDK_CUDA(cudaMemsetAsync(d_len_, 0, sizeof(int), stream_));
    len_ = 0;
    cur_ = 0;
    failed_ = false;
}

DecodeSession::~DecodeSession() {
    cudaSetDevice(device_);
    if (stream_) cudaStreamSynchronize(stream_);
    if (timing_enabled() && len_ > 0)
        std::fprintf(stderr, "fdk session: %lld positions, per position: plan %.3f ms, queueing %.3f ms, waiting %.3f ms; device busy %.3f ms\n",
                     (long long)len_, t_plan_ / (double)len_ * 1e3, t_queue_ / (double)len_ * 1e3, t_wait_ / (double)len_ * 1e3,
                     t_device_ / (double)len_);
    if (ev_begin_) cudaEventDestroy(ev_begin_);
    if (ev_end_) cudaEventDestroy(ev_end_);
    drop_graph();
    cudaFree(d_len_);
    cudaFreeHost(h_pub_);
    cudaFree(d_tokens_); cudaFree(d_next_); cudaFree(d_pos_); cudaFree(d_logits_); cudaFree(d_rows_);
    cudaFree(d_past_[0]); cudaFree(d_past_[1]);
    cudaFree(kv_.k); cudaFree(kv_.v);
    if (stream_) cudaStreamDestroy(stream_);
}

// Launches of one position with the position itself read on the device (cache mode, positions after the first): the
// same sequence whatever the position, so that it can be recorded once and replayed.
void DecodeSession::queue_position_on_device() {
    launch_fill_from_counter(d_pos_, d_len_, batch_, stream_);
    std::vector<const float*> d_in = {d_tokens_, d_pos_};
    std::vector<TShape> shapes = {TShape::from_dims({1}), TShape::from_dims({1})};
    for (int l = 0; l < layers_; ++l) {
        d_in.push_back(d_rows_);  // the past inputs feed only the skipped concatenations: never read
        shapes.push_back(TShape::from_dims({1, dim_}));
    }
    std::vector<float*> d_out((size_t)(1 + layers_), nullptr);  // logits only; the rows live in the cache
    d_out[0] = d_logits_;
    KvCache kv = kv_;
    kv.len_dev = d_len_;
    // FDK_SESSION_PROFILE=1 (with FDK_SESSION_GRAPH=0): the last position of the session is run with events around
    // every operation and the device time per operation is printed (name, milliseconds)
    static const bool prof_on = env_flag("FDK_SESSION_PROFILE", false);
    std::string prof;
    step_.predict_batch_device(0, batch_, d_in.data(), shapes, d_out.data(), stream_, &kv, prof_on && len_ + 1 == max_len_ ? &prof : nullptr);
    if (!prof.empty()) std::fprintf(stderr, "fdk session profile of position %lld:\n%s", (long long)len_, prof.c_str());
    launch_argmax_rows(d_logits_, d_next_, batch_, (int)vocab_, stream_);
    launch_counter_add(d_len_, 1, stream_);
    publish();
    step_.ctx(0).launches += 4;   // position fill, greedy choice, length increment, publish
}

void DecodeSession::publish() {
    launch_publish_position(d_next_, (int)batch_, status_a_, status_b_, d_pub_, reinterpret_cast<int*>(d_pub_ + batch_), stream_);
}

void DecodeSession::drop_graph() {
    if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
    graph_exec_ = nullptr;
}

void DecodeSession::step(const float* tokens, float* next_tokens, float* logits) {
    ensure(!failed_, "decode session: an earlier step failed; the state on the device no longer matches the session's length");
    ensure(len_ < max_len_, "decode session: max_len positions already consumed");
    try {
        step_impl(tokens, next_tokens, logits);
    } catch (...) {
        // part of the position may have been queued (the length on the device advanced, rows written): no further steps
        failed_ = true;
        throw;
    }
}

// Replays the recorded position.  The recording holds the addresses of the step engine's arena and workspace, which
// other callers of that engine use too: the launch is made with the context's mutex held, after the arena's last
// user on another stream (device-side wait), and is itself recorded as the arena's last use.  Returns false when the
// buffers have moved since the recording (the caller records again).
bool DecodeSession::replay_position() {
    DeviceCtx& c = step_.ctx(0);
    std::lock_guard<std::mutex> lk(c.mu);
    if (c.arena != graph_arena_ || c.workspace != graph_workspace_) return false;
    step_.order_after_last_use(c, stream_);
    FDK_CUDA(cudaGraphLaunch(graph_exec_, stream_));
    step_.mark_use(c, stream_);
    c.launches += graph_launches_;
    return true;
}

void DecodeSession::step_impl(const float* tokens, float* next_tokens, float* logits) {
    DeviceSwitch g(device_);
    const size_t B = (size_t)batch_, D = (size_t)dim_, T = (size_t)max_len_;
    const size_t layer_stride = B * T * D;
    if (tokens) FDK_CUDA(cudaMemcpyAsync(d_tokens_, tokens, B * sizeof(float), cudaMemcpyHostToDevice, stream_));
    else {
        ensure(len_ > 0, "decode session: the first step needs tokens");
        FDK_CUDA(cudaMemcpyAsync(d_tokens_, d_next_, B * sizeof(float), cudaMemcpyDeviceToDevice, stream_));
    }
    const bool timing = timing_enabled();
    if (timing) {
        if (!ev_begin_) { FDK_CUDA(cudaEventCreate(&ev_begin_)); FDK_CUDA(cudaEventCreate(&ev_end_)); }
        FDK_CUDA(cudaEventRecord(ev_begin_, stream_));
    }
    double t0 = 0, t1 = 0;
    int new_len = (int)len_ + 1;
    if (cached_ && len_ > 0 && device_len_) {
        if (timing) t0 = t1 = now_s();
        DeviceCtx& c = step_.ctx(0);
        // a recorded position holds the addresses of the engine's arena and workspace: record again if they moved
        if (graph_exec_ && !replay_position()) drop_graph();
        if (graph_exec_) {
            // replayed above
        } else if (use_graph_ && warmed_) {
            // second and later positions of this kind: every buffer has its final size, record the launches
            const int64_t l0 = c.launches;
            cudaGraph_t graph = nullptr;
            FDK_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeRelaxed));
            bool ok = true;
            std::string why;
            try {
                queue_position_on_device();
            } catch (const std::exception& e) {
                ok = false;
                why = e.what();
            }
            const cudaError_t ce = cudaStreamEndCapture(stream_, &graph);
            bool replayed = false;
            const bool recorded = ok && ce == cudaSuccess && graph && cudaGraphInstantiate(&graph_exec_, graph, 0) == cudaSuccess;
            if (recorded) {
                graph_arena_ = c.arena;
                graph_workspace_ = c.workspace;
                graph_launches_ = c.launches - l0;
                c.launches = l0;
                replayed = replay_position();
                if (!replayed) drop_graph();   // another caller made the buffers move in between: launch directly this time
            }
            if (replayed) {
                // done
            } else if (recorded) {
                c.launches = l0;
                queue_position_on_device();
            } else {
                // nothing of a failed recording has run: go on without a graph
                cudaGetLastError();
                graph_exec_ = nullptr;
                use_graph_ = false;
                c.launches = l0;
                if (timing) std::fprintf(stderr, "fdk session: position not recorded as a graph (%s), launching directly\n", why.c_str());
                queue_position_on_device();
            }
            if (graph) cudaGraphDestroy(graph);
        } else {
            queue_position_on_device();
            warmed_ = true;
        }
    } else {
        launch_fill(d_pos_, (float)len_, batch_, stream_);
        std::vector<const float*> d_in;
        std::vector<TShape> shapes;
        d_in.push_back(d_tokens_); shapes.push_back(TShape::from_dims({1}));
        d_in.push_back(d_pos_); shapes.push_back(TShape::from_dims({1}));
        if (len_ > 0) {
            // the caches hold len_ rows per sequence, compact: [batch][len_][dim] per block
            for (int l = 0; l < layers_; ++l) {
                // with the key/value cache the past inputs are not read (their concatenations are skipped): any valid pointer
                d_in.push_back(cached_ ? d_rows_ : d_past_[cur_] + (size_t)l * layer_stride);
                shapes.push_back(TShape::from_dims({len_, dim_}));
            }
        }
        std::vector<float*> d_out;
        d_out.push_back(d_logits_);
        for (int l = 0; l < layers_; ++l) d_out.push_back(cached_ ? nullptr : d_rows_ + (size_t)l * B * D);
        Engine& eng = len_ == 0 ? first_ : step_;
        if (timing) {
            t0 = now_s();
            eng.infer(shapes);  // compiles and caches the plan of this length, so that the call below only looks it up
            t1 = now_s();
            t_plan_ += t1 - t0;
        }
        if (cached_) {
            kv_.len = len_;
            eng.predict_batch_device(0, batch_, d_in.data(), shapes, d_out.data(), stream_, &kv_);
            FDK_CUDA(cudaMemcpyAsync(d_len_, &new_len, sizeof(int), cudaMemcpyHostToDevice, stream_));
        } else {
            eng.predict_batch_device(0, batch_, d_in.data(), shapes, d_out.data(), stream_);
            // append the new rows: [batch][len_][dim] + [batch][1][dim] -> [batch][len_ + 1][dim] in the other buffer
            const int nxt = cur_ ^ 1;
            for (int l = 0; l < layers_; ++l) {
                float* dst = d_past_[nxt] + (size_t)l * layer_stride;
                if (len_ > 0) launch_slab_copy(d_past_[cur_] + (size_t)l * layer_stride, dst, batch_, len_ * dim_, (len_ + 1) * dim_, 0, stream_);
                launch_slab_copy(d_rows_ + (size_t)l * B * D, dst, batch_, dim_, (len_ + 1) * dim_, len_ * dim_, stream_);
            }
            cur_ = nxt;
        }
        launch_argmax_rows(d_logits_, d_next_, batch_, (int)vocab_, stream_);
        publish();
    }
    if (logits) FDK_CUDA(cudaMemcpyAsync(logits, d_logits_, B * (size_t)vocab_ * sizeof(float), cudaMemcpyDeviceToHost, stream_));
    const double t2 = timing ? now_s() : 0;
    if (timing) FDK_CUDA(cudaEventRecord(ev_end_, stream_));
    FDK_CUDA(cudaStreamSynchronize(stream_));
    if (timing) {
        t_queue_ += t2 - t1;
        t_wait_ += now_s() - t2;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, ev_begin_, ev_end_) == cudaSuccess) t_device_ += ms;
    }
    // the position's last kernel left the tokens and the kernels' status words in mapped host memory
    const int* st_words = reinterpret_cast<const int*>(h_pub_ + batch_);
    if (st_words[0] != 0 || st_words[1] != 0) {
        const int st = gemm_tc_take_status(stream_);   // prints what gave up and clears the words
        raise("tensor-core contraction kernel gave up waiting on a barrier (status " + std::to_string(st) + ")");
    }
    if (next_tokens) std::memcpy(next_tokens, h_pub_, B * sizeof(float));
    ++len_;
}

}  // namespace fdk
