// Executor: device contexts, weight upload, plan execution, predict_multi sharding.
#include "engine.hpp"
#include "kernels.cuh"
#include "plan_attrs.hpp"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <thread>

namespace fdk {

static int64_t round_up64(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Text for the device-side input checks (the flag a kernel leaves in DeviceCtx::d_err): the reference's assertions.
std::string input_error_text(int code) {
    if (code == 2) return "Invalid input value (> num_tokens).";   // category_encoding_layer.hpp:44,51
    return "vocabulary item indices must all be strictly less than the value of input_dim";   // embedding_layer.hpp:50
}

static std::atomic<uint64_t> g_h2d_bytes{0}, g_d2h_bytes{0};
void count_transfer(bool host_to_device, uint64_t bytes) { (host_to_device ? g_h2d_bytes : g_d2h_bytes) += bytes; }
void transfer_totals(uint64_t& host_to_device, uint64_t& device_to_host) {
    host_to_device = g_h2d_bytes.load();
    device_to_host = g_d2h_bytes.load();
}

void shard_block(int64_t n_samples, int n_parts, int part, int64_t& begin, int64_t& end) {
    if (n_parts < 1) n_parts = 1;
    const int64_t per = (n_samples + n_parts - 1) / n_parts;
    begin = std::min<int64_t>(n_samples, per * part);
    end = std::min<int64_t>(n_samples, begin + per);
}

struct DeviceGuard {
    int prev = 0;
    explicit DeviceGuard(int dev) {
        FDK_CUDA(cudaGetDevice(&prev));
        if (prev != dev) FDK_CUDA(cudaSetDevice(dev));
    }
    ~DeviceGuard() { cudaSetDevice(prev); }
};

Engine::Engine(LoadedModel&& lm, const std::vector<int>& devices, const EngineOptions& opt) : lm_(std::move(lm)), opt_(opt) {
    int n_dev = 0;
    const cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess || n_dev <= 0)
        raise("no CUDA device available: this engine has no CPU path (" + std::string(cudaGetErrorString(e)) + ")");
    std::vector<int> devs = devices;
    if (devs.empty()) devs.push_back(0);
    for (int d : devs) {
        ensure(d >= 0 && d < n_dev, "invalid device index " + std::to_string(d));
        auto c = std::make_unique<DeviceCtx>();
        c->device = d;
        DeviceGuard g(d);
        FDK_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        FDK_CUDA(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
        FDK_CUDA(cudaStreamCreateWithFlags(&c->aux_stream, cudaStreamNonBlocking));
        FDK_CUDA(cudaEventCreateWithFlags(&c->fork_event, cudaEventDisableTiming));
        FDK_CUDA(cudaEventCreateWithFlags(&c->join_event, cudaEventDisableTiming));
        FDK_CUDA(cudaEventCreateWithFlags(&c->busy, cudaEventDisableTiming));
        FDK_CUDA(cudaMalloc(&c->d_err, sizeof(int)));
        FDK_CUDA(cudaMemset(c->d_err, 0, sizeof(int)));
        FDK_CUDA(cudaMallocHost(&c->h_err, sizeof(int)));
        *c->h_err = 0;
        upload_weights(*c);
        ctx_.push_back(std::move(c));
    }
}

Engine::~Engine() {
    for (auto& c : ctx_) {
        cudaSetDevice(c->device);
        cudaStreamSynchronize(c->stream);
        if (c->busy_valid) cudaEventSynchronize(c->busy);
        if (c->busy) cudaEventDestroy(c->busy);
        cudaFree(c->w.base);
        cudaFree(c->arena);
        cudaFree(c->in_stage);
        cudaFree(c->byte_stage);
        cudaFree(c->workspace);
        cudaFree(c->d_err);
        cudaFreeHost(c->h_in);
        cudaFreeHost(c->h_out);
        cudaFreeHost(c->h_err);
        cudaStreamDestroy(c->stream);
        if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
        if (c->aux_stream) { cudaStreamSynchronize(c->aux_stream); cudaStreamDestroy(c->aux_stream); }
        if (c->fork_event) cudaEventDestroy(c->fork_event);
        if (c->join_event) cudaEventDestroy(c->join_event);
    }
}

void Engine::upload_weights(DeviceCtx& c) {
    const size_t n = lm_.weights.size();
    c.w.offset.assign(n, 0);
    c.w.big_offset.assign(n, -1);
    c.w.small_offset.assign(n, -1);
    int64_t total = 0;
    for (size_t i = 0; i < n; ++i) {
        c.w.offset[i] = total;
        total += round_up64((int64_t)lm_.weights[i].data.size() + 1, 64);
    }
    if (opt_.use_tc)
        for (size_t i = 0; i < n; ++i)
            if (lm_.weights[i].gemm) {
                const int64_t sz = round_up64((int64_t)lm_.weights[i].data.size() + 1, 64);
                c.w.big_offset[i] = total; total += sz;
                c.w.small_offset[i] = total; total += sz;
            }
    FDK_CUDA(cudaMalloc(&c.w.base, (size_t)std::max<int64_t>(total, 64) * sizeof(float)));
    for (size_t i = 0; i < n; ++i) {
        const auto& d = lm_.weights[i].data;
        if (!d.empty()) FDK_CUDA(cudaMemcpyAsync(c.w.base + c.w.offset[i], d.data(), d.size() * sizeof(float), cudaMemcpyHostToDevice, c.stream));
    }
    if (opt_.use_tc)
        for (size_t i = 0; i < n; ++i)
            if (c.w.big_offset[i] >= 0)
                launch_split_tf32(c.w.base + c.w.offset[i], c.w.base + c.w.big_offset[i], c.w.base + c.w.small_offset[i],
                                  (int64_t)lm_.weights[i].data.size(), c.stream);
    FDK_CUDA(cudaStreamSynchronize(c.stream));
}

static std::string signature(const std::vector<TShape>& s) {
    std::string k;
    for (const auto& x : s) {
        k += std::to_string(x.rank) + ":";
        for (int i = 0; i < 5; ++i) k += std::to_string(x.d[i]) + ",";
        k += ";";
    }
    return k;
}

std::shared_ptr<Plan> Engine::get_plan(const std::vector<TShape>& in_shapes) {
    const std::string key = signature(in_shapes);
    std::lock_guard<std::mutex> lk(plan_mu_);
    auto it = plans_.find(key);
    if (it != plans_.end()) return it->second;
    auto p = compile_plan(lm_, opt_, in_shapes);
    plans_[key] = p;
    return p;
}

std::vector<TShape> Engine::infer(const std::vector<TShape>& in_shapes) {
    auto p = get_plan(in_shapes);
    std::vector<TShape> r;
    for (int t : p->outputs) r.push_back(p->tensors[(size_t)t].shape);
    return r;
}
double Engine::plan_flops(const std::vector<TShape>& in_shapes) { return get_plan(in_shapes)->flops_per_sample; }
int64_t Engine::plan_arena_bytes(const std::vector<TShape>& in_shapes) { return get_plan(in_shapes)->arena_elems * 4; }

int64_t Engine::launches() const {
    int64_t n = 0;
    for (const auto& c : ctx_) n += c->launches;
    return n;
}

// The arena, the workspace and the staging buffers of a device serve one call at a time.  Calls may be queued on
// different streams (the engine's own, a caller's, a decode session's) and return before their work is done, so the
// order is kept on the device: every use ends by recording `busy` on its stream, and the next use on another stream
// waits for that event first.  Both are called with c.mu held, never on a stream that is being captured.
void Engine::order_after_last_use(DeviceCtx& c, cudaStream_t s) {
    if (c.busy_valid && c.busy_stream != s) FDK_CUDA(cudaStreamWaitEvent(s, c.busy, 0));
}
void Engine::mark_use(DeviceCtx& c, cudaStream_t s) {
    FDK_CUDA(cudaEventRecord(c.busy, s));
    c.busy_stream = s;
    c.busy_valid = true;
}

void Engine::ensure_arena(DeviceCtx& c, int64_t elems) {
    if (elems <= c.arena_elems) return;
    FDK_CUDA(cudaStreamSynchronize(c.stream));
    if (c.busy_valid) FDK_CUDA(cudaEventSynchronize(c.busy));  // the last user may have been another stream
    if (c.arena) FDK_CUDA(cudaFree(c.arena));
    c.arena = nullptr;
    c.arena_elems = 0;
    const cudaError_t e = cudaMalloc(&c.arena, (size_t)elems * sizeof(float));
    if (e != cudaSuccess) {
        cudaGetLastError();
        raise("device arena allocation of " + std::to_string(elems * 4) + " bytes failed: " + cudaGetErrorString(e));
    }
    c.arena_elems = elems;
}

int64_t Engine::max_batch_for(const std::vector<TShape>& in_shapes, int dev_index) {
    auto p = get_plan(in_shapes);
    DeviceCtx& c = *ctx_[(size_t)dev_index];
    DeviceGuard g(c.device);
    size_t free_b = 0, total_b = 0;
    FDK_CUDA(cudaMemGetInfo(&free_b, &total_b));
    int64_t in_elems = 0;
    for (const auto& s : p->in_shapes) in_elems += round_up64(s.volume(), 64);
    const double budget = opt_.mem_fraction * ((double)free_b + (double)c.arena_elems * 4 + (double)c.in_stage_elems * 4);
    const double per = (double)(std::max<int64_t>(p->arena_elems, 64) + in_elems) * 4.0;
    int64_t b = (int64_t)(budget / per);
    const int64_t cap = opt_.max_batch > 0 ? opt_.max_batch : 8192;
    return std::max<int64_t>(1, std::min(b, cap));
}

// ---------------------------------------------------------------------------------------------------------
// Plan execution
// ---------------------------------------------------------------------------------------------------------
namespace {
// For every operation of the plan: -1, or the index of the attention block it is (OP_MHA).  `x_tensor` receives, per
// block, the tensor whose rows are new at this position; `skip` marks the concatenations made redundant by the cache.
struct KvPlanInfo {
    std::vector<int> block_of_op;
    std::vector<int> x_tensor;
    std::vector<char> skip;
    std::vector<char> cacheable;
};
KvPlanInfo analyse_attention(const Plan& p) {
    KvPlanInfo r;
    r.block_of_op.assign(p.ops.size(), -1);
    r.skip.assign(p.ops.size(), 0);
    std::vector<int> uses(p.tensors.size(), 0), producer(p.tensors.size(), -1);
    for (size_t i = 0; i < p.ops.size(); ++i) {
        for (int t : p.ops[i].in) uses[(size_t)t]++;
        if (p.ops[i].residual >= 0) uses[(size_t)p.ops[i].residual]++;
        for (int t : p.ops[i].out) producer[(size_t)t] = (int)i;
    }
    for (int t : p.outputs) uses[(size_t)t] += 1000;
    for (size_t i = 0; i < p.ops.size(); ++i) {
        const Op& o = p.ops[i];
        if (o.kind != OP_MHA) continue;
        const int blk = (int)r.x_tensor.size();
        r.block_of_op[i] = blk;
        bool ok = o.layer->kv_heads == 0 && o.a[MHA_TQ] == 1 && (o.in.size() == 2 || o.in[2] == o.in[1]);
        int x = o.in.size() > 1 ? o.in[1] : -1;
        if (ok) {
            const int pr = producer[(size_t)o.in[1]];
            if (pr >= 0 && p.ops[(size_t)pr].kind == OP_CONCAT) {
                const Op& cc = p.ops[(size_t)pr];
                const TShape& os = p.tensors[(size_t)cc.out[0]].shape;
                const bool rows_axis = cc.a[0] == 3 && os.d[0] == 1 && os.d[1] == 1 && os.d[2] == 1;
                const bool past_is_input = cc.in.size() == 2 && p.buffers[(size_t)p.tensors[(size_t)cc.in[0]].buf].ext_input >= 0;
                const int n_uses = uses[(size_t)cc.out[0]] - (o.in.size() > 2 ? 1 : 0);
                if (rows_axis && past_is_input && n_uses == 1 && p.tensors[(size_t)cc.in[1]].shape.d[3] == 1) {
                    x = cc.in[1];
                    r.skip[(size_t)pr] = 1;
                } else {
                    ok = false;
                }
            } else {
                ok = o.a[MHA_TK] == 1;  // first position: the key/value input is the new row itself
            }
        }
        r.x_tensor.push_back(x);
        r.cacheable.push_back(ok ? 1 : 0);
    }
    return r;
}

struct Exec {
    Engine& eng;
    DeviceCtx& c;
    const Plan& p;
    int64_t B;
    const float* const* d_in;
    cudaStream_t s;
    bool use_tc;
    bool use_skinny = false;
    bool fuse_cells = false;
    const KvCache* kv = nullptr;   // decode session: attention on the cache
    KvPlanInfo kvi;
    // LayerNormalization folded into the row products that consume it (see plan_norm_folding)
    std::vector<int> norm_of_op;      // per operation: the normalisation its products apply to their input first, or -1
    std::vector<char> norm_folded;    // per operation: 1 = this normalisation runs inside its consumer and is not launched
    const std::vector<char>* wanted = nullptr;   // per plan output: 0 = the caller does not want it (null: all wanted)
    // profiling (off unless `prof` is set): events around operations and contraction launches
    struct Rec { std::string kind, name, path; cudaEvent_t a, b; double flops; int64_t M; int N, K; };
    std::vector<Rec>* prof = nullptr;
    const Op* cur_op = nullptr;
    int cur_index = 0;

    void rec_begin(Rec& r) {
        FDK_CUDA(cudaEventCreate(&r.a));
        FDK_CUDA(cudaEventCreate(&r.b));
        FDK_CUDA(cudaEventRecord(r.a, s));
    }

    float* tptr(int t) const {
        const BufferInfo& b = p.buffers[(size_t)p.tensors[(size_t)t].buf];
        if (b.ext_input >= 0) return const_cast<float*>(d_in[b.ext_input]);
        return c.arena + b.offset * B;
    }
    float* bptr(int buf) const { return c.arena + p.buffers[(size_t)buf].offset * B; }
    const TShape& shape(int t) const { return p.tensors[(size_t)t].shape; }
    const float* wptr(int id) const { return id < 0 ? nullptr : c.w.base + c.w.offset[(size_t)id]; }

    Epilogue epilogue(const Op& o, int64_t ldr) const {
        Epilogue e;
        e.bias = wptr(o.w_bias);
        e.act1 = o.act1;
        e.scale = wptr(o.w_scale);
        e.shift = wptr(o.w_shift);
        if (o.residual >= 0) { e.residual = tptr(o.residual); e.ldr = ldr; }
        e.act2 = o.act2;
        return e;
    }
    // w_off: offset (floats) of the first weight row to use inside weight array w_id (a block of rows of a larger matrix)
    // norm (optional): A is layer-normalised over K inside the product (only passed where plan_norm_folding has
    // checked that the row-product kernel takes this shape)
    void gemm(const float* A, int64_t lda, int w_id, int ldw, float* C, int64_t ldc, int64_t M, int N, int K, const Epilogue& e, int64_t w_off = 0,
              const RowsNorm* norm = nullptr) {
        const float* W = wptr(w_id) + w_off;
        // a handful of rows against a wide matrix: stream the weights over all SMs instead of a few 128-row tiles
        const bool skinny = use_skinny && N >= 256 && gemm_skinny_supported(M, N, K, lda, ldw, A, W);
        const bool rows = skinny && use_tc && gemm_rows_supported(M, N, K, lda, ldw, A, W);
        const bool tc = !skinny && use_tc && c.w.big_offset[(size_t)w_id] >= 0 && gemm_tc_supported(M, N, K, lda, ldw, A, W);
        ensure(norm == nullptr || rows, "internal: a folded normalisation needs the row-product kernel");
        Rec r;
        if (prof) {
            r = Rec{"gemm", cur_op && cur_op->layer ? cur_op->layer->name : "?", rows ? "rows" : skinny ? "skinny" : tc ? "tc" : "ffma", nullptr, nullptr,
                    2.0 * (double)M * N * K, M, N, K};
            rec_begin(r);
        }
        if (rows) {
            // tensor-core form: cluster split-K, reduction on chip, no workspace
            const float* w1[1] = {W};
            float* c1[1] = {C};
            const int64_t l1[1] = {ldc};
            const float* b1[1] = {e.bias};
            launch_gemm_rows(A, lda, 1, w1, ldw, c1, l1, b1, e, M, N, K, norm, s);
        } else if (skinny) {
            int slices = 1, kps = K;
            int64_t ws = 0;
            gemm_skinny_plan(N, K, slices, kps, ws, M);
            ensure_workspace(ws);
            launch_gemm_skinny(A, lda, W, ldw, C, ldc, M, N, K, e, c.workspace, s, use_tc);
        } else if (tc) {
            launch_gemm_tc(A, lda, c.w.base + c.w.big_offset[(size_t)w_id] + w_off, c.w.base + c.w.small_offset[(size_t)w_id] + w_off, ldw, C, ldc, M,
                           N, K, e, s);
        } else {
            launch_gemm_ffma(A, lda, W, ldw, C, ldc, M, N, K, e, s);
        }
        if (prof) {
            FDK_CUDA(cudaEventRecord(r.b, s));
            prof->push_back(r);
        }
        c.launches++;
    }

    // The workspace may move when it grows (a recorded graph that holds the old address must be recorded again: the
    // decode session compares addresses before every replay).
    void ensure_workspace(int64_t ws) {
        if (ws <= c.workspace_elems) return;
        FDK_CUDA(cudaStreamSynchronize(s));
        if (c.busy_valid) FDK_CUDA(cudaEventSynchronize(c.busy));
        if (c.workspace) FDK_CUDA(cudaFree(c.workspace));
        c.workspace = nullptr; c.workspace_elems = 0;
        FDK_CUDA(cudaMalloc(&c.workspace, sizeof(float) * (size_t)ws));
        FDK_CUDA(cudaMemset(c.workspace, 0, sizeof(float) * (size_t)ws));  // the arrival counters start at zero (synchronous)
        c.workspace_elems = ws;
    }
    // Query, key and value projections of one attention block on the same rows: one launch of the skinny kernel when
    // all three qualify for it (same shape, bias-only epilogues).  Returns false when nothing was launched.
    bool rows_three_supported(const float* A, int64_t lda, const int (&w_id)[3], int ldw, int64_t M, int N, int K) const {
        if (!use_skinny || !use_tc || N < 256) return false;
        for (int i = 0; i < 3; ++i)
            if (!gemm_rows_supported(M, N, K, lda, ldw, A, wptr(w_id[i]))) return false;
        return true;
    }
    bool gemm_skinny_three(const float* A, int64_t lda, const int (&w_id)[3], int ldw, float* const (&C)[3], const int64_t (&ldc)[3],
                           const int (&b_id)[3], int64_t M, int N, int K, const RowsNorm* norm = nullptr) {
        ensure(norm == nullptr || rows_three_supported(A, lda, w_id, ldw, M, N, K), "internal: a folded normalisation needs the row-product kernel");
        if (!use_skinny || N < 256) return false;
        const float* W[3];
        const float* bias[3];
        for (int i = 0; i < 3; ++i) {
            W[i] = wptr(w_id[i]);
            bias[i] = wptr(b_id[i]);
            if (!gemm_skinny_supported(M, N, K, lda, ldw, A, W[i])) return false;
        }
        if (use_tc && gemm_rows_supported(M, N, K, lda, ldw, A, W[0]) && gemm_rows_supported(M, N, K, lda, ldw, A, W[1]) &&
            gemm_rows_supported(M, N, K, lda, ldw, A, W[2])) {
            launch_gemm_rows(A, lda, 3, W, ldw, C, ldc, bias, Epilogue(), M, N, K, norm, s);
            c.launches++;
            return true;
        }
        int slices = 1, kps = K;
        int64_t ws = 0;
        gemm_skinny_plan(N, K, slices, kps, ws, M);
        if (((N + 63) / 64) * 3 > 512) return false;
        ensure_workspace(3 * ws);
        launch_gemm_skinny_group(A, lda, 3, W, ldw, C, ldc, bias, M, N, K, c.workspace, s, use_tc);
        c.launches++;
        return true;
    }

    RowsNorm norm_params(const Op& n) const {
        RowsNorm r;
        r.gamma = wptr(n.layer->w_gamma);
        r.beta = wptr(n.layer->w_beta);
        r.eps = n.f[0];
        return r;
    }
    // A LayerNormalization over the last axis whose only reader is a row product (a Dense on at most 64 rows, or the
    // query / key / value projections of an attention block working on the key/value cache) is not launched: the
    // product normalises the rows itself (gemm_rows.cu), which saves a launch and the round trip of the normalised rows.
    // Needs the row-product kernel (load flag "skinny products", tensor cores on), and the normalised tensor must not
    // be an output the caller wants.
    void plan_norm_folding() {
        norm_of_op.assign(p.ops.size(), -1);
        norm_folded.assign(p.ops.size(), 0);
        if (!use_skinny || !use_tc) return;
        std::vector<std::vector<int>> readers(p.tensors.size());
        for (size_t i = 0; i < p.ops.size(); ++i) {
            const Op& o = p.ops[i];
            if (o.dead || (kv && kvi.skip[i])) continue;
            for (int t : o.in) readers[(size_t)t].push_back((int)i);
            if (o.residual >= 0) readers[(size_t)o.residual].push_back((int)i);
            // on the cache an attention block reads the new row itself where the plan has Concatenate([past, row])
            if (kv && o.kind == OP_MHA && kvi.block_of_op[i] >= 0 && kvi.x_tensor[(size_t)kvi.block_of_op[i]] >= 0)
                readers[(size_t)kvi.x_tensor[(size_t)kvi.block_of_op[i]]].push_back((int)i);
        }
        auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
        for (size_t i = 0; i < p.ops.size(); ++i) {
            const Op& o = p.ops[i];
            if (o.dead || o.kind != OP_NORM || o.a[NORM_RMS] != 0) continue;
            const int64_t rows = B * o.a[NORM_ROWS];
            const int64_t n = o.a[NORM_N];
            if (rows > 64 || n % 4 != 0 || n > (1 << 24)) continue;
            const int t = o.out[0];
            bool output_wanted = false;
            for (size_t k = 0; k < p.outputs.size(); ++k)
                if (p.outputs[k] == t && (!wanted || (*wanted)[k])) output_wanted = true;
            if (output_wanted || readers[(size_t)t].empty()) continue;
            const int j = readers[(size_t)t][0];
            bool single = j > (int)i;
            for (int r : readers[(size_t)t]) single = single && r == j;
            if (!single) continue;
            const Op& u = p.ops[(size_t)j];
            const float* X = tptr(o.in[0]);
            const RowsNorm np = norm_params(o);
            if (!aligned(np.gamma) || !aligned(np.beta)) continue;
            if (u.kind == OP_GEMM && u.in[0] == t && u.residual != t && B * u.a[GEMM_ROWS] == rows && u.K == n && u.N >= 256 &&
                gemm_rows_supported(rows, u.N, u.K, u.K, u.ldw, X, wptr(u.w_main)) && gemm_rows_norm_supported(u.N, u.K, 1)) {
                norm_of_op[(size_t)j] = (int)i;
                norm_folded[i] = 1;
            } else if (u.kind == OP_MHA && kv && kvi.block_of_op[(size_t)j] >= 0 && u.residual != t) {
                const Layer& L = *u.layer;
                const int blk = kvi.block_of_op[(size_t)j];
                const int w3[3] = {L.w_q, L.w_k, L.w_v};
                const int HK = L.heads * L.key_dim, HV = L.heads * L.value_dim;
                if (u.in[0] == t && kvi.x_tensor[(size_t)blk] == t && u.a[MHA_TQ] == 1 && rows == B && L.in_feat == n && HK == HV &&
                    rows_three_supported(X, n, w3, L.ldw, rows, HK, (int)n) && gemm_rows_norm_supported(HK, (int)n, 3)) {
                    norm_of_op[(size_t)j] = (int)i;
                    norm_folded[i] = 1;
                }
            }
        }
    }

    void run() {
        if (kv) {
            kvi = analyse_attention(p);
            for (char ok : kvi.cacheable) ensure(ok != 0, "key/value cache: an attention operation of this model does not have the incremental form");
        }
        plan_norm_folding();
        for (size_t oi = 0; oi < p.ops.size(); ++oi) {
            const Op& o = p.ops[oi];
            if (kv && kvi.skip[oi]) continue;  // Concatenate([past, x]): the cache already holds the past rows
            if (norm_folded[oi]) continue;     // runs inside the product that reads it
            cur_op = &o;
            cur_index = (int)oi;
            Rec r;
            if (prof) {
                // an operation's record carries its algorithmic bytes in the M field: every input (and the residual) read
                // once, every output written once
                int64_t bytes = 0;
                for (int t : o.in) bytes += shape(t).volume();
                for (int t : o.out) bytes += shape(t).volume();
                if (o.residual >= 0) bytes += shape(o.residual).volume();
                r = Rec{"op", o.layer ? o.layer->name : "?", std::to_string(o.kind), nullptr, nullptr, 0.0, bytes * B * 4, 0, 0};
                rec_begin(r);
            }
            run_op(o);
            if (prof) {
                FDK_CUDA(cudaEventRecord(r.b, s));
                prof->push_back(r);
            }
        }
    }

    void run_op(const Op& o) {
        {
            switch (o.kind) {
                case OP_CONV: conv(o); break;
                case OP_GEMM: {
                    const int64_t M = B * o.a[GEMM_ROWS];
                    const int nf = norm_of_op[(size_t)cur_index];
                    if (nf >= 0) {
                        const RowsNorm np = norm_params(p.ops[(size_t)nf]);
                        gemm(tptr(p.ops[(size_t)nf].in[0]), o.K, o.w_main, o.ldw, tptr(o.out[0]), o.N, M, o.N, o.K, epilogue(o, o.N), 0, &np);
                    } else {
                        gemm(tptr(o.in[0]), o.K, o.w_main, o.ldw, tptr(o.out[0]), o.N, M, o.N, o.K, epilogue(o, o.N));
                    }
                    break;
                }
                case OP_DWCONV: {
                    const int C = (int)o.a[CONV_C];
                    launch_dwconv(tptr(o.in[0]), wptr(o.w_main), tptr(o.out[0]), B, (int)o.a[CONV_H], (int)o.a[CONV_W], C, (int)o.a[CONV_HO],
                                  (int)o.a[CONV_WO], (int)o.a[CONV_KH], (int)o.a[CONV_KW], (int)o.a[CONV_SY], (int)o.a[CONV_SX],
                                  (int)o.a[CONV_PT], (int)o.a[CONV_PL], epilogue(o, C), s);
                    c.launches++;
                    break;
                }
                case OP_POOL: {
                    const TShape &is = shape(o.in[0]), &os = shape(o.out[0]);
                    const Layer& L = *o.layer;
                    int frame[6];
                    for (int i = 0; i < 6; ++i) frame[i] = (int)o.a[POOL_ZF + i];
                    launch_pool3d(tptr(o.in[0]), tptr(o.out[0]), B, (int)is.d[1], (int)is.d[2], (int)is.d[3], (int)is.d[4], (int)os.d[1],
                                  (int)os.d[2], (int)os.d[3], L.k[0], L.k[1], L.k[2], L.s[0], L.s[1], L.s[2], (int)o.a[POOL_PF],
                                  (int)o.a[POOL_PT], (int)o.a[POOL_PL], o.a[POOL_FRAMED] ? frame : nullptr, o.a[POOL_MAX] != 0, s);
                    c.launches++;
                    break;
                }
                case OP_GPOOL: {
                    const TShape& is = shape(o.in[0]);
                    launch_global_pool(tptr(o.in[0]), tptr(o.out[0]), B, is.d[1] * is.d[2] * is.d[3], (int)is.d[4], o.a[0] != 0, s);
                    c.launches++;
                    break;
                }
                case OP_BINARY: {
                    launch_binary((int)o.a[0], tptr(o.in[0]), shape(o.in[0]).d, tptr(o.in[1]), shape(o.in[1]).d, tptr(o.out[0]),
                                  shape(o.out[0]).d, B, o.f[0], o.act, s);
                    c.launches++;
                    break;
                }
                case OP_UNARY:
                    launch_unary(o.act, tptr(o.in[0]), tptr(o.out[0]), B * shape(o.in[0]).volume(), s);
                    c.launches++;
                    break;
                case OP_AFFINE:
                    if (o.a[AFF_CONST]) launch_scale(tptr(o.in[0]), tptr(o.out[0]), B * shape(o.in[0]).volume(), o.f[0], s);
                    else launch_affine(tptr(o.in[0]), tptr(o.out[0]), wptr(o.w_scale), wptr(o.w_shift), B * o.a[AFF_OUTER], o.a[AFF_NC], o.a[AFF_INNER], o.act, s);
                    c.launches++;
                    break;
                case OP_SOFTMAX: {
                    const TShape& is = shape(o.in[0]);
                    launch_softmax(tptr(o.in[0]), tptr(o.out[0]), B, is.volume() / is.d[4], is.d[2] * is.d[3], (int)is.d[4], o.a[0] != 0, s);
                    c.launches++;
                    break;
                }
                case OP_NORM:
                    if (o.a[NORM_RMS] == 3) {  // group normalisation: rows = spatial positions, n = channels
                        launch_groupnorm(tptr(o.in[0]), tptr(o.out[0]), wptr(o.layer->w_gamma), wptr(o.layer->w_beta), B, o.a[NORM_ROWS],
                                         (int)o.a[NORM_N], o.layer->units, o.f[0], s);
                    } else {
                        launch_layernorm(tptr(o.in[0]), tptr(o.out[0]), wptr(o.layer->w_gamma), wptr(o.layer->w_beta), B * o.a[NORM_ROWS],
                                         (int)o.a[NORM_N], o.f[0], (int)o.a[NORM_RMS], s);
                    }
                    c.launches++;
                    break;
                case OP_WINDOW: {
                    const TShape &is = shape(o.in[0]), &os = shape(o.out[0]);
                    launch_window(tptr(o.in[0]), tptr(o.out[0]), B, (int)is.d[1], (int)is.d[2], (int)is.d[3], (int)is.d[4], (int)os.d[1],
                                  (int)os.d[2], (int)os.d[3], (int)o.a[0], (int)o.a[1], (int)o.a[2], s);
                    c.launches++;
                    break;
                }
                case OP_CONCAT: {
                    const int ax = (int)o.a[0];
                    const TShape& os = shape(o.out[0]);
                    int64_t outer = B, inner = 1;
                    for (int i = 0; i < ax; ++i) outer *= os.d[i];
                    for (int i = ax + 1; i < 5; ++i) inner *= os.d[i];
                    int64_t off = 0;
                    for (int t : o.in) {
                        const int64_t len = shape(t).d[ax] * inner;
                        launch_slab_copy(tptr(t), tptr(o.out[0]), outer, len, os.d[ax] * inner, off, s);
                        c.launches++;
                        off += len;
                    }
                    break;
                }
                case OP_PERMUTE: {
                    int perm[5];
                    for (int i = 0; i < 5; ++i) perm[i] = (int)o.a[i];
                    launch_permute(tptr(o.in[0]), tptr(o.out[0]), B, shape(o.in[0]).d, perm, s);
                    c.launches++;
                    break;
                }
                case OP_EMBED:
                    launch_embedding(tptr(o.in[0]), wptr(o.layer->w_main), tptr(o.out[0]), B * shape(o.in[0]).d[4], o.layer->units,
                                     o.layer->input_dim, c.d_err, s);
                    c.launches++;
                    break;
                case OP_LSTM:
                case OP_GRU:
                case OP_RNN: recurrent(o); break;
                case OP_MHA: mha(o); break;
                case OP_ATTN: {
                    const Layer& L = *o.layer;
                    const TShape &q = shape(o.in[0]), &v = shape(o.in[1]);
                    const int Tq = (int)o.a[MHA_TQ], Tk = (int)o.a[MHA_TK], D = (int)q.d[4], Dv = (int)v.d[4];
                    AttnExtra x;
                    x.mode = L.bin_op;
                    x.w2 = L.f_w2;
                    x.svec = L.w_aux >= 0 ? wptr(L.w_aux) : nullptr;
                    x.sn = L.input_dim;
                    const float* kp = tptr(o.in.size() > 2 ? o.in[2] : o.in[1]);
                    launch_attention(tptr(o.in[0]), D, (int64_t)Tq * D, kp, D, (int64_t)Tk * D, tptr(o.in[1]), Dv, (int64_t)Tk * Dv, tptr(o.out[0]), Dv,
                                     (int64_t)Tq * Dv, B, 1, Tq, Tk, D, Dv, L.f_scale, s, x);
                    c.launches++;
                    break;
                }
                case OP_CONV3D: {
                    Conv3dGeom g;
                    for (int i = 0; i < 3; ++i) {
                        g.in[i] = (int)o.a[i]; g.out[i] = (int)o.a[3 + i]; g.stride[i] = (int)o.a[6 + i]; g.pad_lo[i] = (int)o.a[9 + i];
                        g.spread[i] = (int)o.a[12 + i]; g.off[i] = (int)o.a[15 + i]; g.inner[i] = (int)o.a[18 + i]; g.k[i] = o.layer->k[i];
                    }
                    g.C = o.layer->in_feat; g.Kp = o.ldw;
                    if (o.a[22]) {
                        // no patch matrix: filter taps (kz, ky, kx) walk the input slices through the 4-D tensor map
                        // (dilated filters were spread at load, so the dilation here is 1)
                        ConvTcGeom t;
                        t.B = B; t.D = g.in[0]; t.H = g.in[1]; t.W = g.in[2]; t.C = g.C; t.pix = g.C;
                        t.Do = g.out[0]; t.Ho = g.out[1]; t.Wo = g.out[2];
                        t.kd = g.k[0]; t.kh = g.k[1]; t.kw = g.k[2];
                        t.sz = g.stride[0]; t.sy = g.stride[1]; t.sx = g.stride[2];
                        t.pad_f = g.pad_lo[0]; t.pad_t = g.pad_lo[1]; t.pad_l = g.pad_lo[2];
                        const int w_id = o.w_main;
                        ensure(c.w.big_offset[(size_t)w_id] >= 0 && conv_tc_supported(t, o.N, o.ldw, tptr(o.in[0]), wptr(w_id)),
                               "convolution '" + o.layer->name + "': the tensor-core path needs 16-byte aligned input tensors");
                        const int64_t M3 = B * o.a[21];
                        Rec r;
                        if (prof) {
                            r = Rec{"gemm", o.layer->name, "tc", nullptr, nullptr, 2.0 * (double)M3 * o.N * o.K, M3, o.N, o.K};
                            rec_begin(r);
                        }
                        launch_conv_tc(tptr(o.in[0]), t, c.w.base + c.w.big_offset[(size_t)w_id], c.w.base + c.w.small_offset[(size_t)w_id], o.ldw,
                                       tptr(o.out[0]), o.N, o.N, epilogue(o, o.N), s);
                        if (prof) {
                            FDK_CUDA(cudaEventRecord(r.b, s));
                            prof->push_back(r);
                        }
                        c.launches++;
                        break;
                    }
                    if (o.a[23]) {
                        // transposed, without a patch matrix: per output phase (pz, py, px) a stride-1 walk of the undilated
                        // input slices with the phase's sub-filter, written to every s-th output slice, row and column
                        const Layer& L = *o.layer;
                        const int sz = L.s[0], sy = L.s[1], sx = L.s[2];
                        const int Do = g.out[0], Ho = g.out[1], Wo = g.out[2];
                        const int lead[3] = {transposed_lead(L.k[0], sz, L.pad), transposed_lead(L.k[1], sy, L.pad), transposed_lead(L.k[2], sx, L.pad)};
                        float* out = tptr(o.out[0]);
                        const Epilogue e3 = epilogue(o, o.N);
                        for (int pz = 0; pz < sz; ++pz) for (int py = 0; py < sy && py < Ho; ++py) for (int px = 0; px < sx && px < Wo; ++px) {
                            const TransposedPhase tz = transposed_phase(L.k[0], sz, lead[0], pz), ty = transposed_phase(L.k[1], sy, lead[1], py),
                                                  tx = transposed_phase(L.k[2], sx, lead[2], px);
                            const int w_id = L.w_phases[(size_t)((pz * sy + py) * sx + px)];
                            ConvTcGeom t;
                            t.B = B; t.D = g.in[0]; t.H = g.in[1]; t.W = g.in[2]; t.C = g.C; t.pix = g.C;
                            t.Do = Do / sz; t.Ho = (Ho - py + sy - 1) / sy; t.Wo = (Wo - px + sx - 1) / sx;
                            t.kd = tz.taps; t.kh = ty.taps; t.kw = tx.taps;
                            t.pad_f = -tz.shift; t.pad_t = -ty.shift; t.pad_l = -tx.shift;
                            t.out_sx = (int64_t)sx * o.N; t.out_sy = (int64_t)sy * Wo * o.N; t.out_sb = (int64_t)sz * Ho * Wo * o.N;
                            const int64_t first = (((int64_t)pz * Ho + py) * Wo + px) * o.N;
                            const int kd = tz.taps * ty.taps * tx.taps * g.C;
                            ensure(c.w.big_offset[(size_t)w_id] >= 0 && conv_tc_supported(t, o.N, kd, tptr(o.in[0]), wptr(w_id)),
                                   "convolution '" + L.name + "': the tensor-core path needs 16-byte aligned input tensors");
                            launch_conv_tc(tptr(o.in[0]), t, c.w.base + c.w.big_offset[(size_t)w_id], c.w.base + c.w.small_offset[(size_t)w_id], kd,
                                           out + first, o.N, o.N, e3, s);
                            c.launches++;
                        }
                        break;
                    }
                    float* col = bptr(o.scratch[0]);
                    launch_im2col3d(tptr(o.in[0]), col, B, g, s);
                    c.launches++;
                    gemm(col, o.ldw, o.w_main, o.ldw, tptr(o.out[0]), o.N, B * o.a[21], o.N, o.ldw, epilogue(o, o.N));
                    break;
                }
                case OP_NORMALIZE:
                    launch_normalization(tptr(o.in[0]), tptr(o.out[0]), wptr(o.layer->w_scale), wptr(o.layer->w_shift), B * o.a[0], o.a[1], o.a[2],
                                         o.layer->flag_a, s);
                    c.launches++;
                    break;
                case OP_UPSAMPLE:
                    launch_upsample2d(tptr(o.in[0]), tptr(o.out[0]), B * o.a[3], (int)o.a[0], (int)o.a[1], (int)o.a[2], (int)o.a[4], (int)o.a[5],
                                      o.layer->flag_a, s);
                    c.launches++;
                    break;
                case OP_RESIZE:
                    launch_resize2d(tptr(o.in[0]), tptr(o.out[0]), B, (int)o.a[0], (int)o.a[1], (int)o.a[2], (int)o.a[3], (int)o.a[4], (int)o.a[5],
                                    (int)o.a[6], (int)o.a[7], (int)o.a[8], (int)o.a[9], s);
                    c.launches++;
                    break;
                case OP_DOT:
                    launch_dot(tptr(o.in[0]), tptr(o.in[1]), tptr(o.out[0]), B, o.a[0], o.a[1], o.a[2], o.a[3], o.a[4], o.a[5] != 0, s);
                    c.launches++;
                    break;
                case OP_ADAPTIVE_POOL:
                    launch_adaptive_pool(tptr(o.in[0]), tptr(o.out[0]), B, (int)o.a[0], (int)o.a[1], (int)o.a[2], (int)o.a[3], (int)o.a[4], (int)o.a[5],
                                         (int)o.a[6], o.a[7] != 0, s);
                    c.launches++;
                    break;
                case OP_LOOKUP:
                    launch_lookup((int)o.a[0], tptr(o.in[0]), tptr(o.out[0]), wptr(o.layer->w_main), B, o.a[2], (int)o.a[1], o.a[3] != 0, c.d_err, s);
                    c.launches++;
                    break;
                case OP_CONVLSTM_CELL:
                    launch_convlstm_cell(tptr(o.in[0]), o.in.size() > 1 ? tptr(o.in[1]) : nullptr, o.in.size() > 2 ? tptr(o.in[2]) : nullptr,
                                         tptr(o.out[0]), tptr(o.out[1]), B * o.a[0], (int)o.a[1], o.layer->act_main, o.layer->act_rec, s);
                    c.launches++;
                    break;
                case OP_EINSUM: {
                    EinsumGeom g;
                    g.n_out = (int)o.a[0]; g.n_sum = (int)o.a[1]; g.in_volume = o.a[2]; g.out_volume = o.a[3]; g.sum_volume = o.a[4];
                    size_t e = 0;
                    for (int l = 0; l < g.n_out; ++l) { g.out_size[l] = o.ext[e++]; g.out_in[l] = o.ext[e++]; g.out_k[l] = o.ext[e++]; g.out_b[l] = o.ext[e++]; }
                    for (int l = 0; l < g.n_sum; ++l) { g.sum_size[l] = o.ext[e++]; g.sum_in[l] = o.ext[e++]; g.sum_k[l] = o.ext[e++]; }
                    launch_einsum(tptr(o.in[0]), wptr(o.layer->w_main), wptr(o.layer->w_bias), tptr(o.out[0]), B, g, s);
                    c.launches++;
                    break;
                }
                case OP_PRELU: {
                    const TShape& sh = shape(o.in[0]);
                    launch_prelu(tptr(o.in[0]), tptr(o.out[0]), wptr(o.layer->w_main), B, (int)sh.d[2], (int)sh.d[3], (int)sh.d[4], o.a[0] != 0,
                                 o.a[1] != 0, o.a[2] != 0, s);
                    c.launches++;
                    break;
                }
                default: raise("internal: unknown op kind");
            }
        }
    }

    void conv(const Op& o) {
        const int H = (int)o.a[CONV_H], W = (int)o.a[CONV_W], C = (int)o.a[CONV_C], Ho = (int)o.a[CONV_HO], Wo = (int)o.a[CONV_WO];
        const int64_t M = B * Ho * Wo;
        const Epilogue e = epilogue(o, o.N);
        if (o.a[CONV_DIRECT]) {
            gemm(tptr(o.in[0]), C, o.w_main, o.ldw, tptr(o.out[0]), o.N, M, o.N, o.K, e);
            return;
        }
        if (o.a[CONV_IMPLICIT] || o.a[CONV_ROWWIN]) {
            ConvTcGeom g;
            g.B = B; g.H = H; g.W = W; g.C = C; g.pix = C; g.Ho = Ho; g.Wo = Wo;
            g.kh = (int)o.a[CONV_KH]; g.kw = (int)o.a[CONV_KW]; g.sy = (int)o.a[CONV_SY]; g.sx = (int)o.a[CONV_SX];
            g.dy = (int)o.a[CONV_DY]; g.dx = (int)o.a[CONV_DX]; g.pad_t = (int)o.a[CONV_PT]; g.pad_l = (int)o.a[CONV_PL];
            const float* in = tptr(o.in[0]);
            int w_id = o.w_main, ldw = o.ldw;
            if (o.a[CONV_ROWWIN]) {
                // zero-padded copy with the channels padded to a multiple of 4, then one k block per filter row
                const int hp = (int)o.a[CONV_RW_HP], wp = (int)o.a[CONV_RW_WP], cp = (int)o.a[CONV_RW_CP];
                float* padded = bptr(o.scratch[0]);
                launch_pad_channels(in, padded, B, H, W, C, hp, wp, cp, g.pad_t, g.pad_l, s);
                c.launches++;
                in = padded;
                g.H = hp; g.W = wp; g.C = cp; g.pix = cp;
                g.win_stride = (int64_t)g.sx * cp;
                w_id = o.layer->w_aux;
                ldw = g.kh * 32;
            }
            ensure(c.w.big_offset[(size_t)w_id] >= 0 && conv_tc_supported(g, o.N, ldw, in, wptr(w_id)),
                   "convolution '" + o.layer->name + "': the tensor-core path needs 16-byte aligned input tensors");
            Rec r;
            if (prof) {
                r = Rec{"gemm", o.layer->name, "tc", nullptr, nullptr, 2.0 * (double)M * o.N * o.K, M, o.N, o.K};
                rec_begin(r);
            }
            launch_conv_tc(in, g, c.w.base + c.w.big_offset[(size_t)w_id], c.w.base + c.w.small_offset[(size_t)w_id], ldw,
                           tptr(o.out[0]), o.N, o.N, e, s);
            if (prof) {
                FDK_CUDA(cudaEventRecord(r.b, s));
                prof->push_back(r);
            }
            c.launches++;
            return;
        }
        if (o.a[CONV_PHASES]) {
            // Transposed convolution without a patch matrix: the output positions with the same remainders modulo the
            // strides are a stride-1 convolution of the input with a sub-filter (model.hpp, transposed_phase); one
            // implicit-GEMM launch per phase writes every sy-th / sx-th output pixel.
            const Layer& L = *o.layer;
            const int sy = (int)o.a[CONV_SY], sx = (int)o.a[CONV_SX];
            const int lead_y = transposed_lead(L.k[1], sy, L.pad), lead_x = transposed_lead(L.k[2], sx, L.pad);
            float* out = tptr(o.out[0]);
            for (int py = 0; py < sy && py < Ho; ++py) for (int px = 0; px < sx && px < Wo; ++px) {
                const TransposedPhase ty = transposed_phase(L.k[1], sy, lead_y, py), tx = transposed_phase(L.k[2], sx, lead_x, px);
                const int w_id = L.w_phases[(size_t)(py * sx + px)];
                ConvTcGeom g;
                g.B = B; g.H = H; g.W = W; g.C = C; g.pix = C;
                g.Ho = (Ho - py + sy - 1) / sy; g.Wo = (Wo - px + sx - 1) / sx;
                g.kh = ty.taps; g.kw = tx.taps; g.pad_t = -ty.shift; g.pad_l = -tx.shift;
                g.out_sx = (int64_t)sx * o.N; g.out_sy = (int64_t)sy * Wo * o.N; g.out_sb = (int64_t)Ho * Wo * o.N;
                const int64_t first = ((int64_t)py * Wo + px) * o.N;
                const int kd = ty.taps * tx.taps * C;
                Epilogue ep = e;
                if (ep.residual) ep.residual += first;
                ensure(c.w.big_offset[(size_t)w_id] >= 0 && conv_tc_supported(g, o.N, kd, tptr(o.in[0]), wptr(w_id)),
                       "convolution '" + L.name + "': the tensor-core path needs 16-byte aligned input tensors");
                Rec r;
                if (prof) {
                    r = Rec{"gemm", L.name, "tc phase", nullptr, nullptr, 2.0 * (double)B * g.Ho * g.Wo * o.N * kd, B * g.Ho * g.Wo, o.N, kd};
                    rec_begin(r);
                }
                launch_conv_tc(tptr(o.in[0]), g, c.w.base + c.w.big_offset[(size_t)w_id], c.w.base + c.w.small_offset[(size_t)w_id], kd,
                               out + first, o.N, o.N, ep, s);
                if (prof) {
                    FDK_CUDA(cudaEventRecord(r.b, s));
                    prof->push_back(r);
                }
                c.launches++;
            }
            return;
        }
        float* col = bptr(o.scratch[0]);
        if (o.a[CONV_TRANSPOSED])
            launch_im2col_transposed(tptr(o.in[0]), col, B, H, W, C, Ho, Wo, (int)o.a[CONV_KH], (int)o.a[CONV_KW], (int)o.a[CONV_SY],
                                     (int)o.a[CONV_SX], (int)o.a[CONV_OFFY], (int)o.a[CONV_OFFX], (int)o.a[CONV_PT], (int)o.a[CONV_PL],
                                     (int)o.a[CONV_HD], (int)o.a[CONV_WD], o.ldw, s);
        else
            launch_im2col(tptr(o.in[0]), col, B, H, W, C, Ho, Wo, (int)o.a[CONV_KH], (int)o.a[CONV_KW], (int)o.a[CONV_SY], (int)o.a[CONV_SX],
                          (int)o.a[CONV_DY], (int)o.a[CONV_DX], (int)o.a[CONV_PT], (int)o.a[CONV_PL], o.ldw, s);
        c.launches++;
        gemm(col, o.ldw, o.w_main, o.ldw, tptr(o.out[0]), o.N, M, o.N, o.ldw, e);
    }

    void recurrent(const Op& o) {
        const Layer& L = *o.layer;
        const int64_t T = o.a[RNN_T], F = o.a[RNN_F];
        const int U = (int)o.a[RNN_U];
        const int g = o.kind == OP_LSTM ? 4 : o.kind == OP_GRU ? 3 : 1;
        const int gu = g * U;
        float* X = bptr(o.scratch[0]);
        float* z = bptr(o.scratch[1]);
        float* h = bptr(o.scratch[2]);
        float* c2 = bptr(o.scratch[3]);
        float* out = tptr(o.out[0]);
        // LSTM with the cell in the recurrent product's epilogue: one launch per time step, the gate pre-activations
        // stay on the SM.  Same arithmetic per value as the two-launch form below (bit-identical results), so the
        // choice may depend on the batch.  The new h goes to the other of two buffers (z's, unused in this form).
        const bool cell_fused = o.kind == OP_LSTM && fuse_cells && use_tc && !use_skinny && L.w_cell_rec >= 0 && B > 0 && T > 0 &&
                                c.w.big_offset[(size_t)L.w_cell_rec] >= 0 &&
                                lstm_step_tc_supported(B, U, h, wptr(L.w_cell_rec), L.kdim, X, T * gu, c2, z, out, L.flag_a ? T * U : U);
        Epilogue ex;
        ex.bias = wptr(cell_fused ? L.w_cell_bias : L.w_bias);
        gemm(tptr(o.in[0]), F, cell_fused ? L.w_cell_in : L.w_main, L.ldw, X, gu, B * T, gu, (int)F, ex);  // X = in W (+ b)
        FDK_CUDA(cudaMemsetAsync(h, 0, sizeof(float) * (size_t)(B * U), s));
        FDK_CUDA(cudaMemsetAsync(c2, 0, sizeof(float) * (size_t)(B * U), s));
        float* hc = h;
        float* hn = c2;  // SimpleRNN ping-pong
        // The time steps of rows [r0, r0 + nb) of the batch, queued on the executor's current stream.  h_in / h_out: where
        // this step reads and leaves the state ([B][U]; the same buffer except for SimpleRNN and the fused LSTM step).
        auto rows_step = [&](int64_t r0, int64_t nb, int64_t t, float* o_ptr, int64_t o_stride, float* h_in, float* h_out) {
            float* hr = h_in + r0 * U;
            float* zr = z + r0 * gu;
            float* cr = c2 + r0 * U;
            const float* xr = X + r0 * T * gu + t * gu;
            float* outr = o_ptr ? o_ptr + r0 * o_stride : nullptr;
            if (cell_fused) {
                Rec r;
                if (prof) {
                    r = Rec{"gemm", L.name, "tc+cell", nullptr, nullptr, 2.0 * (double)nb * gu * U, nb, gu, U};
                    rec_begin(r);
                }
                const int w = L.w_cell_rec;
                launch_lstm_step_tc(hr, c.w.base + c.w.big_offset[(size_t)w], c.w.base + c.w.small_offset[(size_t)w], L.kdim, xr, T * gu, cr,
                                    h_out + r0 * U, outr, o_stride, X, nb, U, s);
                if (prof) {
                    FDK_CUDA(cudaEventRecord(r.b, s));
                    prof->push_back(r);
                }
                c.launches++;
            } else if (o.kind == OP_LSTM) {
                Epilogue e;
                e.residual = xr;
                e.ldr = T * gu;
                gemm(hr, U, L.w_rec, L.kdim, zr, gu, nb, gu, U, e);  // z = x_t W + b + h U
                launch_lstm_cell(zr, cr, hr, outr, o_stride, nb, U, L.act_main, L.act_rec, s);
                c.launches++;
            } else if (o.kind == OP_GRU && !L.flag_c) {
                // reset_after = false: the candidate's recurrent product takes r .* h, so two products per step
                Epilogue e;
                gemm(hr, U, L.w_rec, L.kdim, zr, gu, nb, 2 * U, U, e);                     // h U_z | h U_r
                launch_gru_gates(xr, T * gu, zr, gu, hr, nb, U, L.act_rec, s);             // z | r .* h
                gemm(zr + U, gu, L.w_rec, L.kdim, zr + 2 * U, gu, nb, U, U, e, (int64_t)2 * U * L.kdim);  // (r .* h) U_h
                launch_gru_out(xr, T * gu, zr, gu, hr, outr, o_stride, nb, U, L.act_main, s);
                c.launches += 2;
            } else if (o.kind == OP_GRU) {
                Epilogue e;
                e.bias = wptr(L.w_rec_bias);
                gemm(hr, U, L.w_rec, L.kdim, zr, gu, nb, gu, U, e);  // h U + b_h
                launch_gru_cell(xr, T * gu, zr, hr, outr, o_stride, nb, U, L.act_main, L.act_rec, s);
                c.launches++;
            } else {
                Epilogue e;
                e.residual = xr;
                e.ldr = T * gu;
                e.act2 = L.act_main;
                gemm(hr, U, L.w_rec, L.kdim, h_out + r0 * U, U, nb, U, U, e);  // h' = act(x_t W + b + h U)
                if (outr) {
                    launch_slab_copy(h_out + r0 * U, outr, nb, U, o_stride, 0, s);
                    c.launches++;
                }
            }
        };
        // Two chains: the samples are independent, so the two halves of a large batch walk their time steps on two
        // streams.  A step of one half does not wait for the other half's step to drain: the second chain's CTAs take
        // the SMs that the last, partly filled wave of the first leaves idle (4096 x 2048 x 512 is 3.46 waves of tiles),
        // and a cell launch of one chain runs beside the product of the other.  Results per sample do not depend on
        // the batch they are computed in, so the split cannot change them.
        const bool two_chains = prof == nullptr && B >= 256 && c.aux_stream != nullptr && c.aux_stream != s;
        const int64_t first_rows = two_chains ? (B / 2 + 127) / 128 * 128 : B;
        cudaStream_t main_stream = s;
        if (two_chains) {
            FDK_CUDA(cudaEventRecord(c.fork_event, main_stream));
            FDK_CUDA(cudaStreamWaitEvent(c.aux_stream, c.fork_event, 0));
        }
        for (int64_t step = 0; step < T; ++step) {
            const int64_t t = L.reverse ? T - 1 - step : step;  // row of the sequence this step consumes
            float* o_ptr = nullptr;
            int64_t o_stride = 0;
            if (L.flag_a) { o_ptr = out + t * U; o_stride = T * U; }
            else if (step == T - 1) { o_ptr = out; o_stride = U; }
            float* h_in = hc;
            float* h_out = cell_fused ? (hc == h ? z : h) : (o.kind == OP_RNN ? hn : hc);
            try {
                rows_step(0, first_rows, t, o_ptr, o_stride, h_in, h_out);
                if (two_chains) {
                    s = c.aux_stream;
                    rows_step(first_rows, B - first_rows, t, o_ptr, o_stride, h_in, h_out);
                    s = main_stream;
                }
            } catch (...) {
                // nothing of the second chain may still run when the caller's stream goes on (or the arena is reused)
                s = main_stream;
                if (two_chains) cudaStreamSynchronize(c.aux_stream);
                throw;
            }
            if (cell_fused) hc = h_out;
            else if (o.kind == OP_RNN) std::swap(hc, hn);
        }
        if (two_chains) {
            FDK_CUDA(cudaEventRecord(c.join_event, c.aux_stream));
            FDK_CUDA(cudaStreamWaitEvent(main_stream, c.join_event, 0));
        }
        if (T == 0) raise("recurrent layer needs at least one timestep");
        if (L.flag_b) {
            const float* hf = (o.kind == OP_RNN || cell_fused) ? hc : h;
            FDK_CUDA(cudaMemcpyAsync(tptr(o.out[1]), hf, sizeof(float) * (size_t)(B * U), cudaMemcpyDeviceToDevice, s));
            if (o.kind == OP_LSTM) FDK_CUDA(cudaMemcpyAsync(tptr(o.out[2]), c2, sizeof(float) * (size_t)(B * U), cudaMemcpyDeviceToDevice, s));
        }
    }

    void mha(const Op& o) {
        const Layer& L = *o.layer;
        const int64_t Tq = o.a[MHA_TQ], Tk = o.a[MHA_TK];
        const int H = L.heads, dk = L.key_dim, dv = L.value_dim, dim = L.in_feat;
        float* Q = bptr(o.scratch[0]);
        float* K = bptr(o.scratch[1]);
        float* V = bptr(o.scratch[2]);
        float* A = bptr(o.scratch[3]);
        const float* q_in = tptr(o.in[0]);
        const float* v_in = tptr(o.in[1]);
        const float* k_in = o.in.size() > 2 ? tptr(o.in[2]) : v_in;
        Epilogue eq, ek, ev, eo;
        eq.bias = wptr(L.b_q); ek.bias = wptr(L.b_k); ev.bias = wptr(L.b_v); eo.bias = wptr(L.b_o);
        if (o.residual >= 0) { eo.residual = tptr(o.residual); eo.ldr = L.out_dim; }  // a following Add, folded by the plan compiler
        if (kv) {
            // project only the new row of every sample, straight into the cache at row kv->len; attend over the cache
            const int blk = kvi.block_of_op[(size_t)cur_index];
            const float* x_new = tptr(kvi.x_tensor[(size_t)blk]);
            const int64_t HK = (int64_t)H * dk, HV = (int64_t)H * dv;
            // a folded LayerNormalization: the projections read the un-normalised rows and normalise them themselves
            const int nf = norm_of_op[(size_t)cur_index];
            RowsNorm np;
            const float* x_raw = nullptr;
            if (nf >= 0) { np = norm_params(p.ops[(size_t)nf]); x_raw = tptr(p.ops[(size_t)nf].in[0]); }
            float* Kc = kv->k + (int64_t)blk * kv->k_block_stride;
            float* Vc = kv->v + (int64_t)blk * kv->v_block_stride;
            // the three projections: one launch when they share rows and shape, else one each
            auto project = [&](float* Kd, int64_t ldK, float* Vd, int64_t ldV) {
                const int w3[3] = {L.w_q, L.w_k, L.w_v}, b3[3] = {L.b_q, L.b_k, L.b_v};
                float* const c3[3] = {Q, Kd, Vd};
                const int64_t l3[3] = {(int64_t)H * dk, ldK, ldV};
                if (nf >= 0) {
                    gemm_skinny_three(x_raw, dim, w3, L.ldw, c3, l3, b3, B, (int)HK, dim, &np);
                    return;
                }
                if (q_in == x_new && HK == HV && gemm_skinny_three(x_new, dim, w3, L.ldw, c3, l3, b3, B, (int)HK, dim)) return;
                gemm(q_in, dim, L.w_q, L.ldw, Q, H * dk, B, H * dk, dim, eq);
                gemm(x_new, dim, L.w_k, L.ldw, Kd, ldK, B, (int)HK, dim, ek);
                gemm(x_new, dim, L.w_v, L.ldw, Vd, ldV, B, (int)HV, dim, ev);
            };
            if (kv->len_dev) {
                // length on the device: this position's rows go to the scratch, the attention kernel moves them into the cache
                project(K, HK, V, HV);
                AttnExtra x;
                x.len_ptr = kv->len_dev;
                x.k_new = K;
                x.v_new = V;
                const float scale = (float)(1.0 / std::sqrt((double)dk));
                launch_attention(Q, H * dk, H * dk, Kc, HK, kv->max_len * HK, Vc, HV, kv->max_len * HV, A, H * dv, H * dv, B, H, 1, (int)kv->max_len, dk,
                                 dv, scale, s, x);
                c.launches++;
                gemm(A, H * dv, L.w_o, L.kdim, tptr(o.out[0]), L.out_dim, B, L.out_dim, H * dv, eo);
                return;
            }
            ensure(Tk == kv->len + 1 && kv->len < kv->max_len, "key/value cache: the plan's key length does not match the cache");
            project(Kc + kv->len * HK, kv->max_len * HK, Vc + kv->len * HV, kv->max_len * HV);
            const float scale = (float)(1.0 / std::sqrt((double)dk));
            launch_attention(Q, H * dk, H * dk, Kc, HK, kv->max_len * HK, Vc, HV, kv->max_len * HV, A, H * dv, H * dv, B, H, 1, (int)Tk, dk, dv,
                             scale, s);
            c.launches++;
            gemm(A, H * dv, L.w_o, L.kdim, tptr(o.out[0]), L.out_dim, B, L.out_dim, H * dv, eo);
            return;
        }
        // grouped queries (group_query_attention_layer.hpp:125-150): Hk key/value heads serve H query heads
        const int Hk = L.kv_heads ? L.kv_heads : H;
        AttnExtra x;
        x.group = H / Hk;
        gemm(q_in, dim, L.w_q, L.ldw, Q, H * dk, B * Tq, H * dk, dim, eq);
        gemm(k_in, dim, L.w_k, L.ldw, K, Hk * dk, B * Tk, Hk * dk, dim, ek);
        gemm(v_in, dim, L.w_v, L.ldw, V, Hk * dv, B * Tk, Hk * dv, dim, ev);
        if (L.w_g >= 0) {
            float* G = bptr(o.scratch[4]);
            Epilogue eg;
            eg.bias = wptr(L.b_g);
            gemm(q_in, dim, L.w_g, L.ldw, G, H * dv, B * Tq, H * dv, dim, eg);
            x.gate = G;
        }
        const float scale = (float)(1.0 / std::sqrt((double)dk));  // multi_head_attention_layer.hpp:92-93
        launch_attention(Q, H * dk, Tq * H * dk, K, Hk * dk, Tk * Hk * dk, V, Hk * dv, Tk * Hk * dv, A, H * dv, Tq * H * dv, B, H, (int)Tq, (int)Tk,
                         dk, dv, scale, s, x);
        c.launches++;
        gemm(A, H * dv, L.w_o, L.kdim, tptr(o.out[0]), L.out_dim, B * Tq, L.out_dim, H * dv, eo);
    }
};
}  // namespace

void Engine::execute(DeviceCtx& c, const Plan& p, int64_t B, const float* const* d_in, cudaStream_t s, std::string* profile, const KvCache* kv,
                     const std::vector<char>* wanted) {
    ensure_arena(c, std::max<int64_t>(p.arena_elems, 64) * B);
    Exec ex{*this, c, p, B, d_in, s, opt_.use_tc};
    ex.use_skinny = opt_.skinny;
    ex.fuse_cells = opt_.fuse_cells;
    ex.kv = kv;
    ex.wanted = wanted;
    std::vector<Exec::Rec> recs;
    if (profile) ex.prof = &recs;
    ex.run();
    if (profile) {
        FDK_CUDA(cudaStreamSynchronize(s));
        for (auto& r : recs) {
            float ms = 0.f;
            FDK_CUDA(cudaEventElapsedTime(&ms, r.a, r.b));
            *profile += r.kind + " " + r.name + " " + std::to_string(ms) + " " + std::to_string(r.flops) + " " + std::to_string(r.M) + " " +
                        std::to_string(r.N) + " " + std::to_string(r.K) + " " + r.path + "\n";
            cudaEventDestroy(r.a);
            cudaEventDestroy(r.b);
        }
    }
}

std::string Engine::profile_batch_device(int dev_index, int64_t batch, const float* const* d_in, const std::vector<TShape>& in_shapes) {
    ensure(dev_index >= 0 && dev_index < (int)ctx_.size(), "invalid device index");
    ensure(batch > 0, "batch must be positive");
    DeviceCtx& c = *ctx_[(size_t)dev_index];
    std::lock_guard<std::mutex> lk(c.mu);
    DeviceGuard g(c.device);
    auto p = get_plan(in_shapes);
    std::string text;
    order_after_last_use(c, c.stream);
    execute(c, *p, batch, d_in, c.stream, &text);
    mark_use(c, c.stream);
    return text;
}

std::vector<AttentionBlockInfo> Engine::attention_blocks(const std::vector<TShape>& in_shapes) {
    auto p = get_plan(in_shapes);
    const KvPlanInfo info = analyse_attention(*p);
    std::vector<AttentionBlockInfo> r;
    for (size_t i = 0; i < p->ops.size(); ++i) {
        const int blk = info.block_of_op[i];
        if (blk < 0) continue;
        const Layer& L = *p->ops[i].layer;
        AttentionBlockInfo a;
        a.key_width = L.heads * L.key_dim;
        a.value_width = L.heads * L.value_dim;
        a.cacheable = info.cacheable[(size_t)blk] != 0;
        r.push_back(a);
    }
    return r;
}

void Engine::predict_batch_device(int dev_index, int64_t batch, const float* const* d_in, const std::vector<TShape>& in_shapes,
                                  float* const* d_out, cudaStream_t stream, const KvCache* kv, std::string* profile) {
    ensure(dev_index >= 0 && dev_index < (int)ctx_.size(), "invalid device index");
    ensure(batch > 0, "batch must be positive");
    DeviceCtx& c = *ctx_[(size_t)dev_index];
    std::lock_guard<std::mutex> lk(c.mu);
    DeviceGuard g(c.device);
    auto p = get_plan(in_shapes);
    cudaStream_t s = stream ? stream : c.stream;
    // A stream that is being captured (a decode session recording a position) takes no event: the session orders
    // the replays itself.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    FDK_CUDA(cudaStreamIsCapturing(s, &cap));
    const bool live = cap == cudaStreamCaptureStatusNone;
    if (live) order_after_last_use(c, s);
    std::vector<char> wanted(p->outputs.size(), 1);
    for (size_t o = 0; o < p->outputs.size(); ++o) wanted[o] = d_out[o] != nullptr ? 1 : 0;
    execute(c, *p, batch, d_in, s, profile, kv, &wanted);
    for (size_t o = 0; o < p->outputs.size(); ++o) {
        const TensorInfo& t = p->tensors[(size_t)p->outputs[o]];
        const BufferInfo& b = p->buffers[(size_t)t.buf];
        const float* src = b.ext_input >= 0 ? d_in[b.ext_input] : c.arena + b.offset * batch;
        if (!d_out[o]) continue;  // output not wanted
        FDK_CUDA(cudaMemcpyAsync(d_out[o], src, sizeof(float) * (size_t)(batch * t.shape.volume()), cudaMemcpyDeviceToDevice, s));
    }
    if (live) mark_use(c, s);
}

void Engine::run_block(DeviceCtx& c, const Plan& p, const std::vector<int64_t>& ids, const float* const* in_ptrs, float* const* out_ptrs,
                       const ByteScale* bytes) {
    // byte inputs: the pointers are uint8_t arrays; they travel as bytes and become floats on the device
    const size_t esz = bytes ? 1 : sizeof(float);
    std::lock_guard<std::mutex> lk(c.mu);
    DeviceGuard g(c.device);
    const size_t n_in = p.inputs.size(), n_out = p.outputs.size();
    std::vector<int64_t> in_e(n_in), out_e(n_out);
    int64_t in_total = 0, out_total = 0;
    for (size_t i = 0; i < n_in; ++i) { in_e[i] = p.in_shapes[i].volume(); in_total += round_up64(in_e[i], 64); }
    for (size_t o = 0; o < n_out; ++o) { out_e[o] = p.tensors[(size_t)p.outputs[o]].shape.volume(); out_total += round_up64(out_e[o], 64); }
    int dev_index = 0;
    for (size_t i = 0; i < ctx_.size(); ++i) if (ctx_[i].get() == &c) dev_index = (int)i;
    const int64_t maxB = max_batch_for(p.in_shapes, dev_index);
    order_after_last_use(c, c.stream);
    for (size_t start = 0; start < ids.size(); start += (size_t)maxB) {
        const int64_t nb = (int64_t)std::min<size_t>((size_t)maxB, ids.size() - start);
        // staging
        if (c.h_in_elems < nb * in_total) {
            FDK_CUDA(cudaStreamSynchronize(c.stream));
            if (c.h_in) FDK_CUDA(cudaFreeHost(c.h_in));
            c.h_in = nullptr; c.h_in_elems = 0;
            FDK_CUDA(cudaMallocHost(&c.h_in, sizeof(float) * (size_t)(nb * in_total)));
            c.h_in_elems = nb * in_total;
        }
        if (c.in_stage_elems < nb * in_total) {
            FDK_CUDA(cudaStreamSynchronize(c.stream));
            if (c.in_stage) FDK_CUDA(cudaFree(c.in_stage));
            c.in_stage = nullptr; c.in_stage_elems = 0;
            FDK_CUDA(cudaMalloc(&c.in_stage, sizeof(float) * (size_t)(nb * in_total)));
            c.in_stage_elems = nb * in_total;
        }
        if (bytes && c.byte_stage_bytes < nb * in_total) {
            FDK_CUDA(cudaStreamSynchronize(c.stream));
            FDK_CUDA(cudaStreamSynchronize(c.copy_stream));
            if (c.byte_stage) FDK_CUDA(cudaFree(c.byte_stage));
            c.byte_stage = nullptr; c.byte_stage_bytes = 0;
            FDK_CUDA(cudaMalloc(&c.byte_stage, (size_t)(nb * in_total)));
            c.byte_stage_bytes = nb * in_total;
        }
        if (c.h_out_elems < nb * out_total) {
            FDK_CUDA(cudaStreamSynchronize(c.stream));
            if (c.h_out) FDK_CUDA(cudaFreeHost(c.h_out));
            c.h_out = nullptr; c.h_out_elems = 0;
            FDK_CUDA(cudaMallocHost(&c.h_out, sizeof(float) * (size_t)(nb * out_total)));
            c.h_out_elems = nb * out_total;
        }
        // Large blocks go through in a few chunks: the host-to-device copy of a chunk runs on the copy stream while
        // the compute stream works on the chunk before it.  (Chunks are kept large: a chunk of a few images leaves
        // most SMs idle in the late layers.)
        int64_t in_bytes = 0;
        for (size_t i = 0; i < n_in; ++i) in_bytes += nb * in_e[i] * (int64_t)esz;
        // Chunk plan.  Only the first chunk's copy is exposed if every later chunk's copy ends before the work on the
        // chunk before it does, i.e. if chunks grow by at most r = (compute time per sample) / (copy time per sample);
        // every chunk costs something (driver calls, late layers with fewer tiles), so the number of chunks grows only
        // while one more still shortens the exposed copy by more than that.  Both times are estimates: contraction FLOPs
        // at 150 TFLOP/s or twice the layer outputs at 3 TB/s, whichever is longer, and 45 GB/s from host memory.
        // ResNet-50, 256 float images (r = 3.8: a quarter, then the rest), images/s end to end with the chunks in the ratio
        // 1:1 17.5 k, 1:2 18.4 k, 1:3 19.0 k, 1:4 18.7 k, 1:5 18.9 k, 1:7 18.6 k, 2:5 18.9 k, 1:2:3 18.2 k, 1:3:4 18.7 k,
        // 1:1:1:1 17.1 k.
        std::vector<double> weights(1, 1.0);
        if (nb >= 128 && in_bytes >= (8 << 20)) {
            double out_bytes = 0;
            for (const Op& o : p.ops)
                if (!o.dead) for (int t : o.out) out_bytes += 4.0 * (double)p.tensors[(size_t)t].shape.volume();
            const double t_compute = std::max(p.flops_per_sample / 150e12, 2.0 * out_bytes / 3.0e12);
            const double t_copy = (double)in_bytes / (double)nb / 45e9;
            const double g = std::min(4.0, std::max(1.0, t_compute / t_copy));
            auto first_share = [&](int n) {  // first chunk's share of the block with n chunks growing by g
                double sum = 0, w = 1;
                for (int i = 0; i < n; ++i) { sum += w; w *= g; }
                return 1.0 / sum;
            };
            int n = 1;
            while (n < 6) {
                const double now = first_share(n) * (double)nb, next = first_share(n + 1) * (double)nb;
                if (next < 32.0 || (now - next) * t_copy < 0.3e-3) break;
                ++n;
            }
            weights.assign(1, 1.0);
            for (int i = 1; i < n; ++i) weights.push_back(weights.back() * g);
        }
        const int n_chunks = (int)weights.size();
        std::vector<int64_t> bounds(1, 0);  // chunk ch covers samples [bounds[ch], bounds[ch + 1])
        {
            double total_w = 0, acc_w = 0;
            for (double w : weights) total_w += w;
            // chunk ends rounded up to whole groups of 64 samples (tiles of the late layers hold several samples)
            for (double w : weights) {
                acc_w += w;
                const int64_t end = ((int64_t)std::llround((double)nb * acc_w / total_w) + 63) / 64 * 64;
                bounds.push_back(std::max(bounds.back(), std::min<int64_t>(nb, end)));
            }
            bounds.back() = nb;
        }
        std::vector<cudaEvent_t> landed((size_t)n_chunks, nullptr);
        std::vector<char> direct(n_out, 0);  // output o goes straight into the caller's (contiguous) memory
        for (size_t o = 0; o < n_out; ++o) {
            float* first = out_ptrs[(size_t)ids[start] * n_out + o];
            bool contiguous = true;
            for (int64_t k = 1; k < nb && contiguous; ++k)
                contiguous = out_ptrs[(size_t)ids[start + (size_t)k] * n_out + o] == first + k * out_e[o];
            // Only when the block goes through in one piece: a copy into pageable caller memory returns when it is
            // done, which would hold the host back from queueing the next chunk.
            direct[o] = (contiguous && n_chunks == 1) ? 1 : 0;
        }
        FDK_CUDA(cudaMemsetAsync(c.d_err, 0, sizeof(int), c.stream));
        int64_t off = 0;                       // running offset into the input staging buffers (floats)
        std::vector<int64_t> ooffs(n_out);     // offsets of the outputs in h_out: [output][sample] over the whole block
        {
            int64_t ooff = 0;
            for (size_t o = 0; o < n_out; ++o) { ooffs[o] = ooff; ooff += round_up64(nb * out_e[o], 64); }
        }
        try {
            for (int ch = 0; ch < n_chunks; ++ch) {
                const int64_t k0 = bounds[(size_t)ch], k1 = bounds[(size_t)ch + 1], cnb = k1 - k0;
                if (cnb == 0) continue;
                cudaStream_t cs = n_chunks > 1 ? c.copy_stream : c.stream;
                std::vector<const float*> d_in(n_in);
                for (size_t i = 0; i < n_in; ++i) {
                    d_in[i] = c.in_stage + off;
                    auto sample_ptr = [&](int64_t k) { return reinterpret_cast<const char*>(in_ptrs[(size_t)ids[start + (size_t)(k0 + k)] * n_in + i]); };
                    const char* first = sample_ptr(0);
                    bool contiguous = true;  // the samples lie back to back in the caller's memory (a batch array)
                    for (int64_t k = 1; k < cnb && contiguous; ++k) contiguous = sample_ptr(k) == first + (size_t)(k * in_e[i]) * esz;
                    const size_t n_bytes = esz * (size_t)(cnb * in_e[i]);
                    // where the copy lands: the float staging itself, or (byte inputs) the byte staging at the same offset
                    void* d_dst = bytes ? (void*)(c.byte_stage + off) : (void*)(c.in_stage + off);
                    if (contiguous) {
                        // straight from the caller's buffer (a true DMA if it is pinned; the driver stages pageable memory)
                        FDK_CUDA(cudaMemcpyAsync(d_dst, first, n_bytes, cudaMemcpyHostToDevice, cs));
                        count_transfer(true, n_bytes);
                    } else {
                        // gather the samples into the pinned staging buffer, with a few threads when there is much to move
                        char* dst = reinterpret_cast<char*>(c.h_in) + (size_t)off * esz;
                        const int n_thr = n_bytes > (size_t)(8 << 20) ? (int)std::min<int64_t>(8, cnb) : 1;
                        auto gather = [&](int64_t a0, int64_t a1) {
                            for (int64_t k = a0; k < a1; ++k) std::memcpy(dst + (size_t)(k * in_e[i]) * esz, sample_ptr(k), esz * (size_t)in_e[i]);
                        };
                        if (n_thr == 1) {
                            gather(0, cnb);
                        } else {
                            std::vector<std::thread> thr;
                            for (int t = 0; t < n_thr; ++t) thr.emplace_back(gather, cnb * t / n_thr, cnb * (t + 1) / n_thr);
                            for (auto& t : thr) t.join();
                        }
                        FDK_CUDA(cudaMemcpyAsync(d_dst, dst, n_bytes, cudaMemcpyHostToDevice, cs));
                        count_transfer(true, n_bytes);
                    }
                    if (bytes) launch_bytes_to_float(c.byte_stage + off, c.in_stage + off, cnb * in_e[i], bytes->low, bytes->high, cs);
                    off += round_up64(cnb * in_e[i], 64);
                }
                if (n_chunks > 1) {
                    FDK_CUDA(cudaEventCreateWithFlags(&landed[(size_t)ch], cudaEventDisableTiming));
                    FDK_CUDA(cudaEventRecord(landed[(size_t)ch], cs));
                    FDK_CUDA(cudaStreamWaitEvent(c.stream, landed[(size_t)ch], 0));
                }
                execute(c, p, cnb, d_in.data(), c.stream);
                // results of the chunk leave the arena before the next chunk overwrites it (same stream)
                for (size_t o = 0; o < n_out; ++o) {
                    const TensorInfo& t = p.tensors[(size_t)p.outputs[o]];
                    const BufferInfo& b = p.buffers[(size_t)t.buf];
                    const float* src = b.ext_input >= 0 ? d_in[(size_t)b.ext_input] : c.arena + b.offset * cnb;
                    float* dst = direct[o] ? out_ptrs[(size_t)ids[start] * n_out + o] + k0 * out_e[o] : c.h_out + ooffs[o] + k0 * out_e[o];
                    FDK_CUDA(cudaMemcpyAsync(dst, src, sizeof(float) * (size_t)(cnb * out_e[o]), cudaMemcpyDeviceToHost, c.stream));
                    count_transfer(false, sizeof(float) * (size_t)(cnb * out_e[o]));
                }
            }
            FDK_CUDA(cudaMemcpyAsync(c.h_err, c.d_err, sizeof(int), cudaMemcpyDeviceToHost, c.stream));
            FDK_CUDA(cudaStreamSynchronize(c.stream));
            c.busy_valid = false;  // this stream waited for the last user and has finished itself: nothing is in flight
        } catch (...) {
            cudaStreamSynchronize(c.copy_stream);
            cudaStreamSynchronize(c.stream);
            for (cudaEvent_t e : landed) if (e) cudaEventDestroy(e);
            throw;
        }
        for (cudaEvent_t e : landed) if (e) cudaEventDestroy(e);
        if (*c.h_err != 0) raise(input_error_text(*c.h_err));
        const int st = gemm_tc_take_status(c.stream);
        if (st != 0) raise("tensor-core contraction kernel gave up waiting on a barrier (status " + std::to_string(st) + ")");
        for (size_t o = 0; o < n_out; ++o) {
            if (direct[o]) continue;
            for (int64_t k = 0; k < nb; ++k)
                std::memcpy(out_ptrs[(size_t)ids[start + (size_t)k] * n_out + o], c.h_out + ooffs[o] + k * out_e[o], sizeof(float) * (size_t)out_e[o]);
        }
    }
}

void Engine::predict_multi(int64_t n_samples, const float* const* in_ptrs, const TShape* in_shapes, float* const* out_ptrs, const ByteScale* bytes) {
    if (n_samples <= 0) return;
    const size_t n_in = lm_.input_shapes.size();
    // group by shape signature, keeping input order inside each group
    std::vector<std::pair<std::string, std::vector<int64_t>>> groups;
    std::map<std::string, size_t> gi;
    for (int64_t sidx = 0; sidx < n_samples; ++sidx) {
        std::vector<TShape> sh(in_shapes + sidx * (int64_t)n_in, in_shapes + (sidx + 1) * (int64_t)n_in);
        const std::string key = signature(sh);
        auto it = gi.find(key);
        if (it == gi.end()) { gi[key] = groups.size(); groups.emplace_back(key, std::vector<int64_t>{sidx}); }
        else groups[it->second].second.push_back(sidx);
    }
    for (auto& gr : groups) {
        const std::vector<int64_t>& ids = gr.second;
        std::vector<TShape> sh(in_shapes + ids[0] * (int64_t)n_in, in_shapes + (ids[0] + 1) * (int64_t)n_in);
        auto plan = get_plan(sh);
        const size_t nd = std::min(ctx_.size(), ids.size());
        if (nd <= 1) {
            run_block(*ctx_[0], *plan, ids, in_ptrs, out_ptrs, bytes);
            continue;
        }
        // contiguous blocks of ceil(n / G) samples per device, one host thread per device
        std::vector<std::thread> th;
        std::vector<std::string> errs(nd);
        for (size_t d = 0; d < nd; ++d) {
            int64_t blo = 0, bhi = 0;
            shard_block((int64_t)ids.size(), (int)nd, (int)d, blo, bhi);
            const size_t lo = (size_t)blo, hi = (size_t)bhi;
            if (lo >= hi) continue;
            th.emplace_back([&, d, lo, hi]() {
                try {
                    std::vector<int64_t> part(ids.begin() + (long)lo, ids.begin() + (long)hi);
                    run_block(*ctx_[d], *plan, part, in_ptrs, out_ptrs, bytes);
                } catch (const std::exception& e) {
                    errs[d] = e.what();
                    if (errs[d].empty()) errs[d] = "error";
                } catch (...) {
                    errs[d] = "unknown error on device " + std::to_string(ctx_[d]->device);
                }
            });
        }
        for (auto& t : th) t.join();
        for (const auto& e : errs) if (!e.empty()) raise(e);
    }
}

void Engine::run_tests(float eps) {
    // model.hpp:254-267 and check_test_outputs (import_model.hpp:1990-2021): absolute tolerance, NaN == NaN
    const size_t n_in = lm_.input_shapes.size();
    for (size_t t = 0; t < lm_.tests.size(); ++t) {
        const TestCase& tc = lm_.tests[t];
        ensure(tc.in_shapes.size() == n_in, "invalid number of test inputs");
        const std::vector<TShape> outs = infer(tc.in_shapes);
        ensure(outs.size() == tc.out_shapes.size(), "invalid output count");
        std::vector<const float*> ip;
        for (const auto& v : tc.in_values) ip.push_back(v.data());
        std::vector<std::vector<float>> res(outs.size());
        std::vector<float*> op;
        for (size_t o = 0; o < outs.size(); ++o) { res[o].resize((size_t)outs[o].volume()); op.push_back(res[o].data()); }
        predict_multi(1, ip.data(), tc.in_shapes.data(), op.data());
        for (size_t o = 0; o < outs.size(); ++o) {
            if (outs[o] != tc.out_shapes[o])
                raise("test failed: output=" + std::to_string(o) + " Wrong output size. Is " + outs[o].str() + ", should be " + tc.out_shapes[o].str() + ".");
            const TShape& s = outs[o];
            for (int64_t k = 0; k < s.volume(); ++k) {
                const float a = res[o][(size_t)k], b = tc.out_values[o][(size_t)k];
                if (!(std::fabs(a - b) <= eps) && !(std::isnan(a) && std::isnan(b))) {
                    const int64_t z = k % s.d[4], x = (k / s.d[4]) % s.d[3], y = (k / (s.d[4] * s.d[3])) % s.d[2];
                    raise("test failed: output=" + std::to_string(o) + " pos=" + std::to_string(y) + "," + std::to_string(x) + "," + std::to_string(z) +
                          " value=" + std::to_string(a) + " target=" + std::to_string(b));
                }
            }
        }
    }
}

}  // namespace fdk
