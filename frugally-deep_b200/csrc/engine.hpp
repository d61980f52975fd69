// Plan compiler and executor.
//
// The reference evaluates a model by a lazy, memoised pull through layer objects on every predict
// (model_layer.hpp:51-66, layer.hpp:63-80, node.hpp:66-74).  Here the same traversal runs once per
// input-shape signature at plan time and yields a static list of device operations with fused
// epilogues and a liveness-based memory plan; predict then only launches kernels.
#pragma once

#include "common.hpp"
#include "model.hpp"

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace fdk {

enum OpKind : int {
    OP_CONV, OP_GEMM, OP_DWCONV, OP_POOL, OP_GPOOL, OP_BINARY, OP_UNARY, OP_AFFINE, OP_SOFTMAX, OP_NORM,
    OP_WINDOW, OP_CONCAT, OP_PERMUTE, OP_EMBED, OP_LSTM, OP_GRU, OP_RNN, OP_MHA, OP_COPY, OP_ATTN, OP_PRELU, OP_EINSUM, OP_CONV3D, OP_NORMALIZE, OP_UPSAMPLE,
    OP_RESIZE, OP_DOT, OP_ADAPTIVE_POOL, OP_LOOKUP, OP_CONVLSTM_CELL
};

struct TensorInfo {
    TShape shape;
    int buf = -1;
};

struct BufferInfo {
    int64_t elems = 0;        // per sample
    int64_t offset = -1;      // per-sample offset in floats inside the arena (multiplied by the batch at run time)
    int ext_input = -1;       // >= 0: bound to model input i, no arena storage
    int first = -1, last = -1;
    bool pinned_to_end = false;  // model outputs stay alive until the end
};

struct Op {
    int kind = OP_COPY;
    const Layer* layer = nullptr;
    std::vector<int> in, out;   // tensor ids
    std::vector<int> scratch;   // buffer ids
    // fused epilogue (OP_CONV / OP_GEMM / OP_DWCONV)
    int stage = 0;
    int w_bias = -1, w_scale = -1, w_shift = -1;
    ActSpec act1, act2;
    int residual = -1;  // tensor id
    // generic attributes
    int64_t a[32] = {0};
    std::vector<int64_t> ext;   // OP_EINSUM: per output letter (size, input, kernel, bias stride), then per summed letter (size, input, kernel stride)
    float f[4] = {0, 0, 0, 0};
    ActSpec act;
    // OP_GEMM operands
    int w_main = -1, ldw = 0, K = 0, N = 0;
    bool dead = false;
};

struct Plan {
    std::vector<TShape> in_shapes;
    std::vector<TensorInfo> tensors;
    std::vector<BufferInfo> buffers;
    std::vector<Op> ops;
    std::vector<int> inputs, outputs;  // tensor ids
    int64_t arena_elems = 0;           // per sample
    double flops_per_sample = 0;       // contraction FLOPs (2*MACs), for reporting
};

struct DeviceWeights {
    float* base = nullptr;
    std::vector<int64_t> offset;        // floats
    std::vector<int64_t> big_offset;    // TF32 high halves (gemm weights) or -1
    std::vector<int64_t> small_offset;  // TF32 low halves or -1
};

struct DeviceCtx {
    uint8_t* byte_stage = nullptr;   // device staging for byte inputs
    int64_t byte_stage_bytes = 0;
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;  // host-to-device copies of the chunks of a large block
    // second chain of a recurrent layer on a large batch (forked from and joined to the stream of the call)
    cudaStream_t aux_stream = nullptr;
    cudaEvent_t fork_event = nullptr, join_event = nullptr;
    DeviceWeights w;
    float* arena = nullptr;
    int64_t arena_elems = 0;
    float* in_stage = nullptr;     // device staging for host inputs
    int64_t in_stage_elems = 0;
    float* h_in = nullptr;         // pinned host staging
    int64_t h_in_elems = 0;
    float* h_out = nullptr;
    int64_t h_out_elems = 0;
    float* workspace = nullptr;    // partial tiles of split-K products
    int64_t workspace_elems = 0;
    int* d_err = nullptr;          // device error flag (embedding range)
    int* h_err = nullptr;          // pinned
    std::mutex mu;                 // held while a call queues its work on this device
    // Order between calls that use the arena / workspace from different streams: the last use recorded `busy` on
    // `busy_stream`; the next use on another stream waits for it (Engine::order_after_last_use / mark_use).
    cudaEvent_t busy = nullptr;
    cudaStream_t busy_stream = nullptr;
    bool busy_valid = false;
    int64_t launches = 0;          // kernels launched by this context
};

// Key/value cache of a decode session.  It serves the attention operations of a plan whose key/value input is either
// Concatenate([past, x]) with `past` a model input (a later position) or x itself (the first position), one query
// row per sample: the projected key and value rows of x are written into the cache at row `len`, the concatenation
// is skipped, and the attention reads rows 0 .. len of the cache.
struct KvCache {
    float* k = nullptr;            // [blocks][batch][max_len][heads * key_dim]
    float* v = nullptr;            // [blocks][batch][max_len][heads * value_dim]
    int64_t max_len = 0;
    int64_t len = 0;               // rows already in the cache
    // When set, the length is read on the device from this counter instead (the host value above is not used): the
    // launches of a position then do not depend on the position and can be replayed from a CUDA graph.  The plan may
    // be the one of any key length; the attention kernel takes the new key/value rows from the plan's scratch and
    // stores them into the cache itself.
    const int* len_dev = nullptr;
    int64_t k_block_stride = 0;    // floats between the caches of consecutive attention operations
    int64_t v_block_stride = 0;
};
struct AttentionBlockInfo {
    int key_width = 0, value_width = 0;   // heads * key_dim, heads * value_dim
    bool cacheable = false;
};

struct EngineOptions {
    bool use_tc = true;            // tcgen05 contraction path where supported
    bool skinny = false;           // products with <= 64 rows take the weight-streaming split-K kernel (results then differ
                                   // in the last bits between batches of <= 64 and > 64 rows: off unless asked for)
    bool fuse_cells = false;       // LSTM: finish the cell in the recurrent product's epilogue (same results, measured slower)
    int64_t max_batch = 0;         // 0 = derive from memory
    double mem_fraction = 0.5;     // share of free device memory the arena may take
};

// Compiles the plan for one input-shape signature.  Host only: needs no CUDA device.
std::shared_ptr<Plan> compile_plan(const LoadedModel& lm, const EngineOptions& opt, const std::vector<TShape>& in_shapes);
// Sample range [begin, end) of part `part` when n_samples independent samples are split in contiguous
// blocks of ceil(n / parts) over devices or ranks (predict_multi keeps the input order, model.hpp:31-42).
void shard_block(int64_t n_samples, int n_parts, int part, int64_t& begin, int64_t& end);
// Human-readable listing of a plan (one line per operation), used by tests and for debugging.
std::string describe_plan(const Plan& p);

// Message for a non-zero device-side input check flag (1: embedding index, 2: category encoding value).
std::string input_error_text(int code);

// Bytes copied between host and device memory by this library (process-wide counters, for callers that want to
// check that a chain of models stayed on the device).
void count_transfer(bool host_to_device, uint64_t bytes);
void transfer_totals(uint64_t& host_to_device, uint64_t& device_to_host);

// Inputs given as bytes: every input pointer is a uint8_t array that becomes floats on the device by
// tensor_from_bytes' rule (tensor.hpp:1230-1245) before the model runs.
struct ByteScale { float low = 0.f, high = 1.f; };

class Engine {
public:
    Engine(LoadedModel&& lm, const std::vector<int>& devices, const EngineOptions& opt);
    ~Engine();

    const LoadedModel& model() const { return lm_; }
    int num_devices() const { return (int)ctx_.size(); }
    const EngineOptions& options() const { return opt_; }

    // Shape inference only (no GPU work): output shapes for the given input shapes.
    std::vector<TShape> infer(const std::vector<TShape>& in_shapes);

    // predict_multi with host buffers: in_ptrs[s * n_in + i], shapes likewise, out_ptrs[s * n_out + o].
    // Samples are grouped by shape signature, split in contiguous blocks over the devices
    // (model.hpp:31-42 semantics: results in input order).
    void predict_multi(int64_t n_samples, const float* const* in_ptrs, const TShape* in_shapes, float* const* out_ptrs,
                       const ByteScale* bytes = nullptr);

    // One batch on one device with device-resident, batch-major inputs and outputs.
    // kv (optional): the attention operations work on this cache (see KvCache); inputs feeding only the skipped
    // concatenations are not read.
    void predict_batch_device(int dev_index, int64_t batch, const float* const* d_in, const std::vector<TShape>& in_shapes,
                              float* const* d_out, cudaStream_t stream, const KvCache* kv = nullptr, std::string* profile = nullptr);
    // The attention operations of the plan for these input shapes, in execution order.
    std::vector<AttentionBlockInfo> attention_blocks(const std::vector<TShape>& in_shapes);

    // Runs the tests embedded in the model file; throws with the reference's message format on mismatch.
    void run_tests(float eps);

    // One batch on one device with CUDA events around every operation and every contraction launch.
    // Returns one line per record: "<kind> <layer> <ms> <flops> <M> <N> <K> <path>", kind = "op" for a
    // whole operation or "gemm" for one contraction kernel inside it (path: tc or ffma).
    std::string profile_batch_device(int dev_index, int64_t batch, const float* const* d_in, const std::vector<TShape>& in_shapes);

    int64_t launches() const;
    double plan_flops(const std::vector<TShape>& in_shapes);
    int64_t plan_arena_bytes(const std::vector<TShape>& in_shapes);
    int64_t max_batch_for(const std::vector<TShape>& in_shapes, int dev_index);

    // Device-side ordering of the users of a context's arena (see DeviceCtx::busy); call with c.mu held.
    void order_after_last_use(DeviceCtx& c, cudaStream_t s);
    void mark_use(DeviceCtx& c, cudaStream_t s);

    // kernel-level access for tests
    DeviceCtx& ctx(int i) { return *ctx_[(size_t)i]; }
    const float* weight_ptr(const DeviceCtx& c, int id) const { return c.w.base + c.w.offset[(size_t)id]; }

private:
    std::shared_ptr<Plan> get_plan(const std::vector<TShape>& in_shapes);
    std::shared_ptr<Plan> compile(const std::vector<TShape>& in_shapes);
    // wanted (optional, per plan output): 0 = the caller does not read this output, so it need not be computed
    void execute(DeviceCtx& c, const Plan& p, int64_t B, const float* const* d_in, cudaStream_t s, std::string* profile = nullptr,
                 const KvCache* kv = nullptr, const std::vector<char>* wanted = nullptr);
    void ensure_arena(DeviceCtx& c, int64_t elems);
    void run_block(DeviceCtx& c, const Plan& p, const std::vector<int64_t>& sample_ids, const float* const* in_ptrs,
                   float* const* out_ptrs, const ByteScale* bytes = nullptr);
    void upload_weights(DeviceCtx& c);

    LoadedModel lm_;
    EngineOptions opt_;
    std::vector<std::unique_ptr<DeviceCtx>> ctx_;
    std::mutex plan_mu_;
    std::map<std::string, std::shared_ptr<Plan>> plans_;
};

}  // namespace fdk
