/* C ABI of the B200 forward-pass engine for frugally-deep models.
 *
 * This is the boundary a frugally-deep maintainer binds to: plain pointers and sizes, no C++ types.
 * Each entry point names the reference interface it stands in for (paths relative to the reference
 * project root).  Every function returns 0 on success and a non-zero code on failure; the message
 * of the last failure on the calling thread is read with fdk_last_error().  Nothing throws across
 * this boundary.
 *
 * Tensors are float32, channels last, row major, with the reference's right-aligned rank-5 shape
 * convention (include/fdeep/tensor_shape.hpp:23-170): `dims5` arrays hold
 * {dim5, dim4, height, width, depth} and `rank` says how many trailing entries are significant.
 * There is no CPU fallback: without a CUDA device model creation fails.
 */
#ifndef FDEEP_B200_H
#define FDEEP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fdk_model fdk_model;

/* Error text of the last failed call on this thread (include/fdeep/common.hpp:42-57 raises
 * std::runtime_error with the same texts).  Returns the full length of the message. */
size_t fdk_last_error(char* buf, size_t buf_size);

/* Number of visible CUDA devices. */
int fdk_device_count(int* count);

/* fdeep::load_model / fdeep::read_model_from_string (include/fdeep/model.hpp:285-301, :272-281).
 * `devices` lists the CUDA devices predict_multi shards over (NULL / 0 = device 0).
 * flags: bit 0 = disable the tensor-core (3xTF32) contraction path and use exact-fp32 FFMA kernels;
 *        bit 1 = let matrix products with at most 64 rows (a few samples against a wide weight matrix: one decode
 *        position, a dense head) take a kernel that streams the weights over all SMs (3xTF32 tensor-core products,
 *        exact FFMA products when bit 0 is set).  Results then differ in the last bits between batches of at most
 *        64 and of more rows, which is why it is opt-in;
 *        bit 2 = run an LSTM time step (units % 16 == 0, tanh / sigmoid) as ONE launch whose epilogue finishes the cell, so
 *        that the gate pre-activations never leave the SM, instead of the recurrent product followed by a cell launch.
 *        The results are the same bit for bit; the two-launch form is the default because it measured 4-8 % faster at
 *        every batch size tried (the cell's transcendental functions cost more in the product's epilogue than in a
 *        launch that fills the GPU). */
int fdk_model_load_file(const char* path, const int* devices, int n_devices, unsigned flags, fdk_model** out);
int fdk_model_load_json(const char* json_text, size_t json_len, const int* devices, int n_devices, unsigned flags,
                        fdk_model** out);
void fdk_model_destroy(fdk_model* m);

/* model::get_input_shapes / get_output_shapes (include/fdeep/model.hpp:70-78); -1 marks a variable
 * dimension.  model::name / model::hash (:106-114). */
int fdk_model_num_inputs(const fdk_model* m);
int fdk_model_num_outputs(const fdk_model* m);
int fdk_model_input_shape(const fdk_model* m, int index, int64_t dims5[5], int* rank);
int fdk_model_output_shape(const fdk_model* m, int index, int64_t dims5[5], int* rank);
const char* fdk_model_name(const fdk_model* m);
const char* fdk_model_hash(const fdk_model* m);
int fdk_model_num_devices(const fdk_model* m);

/* Output shapes for concrete input shapes (the shape checks of predict_impl,
 * include/fdeep/model.hpp:132-151, without running anything).
 * in_dims5: n_inputs x 5; in_ranks: n_inputs; out_dims5: n_outputs x 5; out_ranks: n_outputs. */
int fdk_model_infer_shapes(fdk_model* m, const int64_t* in_dims5, const int* in_ranks, int64_t* out_dims5,
                           int* out_ranks);

/* model::predict_multi (include/fdeep/model.hpp:31-42); model::predict is the n_samples == 1 case.
 * HOST buffers.  in_ptrs[s * n_inputs + i] is input i of sample s with shape
 * in_dims5[(s * n_inputs + i) * 5 ..], in_ranks[s * n_inputs + i]; out_ptrs[s * n_outputs + o] must
 * hold the volume reported by fdk_model_infer_shapes.  Samples of equal shape are batched; the
 * batches are split in contiguous blocks over the model's devices; results keep the input order. */
int fdk_model_predict_multi(fdk_model* m, int64_t n_samples, const float* const* in_ptrs, const int64_t* in_dims5,
                            const int* in_ranks, float* const* out_ptrs);

/* tensor_from_bytes (include/fdeep/tensor.hpp:1230-1245) followed by model::predict_multi: every input is
 * a uint8_t array of the given shape (an image as it leaves a decoder, row-wise, channels last) that is
 * scaled from [0, 255] into [low, high] exactly like the reference (byte * ((high - low) / 255) + low, in
 * float).  The bytes travel to the GPU as they are and become floats there: a quarter of the host-to-device
 * traffic of converting on the host first.  Otherwise like fdk_model_predict_multi. */
int fdk_model_predict_multi_u8(fdk_model* m, int64_t n_samples, const uint8_t* const* in_ptrs, const int64_t* in_dims5,
                               const int* in_ranks, float low, float high, float* const* out_ptrs);

/* Device-resident variant for callers that keep tensors on the GPU (what a device-backed fdeep::tensor
 * would hand over): one batch on device `device_index` (index into the model's device list).
 * d_in[i] / d_out[o] are device pointers to batch-major arrays [batch][volume]; all samples share
 * the per-sample shapes in in_dims5 / in_ranks (n_inputs entries).  Work is queued on `stream`
 * (a cudaStream_t; NULL = the model's own stream) and NOT synchronised.
 * All calls on one model and device share that device's intermediate buffers.  The library keeps them in order
 * on the device: a call queued on another stream than the previous one first waits (cudaStreamWaitEvent) for the
 * previous call's work, so calls from several threads or streams are safe but do not overlap on the GPU.  What
 * the caller must still do: keep d_in / d_out alive and untouched until the work on `stream` has finished. */
int fdk_model_predict_batch_device(fdk_model* m, int device_index, int64_t batch, const float* const* d_in,
                                   const int64_t* in_dims5, const int* in_ranks, float* const* d_out, void* stream);
/* Waits for the model's stream on that device and reports deferred device-side errors. */
int fdk_model_sync(fdk_model* m, int device_index);

/* ---- device buffers behind device-resident fdeep::tensor values ----
 * The reference's tensor is a shape plus a shared host vector (include/fdeep/tensor.hpp:28-168).  The drop-in tensor
 * may instead keep its values in a buffer on the GPU, so that the outputs of one model feed the next
 * (fdk_model_predict_batch_device) without passing through host memory; it fetches them on first host access
 * (as_vector, get, to_vector).  These calls manage such buffers.  `cuda_device` is a CUDA device ordinal
 * (fdk_model_cuda_device maps a model's device index to it); copies are synchronous.
 * kind: 0 host -> device, 1 device -> host, 2 device -> device. */
int fdk_model_cuda_device(const fdk_model* m, int device_index, int* cuda_device);
int fdk_device_alloc(int cuda_device, size_t bytes, void** d_ptr);
int fdk_device_free(int cuda_device, void* d_ptr);
int fdk_device_copy(int cuda_device, void* dst, const void* src, size_t bytes, int kind);
/* Bytes this library has copied between host and device memory so far, in this process (predict_multi's staging
 * copies and fdk_device_copy): lets a caller check that a chain of models really stayed on the device. */
int fdk_transfer_bytes(uint64_t* host_to_device, uint64_t* device_to_host);

/* The load-time self test of fdeep::load_model(verify = true): runs the `tests` embedded in the model
 * file and compares with absolute tolerance `epsilon` (include/fdeep/model.hpp:254-267,
 * include/fdeep/import_model.hpp:1990-2021).  n_tests may be NULL. */
int fdk_model_run_tests(fdk_model* m, float epsilon, int* n_tests);

/* Bookkeeping for benchmarks: kernels launched so far, contraction FLOPs (2 x MAC) of one sample for
 * the given input shapes, largest batch the arena budget allows on a device. */
int64_t fdk_model_launch_count(const fdk_model* m);
int fdk_model_plan_info(fdk_model* m, const int64_t* in_dims5, const int* in_ranks, double* flops_per_sample,
                        int64_t* arena_bytes_per_sample, int64_t* max_batch);

/* Runs one device-resident batch (arguments as for fdk_model_predict_batch_device, on the model's own
 * stream, synchronised) with CUDA events around every operation and every contraction kernel, and
 * writes one line per record into buf: "<kind> <layer> <ms> <flops> <M> <N> <K> <path>" where kind is
 * "op" (a whole plan operation: path holds the operation kind as a number, M the bytes the operation must move --
 * its inputs, residual and outputs once each) or "gemm" (one contraction kernel; path "tc", "ffma" or "skinny").  This is the
 * per-kernel counterpart of model::test_speed (include/fdeep/model.hpp:98-104).  The text is
 * truncated to buf_size; *needed receives an upper bound for the size of the full text. */
int fdk_model_profile(fdk_model* m, int device_index, int64_t batch, const float* const* d_in, const int64_t* in_dims5,
                      const int* in_ranks, char* buf, size_t buf_size, size_t* needed);

/* Host-only: parses a model, compiles the execution plan for the given input shapes (the walk of
 * include/fdeep/layers/model_layer.hpp:51-66 done once, with shape inference, epilogue fusion and the
 * memory plan) and writes a listing, one operation per line, into buf.  Needs no CUDA device.
 * *needed receives the size required for the whole text. */
int fdk_plan_describe(const char* json_text, size_t json_len, const int64_t* in_dims5, const int* in_ranks,
                      int n_inputs, char* buf, size_t buf_size, size_t* needed);

/* ---- device-resident decode loop ----
 * The reference's MultiHeadAttention has no mask (include/fdeep/layers/multi_head_attention_layer.hpp:74-95), so an
 * autoregressive decoder is exported as two incremental graphs: `first` (inputs: token id (1), position (1);
 * outputs: logits (1, V) and, per attention block, the row (1, D) that later positions attend to) and `step` (the
 * same plus one "past" input (None, D) per block).  With fdeep::model::predict the caller carries the growing past
 * tensors through host memory at every position; a session keeps them on the device (the key/value cache), appends
 * the rows each step emits, leaves the logits on the device and picks the greedy next token there.
 * Both models must be loaded on the same device (the first of their device lists). */
typedef struct fdk_session fdk_session;
int fdk_session_create(fdk_model* first, fdk_model* step, int64_t batch, int64_t max_len, fdk_session** out);
/* One position for all `batch` sequences.  tokens: `batch` host floats (token ids travel as floats,
 * include/fdeep/layers/embedding_layer.hpp:49), or NULL to feed the tokens chosen greedily by the previous step.
 * next_tokens (batch floats) and logits (batch x V floats) are optional host outputs.  Synchronises. */
int fdk_session_step(fdk_session* s, const float* tokens, float* next_tokens, float* logits);
int fdk_session_info(const fdk_session* s, int64_t* length, int64_t* batch, int64_t* vocab);
/* Starts over at length 0 with a new batch of sequences (the next step needs tokens); the device buffers, the cache
 * storage and the recorded position are kept, so that serving batch after batch allocates nothing. */
int fdk_session_reset(fdk_session* s);
void fdk_session_destroy(fdk_session* s);

/* ---- kernel-level entry points (device pointers), used by the parity tests of single kernels ---- */

/* C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) with row strides lda, ldw, ldc (in floats) on `stream`.
 * K <= lda and K <= ldw; only the first K floats of each row are read, so A and W may be blocks of rows (or of
 * columns) of larger matrices that end with the last row's K-th value.
 * path 0: FFMA fp32.  path 1: tcgen05 3xTF32 (needs K, lda, ldw multiples of 4 and 16-byte aligned
 * bases; fails if the shape is unsupported).  path 2: the split-K weight-streaming kernel for M <= 64 (same
 * alignment rules; three TF32 tensor-core products per fp32 product, or exact FFMA products when the environment
 * has FDK_SKINNY_MMA=0).  path 3: the tcgen05 kernel for M <= 64 (weights streamed once over all SMs in blocks of rows
 * and slices of K, the slices of a block summed on chip by a thread-block cluster; same alignment rules; allocates
 * nothing).  Stands in for the Eigen GEMM call sites
 * include/fdeep/convolution.hpp:147,274 and include/fdeep/layers/dense_layer.hpp:85. */
int fdk_gemm(int path, const float* dA, int64_t lda, const float* dW, int64_t ldw, float* dC, int64_t ldc, int64_t M,
             int N, int K, const float* d_bias, int relu, void* stream);

/* The sample range [*begin, *end) that part `part` of `n_parts` (devices of one process, or ranks of a
 * multi-process job) takes of n_samples independent samples: contiguous blocks of ceil(n / parts), so that
 * concatenating the parts' results restores the input order of predict_multi
 * (include/fdeep/model.hpp:31-42).  Host only. */
int fdk_shard_block(int64_t n_samples, int n_parts, int part, int64_t* begin, int64_t* end);

/* Splits n fp32 values into their TF32 high and low halves (big = rna_tf32(w), small = rna_tf32(w - big));
 * the weight operands of the tensor-core path are stored this way.  Queued on `stream`, not synchronised.
 * Corresponds to the load-time weight repack of include/fdeep/convolution.hpp:29-60. */
int fdk_split_tf32(const float* dW, float* d_big, float* d_small, int64_t n, void* stream);

/* The tcgen05 contraction on pre-split weights: C = act(A * (W_big + W_small)^T + bias + residual), with
 * residual (optional) laid out like C.  Allocates nothing and does not synchronise; deferred kernel
 * errors are read with fdk_tc_status.  Same call sites as fdk_gemm. */
int fdk_gemm_presplit(const float* dA, int64_t lda, const float* dW_big, const float* dW_small, int64_t ldw, float* dC,
                      int64_t ldc, int64_t M, int N, int K, const float* d_bias, const float* d_residual, int relu,
                      void* stream);
/* fdk_gemm's tensor-core path for callers that must not allocate device memory.  It has no counterpart in
 * the reference, which runs on the CPU and takes temporaries from the heap wherever it likes.  fdk_gemm(path 1)
 * takes a temporary from cudaMalloc on every call for the two TF32 halves of W; that stalls the other streams
 * of a latency-bound serving loop (cudaFree waits for the whole device) and fails outright in a process whose
 * own memory pool already owns the GPU's memory.  Here the halves go into a fixed array inside the library
 * image instead: no cudaMalloc, cudaFree or allocating library call, ever.
 *   Limit: N * ldw <= fdk_gemm_static_max_weight_floats() (1,048,576 floats; 8 MiB per device for both
 *   halves).  Larger matrices are refused with an error; use fdk_gemm_presplit with your own buffers.
 *   K <= lda and K <= ldw; of every row of W only the first K floats are read (W may end with the last row's
 *   K-th value).
 *   Sharing: every call on a device uses the same array, which keeps the previous call's contents; each call
 *   rewrites all it reads, on `stream`, before the contraction.  Calls on one stream are safe; calls that can
 *   overlap on the GPU (other streams or threads) race on the array and must be serialised by the caller.
 *   First call: on each device the first call looks up the array's address (and may load the kernels), so
 *   make it before any stream capture begins.  The device owning `stream` must be current.
 * Same arguments and arithmetic as fdk_gemm(path 1); queued on `stream`, not synchronised; deferred kernel
 * errors are read with fdk_tc_status. */
int fdk_gemm_static(const float* dA, int64_t lda, const float* dW, int64_t ldw, float* dC, int64_t ldc, int64_t M, int N,
                    int K, const float* d_bias, int relu, void* stream);
int64_t fdk_gemm_static_max_weight_floats(void);

/* Waits for `stream` and returns the sticky status of the tcgen05 kernels in *status (0 = ok; non-zero = a
 * bounded wait inside a kernel gave up), clearing it. */
int fdk_tc_status(void* stream, int* status);

#ifdef __cplusplus
}
#endif
#endif /* FDEEP_B200_H */
