// Device-resident decode session for incremental ("one token per call") decoder graphs.
//
// The reference's MultiHeadAttention has no mask (multi_head_attention_layer.hpp:74-95), so an
// autoregressive decoder is exported as two graphs that the caller loops over:
//   first:  inputs  token id (1), position (1)
//           outputs logits (1, V) and, per attention block l, the row x_l (1, D) that later steps attend to
//   step:   the same inputs plus one "past" tensor (None, D) per block, holding the rows of earlier positions;
//           inside, Concatenate([past_l, x_l]) feeds value and key of the block's attention
// With the reference (and with predict_multi) the caller carries the growing past tensors through host memory
// every step, and every block projects keys and values of ALL earlier rows again.  A session keeps the state on the
// device: the projected key and value rows of each block are cached (each position projects only its own row), the
// logits stay on the device, and the greedy next token is chosen there.
#pragma once

#include "engine.hpp"

namespace fdk {

class DecodeSession {
public:
    DecodeSession(Engine& first, Engine& step, int64_t batch, int64_t max_len);
    ~DecodeSession();
    DecodeSession(const DecodeSession&) = delete;
    DecodeSession& operator=(const DecodeSession&) = delete;

    // One position for every sequence.  tokens: `batch` host floats, or null to continue with the tokens chosen
    // greedily by the previous step.  next_tokens / logits (host, may be null) receive the greedy choice and the
    // logits (batch x vocab) of this position.
    void step(const float* tokens, float* next_tokens, float* logits);
    // Back to length 0 for a new batch of sequences: buffers, cache storage and the recorded position are kept (the
    // recording reads the length from the device, so it serves every position of every batch).  Also clears the
    // failed state of a session whose step threw: the cache is rebuilt from the first position on.
    void reset();
    int64_t length() const { return len_; }
    int64_t batch() const { return batch_; }
    int64_t vocab() const { return vocab_; }

private:
    Engine& first_;
    Engine& step_;
    int64_t batch_, max_len_, len_ = 0;
    int64_t vocab_ = 0, dim_ = 0;
    int layers_ = 0;
    int device_ = 0;
    cudaStream_t stream_ = nullptr;
    float* d_tokens_ = nullptr;      // [batch] current input tokens (as floats)
    float* d_next_ = nullptr;        // [batch] greedy choice of the last step
    float* d_pos_ = nullptr;         // [batch]
    float* d_logits_ = nullptr;      // [batch][vocab]
    float* d_rows_ = nullptr;        // [layers][batch][dim] rows emitted by the last step
    // Host memory mapped into the device's address space: the last kernel of a position leaves the chosen tokens and
    // the kernels' status words here, so that a step needs one stream synchronisation and no copy calls.
    float* h_pub_ = nullptr;         // [batch] tokens, then two ints of status
    float* d_pub_ = nullptr;         // the same memory as the device addresses it
    const int* status_a_ = nullptr;
    const int* status_b_ = nullptr;
    void publish();
    // Either the projected key/value rows (when every attention block has the incremental form): the blocks then
    // project only the new row and attend over the cache ...
    bool cached_ = false;
    KvCache kv_;
    // ... or the raw rows, re-laid out every step as the compact "past" inputs [batch][len][dim] of the step model
    // (ping-pong), for models whose attention is wired differently.
    float* d_past_[2] = {nullptr, nullptr};
    int cur_ = 0;
    // Cache mode, positions after the first: the length is kept on the device (d_len_) so that every position is the
    // same sequence of launches; the second such position is recorded as a CUDA graph and replayed from then on.
    void step_impl(const float* tokens, float* next_tokens, float* logits);
    void queue_position_on_device();
    bool replay_position();
    void drop_graph();
    bool failed_ = false;            // a step threw after queueing work: the session refuses further steps
    int* d_len_ = nullptr;           // rows in the cache, as the kernels see it
    bool device_len_ = true, use_graph_ = true, warmed_ = false;
    cudaGraphExec_t graph_exec_ = nullptr;
    const void* graph_arena_ = nullptr;      // addresses the recorded launches hold
    const void* graph_workspace_ = nullptr;
    int64_t graph_launches_ = 0;
    double t_plan_ = 0, t_queue_ = 0, t_wait_ = 0;  // host seconds, accumulated when FDK_SESSION_TIMING is set
    double t_device_ = 0;                            // device milliseconds between the first and the last launch of a position
    cudaEvent_t ev_begin_ = nullptr, ev_end_ = nullptr;
};

}  // namespace fdk
