// Device-resident decode session for incremental ("one token per call") decoder graphs.
//
// The reference's MultiHeadAttention has no mask (multi_head_attention_layer.hpp:74-95), so an
// autoregressive decoder is exported as two graphs that the caller loops over:
//   first:  inputs  token id (1), position (1)
//           outputs logits (1, V) and, per attention block l, the row x_l (1, D) that later steps attend to
//   step:   the same inputs plus one "past" tensor (None, D) per block, holding the rows of earlier positions;
//           inside, Concatenate([past_l, x_l]) feeds value and key of the block's attention
// With the reference (and with predict_multi) the caller carries the growing past tensors through host memory
// every step.  A session keeps them on the device: after each step the new rows are appended to per-block caches,
// the logits stay on the device, and the greedy next token is chosen there.
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
    float* d_past_[2] = {nullptr, nullptr};  // ping-pong: [layers][batch][max_len][dim], compact per current length
    int cur_ = 0;
};

}  // namespace fdk
