// Launchers of the device kernels (sm_100a).  All tensors are fp32, batch-major:
// [batch][dim5][dim4][height][width][depth], depth contiguous.
#pragma once

#include "common.hpp"

namespace fdk {

// ---- contraction: C[M,N] = epilogue(A[M,K] * W[N,K]^T) ------------------------------------------
// FFMA path (exact fp32 products, sequential-in-k accumulation per thread).
void launch_gemm_ffma(const float* A, int64_t lda, const float* W, int64_t ldw, float* C, int64_t ldc,
                      int64_t M, int N, int K, const Epilogue& e, cudaStream_t s);

// Skinny path (M <= 64): three TF32 tensor-core products per fp32 product (warp-level mma.sync; FDK_SKINNY_MMA=0 in the
// environment, or tensor_cores = false, gives exact fp32 FFMA products instead); the weight matrix is cut into 64-column blocks and slices of K, one
// CTA each; the CTA that finishes last for a column block sums the partial tiles in slice order and applies the
// epilogue (one launch).  gemm_skinny_plan gives the number of slices and the workspace (floats) a launch needs;
// the workspace must have been cleared once after its allocation (it starts with arrival counters that every launch
// leaves at zero) and serves one launch at a time.  K, lda, ldw multiples of 4 and 16-byte aligned bases.
bool gemm_skinny_supported(int64_t M, int N, int K, int64_t lda, int64_t ldw, const void* A, const void* W);
void gemm_skinny_plan(int N, int K, int& slices, int& k_per_slice, int64_t& workspace_floats, int64_t M);
void launch_gemm_skinny(const float* A, int64_t lda, const float* W, int64_t ldw, float* C, int64_t ldc, int64_t M, int N, int K,
                        const Epilogue& e, float* workspace, cudaStream_t s, bool tensor_cores = true);
// `count` (1..3) products of the same A with weight matrices of one shape in ONE launch (the query, key and value
// projections of an attention block): C[i] = A * W[i]^T + bias[i].  The workspace must hold `count` times the
// floats gemm_skinny_plan gives for one product.
void launch_gemm_skinny_group(const float* A, int64_t lda, int count, const float* const* W, int64_t ldw, float* const* C, const int64_t* ldc,
                              const float* const* bias, int64_t M, int N, int K, float* workspace, cudaStream_t s, bool tensor_cores = true);

// Row products (M <= 64) on the 5th-generation tensor cores (gemm_rows.cu): W is streamed once over all SMs in blocks
// of 128 or 64 rows and up to 8 slices of K; the CTAs of a block form a cluster and add their partial tiles through
// distributed shared memory in slice order.  3xTF32 (fp32 semantics) on unsplit weights.  `count` (1..3) products of the
// same X with weight matrices of one shape share a launch (C[i] = epilogue(X * W[i]^T + bias[i]); the epilogue's own
// bias field is not used).  norm (optional): X is layer-normalised over K first (layer_normalization_layer.hpp:37-63),
// which replaces a separate normalisation launch.  Launched with programmatic stream serialisation: the kernel
// prefetches weights while its predecessor in the stream still runs and waits for it before reading X.
// K, ldx, ldw multiples of 4 and 16-byte aligned bases.  Allocates nothing.
struct RowsNorm {
    const float* gamma = nullptr;   // K values or null
    const float* beta = nullptr;
    float eps = 0.f;
};
bool gemm_rows_supported(int64_t M, int N, int K, int64_t ldx, int64_t ldw, const void* X, const void* W);
// The normalised form takes its row statistics from tiles resident in shared memory: whether `count` products of this
// shape can be laid out so that every CTA's K slice fits its ring (asks the current device).
bool gemm_rows_norm_supported(int N, int K, int count);
void gemm_rows_plan(int N, int K, int count, int& block_rows, int& k_slices, int& k_blocks_per_slice, bool normalised = false);
void launch_gemm_rows(const float* X, int64_t ldx, int count, const float* const* W, int64_t ldw, float* const* C, const int64_t* ldc,
                      const float* const* bias, const Epilogue& e, int64_t M, int N, int K, const RowsNorm* norm, cudaStream_t s);
int gemm_rows_take_status(cudaStream_t s);

// tcgen05 path: 3xTF32 split products on the 5th-generation tensor cores, TMEM accumulators, TMA
// operand loads.  `Wbig`/`Wsmall` are the precomputed high/low TF32 halves of the weights.
// Requirements: K % 4 == 0, lda % 4 == 0, ldw % 4 == 0, 16-byte aligned bases.
// Returns false (nothing launched) when the shape is outside what this path supports.
bool gemm_tc_supported(int64_t M, int N, int K, int64_t lda, int64_t ldw, const void* A, const void* W);
void launch_gemm_tc(const float* A, int64_t lda, const float* Wbig, const float* Wsmall, int64_t ldw, float* C,
                    int64_t ldc, int64_t M, int N, int K, const Epilogue& e, cudaStream_t s);
// The same kernel fed straight from a channels-last input [B][H][W][pix] (implicit GEMM: the operand tiles
// are fetched by TMA per filter tap, zero padding comes from out-of-range coordinates, strides from the
// tensor map's element strides; no im2col buffer).  Weights are [N][kh*kw*C] with row stride ldw.
struct ConvTcGeom {
    int64_t B = 1;
    int H = 1, W = 1, C = 1;
    int64_t pix = 1;          // floats between consecutive pixels (= C for a dense NHWC tensor)
    int Ho = 1, Wo = 1;
    int kh = 1, kw = 1, sy = 1, sx = 1, dy = 1, dx = 1, pad_t = 0, pad_l = 0;
    // Row-window form (> 0): the input is a padded copy [B][H][W][C] with C % 4 == 0 and kw * C <= 32; one k block
    // is the 32 floats starting at output column ox * win_stride of input row oy * sy + ky (a whole filter row);
    // weights are [N][kh][32].  sx, dx, pads are not used (the copy is already padded).
    int64_t win_stride = 0;
    // Output pixels that are not dense [B][Ho][Wo][ldc] (> 0: floats between neighbours in x, in y, between samples):
    // one phase of a transposed convolution writes every s-th pixel of the layer's output.  A residual then has the
    // same layout (and the same base offset) as the output.
    int64_t out_sx = 0, out_sy = 0, out_sb = 0;
    // 3-D convolution (D > 1 or kd > 1): every sample is D input slices [H][W][pix] and Do output slices; filter tap
    // (kz, ky, kx) of output slice od reads input slice od * sz - pad_f + kz (none outside 0 .. D - 1: zeros).
    // Weights are [N][kd][kh][kw][C].  A tile then lies within one output slice.
    int D = 1, Do = 1, kd = 1, sz = 1, pad_f = 0;
};
bool conv_tc_supported(const ConvTcGeom& g, int N, int64_t ldw, const void* in, const void* W);
void launch_conv_tc(const float* in, const ConvTcGeom& g, const float* Wbig, const float* Wsmall, int64_t ldw, float* C,
                    int64_t ldc, int N, const Epilogue& e, cudaStream_t s);
// One LSTM time step in one launch: z = h U + x (x = this step's rows of the input product, bias included) never
// leaves the SM; the epilogue applies the cell (tanh / sigmoid) and writes c in place, the new h to h_next (a buffer
// other than h: other CTAs still read h) and, if given, to out.  U's rows (and x's columns) must be in the cell order:
// row 64 * (u / 16) + 16 * gate + u % 16 for gate (i, f, c~, o) of unit u.  z_unused: any 16-byte aligned buffer of
// B x 4U floats (only described, never written).
bool lstm_step_tc_supported(int64_t B, int U, const void* h, const void* W, int64_t ldw, const void* x, int64_t ldx, const void* c,
                            const void* h_next, const void* out, int64_t out_stride);
void launch_lstm_step_tc(const float* h, const float* Wbig, const float* Wsmall, int64_t ldw, const float* x, int64_t ldx, float* c,
                         float* h_next, float* out, int64_t out_stride, float* z_unused, int64_t B, int U, cudaStream_t s);
// Reads and clears the sticky device-side status of the tcgen05 kernels (0 = ok; nonzero = a bounded
// wait on an mbarrier gave up).
int gemm_tc_take_status(cudaStream_t s);
void launch_split_tf32(const float* w, float* big, float* small, int64_t n, cudaStream_t s);
// The tcgen05 contraction on unsplit weights with the TF32 halves kept in a fixed per-device array of the
// library image (gemm_static.cu): allocates nothing; refuses N * ldw > gemm_static_max_weight_floats().
int64_t gemm_static_max_weight_floats();
void launch_gemm_tc_static(const float* A, int64_t lda, const float* W, int64_t ldw, float* C, int64_t ldc, int64_t M, int N, int K,
                           const Epilogue& e, cudaStream_t s);

// ---- convolution helpers -------------------------------------------------------------------------
// out[m][k], m = (b, oy, ox), k = (ky, kx, c) padded with zeros up to Kp columns.
void launch_im2col(const float* in, float* out, int64_t B, int H, int W, int C, int Ho, int Wo, int kh, int kw,
                   int sy, int sx, int dy, int dx, int pad_t, int pad_l, int Kp, cudaStream_t s);
// Transposed-convolution gather: the zero-dilated, padded input of the reference is never materialised;
// out[m][k] reads in[(y - off)/s] where that is an integer sample position, else 0.
void launch_im2col_transposed(const float* in, float* out, int64_t B, int H, int W, int C, int Ho, int Wo, int kh, int kw,
                              int sy, int sx, int offy, int offx, int pad_t, int pad_l, int Hd, int Wd, int Kp, cudaStream_t s);
// Depthwise convolution, weights laid out [kh*kw][C].
void launch_dwconv(const float* in, const float* w, float* out, int64_t B, int H, int W, int C, int Ho, int Wo,
                   int kh, int kw, int sy, int sx, int pad_t, int pad_l, const Epilogue& e, cudaStream_t s);

// Variations of the attention kernel beyond MultiHeadAttention's scaled dot product.
enum AttnMode : int { ATTN_DOT = 0, ATTN_CONCAT = 1, ATTN_ADDITIVE = 2 };
struct AttnExtra {
    int group = 1;                // query heads per key/value head (group_query_attention_layer.hpp:131-133)
    int mode = ATTN_DOT;          // ATTN_CONCAT: w2 * sum tanh(scale (q + k)) (attention_layer.hpp:40-50);
                                  // ATTN_ADDITIVE: sum svec * tanh(q + k) (additive_attention_layer.hpp:33-41)
    float w2 = 1.f;
    const float* svec = nullptr;  // sn = 1 or dk values; nullptr = ones
    int sn = 0;
    const float* gate = nullptr;  // laid out like `out`: out *= sigmoid(gate)
    // Decode on a key/value cache whose length lives in device memory (one query row; a launch recorded in a CUDA
    // graph then serves every position): the key length is *len_ptr + 1; key/value row *len_ptr of every sample is
    // read from k_new / v_new ([batch][heads * dim], this position's projections) and stored into the cache by the
    // kernel; `Tk` of the launch is the capacity of the score buffer (the cache's max_len).
    const int* len_ptr = nullptr;
    const float* k_new = nullptr;
    const float* v_new = nullptr;
};
// ---- memory-bound layers ----------------------------------------------------------------------------
// zero_frame (optional): {front, back, top, bottom, left, right} explicit zeros around the input (a folded
// ZeroPadding layer): those taps read 0 and count as values; pad_f/pad_t/pad_l are the SAME-padding offsets
// of the framed tensor, whose taps outside are skipped.
void launch_pool3d(const float* in, float* out, int64_t B, int D, int H, int W, int C, int Do, int Ho, int Wo,
                   int pd, int ph, int pw, int sd, int sy, int sx, int pad_f, int pad_t, int pad_l, const int* zero_frame,
                   bool is_max, cudaStream_t s);
void launch_global_pool(const float* in, float* out, int64_t B, int64_t spatial, int C, bool is_max, cudaStream_t s);
enum BinaryOp : int { BIN_ADD = 0, BIN_SUB = 1, BIN_MUL = 2, BIN_MAX = 3, BIN_MIN = 4 };
// out = act((a op b) * post_scale); a and b broadcast against out on size-1 dims (per-sample dims5).
void launch_binary(int op, const float* a, const int64_t* adims, const float* b, const int64_t* bdims, float* out,
                   const int64_t* odims, int64_t B, float post_scale, ActSpec act, cudaStream_t s);
void launch_unary(ActSpec act, const float* in, float* out, int64_t n, cudaStream_t s);
// y = act(x * scale[c] + shift[c]); element index = (outer, c, inner).
void launch_affine(const float* in, float* out, const float* scale, const float* shift, int64_t outer, int64_t nc,
                   int64_t inner, ActSpec act, cudaStream_t s);
// Softmax along depth for `rows` rows of `depth` values; rows >= valid_rows are written as zero
// (the reference iterates height and width only, tensor.hpp:1170-1171).
void launch_softmax(const float* in, float* out, int64_t B, int64_t rows_per_sample, int64_t valid_rows, int depth,
                    bool log_form, cudaStream_t s);
// Normalisation over the last `n` contiguous values of each of `rows` rows; gamma/beta may be null.
// mode 0: layer normalisation; 1: x / sqrt(mean(x^2) + eps) * gamma (RMS); 2: x / sqrt(max(sum x^2, FLT_EPSILON)) (unit).
void launch_layernorm(const float* in, float* out, const float* gamma, const float* beta, int64_t rows, int n,
                      float eps, int mode, cudaStream_t s);
// Group normalisation over the channel axis of [B][spatial][C]; gamma / beta (length C) may be null.
void launch_groupnorm(const float* in, float* out, const float* gamma, const float* beta, int64_t B, int64_t spatial, int C, int groups,
                      float eps, cudaStream_t s);
// Window copy used by ZeroPadding and Cropping: out[b, d, y, x, :] = in[b, d - f, y - t, x - l, :] or 0.
void launch_window(const float* in, float* out, int64_t B, int D, int H, int W, int C, int Do, int Ho, int Wo,
                   int off_d, int off_y, int off_x, cudaStream_t s);
// Zero-padded copy in space and channels: out[B][Hp][Wp][Cp] from in[B][H][W][C] shifted by (pad_t, pad_l);
// feeds the row-window form of convolutions with few input channels.
void launch_pad_channels(const float* in, float* out, int64_t B, int H, int W, int C, int Hp, int Wp, int Cp, int pad_t, int pad_l,
                         cudaStream_t s);
// Strided slab copy used by Concatenate: out[o, off + j] = in[o, j], j < in_len, rows of out_len.
void launch_slab_copy(const float* in, float* out, int64_t outer, int64_t in_len, int64_t out_len, int64_t off, cudaStream_t s);
// General permutation of the five per-sample dims: out dims = in dims[perm[i]].
void launch_permute(const float* in, float* out, int64_t B, const int64_t* in_dims, const int* perm, cudaStream_t s);
// Embedding row gather; ids are floats truncated to integers.  An id outside [0, input_dim) sets
// *err to 1 and yields a zero row.
void launch_embedding(const float* ids, const float* table, float* out, int64_t n_ids, int dim, int64_t input_dim,
                      int* err, cudaStream_t s);
// ---- recurrent cells -----------------------------------------------------------------------------------
// z[B,4U] holds x_t W + b + h U (gate order i, f, c~, o); updates c and h in place, writes h to out rows.
void launch_lstm_cell(const float* z, float* c, float* h, float* out, int64_t out_stride, int64_t B, int U,
                      ActSpec act, ActSpec ract, cudaStream_t s);
// GRU with reset_after: xw[B,3U] (= x W + b_x, row stride ldx), hu[B,3U] (= h U + b_h); order z, r, h~.
void launch_gru_cell(const float* xw, int64_t ldx, const float* hu, float* h, float* out, int64_t out_stride,
                     int64_t B, int U, ActSpec act, ActSpec ract, cudaStream_t s);
// GRU without reset_after, two products per step: hu[B, ldh] = h U_z | h U_r becomes z | r .* h (gates), then with
// hu[:, 2U:3U] = (r .* h) U_h the new state h' = (1 - z) act(x W_h + b + hu_h) + z h (out).
void launch_gru_gates(const float* xw, int64_t ldx, float* hu, int64_t ldh, const float* h, int64_t B, int U, ActSpec ract, cudaStream_t s);
void launch_gru_out(const float* xw, int64_t ldx, const float* zr, int64_t ldh, float* h, float* out, int64_t out_stride, int64_t B, int U,
                    ActSpec act, cudaStream_t s);
// ---- attention -------------------------------------------------------------------------------------------
// out[b, tq, h*dv + d] = sum_t softmax_t(scale * q[b,tq,h,:] . k[b,t,h,:]) v[b,t,h,d]
// Row strides are given per tensor; kv_len[b] (optional) bounds Tk per sample for cached decoding.
void launch_attention(const float* q, int64_t ldq, int64_t q_bstride, const float* k, int64_t ldk, int64_t k_bstride,
                      const float* v, int64_t ldv, int64_t v_bstride, float* out, int64_t ldo, int64_t o_bstride,
                      int64_t B, int H, int Tq, int Tk, int dk, int dv, float scale, cudaStream_t s,
                      const AttnExtra& x = AttnExtra());
// PReLU over [B][H][W][C] with alpha indexed (h, w, c), index 0 on shared axes (prelu_layer.hpp:30-68)
void launch_prelu(const float* in, float* out, const float* alpha, int64_t B, int H, int W, int C, bool hs, bool ws, bool cs, cudaStream_t s);
// General "input,kernel->output" contraction of EinsumDense (einsum_dense_layer.hpp:224-258) for equations that
// are not a plain matrix product: every output letter and every summed letter has a size and its stride in the
// input, the kernel and the bias (0 where the letter does not occur).
struct EinsumGeom {
    int n_out = 0, n_sum = 0;
    int64_t out_size[8], out_in[8], out_k[8], out_b[8];
    int64_t sum_size[8], sum_in[8], sum_k[8];
    int64_t in_volume = 0, out_volume = 0, sum_volume = 1;
};
void launch_einsum(const float* in, const float* kernel, const float* bias, float* out, int64_t B, const EinsumGeom& g, cudaStream_t s);
// Patch matrix of a 3-D convolution (convolution3d.hpp:320-506): row (b, od, oy, ox), columns (fd, fy, fx, c), row
// stride Kp.  Per axis i: the window starts at o * stride - pad_lo in a tensor of extent `spread` that holds input
// element j at off + j * inner (inner > 1 for the transposed layer, whose input is spread by its strides).
struct Conv3dGeom {
    int in[3], out[3], k[3], stride[3], pad_lo[3], spread[3], off[3], inner[3];
    int C = 0, Kp = 0;
};
void launch_im2col3d(const float* in, float* out, int64_t B, const Conv3dGeom& g, cudaStream_t s);
// tensor_from_bytes on the device (tensor.hpp:1230-1245): out = byte * ((high - low) / 255) + low, the product and
// the sum rounded separately like the reference's reference_interval.
void launch_bytes_to_float(const uint8_t* in, float* out, int64_t n, float low, float high, cudaStream_t s);
// Normalization layer (normalization_layer.hpp:37-52): x laid out [outer][n][inner]; out = (x - mean[i]) / max(sqrt(var[i]), 1e-7),
// or mean[i] + x * max(sqrt(var[i]), 1e-7) when inverted; the division / product in double like the reference.
void launch_normalization(const float* in, float* out, const float* mean, const float* var, int64_t outer, int64_t n, int64_t inner,
                          bool invert, cudaStream_t s);
// resize2d_nearest with whole-number factors and resize2d_bilinear (tensor.hpp:959-1035) over [B][H][W][C] -> [B][H*fy][W*fx][C]
void launch_upsample2d(const float* in, float* out, int64_t B, int H, int W, int C, int fy, int fx, bool bilinear, cudaStream_t s);
// resize2d_nearest / resize2d_bilinear / resize2d_area (tensor.hpp:959-1111) of the window (y0, x0, ch, cw) of every image
// [H][W][C] into [Ho][Wo][C]; mode 0 nearest, 1 bilinear, 2 area.
void launch_resize2d(const float* in, float* out, int64_t images, int H, int W, int C, int Ho, int Wo, int mode, int y0, int x0, int ch, int cw,
                     cudaStream_t s);
// dot_product_tensors (tensor.hpp:814-884): a = [a_outer][K][a_inner], b = [b_outer][K][b_inner] per sample;
// out[(ao, ai), (bo, bi)] = sum_k a[ao][k][ai] * b[bo][k][bi]; normalize: both operands are L2-normalised along k first.
void launch_dot(const float* a, const float* b, float* out, int64_t B, int64_t a_outer, int64_t a_inner, int64_t b_outer, int64_t b_inner, int64_t K,
                bool normalize, cudaStream_t s);
// adaptive_pooling_3d_layer.hpp:53-113: output index i of an axis covers input [floor(i in / out), ceil((i + 1) in / out)).
void launch_adaptive_pool(const float* in, float* out, int64_t B, int D, int H, int W, int C, int Do, int Ho, int Wo, bool is_max, cudaStream_t s);
// Preprocessing look-ups on `n` values per sample.  mode 0: Discretization (table = `size` sorted boundaries; result = how
// many are <= x, discretization_layer.hpp:37-40); 1: IntegerLookup (table = `size` sorted keys, their results, the mask
// token; integer_lookup_layer.hpp:62-78); 2 / 3 / 4: CategoryEncoding one_hot / multi_hot / count into `size` slots per
// sample (category_encoding_layer.hpp:40-60; a value outside [0, size) sets *err to 2).
void launch_lookup(int mode, const float* in, float* out, const float* table, int64_t B, int64_t n, int size, bool has_mask, int* err,
                   cudaStream_t s);
// Depthwise 3 x 3, stride 1 or 2, from TMA-staged input tiles (dwconv_tma.cu); launch_dwconv takes it when the shape fits.
bool dwconv_tiles_supported(const float* in, const float* w, const float* out, int C, int kh, int kw, int sy, int sx, const Epilogue& e);
void launch_dwconv_tiles(const float* in, const float* w, float* out, int64_t B, int H, int W, int C, int Ho, int Wo, int stride, int pad_t,
                         int pad_l, const Epilogue& e, cudaStream_t s);
int dwconv_tiles_take_status(cudaStream_t s);
// 2-D pooling (2 x 2 / 2, 3 x 3 / 1 or 2) from the same TMA-staged tiles, for windows that never leave the tensor or its
// frame of explicit zeros; launch_pool3d takes it when the shape fits.
bool pool_tiles_supported(const float* in, const float* out, int C, int Hz, int Wz, int Ho, int Wo, int ph, int pw, int sy, int sx, int pad_t,
                          int pad_l);
void launch_pool_tiles(const float* in, float* out, int64_t B, int H, int W, int C, int Ho, int Wo, int window, int stride, int frame_t,
                       int frame_l, bool is_max, cudaStream_t s);
// Gates of a convolutional LSTM step (conv_lstm_2d_layer.hpp:111-131): x and u hold, per spatial position, 4 * U values
// (gates i, f, c~, o; u may be null: zero); c_prev [positions][U] may be null (zero).  c = f c_prev + i c~, h = o act(c).
void launch_convlstm_cell(const float* x, const float* u, const float* c_prev, float* h, float* c, int64_t positions, int U, ActSpec act,
                          ActSpec ract, cudaStream_t s);
void launch_fill(float* p, float v, int64_t n, cudaStream_t s);
// p[0..n) = (float)*counter; *counter += delta (single thread) -- the position of a decode loop kept on the device
void launch_fill_from_counter(float* p, const int* counter, int64_t n, cudaStream_t s);
void launch_counter_add(int* counter, int delta, cudaStream_t s);
// out[r] = index (as a float) of the first largest of the n values of row r: the greedy choice of a decode loop.
void launch_argmax_rows(const float* in, float* out, int64_t rows, int n, cudaStream_t s);
// End of a decode position: copies n floats (the chosen tokens) and the two sticky status words of the tensor-core
// kernels into host memory that is mapped into the device's address space, so that after the stream has been
// synchronised the host reads them without any further call.  host_status receives {status_a, status_b}.
void launch_publish_position(const float* tokens, int n, const int* status_a, const int* status_b, float* host_tokens, int* host_status,
                             cudaStream_t s);
// Device addresses (on the current device) of the status words read by gemm_tc_take_status.
const int* gemm_tc_status_address();
const int* gemm_rows_status_address();
// out = in * f (Average layer: sum * (1 / n), tensor.hpp:886-891)
void launch_scale(const float* in, float* out, int64_t n, float f, cudaStream_t s);

}  // namespace fdk
