// What surrounds the paged attention kernels in a mixer whose projections pass a short convolution
// over time and a norm over all heads at once, and whose softmax weights are mixed over heads.
//
// `conv_norm_rope_write` (one block per new token), in 32-bit throughout:
//   1. a causal convolution over `taps` tokens on each channel of q, k and v: y_t = sum_j w[c][j] u_(t-taps+1+j),
//      u = projection + bias, zero in front of a request's first token. Inputs in front of the step's
//      tokens come from the request's slot (the last taps - 1 projections, bias not yet added);
//   2. one RMS norm over the whole of q (all heads) and one over the whole of k, each with a weight per channel;
//   3. rotation of dims 2i, 2i+1 (i < rot_dims / 2) of every query and key head by position x inv_freq[i];
//   4. queries to a dense buffer, keys and values to the token's page; rows are `row_dim` wide in all
//      three (the arena has one row width for keys and values), the rest zero. The token that starts a
//      page clears the rows its step does not fill.
// `conv_slot_update` (one block per request) moves the slot on.
//
// Mixing the weights over heads: head h applies sum_g M[h][g] softmax_g to the values of its own
// key/value head c(h), which is sum_g M[h][g] (softmax_g applied to the values of head c(h)). The
// attention kernels give A[c][t][g] = softmax_g applied to value head c (one launch per value head);
// `mix_heads_gate` forms out[t][h] = sigmoid(gate[t][h]) (.) sum_g M[h][g] A[c(h)][t][g].
#include "common.cuh"
#include "page_tail.cuh"

namespace {

template <typename T>
__global__ void conv_norm_rope_write_kernel(const T* proj, int ld, const float* __restrict__ bias, const float* __restrict__ taps_w,
                                            int taps, const T* conv_state, const float* __restrict__ q_weight,
                                            const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
                                            int rot_dims, const int* __restrict__ positions, const int* __restrict__ token_seq,
                                            const int* __restrict__ seq_q_start, const int* __restrict__ seq_slot,
                                            const int* __restrict__ seq_kv_len, const int* __restrict__ block_table, int max_pages,
                                            int num_pages, T* k_arena, T* v_arena, T* q_out, int q_heads, int kv_heads, int dim,
                                            int vdim, int row_dim, int page_size, int write_kv, int* err) {
  extern __shared__ float y[];  // [channels]
  __shared__ float scratch[32];
  let_successor_start();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int qw = q_heads * dim, kw = kv_heads * dim, vw = kv_heads * vdim;
  const int channels = qw + kw + vw;
  const int seq = token_seq[t];
  const int pos = positions[t];
  const int run = t - seq_q_start[seq];  // tokens of this request in front of t within the step
  int page = -1;
  if (write_kv) {
    const int logical = pos / page_size;
    if (pos < 0 || logical >= max_pages) {
      if (tid == 0) atomicOr(err, ERRBIT_BAD_POSITION);
    } else {
      page = block_table[static_cast<int64_t>(seq) * max_pages + logical];
      if (page < 0 || page >= num_pages) {
        if (tid == 0) atomicOr(err, ERRBIT_BAD_PAGE);
        page = -1;
      }
    }
  }
  wait_for_predecessor();
  const T* state = conv_state + static_cast<int64_t>(seq_slot[seq]) * (taps - 1) * channels;
  for (int c = tid; c < channels; c += blockDim.x) {
    const float b = bias ? bias[c] : 0.f;
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;  // how many tokens before t
      if (back > pos) continue;       // in front of the request's first token
      const float x = back <= run ? to_f32<T>(proj[static_cast<int64_t>(t - back) * ld + c])
                                  : to_f32<T>(state[static_cast<int64_t>(taps - 1 + run - back) * channels + c]);
      acc = fmaf(taps_w[c * taps + j], x + b, acc);
    }
    y[c] = acc;
  }
  __syncthreads();
  float sq = 0.f, sk = 0.f;
  for (int c = tid; c < qw; c += blockDim.x) sq = fmaf(y[c], y[c], sq);
  for (int c = qw + tid; c < qw + kw; c += blockDim.x) sk = fmaf(y[c], y[c], sk);
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);
  const float inv_q = 1.f / sqrtf(sq / static_cast<float>(qw) + eps);
  const float inv_k = 1.f / sqrtf(sk / static_cast<float>(kw) + eps);
  __syncthreads();
  for (int c = tid; c < qw + kw; c += blockDim.x) y[c] *= (c < qw ? inv_q * q_weight[c] : inv_k * k_weight[c - qw]);
  __syncthreads();
  const float p = static_cast<float>(pos);
  // queries and keys: (q_heads + kv_heads) rows of row_dim numbers
  const int qk_rows = q_heads + kv_heads;
  for (int idx = tid; idx < qk_rows * row_dim; idx += blockDim.x) {
    const int head = idx / row_dim, i = idx - head * row_dim;
    const bool is_q = head < q_heads;
    float value = 0.f;
    if (i < dim) {
      const float* src = y + head * dim;  // keys follow the queries in y
      value = src[i];
      if (i < rot_dims) {
        float sn, cs;
        sincosf(p * inv_freq[i >> 1], &sn, &cs);
        const float other = src[i ^ 1];
        value = (i & 1) ? fmaf(value, cs, other * sn) : fmaf(value, cs, -other * sn);
      }
    }
    if (is_q) {
      q_out[(static_cast<int64_t>(t) * q_heads + head) * row_dim + i] = from_f32<T>(value);
    } else if (page >= 0) {
      k_arena[kv_row_offset(page, head - q_heads, pos % page_size, kv_heads, page_size, row_dim) + i] = from_f32<T>(value);
    }
  }
  if (page >= 0) {
    for (int idx = tid; idx < kv_heads * row_dim; idx += blockDim.x) {
      const int head = idx / row_dim, i = idx - head * row_dim;
      const float value = i < vdim ? y[qw + kw + head * vdim + i] : 0.f;
      v_arena[kv_row_offset(page, head, pos % page_size, kv_heads, page_size, row_dim) + i] = from_f32<T>(value);
    }
    if (pos % page_size == 0 && seq_kv_len != nullptr) {
      const int clear_from = max(1, seq_kv_len[seq] - pos);
      for (int head = 0; head < kv_heads; ++head) {
        clear_page_tail(k_arena + kv_row_offset(page, head, 0, kv_heads, page_size, row_dim), clear_from, page_size, row_dim);
        clear_page_tail(v_arena + kv_row_offset(page, head, 0, kv_heads, page_size, row_dim), clear_from, page_size, row_dim);
      }
    }
  }
}

// After a step the slot holds the last taps - 1 rows of [old slot | the step's projections].
template <typename T>
__global__ void conv_slot_update_kernel(const T* proj, int ld, int channels, int taps, const int* seq_q_start, const int* seq_q_len,
                                        const int* seq_slot, T* conv_state) {
  wait_for_predecessor();
  let_successor_start();
  const int seq = blockIdx.x;
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  const int keep = taps - 1;
  T* state = conv_state + static_cast<int64_t>(seq_slot[seq]) * keep * channels;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    for (int r = 0; r < keep; ++r) {
      const int at = len + r;  // index into [old slot (keep) | inputs (len)]
      state[static_cast<int64_t>(r) * channels + c] =
          at < keep ? state[static_cast<int64_t>(at) * channels + c] : proj[static_cast<int64_t>(start + at - keep) * ld + c];
    }
  }
}

// attn [kv_heads][tokens][heads][row_dim]; gate logits at gate[t * gate_ld + h * vdim + i].
template <typename T>
__global__ void mix_heads_gate_kernel(const T* attn, const float* __restrict__ mix, const T* gate, int gate_ld, int tokens, int heads,
                                      int kv_heads, int vdim, int row_dim, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int group = heads / kv_heads;
  const int64_t total = static_cast<int64_t>(tokens) * heads * vdim;
  const int64_t plane = static_cast<int64_t>(tokens) * heads * row_dim;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % vdim);
    const int64_t th = idx / vdim;
    const int h = static_cast<int>(th % heads);
    const int64_t t = th / heads;
    const T* src = attn + (h / group) * plane + t * heads * row_dim + i;
    float acc = 0.f;
    for (int g = 0; g < heads; ++g) acc = fmaf(mix[h * heads + g], to_f32<T>(src[static_cast<int64_t>(g) * row_dim]), acc);
    const float gv = gate ? 1.f / (1.f + expf(-to_f32<T>(gate[t * gate_ld + h * vdim + i]))) : 1.f;
    out[idx] = from_f32<T>(acc * gv);
  }
}

template <typename T>
int run_conv_norm_rope_write(const T* proj, int ld, const float* bias, const float* taps_w, int taps, T* conv_state, const float* q_weight,
                             const float* k_weight, float eps, const float* inv_freq, int rot_dims, const int* positions,
                             const int* token_seq, const int* seq_q_start, const int* seq_q_len, const int* seq_slot,
                             const int* seq_kv_len, const int* block_table, int max_pages, int num_pages, T* k_arena, T* v_arena,
                             T* q_out, int tokens, int seqs, int q_heads, int kv_heads, int dim, int vdim, int row_dim, int page_size,
                             int write_kv, int* err, cudaStream_t stream) {
  const int channels = (q_heads + kv_heads) * dim + kv_heads * vdim;
  const int threads = channels >= 1024 ? 256 : 128;
  const size_t smem = sizeof(float) * channels;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(conv_norm_rope_write_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  launch_kernel(conv_norm_rope_write_kernel<T>, dim3(tokens), dim3(threads), smem, stream, proj, ld, bias, taps_w, taps,
                static_cast<const T*>(conv_state), q_weight, k_weight, eps, inv_freq, rot_dims, positions, token_seq, seq_q_start, seq_slot,
                seq_kv_len, block_table, max_pages, num_pages, k_arena, v_arena, q_out, q_heads, kv_heads, dim, vdim, row_dim, page_size,
                write_kv, err);
  if (int status = b200_check_launch("conv_norm_rope_write")) return status;
  if (taps > 1) {
    launch_kernel(conv_slot_update_kernel<T>, dim3(seqs), dim3(threads), 0, stream, proj, ld, channels, taps, seq_q_start, seq_q_len, seq_slot,
                  conv_state);
    return b200_check_launch("conv_slot_update");
  }
  return 0;
}

}  // namespace

B200_API int b200_conv_norm_rope_write(const void* proj, int ld, const float* bias, const float* taps_w, int taps, void* conv_state,
                                       const float* q_weight, const float* k_weight, float eps, const float* inv_freq, int rot_dims,
                                       const int* positions, const int* token_seq, const int* seq_q_start, const int* seq_q_len,
                                       const int* seq_slot, const int* seq_kv_len, const int* block_table, int max_pages, int num_pages,
                                       void* k_arena, void* v_arena, void* q_out, int tokens, int seqs, int q_heads, int kv_heads,
                                       int dim, int vdim, int row_dim, int page_size, int write_kv, int dtype, int* err,
                                       cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && seqs > 0 && q_heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && row_dim >= dim && row_dim >= vdim && taps >= 1,
               "conv_norm_rope_write: bad sizes");
  B200_REQUIRE(ld >= (q_heads + kv_heads) * dim + kv_heads * vdim, "conv_norm_rope_write: rows of %d numbers do not hold the projections", ld);
  B200_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim && (rot_dims == 0 || inv_freq != nullptr),
               "conv_norm_rope_write: %d rotated dims of %d", rot_dims, dim);
  B200_REQUIRE(sizeof(float) * ((q_heads + kv_heads) * dim + kv_heads * vdim) <= 200 * 1024, "conv_norm_rope_write: a token's projections do not fit shared memory");
  if (dtype == DTYPE_F32)
    return run_conv_norm_rope_write(static_cast<const float*>(proj), ld, bias, taps_w, taps, static_cast<float*>(conv_state), q_weight,
                                    k_weight, eps, inv_freq, rot_dims, positions, token_seq, seq_q_start, seq_q_len, seq_slot, seq_kv_len,
                                    block_table, max_pages, num_pages, static_cast<float*>(k_arena), static_cast<float*>(v_arena),
                                    static_cast<float*>(q_out), tokens, seqs, q_heads, kv_heads, dim, vdim, row_dim, page_size, write_kv, err,
                                    stream);
  if (dtype == DTYPE_BF16)
    return run_conv_norm_rope_write(static_cast<const __nv_bfloat16*>(proj), ld, bias, taps_w, taps, static_cast<__nv_bfloat16*>(conv_state),
                                    q_weight, k_weight, eps, inv_freq, rot_dims, positions, token_seq, seq_q_start, seq_q_len, seq_slot,
                                    seq_kv_len, block_table, max_pages, num_pages, static_cast<__nv_bfloat16*>(k_arena),
                                    static_cast<__nv_bfloat16*>(v_arena), static_cast<__nv_bfloat16*>(q_out), tokens, seqs, q_heads, kv_heads,
                                    dim, vdim, row_dim, page_size, write_kv, err, stream);
  return b200_fail("conv_norm_rope_write: unknown dtype %d", dtype);
}

B200_API int b200_mix_heads_gate(const void* attn, const float* mix, const void* gate, int gate_ld, int tokens, int heads, int kv_heads,
                                 int vdim, int row_dim, void* out, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && vdim > 0 && row_dim >= vdim, "mix_heads_gate: bad sizes");
  const int threads = 256;
  const int64_t total = static_cast<int64_t>(tokens) * heads * vdim;
  const int64_t want = (total + threads - 1) / threads;
  const dim3 grid(static_cast<unsigned>(want < 65535 ? want : 65535));
  if (dtype == DTYPE_F32) {
    launch_kernel(mix_heads_gate_kernel<float>, grid, dim3(threads), 0, stream, static_cast<const float*>(attn), mix,
                  static_cast<const float*>(gate), gate_ld, tokens, heads, kv_heads, vdim, row_dim, static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(mix_heads_gate_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(attn), mix,
                  static_cast<const __nv_bfloat16*>(gate), gate_ld, tokens, heads, kv_heads, vdim, row_dim, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("mix_heads_gate: unknown dtype %d", dtype);
  }
  return b200_check_launch("mix_heads_gate");
}
