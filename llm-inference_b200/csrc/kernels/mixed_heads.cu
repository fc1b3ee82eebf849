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
#include <type_traits>

#include "common.cuh"
#include "page_tail.cuh"

namespace {

// kWide neighbouring numbers as one load or store (kWide = 2 where every size involved is even).
template <typename T, int kWide>
__device__ __forceinline__ void load_wide(const T* p, float (&v)[kWide]) {
  if constexpr (kWide == 1) {
    v[0] = to_f32<T>(*p);
  } else if constexpr (sizeof(T) == 2) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    v[0] = f.x, v[1] = f.y;
  } else {
    const float2 f = *reinterpret_cast<const float2*>(p);
    v[0] = f.x, v[1] = f.y;
  }
}
template <typename T, int kWide>
__device__ __forceinline__ void store_wide(T* p, const float (&v)[kWide]) {
  if constexpr (kWide == 1) {
    *p = from_f32<T>(v[0]);
  } else if constexpr (sizeof(T) == 2) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
  } else {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  }
}

template <typename T, int kWide>
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
  float sq = 0.f, sk = 0.f;
  for (int c = tid * kWide; c < channels; c += blockDim.x * kWide) {
    float acc[kWide];
#pragma unroll
    for (int e = 0; e < kWide; ++e) acc[e] = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;  // how many tokens before t
      if (back > pos) continue;       // in front of the request's first token
      float x[kWide];
      load_wide<T, kWide>(back <= run ? proj + static_cast<int64_t>(t - back) * ld + c
                                      : state + static_cast<int64_t>(taps - 1 + run - back) * channels + c, x);
#pragma unroll
      for (int e = 0; e < kWide; ++e) acc[e] = fmaf(taps_w[(c + e) * taps + j], x[e] + (bias ? bias[c + e] : 0.f), acc[e]);
    }
#pragma unroll
    for (int e = 0; e < kWide; ++e) {
      y[c + e] = acc[e];
      if (c < qw) sq = fmaf(acc[e], acc[e], sq);
      else if (c < qw + kw) sk = fmaf(acc[e], acc[e], sk);
    }
  }
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);  // (its barriers also make y visible to the whole block)
  const float inv_q = 1.f / sqrtf(sq / static_cast<float>(qw) + eps);
  const float inv_k = 1.f / sqrtf(sk / static_cast<float>(kw) + eps);
  const float p = static_cast<float>(pos);
  // queries and keys: (q_heads + kv_heads) rows of row_dim numbers; a pair of neighbours (2i, 2i + 1) is rotated together
  const int qk_rows = q_heads + kv_heads;
  for (int idx = tid * kWide; idx < qk_rows * row_dim; idx += blockDim.x * kWide) {
    const int head = idx / row_dim, i = idx - head * row_dim;
    const bool is_q = head < q_heads;
    float value[kWide];
#pragma unroll
    for (int e = 0; e < kWide; ++e) value[e] = 0.f;
    if (i < dim) {
      const int c = head * dim + i;  // keys follow the queries in y
      const float* weight = is_q ? q_weight + c : k_weight + (c - qw);
      const float inv = is_q ? inv_q : inv_k;
      if constexpr (kWide == 2) {
        const float a = y[c] * inv * weight[0], b = y[c + 1] * inv * weight[1];
        value[0] = a, value[1] = b;
        if (i < rot_dims) {
          float sn, cs;
          sincosf(p * inv_freq[i >> 1], &sn, &cs);
          value[0] = fmaf(a, cs, -b * sn);
          value[1] = fmaf(b, cs, a * sn);
        }
      } else {
        value[0] = y[c] * inv * weight[0];
        if (i < rot_dims) {
          float sn, cs;
          sincosf(p * inv_freq[i >> 1], &sn, &cs);
          const int o = (i ^ 1) - i;
          const float other = y[c + o] * inv * weight[o];
          value[0] = (i & 1) ? fmaf(value[0], cs, other * sn) : fmaf(value[0], cs, -other * sn);
        }
      }
    }
    if (is_q) {
      store_wide<T, kWide>(q_out + (static_cast<int64_t>(t) * q_heads + head) * row_dim + i, value);
    } else if (page >= 0) {
      store_wide<T, kWide>(k_arena + kv_row_offset(page, head - q_heads, pos % page_size, kv_heads, page_size, row_dim) + i, value);
    }
  }
  if (page >= 0) {
    for (int idx = tid * kWide; idx < kv_heads * row_dim; idx += blockDim.x * kWide) {
      const int head = idx / row_dim, i = idx - head * row_dim;
      float value[kWide];
#pragma unroll
      for (int e = 0; e < kWide; ++e) value[e] = i + e < vdim ? y[qw + kw + head * vdim + i + e] : 0.f;
      store_wide<T, kWide>(v_arena + kv_row_offset(page, head, pos % page_size, kv_heads, page_size, row_dim) + i, value);
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

// attn [kv_heads][tokens][heads][row_dim]; gate logits at gate[t * gate_ld + h * vdim + i]. A thread forms kVec
// neighbouring numbers of one head's output from 16-byte loads (kVec = 8 bfloat16 or 4 floats); with sizes or
// addresses that do not allow those, kVec = 1.
template <typename T, int kVec>
__global__ void mix_heads_gate_kernel(const T* attn, const float* __restrict__ mix, const T* gate, int gate_ld, int tokens, int heads,
                                      int kv_heads, int vdim, int row_dim, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int group = heads / kv_heads;
  const int chunks = vdim / kVec;
  const int64_t total = static_cast<int64_t>(tokens) * heads * chunks;
  const int64_t plane = static_cast<int64_t>(tokens) * heads * row_dim;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % chunks) * kVec;
    const int64_t th = idx / chunks;
    const int h = static_cast<int>(th % heads);
    const int64_t t = th / heads;
    const T* src = attn + (h / group) * plane + t * heads * row_dim + i;
    float acc[kVec];
#pragma unroll
    for (int e = 0; e < kVec; ++e) acc[e] = 0.f;
    for (int g = 0; g < heads; ++g) {
      const float m = mix[h * heads + g];
      alignas(16) T values[kVec];
      if constexpr (kVec > 1) {
        *reinterpret_cast<uint4*>(values) = *reinterpret_cast<const uint4*>(src + static_cast<int64_t>(g) * row_dim);
      } else {
        values[0] = src[static_cast<int64_t>(g) * row_dim];
      }
#pragma unroll
      for (int e = 0; e < kVec; ++e) acc[e] = fmaf(m, to_f32<T>(values[e]), acc[e]);
    }
    alignas(16) T gates[kVec];
    alignas(16) T result[kVec];
    if (gate) {
      if constexpr (kVec > 1) {
        *reinterpret_cast<uint4*>(gates) = *reinterpret_cast<const uint4*>(gate + t * gate_ld + h * vdim + i);
      } else {
        gates[0] = gate[t * gate_ld + h * vdim + i];
      }
    }
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      const float gv = gate ? 1.f / (1.f + expf(-to_f32<T>(gates[e]))) : 1.f;
      result[e] = from_f32<T>(acc[e] * gv);
    }
    T* dst = out + (t * heads + h) * vdim + i;
    if constexpr (kVec > 1) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(result);
    } else {
      dst[0] = result[0];
    }
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
  // Pairs of neighbours where every size is even (two numbers per load and store, one sine and cosine per rotated pair).
  const bool pairs = dim % 2 == 0 && vdim % 2 == 0 && row_dim % 2 == 0 && ld % 2 == 0;
  // A step of few tokens has few blocks: each then gets as many threads as it has pairs, up to 1,024.
  int threads = channels >= 1024 ? 256 : 128;
  if (tokens <= 64) {
    const int items = (q_heads + kv_heads) * row_dim / (pairs ? 2 : 1);
    threads = items >= 1024 ? 1024 : (items >= 512 ? 512 : threads);
  }
  const size_t smem = sizeof(float) * channels;
  auto launch = [&](auto kernel) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_kernel(kernel, dim3(tokens), dim3(threads), smem, stream, proj, ld, bias, taps_w, taps, static_cast<const T*>(conv_state), q_weight,
                  k_weight, eps, inv_freq, rot_dims, positions, token_seq, seq_q_start, seq_slot, seq_kv_len, block_table, max_pages,
                  num_pages, k_arena, v_arena, q_out, q_heads, kv_heads, dim, vdim, row_dim, page_size, write_kv, err);
  };
  if (pairs) launch(conv_norm_rope_write_kernel<T, 2>);
  else launch(conv_norm_rope_write_kernel<T, 1>);
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
  B200_REQUIRE(dtype == DTYPE_F32 || dtype == DTYPE_BF16, "mix_heads_gate: unknown dtype %d", dtype);
  const int threads = 256;
  const int wide = dtype == DTYPE_F32 ? 4 : 8;  // numbers in 16 bytes
  const auto aligned = [](const void* p) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = vdim % wide == 0 && row_dim % wide == 0 && gate_ld % wide == 0 && aligned(attn) && aligned(gate) && aligned(out);
  const int64_t total = static_cast<int64_t>(tokens) * heads * (vec ? vdim / wide : vdim);
  const int64_t want = (total + threads - 1) / threads;
  const dim3 grid(static_cast<unsigned>(want < 65535 * 8 ? want : 65535 * 8));
  auto launch = [&](auto kernel, auto* typed) {
    using P = decltype(typed);
    launch_kernel(kernel, grid, dim3(threads), 0, stream, static_cast<const std::remove_pointer_t<P>*>(attn), mix,
                  static_cast<const std::remove_pointer_t<P>*>(gate), gate_ld, tokens, heads, kv_heads, vdim, row_dim, static_cast<P>(out));
  };
  if (dtype == DTYPE_F32) {
    if (vec) launch(mix_heads_gate_kernel<float, 4>, static_cast<float*>(nullptr));
    else launch(mix_heads_gate_kernel<float, 1>, static_cast<float*>(nullptr));
  } else {
    if (vec) launch(mix_heads_gate_kernel<__nv_bfloat16, 8>, static_cast<__nv_bfloat16*>(nullptr));
    else launch(mix_heads_gate_kernel<__nv_bfloat16, 1>, static_cast<__nv_bfloat16*>(nullptr));
  }
  return b200_check_launch("mix_heads_gate");
}
