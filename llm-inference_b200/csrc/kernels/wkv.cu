// A recurrent mixer with a matrix state per head and a decay per head and key channel, read out
// before the token's own write except for a bonus on the current token.
//
// Per head, with a state S [dk][dv] (32-bit, zero at a request's start) carried from token to token:
//   o_t = (S + diag(u) k_t v_t^T)^T r_t = S^T r_t + (sum_i r_i u_i k_i) v_t;   S <- diag(w_t) S + k_t v_t^T.
// Each of the five projections in front reads its own blend of the token's input h and the previous
// token's: h + (h' - h) mu (h' = 0 for a request's first token); the last input of a request lives in
// its state slot next to S. w = exp(-exp(lw + w0)) with lw a low-rank projection. Each head's o is
// divided by its root mean square, multiplied by a weight per channel and by silu(gate).
//
// Kernels: `wkv_shift_mix` (one block per token: the five blends), `wkv_shift_update` (one block per
// request: the slot's last input), `wkv_prepare` (one block per token: r, k, v as 32-bit, the decay,
// the bonus scalar), `wkv_recurrence` (the columns of S are independent, so a thread group owns a
// column and walks the request's tokens), `wkv_output`.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// out[s][t][:] = h[t] + (prev - h[t]) * mu[s], s < blends; prev is row t - 1 of the step when that is
// the same request's, else the request's slot (zeros after admission).
template <typename T>
__global__ void wkv_shift_mix_kernel(const T* h, const T* shift, const float* __restrict__ mu, const int* __restrict__ token_seq,
                                     const int* seq_q_start, const int* seq_slot, int tokens, int hidden, int blends, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x;
  const int seq = token_seq[t];
  const T* prev = t > seq_q_start[seq] ? h + static_cast<int64_t>(t - 1) * hidden : shift + static_cast<int64_t>(seq_slot[seq]) * hidden;
  const T* cur = h + static_cast<int64_t>(t) * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float x = to_f32<T>(cur[d]);
    const float diff = to_f32<T>(prev[d]) - x;
    for (int s = 0; s < blends; ++s)
      out[(static_cast<int64_t>(s) * tokens + t) * hidden + d] = from_f32<T>(fmaf(diff, mu[s * hidden + d], x));
  }
}

// x <- tanh(x) in place (the activation between the decay's two small projections).
template <typename T>
__global__ void tanh_rows_kernel(T* x, int64_t count) {
  wait_for_predecessor();
  let_successor_start();
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    x[i] = from_f32<T>(tanhf(to_f32<T>(x[i])));
}

template <typename T>
__global__ void wkv_shift_update_kernel(const T* h, T* shift, const int* seq_q_start, const int* seq_q_len, const int* seq_slot,
                                        int hidden) {
  wait_for_predecessor();
  let_successor_start();
  const int seq = blockIdx.x;
  const int len = seq_q_len[seq];
  if (len <= 0) return;
  const T* last = h + static_cast<int64_t>(seq_q_start[seq] + len - 1) * hidden;
  T* dst = shift + static_cast<int64_t>(seq_slot[seq]) * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) dst[d] = last[d];
}

// r, k, v [tokens][heads*dim] in T -> 32-bit copies; decay = exp(-exp(lw + w0)); bonus[t][h] = sum_i r_i u_i k_i.
template <typename T>
__global__ void wkv_prepare_kernel(const T* r, const T* k, const T* v, const float* lw, const float* __restrict__ w0,
                                   const float* __restrict__ u, int heads, int dim, float* r_out, float* k_out, float* v_out,
                                   float* decay_out, float* bonus_out) {
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int64_t base = static_cast<int64_t>(t) * heads * dim;
  for (int head = warp; head < heads; head += warps) {
    float acc = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const int c = head * dim + i;
      const float rv = to_f32<T>(r[base + c]), kv = to_f32<T>(k[base + c]);
      r_out[base + c] = rv;
      k_out[base + c] = kv;
      v_out[base + c] = to_f32<T>(v[base + c]);
      decay_out[base + c] = expf(-expf(lw[base + c] + w0[c]));
      acc = fmaf(rv * u[c], kv, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) bonus_out[static_cast<int64_t>(t) * heads + head] = acc;
  }
}

// A block owns `cols` columns of one head of one request; a column's dk rows are spread over
// `lanes_per_col` neighbouring lanes (row r on lane r % lanes_per_col), PER rows per lane in
// registers. The tokens' r, k, w, v and bonus arrive kStage at a time by cp.async in a ring of two
// stages, so the next tokens load while these are worked on.
constexpr int kRecurrenceThreads = 128;
constexpr int kStage = 8;

template <int kBytes>
__device__ __forceinline__ void stage_copy(float* smem, const float* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? kBytes : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(s), "l"(gmem), "n"(kBytes), "r"(bytes) : "memory");
}

template <int PER, int LANES>
__global__ void __launch_bounds__(kRecurrenceThreads)
wkv_recurrence_kernel(const float* r, const float* k, const float* v, const float* bonus, const float* decay, const int* seq_q_start,
                      const int* seq_q_len, const int* seq_slot, int heads, int dk, int dv, int vec, float* state, float* out) {
  extern __shared__ __align__(16) float stage[];
  let_successor_start();
  constexpr int lanes_per_col = LANES;
  constexpr int cols = kRecurrenceThreads / lanes_per_col;
  const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
  const int tid = threadIdx.x;
  const int part = tid % lanes_per_col, col = col0 + tid / lanes_per_col;
  constexpr int padded = PER * lanes_per_col;
  constexpr int per_stage = kStage * (3 * padded + cols) + kStage;
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  const bool live = col < dv;
  float* s_base = state + (static_cast<int64_t>(seq_slot[seq]) * heads + head) * dk * dv;
  wait_for_predecessor();
  // Rows past dk (when dk is no multiple of the lanes) hold zeros in r, k and w and stay zero.
  auto fetch = [&](int buffer, int t0) {
    float* sr = stage + buffer * per_stage;
    float* sk = sr + kStage * padded;
    float* sw = sk + kStage * padded;
    float* sv = sw + kStage * padded;
    float* sb = sv + kStage * cols;
    const int count = min(kStage, len - t0);
    const int64_t first = static_cast<int64_t>(start) + t0;
    if (vec) {
      for (int idx = tid * 4; idx < count * padded; idx += kRecurrenceThreads * 4) {
        const int j = idx / padded, row = idx % padded;
        const int64_t at = ((first + j) * heads + head) * dk + (row < dk ? row : 0);
        stage_copy<16>(sr + idx, r + at, row < dk);
        stage_copy<16>(sk + idx, k + at, row < dk);
        stage_copy<16>(sw + idx, decay + at, row < dk);
      }
      for (int idx = tid * 4; idx < count * cols; idx += kRecurrenceThreads * 4) {
        const int j = idx / cols, c = col0 + idx % cols;
        stage_copy<16>(sv + idx, v + ((first + j) * heads + head) * dv + (c < dv ? c : 0), c < dv);
      }
    } else {
      for (int idx = tid; idx < count * padded; idx += kRecurrenceThreads) {
        const int j = idx / padded, row = idx % padded;
        const int64_t at = ((first + j) * heads + head) * dk + (row < dk ? row : 0);
        stage_copy<4>(sr + idx, r + at, row < dk);
        stage_copy<4>(sk + idx, k + at, row < dk);
        stage_copy<4>(sw + idx, decay + at, row < dk);
      }
      for (int idx = tid; idx < count * cols; idx += kRecurrenceThreads) {
        const int j = idx / cols, c = col0 + idx % cols;
        stage_copy<4>(sv + idx, v + ((first + j) * heads + head) * dv + (c < dv ? c : 0), c < dv);
      }
    }
    if (tid < count) stage_copy<4>(sb + tid, bonus + (first + tid) * heads + head, true);
  };
  float s[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int row = i * lanes_per_col + part;
    s[i] = (live && row < dk) ? s_base[static_cast<int64_t>(row) * dv + col] : 0.f;
  }
  if (len > 0) fetch(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int t0 = 0, buffer = 0; t0 < len; t0 += kStage, buffer ^= 1) {
    if (t0 + kStage < len) fetch(buffer ^ 1, t0 + kStage);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const float* sr = stage + buffer * per_stage;
    const float* sk = sr + kStage * padded;
    const float* sw = sk + kStage * padded;
    const float* sv = sw + kStage * padded;
    const float* sb = sv + kStage * cols;
    const int count = min(kStage, len - t0);
    for (int j = 0; j < count; ++j) {
      const float* rj = sr + j * padded + part;
      const float* kj = sk + j * padded + part;
      const float* wj = sw + j * padded + part;
      const float vc = sv[j * cols + tid / lanes_per_col];
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int i = 0; i < PER; i += 2) {
        rs0 = fmaf(rj[i * lanes_per_col], s[i], rs0), rs1 = fmaf(rj[(i + 1) * lanes_per_col], s[i + 1], rs1);
        s[i] = fmaf(wj[i * lanes_per_col], s[i], kj[i * lanes_per_col] * vc);
        s[i + 1] = fmaf(wj[(i + 1) * lanes_per_col], s[i + 1], kj[(i + 1) * lanes_per_col] * vc);
      }
      float rs = rs0 + rs1;
#pragma unroll
      for (int o = lanes_per_col >> 1; o > 0; o >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
      if (live && part == 0) out[(static_cast<int64_t>(start) + t0 + j) * heads * dv + head * dv + col] = fmaf(sb[j], vc, rs);
    }
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int row = i * lanes_per_col + part;
    if (live && row < dk) s_base[static_cast<int64_t>(row) * dv + col] = s[i];
  }
}

// out[t, h, :] = o / rms(o) * weight[h, :] * act(gate[t, h, :]), act = silu, or sigmoid with `sigmoid_gate`; one warp
// per (token, head). Gate rows are `gate_ld` numbers apart.
template <typename T>
__global__ void wkv_output_kernel(const float* o, const float* __restrict__ weight, const T* gate, int gate_ld, int rows, int heads,
                                  int dv, float eps, int sigmoid_gate, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<int64_t>(rows) * heads) return;
  const int h = static_cast<int>(item % heads);
  const float* src = o + item * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(src[i], src[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(dv) + eps);
  const T* g = gate + (item / heads) * gate_ld + h * dv;
  T* dst = out + item * dv;
  for (int i = lane; i < dv; i += 32) {
    const float gv = to_f32<T>(g[i]);
    dst[i] = from_f32<T>(src[i] * inv * weight[h * dv + i] * (sigmoid_gate ? sigmoid_f(gv) : gv * sigmoid_f(gv)));
  }
}

}  // namespace

B200_API int b200_wkv_shift_mix(const void* h, void* shift, const float* mu, const int* token_seq, const int* seq_q_start,
                                const int* seq_q_len, const int* seq_slot, int tokens, int seqs, int hidden, int blends, void* out,
                                int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && seqs > 0 && hidden > 0 && blends > 0, "wkv_shift_mix: bad sizes");
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == DTYPE_F32) {
    launch_kernel(wkv_shift_mix_kernel<float>, dim3(tokens), dim3(threads), 0, stream, static_cast<const float*>(h),
                  static_cast<const float*>(shift), mu, token_seq, seq_q_start, seq_slot, tokens, hidden, blends, static_cast<float*>(out));
    if (int status = b200_check_launch("wkv_shift_mix")) return status;
    launch_kernel(wkv_shift_update_kernel<float>, dim3(seqs), dim3(threads), 0, stream, static_cast<const float*>(h),
                  static_cast<float*>(shift), seq_q_start, seq_q_len, seq_slot, hidden);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(wkv_shift_mix_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(h),
                  static_cast<const __nv_bfloat16*>(shift), mu, token_seq, seq_q_start, seq_slot, tokens, hidden, blends,
                  static_cast<__nv_bfloat16*>(out));
    if (int status = b200_check_launch("wkv_shift_mix")) return status;
    launch_kernel(wkv_shift_update_kernel<__nv_bfloat16>, dim3(seqs), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(h),
                  static_cast<__nv_bfloat16*>(shift), seq_q_start, seq_q_len, seq_slot, hidden);
  } else {
    return b200_fail("wkv_shift_mix: unknown dtype %d", dtype);
  }
  return b200_check_launch("wkv_shift_update");
}

B200_API int b200_tanh_rows(void* x, int64_t count, int dtype, cudaStream_t stream) {
  if (count == 0) return 0;
  B200_REQUIRE(count > 0, "tanh_rows: bad size");
  const int threads = 256;
  const int64_t want = (count + threads - 1) / threads;
  const dim3 grid(static_cast<unsigned>(want < 65535 ? want : 65535));
  if (dtype == DTYPE_F32) launch_kernel(tanh_rows_kernel<float>, grid, dim3(threads), 0, stream, static_cast<float*>(x), count);
  else if (dtype == DTYPE_BF16) launch_kernel(tanh_rows_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, static_cast<__nv_bfloat16*>(x), count);
  else return b200_fail("tanh_rows: unknown dtype %d", dtype);
  return b200_check_launch("tanh_rows");
}

B200_API int b200_wkv_prepare(const void* r, const void* k, const void* v, const float* lw, const float* w0, const float* u, int tokens,
                              int heads, int dim, float* r_out, float* k_out, float* v_out, float* decay_out, float* bonus_out,
                              int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && heads > 0 && dim > 0, "wkv_prepare: bad sizes");
  const int threads = 128;
  if (dtype == DTYPE_F32) {
    launch_kernel(wkv_prepare_kernel<float>, dim3(tokens), dim3(threads), 0, stream, static_cast<const float*>(r),
                  static_cast<const float*>(k), static_cast<const float*>(v), lw, w0, u, heads, dim, r_out, k_out, v_out, decay_out,
                  bonus_out);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(wkv_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(r),
                  static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), lw, w0, u, heads, dim, r_out, k_out, v_out,
                  decay_out, bonus_out);
  } else {
    return b200_fail("wkv_prepare: unknown dtype %d", dtype);
  }
  return b200_check_launch("wkv_prepare");
}

B200_API int b200_wkv_recurrence(const float* r, const float* k, const float* v, const float* bonus, const float* decay,
                                 const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int seqs, int heads, int dk, int dv,
                                 float* state, float* out, cudaStream_t stream) {
  if (seqs == 0) return 0;
  B200_REQUIRE(seqs > 0 && heads > 0 && heads <= 65535 && dk > 0 && dv > 0, "wkv_recurrence: bad sizes");
  B200_REQUIRE(dk <= 1024, "wkv_recurrence: %d key channels per head, at most 1024", dk);
  // Lanes per column: enough that a lane holds at most 8 rows (up to 32 rows when even a whole warp
  // per column leaves more).
  int lanes = 1;
  while ((dk + lanes - 1) / lanes > 8 && lanes < 32) lanes *= 2;
  const int rows = (dk + lanes - 1) / lanes;
  const int per = rows <= 8 ? 8 : (rows <= 16 ? 16 : 32);
  const int cols = kRecurrenceThreads / lanes;
  const dim3 grid(seqs, heads, (dv + cols - 1) / cols);
  B200_REQUIRE(grid.z <= 65535, "wkv_recurrence: too many columns");
  const size_t smem = sizeof(float) * 2 * (kStage * (3 * per * lanes + cols) + kStage);
  const auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const int vec = dk % 4 == 0 && dv % 4 == 0 && aligned(r) && aligned(k) && aligned(v) && aligned(decay) ? 1 : 0;
  B200_REQUIRE(smem <= 200 * 1024, "wkv_recurrence: the staged tokens do not fit shared memory");
  auto launch = [&](auto kernel) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_kernel(kernel, grid, dim3(kRecurrenceThreads), smem, stream, r, k, v, bonus, decay, seq_q_start, seq_q_len, seq_slot, heads,
                  dk, dv, vec, state, out);
  };
  if (per == 32) launch(wkv_recurrence_kernel<32, 32>);
  else if (per == 16) launch(wkv_recurrence_kernel<16, 32>);
  else if (lanes == 32) launch(wkv_recurrence_kernel<8, 32>);
  else if (lanes == 16) launch(wkv_recurrence_kernel<8, 16>);
  else if (lanes == 8) launch(wkv_recurrence_kernel<8, 8>);
  else if (lanes == 4) launch(wkv_recurrence_kernel<8, 4>);
  else if (lanes == 2) launch(wkv_recurrence_kernel<8, 2>);
  else launch(wkv_recurrence_kernel<8, 1>);
  return b200_check_launch("wkv_recurrence");
}

B200_API int b200_wkv_output(const float* o, const float* weight, const void* gate, int gate_ld, int rows, int heads, int dv, float eps,
                             int sigmoid_gate, void* out, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && heads > 0 && dv > 0 && gate_ld >= heads * dv, "wkv_output: bad sizes");
  const int threads = 128;
  const int64_t items = static_cast<int64_t>(rows) * heads;
  const unsigned blocks = static_cast<unsigned>((items + 3) / 4);
  if (dtype == DTYPE_F32) {
    launch_kernel(wkv_output_kernel<float>, dim3(blocks), dim3(threads), 0, stream, o, weight, static_cast<const float*>(gate), gate_ld,
                  rows, heads, dv, eps, sigmoid_gate, static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(wkv_output_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, o, weight,
                  static_cast<const __nv_bfloat16*>(gate), gate_ld, rows, heads, dv, eps, sigmoid_gate, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("wkv_output: unknown dtype %d", dtype);
  }
  return b200_check_launch("wkv_output");
}
