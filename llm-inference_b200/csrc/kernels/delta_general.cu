// The generalized delta rule: a matrix state per head with a decay per key channel and the removal of
// a learned share of what the state holds along the current key's direction.
//
// Per head, with a state S [dk][dv] (32-bit, zero at a request's start) carried from token to token:
//   S <- diag(w) S - (a (.) u) (u^T S) + k v^T   (both terms read the old S),   o = S^T r   (the new S),
// u = k / sqrt(sum k^2 + 1e-6) the key's direction, w = exp(-e^(-1/2) sigmoid(lw + w0)) with lw a
// low-rank projection, a = sigmoid(pa + a_bias) the share removed per key channel. Everything the
// recurrence reads is 32-bit.
//
// Kernels: `delta_general_prepare` (one warp per token and head: r, k, v as 32-bit, w, a (.) u and u),
// `delta_general_recurrence` (the columns of S are independent: column c follows
// s <- w (.) s - (a (.) u) (u . s) + k v_c, so a thread group owns a column and walks the request's tokens).
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

constexpr float kDecayRate = 0.60653065971263342f;  // e^(-1/2)

// proj rows: r, k, v, pa at column offsets r_at, k_at, v_at, a_at (heads*dim numbers each), `ld` apart.
template <typename T>
__global__ void delta_general_prepare_kernel(const T* proj, int ld, int r_at, int k_at, int v_at, int a_at, const float* lw,
                                             const float* __restrict__ w0, const float* __restrict__ a_bias, int heads, int dim,
                                             float* r_out, float* k_out, float* v_out, float* w_out, float* au_out, float* u_out) {
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const T* row = proj + static_cast<int64_t>(t) * ld;
  const int64_t base = static_cast<int64_t>(t) * heads * dim;
  for (int head = blockIdx.y * warps + warp; head < heads; head += gridDim.y * warps) {
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float kv = to_f32<T>(row[k_at + head * dim + i]);
      ss = fmaf(kv, kv, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss + 1e-6f);
    for (int i = lane; i < dim; i += 32) {
      const int c = head * dim + i;
      const float kv = to_f32<T>(row[k_at + c]);
      const float u = kv * inv;
      r_out[base + c] = to_f32<T>(row[r_at + c]);
      k_out[base + c] = kv;
      v_out[base + c] = to_f32<T>(row[v_at + c]);
      w_out[base + c] = expf(-kDecayRate * sigmoid_f(lw[base + c] + w0[c]));
      au_out[base + c] = sigmoid_f(to_f32<T>(row[a_at + c]) + a_bias[c]) * u;
      u_out[base + c] = u;
    }
  }
}

// A block owns `cols` columns of one head of one request; a column's dk rows are spread over
// `lanes_per_col` neighbouring lanes, PER neighbouring rows per lane in registers (rows lane * PER ..).
// A lane reads four neighbouring numbers of each vector with one 16-byte load; in shared memory a lane's
// rows are followed by four unused numbers, which puts the eight lanes that load together on different
// banks. (Four rows per lane instead of eight, with twice the lanes per column, was slower: 0.36 against
// 0.28 us per token for 24 heads of 64 x 64, more blocks than SMs and one more step in both sums over lanes.)
// The tokens' r, k, w, a (.) u, u and v arrive kStage at a time by cp.async in a ring of two stages,
// so the next tokens load while these are worked on.
constexpr int kRecurrenceThreads = 128;
constexpr int kStage = 8;
constexpr int kVectors = 5;  // r, k, w, au, u

template <int kBytes>
__device__ __forceinline__ void stage_copy(float* smem, const float* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? kBytes : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(s), "l"(gmem), "n"(kBytes), "r"(bytes) : "memory");
}

template <int PER, int LANES>
__global__ void __launch_bounds__(kRecurrenceThreads)
delta_general_recurrence_kernel(const float* r, const float* k, const float* v, const float* w, const float* au, const float* u,
                                const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int heads, int dk, int dv, int vec,
                                float* state, float* out) {
  extern __shared__ __align__(16) float stage[];
  let_successor_start();
  constexpr int lanes_per_col = LANES;
  constexpr int cols = kRecurrenceThreads / lanes_per_col;
  const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
  const int tid = threadIdx.x;
  const int part = tid % lanes_per_col, col = col0 + tid / lanes_per_col;
  constexpr int lane_span = PER + 4;  // a lane's rows in shared memory, and four numbers nobody reads
  constexpr int padded = lane_span * lanes_per_col;
  constexpr int per_stage = kStage * (kVectors * padded + cols);
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  const bool live = col < dv;
  float* s_base = state + (static_cast<int64_t>(seq_slot[seq]) * heads + head) * dk * dv;
  wait_for_predecessor();
  const float* sources[kVectors] = {r, k, w, au, u};
  // Rows past dk (when dk is no multiple of the lanes) hold zeros in all five vectors and stay zero.
  auto fetch = [&](int buffer, int t0) {
    float* base = stage + buffer * per_stage;
    float* sv = base + kVectors * kStage * padded;
    const int count = min(kStage, len - t0);
    const int64_t first = static_cast<int64_t>(start) + t0;
    if (vec) {
      for (int idx = tid * 4; idx < count * padded; idx += kRecurrenceThreads * 4) {
        const int j = idx / padded, place = idx % padded;
        if (place % lane_span >= PER) continue;
        const int row = place / lane_span * PER + place % lane_span;
        const int64_t at = ((first + j) * heads + head) * dk + (row < dk ? row : 0);
#pragma unroll
        for (int n = 0; n < kVectors; ++n) stage_copy<16>(base + n * kStage * padded + idx, sources[n] + at, row < dk);
      }
      for (int idx = tid * 4; idx < count * cols; idx += kRecurrenceThreads * 4) {
        const int j = idx / cols, c = col0 + idx % cols;
        stage_copy<16>(sv + idx, v + ((first + j) * heads + head) * dv + (c < dv ? c : 0), c < dv);
      }
    } else {
      for (int idx = tid; idx < count * padded; idx += kRecurrenceThreads) {
        const int j = idx / padded, place = idx % padded;
        if (place % lane_span >= PER) continue;
        const int row = place / lane_span * PER + place % lane_span;
        const int64_t at = ((first + j) * heads + head) * dk + (row < dk ? row : 0);
#pragma unroll
        for (int n = 0; n < kVectors; ++n) stage_copy<4>(base + n * kStage * padded + idx, sources[n] + at, row < dk);
      }
      for (int idx = tid; idx < count * cols; idx += kRecurrenceThreads) {
        const int j = idx / cols, c = col0 + idx % cols;
        stage_copy<4>(sv + idx, v + ((first + j) * heads + head) * dv + (c < dv ? c : 0), c < dv);
      }
    }
  };
  float s[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int row = part * PER + i;
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
    const float* sa = sw + kStage * padded;
    const float* su = sa + kStage * padded;
    const float* sv = su + kStage * padded;
    const int count = min(kStage, len - t0);
    // The read-out of a token is summed over the lanes together with the next token's u . s: the two sums do not
    // depend on each other, so their shuffles go out in pairs and the warp waits for half as many.
    float pending = 0.f;
    int pending_at = -1;
    auto token = [&](int j) {
      const int at = j * padded + part * lane_span;
      const float vc = sv[j * cols + tid / lanes_per_col];
      float rv[PER], kv[PER], wv[PER], av[PER], uv[PER];
#pragma unroll
      for (int i = 0; i < PER; i += 4) {
        *reinterpret_cast<float4*>(rv + i) = *reinterpret_cast<const float4*>(sr + at + i);
        *reinterpret_cast<float4*>(kv + i) = *reinterpret_cast<const float4*>(sk + at + i);
        *reinterpret_cast<float4*>(wv + i) = *reinterpret_cast<const float4*>(sw + at + i);
        *reinterpret_cast<float4*>(av + i) = *reinterpret_cast<const float4*>(sa + at + i);
        *reinterpret_cast<float4*>(uv + i) = *reinterpret_cast<const float4*>(su + at + i);
      }
      // u . s over the old state
      float d0 = 0.f, d1 = 0.f;
#pragma unroll
      for (int i = 0; i < PER; i += 2) {
        d0 = fmaf(uv[i], s[i], d0);
        d1 = fmaf(uv[i + 1], s[i + 1], d1);
      }
      float dot = d0 + d1;
#pragma unroll
      for (int o = lanes_per_col >> 1; o > 0; o >>= 1) {
        const float from_dot = __shfl_xor_sync(0xffffffffu, dot, o), from_pending = __shfl_xor_sync(0xffffffffu, pending, o);
        dot += from_dot;
        pending += from_pending;
      }
      if (live && part == 0 && pending_at >= 0) out[(static_cast<int64_t>(start) + pending_at) * heads * dv + head * dv + col] = pending;
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int i = 0; i < PER; i += 2) {
        s[i] = fmaf(wv[i], s[i], fmaf(kv[i], vc, -av[i] * dot));
        s[i + 1] = fmaf(wv[i + 1], s[i + 1], fmaf(kv[i + 1], vc, -av[i + 1] * dot));
        rs0 = fmaf(rv[i], s[i], rs0);
        rs1 = fmaf(rv[i + 1], s[i + 1], rs1);
      }
      pending = rs0 + rs1;
      pending_at = t0 + j;
    };
    if (count == kStage) {  // a full stage is unrolled: one token's read-out overlaps the next token's update
#pragma unroll
      for (int j = 0; j < kStage; ++j) token(j);
    } else {
      for (int j = 0; j < count; ++j) token(j);
    }
#pragma unroll
    for (int o = lanes_per_col >> 1; o > 0; o >>= 1) pending += __shfl_xor_sync(0xffffffffu, pending, o);
    if (live && part == 0 && pending_at >= 0) out[(static_cast<int64_t>(start) + pending_at) * heads * dv + head * dv + col] = pending;
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int row = part * PER + i;
    if (live && row < dk) s_base[static_cast<int64_t>(row) * dv + col] = s[i];
  }
}

}  // namespace

B200_API int b200_delta_general_prepare(const void* proj, int ld, int r_at, int k_at, int v_at, int a_at, const float* lw,
                                        const float* w0, const float* a_bias, int tokens, int heads, int dim, float* r_out,
                                        float* k_out, float* v_out, float* w_out, float* au_out, float* u_out, int dtype,
                                        cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && heads > 0 && dim > 0, "delta_general_prepare: bad sizes");
  const int inner = heads * dim;
  B200_REQUIRE(r_at >= 0 && k_at >= 0 && v_at >= 0 && a_at >= 0 && r_at + inner <= ld && k_at + inner <= ld && v_at + inner <= ld &&
                   a_at + inner <= ld,
               "delta_general_prepare: rows of %d numbers do not hold the projections", ld);
  const int threads = 128;
  const dim3 grid(tokens, static_cast<unsigned>(min((heads + 3) / 4, 65535)));  // four warps, a head each
  if (dtype == DTYPE_F32) {
    launch_kernel(delta_general_prepare_kernel<float>, grid, dim3(threads), 0, stream, static_cast<const float*>(proj), ld, r_at,
                  k_at, v_at, a_at, lw, w0, a_bias, heads, dim, r_out, k_out, v_out, w_out, au_out, u_out);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(delta_general_prepare_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream,
                  static_cast<const __nv_bfloat16*>(proj), ld, r_at, k_at, v_at, a_at, lw, w0, a_bias, heads, dim, r_out, k_out, v_out,
                  w_out, au_out, u_out);
  } else {
    return b200_fail("delta_general_prepare: unknown dtype %d", dtype);
  }
  return b200_check_launch("delta_general_prepare");
}

B200_API int b200_delta_general_recurrence(const float* r, const float* k, const float* v, const float* w, const float* au,
                                           const float* u, const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int seqs,
                                           int max_q_len, int heads, int dk, int dv, float* state, float* out, cudaStream_t stream) {
  if (seqs == 0) return 0;
  B200_REQUIRE(seqs > 0 && heads > 0 && heads <= 65535 && dk > 0 && dv > 0, "delta_general_recurrence: bad sizes");
  B200_REQUIRE(dk <= 1024, "delta_general_recurrence: %d key channels per head, at most 1024", dk);
  // Lanes per column: enough that a lane holds at most 8 rows (up to 32 rows when even a whole warp
  // per column leaves more).
  int lanes = 1;
  while ((dk + lanes - 1) / lanes > 8 && lanes < 32) lanes *= 2;
  const int rows = (dk + lanes - 1) / lanes;
  const int per = rows <= 8 ? 8 : (rows <= 16 ? 16 : 32);
  const int cols = kRecurrenceThreads / lanes;
  const dim3 grid(seqs, heads, (dv + cols - 1) / cols);
  B200_REQUIRE(grid.z <= 65535, "delta_general_recurrence: too many columns");
  const size_t smem = sizeof(float) * 2 * (kStage * (kVectors * (per + 4) * lanes + cols));
  const auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const int vec = dk % 4 == 0 && dv % 4 == 0 && aligned(r) && aligned(k) && aligned(v) && aligned(w) && aligned(au) && aligned(u) ? 1 : 0;
  B200_REQUIRE(smem <= 227 * 1024, "delta_general_recurrence: the staged tokens of %d key channels per head do not fit shared memory", dk);
  // A step with prompt portions launches the ordinary way, after the kernel in front has left the SMs. Made resident
  // early, the few blocks of this kernel are packed onto the few SMs the predecessor's last wave leaves free, several
  // to an SM, and walk their tokens there to the end: measured on a B200, 2,048 tokens of 24 heads of 64 x 64 took
  // 1.8 ms that way and 0.63 ms spread one block to an SM. Steps of single tokens keep the early start.
  const bool ordered = max_q_len > kStage;
  auto launch = [&](auto kernel) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_kernel_as(ordered, kernel, grid, dim3(kRecurrenceThreads), smem, stream, r, k, v, w, au, u, seq_q_start, seq_q_len, seq_slot, heads,
                     dk, dv, vec, state, out);
  };
  if (per == 32) launch(delta_general_recurrence_kernel<32, 32>);
  else if (per == 16) launch(delta_general_recurrence_kernel<16, 32>);
  else if (lanes == 32) launch(delta_general_recurrence_kernel<8, 32>);
  else if (lanes == 16) launch(delta_general_recurrence_kernel<8, 16>);
  else if (lanes == 8) launch(delta_general_recurrence_kernel<8, 8>);
  else if (lanes == 4) launch(delta_general_recurrence_kernel<8, 4>);
  else if (lanes == 2) launch(delta_general_recurrence_kernel<8, 2>);
  else launch(delta_general_recurrence_kernel<8, 1>);
  return b200_check_launch("delta_general_recurrence");
}
