// Norms that act on a branch's output, a scaled embedding, and the PolyNorm activation.
//
// A "post-norm" layer adds norm(branch(x)) to its residual stream instead of feeding norm(x) to
// the branch:  x <- x + mult * scale[i] * w[i] * d[i] / sqrt(mean_g(d^2) + eps), where d is the
// branch's output and mean_g runs over the consecutive part of the row that holds column i (the
// row is cut into `groups` equal parts, each with a root mean square of its own). The same
// kernel can finish a layer whose stream is a weighted average over depth: with X_0 the
// embedding's output and X_j the stream that left layer j - 1, layer i hands on
// sum_{j <= i + 1} mix[j] * X_j; the X_j live in a history buffer, the newest one still in
// registers. Everything here is 32-bit; `cast` is the stream rounded once to the compute dtype,
// the operand of the next matrix product.
#include "common.cuh"

namespace {

constexpr int kMaxGroups = 1024;

// 1 / sqrt(mean(d^2) + eps) of every group of row `d`, by the block's warps (one group per warp
// and turn, lanes stride through it, a fixed tree adds the lanes), into rstd[groups].
template <typename T>
__device__ __forceinline__ void group_rstd(const T* d, int hidden, int groups, float eps, float* rstd) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int size = hidden / groups;
  for (int g = warp; g < groups; g += warps) {
    const T* part = d + g * size;
    float ss = 0.f;
    for (int i = lane; i < size; i += 32) {
      const float v = to_f32<T>(part[i]);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) rstd[g] = 1.f / sqrtf(ss / static_cast<float>(size) + eps);
  }
  __syncthreads();
}

template <typename T>
__global__ void branch_norm_add_kernel(const float* in_x, const T* delta, const float* __restrict__ weight,
                                       const float* __restrict__ scale, float mult, int hidden, int groups, float eps,
                                       float* out_x, float* copy_in, const float* history, int64_t history_stride,
                                       const float* __restrict__ mix, int mix_count, float* mixed_x, T* cast) {
  __shared__ float rstd[kMaxGroups];
  wait_for_predecessor();
  let_successor_start();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * hidden;
  const T* d = delta + row;
  group_rstd<T>(d, hidden, groups, eps, rstd);
  const int size = hidden / groups;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float before = in_x[row + i];
    const float normed = to_f32<T>(d[i]) * rstd[i / size] * weight[i];
    const float v = before + mult * (scale ? scale[i] : 1.f) * normed;
    if (copy_in) copy_in[row + i] = before;
    out_x[row + i] = v;
    float next = v;
    if (mix) {
      float acc = 0.f;
      for (int j = 0; j + 1 < mix_count; ++j) acc = fmaf(mix[j], history[j * history_stride + row + i], acc);
      next = fmaf(mix[mix_count - 1], v, acc);
      mixed_x[row + i] = next;
    }
    if (cast) cast[row + i] = from_f32<T>(next);
  }
}

// out[r] = x[rows ? rows[r] : r] normalised in groups, times w; x is the 32-bit stream.
template <typename T>
__global__ void grouped_rmsnorm_kernel(const float* x, const float* __restrict__ weight, const int* rows, int hidden,
                                       int groups, float eps, T* out) {
  __shared__ float rstd[kMaxGroups];
  wait_for_predecessor();
  let_successor_start();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + static_cast<int64_t>(r) * hidden;
  group_rstd<float>(xr, hidden, groups, eps, rstd);
  const int size = hidden / groups;
  T* o = out + static_cast<int64_t>(blockIdx.x) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(xr[i] * rstd[i / size] * weight[i]);
}

// x[t] = table[ids[t]] * scale in 32-bit; `cast` (optional) is x rounded to the compute dtype.
template <typename T>
__global__ void embedding_scaled_kernel(const T* __restrict__ table, const int* ids, float scale, float* out, T* cast,
                                        int hidden, int vocab, int* err) {
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_TOKEN);
  const T* src = table + static_cast<int64_t>(bad ? 0 : id) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = bad ? 0.f : to_f32<T>(src[i]) * scale;
    out[static_cast<int64_t>(t) * hidden + i] = v;
    if (cast) cast[static_cast<int64_t>(t) * hidden + i] = from_f32<T>(v);
  }
}

// PolyNorm: out = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(y) = y divided by
// the root mean square of the token's row of y (epsilon inside the root). One block per token:
// the three sums of squares (z^2, z^4, z^6) in one pass, the output in a second.
template <typename T>
__global__ void poly_norm_kernel(const T* z, const float* __restrict__ coefficients, int width, float eps, T* out) {
  __shared__ float scratch[32];
  const float a = coefficients[0], b = coefficients[1], c = coefficients[2], e = coefficients[3];
  wait_for_predecessor();
  let_successor_start();
  const T* zr = z + static_cast<int64_t>(blockIdx.x) * width;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_f32<T>(zr[i]);
    const float v2 = v * v;
    s1 += v2;
    s2 = fmaf(v2, v2, s2);
    s3 = fmaf(v2 * v, v2 * v, s3);
  }
  const float n = static_cast<float>(width);
  const float r1 = 1.f / sqrtf(block_sum(s1, scratch) / n + eps);
  const float r2 = 1.f / sqrtf(block_sum(s2, scratch) / n + eps);
  const float r3 = 1.f / sqrtf(block_sum(s3, scratch) / n + eps);
  T* o = out + static_cast<int64_t>(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_f32<T>(zr[i]);
    const float v2 = v * v;
    o[i] = from_f32<T>(a * (v * r1) + b * (v2 * r2) + c * (v2 * v * r3) + e);
  }
}

// Four neighbouring values as one access (16 bytes of float, 8 of bfloat16).
template <typename T>
struct Four;
template <>
struct Four<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Four<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

constexpr int kFoursPerThread = 4;  // a thread keeps up to this many groups of four of its row in registers

// branch_norm_add with 16-byte accesses: rows whose groups are multiples of four long and fit the
// registers (hidden <= 16 * threads). The row of the branch output is read once: each thread's
// sums of squares go to shared memory by position, one warp per norm group adds its range in a
// fixed order.
template <typename T>
__global__ void branch_norm_add_vec_kernel(const float* in_x, const T* delta, const float* __restrict__ weight,
                                           const float* __restrict__ scale, float mult, int hidden, int groups, float eps,
                                           float* out_x, float* copy_in, const float* history, int64_t history_stride,
                                           const float* __restrict__ mix, int mix_count, float* mixed_x, T* cast) {
  extern __shared__ float squares[];  // [hidden / 4]
  __shared__ float rstd[kMaxGroups];
  wait_for_predecessor();
  let_successor_start();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * hidden;
  const int fours = hidden / 4, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  float4 d[kFoursPerThread];
#pragma unroll
  for (int j = 0; j < kFoursPerThread; ++j) {
    const int f = threadIdx.x + j * blockDim.x;
    if (f < fours) {
      d[j] = Four<T>::load(delta + row + 4 * f);
      squares[f] = d[j].x * d[j].x + d[j].y * d[j].y + d[j].z * d[j].z + d[j].w * d[j].w;
    }
  }
  __syncthreads();
  const int per_group = fours / groups;
  for (int g = warp; g < groups; g += warps) {
    float ss = 0.f;
    for (int f = lane; f < per_group; f += 32) ss += squares[g * per_group + f];
    ss = warp_sum(ss);
    if (lane == 0) rstd[g] = 1.f / sqrtf(ss / static_cast<float>(4 * per_group) + eps);
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kFoursPerThread; ++j) {
    const int f = threadIdx.x + j * blockDim.x;
    if (f >= fours) continue;
    const int i = 4 * f;
    const float r = rstd[f / per_group];
    const float4 before = *reinterpret_cast<const float4*>(in_x + row + i);
    const float4 w = *reinterpret_cast<const float4*>(weight + i);
    const float4 sc = scale ? *reinterpret_cast<const float4*>(scale + i) : make_float4(1.f, 1.f, 1.f, 1.f);
    float4 v;
    v.x = before.x + mult * sc.x * (d[j].x * r * w.x);
    v.y = before.y + mult * sc.y * (d[j].y * r * w.y);
    v.z = before.z + mult * sc.z * (d[j].z * r * w.z);
    v.w = before.w + mult * sc.w * (d[j].w * r * w.w);
    if (copy_in) *reinterpret_cast<float4*>(copy_in + row + i) = before;
    *reinterpret_cast<float4*>(out_x + row + i) = v;
    float4 next = v;
    if (mix) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k + 1 < mix_count; ++k) {
        const float m = mix[k];
        const float4 h = *reinterpret_cast<const float4*>(history + k * history_stride + row + i);
        acc.x = fmaf(m, h.x, acc.x), acc.y = fmaf(m, h.y, acc.y), acc.z = fmaf(m, h.z, acc.z), acc.w = fmaf(m, h.w, acc.w);
      }
      const float m = mix[mix_count - 1];
      next = make_float4(fmaf(m, v.x, acc.x), fmaf(m, v.y, acc.y), fmaf(m, v.z, acc.z), fmaf(m, v.w, acc.w));
      *reinterpret_cast<float4*>(mixed_x + row + i) = next;
    }
    if (cast) Four<T>::store(cast + row + i, next);
  }
}

// PolyNorm with 16-byte (float) or 8-byte (bfloat16) accesses. The row is read twice (the second
// time from L1 / L2): kept in registers it cost 72 registers a thread and left one block per SM.
template <typename T>
__global__ void poly_norm_vec_kernel(const T* z, const float* __restrict__ coefficients, int width, float eps, T* out) {
  __shared__ float scratch[32];
  const float a = coefficients[0], b = coefficients[1], c = coefficients[2], e = coefficients[3];
  wait_for_predecessor();
  let_successor_start();
  const T* zr = z + static_cast<int64_t>(blockIdx.x) * width;
  const int fours = width / 4;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int f = threadIdx.x; f < fours; f += blockDim.x) {
    const float4 v = Four<T>::load(zr + 4 * f);
    const float x2 = v.x * v.x, y2 = v.y * v.y, z2 = v.z * v.z, w2 = v.w * v.w;
    s1 += x2 + y2 + z2 + w2;
    s2 += x2 * x2 + y2 * y2 + z2 * z2 + w2 * w2;
    s3 += x2 * x2 * x2 + y2 * y2 * y2 + z2 * z2 * z2 + w2 * w2 * w2;
  }
  const float n = static_cast<float>(width);
  const float r1 = 1.f / sqrtf(block_sum(s1, scratch) / n + eps);
  const float r2 = 1.f / sqrtf(block_sum(s2, scratch) / n + eps);
  const float r3 = 1.f / sqrtf(block_sum(s3, scratch) / n + eps);
  T* o = out + static_cast<int64_t>(blockIdx.x) * width;
  const auto act = [&](float x) { return a * (x * r1) + b * (x * x * r2) + c * (x * x * x * r3) + e; };
  for (int f = threadIdx.x; f < fours; f += blockDim.x) {
    const float4 v = Four<T>::load(zr + 4 * f);
    Four<T>::store(o + 4 * f, make_float4(act(v.x), act(v.y), act(v.z), act(v.w)));
  }
}

// A layer whose mixer is two mixers side by side: y = (wa (.) a / rms(a) + wb (.) b / rms(b)) / 2 is the mixer's
// output, and x <- x + w (.) y / rms(y) adds its norm to the stream. One block per row; y stays in shared
// memory in 32-bit between the two norms. `cast` is the stream rounded once to the compute dtype.
template <typename T>
__global__ void pair_norm_add_kernel(const float* in_x, const T* a, const T* b, const float* __restrict__ wa,
                                     const float* __restrict__ wb, const float* __restrict__ weight, int hidden, float eps_pair,
                                     float eps, float* out_x, T* cast) {
  extern __shared__ float pair_y[];  // [hidden]
  __shared__ float scratch[32];
  wait_for_predecessor();
  let_successor_start();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * hidden;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float av = to_f32<T>(a[row + i]), bv = to_f32<T>(b[row + i]);
    sa = fmaf(av, av, sa);
    sb = fmaf(bv, bv, sb);
  }
  const float n = static_cast<float>(hidden);
  const float ra = 1.f / sqrtf(block_sum(sa, scratch) / n + eps_pair);
  const float rb = 1.f / sqrtf(block_sum(sb, scratch) / n + eps_pair);
  float sy = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float y = 0.5f * (to_f32<T>(a[row + i]) * ra * wa[i] + to_f32<T>(b[row + i]) * rb * wb[i]);
    pair_y[i] = y;
    sy = fmaf(y, y, sy);
  }
  const float ry = 1.f / sqrtf(block_sum(sy, scratch) / n + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = in_x[row + i] + pair_y[i] * ry * weight[i];
    out_x[row + i] = v;
    if (cast) cast[row + i] = from_f32<T>(v);
  }
}

// x[t] = table[ids[t]] + pairs[row(t)] in 32-bit, row(t) = (previous * mul_prev + ids[t] * mul_cur) mod buckets with
// `previous` the token in front of t in its request, or row `buckets` (the table's last) for a request's first
// token. The token in front of a step's first one comes from the request's slot in `last_token`.
template <typename T>
__global__ void embedding_bigram_kernel(const T* __restrict__ table, const T* __restrict__ pairs, const int* ids,
                                        const int* __restrict__ positions, const int* __restrict__ token_seq,
                                        const int* __restrict__ seq_q_start, const int* __restrict__ seq_slot, const int* last_token,
                                        int buckets, int64_t mul_prev, int64_t mul_cur, float* out, T* cast, int hidden, int vocab,
                                        int* err) {
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_TOKEN);
  const int seq = token_seq[t];
  int64_t pair_row = buckets;
  if (positions[t] > 0) {
    const int previous = t > seq_q_start[seq] ? ids[t - 1] : last_token[seq_slot[seq]];
    pair_row = (static_cast<int64_t>(previous) * mul_prev + static_cast<int64_t>(id) * mul_cur) % buckets;
    if (pair_row < 0) pair_row += buckets;
  }
  const T* src = table + static_cast<int64_t>(bad ? 0 : id) * hidden;
  const T* add = pairs + pair_row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = bad ? 0.f : to_f32<T>(src[i]) + to_f32<T>(add[i]);
    out[static_cast<int64_t>(t) * hidden + i] = v;
    if (cast) cast[static_cast<int64_t>(t) * hidden + i] = from_f32<T>(v);
  }
}

// Each request's slot takes the step's last token of the request.
__global__ void last_token_update_kernel(const int* ids, const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                                         const int* __restrict__ seq_slot, int seqs, int* last_token) {
  wait_for_predecessor();
  let_successor_start();
  const int seq = blockIdx.x * blockDim.x + threadIdx.x;
  if (seq >= seqs || seq_q_len[seq] <= 0) return;
  last_token[seq_slot[seq]] = ids[seq_q_start[seq] + seq_q_len[seq] - 1];
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

int row_threads(int hidden) { return hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128); }

}  // namespace

B200_API int b200_branch_norm_add(const float* in_x, const void* delta, const float* weight, const float* scale, float mult,
                                  int rows, int hidden, int groups, float eps, float* out_x, float* copy_in,
                                  const float* history, int64_t history_stride, const float* mix, int mix_count,
                                  float* mixed_x, void* cast, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && hidden > 0 && groups > 0 && groups <= kMaxGroups && hidden % groups == 0,
               "branch_norm_add: %d columns do not cut into %d groups", hidden, groups);
  B200_REQUIRE(!mix || (mix_count >= 1 && mixed_x && (mix_count == 1 || history)), "branch_norm_add: bad depth mix");
  const int threads = row_threads(hidden);
  const bool vec = (hidden / groups) % 4 == 0 && hidden <= 4 * kFoursPerThread * threads && aligned16(in_x) && aligned16(delta) &&
                   aligned16(weight) && aligned16(scale) && aligned16(out_x) && aligned16(copy_in) && aligned16(history) &&
                   aligned16(mixed_x) && aligned16(cast) && history_stride % 4 == 0;
  if (vec && (dtype == DTYPE_F32 || dtype == DTYPE_BF16)) {
    const size_t smem = sizeof(float) * (hidden / 4);
    if (dtype == DTYPE_F32)
      launch_kernel(branch_norm_add_vec_kernel<float>, dim3(rows), dim3(threads), smem, stream, in_x,
                    static_cast<const float*>(delta), weight, scale, mult, hidden, groups, eps, out_x, copy_in, history,
                    history_stride, mix, mix_count, mixed_x, static_cast<float*>(cast));
    else
      launch_kernel(branch_norm_add_vec_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), smem, stream, in_x,
                    static_cast<const __nv_bfloat16*>(delta), weight, scale, mult, hidden, groups, eps, out_x, copy_in, history,
                    history_stride, mix, mix_count, mixed_x, static_cast<__nv_bfloat16*>(cast));
    return b200_check_launch("branch_norm_add");
  }
  if (dtype == DTYPE_F32) {
    launch_kernel(branch_norm_add_kernel<float>, dim3(rows), dim3(threads), 0, stream, in_x, static_cast<const float*>(delta),
                  weight, scale, mult, hidden, groups, eps, out_x, copy_in, history, history_stride, mix, mix_count, mixed_x,
                  static_cast<float*>(cast));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(branch_norm_add_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, in_x,
                  static_cast<const __nv_bfloat16*>(delta), weight, scale, mult, hidden, groups, eps, out_x, copy_in, history,
                  history_stride, mix, mix_count, mixed_x, static_cast<__nv_bfloat16*>(cast));
  } else {
    return b200_fail("branch_norm_add: unknown dtype %d", dtype);
  }
  return b200_check_launch("branch_norm_add");
}

B200_API int b200_grouped_rmsnorm(const float* x, const float* weight, const int* rows, int num_rows, int hidden, int groups,
                                  float eps, void* out, int dtype, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  B200_REQUIRE(num_rows > 0 && hidden > 0 && groups > 0 && groups <= kMaxGroups && hidden % groups == 0,
               "grouped_rmsnorm: %d columns do not cut into %d groups", hidden, groups);
  const int threads = row_threads(hidden);
  if (dtype == DTYPE_F32) {
    launch_kernel(grouped_rmsnorm_kernel<float>, dim3(num_rows), dim3(threads), 0, stream, x, weight, rows, hidden, groups, eps,
                  static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(grouped_rmsnorm_kernel<__nv_bfloat16>, dim3(num_rows), dim3(threads), 0, stream, x, weight, rows, hidden,
                  groups, eps, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("grouped_rmsnorm: unknown dtype %d", dtype);
  }
  return b200_check_launch("grouped_rmsnorm");
}

B200_API int b200_embedding_scaled(const void* table, const int* ids, float scale, float* out, void* cast, int tokens,
                                   int hidden, int vocab, int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && hidden > 0 && vocab > 0, "embedding_scaled: bad sizes");
  const int threads = row_threads(hidden);
  if (dtype == DTYPE_F32) {
    launch_kernel(embedding_scaled_kernel<float>, dim3(tokens), dim3(threads), 0, stream, static_cast<const float*>(table), ids,
                  scale, out, static_cast<float*>(cast), hidden, vocab, err);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(embedding_scaled_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                  static_cast<const __nv_bfloat16*>(table), ids, scale, out, static_cast<__nv_bfloat16*>(cast), hidden, vocab,
                  err);
  } else {
    return b200_fail("embedding_scaled: unknown dtype %d", dtype);
  }
  return b200_check_launch("embedding_scaled");
}

B200_API int b200_poly_norm(const void* z, const float* coefficients, int rows, int width, float eps, void* out, int dtype,
                            cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && width > 0, "poly_norm: bad sizes");
  const int threads = row_threads(width);
  if (width % 4 == 0 && aligned16(z) && aligned16(out) &&
      (dtype == DTYPE_F32 || (dtype == DTYPE_BF16 && width % 8 == 0))) {
    if (dtype == DTYPE_F32)
      launch_kernel(poly_norm_vec_kernel<float>, dim3(rows), dim3(threads), 0, stream, static_cast<const float*>(z), coefficients,
                    width, eps, static_cast<float*>(out));
    else
      launch_kernel(poly_norm_vec_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream,
                    static_cast<const __nv_bfloat16*>(z), coefficients, width, eps, static_cast<__nv_bfloat16*>(out));
    return b200_check_launch("poly_norm");
  }
  if (dtype == DTYPE_F32) {
    launch_kernel(poly_norm_kernel<float>, dim3(rows), dim3(threads), 0, stream, static_cast<const float*>(z), coefficients,
                  width, eps, static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(poly_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(z),
                  coefficients, width, eps, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("poly_norm: unknown dtype %d", dtype);
  }
  return b200_check_launch("poly_norm");
}

B200_API int b200_pair_norm_add(const float* in_x, const void* a, const void* b, const float* wa, const float* wb, const float* weight,
                                int rows, int hidden, float eps_pair, float eps, float* out_x, void* cast, int dtype,
                                cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && hidden > 0 && hidden <= 48 * 1024, "pair_norm_add: bad sizes");
  const int threads = row_threads(hidden);
  const size_t smem = sizeof(float) * hidden;
  auto launch = [&](auto kernel, auto* pa, auto* pb, auto* pc) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_kernel(kernel, dim3(rows), dim3(threads), smem, stream, in_x, pa, pb, wa, wb, weight, hidden, eps_pair, eps, out_x, pc);
  };
  if (dtype == DTYPE_F32)
    launch(pair_norm_add_kernel<float>, static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(cast));
  else if (dtype == DTYPE_BF16)
    launch(pair_norm_add_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b),
           static_cast<__nv_bfloat16*>(cast));
  else
    return b200_fail("pair_norm_add: unknown dtype %d", dtype);
  return b200_check_launch("pair_norm_add");
}

B200_API int b200_embedding_bigram(const void* table, const void* pairs, const int* ids, const int* positions, const int* token_seq,
                                   const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int* last_token, int buckets,
                                   int64_t mul_prev, int64_t mul_cur, float* out, void* cast, int tokens, int seqs, int hidden, int vocab,
                                   int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && seqs > 0 && hidden > 0 && vocab > 0 && buckets > 0, "embedding_bigram: bad sizes");
  const int threads = row_threads(hidden);
  if (dtype == DTYPE_F32) {
    launch_kernel(embedding_bigram_kernel<float>, dim3(tokens), dim3(threads), 0, stream, static_cast<const float*>(table),
                  static_cast<const float*>(pairs), ids, positions, token_seq, seq_q_start, seq_slot, static_cast<const int*>(last_token),
                  buckets, mul_prev, mul_cur, out, static_cast<float*>(cast), hidden, vocab, err);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(embedding_bigram_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(table),
                  static_cast<const __nv_bfloat16*>(pairs), ids, positions, token_seq, seq_q_start, seq_slot,
                  static_cast<const int*>(last_token), buckets, mul_prev, mul_cur, out, static_cast<__nv_bfloat16*>(cast), hidden, vocab,
                  err);
  } else {
    return b200_fail("embedding_bigram: unknown dtype %d", dtype);
  }
  if (int status = b200_check_launch("embedding_bigram")) return status;
  launch_kernel(last_token_update_kernel, dim3((seqs + 127) / 128), dim3(128), 0, stream, ids, seq_q_start, seq_q_len, seq_slot, seqs,
                last_token);
  return b200_check_launch("last_token_update");
}
