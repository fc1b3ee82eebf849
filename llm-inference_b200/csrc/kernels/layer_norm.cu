// Layer norm (mean taken off, a weight and no bias) of the 32-bit residual stream, the embedding that
// ends in one, and three small row kernels that layers built around it use.
//
// `layernorm`: v = x + a + b (the pending branch outputs, either may be absent; the sum is 32-bit and is
// written back into the stream), y = (v - mean(v)) / sqrt(mean((v - mean)^2) + eps) * w, rounded to the
// compute dtype. With `rows` only those rows are normed (pending outputs included) and the stream is left alone. The row stays in
// shared memory between the passes, so the variance is the mean of the squared deviations themselves.
//
// `embedding_layernorm`: x[t] = layer norm of table[token[t]], straight into the 32-bit stream.
// `rms_rows`: y = v / sqrt(mean(v^2) + eps) * w on rows of a matrix in the compute dtype (any row stride).
// `sigmoid_mul`: out = a * sigmoid(g), element by element, the gate logits with a row stride of their own.
// `scale_values`: v <- v * s on 32-bit numbers (logits).
#include "common.cuh"

namespace {

template <typename T>
__global__ void layernorm_kernel(float* x, const T* delta_a, const T* delta_b, const float* __restrict__ weight,
                                 const int* rows, int hidden, float eps, T* out) {
  extern __shared__ float ln_row[];
  __shared__ float scratch[32];
  wait_for_predecessor();
  let_successor_start();
  const int64_t r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = x + r * hidden;
  const bool pending = delta_a != nullptr || delta_b != nullptr;
  float sum = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    float v = xr[d];
    if (pending) {
      float add = delta_a ? to_f32<T>(delta_a[r * hidden + d]) : 0.f;
      if (delta_b) add += to_f32<T>(delta_b[r * hidden + d]);
      v += add;
      if (!rows) xr[d] = v;
    }
    ln_row[d] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / static_cast<float>(hidden);
  float ss = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float c = ln_row[d] - mean;
    ss = fmaf(c, c, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
  T* dst = out + static_cast<int64_t>(blockIdx.x) * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) dst[d] = from_f32<T>((ln_row[d] - mean) * inv * weight[d]);
}

template <typename T>
__global__ void embedding_layernorm_kernel(const T* __restrict__ table, const int* ids, const float* __restrict__ weight,
                                           float eps, float* x, int hidden, int vocab, int* err) {
  extern __shared__ float ln_row[];
  __shared__ float scratch[32];
  wait_for_predecessor();
  let_successor_start();
  const int id = ids[blockIdx.x];
  const bool good = id >= 0 && id < vocab;
  if (!good && threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_TOKEN);
  const T* src = table + static_cast<int64_t>(good ? id : 0) * hidden;
  float sum = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float v = good ? to_f32<T>(src[d]) : 0.f;
    ln_row[d] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / static_cast<float>(hidden);
  float ss = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float c = ln_row[d] - mean;
    ss = fmaf(c, c, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
  float* dst = x + static_cast<int64_t>(blockIdx.x) * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) dst[d] = (ln_row[d] - mean) * inv * weight[d];
}

template <typename T>
__global__ void rms_rows_kernel(const T* in, int64_t in_ld, const float* __restrict__ weight, float eps, int width, T* out, int64_t out_ld) {
  __shared__ float scratch[32];
  wait_for_predecessor();
  let_successor_start();
  const T* src = in + blockIdx.x * in_ld;
  float ss = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float v = to_f32<T>(src[d]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / static_cast<float>(width) + eps);
  T* dst = out + blockIdx.x * out_ld;
  for (int d = threadIdx.x; d < width; d += blockDim.x) dst[d] = from_f32<T>(to_f32<T>(src[d]) * inv * weight[d]);
}

template <typename T>
__global__ void sigmoid_mul_kernel(const T* a, const T* gate, int64_t gate_ld, int64_t rows, int width, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int64_t total = rows * width;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / width;
    const int c = static_cast<int>(idx - r * width);
    const float g = to_f32<T>(gate[r * gate_ld + c]);
    out[idx] = from_f32<T>(to_f32<T>(a[idx]) / (1.f + expf(-g)));
  }
}

// bfloat16, eight numbers a thread: the width and the gate's row stride are multiples of eight and all three
// pointers are 16-byte aligned (the launcher checks).
__global__ void sigmoid_mul_wide_kernel(const __nv_bfloat16* a, const __nv_bfloat16* gate, int64_t gate_ld, int64_t rows, int width,
                                        __nv_bfloat16* out) {
  wait_for_predecessor();
  let_successor_start();
  const int chunks = width / 8;
  const int64_t total = rows * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / chunks;
    const int c = static_cast<int>(idx - r * chunks) * 8;
    const uint4 raw_a = *reinterpret_cast<const uint4*>(a + r * width + c);
    const uint4 raw_g = *reinterpret_cast<const uint4*>(gate + r * gate_ld + c);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&raw_a);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&raw_g);
    uint4 packed;
    __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 av = __bfloat1622float2(a2[j]), gv = __bfloat1622float2(g2[j]);
      y2[j] = __floats2bfloat162_rn(av.x / (1.f + expf(-gv.x)), av.y / (1.f + expf(-gv.y)));
    }
    *reinterpret_cast<uint4*>(out + r * width + c) = packed;
  }
}

__global__ void scale_values_kernel(float* values, int64_t count, float scale) {
  wait_for_predecessor();
  let_successor_start();
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    values[i] *= scale;
}

int row_threads(int width) { return width >= 2048 ? 512 : (width >= 512 ? 256 : 128); }

template <typename T>
int launch_layernorm(float* x, const void* a, const void* b, const float* weight, const int* rows, int count, int hidden, float eps,
                     void* out, cudaStream_t stream) {
  const size_t smem = sizeof(float) * hidden;
  if (smem > 48 * 1024) cudaFuncSetAttribute(layernorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  launch_kernel(layernorm_kernel<T>, dim3(count), dim3(row_threads(hidden)), smem, stream, x, static_cast<const T*>(a),
                static_cast<const T*>(b), weight, rows, hidden, eps, static_cast<T*>(out));
  return b200_check_launch("layernorm");
}

template <typename T>
int launch_embedding_layernorm(const void* table, const int* ids, const float* weight, float eps, float* x, int tokens, int hidden,
                               int vocab, int* err, cudaStream_t stream) {
  const size_t smem = sizeof(float) * hidden;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(embedding_layernorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  launch_kernel(embedding_layernorm_kernel<T>, dim3(tokens), dim3(row_threads(hidden)), smem, stream, static_cast<const T*>(table), ids,
                weight, eps, x, hidden, vocab, err);
  return b200_check_launch("embedding_layernorm");
}

}  // namespace

B200_API int b200_layernorm(float* x, const void* delta_a, const void* delta_b, const float* weight, const int* rows, int count,
                            int hidden, float eps, void* out, int dtype, cudaStream_t stream) {
  if (count == 0) return 0;
  B200_REQUIRE(count > 0 && hidden > 0 && hidden <= 48 * 1024, "layernorm: %d rows of %d", count, hidden);
  if (dtype == DTYPE_F32) return launch_layernorm<float>(x, delta_a, delta_b, weight, rows, count, hidden, eps, out, stream);
  if (dtype == DTYPE_BF16) return launch_layernorm<__nv_bfloat16>(x, delta_a, delta_b, weight, rows, count, hidden, eps, out, stream);
  return b200_fail("layernorm: unknown dtype %d", dtype);
}

B200_API int b200_embedding_layernorm(const void* table, const int* ids, const float* weight, float eps, float* x, int tokens,
                                      int hidden, int vocab, int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && hidden > 0 && hidden <= 48 * 1024 && vocab > 0, "embedding_layernorm: bad sizes");
  if (dtype == DTYPE_F32) return launch_embedding_layernorm<float>(table, ids, weight, eps, x, tokens, hidden, vocab, err, stream);
  if (dtype == DTYPE_BF16) return launch_embedding_layernorm<__nv_bfloat16>(table, ids, weight, eps, x, tokens, hidden, vocab, err, stream);
  return b200_fail("embedding_layernorm: unknown dtype %d", dtype);
}

B200_API int b200_rms_rows(const void* in, int64_t in_ld, const float* weight, float eps, int rows, int width, void* out, int64_t out_ld,
                           int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && width > 0 && in_ld >= width && out_ld >= width, "rms_rows: bad sizes");
  if (dtype == DTYPE_F32) {
    launch_kernel(rms_rows_kernel<float>, dim3(rows), dim3(row_threads(width)), 0, stream, static_cast<const float*>(in), in_ld, weight,
                  eps, width, static_cast<float*>(out), out_ld);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(rms_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(row_threads(width)), 0, stream, static_cast<const __nv_bfloat16*>(in),
                  in_ld, weight, eps, width, static_cast<__nv_bfloat16*>(out), out_ld);
  } else {
    return b200_fail("rms_rows: unknown dtype %d", dtype);
  }
  return b200_check_launch("rms_rows");
}

B200_API int b200_sigmoid_mul(const void* a, const void* gate, int64_t gate_ld, int rows, int width, void* out, int dtype,
                              cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && width > 0 && gate_ld >= width, "sigmoid_mul: bad sizes");
  const int threads = 256;
  const int64_t total = static_cast<int64_t>(rows) * width;
  auto blocks = [&](int64_t items) {
    const int64_t want = (items + threads - 1) / threads;
    return dim3(static_cast<unsigned>(want < 65535 ? want : 65535));
  };
  auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (dtype == DTYPE_F32) {
    launch_kernel(sigmoid_mul_kernel<float>, blocks(total), dim3(threads), 0, stream, static_cast<const float*>(a),
                  static_cast<const float*>(gate), gate_ld, static_cast<int64_t>(rows), width, static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16 && width % 8 == 0 && gate_ld % 8 == 0 && aligned(a) && aligned(gate) && aligned(out)) {
    launch_kernel(sigmoid_mul_wide_kernel, blocks(total / 8), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(a),
                  static_cast<const __nv_bfloat16*>(gate), gate_ld, static_cast<int64_t>(rows), width, static_cast<__nv_bfloat16*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(sigmoid_mul_kernel<__nv_bfloat16>, blocks(total), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(a),
                  static_cast<const __nv_bfloat16*>(gate), gate_ld, static_cast<int64_t>(rows), width, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("sigmoid_mul: unknown dtype %d", dtype);
  }
  return b200_check_launch("sigmoid_mul");
}

B200_API int b200_scale_values(float* values, int64_t count, float scale, cudaStream_t stream) {
  if (count == 0) return 0;
  B200_REQUIRE(count > 0, "scale_values: bad size");
  const int threads = 256;
  const int64_t blocks = (count + threads - 1) / threads;
  launch_kernel(scale_values_kernel, dim3(static_cast<unsigned>(blocks < 4096 ? blocks : 4096)), dim3(threads), 0, stream, values, count,
                scale);
  return b200_check_launch("scale_values");
}
