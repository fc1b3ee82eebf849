// Attention over a cache of low-rank latents.
//
// Every token leaves one row [latent (rank) | rotated key part (rot_dim)] in a paged arena
// [pages][page_size][rank + rot_dim]; all query heads read the same rows. A head's key is
// W_uk latent (plus the shared rotated part) and its value W_uv latent, so with
// q' = W_uk^T q_plain the score is (q' . latent + q_rot . k_rot) * scale and the head's output is
// W_uv (sum_j p_j latent_j): the kernels here work on the rows as they are cached, the two small
// products around them are matrix products of their own. The softmax's denominator also holds
// exp(sink[h]), a term without key or value; the head's output is multiplied by
// sigmoid(gate[t, h]). Scores, weights and sums are 32-bit.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kMaxValuesPerThread = 8;  // rank <= 1024 in the plain kernel

// The pair (u, v) of dims (2i, 2i + 1), or (i, i + rot_dims / 2) in the layout of halves, at position p becomes
// (u cos a - v sin a, v cos a + u sin a), a = p * inv_freq[i], sine and cosine both times `magnitude`; dims from
// `rot_dims` on pass unchanged.
__device__ __forceinline__ void rotate_pair(float u, float v, int position, float inv_freq, float magnitude, float* ru, float* rv) {
  float s, c;
  sincosf(static_cast<float>(position) * inv_freq, &s, &c);
  s *= magnitude;
  c *= magnitude;
  *ru = u * c - v * s;
  *rv = v * c + u * s;
}

// One block per token. The token's queries [heads x (dim | rot_dim)] start at q_offset of its row of `q_proj`, its
// [latent (rank) | key part (rot_dim)] at kv_offset of its row of `proj` (the two may be one matrix).
// Writes the normalised latent and the rotated key part to the token's cache row and the rotated
// query parts to q_rot [tokens][heads][rot_dim].
template <typename T>
__global__ void latent_kv_write_kernel(const T* q_proj, int q_ld, const T* proj, int ld, int q_offset, int kv_offset, int heads, int dim,
                                       int rot_dim, int rank, const float* __restrict__ norm_weight, float eps,
                                       const float* __restrict__ inv_freq, int rot_dims, int halves, float magnitude, const int* positions,
                                       const int* token_seq, const int* block_table, int max_pages, int num_pages,
                                       T* arena, int page_size, int writes, T* q_rot, int* err) {
  __shared__ float scratch[32];
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = positions[t];
  const T* row = proj + static_cast<int64_t>(t) * ld;
  const T* q_row = q_proj + static_cast<int64_t>(t) * q_ld;
  const int half = rot_dims / 2;
  // queries: rotate each head's last rot_dim dims
  for (int idx = tid; idx < heads * (rot_dim - half); idx += blockDim.x) {
    const int h = idx / (rot_dim - half), i = idx % (rot_dim - half);
    const T* src = q_row + q_offset + h * (dim + rot_dim) + dim;
    T* dst = q_rot + (static_cast<int64_t>(t) * heads + h) * rot_dim;
    if (i < half) {
      const int a = halves ? i : 2 * i, b = halves ? i + half : 2 * i + 1;
      float u, v;
      rotate_pair(to_f32<T>(src[a]), to_f32<T>(src[b]), pos, inv_freq[i], magnitude, &u, &v);
      dst[a] = from_f32<T>(u);
      dst[b] = from_f32<T>(v);
    } else {
      dst[rot_dims + i - half] = src[rot_dims + i - half];
    }
  }
  if (!writes) return;
  const int seq = token_seq[t];
  const int logical = pos / page_size;
  const int page = (pos >= 0 && logical < max_pages) ? block_table[static_cast<int64_t>(seq) * max_pages + logical] : -1;
  const T* kv = row + kv_offset;
  float ss = 0.f;
  for (int i = tid; i < rank; i += blockDim.x) {
    const float v = to_f32<T>(kv[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / static_cast<float>(rank) + eps);
  if (page < 0 || page >= num_pages) {
    if (tid == 0) atomicOr(err, pos >= 0 && logical < max_pages ? ERRBIT_BAD_PAGE : ERRBIT_BAD_POSITION);
    return;
  }
  T* dst = arena + (static_cast<int64_t>(page) * page_size + pos % page_size) * (rank + rot_dim);
  for (int i = tid; i < rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32<T>(kv[i]) * inv * norm_weight[i]);
  for (int i = tid; i < rot_dim - half; i += blockDim.x) {
    if (i < half) {
      const int a = halves ? i : 2 * i, b = halves ? i + half : 2 * i + 1;
      float u, v;
      rotate_pair(to_f32<T>(kv[rank + a]), to_f32<T>(kv[rank + b]), pos, inv_freq[i], magnitude, &u, &v);
      dst[rank + a] = from_f32<T>(u);
      dst[rank + b] = from_f32<T>(v);
    } else {
      dst[rank + rot_dims + i - half] = kv[rank + rot_dims + i - half];
    }
  }
}

template <typename T>
__device__ __forceinline__ float dot_latent(const float* q, const T* k, int n) {
  float acc = 0.f;
  for (int i = 0; i < n; ++i) acc = fmaf(q[i], to_f32<T>(k[i]), acc);
  return acc;
}

// The plain kernel: one block per (token, head); keys 128 at a time with a running maximum and
// sum that start at (sink, 1), which is the sink's term. Serves the 32-bit path and every shape.
template <typename T>
__global__ void __launch_bounds__(kThreads)
latent_attention_plain_kernel(const T* q_lat, int64_t q_lat_token, int64_t q_lat_head, const T* q_rot, const T* arena,
                              const int* positions, const int* token_seq, const int* block_table, int max_pages,
                              int num_pages, const float* __restrict__ sink, const T* gate, int64_t gate_ld, T* out,
                              int64_t out_token, int64_t out_head, int heads, int rank, int rot_dim, int page_size,
                              int window, float scale, int* err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int width = rank + rot_dim;
  float* qs = reinterpret_cast<float*>(smem_raw);                     // [width]
  float* probs = qs + ((width + 3) & ~3);                             // [kThreads]
  int64_t* offsets = reinterpret_cast<int64_t*>(probs + kThreads);    // [kThreads]
  __shared__ float scratch[32];
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int pos = positions[t];
  const int seq = token_seq[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = block_table + static_cast<int64_t>(seq) * max_pages;
  const T* ql = q_lat + t * q_lat_token + h * q_lat_head;
  const T* qr = q_rot + (static_cast<int64_t>(t) * heads + h) * rot_dim;
  for (int i = tid; i < rank; i += kThreads) qs[i] = to_f32<T>(ql[i]);
  for (int i = tid; i < rot_dim; i += kThreads) qs[rank + i] = to_f32<T>(qr[i]);
  __syncthreads();

  float acc[kMaxValuesPerThread];
#pragma unroll
  for (int i = 0; i < kMaxValuesPerThread; ++i) acc[i] = 0.f;
  float running_max = sink ? sink[h] : -INFINITY;
  float running_sum = sink ? 1.f : 0.f;

  for (int k0 = lo; k0 <= pos; k0 += kThreads) {
    const int j = k0 + tid;
    float s = -INFINITY;
    int64_t off = -1;
    if (j <= pos) {
      const int logical = j / page_size;
      const int page = logical < max_pages ? table[logical] : -1;
      if (page < 0 || page >= num_pages) {
        atomicOr(err, ERRBIT_BAD_PAGE);
      } else {
        off = (static_cast<int64_t>(page) * page_size + j % page_size) * width;
        s = dot_latent<T>(qs, arena + off, width) * scale;
      }
    }
    offsets[tid] = off;
    const float new_max = fmaxf(running_max, block_max(s, scratch));
    const float p = (off >= 0 && new_max > -INFINITY) ? expf(s - new_max) : 0.f;
    probs[tid] = p;
    const float chunk_sum = block_sum(p, scratch);
    const float alpha = (running_max > -INFINITY) ? expf(running_max - new_max) : 0.f;
    running_sum = running_sum * alpha + chunk_sum;
    running_max = new_max;
    __syncthreads();
    const int count = min(kThreads, pos - k0 + 1);
#pragma unroll
    for (int i = 0; i < kMaxValuesPerThread; ++i) {
      const int d = tid + i * kThreads;
      if (d < rank) {
        float a = acc[i] * alpha;
        for (int jj = 0; jj < count; ++jj) {
          const int64_t o = offsets[jj];
          if (o >= 0) a = fmaf(probs[jj], to_f32<T>(arena[o + d]), a);
        }
        acc[i] = a;
      }
    }
    __syncthreads();
  }
  float factor = running_sum > 0.f ? 1.f / running_sum : 0.f;
  if (gate) factor *= 1.f / (1.f + expf(-to_f32<T>(gate[t * gate_ld + h])));
  T* o = out + t * out_token + h * out_head;
#pragma unroll
  for (int i = 0; i < kMaxValuesPerThread; ++i) {
    const int d = tid + i * kThreads;
    if (d < rank) o[d] = from_f32<T>(acc[i] * factor);
  }
}

}  // namespace

B200_API int b200_latent_kv_write(const void* q_proj, int q_ld, const void* proj, int ld, int q_offset, int kv_offset, int tokens, int heads,
                                  int dim, int rot_dim, int rank, const float* norm_weight, float eps, const float* inv_freq,
                                  int rot_dims, int halves, float magnitude, const int* positions, const int* token_seq, const int* block_table,
                                  int max_pages, int num_pages, void* arena, int page_size, int writes, void* q_rot,
                                  int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && heads > 0 && dim >= 0 && rank > 0 && rot_dim >= 0, "latent_kv_write: bad sizes");
  B200_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot_dim, "latent_kv_write: %d rotated dims of %d", rot_dims,
               rot_dim);
  B200_REQUIRE(page_size > 0 && max_pages > 0, "latent_kv_write: bad geometry");
  const int threads = rank >= 512 ? 256 : 128;
  if (dtype == DTYPE_F32) {
    launch_kernel(latent_kv_write_kernel<float>, dim3(tokens), dim3(threads), 0, stream, static_cast<const float*>(q_proj), q_ld,
                  static_cast<const float*>(proj), ld, q_offset, kv_offset, heads, dim, rot_dim, rank, norm_weight, eps, inv_freq, rot_dims,
                  halves, magnitude, positions, token_seq,
                  block_table, max_pages, num_pages, static_cast<float*>(arena), page_size, writes, static_cast<float*>(q_rot),
                  err);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(latent_kv_write_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                  static_cast<const __nv_bfloat16*>(q_proj), q_ld, static_cast<const __nv_bfloat16*>(proj), ld, q_offset, kv_offset, heads,
                  dim, rot_dim, rank, norm_weight, eps, inv_freq, rot_dims, halves, magnitude, positions, token_seq, block_table, max_pages, num_pages,
                  static_cast<__nv_bfloat16*>(arena), page_size, writes, static_cast<__nv_bfloat16*>(q_rot), err);
  } else {
    return b200_fail("latent_kv_write: unknown dtype %d", dtype);
  }
  return b200_check_launch("latent_kv_write");
}

B200_API int b200_latent_attention_plain(const void* q_lat, int64_t q_lat_token, int64_t q_lat_head, const void* q_rot,
                                         const void* arena, const int* positions, const int* token_seq,
                                         const int* block_table, int max_pages, int num_pages, const float* sink,
                                         const void* gate, int64_t gate_ld, void* out, int64_t out_token, int64_t out_head,
                                         int tokens, int heads, int rank, int rot_dim, int page_size, int window, float scale,
                                         int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && heads > 0 && heads <= 65535 && rank > 0 && rot_dim >= 0, "latent_attention_plain: bad sizes");
  B200_REQUIRE(rank <= kThreads * kMaxValuesPerThread, "latent_attention_plain: latent size %d above %d", rank,
               kThreads * kMaxValuesPerThread);
  B200_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "latent_attention_plain: bad geometry");
  const dim3 grid(tokens, heads);
  const size_t smem = sizeof(float) * (((rank + rot_dim + 3) & ~3) + kThreads) + sizeof(int64_t) * kThreads;
  if (dtype == DTYPE_F32) {
    launch_kernel(latent_attention_plain_kernel<float>, grid, dim3(kThreads), smem, stream, static_cast<const float*>(q_lat),
                  q_lat_token, q_lat_head, static_cast<const float*>(q_rot), static_cast<const float*>(arena), positions,
                  token_seq, block_table, max_pages, num_pages, sink, static_cast<const float*>(gate), gate_ld,
                  static_cast<float*>(out), out_token, out_head, heads, rank, rot_dim, page_size, window, scale, err);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(latent_attention_plain_kernel<__nv_bfloat16>, grid, dim3(kThreads), smem, stream,
                  static_cast<const __nv_bfloat16*>(q_lat), q_lat_token, q_lat_head, static_cast<const __nv_bfloat16*>(q_rot),
                  static_cast<const __nv_bfloat16*>(arena), positions, token_seq, block_table, max_pages, num_pages, sink,
                  static_cast<const __nv_bfloat16*>(gate), gate_ld, static_cast<__nv_bfloat16*>(out), out_token, out_head,
                  heads, rank, rot_dim, page_size, window, scale, err);
  } else {
    return b200_fail("latent_attention_plain: unknown dtype %d", dtype);
  }
  return b200_check_launch("latent_attention_plain");
}
