// What stands in front of the paged attention kernels in a mixer that norms all of its queries (and all of its
// keys) as one vector and may rotate part of each head: bias, the two norms, the rotation and the cache write.
//
// `qk_norm_rope_write`, one block per new token. The token's row of the fused input product holds
// [q (q_heads * dim) | k (kv_heads * dim) | v (kv_heads * vdim) | ...]; with `values_from_keys` there is no v part and
// the values are the keys as projected (bias added, before norm and rotation). In 32-bit: bias; the whole of q is
// divided by its root mean square over all q_heads * dim numbers (eps inside the root) and multiplied by a weight
// per number, likewise the whole of k (either norm may be absent); the first `rot_dims` numbers of every head are
// rotated, number i with number i + rot_dims / 2, by the angle position * inv_freq[i], sine and cosine both
// multiplied by `magnitude`; the rest of the head passes unchanged. Queries go to a dense buffer and keys and values
// into the token's page, all in rows of `row_dim` numbers padded with zeros (the arena has one row width for keys
// and values). The token that starts a page clears the rows its step does not fill.
#include "common.cuh"
#include "page_tail.cuh"

namespace {

template <typename T>
__global__ void qk_norm_rope_write_kernel(const T* proj, int ld, const float* __restrict__ bias, const float* __restrict__ q_weight,
                                          const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq, int rot_dims,
                                          float magnitude, int values_from_keys, const int* __restrict__ positions,
                                          const int* __restrict__ token_seq, const int* __restrict__ seq_kv_len,
                                          const int* __restrict__ block_table, int max_pages, int num_pages, T* k_arena, T* v_arena,
                                          T* q_out, int q_heads, int kv_heads, int dim, int vdim, int row_dim, int page_size,
                                          int write_kv, int* err) {
  extern __shared__ float qk_row[];  // [q_heads * dim + kv_heads * dim]: q and k with their biases
  __shared__ float scratch[32];
  let_successor_start();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = positions[t];
  const int q_width = q_heads * dim, k_width = kv_heads * dim;
  int page = -1, clear_from = 0;
  if (write_kv) {
    const int logical = pos / page_size;
    if (pos < 0 || logical >= max_pages) {
      if (tid == 0) atomicOr(err, ERRBIT_BAD_POSITION);
    } else {
      page = block_table[static_cast<int64_t>(token_seq[t]) * max_pages + logical];
      if (page < 0 || page >= num_pages) {
        if (tid == 0) atomicOr(err, ERRBIT_BAD_PAGE);
        page = -1;
      } else if (pos % page_size == 0 && seq_kv_len != nullptr) {
        clear_from = max(1, seq_kv_len[token_seq[t]] - pos);
      }
    }
  }
  wait_for_predecessor();
  const T* row = proj + static_cast<int64_t>(t) * ld;
  float ss_q = 0.f, ss_k = 0.f;
  for (int i = tid; i < q_width + k_width; i += blockDim.x) {
    const float v = to_f32<T>(row[i]) + (bias ? bias[i] : 0.f);
    qk_row[i] = v;
    if (i < q_width) ss_q = fmaf(v, v, ss_q);
    else ss_k = fmaf(v, v, ss_k);
  }
  ss_q = block_sum(ss_q, scratch);
  ss_k = block_sum(ss_k, scratch);
  const float inv_q = q_weight ? 1.f / sqrtf(ss_q / static_cast<float>(q_width) + eps) : 1.f;
  const float inv_k = k_weight ? 1.f / sqrtf(ss_k / static_cast<float>(k_width) + eps) : 1.f;
  const int row_in_page = pos % page_size;
  T* k_tile = page >= 0 ? k_arena + kv_row_offset(page, 0, 0, kv_heads, page_size, row_dim) : nullptr;
  T* v_tile = page >= 0 ? v_arena + kv_row_offset(page, 0, 0, kv_heads, page_size, row_dim) : nullptr;
  const int64_t head_stride = static_cast<int64_t>(page_size) * row_dim;
  if (clear_from > 0 && page >= 0) {
    for (int h = 0; h < kv_heads; ++h) {
      clear_page_tail(k_tile + h * head_stride, clear_from, page_size, row_dim);  // the token sits in row 0 of the page
      clear_page_tail(v_tile + h * head_stride, clear_from, page_size, row_dim);
    }
  }
  // Values: the keys as projected, or the v part of the row (with its bias).
  if (page >= 0) {
    for (int idx = tid; idx < kv_heads * row_dim; idx += blockDim.x) {
      const int h = idx / row_dim, i = idx - h * row_dim;
      float v = 0.f;
      if (i < vdim) {
        if (values_from_keys) v = qk_row[q_width + h * dim + i];
        else v = to_f32<T>(row[q_width + k_width + h * vdim + i]) + (bias ? bias[q_width + k_width + h * vdim + i] : 0.f);
      }
      v_tile[h * head_stride + static_cast<int64_t>(row_in_page) * row_dim + i] = from_f32<T>(v);
    }
  }
  // Queries and keys: an item is one number of a head's unrotated part or one rotated pair; items past `dim` pad.
  const int half = rot_dims / 2;
  const int items = row_dim - half;  // per head: `half` pairs, then the numbers from rot_dims on, then the padding
  for (int idx = tid; idx < (q_heads + kv_heads) * items; idx += blockDim.x) {
    const int head = idx / items, i = idx - head * items;
    const bool is_q = head < q_heads;
    if (!is_q && page < 0) continue;
    const float* src = qk_row + head * dim;  // k heads follow the q heads in the shared row
    const bool weighted = is_q ? q_weight != nullptr : k_weight != nullptr;
    const float* w = !weighted ? nullptr : (is_q ? q_weight + head * dim : k_weight + (head - q_heads) * dim);
    const float inv = is_q ? inv_q : inv_k;
    T* dst = is_q ? q_out + (static_cast<int64_t>(t) * q_heads + head) * row_dim
                  : k_tile + (head - q_heads) * head_stride + static_cast<int64_t>(row_in_page) * row_dim;
    if (i < half) {
      const float u = src[i] * inv * (weighted ? w[i] : 1.f), v = src[i + half] * inv * (weighted ? w[i + half] : 1.f);
      float s, c;
      sincosf(static_cast<float>(pos) * inv_freq[i], &s, &c);
      s *= magnitude;
      c *= magnitude;
      dst[i] = from_f32<T>(u * c - v * s);
      dst[i + half] = from_f32<T>(v * c + u * s);
    } else {
      const int d = i + half;
      dst[d] = from_f32<T>(d < dim ? src[d] * inv * (weighted ? w[d] : 1.f) : 0.f);
    }
  }
}

}  // namespace

B200_API int b200_qk_norm_rope_write(const void* proj, int ld, const float* bias, const float* q_weight, const float* k_weight, float eps,
                                     const float* inv_freq, int rot_dims, float magnitude, int values_from_keys, const int* positions,
                                     const int* token_seq, const int* seq_kv_len, const int* block_table, int max_pages, int num_pages,
                                     void* k_arena, void* v_arena, void* q_out, int tokens, int q_heads, int kv_heads, int dim, int vdim,
                                     int row_dim, int page_size, int write_kv, int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && q_heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && row_dim >= dim && row_dim >= vdim,
               "qk_norm_rope_write: bad sizes");
  B200_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim && (rot_dims == 0 || inv_freq != nullptr),
               "qk_norm_rope_write: %d of %d numbers of a head cannot be rotated in halves", rot_dims, dim);
  B200_REQUIRE(!values_from_keys || vdim == dim, "qk_norm_rope_write: values that are the keys have the keys' size");
  B200_REQUIRE(ld >= (q_heads + kv_heads) * dim + (values_from_keys ? 0 : kv_heads * vdim),
               "qk_norm_rope_write: rows of %d numbers do not hold the projections", ld);
  const size_t smem = sizeof(float) * (q_heads + kv_heads) * dim;
  B200_REQUIRE(smem <= 160 * 1024, "qk_norm_rope_write: %d numbers of q and k do not fit one block", (q_heads + kv_heads) * dim);
  const int work = (q_heads + kv_heads) * dim;
  const int threads = work >= 4096 ? 512 : (work >= 1024 ? 256 : 128);
  if (dtype == DTYPE_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(qk_norm_rope_write_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_kernel(qk_norm_rope_write_kernel<float>, dim3(tokens), dim3(threads), smem, stream, static_cast<const float*>(proj), ld, bias,
                  q_weight, k_weight, eps, inv_freq, rot_dims, magnitude, values_from_keys, positions, token_seq, seq_kv_len, block_table,
                  max_pages, num_pages, static_cast<float*>(k_arena), static_cast<float*>(v_arena), static_cast<float*>(q_out), q_heads,
                  kv_heads, dim, vdim, row_dim, page_size, write_kv, err);
  } else if (dtype == DTYPE_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(qk_norm_rope_write_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_kernel(qk_norm_rope_write_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), smem, stream,
                  static_cast<const __nv_bfloat16*>(proj), ld, bias, q_weight, k_weight, eps, inv_freq, rot_dims, magnitude,
                  values_from_keys, positions, token_seq, seq_kv_len, block_table, max_pages, num_pages,
                  static_cast<__nv_bfloat16*>(k_arena), static_cast<__nv_bfloat16*>(v_arena), static_cast<__nv_bfloat16*>(q_out), q_heads,
                  kv_heads, dim, vdim, row_dim, page_size, write_kv, err);
  } else {
    return b200_fail("qk_norm_rope_write: unknown dtype %d", dtype);
  }
  return b200_check_launch("qk_norm_rope_write");
}
