// minGRU: a gated recurrence whose gates and candidates read only the current token.
//
// Per channel, with a state S (32-bit, zero at a request's start) carried from token to token:
//   z = sigmoid(pz + bz);  u = px + bx;  c = u + 1/2 where u >= 0, sigmoid(u) where u < 0;
//   S <- (1 - z) S + z c;  y = S * silu(pg).
// `proj` rows hold [pz | px | pg] (the three projections of the token, `width` numbers each, bias
// not yet added). Gates, candidates and the state are 32-bit; y leaves in the compute dtype.
//
// S_t = A_t S_(t-1) + B_t with A = 1 - z and B = z c is a chain of affine maps, and affine maps
// compose: (A2, B2) o (A1, B1) = (A2 A1, A2 B1 + B2). A prompt portion is therefore cut into
// pieces of kPiece tokens that run at the same time: pass 1 composes each piece's maps, pass 2
// walks the pieces' results in order (a short chain), pass 3 replays each piece from its true
// start value and writes y. Short runs (decoded tokens, short portions) take the one-pass kernel.
// Both forms apply the maps to the state in token order, so a request's result does not depend on
// which form ran beyond rounding of the composed products.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kUnroll = 8;
constexpr int kPiece = 64;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ void gate_and_candidate(float pz, float px, float bz, float bx, float& a, float& b) {
  const float z = sigmoid_f(pz + bz);
  const float u = px + bx;
  const float c = u >= 0.f ? u + 0.5f : sigmoid_f(u);
  a = 1.f - z;
  b = z * c;
}

// One thread per (request, channel) walks the request's tokens.
template <typename T>
__global__ void __launch_bounds__(kThreads)
mingru_scan_kernel(const T* proj, int ld, const float* __restrict__ bias, const int* __restrict__ seq_q_start,
                   const int* __restrict__ seq_q_len, const int* __restrict__ seq_slot, int width, float* state, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int c = blockIdx.x * kThreads + threadIdx.x;
  const int seq = blockIdx.y;
  if (c >= width) return;
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  if (len <= 0) return;
  float* slot = state + static_cast<int64_t>(seq_slot[seq]) * width;
  const float bz = bias[c], bx = bias[width + c];
  float s = slot[c];
  for (int t0 = 0; t0 < len; t0 += kUnroll) {
    float pz[kUnroll], px[kUnroll], pg[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const int t = min(t0 + j, len - 1);
      const T* row = proj + static_cast<int64_t>(start + t) * ld;
      pz[j] = to_f32<T>(row[c]);
      px[j] = to_f32<T>(row[width + c]);
      pg[j] = to_f32<T>(row[2 * width + c]);
    }
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      if (t0 + j < len) {
        float a, b;
        gate_and_candidate(pz[j], px[j], bz, bx, a, b);
        s = fmaf(a, s, b);
        out[static_cast<int64_t>(start + t0 + j) * width + c] = from_f32<T>(s * (pg[j] * sigmoid_f(pg[j])));
      }
    }
  }
  slot[c] = s;
}

// Pass 1 of the long form: piece p of request `seq` composes its tokens' maps into (A, B).
template <typename T>
__global__ void __launch_bounds__(kThreads)
mingru_compose_kernel(const T* proj, int ld, const float* __restrict__ bias, const int* __restrict__ seq_q_start,
                      const int* __restrict__ seq_q_len, int first_seq, int width, int max_pieces, float* maps) {
  wait_for_predecessor();
  let_successor_start();
  const int c = blockIdx.x * kThreads + threadIdx.x;
  const int piece = blockIdx.y, seq = first_seq + blockIdx.z;
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  const int t0 = piece * kPiece;
  if (c >= width || t0 >= len) return;
  const int count = min(kPiece, len - t0);
  const float bz = bias[c], bx = bias[width + c];
  float a_all = 1.f, b_all = 0.f;
  for (int j0 = 0; j0 < count; j0 += kUnroll) {
    float pz[kUnroll], px[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const T* row = proj + static_cast<int64_t>(start + t0 + min(j0 + j, count - 1)) * ld;
      pz[j] = to_f32<T>(row[c]);
      px[j] = to_f32<T>(row[width + c]);
    }
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      if (j0 + j < count) {
        float a, b;
        gate_and_candidate(pz[j], px[j], bz, bx, a, b);
        a_all *= a;
        b_all = fmaf(a, b_all, b);
      }
    }
  }
  float* dst = maps + ((static_cast<int64_t>(blockIdx.z) * max_pieces + piece) * 2) * width;
  dst[c] = a_all;
  dst[width + c] = b_all;
}

// Pass 2: the state in front of every piece (written over the piece's A), and the slot's new state.
__global__ void __launch_bounds__(kThreads)
mingru_carry_kernel(const int* __restrict__ seq_q_len, const int* __restrict__ seq_slot, int first_seq, int width, int max_pieces,
                    float* maps, float* state) {
  wait_for_predecessor();
  let_successor_start();
  const int c = blockIdx.x * kThreads + threadIdx.x;
  const int seq = first_seq + blockIdx.y;
  const int len = seq_q_len[seq];
  if (c >= width || len <= 0) return;
  const int pieces = (len + kPiece - 1) / kPiece;
  float* slot = state + static_cast<int64_t>(seq_slot[seq]) * width;
  float s = slot[c];
  float* m = maps + static_cast<int64_t>(blockIdx.y) * max_pieces * 2 * width;
  for (int p = 0; p < pieces; ++p) {
    const float a = m[(2 * p) * width + c], b = m[(2 * p + 1) * width + c];
    m[(2 * p) * width + c] = s;
    s = fmaf(a, s, b);
  }
  slot[c] = s;
}

// Pass 3: every piece again, from the state in front of it.
template <typename T>
__global__ void __launch_bounds__(kThreads)
mingru_replay_kernel(const T* proj, int ld, const float* __restrict__ bias, const int* __restrict__ seq_q_start,
                     const int* __restrict__ seq_q_len, int first_seq, int width, int max_pieces, const float* maps, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int c = blockIdx.x * kThreads + threadIdx.x;
  const int piece = blockIdx.y, seq = first_seq + blockIdx.z;
  const int start = seq_q_start[seq], len = seq_q_len[seq];
  const int t0 = piece * kPiece;
  if (c >= width || t0 >= len) return;
  const int count = min(kPiece, len - t0);
  const float bz = bias[c], bx = bias[width + c];
  float s = maps[((static_cast<int64_t>(blockIdx.z) * max_pieces + piece) * 2) * width + c];
  for (int j0 = 0; j0 < count; j0 += kUnroll) {
    float pz[kUnroll], px[kUnroll], pg[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const T* row = proj + static_cast<int64_t>(start + t0 + min(j0 + j, count - 1)) * ld;
      pz[j] = to_f32<T>(row[c]);
      px[j] = to_f32<T>(row[width + c]);
      pg[j] = to_f32<T>(row[2 * width + c]);
    }
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      if (j0 + j < count) {
        float a, b;
        gate_and_candidate(pz[j], px[j], bz, bx, a, b);
        s = fmaf(a, s, b);
        out[static_cast<int64_t>(start + t0 + j0 + j) * width + c] = from_f32<T>(s * (pg[j] * sigmoid_f(pg[j])));
      }
    }
  }
}

template <typename T>
int run_mingru(const T* proj, int ld, const float* bias, const int* seq_q_start, const int* seq_q_len, const int* seq_slot,
               int first_long, int seqs, int max_q_len, int width, float* state, float* maps, T* out, cudaStream_t stream) {
  const unsigned col_blocks = static_cast<unsigned>((width + kThreads - 1) / kThreads);
  // Requests [0, first_long) feed few tokens and take the one-pass kernel; the rest take the three passes.
  if (first_long > 0) {
    launch_kernel(mingru_scan_kernel<T>, dim3(col_blocks, first_long), dim3(kThreads), 0, stream, proj, ld, bias, seq_q_start, seq_q_len,
                  seq_slot, width, state, out);
    if (int status = b200_check_launch("mingru_scan")) return status;
  }
  const int long_seqs = seqs - first_long;
  if (long_seqs > 0) {
    const int max_pieces = (max_q_len + kPiece - 1) / kPiece;
    launch_kernel(mingru_compose_kernel<T>, dim3(col_blocks, max_pieces, long_seqs), dim3(kThreads), 0, stream, proj, ld, bias,
                  seq_q_start, seq_q_len, first_long, width, max_pieces, maps);
    if (int status = b200_check_launch("mingru_compose")) return status;
    launch_kernel(mingru_carry_kernel, dim3(col_blocks, long_seqs), dim3(kThreads), 0, stream, seq_q_len, seq_slot, first_long, width,
                  max_pieces, maps, state);
    if (int status = b200_check_launch("mingru_carry")) return status;
    launch_kernel(mingru_replay_kernel<T>, dim3(col_blocks, max_pieces, long_seqs), dim3(kThreads), 0, stream, proj, ld, bias,
                  seq_q_start, seq_q_len, first_long, width, max_pieces, static_cast<const float*>(maps), out);
    if (int status = b200_check_launch("mingru_replay")) return status;
  }
  return 0;
}

}  // namespace

// Floats of scratch the three-pass form needs for `long_seqs` requests of up to `max_q_len` tokens.
B200_API int64_t b200_mingru_scratch(int long_seqs, int max_q_len, int width) {
  const int64_t pieces = (max_q_len + kPiece - 1) / kPiece;
  return static_cast<int64_t>(long_seqs) * pieces * 2 * width;
}

// Requests [0, first_long) of the step run the one-pass kernel, [first_long, seqs) the three passes
// (`maps` holds b200_mingru_scratch floats; it may be null when first_long == seqs).
B200_API int b200_mingru(const void* proj, int ld, const float* bias, const int* seq_q_start, const int* seq_q_len,
                         const int* seq_slot, int first_long, int seqs, int max_q_len, int width, float* state, float* maps,
                         void* out, int dtype, cudaStream_t stream) {
  if (seqs == 0) return 0;
  B200_REQUIRE(seqs > 0 && width > 0 && ld >= 3 * width && first_long >= 0 && first_long <= seqs && max_q_len > 0,
               "mingru: bad sizes");
  B200_REQUIRE(seqs <= 65535, "mingru: too many requests in one step");
  B200_REQUIRE(first_long == seqs || maps != nullptr, "mingru: the three-pass form needs its scratch");
  B200_REQUIRE((max_q_len + kPiece - 1) / kPiece <= 65535, "mingru: a portion of %d tokens is too long", max_q_len);
  if (dtype == DTYPE_F32)
    return run_mingru(static_cast<const float*>(proj), ld, bias, seq_q_start, seq_q_len, seq_slot, first_long, seqs, max_q_len, width,
                      state, maps, static_cast<float*>(out), stream);
  if (dtype == DTYPE_BF16)
    return run_mingru(static_cast<const __nv_bfloat16*>(proj), ld, bias, seq_q_start, seq_q_len, seq_slot, first_long, seqs, max_q_len,
                      width, state, maps, static_cast<__nv_bfloat16*>(out), stream);
  return b200_fail("mingru: unknown dtype %d", dtype);
}
