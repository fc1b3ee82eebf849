// A routed feed-forward: the router's choice, the tokens grouped by expert, the experts' two
// products over those groups, and the weighted sum; plus the clamped gated activation of a dense
// expert of the same form.
//
// Router (one warp per token, all 32-bit): s = sigmoid(z); the experts form `groups` equal groups of
// neighbours, a group scores the sum of its two largest s, only experts of the `keep` best groups can
// be chosen; the `top` largest s among them are chosen (ties: the lower index), and their weights are
// s / (sum of the chosen s + 1e-20) * scale. A second kind of router (`softmax_chosen`) scores an expert by its logit
// itself, z plus a learned bias per expert, chooses the `top` largest and weighs them by the softmax over the chosen
// logits only, times scale. A bias may be given to either kind.
//
// Expert: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), y = g sigmoid(1.702 g) (u + 1),
// output W_down y. A limit of zero means the unclamped form y = silu(W_gate h) * (W_up h).
//
// Grouping: every (token, choice) pair is a slot. `moe_sort` (one block) counts the slots of each
// expert, gives each expert a run of whole tiles of `tile_rows` sorted places (kTileM, or four times
// that for prompt portions on tensor cores) and writes, per place, the
// slot it holds (-1: padding) and, per tile, its expert. The two product kernels walk tiles: a tile's
// rows share one expert's weights. Each output number is one thread's sum over K in a fixed order, so
// a slot's result does not depend on which other slots share its tile, and the final sum over a
// token's choices runs in the router's order: nothing depends on the batch.
#include "common.cuh"

namespace {

constexpr int kTileM = 32;
constexpr int kTileN = 32;
constexpr int kTileK = 32;
constexpr int kGemmThreads = 256;  // 8 row groups of 4 rows x 32 columns

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ float clamped_glu(float g, float u, float limit) {
  if (limit <= 0.f) return g * sigmoid_f(g) * u;  // no clamps: silu(g) * u
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoid_f(1.702f * g) * (u + 1.f);
}

// The lane holding the largest value (ties: the lowest index) among the lanes' candidates.
__device__ __forceinline__ void warp_argmax(float& value, int& index) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, value, o);
    const int other_index = __shfl_xor_sync(0xffffffffu, index, o);
    if (other > value || (other == value && other_index < index)) {
      value = other;
      index = other_index;
    }
  }
}

// z [tokens][experts] -> ids [tokens][top], weights [tokens][top]. Shared memory per warp:
// experts scores + groups group scores.
__global__ void moe_route_kernel(const float* z, const float* __restrict__ bias, int softmax_chosen, int tokens, int experts, int groups,
                                 int keep, int top, float scale, int* ids, float* weights) {
  extern __shared__ float route_smem[];
  wait_for_predecessor();
  let_successor_start();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int t = blockIdx.x * warps + warp;
  if (t >= tokens) return;
  float* s = route_smem + warp * (experts + groups);
  float* gs = s + experts;
  const int size = experts / groups;
  for (int e = lane; e < experts; e += 32) {
    const float logit = z[static_cast<int64_t>(t) * experts + e] + (bias ? bias[e] : 0.f);
    s[e] = softmax_chosen ? logit : sigmoid_f(logit);
  }
  __syncwarp();
  for (int g = lane; g < groups; g += 32) {
    float first = -INFINITY, second = -INFINITY;
    for (int i = 0; i < size; ++i) {
      const float v = s[g * size + i];
      if (v > first) {
        second = first;
        first = v;
      } else if (v > second) {
        second = v;
      }
    }
    gs[g] = size > 1 ? first + second : first;
  }
  __syncwarp();
  // Keep the best groups: the others' experts leave the contest.
  if (keep < groups) {
    for (int round = 0; round < keep; ++round) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (gs[g] > best) best = gs[g], at = g;  // indices grow along a lane: the first maximum stays
      warp_argmax(best, at);
      if (lane == 0) gs[at] = -INFINITY;  // marks a kept group
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gs[e / size] != -INFINITY) s[e] = -INFINITY;
    __syncwarp();
  }
  float sum = 0.f, mine = 0.f;
  int mine_id = 0;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32)
      if (s[e] > best) best = s[e], at = e;
    warp_argmax(best, at);
    if (at >= experts) at = 0, best = 0.f;  // cannot happen with a valid configuration and finite logits
    sum += best;
    if (lane == j % 32 && j < 32) mine = best, mine_id = at;
    if (j >= 32 && lane == 0) {  // more than 32 choices: written unnormalised, fixed up below
      ids[static_cast<int64_t>(t) * top + j] = at;
      weights[static_cast<int64_t>(t) * top + j] = best;
    }
    if (lane == 0) s[at] = -INFINITY;
    __syncwarp();
  }
  if (softmax_chosen) {
    // The first choice is the largest logit. exp(logit - largest) over the chosen, then their share of the sum.
    const float largest = __shfl_sync(0xffffffffu, mine, 0);
    float e_mine = lane < top ? expf(mine - largest) : 0.f;
    float total = warp_sum(e_mine);
    if (lane == 0)
      for (int j = 32; j < top; ++j) {
        const float e = expf(weights[static_cast<int64_t>(t) * top + j] - largest);
        weights[static_cast<int64_t>(t) * top + j] = e;
        total += e;
      }
    total = __shfl_sync(0xffffffffu, total, 0);
    const float share = scale / total;
    if (lane < top) {
      ids[static_cast<int64_t>(t) * top + lane] = mine_id;
      weights[static_cast<int64_t>(t) * top + lane] = e_mine * share;
    }
    if (lane == 0)
      for (int j = 32; j < top; ++j) weights[static_cast<int64_t>(t) * top + j] *= share;
    return;
  }
  const float factor = scale / (sum + 1e-20f);
  if (lane < top) {
    ids[static_cast<int64_t>(t) * top + lane] = mine_id;
    weights[static_cast<int64_t>(t) * top + lane] = mine * factor;
  }
  if (lane == 0)
    for (int j = 32; j < top; ++j) weights[static_cast<int64_t>(t) * top + j] *= factor;
}

// One block. ids [slots]; place_slot [capacity]; tile_expert [max_tiles]; num_tiles [1].
__global__ void moe_sort_kernel(const int* ids, int slots, int experts, int capacity, int tile_rows, int* place_slot, int* tile_expert,
                                int* num_tiles) {
  extern __shared__ int sort_smem[];  // counts [experts], cursor [experts]
  int* counts = sort_smem;
  int* cursor = counts + experts;
  wait_for_predecessor();
  let_successor_start();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  for (int i = threadIdx.x; i < capacity; i += blockDim.x) place_slot[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < slots; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tile = 0;
    for (int e = 0; e < experts; ++e) {
      cursor[e] = tile * tile_rows;
      const int tiles = (counts[e] + tile_rows - 1) / tile_rows;
      for (int i = 0; i < tiles; ++i) tile_expert[tile + i] = e;
      tile += tiles;
    }
    *num_tiles = tile;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < slots; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) place_slot[atomicAdd(&cursor[e], 1)] = i;
  }
}

// act[place][n] = glu(h[token(place)] . W_gate[e][n], h . W_up[e][n]) for the tile's expert e.
// w_gate_up [experts][2 * ff][width]: rows 0 .. ff are the gate's, the rest the up projection's.
template <typename T>
__global__ void __launch_bounds__(kGemmThreads)
moe_gate_up_kernel(const T* h, const T* __restrict__ weight, const int* place_slot, const int* tile_expert, const int* num_tiles, int top,
                   int width, int ff, float limit, T* act) {
  __shared__ float a_tile[kTileM][kTileK + 1];
  __shared__ float g_tile[kTileN][kTileK + 1];
  __shared__ float u_tile[kTileN][kTileK + 1];
  __shared__ int row_token[kTileM];
  wait_for_predecessor();
  let_successor_start();
  const int tile = blockIdx.x;
  if (tile >= *num_tiles) return;
  const int expert = tile_expert[tile];
  const int n0 = blockIdx.y * kTileN;
  const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
  if (tid < kTileM) {
    const int slot = place_slot[tile * kTileM + tid];
    row_token[tid] = slot < 0 ? -1 : slot / top;
  }
  __syncthreads();
  const T* wg = weight + static_cast<int64_t>(expert) * 2 * ff * width;
  const T* wu = wg + static_cast<int64_t>(ff) * width;
  float acc_g[4] = {0.f, 0.f, 0.f, 0.f}, acc_u[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < width; k0 += kTileK) {
    for (int idx = tid; idx < kTileM * kTileK; idx += kGemmThreads) {
      const int r = idx / kTileK, c = idx % kTileK;
      const int token = row_token[r];
      a_tile[r][c] = (token >= 0 && k0 + c < width) ? to_f32<T>(h[static_cast<int64_t>(token) * width + k0 + c]) : 0.f;
      const int n = n0 + r;
      const bool in = n < ff && k0 + c < width;
      g_tile[r][c] = in ? to_f32<T>(wg[static_cast<int64_t>(n) * width + k0 + c]) : 0.f;
      u_tile[r][c] = in ? to_f32<T>(wu[static_cast<int64_t>(n) * width + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kTileK; ++kk) {
      const float bg = g_tile[tx][kk], bu = u_tile[tx][kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = a_tile[ty * 4 + i][kk];
        acc_g[i] = fmaf(a, bg, acc_g[i]);
        acc_u[i] = fmaf(a, bu, acc_u[i]);
      }
    }
    __syncthreads();
  }
  const int n = n0 + tx;
  if (n >= ff) return;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (row_token[r] >= 0)
      act[(static_cast<int64_t>(tile) * kTileM + r) * ff + n] = from_f32<T>(clamped_glu(acc_g[i], acc_u[i], limit));
  }
}

// out[slot(place)][n] = act[place] . W_down[e][n] (32-bit, not yet weighted). w_down [experts][width][ff].
template <typename T>
__global__ void __launch_bounds__(kGemmThreads)
moe_down_kernel(const T* act, const T* __restrict__ weight, const int* place_slot, const int* tile_expert, const int* num_tiles,
                int width, int ff, float* out) {
  __shared__ float a_tile[kTileM][kTileK + 1];
  __shared__ float b_tile[kTileN][kTileK + 1];
  __shared__ int row_slot[kTileM];
  wait_for_predecessor();
  let_successor_start();
  const int tile = blockIdx.x;
  if (tile >= *num_tiles) return;
  const int expert = tile_expert[tile];
  const int n0 = blockIdx.y * kTileN;
  const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
  if (tid < kTileM) row_slot[tid] = place_slot[tile * kTileM + tid];
  __syncthreads();
  const T* w = weight + static_cast<int64_t>(expert) * width * ff;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < ff; k0 += kTileK) {
    for (int idx = tid; idx < kTileM * kTileK; idx += kGemmThreads) {
      const int r = idx / kTileK, c = idx % kTileK;
      a_tile[r][c] = (row_slot[r] >= 0 && k0 + c < ff) ? to_f32<T>(act[(static_cast<int64_t>(tile) * kTileM + r) * ff + k0 + c]) : 0.f;
      const int n = n0 + r;
      b_tile[r][c] = (n < width && k0 + c < ff) ? to_f32<T>(w[static_cast<int64_t>(n) * ff + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kTileK; ++kk) {
      const float b = b_tile[tx][kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(a_tile[ty * 4 + i][kk], b, acc[i]);
    }
    __syncthreads();
  }
  const int n = n0 + tx;
  if (n >= width) return;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int slot = row_slot[ty * 4 + i];
    if (slot >= 0) out[static_cast<int64_t>(slot) * width + n] = acc[i];
  }
}

// The same two products on tensor cores (bfloat16 operands, 32-bit sums): a block takes one tile of
// 32 * MT sorted places and kMmaN output columns of each of its MATS matrices (2: gate and up with the
// activation as epilogue; 1: down) and walks K in steps of kMmaK through a ring of kMmaStages cp.async stages
// in dynamic shared memory (one block barrier a step: a stage is refilled right after the barrier that
// follows its last use);
// fragments by ldmatrix, `mma.sync` m16n8k16. MT = 1 (steps with few tokens per expert: four warps, 16
// columns each) or 4 (prompt portions: eight warps as 4 x 2, each 32 rows x 32 columns, so that a
// weight tile fetched from L2 serves 128 rows). A row's sums depend on the row, the weights and K only
// (a fixed order of k steps), not on the tile's other rows or on MT. Rows of A start at `a_rows[r]`
// (null: zeros); K must be a multiple of 8 (16-byte copies).
constexpr int kMmaN = 64;
constexpr int kMmaK = 64;
constexpr int kMmaPitch = kMmaK + 8;  // 144 bytes a row: ldmatrix reads without bank conflicts
constexpr int kMmaStages = 3;
constexpr int kWideTiles = 4;         // MT of the prompt form

template <int MT>
struct MmaShape {
  static constexpr int rows = 32 * MT;
  static constexpr int threads = MT == 1 ? 128 : 256;
  static constexpr int warps_n = MT == 1 ? 4 : 2;
  static constexpr int n_tiles = kMmaN / warps_n / 8;  // n8 tiles a warp: 2 or 4
  static constexpr size_t smem(int mats) { return sizeof(__nv_bfloat16) * kMmaStages * (rows + mats * kMmaN) * kMmaPitch; }
};

__device__ __forceinline__ void copy16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// acc[mat][m16 tile][n8 tile][4] of this warp's 32 rows (`warp_m`) and columns (`warp_n`); `b_rows[mat]` is row n0
// of matrix `mat` ([.][K], K contiguous), `n_valid` how many of the kMmaN rows exist.
template <int MATS, int MT>
__device__ __forceinline__ void tile_product(const __nv_bfloat16* const* a_rows, const __nv_bfloat16* const (&b_rows)[MATS], int n_valid, int K,
                                             __nv_bfloat16 (*a_smem)[32 * MT][kMmaPitch], __nv_bfloat16 (*b_smem)[MATS][kMmaN][kMmaPitch],
                                             float (&acc)[MATS][2][MmaShape<MT>::n_tiles][4]) {
  using Shape = MmaShape<MT>;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int warp_m = warp / Shape::warps_n, warp_n = warp % Shape::warps_n;
#pragma unroll
  for (int mat = 0; mat < MATS; ++mat)
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int n = 0; n < Shape::n_tiles; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mat][m][n][i] = 0.f;
  auto fetch = [&](int stage, int k0) {
#pragma unroll
    for (int i = 0; i < Shape::rows * (kMmaK / 8) / Shape::threads; ++i) {
      const int chunk = tid + i * Shape::threads;
      const int r = chunk / (kMmaK / 8), c = (chunk % (kMmaK / 8)) * 8;
      const __nv_bfloat16* src = a_rows[r];
      const bool in = src != nullptr && k0 + c < K;
      copy16(&a_smem[stage][r][c], in ? src + k0 + c : b_rows[0], in);
    }
#pragma unroll
    for (int mat = 0; mat < MATS; ++mat)
#pragma unroll
      for (int i = 0; i < kMmaN * (kMmaK / 8) / Shape::threads; ++i) {
        const int chunk = tid + i * Shape::threads;
        const int r = chunk / (kMmaK / 8), c = (chunk % (kMmaK / 8)) * 8;
        const bool in = r < n_valid && k0 + c < K;
        copy16(&b_smem[stage][mat][r][c], in ? b_rows[mat] + static_cast<int64_t>(r) * K + k0 + c : b_rows[0], in);
      }
  };
  const int steps = (K + kMmaK - 1) / kMmaK;
#pragma unroll
  for (int ahead = 0; ahead < kMmaStages - 1; ++ahead) {
    if (ahead < steps) fetch(ahead, ahead * kMmaK);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int step = 0; step < steps; ++step) {
    const int stage = step % kMmaStages;
    asm volatile("cp.async.wait_group %0;" ::"n"(kMmaStages - 2) : "memory");
    __syncthreads();  // this step's stage has landed for everyone, and everyone is done with the stage refilled next
    if (step + kMmaStages - 1 < steps) fetch((step + kMmaStages - 1) % kMmaStages, (step + kMmaStages - 1) * kMmaK);
    asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
    for (int kk = 0; kk < kMmaK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int m = 0; m < 2; ++m)
        ldmatrix4(a[m], &a_smem[stage][warp_m * 32 + m * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int mat = 0; mat < MATS; ++mat)
#pragma unroll
        for (int pair = 0; pair < Shape::n_tiles / 2; ++pair) {
          uint32_t b[4];  // two n8 tiles: (b0, b1) of columns 0..7 and of columns 8..15 of this pair's 16
          ldmatrix4(b, &b_smem[stage][mat][warp_n * (8 * Shape::n_tiles) + pair * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            mma_bf16(acc[mat][m][2 * pair], a[m], b[0], b[1]);
            mma_bf16(acc[mat][m][2 * pair + 1], a[m], b[2], b[3]);
          }
        }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int MT>
__global__ void __launch_bounds__(MmaShape<MT>::threads)
moe_gate_up_mma_kernel(const __nv_bfloat16* h, const __nv_bfloat16* __restrict__ weight, const int* place_slot, const int* tile_expert,
                       const int* num_tiles, int top, int width, int ff, float limit, __nv_bfloat16* act) {
  using Shape = MmaShape<MT>;
  extern __shared__ __align__(16) unsigned char mma_smem[];
  auto a_smem = reinterpret_cast<__nv_bfloat16(*)[Shape::rows][kMmaPitch]>(mma_smem);
  auto b_smem = reinterpret_cast<__nv_bfloat16(*)[2][kMmaN][kMmaPitch]>(mma_smem + sizeof(__nv_bfloat16) * kMmaStages * Shape::rows * kMmaPitch);
  __shared__ const __nv_bfloat16* a_rows[Shape::rows];
  wait_for_predecessor();
  let_successor_start();
  const int tile = blockIdx.x;
  if (tile >= *num_tiles) return;
  const int expert = tile_expert[tile];
  const int n0 = blockIdx.y * kMmaN;
  if (threadIdx.x < Shape::rows) {
    const int slot = place_slot[tile * Shape::rows + threadIdx.x];
    a_rows[threadIdx.x] = slot < 0 ? nullptr : h + static_cast<int64_t>(slot / top) * width;
  }
  __syncthreads();
  const __nv_bfloat16* wg = weight + (static_cast<int64_t>(expert) * 2 * ff + n0) * width;
  const __nv_bfloat16* const b_rows[2] = {wg, wg + static_cast<int64_t>(ff) * width};
  float acc[2][2][Shape::n_tiles][4];
  tile_product<2, MT>(a_rows, b_rows, min(kMmaN, ff - n0), width, a_smem, b_smem, acc);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warp_m = warp / Shape::warps_n, warp_n = warp % Shape::warps_n;
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < Shape::n_tiles; ++n)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = warp_m * 32 + m * 16 + (lane >> 2) + half * 8;
        const int col = n0 + warp_n * (8 * Shape::n_tiles) + n * 8 + (lane & 3) * 2;
        if (a_rows[r] == nullptr || col >= ff) continue;  // ff is even: the pair is whole
        const float y0 = clamped_glu(acc[0][m][n][half * 2], acc[1][m][n][half * 2], limit);
        const float y1 = clamped_glu(acc[0][m][n][half * 2 + 1], acc[1][m][n][half * 2 + 1], limit);
        *reinterpret_cast<__nv_bfloat162*>(act + (static_cast<int64_t>(tile) * Shape::rows + r) * ff + col) = __floats2bfloat162_rn(y0, y1);
      }
}

template <int MT>
__global__ void __launch_bounds__(MmaShape<MT>::threads)
moe_down_mma_kernel(const __nv_bfloat16* act, const __nv_bfloat16* __restrict__ weight, const int* place_slot, const int* tile_expert,
                    const int* num_tiles, int width, int ff, float* out) {
  using Shape = MmaShape<MT>;
  extern __shared__ __align__(16) unsigned char mma_smem[];
  auto a_smem = reinterpret_cast<__nv_bfloat16(*)[Shape::rows][kMmaPitch]>(mma_smem);
  auto b_smem = reinterpret_cast<__nv_bfloat16(*)[1][kMmaN][kMmaPitch]>(mma_smem + sizeof(__nv_bfloat16) * kMmaStages * Shape::rows * kMmaPitch);
  __shared__ const __nv_bfloat16* a_rows[Shape::rows];
  __shared__ int row_slot[Shape::rows];
  wait_for_predecessor();
  let_successor_start();
  const int tile = blockIdx.x;
  if (tile >= *num_tiles) return;
  const int expert = tile_expert[tile];
  const int n0 = blockIdx.y * kMmaN;
  if (threadIdx.x < Shape::rows) {
    const int slot = place_slot[tile * Shape::rows + threadIdx.x];
    row_slot[threadIdx.x] = slot;
    a_rows[threadIdx.x] = slot < 0 ? nullptr : act + (static_cast<int64_t>(tile) * Shape::rows + threadIdx.x) * ff;
  }
  __syncthreads();
  const __nv_bfloat16* const b_rows[1] = {weight + (static_cast<int64_t>(expert) * width + n0) * ff};
  float acc[1][2][Shape::n_tiles][4];
  tile_product<1, MT>(a_rows, b_rows, min(kMmaN, width - n0), ff, a_smem, b_smem, acc);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warp_m = warp / Shape::warps_n, warp_n = warp % Shape::warps_n;
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < Shape::n_tiles; ++n)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = warp_m * 32 + m * 16 + (lane >> 2) + half * 8;
        const int col = n0 + warp_n * (8 * Shape::n_tiles) + n * 8 + (lane & 3) * 2;
        if (row_slot[r] < 0 || col >= width) continue;  // width is even: the pair is whole
        *reinterpret_cast<float2*>(out + static_cast<int64_t>(row_slot[r]) * width + col) = make_float2(acc[0][m][n][half * 2], acc[0][m][n][half * 2 + 1]);
      }
}

// out[t] = sum_j weights[t][j] * expert_out[t * top + j] (+ shared[t]), in the order of j.
template <typename T>
__global__ void moe_combine_kernel(const float* expert_out, const float* weights, const T* shared, int top, int width, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j)
      acc = fmaf(weights[static_cast<int64_t>(t) * top + j], expert_out[(static_cast<int64_t>(t) * top + j) * width + d], acc);
    if (shared) acc += to_f32<T>(shared[static_cast<int64_t>(t) * width + d]);
    out[static_cast<int64_t>(t) * width + d] = from_f32<T>(acc);
  }
}

// gate_up rows are [gate (ff) | up (ff)].
template <typename T>
__global__ void clamped_glu_kernel(const T* gate_up, int64_t rows, int ff, float limit, T* out) {
  wait_for_predecessor();
  let_successor_start();
  const int64_t total = rows * ff;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / ff;
    const int c = static_cast<int>(idx % ff);
    out[idx] = from_f32<T>(clamped_glu(to_f32<T>(gate_up[r * 2 * ff + c]), to_f32<T>(gate_up[r * 2 * ff + ff + c]), limit));
  }
}

// The same for bfloat16 rows whose halves start on 16-byte boundaries (ff a multiple of 8): eight outputs a thread.
__global__ void clamped_glu_wide_kernel(const __nv_bfloat16* gate_up, int64_t rows, int ff, float limit, __nv_bfloat16* out) {
  wait_for_predecessor();
  let_successor_start();
  const int chunks = ff / 8;
  const int64_t total = rows * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / chunks;
    const int c = static_cast<int>(idx % chunks) * 8;
    const uint4 graw = *reinterpret_cast<const uint4*>(gate_up + r * 2 * ff + c);
    const uint4 uraw = *reinterpret_cast<const uint4*>(gate_up + r * 2 * ff + ff + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 packed;
    __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      y2[j] = __floats2bfloat162_rn(clamped_glu(g.x, u.x, limit), clamped_glu(g.y, u.y, limit));
    }
    *reinterpret_cast<uint4*>(out + r * ff + c) = packed;
  }
}

}  // namespace

B200_API int b200_moe_tile_rows() { return kTileM; }

B200_API int b200_moe_route(const float* z, const float* bias, int softmax_chosen, int tokens, int experts, int groups, int keep, int top,
                            float scale, int* ids, float* weights, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && experts > 0 && groups > 0 && experts % groups == 0 && keep > 0 && keep <= groups && top > 0 &&
                   top <= keep * (experts / groups),
               "moe_route: %d experts in %d groups, %d kept, %d chosen", experts, groups, keep, top);
  const int warps = 4;
  const size_t smem = sizeof(float) * warps * (experts + groups);
  B200_REQUIRE(smem <= 48 * 1024, "moe_route: %d experts do not fit shared memory", experts);
  launch_kernel(moe_route_kernel, dim3((tokens + warps - 1) / warps), dim3(32 * warps), smem, stream, z, bias, softmax_chosen, tokens, experts,
                groups, keep, top, scale, ids, weights);
  return b200_check_launch("moe_route");
}

B200_API int b200_moe_sort(const int* ids, int slots, int experts, int capacity, int tile_rows, int* place_slot, int* tile_expert,
                           int* num_tiles, cudaStream_t stream) {
  if (slots == 0) return 0;
  B200_REQUIRE(slots > 0 && experts > 0 && capacity >= slots, "moe_sort: bad sizes");
  B200_REQUIRE(tile_rows == kTileM || tile_rows == kTileM * kWideTiles, "moe_sort: tiles of %d or %d rows", kTileM, kTileM * kWideTiles);
  B200_REQUIRE(capacity % tile_rows == 0 && capacity / tile_rows >= (slots + experts * (tile_rows - 1)) / tile_rows,
               "moe_sort: %d places do not hold %d slots of %d experts in whole tiles", capacity, slots, experts);
  const size_t smem = sizeof(int) * 2 * experts;
  B200_REQUIRE(smem <= 48 * 1024, "moe_sort: too many experts");
  launch_kernel(moe_sort_kernel, dim3(1), dim3(1024), smem, stream, ids, slots, experts, capacity, tile_rows, place_slot, tile_expert,
                num_tiles);
  return b200_check_launch("moe_sort");
}

static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// Whether the tensor-core form takes these sizes (bfloat16; K a multiple of 8 for both products).
B200_API int b200_moe_mma_supported(int width, int ff) { return width % 8 == 0 && ff % 8 == 0 ? 1 : 0; }

// `tile_rows`: what `moe_sort` was given. kTileM: the plain kernels, or with `use_mma` (bfloat16, sizes that
// `moe_mma_supported` takes) the tensor-core form; four times kTileM: the tensor-core form only.
B200_API int b200_moe_gate_up(const void* h, const void* weight, const int* place_slot, const int* tile_expert, const int* num_tiles,
                              int max_tiles, int tile_rows, int top, int width, int ff, float limit, void* act, int dtype, int use_mma,
                              cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  B200_REQUIRE(max_tiles > 0 && top > 0 && width > 0 && ff > 0 && limit >= 0.f, "moe_gate_up: bad sizes");
  const bool mma = dtype == DTYPE_BF16 && use_mma && b200_moe_mma_supported(width, ff) && aligned16(h) && aligned16(weight) && aligned16(act);
  B200_REQUIRE(tile_rows == kTileM || (mma && tile_rows == kTileM * kWideTiles), "moe_gate_up: tiles of %d rows are not taken here", tile_rows);
  const dim3 grid(max_tiles, (ff + kTileN - 1) / kTileN);
  B200_REQUIRE(grid.y <= 65535, "moe_gate_up: too many columns");
  if (dtype == DTYPE_F32) {
    launch_kernel(moe_gate_up_kernel<float>, grid, dim3(kGemmThreads), 0, stream, static_cast<const float*>(h),
                  static_cast<const float*>(weight), place_slot, tile_expert, num_tiles, top, width, ff, limit, static_cast<float*>(act));
  } else if (mma) {
    const dim3 mma_grid(max_tiles, (ff + kMmaN - 1) / kMmaN);
    auto launch = [&](auto kernel, int threads, size_t smem) {
      if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      launch_kernel(kernel, mma_grid, dim3(threads), smem, stream, static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(weight),
                    place_slot, tile_expert, num_tiles, top, width, ff, limit, static_cast<__nv_bfloat16*>(act));
    };
    if (tile_rows == kTileM) launch(moe_gate_up_mma_kernel<1>, MmaShape<1>::threads, MmaShape<1>::smem(2));
    else launch(moe_gate_up_mma_kernel<kWideTiles>, MmaShape<kWideTiles>::threads, MmaShape<kWideTiles>::smem(2));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(moe_gate_up_kernel<__nv_bfloat16>, grid, dim3(kGemmThreads), 0, stream, static_cast<const __nv_bfloat16*>(h),
                  static_cast<const __nv_bfloat16*>(weight), place_slot, tile_expert, num_tiles, top, width, ff, limit,
                  static_cast<__nv_bfloat16*>(act));
  } else {
    return b200_fail("moe_gate_up: unknown dtype %d", dtype);
  }
  return b200_check_launch("moe_gate_up");
}

B200_API int b200_moe_down(const void* act, const void* weight, const int* place_slot, const int* tile_expert, const int* num_tiles,
                           int max_tiles, int tile_rows, int width, int ff, float* out, int dtype, int use_mma, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  B200_REQUIRE(max_tiles > 0 && width > 0 && ff > 0, "moe_down: bad sizes");
  const bool mma = dtype == DTYPE_BF16 && use_mma && b200_moe_mma_supported(width, ff) && aligned16(act) && aligned16(weight) && aligned16(out);
  B200_REQUIRE(tile_rows == kTileM || (mma && tile_rows == kTileM * kWideTiles), "moe_down: tiles of %d rows are not taken here", tile_rows);
  const dim3 grid(max_tiles, (width + kTileN - 1) / kTileN);
  B200_REQUIRE(grid.y <= 65535, "moe_down: too many columns");
  if (dtype == DTYPE_F32) {
    launch_kernel(moe_down_kernel<float>, grid, dim3(kGemmThreads), 0, stream, static_cast<const float*>(act),
                  static_cast<const float*>(weight), place_slot, tile_expert, num_tiles, width, ff, out);
  } else if (mma) {
    const dim3 mma_grid(max_tiles, (width + kMmaN - 1) / kMmaN);
    auto launch = [&](auto kernel, int threads, size_t smem) {
      if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      launch_kernel(kernel, mma_grid, dim3(threads), smem, stream, static_cast<const __nv_bfloat16*>(act), static_cast<const __nv_bfloat16*>(weight),
                    place_slot, tile_expert, num_tiles, width, ff, out);
    };
    if (tile_rows == kTileM) launch(moe_down_mma_kernel<1>, MmaShape<1>::threads, MmaShape<1>::smem(1));
    else launch(moe_down_mma_kernel<kWideTiles>, MmaShape<kWideTiles>::threads, MmaShape<kWideTiles>::smem(1));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(moe_down_kernel<__nv_bfloat16>, grid, dim3(kGemmThreads), 0, stream, static_cast<const __nv_bfloat16*>(act),
                  static_cast<const __nv_bfloat16*>(weight), place_slot, tile_expert, num_tiles, width, ff, out);
  } else {
    return b200_fail("moe_down: unknown dtype %d", dtype);
  }
  return b200_check_launch("moe_down");
}

B200_API int b200_moe_combine(const float* expert_out, const float* weights, const void* shared, int tokens, int top, int width, void* out,
                              int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && top > 0 && width > 0, "moe_combine: bad sizes");
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == DTYPE_F32) {
    launch_kernel(moe_combine_kernel<float>, dim3(tokens), dim3(threads), 0, stream, expert_out, weights, static_cast<const float*>(shared),
                  top, width, static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(moe_combine_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, expert_out, weights,
                  static_cast<const __nv_bfloat16*>(shared), top, width, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("moe_combine: unknown dtype %d", dtype);
  }
  return b200_check_launch("moe_combine");
}

B200_API int b200_clamped_glu(const void* gate_up, int rows, int ff, float limit, void* out, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && ff > 0 && limit >= 0.f, "clamped_glu: bad sizes");
  const int threads = 256;
  const int64_t total = static_cast<int64_t>(rows) * ff;
  const int64_t want = (total + threads - 1) / threads;
  const dim3 grid(static_cast<unsigned>(want < 65535 ? want : 65535));
  if (dtype == DTYPE_F32) {
    launch_kernel(clamped_glu_kernel<float>, grid, dim3(threads), 0, stream, static_cast<const float*>(gate_up), static_cast<int64_t>(rows),
                  ff, limit, static_cast<float*>(out));
  } else if (dtype == DTYPE_BF16 && ff % 8 == 0 && aligned16(gate_up) && aligned16(out)) {
    const int64_t wide = (total / 8 + threads - 1) / threads;
    launch_kernel(clamped_glu_wide_kernel, dim3(static_cast<unsigned>(wide < 65535 ? wide : 65535)), dim3(threads), 0, stream,
                  static_cast<const __nv_bfloat16*>(gate_up), static_cast<int64_t>(rows), ff, limit, static_cast<__nv_bfloat16*>(out));
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(clamped_glu_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(gate_up),
                  static_cast<int64_t>(rows), ff, limit, static_cast<__nv_bfloat16*>(out));
  } else {
    return b200_fail("clamped_glu: unknown dtype %d", dtype);
  }
  return b200_check_launch("clamped_glu");
}
