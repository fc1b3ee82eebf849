// The routed experts' two products for prompt portions on the fifth-generation tensor cores.
//
// `moe_sort` (moe.cu) has given every expert a run of whole tiles of 128 sorted places. A block takes
// one tile and 128 rows of the tile's expert's matrix and computes D[row of W][place] = W_tile X_tile^T
// with `tcgen05.mma` (cta_group::1, kind::f16, bfloat16 operands, 32-bit accumulators in TMEM): one
// thread feeds a ring of stages by TMA (W rows straight from the stacked expert matrices, X rows from
// the sorted activations, both K-major with 128-byte swizzle), one elected thread of a warp issues the
// products, four warps read the accumulators back with `tcgen05.ld` and write the result. With two
// matrices (gate and up) the block keeps two accumulators over the same X tile and its epilogue is the
// clamped gated activation; with one (down) it stores 32-bit rows by slot. The gate/up product reads
// rows gathered into sorted order by `moe_gather_rows` in front (TMA does not gather rows); the down
// product reads the activations where the first product wrote them. Places of padding hold whatever
// the buffer held: a place is a column of D, so it harms no other place, and it is never stored.
// Every wait is bounded; a block that gives up sets the timeout bit, frees its TMEM and leaves.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int kBlockRows = 128;  // rows of W per block = MMA M
constexpr int kPlaces = 128;     // sorted places per tile = MMA N
constexpr int kBlockK = 64;      // k per stage: 128 bytes of bf16 = one swizzle row
constexpr int kMmaK = 16;
constexpr int kThreads = 192;    // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue
constexpr uint32_t kTileBytes = kBlockRows * kBlockK * 2;  // 16 KB, for W and for X tiles alike
constexpr long long kWaitCycles = 4000000000LL;            // about two seconds
constexpr int ERRBIT_TIMEOUT = 8;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity to complete.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_addr(bar);
  const long long start = clock64();
  while (true) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (clock64() - start > kWaitCycles) return false;
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
      : "memory");
}
// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle:
// groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);   // start address
  desc |= static_cast<uint64_t>(1) << 16;                  // leading byte offset (unused for swizzled K-major)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;          // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;                  // descriptor version (sm_100)
  desc |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
  return desc;
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kBlockRows >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float clamped_glu(float g, float u, float limit) {
  if (limit <= 0.f) return g * (1.f / (1.f + expf(-g))) * u;  // a limit of zero: the unclamped form silu(g) * u
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.f / (1.f + expf(-1.702f * g))) * (u + 1.f);
}

struct ExpertProduct {
  const int* place_slot;   // [tiles * kPlaces]: the slot a sorted place holds, -1 for padding
  const int* tile_expert;  // [tiles]
  const int* num_tiles;    // [1]
  int* err;
  int stages;
  int K;
  int rows_per_expert;  // rows of the stacked matrix that belong to one expert
  int second_offset;    // rows from an expert's first matrix to its second (MATS = 2)
  int n_total;          // output columns an expert has (rows of one of its matrices)
  float limit;
  void* out;            // MATS = 2: bfloat16 [places][n_total]; MATS = 1: float [slots][n_total]
};

template <int MATS>
__global__ void __launch_bounds__(kThreads)
moe_tcgen05_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map, const ExpertProduct p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int kMaxStages = 6;
  constexpr uint32_t stage_bytes = (MATS + 1) * kTileBytes;  // W tile(s), then the X tile; all 1024-byte aligned
  constexpr uint32_t tmem_cols = MATS * kPlaces;              // 128 or 256: a power of two
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_shared;
  __shared__ int slot_of[kPlaces];

  // Which tile exists and whose it is comes from the sort kernel in front.
  wait_for_predecessor();
  let_successor_start();
  // Row blocks of W run fastest in the grid: neighbouring blocks share the tile's X rows, and the other tiles of the
  // expert, which want the same rows of W, are in flight at the same time.
  const int tile = blockIdx.y;
  if (tile >= *p.num_tiles) return;  // the whole block, before anything is allocated
  const int expert = p.tile_expert[tile];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int n0 = blockIdx.x * kBlockRows;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int w_row = expert * p.rows_per_expert + n0;
  const int x_row = tile * kPlaces;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x >= 64 && threadIdx.x < 64 + kPlaces) slot_of[threadIdx.x - 64] = p.place_slot[x_row + threadIdx.x - 64];
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_shared)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_shared;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer ----
    for (int i = 0; i < num_kb; ++i) {
      const int s = i % stages;
      if (i >= stages && !mbar_wait(&empty_bar[s], ((i / stages) - 1) & 1)) {
        atomicOr(p.err, ERRBIT_TIMEOUT);
        break;
      }
      unsigned char* stage = tiles + static_cast<size_t>(s) * stage_bytes;
      mbar_expect_tx(&full_bar[s], stage_bytes);
      tma_load_2d(stage, &w_map, &full_bar[s], i * kBlockK, w_row);
      if (MATS == 2) tma_load_2d(stage + kTileBytes, &w_map, &full_bar[s], i * kBlockK, w_row + p.second_offset);
      tma_load_2d(stage + MATS * kTileBytes, &x_map, &full_bar[s], i * kBlockK, x_row);
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the whole warp walks the loop, one elected lane issues ----
    uint32_t chosen;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(chosen));
    const bool leader = chosen != 0;
    const uint32_t idesc = umma_instr_desc(kPlaces);
    const uint64_t a_first = umma_smem_desc(smem_addr(tiles));
    const uint64_t b_first = umma_smem_desc(smem_addr(tiles) + MATS * kTileBytes);
    for (int i = 0; i < num_kb; ++i) {
      const int s = i % stages;
      if (!mbar_wait(&full_bar[s], (i / stages) & 1)) {
        if (leader) atomicOr(p.err, ERRBIT_TIMEOUT);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t stage_units = static_cast<uint64_t>(s) * (stage_bytes >> 4);
#pragma unroll
      for (int k = 0; k < kBlockK / kMmaK; ++k) {
        const uint64_t step = stage_units + static_cast<uint64_t>(k * (kMmaK * 2 >> 4));
        if (leader) {
          umma_bf16(tmem_base, a_first + step, b_first + step, idesc, i > 0 || k > 0);
          if (MATS == 2) umma_bf16(tmem_base + kPlaces, a_first + (kTileBytes >> 4) + step, b_first + step, idesc, i > 0 || k > 0);
        }
      }
      if (leader) umma_commit(&empty_bar[s]);  // the stage may be refilled once these products have read it
      __syncwarp();
    }
    if (leader) umma_commit(&accum_bar);  // the accumulators are complete once every product has retired
  }
  __syncwarp();

  if (warp >= 2) {
    // ---- epilogue: TMEM lanes 32 * quarter .. + 31 are rows of W, columns are places ----
    const int quarter = warp & 3;
    const int n = n0 + quarter * 32 + lane;
    bool have = num_kb > 0;
    if (have && !mbar_wait(&accum_bar, 0)) {
      if (lane == 0) atomicOr(p.err, ERRBIT_TIMEOUT);
      have = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (have) {
      for (int c0 = 0; c0 < kPlaces; c0 += 16) {
        float first[16], second[16];
        tmem_load_16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c0, first);
        if (MATS == 2) tmem_load_16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kPlaces + c0, second);
        if (n < p.n_total) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int slot = slot_of[c0 + i];
            if (slot < 0) continue;
            if (MATS == 2)
              static_cast<__nv_bfloat16*>(p.out)[static_cast<int64_t>(x_row + c0 + i) * p.n_total + n] =
                  __float2bfloat16_rn(clamped_glu(first[i], second[i], p.limit));
            else
              static_cast<float*>(p.out)[static_cast<int64_t>(slot) * p.n_total + n] = first[i];
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// sorted[place] = rows[slot / top] for the slot a place holds, zeros for padding; 16 bytes a thread.
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* rows, const int* place_slot, int places, int top, int width,
                                       __nv_bfloat16* sorted) {
  wait_for_predecessor();
  let_successor_start();
  const int chunks = width / 8;
  const int64_t total = static_cast<int64_t>(places) * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t place = idx / chunks;
    const int c = static_cast<int>(idx % chunks) * 8;
    const int slot = place_slot[place];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (slot >= 0) v = *reinterpret_cast<const uint4*>(rows + static_cast<int64_t>(slot / top) * width + c);
    *reinterpret_cast<uint4*>(sorted + place * width + c) = v;
  }
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(ptr);
  }
  return fn;
}

// A [rows, K] bfloat16 row-major matrix as a 2-D tensor map with boxes of 64 k x 128 rows.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int K) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return b200_fail("moe_tcgen05: the driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t box[2] = {kBlockK, kBlockRows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult status = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) return b200_fail("moe_tcgen05: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(status));
  return 0;
}

template <int MATS>
int launch_product(const CUtensorMap& w_map, const CUtensorMap& x_map, const ExpertProduct& p, int max_tiles, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(p.stages) * (MATS + 1) * kTileBytes + 1024;
  if (cudaFuncSetAttribute(moe_tcgen05_kernel<MATS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return b200_fail("moe_tcgen05: cannot size shared memory (%zu bytes)", smem);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((p.n_total + kBlockRows - 1) / kBlockRows, max_tiles);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = b200_overlap_enabled() ? 1 : 0;
  const cudaError_t status = cudaLaunchKernelEx(&config, moe_tcgen05_kernel<MATS>, w_map, x_map, p);
  if (status != cudaSuccess) return b200_fail("moe_tcgen05: %s", cudaGetErrorString(status));
  return 0;
}

}  // namespace

// Whether the tcgen05 form takes these sizes: both products' K a multiple of 8 (rows of whole 16 bytes).
B200_API int b200_moe_tcgen05_supported(int width, int ff) { return width > 0 && ff > 0 && width % 8 == 0 && ff % 8 == 0 ? 1 : 0; }

B200_API int b200_moe_gather_rows(const void* rows, const int* place_slot, int places, int top, int width, void* sorted,
                                  cudaStream_t stream) {
  if (places == 0) return 0;
  B200_REQUIRE(places > 0 && top > 0 && width > 0 && width % 8 == 0, "moe_gather_rows: bad sizes");
  B200_REQUIRE(reinterpret_cast<uintptr_t>(rows) % 16 == 0 && reinterpret_cast<uintptr_t>(sorted) % 16 == 0, "moe_gather_rows: operands must be 16-byte aligned");
  const int threads = 256;
  const int64_t want = (static_cast<int64_t>(places) * (width / 8) + threads - 1) / threads;
  launch_kernel(moe_gather_rows_kernel, dim3(static_cast<unsigned>(want < 65535 ? want : 65535)), dim3(threads), 0, stream,
                static_cast<const __nv_bfloat16*>(rows), place_slot, places, top, width, static_cast<__nv_bfloat16*>(sorted));
  return b200_check_launch("moe_gather_rows");
}

// One of the two products over tiles of 128 sorted places. `weight`: the experts' matrices stacked, [experts * rows_per_expert][K];
// `x`: [capacity][K] rows in sorted order. mats = 2: rows n and second_offset + n of an expert are gate and up of output column n,
// `out` is bfloat16 [capacity][n_total] (the clamped gated activation); mats = 1: `out` is float [slots][n_total].
B200_API int b200_moe_product_tcgen05(const void* weight, const void* x, const int* place_slot, const int* tile_expert, const int* num_tiles,
                                      int max_tiles, int experts, int rows_per_expert, int second_offset, int n_total, int K, int mats,
                                      float limit, void* out, int stages, int* err, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  B200_REQUIRE(max_tiles > 0 && max_tiles <= 65535 && experts > 0 && rows_per_expert > 0 && n_total > 0 && K > 0 && K % 8 == 0 && (mats == 1 || mats == 2),
               "moe_product_tcgen05: bad sizes");
  B200_REQUIRE(mats == 1 || (second_offset > 0 && second_offset + n_total <= rows_per_expert && limit >= 0.f), "moe_product_tcgen05: bad second matrix");
  B200_REQUIRE(reinterpret_cast<uintptr_t>(weight) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0, "moe_product_tcgen05: operands must be 16-byte aligned");
  // Two stages: 96 KB (gate and up) or 64 KB (down) a block, so that two or three blocks share an SM and one's epilogue runs
  // beside the others' products. Measured on a B200 (2,048 tokens, width 3,584, 32 experts, 4 a token): 630 us for both
  // products with 2 stages, 815 with 3, 844 with 4.
  if (stages <= 0) stages = 2;
  B200_REQUIRE(stages >= 2 && stages <= 6 && static_cast<size_t>(stages) * (mats + 1) * kTileBytes + 1024 <= 200 * 1024,
               "moe_product_tcgen05: %d stages do not fit", stages);
  CUtensorMap w_map, x_map;
  if (make_map(&w_map, weight, static_cast<int64_t>(experts) * rows_per_expert, K) != 0) return -1;
  if (make_map(&x_map, x, static_cast<int64_t>(max_tiles) * kPlaces, K) != 0) return -1;
  ExpertProduct p;
  p.place_slot = place_slot;
  p.tile_expert = tile_expert;
  p.num_tiles = num_tiles;
  p.err = err;
  p.stages = stages;
  p.K = K;
  p.rows_per_expert = rows_per_expert;
  p.second_offset = second_offset;
  p.n_total = n_total;
  p.limit = limit;
  p.out = out;
  return mats == 2 ? launch_product<2>(w_map, x_map, p, max_tiles, stream) : launch_product<1>(w_map, x_map, p, max_tiles, stream);
}
