// The routed experts' products on the tensor cores (bfloat16): tcgen05.mma with the accumulator in
// tensor memory, operands by TMA, as the dense product kernel (gemm_tc.cu) does it, for rows that are
// grouped by expert ON THE DEVICE.
//
// Rows of all (token, choice) pairs lie ordered by expert in one matrix; offsets[e] .. offsets[e + 1]
// is expert e's range, known to the device only.  So the launch covers the most row tiles any routing
// can produce, and every CTA finds its (expert, first row) from the offsets; a CTA beyond the last
// tile returns.  One tensor map covers all rows and one the stacked weights of all experts
// [E * rows_per_expert, K]: a tile of token rows may start at any row (TMA's alignment rule is about
// the innermost coordinate only) and may run into the next expert's rows or weights; what it computes
// for those is not stored.
//
// The weight is the M side of the MMA (128 weight rows per tile, one accumulator lane each), the
// token rows the N side (BN per tile), as in gemm_tc.cu.  Two epilogues:
//   plain   out[row, n] = acc            (32-bit; the experts' down projections)
//   GLU     act[row, f] = g' sigmoid(alpha g') (u' + up_add), g' = min(g, limit), u' = clamp(u, +-limit),
//           for weights whose rows alternate in blocks of 64 between gate and up of the same 64 features
//           (lanes 0-63 of a tile hold g, lanes 64-127 u).
#include <mutex>
#include <unordered_map>

#include "hybrid.cuh"
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128, BK = 64, UMMA_K = 16, STAGES = 4;
constexpr int W_TILE_BYTES = BM * BK * 2;
constexpr int STATUS_TIMEOUT = 24;

struct GroupedParams {
  const int* offsets;
  int E, rows_per_expert, n_valid;   // weight rows per expert in the stacked matrix; rows that exist per expert
  int mode;                          // 0 GLU, 1 plain
  void* out; long long ldo;
  int total_kb;
  float alpha, limit, up_add;
  int* status;
};

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int BN>
__global__ void __launch_bounds__(192)
moe_experts_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                      const GroupedParams p) {
  constexpr int X_TILE_BYTES = BN * BK * 2, STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], tmem_full_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;
  pdl_wait();                                   // the offsets and the rows come from the kernels before

  // this CTA's expert and rows (the same walk in every thread; E is small)
  int e = 0, r0 = 0, r1 = 0;
  {
    int tile = blockIdx.y;
    bool found = false;
    for (e = 0; e < p.E; ++e) {
      const int lo = p.offsets[e], hi = p.offsets[e + 1];
      const int tiles = (hi - lo + BN - 1) / BN;
      if (tile < tiles) { r0 = lo + BN * tile; r1 = hi; found = true; break; }
      tile -= tiles;
    }
    if (!found) return;                         // (before any barrier or tensor-memory allocation)
  }
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = e * p.rows_per_expert + blockIdx.x * BM;     // row of the stacked weights
  const int nkb = p.total_kb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full_bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES) {
          const uint32_t ph = (i / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            abort_flag = 1;
            atomicExch(p.status, STATUS_TIMEOUT);
            break;
          }
          if (abort_flag) break;
        }
        uint8_t* st = tiles + (size_t)s * STAGE_BYTES;
        mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(st, &tmap_w, i * BK, n0, &full_bar[s]);
        tma_load_2d(st + W_TILE_BYTES, &tmap_x, i * BK, r0, &full_bar[s]);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph)) {
          abort_flag = 1;
          atomicExch(p.status, STATUS_TIMEOUT + 1);
          break;
        }
        if (abort_flag) break;
        tc_fence_after();
        uint8_t* st = tiles + (size_t)s * STAGE_BYTES;
        const uint64_t da = smem_desc_sw128(st);
        const uint64_t db = smem_desc_sw128(st + W_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (uint32_t)((i | k) != 0));
        umma_commit(&empty_bar[s]);
      }
      umma_commit(&tmem_full_bar);
    }
    __syncwarp();
  } else {
    // ---- epilogue warps (threads 64..191) ----
    const bool ok = mbar_wait(&tmem_full_bar, 0);
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicExch(p.status, STATUS_TIMEOUT + 2);
    }
    tc_fence_after();
    epilogue_barrier();
    const bool good = !abort_flag;
    const int q = warp & 3;                      // tensor-memory lanes 32q .. 32q + 31
    const int row = 32 * q + lane;               // weight row within the tile
    const int cols = min(BN, r1 - r0);           // token rows of this tile that belong to the expert
    if (good && p.mode == 1) {
      const int n = blockIdx.x * BM + row;       // output feature
      float* out = (float*)p.out;
#pragma unroll 1
      for (int c0 = 0; c0 < cols; c0 += 16) {
        float v[16];
        tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
        if (n < p.n_valid) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < cols) out[(size_t)(r0 + c0 + j) * p.ldo + n] = v[j];
        }
      }
    } else if (good) {
      // u of one 16-column chunk through shared memory (the pipeline's first stage is free once the
      // accumulator is complete); the threads of lanes 0-63 hold g and finish the unit
      float (*ubuf)[17] = reinterpret_cast<float (*)[17]>(tiles);
      bf16* act = (bf16*)p.out;
      const int f = blockIdx.x * 64 + (row & 63);        // feature
#pragma unroll 1
      for (int c0 = 0; c0 < cols; c0 += 16) {
        float v[16];
        tmem_ld_16(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
        if (row >= 64) {
#pragma unroll
          for (int j = 0; j < 16; ++j) ubuf[row - 64][j] = v[j];
        }
        epilogue_barrier();
        if (row < 64 && f < p.n_valid) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < cols)
              act[(size_t)(r0 + c0 + j) * p.ldo + f] =
                  __float2bfloat16_rn(hy_clamped_glu(v[j], ubuf[row][j], p.alpha, p.limit, p.up_add));
        }
        if (c0 + 16 < cols) epilogue_barrier();          // ubuf is rewritten by the next chunk
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // give copies that are still in flight time to land before the shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld (elements), read in boxes of box_rows x 64, 128-byte swizzle.
bool make_tmap(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct WKey {
  const void* p; long long rows, k;
  bool operator==(const WKey& o) const { return p == o.p && rows == o.rows && k == o.k; }
};
struct WKeyHash {
  size_t operator()(const WKey& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.rows) * 31) ^ (std::hash<long long>()(k.k) * 131);
  }
};
std::mutex g_wmap_mutex;
std::unordered_map<WKey, CUtensorMap, WKeyHash> g_wmaps;   // weights do not move: their maps are made once

template <int BN>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, const GroupedParams& p, int weight_tiles, int row_tiles,
           cudaStream_t stream) {
  constexpr int SMEM = STAGES * (W_TILE_BYTES + BN * BK * 2) + 1024;
  static bool raised = false;
  if (!raised) {
    GB_CUDA(cudaFuncSetAttribute(moe_experts_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    raised = true;
  }
  gb_launch(moe_experts_tc_kernel<BN>, dim3(weight_tiles, row_tiles), dim3(192), SMEM, stream, tw, tx, p);
  GB_CHECK_LAUNCH("moe_experts_tc");
  return 1;
}

}  // namespace

// Whether gb_op_moe_experts_tc takes these sizes (mode 0: GLU, the weights' gate and up rows alternating
// in blocks of 64; mode 1: plain).  K: features in; ld: row strides of the rows and of the weights.
GB_API int gb_moe_experts_tc_supported(int mode, int n_out, int K, long long ld_rows, long long ld_w) {
  if (K % 8 || ld_rows % 8 || ld_w % 8) return 0;
  if (mode == 0 && n_out % 64) return 0;
  return 1;
}

// a0 input rows (bf16), a1 their stride, a2 rows the matrix has room for, a3 weights [E, rows per expert, K]
// (bf16, contiguous), a4 unused, a5 offsets [E + 1], a6 experts, a7 out, a8 its row stride, a9 tokens, a10 features out
// (GLU: ff), a11 features in (K), a12 mode (0: GLU, out bf16 [rows, ff]; 1: plain, out f32), a13 top; f0 alpha,
// f1 limit, f2 what is added to u
GB_OP(gb_op_moe_experts_tc) {
  const int pairs = (int)(a[9] * a[13]), E = (int)a[6], n_out = (int)a[10], K = (int)a[11], mode = (int)a[12];
  if (pairs <= 0) return 0;
  if (!gb_moe_experts_tc_supported(mode, n_out, K, a[1], K) || (a[0] & 15) || (a[3] & 15))
    GB_FAIL(GB_ERR_ARG, "moe_experts_tc: sizes or alignment the tensor-core kernel does not take");
  const int rows_per_expert = mode == 0 ? 2 * n_out : n_out;
  CUtensorMap tw, tx;
  {
    std::lock_guard<std::mutex> lock(g_wmap_mutex);
    const WKey key{op_ptr<const void>(a[3]), (long long)E * rows_per_expert, K};
    auto it = g_wmaps.find(key);
    if (it == g_wmaps.end()) {
      if (!make_tmap(&tw, key.p, key.rows, K, K, BM)) GB_FAIL(GB_ERR_CUDA, "moe_experts_tc: cuTensorMapEncodeTiled failed (W)");
      g_wmaps.emplace(key, tw);
    } else {
      tw = it->second;
    }
  }
  // few rows an expert (decoding): narrow token tiles
  const int BN = pairs <= 16 * E ? 16 : 64;
  if (!make_tmap(&tx, op_ptr<const void>(a[0]), a[2], K, a[1], BN))
    GB_FAIL(GB_ERR_CUDA, "moe_experts_tc: cuTensorMapEncodeTiled failed (rows)");
  GroupedParams p;
  p.offsets = op_ptr<const int>(a[5]);
  p.E = E; p.rows_per_expert = rows_per_expert; p.n_valid = n_out; p.mode = mode;
  p.out = op_ptr<void>(a[7]); p.ldo = a[8];
  p.total_kb = gb_div_up(K, BK);
  p.alpha = (float)f[0]; p.limit = (float)f[1]; p.up_add = (float)f[2];
  p.status = ctx->status;
  const int weight_tiles = gb_div_up(rows_per_expert, BM);
  const int row_tiles = gb_div_up(pairs, BN) + E;          // at most this many over all experts
  return BN == 16 ? launch<16>(tw, tx, p, weight_tiles, row_tiles, ctx->stream)
                  : launch<64>(tw, tx, p, weight_tiles, row_tiles, ctx->stream);
}

// Forget the tensor maps of weights (a model was unloaded).
GB_API void gb_moe_experts_tc_forget() {
  std::lock_guard<std::mutex> lock(g_wmap_mutex);
  g_wmaps.clear();
}
