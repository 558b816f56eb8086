// Shared pieces of the "hybrid" kernel library: layer norms, gated linear units with clamps, latent
// attention, state-space recurrences and routed experts.
//
// Every exported operation has the signature of a step-plan operation (gb_plan_op.h):
//
//     int gb_op_xxx(const GbPlanCtx* ctx, const long long* a, const double* f, int flags)
//
// so that ONE entry point serves both ways of running a model: the step walker calls it with a
// record's operands (symbols already replaced by the step's values), and the Python wrappers call it
// directly with the same operand list.  It launches on ctx->stream and returns the number of kernels
// launched, or a negative code with the message in gb_last_error().
#pragma once
#include "common.cuh"
#include "gb_plan_op.h"

#define GB_OP(name) GB_API int name(const GbPlanCtx* ctx, const long long* a, const double* f, int flags)

template <typename T> static inline T* op_ptr(long long v) { return reinterpret_cast<T*>(v); }

__device__ __forceinline__ float hy_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float hy_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float hy_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float hy_gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
// g' = min(g, limit), u' = clamp(u, -limit, limit): g' * sigmoid(alpha * g') * (u' + up_add)
__device__ __forceinline__ float hy_clamped_glu(float g, float u, float alpha, float limit, float up_add) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * hy_sigmoid(alpha * g) * (u + up_add);
}

// A 64 x 64 tile of C = A . B^T on the CUDA cores in 32-bit, for 256 threads.  Row i of the tile is
// A[arow(i)] (null: a row of zeros), column j is B[brow(j)] (null likewise), both of K contiguous
// elements.  Every output is one accumulator walking k upwards, so a row's result does not depend on
// which other rows share its tile.  acc[r][c] belongs to tile row ty*4+r, column tx*4+c.
template <typename TA, typename TB, typename ARow, typename BRow>
__device__ __forceinline__ void hy_tile_64x64(ARow arow, BRow brow, int K, float (&acc)[4][4], int& ty, int& tx) {
  __shared__ float As[32][65];          // [k][row]
  __shared__ float Bs[32][65];          // [k][col]
  const int tid = threadIdx.x;
  ty = tid >> 4;
  tx = tid & 15;
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
  // loading: thread (lr, lk) fetches rows lr, lr+8, ... at k offset lk
  const int lk = tid & 31, lr = tid >> 5;
  for (int k0 = 0; k0 < K; k0 += 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = lr + 8 * i;
      const TA* ap = arow(row);
      const TB* bp = brow(row);
      const int k = k0 + lk;
      As[lk][row] = (ap != nullptr && k < K) ? to_f32(ap[k]) : 0.f;
      Bs[lk][row] = (bp != nullptr && k < K) ? to_f32(bp[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) av[r] = As[kk][ty * 4 + r];
#pragma unroll
      for (int c = 0; c < 4; ++c) bv[c] = Bs[kk][tx * 4 + c];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(av[r], bv[c], acc[r][c]);
    }
    __syncthreads();
  }
}
