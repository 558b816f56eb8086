// A selective state-space mixer (the scalar-decay, multi-head form) over a ragged batch of prompt
// portions and single decoded tokens, with per-request state in slots.
//
//  gb_op_causal_conv_silu   per channel: silu(bias + sum_j taps[c][j] * in[t - (K-1) + j]); the K-1 inputs
//                           before a portion come from the request's slot (zeros for a new request), and
//                           the slot then receives the portion's last K-1 inputs.
//  gb_op_ssm_scan           per head h (group g = h / (heads/groups)), token after token:
//                             dt = softplus(dt_raw + dt_bias[h]);  a = exp(-exp(A_log[h]) * dt)
//                             S  = a * S + dt * B_t x_t^T          (S: [state, head_dim], 32-bit, in the slot)
//                             y_t = S^T C_t + D[h] * x_t
//                           Everything here is 32-bit.
//
// State layout in a slot: conv [K-1][channels] (oldest first); recurrence [heads][head_dim][state], or
// [heads][state][head_dim] where the column-per-thread kernel runs (which kernel runs depends on the layer's
// sizes only, so a layer's state always has one layout).
#include "hybrid.cuh"

namespace {

__global__ void causal_conv_silu_kernel(const float* in, long long ld, const float* __restrict__ taps,
                                        const float* __restrict__ bias, const float* state, long long slot_stride,
                                        const int* slot_ids, const int* tok_req, const int* q_start, float* out,
                                        long long ldo, int n, int C, int K) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n * C) return;
  const int t = (int)(i / C), c = (int)(i - (long long)t * C);
  const int r = tok_req[t];
  const int first = q_start[r];
  const int li = t - first;                               // index within the portion
  const float* st = state + (size_t)slot_ids[r] * slot_stride;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j) {
    const int s = li - (K - 1) + j;
    const float v = s >= 0 ? in[(size_t)(first + s) * ld + c] : st[(size_t)(K - 1 + s) * C + c];
    acc = fmaf(taps[(size_t)c * K + j], v, acc);
  }
  out[(size_t)t * ldo + c] = hy_silu(acc);
}

// one thread per (request, channel): the slot's K-1 rows become the last K-1 inputs seen
__global__ void conv_state_update_kernel(const float* in, long long ld, float* state, long long slot_stride,
                                         const int* slot_ids, const int* q_start, const int* q_len, int R, int C, int K) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)R * C) return;
  const int r = (int)(i / C), c = (int)(i - (long long)r * C);
  const int first = q_start[r], len = q_len[r];
  float* st = state + (size_t)slot_ids[r] * slot_stride;
  for (int j = 0; j < K - 1; ++j) {                        // ascending: row j reads row j + len (> j) or the portion
    const int s = len - (K - 1) + j;
    st[(size_t)j * C + c] = s >= 0 ? in[(size_t)(first + s) * ld + c] : st[(size_t)(K - 1 + s) * C + c];
  }
}

// Block: 4 warps, each with PC columns p of one head; lane l holds S[p][n] for n = l + 32 i, i < NPL.
// The inputs of SCAN_TOKENS tokens at a time are staged in shared memory by the whole block (B and C of
// the head's group, the block's columns of x, the step size and the decay), so that the recurrence
// itself reads nothing from global memory.
constexpr int SCAN_WARPS = 4, SCAN_PC = 2, SCAN_COLS = SCAN_WARPS * SCAN_PC, SCAN_TOKENS = 16;

template <int NPL>
__global__ void ssm_scan_kernel(const float* xbc, long long ld, const float* dt_raw, long long ld_dt,
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                const float* __restrict__ dskip, float* state, long long slot_stride,
                                const int* slot_ids, const int* q_start, const int* q_len, float* y, long long ldy, int H,
                                int P, int N, int G) {
  extern __shared__ float staged[];
  float* sB = staged;                                   // [SCAN_TOKENS][N]  (B, not yet times dt)
  float* sC = sB + SCAN_TOKENS * N;                     // [SCAN_TOKENS][N]
  float* sX = sC + SCAN_TOKENS * N;                     // [SCAN_TOKENS][SCAN_COLS]
  float* sDt = sX + SCAN_TOKENS * SCAN_COLS;            // [SCAN_TOKENS] step size
  float* sDecay = sDt + SCAN_TOKENS;                    // [SCAN_TOKENS]
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pb = blockIdx.z * SCAN_COLS, p0 = pb + warp * SCAN_PC;
  const int g = h / (H / G);
  const int inner = H * P;
  const float bias = dt_bias[h], neg_a = -expf(a_log[h]), dsk = dskip[h];
  const int first = q_start[r], len = q_len[r];
  float* S = state + (size_t)slot_ids[r] * slot_stride + (size_t)h * P * N;
  pdl_wait();
  float s[SCAN_PC][NPL];
#pragma unroll
  for (int c = 0; c < SCAN_PC; ++c)
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = lane + 32 * i;
      s[c][i] = (p0 + c < P && n < N) ? S[(size_t)(p0 + c) * N + n] : 0.f;
    }
  for (int t0 = 0; t0 < len; t0 += SCAN_TOKENS) {
    const int nt = min(SCAN_TOKENS, len - t0);
    __syncthreads();                                    // the chunk before has been used
    // (four loads of B and of C are requested before any is stored: a store to shared memory in between
    // would make every load wait for the one before it)
    for (int i0 = threadIdx.x; i0 < nt * N; i0 += 4 * blockDim.x) {
      float b[4], c[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        b[u] = c[u] = 0.f;
        if (i < nt * N) {
          const int tt = i / N, n = i - tt * N;
          const float* row = xbc + (size_t)(first + t0 + tt) * ld + inner;
          b[u] = row[g * N + n];
          c[u] = row[(G + g) * N + n];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < nt * N) { sB[i] = b[u]; sC[i] = c[u]; }
      }
    }
    for (int i = threadIdx.x; i < nt * SCAN_COLS; i += blockDim.x) {
      const int tt = i / SCAN_COLS, c = i - tt * SCAN_COLS;
      sX[i] = pb + c < P ? xbc[(size_t)(first + t0 + tt) * ld + h * P + pb + c] : 0.f;
    }
    if ((int)threadIdx.x < nt) {
      const float dt = hy_softplus(dt_raw[(size_t)(first + t0 + threadIdx.x) * ld_dt + h] + bias);
      sDt[threadIdx.x] = dt;
      sDecay[threadIdx.x] = expf(neg_a * dt);
    }
    __syncthreads();
    if (p0 >= P) continue;                              // (a warp without columns only helps to stage)
    for (int tt = 0; tt < nt; ++tt) {
      const float dt = sDt[tt], decay = sDecay[tt];
      float bv[NPL], cv[NPL];
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int n = lane + 32 * i;
        bv[i] = n < N ? sB[tt * N + n] * dt : 0.f;
        cv[i] = n < N ? sC[tt * N + n] : 0.f;
      }
#pragma unroll
      for (int c = 0; c < SCAN_PC; ++c) {
        const float xv = sX[tt * SCAN_COLS + warp * SCAN_PC + c];
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          s[c][i] = fmaf(decay, s[c][i], bv[i] * xv);
          part = fmaf(s[c][i], cv[i], part);
        }
        part = warp_sum(part);
        if (lane == 0 && p0 + c < P) y[(size_t)(first + t0 + tt) * ldy + h * P + p0 + c] = part + dsk * xv;
      }
    }
  }
#pragma unroll
  for (int c = 0; c < SCAN_PC; ++c)
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = lane + 32 * i;
      if (p0 + c < P && n < N) S[(size_t)(p0 + c) * N + n] = s[c][i];
    }
}

// The same recurrence with the state in registers and (almost) no exchange between lanes: SPLIT neighbouring
// lanes share a column p of a head, each with 32 of the column's state values (N up to 32 * SPLIT), so a token
// costs a thread 64 multiply-adds and the column log2(SPLIT) shuffles; B_t and C_t are read from shared memory
// four values an instruction.  The inputs of SCOL_TOKENS tokens at a time arrive by asynchronous copies into
// one of two buffers while the tokens of the other are consumed.
constexpr int SCOL_TOKENS = 16, SCOL_THREADS = 64;

__device__ __forceinline__ void scol_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT> __device__ __forceinline__ void scol_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory");
}

template <int SPLIT>
__global__ void ssm_scan_cols_kernel(const float* xbc, long long ld, const float* dt_raw, long long ld_dt,
                                     const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                     const float* __restrict__ dskip, float* state, long long slot_stride,
                                     const int* slot_ids, const int* q_start, const int* q_len, float* y, long long ldy,
                                     int H, int P, int N, int G) {
  constexpr int NR = 32 * SPLIT, COLS = SCOL_THREADS / SPLIT;
  extern __shared__ __align__(16) float scol[];
  constexpr int PER = SCOL_TOKENS * (2 * NR + COLS);      // one buffer: B [T][NR] | C [T][NR] | x [T][COLS]
  float* sRaw = scol + 2 * PER;                            // [2][T] dt before the bias
  float* sDt = sRaw + 2 * SCOL_TOKENS;                     // [T] step size, [T] decay
  float* sDecay = sDt + SCOL_TOKENS;
  pdl_trigger();
  const int col = threadIdx.x / SPLIT, q = threadIdx.x % SPLIT;
  const int r = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * COLS, p = p0 + col;
  const bool active = p < P;
  const int g = h / (H / G);
  const int inner = H * P;
  const float bias = dt_bias[h], neg_a = -expf(a_log[h]), dsk = dskip[h];
  const int first = q_start[r], len = q_len[r];
  // (this kernel keeps a head's state as [state][head_dim], so that neighbouring columns lie side by side)
  float* S = state + (size_t)slot_ids[r] * slot_stride + (size_t)h * P * N + (active ? p : 0);
  if (N < NR)                                              // the padding N .. NR of B and C stays zero
    for (int i = threadIdx.x; i < 2 * PER; i += blockDim.x) scol[i] = 0.f;
  pdl_wait();
  // this thread's state values: n = 4 (q + SPLIT i) + e, i < 8, e < 4
  float s[32];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int n = 4 * (q + SPLIT * i) + e;
      s[4 * i + e] = (active && n < N) ? S[(size_t)n * P] : 0.f;
    }
  __syncthreads();

  const int pieces = N >> 2, xpieces = min(COLS, P - p0) >> 2;
  auto stage = [&](int t0, int b) {
    const int nt = min(SCOL_TOKENS, len - t0);
    float* B = scol + b * PER;
    float* C = B + SCOL_TOKENS * NR;
    float* X = C + SCOL_TOKENS * NR;
    for (int i = threadIdx.x; i < 2 * nt * pieces; i += blockDim.x) {
      const int which = i / (nt * pieces), rem = i - which * nt * pieces;
      const int tt = rem / pieces, c4 = rem - tt * pieces;
      const float* src = xbc + (size_t)(first + t0 + tt) * ld + inner + (which ? G + g : g) * N + 4 * c4;
      gb_cp_async_16((which ? C : B) + tt * NR + 4 * c4, src);
    }
    for (int i = threadIdx.x; i < nt * xpieces; i += blockDim.x) {
      const int tt = i / xpieces, c4 = i - tt * xpieces;
      gb_cp_async_16(X + tt * COLS + 4 * c4, xbc + (size_t)(first + t0 + tt) * ld + h * P + p0 + 4 * c4);
    }
    if ((int)threadIdx.x < nt)
      gb_cp_async_4(sRaw + b * SCOL_TOKENS + threadIdx.x, dt_raw + (size_t)(first + t0 + threadIdx.x) * ld_dt + h);
    scol_commit();
  };

  if (len > 0) stage(0, 0);
  int b = 0;
  for (int t0 = 0; t0 < len; t0 += SCOL_TOKENS, b ^= 1) {
    const int nt = min(SCOL_TOKENS, len - t0);
    if (t0 + SCOL_TOKENS < len) {
      stage(t0 + SCOL_TOKENS, b ^ 1);
      scol_wait<1>();                                      // this chunk has landed, the next is on its way
    } else {
      scol_wait<0>();
    }
    __syncthreads();
    if ((int)threadIdx.x < nt) {
      const float dt = hy_softplus(sRaw[b * SCOL_TOKENS + threadIdx.x] + bias);
      sDt[threadIdx.x] = dt;
      sDecay[threadIdx.x] = expf(neg_a * dt);
    }
    __syncthreads();
    const float* B = scol + b * PER;
    const float* C = B + SCOL_TOKENS * NR;
    const float* X = C + SCOL_TOKENS * NR;
    for (int tt = 0; tt < nt; ++tt) {                      // (every lane, also of a column beyond P: the shuffles below)
      const float decay = sDecay[tt], xv = active ? X[tt * COLS + col] : 0.f, dx = sDt[tt] * xv;
      float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;        // four chains; added in a fixed order
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 b4 = *reinterpret_cast<const float4*>(B + tt * NR + 4 * (q + SPLIT * i));
        const float4 c4 = *reinterpret_cast<const float4*>(C + tt * NR + 4 * (q + SPLIT * i));
        s[4 * i] = fmaf(decay, s[4 * i], b4.x * dx);
        y0 = fmaf(s[4 * i], c4.x, y0);
        s[4 * i + 1] = fmaf(decay, s[4 * i + 1], b4.y * dx);
        y1 = fmaf(s[4 * i + 1], c4.y, y1);
        s[4 * i + 2] = fmaf(decay, s[4 * i + 2], b4.z * dx);
        y2 = fmaf(s[4 * i + 2], c4.z, y2);
        s[4 * i + 3] = fmaf(decay, s[4 * i + 3], b4.w * dx);
        y3 = fmaf(s[4 * i + 3], c4.w, y3);
      }
      float ys = (y0 + y1) + (y2 + y3);
#pragma unroll
      for (int o = 1; o < SPLIT; o <<= 1) ys += __shfl_xor_sync(0xffffffffu, ys, o);
      if (active && q == 0) y[(size_t)(first + t0 + tt) * ldy + h * P + p] = ys + dsk * xv;
    }
    __syncthreads();                                       // before the copies of the chunk after next land here
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = 4 * (q + SPLIT * i) + e;
        if (n < N) S[(size_t)n * P] = s[4 * i + e];
      }
  }
}

}  // namespace

// a0 in (f32; the convolved columns of a wider row), a1 its row stride, a2 taps [C, K], a3 bias [C] or 0, a4 conv
// state of slot 0, a5 elements between slots, a6 slot ids, a7 token -> request, a8 first row per request, a9 rows per
// request, a10 out (f32), a11 its row stride, a12 tokens, a13 channels, a14 taps per channel, a15 requests
GB_OP(gb_op_causal_conv_silu) {
  const int n = (int)a[12], C = (int)a[13], K = (int)a[14], R = (int)a[15];
  if (n <= 0) return 0;
  if (K < 1) GB_FAIL(GB_ERR_ARG, "causal_conv_silu: %d taps", K);
  gb_launch(causal_conv_silu_kernel, dim3(gb_div_up((long long)n * C, 256)), dim3(256), 0, ctx->stream,
            op_ptr<const float>(a[0]), a[1], op_ptr<const float>(a[2]), op_ptr<const float>(a[3]), op_ptr<const float>(a[4]),
            a[5], op_ptr<const int>(a[6]), op_ptr<const int>(a[7]), op_ptr<const int>(a[8]), op_ptr<float>(a[10]), a[11], n,
            C, K);
  GB_CHECK_LAUNCH("causal_conv_silu");
  if (K == 1) return 1;
  gb_launch(conv_state_update_kernel, dim3(gb_div_up((long long)R * C, 256)), dim3(256), 0, ctx->stream,
            op_ptr<const float>(a[0]), a[1], op_ptr<float>(a[4]), a[5], op_ptr<const int>(a[6]), op_ptr<const int>(a[8]),
            op_ptr<const int>(a[9]), R, C, K);
  GB_CHECK_LAUNCH("conv_state_update");
  return 2;
}

// a0 rows [x | B | C] after the convolution (f32), a1 their stride, a2 dt before the bias (f32; a column of a wider
// row), a3 its row stride, a4 dt_bias [H], a5 A_log [H], a6 D [H], a7 recurrent state of slot 0, a8 elements between
// slots, a9 slot ids, a10 first row per request, a11 rows per request, a12 y (f32), a13 its row stride, a14 requests,
// a15 heads, a16 head_dim, a17 state size, a18 groups
GB_OP(gb_op_ssm_scan) {
  const int R = (int)a[14], H = (int)a[15], P = (int)a[16], N = (int)a[17], G = (int)a[18];
  if (R <= 0) return 0;
  if (G <= 0 || H % G) GB_FAIL(GB_ERR_ARG, "ssm_scan: %d heads in %d groups", H, G);
  if (N > 256) GB_FAIL(GB_ERR_ARG, "ssm_scan: state size %d (at most 256)", N);
  // states of up to 128 values whose rows can be copied in 16-byte pieces: state in registers, 32 values a thread
  if (N <= 128 && N % 4 == 0 && P % 4 == 0 && a[1] % 4 == 0 && (a[0] & 15) == 0) {
    const int split = N <= 32 ? 1 : (N <= 64 ? 2 : 4);
    const int cols = SCOL_THREADS / split;
    const size_t smem_cols = sizeof(float) * (2 * (size_t)SCOL_TOKENS * (2 * 32 * split + cols) + 4 * SCOL_TOKENS);
    const dim3 grid_cols(R, H, gb_div_up(P, cols));
#define SCOL_LAUNCH(SP)                                                                                               \
    gb_launch(ssm_scan_cols_kernel<SP>, grid_cols, dim3(SCOL_THREADS), smem_cols, ctx->stream, op_ptr<const float>(a[0]), \
              a[1], op_ptr<const float>(a[2]), a[3], op_ptr<const float>(a[4]), op_ptr<const float>(a[5]),              \
              op_ptr<const float>(a[6]), op_ptr<float>(a[7]), a[8], op_ptr<const int>(a[9]), op_ptr<const int>(a[10]),   \
              op_ptr<const int>(a[11]), op_ptr<float>(a[12]), a[13], H, P, N, G)
    if (split == 1) SCOL_LAUNCH(1); else if (split == 2) SCOL_LAUNCH(2); else SCOL_LAUNCH(4);
#undef SCOL_LAUNCH
    GB_CHECK_LAUNCH("ssm_scan (columns)");
    return 1;
  }
  const dim3 grid(R, H, gb_div_up(P, SCAN_COLS)), block(32 * SCAN_WARPS);
  const size_t smem = sizeof(float) * (size_t)SCAN_TOKENS * (2 * N + SCAN_COLS + 2);      // at most 34 KB
#define SCAN_LAUNCH(NPL)                                                                                              \
  gb_launch(ssm_scan_kernel<NPL>, grid, block, smem, ctx->stream, op_ptr<const float>(a[0]), a[1], op_ptr<const float>(a[2]), \
            a[3], op_ptr<const float>(a[4]), op_ptr<const float>(a[5]), op_ptr<const float>(a[6]), op_ptr<float>(a[7]),   \
            a[8], op_ptr<const int>(a[9]), op_ptr<const int>(a[10]), op_ptr<const int>(a[11]), op_ptr<float>(a[12]),    \
            a[13], H, P, N, G)
  if (N <= 32) SCAN_LAUNCH(1);
  else if (N <= 64) SCAN_LAUNCH(2);
  else if (N <= 128) SCAN_LAUNCH(4);
  else SCAN_LAUNCH(8);
#undef SCAN_LAUNCH
  GB_CHECK_LAUNCH("ssm_scan");
  return 1;
}
