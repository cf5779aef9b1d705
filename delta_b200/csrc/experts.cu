// A mixture of small feed-forward experts, and the gated activation its experts and dense layers share.
//
//   glu_clamped     y = g' * sigmoid(alpha (g' + cubic g'^3)) * (u' + shift),  g' = min(g, limit), u' = clamp(u, -limit, limit)
//                   from rows [g (F) | u (F)] (limit < 0: nothing is clamped);
//   router          per token the router's logits z = W x in 32 bit, the `top` largest of the E experts' logits (the lowest
//                   index among equals) and the softmax over the chosen logits only (router_topk: the choice alone, from
//                   logits that are there already);
//   experts_align   sorts the (token, choice) slots by expert into tiles of `tile_m` rows that each belong to one expert
//                   (every expert's rows padded to whole tiles with -1), so that the products run as one launch and
//                   nothing about the routing is read on the host;
//   experts_gemm    for every tile the product of its rows with its expert's matrix.  First product: rows are gathered
//                   from the tokens, the matrix is [gate (F) | up (F)] x d, and the gated activation is applied before
//                   the result is stored at the row's place in the sorted order (row_scale: the product of a slot is multiplied by
//                   the slot's weight first, which is what an expert that reads weight * x gets).  Second product: rows are read in the
//                   sorted order and the result goes to the slot's own place, in 32 bit;
//   experts_combine out[t] = sum_j weight[t][j] * z[t*top + j]  (+ sigmoid(gate logit of t) * shared[t]), summed in 32 bit in
//                   the order of the choices, so the result does not depend on what else is in the batch.
//
// The products run on the tensor cores for bfloat16 (warp-level MMA, 32-bit accumulation) and on the FMA units in 32 bit
// (and for bfloat16 rows whose length is no multiple of 8).
#include "common.cuh"
#include "mma_helpers.cuh"

namespace {
constexpr int TILE_M = 64;
constexpr int TILE_N = 64;
constexpr int TILE_K = 16;
constexpr int GEMM_THREADS = 256;
constexpr int MAX_TOP = 32;
constexpr int MAX_EXPERTS = 1024;

__device__ __forceinline__ float glu_value(float g, float u, float limit, float alpha, float shift, float cubic = 0.f) {
  return dk_glu_value(g, u, limit, alpha, shift, cubic);
}

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ y, long long rows, int F, float limit, float alpha, float shift,
                                   float cubic) {
  const long long n = rows * F;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / F;
    const int i = (int)(idx - r * F);
    const T* row = gu + r * 2 * F;
    y[idx] = from_f32<T>(glu_value(to_f32<T>(row[i]), to_f32<T>(row[F + i]), limit, alpha, shift, cubic));
  }
}

// The same for F a multiple of 8 and 16-byte aligned rows: eight entries a thread, 16-byte accesses.
template <typename T>
__global__ void glu_clamped_vec_kernel(const T* __restrict__ gu, T* __restrict__ y, long long rows, int F, float limit, float alpha, float shift,
                                       float cubic) {
  const int per_row = F / 8;
  const long long n = rows * per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / per_row;
    const int i = (int)(idx - r * per_row) * 8;
    float g[8], u[8], o[8];
    load8<T>(gu + r * 2 * F + i, g);
    load8<T>(gu + r * 2 * F + F + i, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = glu_value(g[e], u[e], limit, alpha, shift, cubic);
    store8<T>(y + r * F + i, o);
  }
}

// The `top` largest of z[0..E) (the lowest index among equals) and the softmax over them, by one warp.  z is the warp's own
// copy (shared memory) and is used up: a chosen entry is set to -inf.
__device__ void pick_top(float* z, int E, int top, int* __restrict__ choice, float* __restrict__ weight, int lane) {
  float largest = 0.f, sum = 0.f, my_weight = 0.f;
  int my_choice = -1;
  for (int j = 0; j < top; ++j) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > bv) {
        bv = v;
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    if (j == 0) largest = bv;
    const float ex = expf(bv - largest);
    sum += ex;
    if (lane == j) {
      my_weight = ex;
      my_choice = be < E ? be : -1;
    }
    if (lane == 0 && be < E) z[be] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    choice[lane] = my_choice;
    weight[lane] = my_weight / sum;
  }
}

// The choice by sigmoid scores: `pick` [E] holds score + correction and is used up, `score` [E] the scores s = sigmoid(z).  The
// `top` largest of pick are chosen (the lowest index among equals); a chosen expert's weight is its score without the
// correction, divided by the sum of the chosen scores (+ 1e-20) when `normalize`, times `scale`.
__device__ void pick_top_scored(float* pick, const float* score, int E, int top, float scale, int normalize, int* __restrict__ choice,
                                float* __restrict__ weight, int lane) {
  float sum = 0.f, my_weight = 0.f;
  int my_choice = -1;
  for (int j = 0; j < top; ++j) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = pick[e];
      if (v > bv) {
        bv = v;
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    const float sc = be < E ? score[be] : 0.f;
    sum += sc;
    if (lane == j) {
      my_weight = sc;
      my_choice = be < E ? be : -1;
    }
    __syncwarp();
    if (lane == 0 && be < E) pick[be] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    choice[lane] = my_choice;
    weight[lane] = (normalize ? my_weight / (sum + 1e-20f) : my_weight) * scale;
  }
}

constexpr int ROUTER_WARPS = 8;

// One warp per token; the logits are copied to the warp's shared memory first.
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_topk_kernel(const float* __restrict__ logits, int ld, int* __restrict__ choice, float* __restrict__ weight, int T_, int E, int top) {
  extern __shared__ float zs[];      // [warps][E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTER_WARPS + warp;
  if (t >= T_) return;
  float* z = zs + (size_t)warp * E;
  for (int e = lane; e < E; e += 32) z[e] = logits[(size_t)t * ld + e];
  __syncwarp();
  pick_top(z, E, top, choice + (size_t)t * top, weight + (size_t)t * top, lane);
}

// The router's product and its choice in one kernel: the n_rows logits z = W x of a token in 32 bit (the first E are the
// experts'; further rows, such as a gate's, are only stored), then the choice.  A block takes `tpb` tokens (1, 2, 4 or 8); the
// 8 / tpb warps of a token share its rows in groups of ROUTER_ROWS, so that a step of few tokens still has many loads under way.
constexpr int ROUTER_ROWS = 8;      // rows of the matrix whose products a warp has under way at a time

template <typename T, bool VEC>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_kernel(const T* __restrict__ x, const T* __restrict__ w, float* __restrict__ logits, int* __restrict__ choice,
              float* __restrict__ weight, int T_, int d, int n_rows, int E, int top, int tpb, const float* __restrict__ correction,
              float route_scale, int scored) {
  extern __shared__ float zs[];      // [tpb][n_rows] (scored: and [tpb][E] behind them)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int local = warp % tpb, share = warp / tpb, sharers = ROUTER_WARPS / tpb;
  const int t = blockIdx.x * tpb + local;
  const bool live = t < T_;
  float* z = zs + (size_t)local * n_rows;
  const T* xr = x + (size_t)(live ? t : 0) * d;
  for (int r0 = share * ROUTER_ROWS; live && r0 < n_rows; r0 += sharers * ROUTER_ROWS) {
    float acc[ROUTER_ROWS];
#pragma unroll
    for (int q = 0; q < ROUTER_ROWS; ++q) acc[q] = 0.f;
    if (VEC) {      // d is a multiple of 8 and the rows are 16-byte aligned: eight entries a load
#pragma unroll 2
      for (int c = lane * 8; c < d; c += 256) {
        float xv[8];
        load8<T>(xr + c, xv);
#pragma unroll
        for (int q = 0; q < ROUTER_ROWS; ++q) {
          if (r0 + q < n_rows) {
            float wv[8];
            load8<T>(w + (size_t)(r0 + q) * d + c, wv);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[q] = fmaf(xv[i], wv[i], acc[q]);
          }
        }
      }
    } else {
      for (int i = lane; i < d; i += 32) {
        const float xv = to_f32<T>(xr[i]);
#pragma unroll
        for (int q = 0; q < ROUTER_ROWS; ++q)
          if (r0 + q < n_rows) acc[q] = fmaf(xv, to_f32<T>(w[(size_t)(r0 + q) * d + i]), acc[q]);
      }
    }
#pragma unroll
    for (int q = 0; q < ROUTER_ROWS; ++q) {
      const float v = warp_sum(acc[q]);
      if (lane == 0 && r0 + q < n_rows) {
        z[r0 + q] = v;
        logits[(size_t)t * n_rows + r0 + q] = v;
      }
    }
  }
  __syncthreads();
  if (!live || share != 0) return;
  if (scored) {      // sigmoid scores; the correction joins the choice only
    float* score = zs + (size_t)tpb * n_rows + (size_t)local * E;
    for (int e = lane; e < E; e += 32) {
      const float sc = 1.f / (1.f + expf(-z[e]));
      score[e] = sc;
      // without a correction the logits themselves are compared: the same order, and no ties where the sigmoid saturates
      if (correction != nullptr) z[e] = sc + correction[e];
    }
    __syncwarp();
    pick_top_scored(z, score, E, top, route_scale, scored == 1, choice + (size_t)t * top, weight + (size_t)t * top, lane);
  } else {
    pick_top(z, E, top, choice + (size_t)t * top, weight + (size_t)t * top, lane);
  }
}

// One block.  sorted[p] = slot (token * top + choice) or -1; tile_expert[tile] = expert or -1.
__global__ void experts_align_kernel(const int* __restrict__ choice, int n_slots, int E, int* __restrict__ sorted, int capacity,
                                     int* __restrict__ tile_expert, int max_tiles, int tile_m) {
  __shared__ int count[MAX_EXPERTS], start[MAX_EXPERTS];
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x) {
    const int e = choice[s];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  for (int p = threadIdx.x; p < capacity; p += blockDim.x) sorted[p] = -1;
  for (int q = threadIdx.x; q < max_tiles; q += blockDim.x) tile_expert[q] = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      const int tiles = (count[e] + tile_m - 1) / tile_m;
      for (int q = 0; q < tiles; ++q) tile_expert[at / tile_m + q] = e;
      at += tiles * tile_m;
      count[e] = 0;
    }
  }
  __syncthreads();
  // the order of an expert's rows is whatever the atomics give: every row is computed alone, so it changes no value
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x) {
    const int e = choice[s];
    if (e < 0 || e >= E) continue;
    sorted[start[e] + atomicAdd(&count[e], 1)] = s;
  }
}

// MODE 1 (gated): A = tokens [*, K] gathered by sorted[p] / top, W = [E][2N][K] (gate rows, then up rows), out Y[p][N] of type T.
// MODE 2 (one branch): the same gather, W = [E][N][K], out Y[p][N] = relu(product)^2 of type T.
// MODE 0: A = Y [capacity, K] in sorted order, W = [E][N][K], out Z[slot][N] in float.
__device__ __forceinline__ float relu_squared(float x) { return x > 0.f ? x * x : 0.f; }

template <typename T, int MODE>
__global__ void __launch_bounds__(GEMM_THREADS)
experts_gemm_kernel(const T* __restrict__ A, const T* __restrict__ W, void* __restrict__ out, const int* __restrict__ sorted,
                    const int* __restrict__ tile_expert, int top, int N, int K, float limit, float alpha, float shift,
                    const float* __restrict__ row_scale) {
  constexpr bool ACT = MODE == 1, FIRST = MODE != 0;
  const int tile = blockIdx.y;
  const int e = tile_expert[tile];
  if (e < 0) return;
  const int n0 = blockIdx.x * TILE_N, p0 = tile * TILE_M;
  __shared__ float As[TILE_M][TILE_K + 1];
  __shared__ float Ws[ACT ? 2 : 1][TILE_N][TILE_K + 1];
  __shared__ int src_row[TILE_M];
  const int tid = threadIdx.x;
  if (tid < TILE_M) {
    const int s = sorted[p0 + tid];
    src_row[tid] = s < 0 ? -1 : (FIRST ? s / top : p0 + tid);
  }
  __syncthreads();
  const T* We = W + (size_t)e * (ACT ? 2 : 1) * N * K;
  const int ty = tid / 16, tx = tid % 16;      // rows 4*ty .. 4*ty+3; columns tx + 16*c
  float acc[ACT ? 2 : 1][4][4];
#pragma unroll
  for (int a = 0; a < (ACT ? 2 : 1); ++a)
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][r][c] = 0.f;
  for (int k0 = 0; k0 < K; k0 += TILE_K) {
    for (int idx = tid; idx < TILE_M * TILE_K; idx += GEMM_THREADS) {
      const int r = idx / TILE_K, k = idx - r * TILE_K;
      const int row = src_row[r];
      As[r][k] = (row >= 0 && k0 + k < K) ? to_f32<T>(A[(size_t)row * K + k0 + k]) : 0.f;
    }
    for (int idx = tid; idx < TILE_N * TILE_K; idx += GEMM_THREADS) {
      const int c = idx / TILE_K, k = idx - c * TILE_K;
      const bool ok = n0 + c < N && k0 + k < K;
      Ws[0][c][k] = ok ? to_f32<T>(We[(size_t)(n0 + c) * K + k0 + k]) : 0.f;
      if (ACT) Ws[ACT ? 1 : 0][c][k] = ok ? to_f32<T>(We[(size_t)(N + n0 + c) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TILE_K; ++k) {
      float a[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) a[r] = As[4 * ty + r][k];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float w0 = Ws[0][tx + 16 * c][k];
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[0][r][c] = fmaf(a[r], w0, acc[0][r][c]);
        if (ACT) {
          const float w1 = Ws[ACT ? 1 : 0][tx + 16 * c][k];
#pragma unroll
          for (int r = 0; r < 4; ++r) acc[ACT ? 1 : 0][r][c] = fmaf(a[r], w1, acc[ACT ? 1 : 0][r][c]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int lr = 4 * ty + r;
    const int s = sorted[p0 + lr];
    if (s < 0) continue;
    const float rs = (FIRST && row_scale != nullptr) ? row_scale[s] : 1.f;      // (w x) W^T = w (x W^T)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = n0 + tx + 16 * c;
      if (n >= N) continue;
      if (ACT) {
        // the two products are rounded to the element type before the activation, as separate products would be
        const float g = to_f32<T>(from_f32<T>(acc[0][r][c] * rs)), u = to_f32<T>(from_f32<T>(acc[ACT ? 1 : 0][r][c] * rs));
        ((T*)out)[(size_t)(p0 + lr) * N + n] = from_f32<T>(glu_value(g, u, limit, alpha, shift));
      } else if (FIRST) {
        ((T*)out)[(size_t)(p0 + lr) * N + n] = from_f32<T>(relu_squared(to_f32<T>(from_f32<T>(acc[0][r][c] * rs))));
      } else {
        ((float*)out)[(size_t)s * N + n] = acc[0][r][c];
      }
    }
  }
}

// The same products on the tensor cores (warp-level MMA, bfloat16 operands, 32-bit accumulation) for K a multiple of 8:
// a block of 8 warps takes TILE_M rows x 128 columns, K in steps of 32 through a ring of cp.async stages.  With ACT the 128
// columns are 64 gate columns and the 64 up columns that belong to them, laid out so that a thread holds both values of an
// entry and applies the gated activation in registers.
constexpr int MMA_BN = 128;
constexpr int MMA_BK = 32;
constexpr int MMA_LD = MMA_BK + 8;      // padded row: ldmatrix reads eight rows without a bank conflict
constexpr int MMA_STAGES = 4;
constexpr int MMA_SMEM = MMA_STAGES * (TILE_M + MMA_BN) * MMA_LD * 2;

template <int MODE>
__global__ void __launch_bounds__(256)
experts_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W, void* __restrict__ out,
                        const int* __restrict__ sorted, const int* __restrict__ tile_expert, int top, int N, int K, float limit,
                        float alpha, float shift, const float* __restrict__ row_scale) {
  constexpr bool ACT = MODE == 1, FIRST = MODE != 0;
  const int tile = blockIdx.y;
  const int e = tile_expert[tile];
  if (e < 0) return;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* As = (__nv_bfloat16*)smem_raw;                              // [STAGES][TILE_M][LD]
  __nv_bfloat16* Bs = As + MMA_STAGES * TILE_M * MMA_LD;                     // [STAGES][BN][LD]
  __shared__ int src_row[TILE_M];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 2, wn = warp & 3;                                   // 2 x 4 warps: 32 rows x 32 columns each
  const int cols = ACT ? MMA_BN / 2 : MMA_BN;                                // output columns of the block
  const int n0 = blockIdx.x * cols, p0 = tile * TILE_M;
  if (tid < TILE_M) {
    const int s = sorted[p0 + tid];
    src_row[tid] = s < 0 ? -1 : (FIRST ? s / top : p0 + tid);
  }
  __syncthreads();
  const __nv_bfloat16* We = W + (size_t)e * (ACT ? 2 : 1) * N * K;
  // what this thread fetches in every stage: one 16-byte piece of A, two of B
  const int a_r = tid >> 2, a_c = (tid & 3) * 8;
  const int a_src = src_row[a_r];
  const __nv_bfloat16* a_ptr = A + (size_t)(a_src < 0 ? 0 : a_src) * K + a_c;
  const __nv_bfloat16* b_ptr[2];
  bool b_ok[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = (tid >> 2) + 64 * i;                                       // row of the B tile
    int n;                                                                   // row of the expert's matrix
    if (ACT) n = r < 64 ? n0 + r : N + n0 + (r - 64);
    else n = n0 + r;
    b_ok[i] = ACT ? (n0 + (r & 63) < N) : (n < N);
    b_ptr[i] = We + (size_t)(b_ok[i] ? n : 0) * K + a_c;
  }
  const int ksteps = (K + MMA_BK - 1) / MMA_BK;
  auto fetch = [&](int ks) {
    const int st = ks % MMA_STAGES, k0 = ks * MMA_BK;
    const bool kin = k0 + a_c < K;
    cp_async_16(smem_u32(As + ((size_t)st * TILE_M + a_r) * MMA_LD + a_c), kin ? a_ptr + k0 : A, kin && a_src >= 0);
#pragma unroll
    for (int i = 0; i < 2; ++i)
      cp_async_16(smem_u32(Bs + ((size_t)st * MMA_BN + (tid >> 2) + 64 * i) * MMA_LD + a_c), kin ? b_ptr[i] + k0 : W, kin && b_ok[i]);
  };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.f;
#pragma unroll
  for (int s = 0; s < MMA_STAGES - 1; ++s) {
    if (s < ksteps) fetch(s);
    cp_async_commit();
  }
  // n-tiles of this warp in the B tile: ACT: two of the gate half and the two up tiles that belong to them
  int bn[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) bn[j] = ACT ? ((j >> 1) * 64 + wn * 16 + (j & 1) * 8) : (wn * 32 + j * 8);
  for (int ks = 0; ks < ksteps; ++ks) {
    cp_async_wait<MMA_STAGES - 2>();
    __syncthreads();
    if (ks + MMA_STAGES - 1 < ksteps) fetch(ks + MMA_STAGES - 1);
    cp_async_commit();
    const int st = ks % MMA_STAGES;
    const __nv_bfloat16* as = As + (size_t)st * TILE_M * MMA_LD;
    const __nv_bfloat16* bs = Bs + (size_t)st * MMA_BN * MMA_LD;
#pragma unroll
    for (int kk = 0; kk < MMA_BK; kk += 16) {
      uint32_t a[2][4], b[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        ldmatrix_x4(a[i][0], a[i][1], a[i][2], a[i][3],
                    smem_u32(as + (size_t)(wm * 32 + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * MMA_LD + kk + (lane >> 4) * 8));
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        // two n-tiles that lie 8 rows apart in the B tile: (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
        ldmatrix_x4(b[j][0], b[j][1], b[j + 1][0], b[j + 1][1],
                    smem_u32(bs + (size_t)(bn[j] + (lane & 7) + (lane >> 4) * 8) * MMA_LD + kk + ((lane >> 3) & 1) * 8));
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], a[i], b[j][0], b[j][1]);
    }
  }
  cp_async_wait<0>();
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int lr = wm * 32 + i * 16 + g + half * 8;
      const int s = sorted[p0 + lr];
      if (s < 0) continue;
      const float rs = (FIRST && row_scale != nullptr) ? row_scale[s] : 1.f;      // (w x) W^T = w (x W^T)
      if (ACT) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = n0 + wn * 16 + j * 8 + 2 * t4;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            if (n + q >= N) continue;
            const float gv = __bfloat162float(__float2bfloat16_rn(acc[i][j][half * 2 + q] * rs));
            const float uv = __bfloat162float(__float2bfloat16_rn(acc[i][j + 2][half * 2 + q] * rs));
            ((__nv_bfloat16*)out)[(size_t)(p0 + lr) * N + n + q] = __float2bfloat16_rn(glu_value(gv, uv, limit, alpha, shift));
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + wn * 32 + j * 8 + 2 * t4;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            if (n + q >= N) continue;
            if (FIRST)      // the product rounded to bfloat16 first, as a separate product would be
              ((__nv_bfloat16*)out)[(size_t)(p0 + lr) * N + n + q] =
                  __float2bfloat16_rn(relu_squared(__bfloat162float(__float2bfloat16_rn(acc[i][j][half * 2 + q] * rs))));
            else
              ((float*)out)[(size_t)s * N + n + q] = acc[i][j][half * 2 + q];
          }
        }
      }
    }
}

// rows[p] = x[sorted[p] / top] (zeros where sorted[p] < 0): the tokens in the sorted order, for products that want their rows
// side by side (csrc/gemm_tc.cu).  K is a multiple of 8.
// row_scale (or null): rows[p] = row_scale[sorted[p]] * x[sorted[p] / top], rounded once: a choice's weight multiplies what its
// expert reads.
__global__ void experts_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted, int top,
                                      __nv_bfloat16* __restrict__ rows, int K, const float* __restrict__ row_scale) {
  const int p = blockIdx.x;
  const int s = sorted[p];
  const uint4* src = s < 0 ? nullptr : reinterpret_cast<const uint4*>(x + (size_t)(s / top) * K);
  uint4* dst = reinterpret_cast<uint4*>(rows + (size_t)p * K);
  if (src == nullptr || row_scale == nullptr) {
    for (int c = threadIdx.x; c < K / 8; c += blockDim.x) dst[c] = src ? src[c] : make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const float w = row_scale[s];
  for (int c = threadIdx.x; c < K / 8; c += blockDim.x) {
    float v[8];
    load8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(src + c), v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= w;
    store8<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(dst + c), v);
  }
}

template <typename T>
__global__ void experts_combine_kernel(const float* __restrict__ z, const float* __restrict__ weight, int top, const T* __restrict__ shared,
                                       const float* __restrict__ gate_logit, int gate_stride, T* __restrict__ out, int d) {
  const int t = blockIdx.x;
  float gate = 0.f;
  if (shared != nullptr) gate = gate_logit != nullptr ? 1.f / (1.f + expf(-gate_logit[(size_t)t * gate_stride])) : 1.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < top; ++j) a = fmaf(weight != nullptr ? weight[(size_t)t * top + j] : 1.f, z[((size_t)t * top + j) * d + i], a);
    if (shared != nullptr) a = fmaf(gate, to_f32<T>(shared[(size_t)t * d + i]), a);
    out[(size_t)t * d + i] = from_f32<T>(a);
  }
}
}  // namespace

extern "C" int dk_experts_tile_rows() { return TILE_M; }

extern "C" int dk_glu_clamped(const void* gu, void* y, long long rows, int F, float limit, float alpha, float shift, float cubic, int dtype,
                              cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && F > 0, "glu_clamped: bad sizes rows=%lld F=%d", rows, F);
  const bool vec = F % 8 == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)y % 16) == 0;
  const long long n = vec ? rows * (F / 8) : rows * F;
  long long blocks = (n + 255) / 256;
  const long long most = (long long)dk_sm_count() * 16;
  if (blocks > most) blocks = most;
#define LAUNCH(T)                                                                                                              \
  do {                                                                                                                         \
    if (vec) glu_clamped_vec_kernel<T><<<(int)blocks, 256, 0, stream>>>((const T*)gu, (T*)y, rows, F, limit, alpha, shift, cubic); \
    else glu_clamped_kernel<T><<<(int)blocks, 256, 0, stream>>>((const T*)gu, (T*)y, rows, F, limit, alpha, shift, cubic);       \
  } while (0)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "glu_clamped: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("glu_clamped");
}

extern "C" int dk_router_topk(const float* logits, int ld, int* choice, float* weight, int T_, int E, int top, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && E > 0 && top > 0 && top <= E && ld >= E, "router_topk: bad sizes T=%d E=%d top=%d ld=%d", T_, E, top, ld);
  DK_REQUIRE(top <= MAX_TOP, "router_topk: %d choices a token are above the %d this kernel takes", top, MAX_TOP);
  const size_t smem = (size_t)ROUTER_WARPS * E * sizeof(float);
  DK_REQUIRE(smem <= 48 * 1024, "router_topk: %d logits a token do not fit the shared memory", E);
  router_topk_kernel<<<(T_ + ROUTER_WARPS - 1) / ROUTER_WARPS, ROUTER_WARPS * 32, smem, stream>>>(logits, ld, choice, weight, T_, E, top);
  return dk_check_launch("router_topk");
}

// scored == 0: the softmax over the chosen logits.  scored == 1: sigmoid scores, `correction` [E] (or null) added for the choice
// only, weights = chosen scores / their sum * route_scale.  scored == 2: the same with weights = chosen scores * route_scale.
extern "C" int dk_router(const void* x, const void* w, float* logits, int* choice, float* weight, int T_, int d, int n_rows, int E, int top,
                         const float* correction, float route_scale, int scored, int dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && d > 0 && E > 0 && top > 0 && top <= E && n_rows >= E, "router: bad sizes T=%d d=%d E=%d top=%d rows=%d", T_, d, E, top, n_rows);
  DK_REQUIRE(top <= MAX_TOP, "router: %d choices a token are above the %d this kernel takes", top, MAX_TOP);
  // few tokens: one token a block, its rows shared by the block's warps; many: eight tokens a block
  const int groups = (n_rows + ROUTER_ROWS - 1) / ROUTER_ROWS;
  int tpb = ROUTER_WARPS;
  while (tpb > 1 && (ROUTER_WARPS / tpb < groups) && (long long)T_ * (ROUTER_WARPS / tpb) < 16LL * dk_sm_count()) tpb /= 2;
  const size_t smem = (size_t)tpb * (n_rows + (scored ? E : 0)) * sizeof(float);
  DK_REQUIRE(smem <= 48 * 1024, "router: %d logits a token do not fit the shared memory", n_rows);
  const int blocks = (T_ + tpb - 1) / tpb;
  const bool vec = d % 8 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0;
#define LAUNCH(T, V) router_kernel<T, V><<<blocks, ROUTER_WARPS * 32, smem, stream>>>((const T*)x, (const T*)w, logits, choice, weight, T_, d, n_rows, E, top, tpb, correction, route_scale, scored)
  if (dtype == DK_F32) {
    if (vec) LAUNCH(float, true);
    else LAUNCH(float, false);
  } else if (dtype == DK_BF16) {
    if (vec) LAUNCH(__nv_bfloat16, true);
    else LAUNCH(__nv_bfloat16, false);
  }
#undef LAUNCH
  else DK_REQUIRE(false, "router: unknown dtype %d", dtype);
  return dk_check_launch("router");
}

extern "C" int dk_experts_align(const int* choice, int n_slots, int E, int* sorted, int capacity, int* tile_expert, int max_tiles,
                                int tile_m, cudaStream_t stream) {
  if (n_slots == 0) return 0;
  DK_REQUIRE(n_slots > 0 && E > 0 && E <= MAX_EXPERTS, "experts_align: bad sizes slots=%d E=%d (at most %d experts)", n_slots, E, MAX_EXPERTS);
  DK_REQUIRE(tile_m > 0 && capacity % tile_m == 0 && max_tiles * tile_m == capacity && capacity >= n_slots + (tile_m - 1) * (E < n_slots ? E : n_slots),
             "experts_align: %d rows in %d tiles do not hold %d slots of %d experts", capacity, max_tiles, n_slots, E);
  experts_align_kernel<<<1, 1024, 0, stream>>>(choice, n_slots, E, sorted, capacity, tile_expert, max_tiles, tile_m);
  return dk_check_launch("experts_align");
}

// row_scale (float [slots] or null): in a first product (act != 0) the row of slot s is multiplied by row_scale[s] before the
// activation, as if the expert had read row_scale[s] * x.
extern "C" int dk_experts_gemm(const void* A, const void* W, void* out, const int* sorted, const int* tile_expert, int max_tiles, int top,
                               int N, int K, int act, float limit, float alpha, float shift, const float* row_scale, int dtype,
                               cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  DK_REQUIRE(max_tiles > 0 && N > 0 && K > 0 && top > 0, "experts_gemm: bad sizes tiles=%d N=%d K=%d top=%d", max_tiles, N, K, top);
  DK_REQUIRE(act >= 0 && act <= 2, "experts_gemm: activation %d is not known (0 none, 1 gated, 2 relu squared)", act);
  DK_REQUIRE(max_tiles <= 65535, "experts_gemm: %d tiles are above the grid's limit", max_tiles);
  if (dtype == DK_BF16 && K % 8 == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0) {
    const int cols = act == 1 ? MMA_BN / 2 : MMA_BN;
    const dim3 mgrid((N + cols - 1) / cols, max_tiles);
    static bool granted[DK_MAX_DEVICES] = {false};
    const int dev = dk_current_device();
    if (!granted[dev]) {
      if (cudaFuncSetAttribute(experts_gemm_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM) != cudaSuccess ||
          cudaFuncSetAttribute(experts_gemm_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM) != cudaSuccess ||
          cudaFuncSetAttribute(experts_gemm_mma_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM) != cudaSuccess) {
        cudaGetLastError();
        DK_REQUIRE(false, "experts_gemm: %d bytes of shared memory were not granted", MMA_SMEM);
      }
      granted[dev] = true;
    }
#define MMA_LAUNCH(MODE)                                                                                                          \
  experts_gemm_mma_kernel<MODE><<<mgrid, 256, MMA_SMEM, stream>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)W, out, sorted, tile_expert, \
                                                                  top, N, K, limit, alpha, shift, row_scale)
    if (act == 1) MMA_LAUNCH(1);
    else if (act == 2) MMA_LAUNCH(2);
    else MMA_LAUNCH(0);
#undef MMA_LAUNCH
    return dk_check_launch("experts_gemm");
  }
  const dim3 grid((N + TILE_N - 1) / TILE_N, max_tiles);
#define LAUNCH(T)                                                                                                                  \
  do {                                                                                                                             \
    if (act == 1) experts_gemm_kernel<T, 1><<<grid, GEMM_THREADS, 0, stream>>>((const T*)A, (const T*)W, out, sorted, tile_expert, top, N, K, limit, alpha, shift, row_scale); \
    else if (act == 2) experts_gemm_kernel<T, 2><<<grid, GEMM_THREADS, 0, stream>>>((const T*)A, (const T*)W, out, sorted, tile_expert, top, N, K, limit, alpha, shift, row_scale); \
    else experts_gemm_kernel<T, 0><<<grid, GEMM_THREADS, 0, stream>>>((const T*)A, (const T*)W, out, sorted, tile_expert, top, N, K, limit, alpha, shift, row_scale);    \
  } while (0)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "experts_gemm: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("experts_gemm");
}

extern "C" int dk_experts_gather(const void* x, const int* sorted, int top, void* rows, int capacity, int K, const float* row_scale,
                                 cudaStream_t stream) {
  if (capacity == 0) return 0;
  DK_REQUIRE(capacity > 0 && K > 0 && K % 8 == 0 && top > 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)rows % 16) == 0,
             "experts_gather: bad arguments capacity=%d K=%d top=%d", capacity, K, top);
  experts_gather_kernel<<<capacity, K >= 2048 ? 256 : 128, 0, stream>>>((const __nv_bfloat16*)x, sorted, top, (__nv_bfloat16*)rows, K, row_scale);
  return dk_check_launch("experts_gather");
}

extern "C" int dk_experts_combine(const float* z, const float* weight, int top, const void* shared, const float* gate_logit,
                                  int gate_stride, void* out, int T_, int d, int dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && d > 0 && top > 0, "experts_combine: bad sizes T=%d d=%d top=%d", T_, d, top);
  const int threads = d >= 1024 ? 256 : 128;
  if (dtype == DK_F32)
    experts_combine_kernel<float><<<T_, threads, 0, stream>>>(z, weight, top, (const float*)shared, gate_logit, gate_stride, (float*)out, d);
  else if (dtype == DK_BF16)
    experts_combine_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(z, weight, top, (const __nv_bfloat16*)shared, gate_logit, gate_stride,
                                                                      (__nv_bfloat16*)out, d);
  else DK_REQUIRE(false, "experts_combine: unknown dtype %d", dtype);
  return dk_check_launch("experts_combine");
}
