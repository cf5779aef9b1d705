// The matrix memory with exponential gates (see gated_recurrence.cu) for long portions: a row's chunks run in parallel.
//
// Per head, with the log gates li_t, lf_t, the memory is C_t = e^(lf_t) C_(t-1) + e^(li_t) k_t v_t^T and what is kept is
// S_t = e^(-m_t) C_t with the running maximum m_t = max(lf_t + m_(t-1), li_t).  Inside a chunk of n tokens, with
//     F_t = lf_0 + ... + lf_t,   g_s = li_s - F_s,   M_t = max(m_in, max_{s<=t} g_s)       (m_in: the maximum before the chunk)
// the recurrence for m gives m_t = F_t + M_t, and F_t drops out of every weight:
//     S_t = e^(m_in - M_t) S_in + sum_{s<=t} e^(g_s - M_t) k_s v_s^T                  (no exponent is positive)
//     o_t = [e^(m_in - M_t) S_in^T q_t + sum_{s<=t} e^(g_s - M_t) (q_t . k_s) v_s] / (max(|same with z and k|, e^(-F_t - M_t)) + guard)
// The recurrence is linear in (S, z) once the maxima are known, so, as for the linear attention with a constant decay:
//   1. mm_chunk_state: every chunk taken alone from a zero state, U_c = sum_s e^(F_(n-1) + g_s - a_c) k_s v_s^T with its own maximum
//                      a_c = max_s (F_(n-1) + g_s), the same sum of the keys alone, and (F_(n-1), a_c);
//   2. mm_chunk_scan:  along a row, m_out = max(F_(n-1) + m_in, a_c), S_out = e^(F_(n-1) + m_in - m_out) S_in + e^(a_c - m_out) U_c,
//                      element by element; the state BEFORE chunk c takes the place of U_c, m_in is kept per chunk;
//   3. mm_chunk_out:   every chunk's outputs from the state before it, in parallel; the last chunk stores the row's maximum.
// Everything is 32-bit FMA.  Threads hold 4 x 4 tiles of outputs in registers.
#include "common.cuh"

namespace {

constexpr int MC = 32;             // tokens of a chunk: one lane of a warp per token when the gates are prepared
constexpr int MCP = MC + 4;        // padded row of the transposed tiles
constexpr size_t MMC_SMEM_LIMIT = 200 * 1024;

__device__ __forceinline__ int mm_up4(int n) { return (n + 3) & ~3; }
__device__ __forceinline__ float mm_log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// Lane s of a full warp: the log gates of token s of the chunk (li = -inf, lf = 0 behind the chunk's end), F_s and g_s.
__device__ __forceinline__ void mm_chunk_gates(const float* __restrict__ gates, const float* __restrict__ gate_bias, float cap, int H, int h,
                                               int t0, int n, int lane, float& F, float& g) {
  float li = -INFINITY, lf = 0.f;
  if (lane < n) {
    const size_t tok = (size_t)(t0 + lane);
    const float gi = gates[tok * 2 * H + h] + gate_bias[h], gf = gates[tok * 2 * H + H + h] + gate_bias[H + h];
    li = cap * tanhf(gi / cap);
    lf = mm_log_sigmoid(cap * tanhf(gf / cap));
  }
  F = lf;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, F, d);
    if (lane >= d) F += up;
  }
  g = li - F;      // -inf behind the end
}

// ---- 1. every chunk alone ------------------------------------------------------------------------------------------------
// grid (most chunks of a row, rows * H, slices of the value entries), 256 threads.
template <typename T>
__global__ void __launch_bounds__(256)
mm_chunk_state_kernel(const T* __restrict__ src, int src_stride, int k_off, int v_off, const float* __restrict__ gates,
                      const float* __restrict__ gate_bias, float cap, float* __restrict__ U, float* __restrict__ Z, float* __restrict__ info,
                      const int* __restrict__ row_q_start, const int* __restrict__ row_q_len, const int* __restrict__ chunk_base, int H, int dk,
                      int dv, int dvs, int vec) {
  extern __shared__ __align__(16) float sm[];
  const int row = blockIdx.y / H, h = blockIdx.y % H, j0 = blockIdx.z * dvs;
  const int jn = min(dvs, dv - j0), c0 = blockIdx.x * MC, n_new = row_q_len[row];
  if (c0 >= n_new || jn <= 0) return;
  const int n = min(MC, n_new - c0), t0 = row_q_start[row] + c0;
  const int dkp = mm_up4(dk), dvp = mm_up4(dvs), tid = threadIdx.x;
  float* Kd = sm;                    // [MC][dkp]: keys times their weight at the chunk's end
  float* V = Kd + MC * dkp;          // [MC][dvp]
  float* wt = V + MC * dvp;          // [MC]
  const size_t chunk = (size_t)(chunk_base[row] + blockIdx.x) * H + h;
  if (tid < 32) {
    float F, g;
    mm_chunk_gates(gates, gate_bias, cap, H, h, t0, n, tid, F, g);
    const float F_end = __shfl_sync(0xffffffffu, F, n - 1);
    const float e = F_end + g;                       // -inf behind the end
    const float a = warp_max(e);
    wt[tid] = expf(e - a);                           // 0 behind the end
    if (tid == 0 && blockIdx.z == 0) {
      info[chunk * 4 + 0] = F_end;
      info[chunk * 4 + 1] = a;
    }
  }
  __syncthreads();
  if (vec) {      // sizes and offsets are multiples of 8: sixteen-byte loads
    const int kc = dk / 8, vc = dvp / 8;
    for (int idx = tid; idx < MC * kc; idx += 256) {
      const int s = idx / kc, c = (idx - s * kc) * 8;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (s < n) {
        load8<T>(src + (size_t)(t0 + s) * src_stride + k_off + (size_t)h * dk + c, v);
        const float f = wt[s];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] *= f;
      }
      *reinterpret_cast<float4*>(Kd + s * dkp + c) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(Kd + s * dkp + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    for (int idx = tid; idx < MC * vc; idx += 256) {
      const int s = idx / vc, c = (idx - s * vc) * 8;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (s < n && c < jn) load8<T>(src + (size_t)(t0 + s) * src_stride + v_off + (size_t)h * dv + j0 + c, v);
      *reinterpret_cast<float4*>(V + s * dvp + c) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(V + s * dvp + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  } else {
    for (int idx = tid; idx < MC * dkp; idx += 256) {
      const int s = idx / dkp, i = idx - s * dkp;
      Kd[idx] = (s < n && i < dk) ? to_f32<T>(src[(size_t)(t0 + s) * src_stride + k_off + (size_t)h * dk + i]) * wt[s] : 0.f;
    }
    for (int idx = tid; idx < MC * dvp; idx += 256) {
      const int s = idx / dvp, j = idx - s * dvp;
      V[idx] = (s < n && j < jn) ? to_f32<T>(src[(size_t)(t0 + s) * src_stride + v_off + (size_t)h * dv + j0 + j]) : 0.f;
    }
  }
  __syncthreads();
  float* Uc = U + chunk * dk * dv;
  const int tiles_j = dvp / 4, tiles = (dkp / 4) * tiles_j;
  for (int tile = tid; tile < tiles; tile += 256) {
    const int ti = tile / tiles_j, tj = tile - ti * tiles_j;
    float acc[4][4] = {};
#pragma unroll 4
    for (int s = 0; s < n; ++s) {
      const float4 a = *reinterpret_cast<const float4*>(Kd + s * dkp + 4 * ti);
      const float4 b = *reinterpret_cast<const float4*>(V + s * dvp + 4 * tj);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(av[x], bv[y], acc[x][y]);
    }
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y)
        if (4 * ti + x < dk && 4 * tj + y < jn) Uc[(size_t)(4 * ti + x) * dv + j0 + 4 * tj + y] = acc[x][y];
  }
  if (blockIdx.z == 0)
    for (int i = tid; i < dk; i += 256) {
      float z = 0.f;
      for (int s = 0; s < n; ++s) z += Kd[s * dkp + i];
      Z[chunk * dk + i] = z;
    }
}

// ---- 2. the states before the chunks, in order -----------------------------------------------------------------------------
// grid (ceil((dk * dv + dk) / 256), rows * H): entry e < dk * dv of the memory, the others of the keys' sum.  Every thread
// follows the row's maxima itself (a few numbers per chunk); the request's maximum is stored by the third kernel, since
// blocks of this one still read it.
__global__ void mm_chunk_scan_kernel(float* __restrict__ U, float* __restrict__ Z, float* __restrict__ info, float* __restrict__ S_state,
                                     float* __restrict__ z_state, const float* __restrict__ m_state, const int* __restrict__ row_slot,
                                     const int* __restrict__ row_q_len, const int* __restrict__ chunk_base, int H, int dk, int dv) {
  const int row = blockIdx.y / H, h = blockIdx.y % H;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int per_head = dk * dv, n_new = row_q_len[row];
  if (e >= per_head + dk || n_new <= 0) return;
  const int chunks = (n_new + MC - 1) / MC;
  const size_t slot = (size_t)row_slot[row] * H + h, first = (size_t)chunk_base[row] * H + h;
  const bool memory = e < per_head;
  float* st = memory ? S_state + slot * per_head + e : z_state + slot * dk + (e - per_head);
  float* u = memory ? U + first * per_head + e : Z + first * dk + (e - per_head);
  const size_t step = (size_t)H * (memory ? per_head : dk);
  float S = *st, m = m_state[slot];
  float next = u[0];
  for (int c = 0; c < chunks; ++c) {
    const float cur = next;
    if (c + 1 < chunks) next = u[(size_t)(c + 1) * step];
    float* inf = info + (first + (size_t)c * H) * 4;
    const float F_end = inf[0], a = inf[1];
    const float m_out = fmaxf(F_end + m, a);
    u[(size_t)c * step] = S;
    if (e == 0) inf[2] = m;
    S = fmaf(expf(F_end + m - m_out), S, expf(a - m_out) * cur);
    m = m_out;
  }
  *st = S;
}

// ---- 3. every chunk's outputs ----------------------------------------------------------------------------------------------
// grid as the first kernel's, 128 threads.  U and Z hold the state before each chunk, info[2] its maximum.
template <typename T>
__global__ void __launch_bounds__(128)
mm_chunk_out_kernel(const T* __restrict__ src, int src_stride, int q_off, int k_off, int v_off, float q_scale, const float* __restrict__ gates,
                    const float* __restrict__ gate_bias, float cap, float guard, const float* __restrict__ U, const float* __restrict__ Z,
                    const float* __restrict__ info, float* __restrict__ m_state, float* __restrict__ out, const int* __restrict__ row_slot,
                    const int* __restrict__ row_q_start, const int* __restrict__ row_q_len, const int* __restrict__ chunk_base, int H, int dk,
                    int dv, int dvs, int vec) {
  extern __shared__ __align__(16) float sm[];
  const int row = blockIdx.y / H, h = blockIdx.y % H, j0 = blockIdx.z * dvs;
  const int jn = min(dvs, dv - j0), c0 = blockIdx.x * MC, n_new = row_q_len[row];
  if (c0 >= n_new || jn <= 0) return;
  const int n = min(MC, n_new - c0), t0 = row_q_start[row] + c0;
  const int dkp = mm_up4(dk), dvp = mm_up4(dvs), tid = threadIdx.x;
  float* Qt = sm;                    // [dkp][MCP]: scaled queries, transposed
  float* Kt = Qt + dkp * MCP;        // [dkp][MCP]
  float* S = Kt + dkp * MCP;         // [dkp][dvp]: the memory before the chunk
  float* V = S + dkp * dvp;          // [MC][dvp]
  float* At = V + MC * dvp;          // [MC][MCP]: At[s][t] = e^(g_s - M_t) q_t . k_s for s <= t, else 0
  float* zs = At + MC * MCP;         // [dkp]: the keys' sum before the chunk
  float* gs = zs + dkp;              // [MC]: g_s
  float* Ms = gs + MC;               // [MC]: M_t
  float* far = Ms + MC;              // [MC]: e^(m_in - M_t), the weight of the state before the chunk
  float* low = far + MC;             // [MC]: e^(-m_t), the denominator's floor
  float* den = low + MC;             // [MC]
  const size_t chunk = (size_t)(chunk_base[row] + blockIdx.x) * H + h;
  const float* Sc = U + chunk * dk * dv;
  if (tid < 32) {
    float F, g;
    mm_chunk_gates(gates, gate_bias, cap, H, h, t0, n, tid, F, g);
    const float m_in = info[chunk * 4 + 2];
    float M = g;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, M, d);
      if (tid >= d) M = fmaxf(M, up);
    }
    M = fmaxf(M, m_in);
    gs[tid] = g;
    Ms[tid] = M;
    far[tid] = expf(m_in - M);
    low[tid] = expf(-(F + M));
    if (tid == n - 1 && blockIdx.z == 0 && c0 + n == n_new) m_state[(size_t)row_slot[row] * H + h] = F + M;
  }
  for (int i = tid; i < dkp; i += 128) zs[i] = i < dk ? Z[chunk * dk + i] : 0.f;
  if (vec) {      // sizes and offsets are multiples of 8: sixteen-byte loads
    const int kc = dk / 8, vc = dvp / 8, sc = dvp / 4;
    for (int idx = tid; idx < MC * kc; idx += 128) {      // a warp takes eight entries of all 32 tokens: stores without conflicts
      const int t = idx % MC, c = (idx / MC) * 8;
      float q[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, k[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (t < n) {
        const T* p = src + (size_t)(t0 + t) * src_stride + (size_t)h * dk + c;
        load8<T>(p + q_off, q);
        load8<T>(p + k_off, k);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        Qt[(c + e) * MCP + t] = q[e] * q_scale;
        Kt[(c + e) * MCP + t] = k[e];
      }
    }
    for (int idx = tid; idx < dk * sc; idx += 128) {
      const int i = idx / sc, j = (idx - i * sc) * 4;
      *reinterpret_cast<float4*>(S + i * dvp + j) =
          j < jn ? *reinterpret_cast<const float4*>(Sc + (size_t)i * dv + j0 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int idx = tid; idx < MC * vc; idx += 128) {
      const int s2 = idx / vc, c = (idx - s2 * vc) * 8;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (s2 < n && c < jn) load8<T>(src + (size_t)(t0 + s2) * src_stride + v_off + (size_t)h * dv + j0 + c, v);
      *reinterpret_cast<float4*>(V + s2 * dvp + c) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(V + s2 * dvp + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  } else {
    for (int idx = tid; idx < dkp * MC; idx += 128) {
      const int t = idx / dkp, i = idx - t * dkp;
      float qv = 0.f, kv = 0.f;
      if (t < n && i < dk) {
        const T* p = src + (size_t)(t0 + t) * src_stride + (size_t)h * dk + i;
        qv = to_f32<T>(p[q_off]) * q_scale;
        kv = to_f32<T>(p[k_off]);
      }
      Qt[i * MCP + t] = qv;
      Kt[i * MCP + t] = kv;
    }
    for (int idx = tid; idx < dkp * dvp; idx += 128) {
      const int i = idx / dvp, j = idx - i * dvp;
      S[idx] = (i < dk && j < jn) ? Sc[(size_t)i * dv + j0 + j] : 0.f;
    }
    for (int idx = tid; idx < MC * dvp; idx += 128) {
      const int s2 = idx / dvp, j = idx - s2 * dvp;
      V[idx] = (s2 < n && j < jn) ? to_f32<T>(src[(size_t)(t0 + s2) * src_stride + v_off + (size_t)h * dv + j0 + j]) : 0.f;
    }
  }
  __syncthreads();
  // weighted scores inside the chunk: tiles on and below the diagonal
  for (int tile = tid; tile < (MC / 4) * (MC / 4); tile += 128) {
    const int tt = tile / (MC / 4), ts = tile - tt * (MC / 4);
    float acc[4][4] = {};
    if (ts <= tt) {
#pragma unroll 4
      for (int i = 0; i < dk; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(Qt + i * MCP + 4 * tt);
        const float4 b = *reinterpret_cast<const float4*>(Kt + i * MCP + 4 * ts);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
          for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(av[x], bv[y], acc[x][y]);
      }
    }
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int t = 4 * tt + x, s2 = 4 * ts + y;
        At[s2 * MCP + t] = (s2 <= t && t < n) ? acc[x][y] * expf(gs[s2] - Ms[t]) : 0.f;
      }
  }
  __syncthreads();
  // the denominators: |z_t . q_t| against the floor, z_t = far_t z_in + sum_{s<=t} e^(g_s - M_t) k_s
  if (tid < MC) {
    float zq = 0.f, inside = 0.f;
    for (int i = 0; i < dk; ++i) zq = fmaf(zs[i], Qt[i * MCP + tid], zq);
    for (int s2 = 0; s2 <= tid; ++s2) inside += At[s2 * MCP + tid];
    den[tid] = fmaxf(fabsf(fmaf(far[tid], zq, inside)), low[tid]) + guard;
  }
  __syncthreads();
  const int tiles_j = dvp / 4;
  for (int tile = tid; tile < (MC / 4) * tiles_j; tile += 128) {
    const int tt = tile / tiles_j, tj = tile - tt * tiles_j;
    if (4 * tt >= n) continue;
    float before[4][4] = {}, inside[4][4] = {};
#pragma unroll 4
    for (int i = 0; i < dk; ++i) {
      const float4 a = *reinterpret_cast<const float4*>(Qt + i * MCP + 4 * tt);
      const float4 b = *reinterpret_cast<const float4*>(S + i * dvp + 4 * tj);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) before[x][y] = fmaf(av[x], bv[y], before[x][y]);
    }
    const int s_end = min(n, 4 * tt + 4);
    for (int s2 = 0; s2 < s_end; ++s2) {
      const float4 a = *reinterpret_cast<const float4*>(At + s2 * MCP + 4 * tt);
      const float4 b = *reinterpret_cast<const float4*>(V + s2 * dvp + 4 * tj);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) inside[x][y] = fmaf(av[x], bv[y], inside[x][y]);
    }
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int t = 4 * tt + x, j = 4 * tj + y;
        if (t < n && j < jn)
          out[(size_t)(t0 + t) * ((size_t)H * dv) + (size_t)h * dv + j0 + j] = fmaf(far[t], before[x][y], inside[x][y]) / den[t];
      }
  }
}

size_t mmc_out_smem(int dk, int dvs) {
  const int dkp = (dk + 3) & ~3, dvp = (dvs + 3) & ~3;
  return ((size_t)2 * dkp * MCP + (size_t)dkp * dvp + (size_t)MC * dvp + (size_t)MC * MCP + dkp + 5 * MC) * sizeof(float);
}
size_t mmc_state_smem(int dk, int dvs) {
  const int dkp = (dk + 3) & ~3, dvp = (dvs + 3) & ~3;
  return ((size_t)MC * dkp + (size_t)MC * dvp + MC) * sizeof(float);
}
int mmc_slice(int dv) { return dv <= 64 ? dv : 64; }

}  // namespace

extern "C" int dk_matrix_memory_chunk() { return MC; }

extern "C" int dk_matrix_memory_chunked_supported(int dk, int dv) {
  return mmc_out_smem(dk, mmc_slice(dv)) <= MMC_SMEM_LIMIT && mmc_state_smem(dk, mmc_slice(dv)) <= MMC_SMEM_LIMIT;
}

// `chunk_base` [rows]: the number of chunks (of dk_matrix_memory_chunk() tokens) of all rows before this one; `total_chunks`: of all
// rows; `max_chunks`: the most of any row; `work`: total_chunks * H * (dk * dv + dk + 4) floats (every chunk's memory, keys' sum and
// four numbers).  The other arguments are dk_matrix_memory's.
extern "C" int dk_matrix_memory_chunked(const void* src, int src_stride, int q_off, int k_off, int v_off, float q_scale, const float* gates,
                                        const float* gate_bias, float cap, float guard, float* S_state, float* z_state, float* m_state,
                                        float* out, float* work, const int* row_slot, const int* row_q_start, const int* row_q_len,
                                        const int* chunk_base, int rows, int total_chunks, int max_chunks, int H, int dk, int dv, int dtype,
                                        cudaStream_t stream) {
  if (rows == 0 || max_chunks == 0) return 0;
  DK_REQUIRE(rows > 0 && max_chunks > 0 && total_chunks >= max_chunks && H > 0 && dk > 0 && dv > 0,
             "matrix_memory_chunked: bad sizes rows=%d chunks=%d of %d H=%d dk=%d dv=%d", rows, max_chunks, total_chunks, H, dk, dv);
  DK_REQUIRE(cap > 0.f, "matrix_memory_chunked: the gates' cap must be positive");
  DK_REQUIRE((long long)rows * H <= 65535, "matrix_memory_chunked: %d rows of %d heads are above the grid's limit", rows, H);
  const int dvs = mmc_slice(dv);
  const size_t sm1 = mmc_state_smem(dk, dvs), sm3 = mmc_out_smem(dk, dvs);
  DK_REQUIRE(sm1 <= MMC_SMEM_LIMIT && sm3 <= MMC_SMEM_LIMIT, "matrix_memory_chunked: heads of %d x %d do not fit the shared memory", dk, dv);
  float* U = work;
  float* Z = U + (size_t)total_chunks * H * dk * dv;
  float* info = Z + (size_t)total_chunks * H * dk;
  const dim3 grid(max_chunks, rows * H, (dv + dvs - 1) / dvs);
  const int vec = dk % 8 == 0 && dv % 8 == 0 && dvs % 8 == 0 && src_stride % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 &&
                  ((uintptr_t)src % 16) == 0 && ((uintptr_t)U % 16) == 0;
  const dim3 scan_grid((dk * dv + dk + 255) / 256, rows * H);
#define LAUNCH(T)                                                                                                                       \
  do {                                                                                                                                  \
    if (cudaFuncSetAttribute(mm_chunk_state_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1) != cudaSuccess ||        \
        cudaFuncSetAttribute(mm_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm3) != cudaSuccess) {          \
      cudaGetLastError();                                                                                                               \
      DK_REQUIRE(false, "matrix_memory_chunked: shared memory was not granted");                                                        \
    }                                                                                                                                   \
    mm_chunk_state_kernel<T><<<grid, 256, sm1, stream>>>((const T*)src, src_stride, k_off, v_off, gates, gate_bias, cap, U, Z, info,   \
                                                         row_q_start, row_q_len, chunk_base, H, dk, dv, dvs, vec);                     \
    mm_chunk_scan_kernel<<<scan_grid, 256, 0, stream>>>(U, Z, info, S_state, z_state, m_state, row_slot, row_q_len, chunk_base, H, dk, \
                                                        dv);                                                                           \
    mm_chunk_out_kernel<T><<<grid, 128, sm3, stream>>>((const T*)src, src_stride, q_off, k_off, v_off, q_scale, gates, gate_bias, cap, \
                                                       guard, U, Z, info, m_state, out, row_slot, row_q_start, row_q_len, chunk_base,  \
                                                       H, dk, dv, dvs, vec);                                                           \
  } while (0)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "matrix_memory_chunked: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("matrix_memory_chunked");
}
