// Linear attention with a constant decay per head ("lightning attention"), and the gated norm behind it.
//
// Per head, with a state S [dk, dv] in 32 bit that a request carries from token to token:
//     S_t = lambda * S_(t-1) + k_t v_t^T ,      o_t = S_t^T q_t .
// A row's new tokens are taken in chunks of C.  With the chunk's tokens numbered 0..n-1 and S the state before it,
//     o_t = lambda^(t+1) * S^T q_t + sum_{s<=t} lambda^(t-s) (q_t . k_s) v_s
//     S  <- lambda^n * S + sum_s lambda^(n-1-s) k_s v_s^T
// which is the recurrence itself, summed in another order.  No power of lambda is ever divided by: the powers
// lambda^0..lambda^C are tabulated from the 64-bit decay.  q, k and v may get an activation (silu) as they are read;
// all arithmetic is 32-bit FMA, whatever the type of the inputs.
//
// decay_attention: one block per (row, head, slice of the value entries); the slice's part of the state stays in
// shared memory over the row's chunks and goes back to the request's slot at the end.
// gated_rms_norm:  out = rmsnorm(o over all heads) * w * sigmoid(gate), one block per token.
#include "common.cuh"

namespace {
constexpr int C = 32;            // tokens of a chunk
constexpr int THREADS = 256;

__device__ __forceinline__ float act_silu(float z) { return z / (1.f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(THREADS)
decay_attention_kernel(const T* __restrict__ src, int src_stride, int q_off, int k_off, int v_off, int act,
                       const double* __restrict__ decays, float* __restrict__ state, float* __restrict__ out,
                       const int* __restrict__ row_slot, const int* __restrict__ row_q_start, const int* __restrict__ row_q_len,
                       int H, int dk, int dv, int dvs) {
  extern __shared__ __align__(16) float sm[];
  const int kp = dk + 1;                    // padded row of Q and K
  float* S = sm;                            // [dk][dvs]
  float* Q = S + (size_t)dk * dvs;          // [C][kp]
  float* K = Q + C * kp;                    // [C][kp]
  float* V = K + C * kp;                    // [C][dvs]
  float* A = V + C * dvs;                   // [C][C + 1]
  float* pw = A + C * (C + 1);              // [C + 1]
  const int row = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * dvs;
  const int jn = min(dvs, dv - j0);
  const int tid = threadIdx.x;
  const int n_new = row_q_len[row];
  if (n_new <= 0 || jn <= 0) return;
  const int t0 = row_q_start[row];
  float* st = state + (((size_t)row_slot[row] * H + h) * dk) * dv + j0;
  if (tid <= C) pw[tid] = (float)pow(decays[h], (double)tid);
  for (int idx = tid; idx < dk * jn; idx += THREADS) {
    const int i = idx / jn, j = idx - i * jn;
    S[i * dvs + j] = st[(size_t)i * dv + j];
  }
  for (int c0 = 0; c0 < n_new; c0 += C) {
    const int n = min(C, n_new - c0);
    __syncthreads();
    for (int idx = tid; idx < n * dk; idx += THREADS) {
      const int t = idx / dk, i = idx - t * dk;
      const T* p = src + (size_t)(t0 + c0 + t) * src_stride + (size_t)h * dk + i;
      const float qv = to_f32<T>(p[q_off]), kv = to_f32<T>(p[k_off]);
      Q[t * kp + i] = act ? act_silu(qv) : qv;
      K[t * kp + i] = act ? act_silu(kv) : kv;
    }
    for (int idx = tid; idx < n * jn; idx += THREADS) {
      const int t = idx / jn, j = idx - t * jn;
      const float vv = to_f32<T>(src[(size_t)(t0 + c0 + t) * src_stride + v_off + (size_t)h * dv + j0 + j]);
      V[t * dvs + j] = act ? act_silu(vv) : vv;
    }
    __syncthreads();
    // A[t][s] = lambda^(t-s) q_t . k_s for s <= t
    for (int idx = tid; idx < n * n; idx += THREADS) {
      const int t = idx / n, s = idx - t * n;
      if (s > t) continue;
      const float* qt = Q + t * kp;
      const float* ks = K + s * kp;
      float a = 0.f;
      for (int i = 0; i < dk; ++i) a = fmaf(qt[i], ks[i], a);
      A[t * (C + 1) + s] = a * pw[t - s];
    }
    __syncthreads();
    // o_t[j] = lambda^(t+1) sum_i q_t[i] S[i][j] + sum_{s<=t} A[t][s] v_s[j]
    for (int idx = tid; idx < n * jn; idx += THREADS) {
      const int t = idx / jn, j = idx - t * jn;
      const float* qt = Q + t * kp;
      float far = 0.f;
      for (int i = 0; i < dk; ++i) far = fmaf(qt[i], S[i * dvs + j], far);
      float near = 0.f;
      for (int s = 0; s <= t; ++s) near = fmaf(A[t * (C + 1) + s], V[s * dvs + j], near);
      out[(size_t)(t0 + c0 + t) * ((size_t)H * dv) + (size_t)h * dv + j0 + j] = fmaf(pw[t + 1], far, near);
    }
    __syncthreads();
    // S[i][j] = lambda^n S[i][j] + sum_s lambda^(n-1-s) k_s[i] v_s[j]
    for (int idx = tid; idx < dk * jn; idx += THREADS) {
      const int i = idx / jn, j = idx - i * jn;
      float a = 0.f;
      for (int s = 0; s < n; ++s) a = fmaf(pw[n - 1 - s] * K[s * kp + i], V[s * dvs + j], a);
      S[i * dvs + j] = fmaf(pw[n], S[i * dvs + j], a);
    }
  }
  __syncthreads();
  for (int idx = tid; idx < dk * jn; idx += THREADS) {
    const int i = idx / jn, j = idx - i * jn;
    st[(size_t)i * dv + j] = S[i * dvs + j];
  }
}

// ---- single tokens (decode steps): the state streams through registers once ---------------------------------------------
// One block per (row, head, 128 value entries): 8 groups of 32 lanes; a lane owns four neighbouring value entries (16-byte
// accesses, a state row is read by consecutive lanes), group g the key entries g, g + 8, ...  Every thread has all its loads
// under way at once; S <- lambda S + k v^T is written back in place and o = S^T q is summed over the groups in shared memory.
// The value size is a multiple of 4.
template <typename T>
__global__ void __launch_bounds__(256)
decay_step_kernel(const T* __restrict__ src, int src_stride, int q_off, int k_off, int v_off, int act, const double* __restrict__ decays,
                  float* __restrict__ state, float* __restrict__ out, const int* __restrict__ row_slot,
                  const int* __restrict__ row_q_start, int H, int dk, int dv) {
  extern __shared__ __align__(16) float sm[];
  float* q = sm;                       // [dk]
  float* k = q + dk;                   // [dk]
  float4* red = reinterpret_cast<float4*>(k + dk + ((2 * dk) & 2));   // [8][32], on the next 16-byte boundary
  const int row = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, grp = tid >> 5;
  const int t = row_q_start[row];
  const T* tok = src + (size_t)t * src_stride;
  for (int i = tid; i < dk; i += 256) {
    const float qv = to_f32<T>(tok[q_off + (size_t)h * dk + i]), kv = to_f32<T>(tok[k_off + (size_t)h * dk + i]);
    q[i] = act ? act_silu(qv) : qv;
    k[i] = act ? act_silu(kv) : kv;
  }
  const int j = blockIdx.z * 128 + lane * 4;
  const bool live = j < dv;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    const T* vp = tok + v_off + (size_t)h * dv + j;
    v = make_float4(to_f32<T>(vp[0]), to_f32<T>(vp[1]), to_f32<T>(vp[2]), to_f32<T>(vp[3]));
    if (act) v = make_float4(act_silu(v.x), act_silu(v.y), act_silu(v.z), act_silu(v.w));
  }
  const float lam = (float)decays[h];
  __syncthreads();
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    float* st = state + (((size_t)row_slot[row] * H + h) * dk) * dv + j;
#pragma unroll 4
    for (int i = grp; i < dk; i += 8) {
      float4 s4 = *reinterpret_cast<const float4*>(st + (size_t)i * dv);
      const float ki = k[i], qi = q[i];
      s4.x = fmaf(lam, s4.x, ki * v.x);
      s4.y = fmaf(lam, s4.y, ki * v.y);
      s4.z = fmaf(lam, s4.z, ki * v.z);
      s4.w = fmaf(lam, s4.w, ki * v.w);
      *reinterpret_cast<float4*>(st + (size_t)i * dv) = s4;
      o.x = fmaf(qi, s4.x, o.x);
      o.y = fmaf(qi, s4.y, o.y);
      o.z = fmaf(qi, s4.z, o.z);
      o.w = fmaf(qi, s4.w, o.w);
    }
  }
  red[grp * 32 + lane] = o;
  __syncthreads();
  if (grp == 0 && live) {
    float4 a = red[lane];
#pragma unroll
    for (int g = 1; g < 8; ++g) {
      const float4 b = red[g * 32 + lane];
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)t * ((size_t)H * dv) + (size_t)h * dv + j) = a;
  }
}

// ---- long portions: the chunks of a row run in parallel --------------------------------------------------------------
// The recurrence is linear in the state, so with U_c = sum_s lambda^(n-1-s) k_s v_s^T of chunk c taken alone:
//   1. decay_chunk_state: U_c for every chunk of every row, in parallel;
//   2. decay_chunk_scan:  S_c = lambda^n S_(c-1) + U_c along a row, element by element; the state BEFORE chunk c takes the
//                         place of U_c, the last one goes to the request's slot;
//   3. decay_chunk_out:   o_t = lambda^(t+1) S^T q_t + sum_{s<=t} lambda^(t-s) (q_t . k_s) v_s  for every chunk, in parallel.
// Threads hold 4 x 4 tiles of outputs in registers and read shared memory sixteen bytes at a time.
constexpr int PC = 32;             // tokens of a chunk on this path
constexpr int PCP = PC + 4;        // padded row of the transposed tiles

__device__ __forceinline__ int up4(int n) { return (n + 3) & ~3; }

template <typename T>
__global__ void __launch_bounds__(256)
decay_chunk_state_kernel(const T* __restrict__ src, int src_stride, int k_off, int v_off, int act, const double* __restrict__ decays,
                         float* __restrict__ U, const int* __restrict__ row_q_start, const int* __restrict__ row_q_len,
                         const int* __restrict__ chunk_base, int H, int dk, int dv, int dvs, int vec) {
  extern __shared__ __align__(16) float sm[];
  const int row = blockIdx.y / H, h = blockIdx.y % H, j0 = blockIdx.z * dvs;
  const int jn = min(dvs, dv - j0), c0 = blockIdx.x * PC, n_new = row_q_len[row];
  if (c0 >= n_new || jn <= 0) return;
  const int n = min(PC, n_new - c0), t0 = row_q_start[row] + c0;
  const int dkp = up4(dk), dvp = up4(dvs), tid = threadIdx.x;
  float* Kd = sm;                    // [PC][dkp]: keys times lambda^(n-1-s)
  float* V = Kd + PC * dkp;          // [PC][dvp]
  float* pw = V + PC * dvp;          // [PC + 1]
  if (tid <= PC) pw[tid] = (float)pow(decays[h], (double)tid);
  __syncthreads();
  if (vec) {      // sizes and offsets are multiples of 8: sixteen-byte loads, all of a thread's loads under way at once
    const int kc = dk / 8, vc = dvp / 8;
    for (int idx = tid; idx < PC * kc; idx += 256) {
      const int s = idx / kc, c = (idx - s * kc) * 8;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (s < n) {
        load8<T>(src + (size_t)(t0 + s) * src_stride + k_off + (size_t)h * dk + c, v);
        const float f = pw[n - 1 - s];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (act ? act_silu(v[e]) : v[e]) * f;
      }
      *reinterpret_cast<float4*>(Kd + s * dkp + c) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(Kd + s * dkp + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    for (int idx = tid; idx < PC * vc; idx += 256) {
      const int s = idx / vc, c = (idx - s * vc) * 8;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (s < n && c < jn) {
        load8<T>(src + (size_t)(t0 + s) * src_stride + v_off + (size_t)h * dv + j0 + c, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = act ? act_silu(v[e]) : v[e];
      }
      *reinterpret_cast<float4*>(V + s * dvp + c) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(V + s * dvp + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  } else {
  for (int idx = tid; idx < PC * dkp; idx += 256) {
    const int s = idx / dkp, i = idx - s * dkp;
    float v = 0.f;
    if (s < n && i < dk) {
      v = to_f32<T>(src[(size_t)(t0 + s) * src_stride + k_off + (size_t)h * dk + i]);
      if (act) v = act_silu(v);
      v *= pw[n - 1 - s];
    }
    Kd[idx] = v;
  }
  for (int idx = tid; idx < PC * dvp; idx += 256) {
    const int s = idx / dvp, j = idx - s * dvp;
    float v = 0.f;
    if (s < n && j < jn) {
      v = to_f32<T>(src[(size_t)(t0 + s) * src_stride + v_off + (size_t)h * dv + j0 + j]);
      if (act) v = act_silu(v);
    }
    V[idx] = v;
  }
  }
  __syncthreads();
  float* Uc = U + ((size_t)(chunk_base[row] + blockIdx.x) * H + h) * dk * dv;
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
}

__global__ void decay_chunk_scan_kernel(float* __restrict__ U, float* __restrict__ state, const double* __restrict__ decays,
                                        const int* __restrict__ row_slot, const int* __restrict__ row_q_len,
                                        const int* __restrict__ chunk_base, int H, int per_head) {
  const int row = blockIdx.y / H, h = blockIdx.y % H;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int n_new = row_q_len[row];
  if (e >= per_head || n_new <= 0) return;
  const int chunks = (n_new + PC - 1) / PC;
  const float lam_full = (float)pow(decays[h], (double)PC), lam_last = (float)pow(decays[h], (double)(n_new - (chunks - 1) * PC));
  float* st = state + ((size_t)row_slot[row] * H + h) * per_head + e;
  float* u = U + ((size_t)chunk_base[row] * H + h) * per_head + e;
  const size_t step = (size_t)H * per_head;
  float S = *st;
  float next = u[0];
  for (int c = 0; c < chunks; ++c) {
    const float cur = next;
    if (c + 1 < chunks) next = u[(size_t)(c + 1) * step];
    u[(size_t)c * step] = S;
    S = fmaf(c + 1 < chunks ? lam_full : lam_last, S, cur);
  }
  *st = S;
}

template <typename T>
__global__ void __launch_bounds__(128)
decay_chunk_out_kernel(const T* __restrict__ src, int src_stride, int q_off, int k_off, int v_off, int act,
                       const double* __restrict__ decays, const float* __restrict__ U, float* __restrict__ out,
                       const int* __restrict__ row_q_start, const int* __restrict__ row_q_len, const int* __restrict__ chunk_base,
                       int H, int dk, int dv, int dvs, int vec) {
  extern __shared__ __align__(16) float sm[];
  const int row = blockIdx.y / H, h = blockIdx.y % H, j0 = blockIdx.z * dvs;
  const int jn = min(dvs, dv - j0), c0 = blockIdx.x * PC, n_new = row_q_len[row];
  if (c0 >= n_new || jn <= 0) return;
  const int n = min(PC, n_new - c0), t0 = row_q_start[row] + c0;
  const int dkp = up4(dk), dvp = up4(dvs), tid = threadIdx.x;
  float* Qt = sm;                    // [dkp][PCP]: queries, transposed
  float* Kt = Qt + dkp * PCP;        // [dkp][PCP]
  float* S = Kt + dkp * PCP;         // [dkp][dvp]: the state before the chunk
  float* V = S + dkp * dvp;          // [PC][dvp]
  float* At = V + PC * dvp;          // [PC][PCP]: At[s][t] = lambda^(t-s) q_t . k_s for s <= t, else 0
  float* pw = At + PC * PCP;         // [PC + 1]
  if (tid <= PC) pw[tid] = (float)pow(decays[h], (double)tid);
  const float* Sc = U + ((size_t)(chunk_base[row] + blockIdx.x) * H + h) * dk * dv;
  if (vec) {      // sizes and offsets are multiples of 8: sixteen-byte loads, all of a thread's loads under way at once
    const int kc = dk / 8, vc = dvp / 8, sc = dvp / 4;
    for (int idx = tid; idx < PC * kc; idx += 128) {      // a warp takes eight entries of all 32 tokens: stores without conflicts
      const int t = idx % PC, c = (idx / PC) * 8;
      float q[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, k[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (t < n) {
        const T* p = src + (size_t)(t0 + t) * src_stride + (size_t)h * dk + c;
        load8<T>(p + q_off, q);
        load8<T>(p + k_off, k);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        Qt[(c + e) * PCP + t] = (act && t < n) ? act_silu(q[e]) : q[e];
        Kt[(c + e) * PCP + t] = (act && t < n) ? act_silu(k[e]) : k[e];
      }
    }
    for (int idx = tid; idx < dk * sc; idx += 128) {
      const int i = idx / sc, j = (idx - i * sc) * 4;
      *reinterpret_cast<float4*>(S + i * dvp + j) =
          j < jn ? *reinterpret_cast<const float4*>(Sc + (size_t)i * dv + j0 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int idx = tid; idx < PC * vc; idx += 128) {
      const int s2 = idx / vc, c = (idx - s2 * vc) * 8;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (s2 < n && c < jn) {
        load8<T>(src + (size_t)(t0 + s2) * src_stride + v_off + (size_t)h * dv + j0 + c, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = act ? act_silu(v[e]) : v[e];
      }
      *reinterpret_cast<float4*>(V + s2 * dvp + c) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(V + s2 * dvp + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  } else {
  for (int idx = tid; idx < dkp * PC; idx += 128) {
    const int t = idx / dkp, i = idx - t * dkp;
    float qv = 0.f, kv = 0.f;
    if (t < n && i < dk) {
      const T* p = src + (size_t)(t0 + t) * src_stride + (size_t)h * dk + i;
      qv = to_f32<T>(p[q_off]);
      kv = to_f32<T>(p[k_off]);
      if (act) {
        qv = act_silu(qv);
        kv = act_silu(kv);
      }
    }
    Qt[i * PCP + t] = qv;
    Kt[i * PCP + t] = kv;
  }
  for (int idx = tid; idx < dkp * dvp; idx += 128) {
    const int i = idx / dvp, j = idx - i * dvp;
    S[idx] = (i < dk && j < jn) ? Sc[(size_t)i * dv + j0 + j] : 0.f;
  }
  for (int idx = tid; idx < PC * dvp; idx += 128) {
    const int s = idx / dvp, j = idx - s * dvp;
    float v = 0.f;
    if (s < n && j < jn) {
      v = to_f32<T>(src[(size_t)(t0 + s) * src_stride + v_off + (size_t)h * dv + j0 + j]);
      if (act) v = act_silu(v);
    }
    V[idx] = v;
  }
  }
  __syncthreads();
  // scores of the chunk: tiles on and below the diagonal
  for (int tile = tid; tile < (PC / 4) * (PC / 4); tile += 128) {
    const int tt = tile / (PC / 4), ts = tile - tt * (PC / 4);
    float acc[4][4] = {};
    if (ts <= tt) {
#pragma unroll 4
      for (int i = 0; i < dk; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(Qt + i * PCP + 4 * tt);
        const float4 b = *reinterpret_cast<const float4*>(Kt + i * PCP + 4 * ts);
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
        At[s2 * PCP + t] = (s2 <= t) ? acc[x][y] * pw[t - s2] : 0.f;
      }
  }
  __syncthreads();
  const int tiles_j = dvp / 4;
  for (int tile = tid; tile < (PC / 4) * tiles_j; tile += 128) {
    const int tt = tile / tiles_j, tj = tile - tt * tiles_j;
    if (4 * tt >= n) continue;
    float far[4][4] = {}, near[4][4] = {};
#pragma unroll 4
    for (int i = 0; i < dk; ++i) {
      const float4 a = *reinterpret_cast<const float4*>(Qt + i * PCP + 4 * tt);
      const float4 b = *reinterpret_cast<const float4*>(S + i * dvp + 4 * tj);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) far[x][y] = fmaf(av[x], bv[y], far[x][y]);
    }
    const int s_end = min(n, 4 * tt + 4);
    for (int s2 = 0; s2 < s_end; ++s2) {
      const float4 a = *reinterpret_cast<const float4*>(At + s2 * PCP + 4 * tt);
      const float4 b = *reinterpret_cast<const float4*>(V + s2 * dvp + 4 * tj);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) near[x][y] = fmaf(av[x], bv[y], near[x][y]);
    }
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int t = 4 * tt + x, j = 4 * tj + y;
        if (t < n && j < jn) out[(size_t)(t0 + t) * ((size_t)H * dv) + (size_t)h * dv + j0 + j] = fmaf(pw[t + 1], far[x][y], near[x][y]);
      }
  }
}

size_t chunk_out_smem(int dk, int dvs) {
  const int dkp = (dk + 3) & ~3, dvp = (dvs + 3) & ~3;
  return ((size_t)2 * dkp * PCP + (size_t)dkp * dvp + (size_t)PC * dvp + (size_t)PC * PCP + PC + 1) * sizeof(float);
}
size_t chunk_state_smem(int dk, int dvs) {
  const int dkp = (dk + 3) & ~3, dvp = (dvs + 3) & ~3;
  return ((size_t)PC * dkp + (size_t)PC * dvp + PC + 1) * sizeof(float);
}
int chunk_slice(int dv) { return dv <= 64 ? dv : 64; }

template <typename T>
__global__ void gated_rms_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride,
                                      const float* __restrict__ w, T* __restrict__ out, int n, float eps) {
  __shared__ float scratch[34];
  const int t = blockIdx.x;
  const float* x = o + (size_t)t * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += x[i] * x[i];
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float g = to_f32<T>(gate[(size_t)t * gate_stride + i]);
    out[(size_t)t * n + i] = from_f32<T>(x[i] * inv * w[i] * (1.f / (1.f + expf(-g))));
  }
}

// The same with the statistics taken per group of `group` consecutive entries (a head): one warp per group.
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride,
                                        const float* __restrict__ w, T* __restrict__ out, int n, int group, float eps) {
  const int t = blockIdx.x, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const float* x = o + (size_t)t * n;
  for (int g0 = (threadIdx.x >> 5) * group; g0 < n; g0 += warps * group) {
    float ss = 0.f;
    for (int i = lane; i < group; i += 32) ss += x[g0 + i] * x[g0 + i];
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float)group + eps);
    for (int i = g0 + lane; i < g0 + group; i += 32) {
      const float g = to_f32<T>(gate[(size_t)t * gate_stride + i]);
      out[(size_t)t * n + i] = from_f32<T>(x[i] * inv * w[i] * (1.f / (1.f + expf(-g))));
    }
  }
}

size_t smem_floats(int dk, int dvs) { return (size_t)dk * dvs + 2 * (size_t)C * (dk + 1) + (size_t)C * dvs + C * (C + 1) + C + 1; }
constexpr size_t SMEM_LIMIT = 200 * 1024;
}  // namespace

// The slice of value entries a block takes: the whole head when its state fits the shared memory, and a smaller one
// while the grid would leave SMs without a block.
extern "C" int dk_decay_attention_slice(int rows, int H, int dk, int dv) {
  int dvs = dv;
  while (dvs > 1 && smem_floats(dk, dvs) * sizeof(float) > SMEM_LIMIT) dvs = (dvs + 1) / 2;
  const int sms = dk_sm_count();
  while (dvs > 32 && (long long)rows * H * ((dv + dvs - 1) / dvs) < sms) dvs = (dvs + 1) / 2;
  return dvs;
}

extern "C" int dk_decay_attention(const void* src, int src_stride, int q_off, int k_off, int v_off, int act, const double* decays,
                                  float* state, float* out, const int* row_slot, const int* row_q_start, const int* row_q_len,
                                  int rows, int H, int dk, int dv, int dvs, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && H > 0 && dk > 0 && dv > 0 && dvs > 0 && dvs <= dv, "decay_attention: bad sizes rows=%d H=%d dk=%d dv=%d slice=%d", rows, H, dk, dv, dvs);
  const size_t smem = smem_floats(dk, dvs) * sizeof(float);
  DK_REQUIRE(smem <= SMEM_LIMIT, "decay_attention: a state slice of %d x %d does not fit the shared memory", dk, dvs);
  DK_REQUIRE(H <= 65535, "decay_attention: %d heads are above the grid's limit", H);
  const dim3 grid(rows, H, (dv + dvs - 1) / dvs);
#define LAUNCH(T)                                                                                                                   \
  do {                                                                                                                              \
    if (smem > 48 * 1024 &&                                                                                                         \
        cudaFuncSetAttribute(decay_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { \
      cudaGetLastError();                                                                                                           \
      DK_REQUIRE(false, "decay_attention: %zu bytes of shared memory were not granted", smem);                                      \
    }                                                                                                                               \
    decay_attention_kernel<T><<<grid, THREADS, smem, stream>>>((const T*)src, src_stride, q_off, k_off, v_off, act, decays, state,  \
                                                                out, row_slot, row_q_start, row_q_len, H, dk, dv, dvs);            \
  } while (0)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "decay_attention: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("decay_attention");
}

// group: the entries whose root mean square is taken together (n: the whole row; a divisor of n: one head at a time)
extern "C" int dk_gated_rms_norm(const float* o, const void* gate, int gate_stride, const float* w, void* out, int T_, int n, float eps,
                                 int group, int dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && n > 0 && gate_stride >= n, "gated_rms_norm: bad sizes T=%d n=%d stride=%d", T_, n, gate_stride);
  DK_REQUIRE(group > 0 && n % group == 0, "gated_rms_norm: groups of %d entries do not divide a row of %d", group, n);
  const int threads = n >= 2048 ? 256 : 128;
  if (group != n) {
    if (dtype == DK_F32)
      gated_group_norm_kernel<float><<<T_, threads, 0, stream>>>(o, (const float*)gate, gate_stride, w, (float*)out, n, group, eps);
    else if (dtype == DK_BF16)
      gated_group_norm_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(o, (const __nv_bfloat16*)gate, gate_stride, w, (__nv_bfloat16*)out, n, group, eps);
    else DK_REQUIRE(false, "gated_rms_norm: unknown dtype %d", dtype);
    return dk_check_launch("gated_rms_norm");
  }
  if (dtype == DK_F32)
    gated_rms_norm_kernel<float><<<T_, threads, 0, stream>>>(o, (const float*)gate, gate_stride, w, (float*)out, n, eps);
  else if (dtype == DK_BF16)
    gated_rms_norm_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(o, (const __nv_bfloat16*)gate, gate_stride, w, (__nv_bfloat16*)out, n, eps);
  else DK_REQUIRE(false, "gated_rms_norm: unknown dtype %d", dtype);
  return dk_check_launch("gated_rms_norm");
}

// The chunk-parallel path.  `chunk_base` [rows]: the number of chunks (of dk_decay_attention_chunk() tokens) of all rows
// before this one; `U` holds total chunks x H x dk x dv floats; `max_chunks`: the most chunks of any row.
extern "C" int dk_decay_attention_chunk() { return PC; }

extern "C" int dk_decay_attention_chunked_supported(int dk, int dv) {
  return chunk_out_smem(dk, chunk_slice(dv)) <= SMEM_LIMIT && chunk_state_smem(dk, chunk_slice(dv)) <= SMEM_LIMIT;
}

extern "C" int dk_decay_attention_chunked(const void* src, int src_stride, int q_off, int k_off, int v_off, int act, const double* decays,
                                          float* state, float* out, float* U, const int* row_slot, const int* row_q_start,
                                          const int* row_q_len, const int* chunk_base, int rows, int max_chunks, int H, int dk, int dv,
                                          int dtype, cudaStream_t stream) {
  if (rows == 0 || max_chunks == 0) return 0;
  DK_REQUIRE(rows > 0 && max_chunks > 0 && H > 0 && dk > 0 && dv > 0, "decay_attention_chunked: bad sizes rows=%d chunks=%d H=%d dk=%d dv=%d", rows,
             max_chunks, H, dk, dv);
  DK_REQUIRE((long long)rows * H <= 65535, "decay_attention_chunked: %d rows of %d heads are above the grid's limit", rows, H);
  const int dvs = chunk_slice(dv);
  const size_t sm1 = chunk_state_smem(dk, dvs), sm3 = chunk_out_smem(dk, dvs);
  DK_REQUIRE(sm1 <= SMEM_LIMIT && sm3 <= SMEM_LIMIT, "decay_attention_chunked: heads of %d x %d do not fit the shared memory", dk, dv);
  const dim3 grid(max_chunks, rows * H, (dv + dvs - 1) / dvs);
  const int per_head = dk * dv;
  const int vec = dk % 8 == 0 && dv % 8 == 0 && dvs % 8 == 0 && src_stride % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 &&
                  ((uintptr_t)src % 16) == 0 && ((uintptr_t)U % 16) == 0;
  const dim3 scan_grid((per_head + 255) / 256, rows * H);
#define LAUNCH(T)                                                                                                                       \
  do {                                                                                                                                  \
    if (cudaFuncSetAttribute(decay_chunk_state_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1) != cudaSuccess ||     \
        cudaFuncSetAttribute(decay_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm3) != cudaSuccess) {       \
      cudaGetLastError();                                                                                                               \
      DK_REQUIRE(false, "decay_attention_chunked: shared memory was not granted");                                                      \
    }                                                                                                                                   \
    decay_chunk_state_kernel<T><<<grid, 256, sm1, stream>>>((const T*)src, src_stride, k_off, v_off, act, decays, U, row_q_start,     \
                                                            row_q_len, chunk_base, H, dk, dv, dvs, vec);                              \
    decay_chunk_scan_kernel<<<scan_grid, 256, 0, stream>>>(U, state, decays, row_slot, row_q_len, chunk_base, H, per_head);            \
    decay_chunk_out_kernel<T><<<grid, 128, sm3, stream>>>((const T*)src, src_stride, q_off, k_off, v_off, act, decays, U, out,         \
                                                          row_q_start, row_q_len, chunk_base, H, dk, dv, dvs, vec);                    \
  } while (0)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "decay_attention_chunked: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("decay_attention_chunked");
}

// Decode steps: every row brings one token.  The value size is a multiple of 4 and state and output are 16-byte aligned.
extern "C" int dk_decay_attention_step_supported(int dk, int dv) { return dv % 4 == 0 && (size_t)(2 * dk + 4) * 4 + 8 * 32 * 16 <= 48 * 1024; }

extern "C" int dk_decay_attention_step(const void* src, int src_stride, int q_off, int k_off, int v_off, int act, const double* decays,
                                       float* state, float* out, const int* row_slot, const int* row_q_start, int rows, int H, int dk,
                                       int dv, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && H > 0 && dk > 0 && dv > 0, "decay_attention_step: bad sizes rows=%d H=%d dk=%d dv=%d", rows, H, dk, dv);
  DK_REQUIRE(dk_decay_attention_step_supported(dk, dv) && ((uintptr_t)state % 16) == 0 && ((uintptr_t)out % 16) == 0,
             "decay_attention_step: heads of %d x %d are not taken (the value size must be a multiple of 4)", dk, dv);
  DK_REQUIRE(H <= 65535, "decay_attention_step: %d heads are above the grid's limit", H);
  const dim3 grid(rows, H, (dv + 127) / 128);
  const size_t smem = (size_t)(2 * dk + 4) * sizeof(float) + 8 * 32 * sizeof(float4);
  if (dtype == DK_F32)
    decay_step_kernel<float><<<grid, 256, smem, stream>>>((const float*)src, src_stride, q_off, k_off, v_off, act, decays, state, out, row_slot,
                                                          row_q_start, H, dk, dv);
  else if (dtype == DK_BF16)
    decay_step_kernel<__nv_bfloat16><<<grid, 256, smem, stream>>>((const __nv_bfloat16*)src, src_stride, q_off, k_off, v_off, act, decays, state,
                                                                  out, row_slot, row_q_start, H, dk, dv);
  else DK_REQUIRE(false, "decay_attention_step: unknown dtype %d", dtype);
  return dk_check_launch("decay_attention_step");
}
