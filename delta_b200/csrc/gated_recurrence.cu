// Two recurrent mixers whose state is carried per request in 32 bit.
//
// gated_recurrence: a diagonal linear recurrence with a gate on its decay and one on its input (the real-gated linear
// recurrent unit).  Per token and channel c, with the gates' products gr, gi given (32 bit) and D_c <= 0 a constant:
//     r = sigmoid(gr + rb_c),  i = sigmoid(gi + ib_c),  a = exp(D_c r)
//     S_c <- a S_c + sqrt(1 - a^2) (i u_c),     out_c = S_c * act(y_c + yb_c)        act: the tanh form of gelu, or none
// 1 - a^2 is taken as -expm1(2 D r), which keeps its digits when a is close to one.
//
// matrix_memory: a matrix memory per head with exponential gating and a running maximum (mLSTM).  Per token and head, with
// the log input gate li and the log forget gate lf (32 bit), q [dk] (scaled), k [dk], v [dv]:
//     m' = max(lf + m, li);  keep = exp(lf + m - m'),  take = exp(li - m')
//     S <- keep S + take k v^T   [dk, dv];   z <- keep z + take k   [dk]
//     o = S^T q / (max(|z . q|, exp(-m')) + guard)
// S, z and m start at zero.  The gates arrive as products g (before the bias); li = cap tanh((g_i + b_i) / cap),
// lf = logsigmoid(cap tanh((g_f + b_f) / cap)).
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// One thread per (row, channel): the row's tokens in turn.  grid (ceil(C / blockDim), rows).
// SEG > 0: the row is cut into segments of SEG tokens, blockIdx.z names the segment.
//   PHASE 1: the segment from a zero state; its end state and the product of its decays are kept.
//   PHASE 2: the segment from its start state (made by the combine kernel), writing the outputs.
// PHASE 0: the whole row from and into the request's state.
template <typename T, int PHASE>
__global__ void __launch_bounds__(128) gated_recurrence_kernel(
    const T* __restrict__ u, const float* __restrict__ gates, long long g_tok, long long g_block, int block_size, const float* __restrict__ rb, const float* __restrict__ ib,
    const float* __restrict__ decay, const T* __restrict__ y, int y_stride, const float* __restrict__ yb, int act,
    float* __restrict__ state, T* __restrict__ out, const int* __restrict__ row_slot, const int* __restrict__ row_q_start,
    const int* __restrict__ row_q_len, int C, int seg_len, int segs, float* __restrict__ seg_state, float* __restrict__ seg_decay) {
  const int row = blockIdx.y, seg = blockIdx.z;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int len = row_q_len[row];
  const int first = PHASE == 0 ? 0 : seg * seg_len;
  if (first >= len && PHASE != 0) return;
  const int last = PHASE == 0 ? len : min(len, first + seg_len);
  const int q0 = row_q_start[row];
  const int b = c / block_size, j = c - b * block_size;
  const size_t goff = (size_t)b * g_block + j;
  const float bias_r = rb ? rb[c] : 0.f, bias_i = ib ? ib[c] : 0.f, D = decay[c], bias_y = yb ? yb[c] : 0.f;
  const size_t sidx = ((size_t)row * segs + seg) * C + c;
  float S = PHASE == 0 ? state[(size_t)row_slot[row] * C + c] : (PHASE == 2 ? seg_state[sidx] : 0.f);
  float prod = 1.f;
  for (int t = first; t < last; ++t) {
    const size_t tok = (size_t)(q0 + t);
    const float r = sigmoid_f(gates[tok * g_tok + goff] + bias_r);
    const float i = sigmoid_f(gates[tok * g_tok + goff + block_size] + bias_i);
    const float la = D * r;
    const float a = expf(la);
    const float in = sqrtf(fmaxf(-expm1f(2.f * la), 0.f)) * (i * to_f32<T>(u[tok * C + c]));
    S = fmaf(a, S, in);
    if (PHASE == 1) prod *= a;
    if (PHASE != 1) {
      const float yv = to_f32<T>(y[tok * y_stride + c]) + bias_y;
      out[tok * C + c] = from_f32<T>(S * (act ? gelu_tanh_f(yv) : yv));
    }
  }
  if (PHASE == 0) state[(size_t)row_slot[row] * C + c] = S;
  if (PHASE == 1) {
    seg_state[sidx] = S;
    seg_decay[sidx] = prod;
  }
}

// grid (ceil(C / 128), rows): the segments' end states become their start states, in order; the last value is the request's
__global__ void gated_recurrence_combine_kernel(float* __restrict__ state, float* __restrict__ seg_state, const float* __restrict__ seg_decay,
                                                const int* __restrict__ row_slot, const int* __restrict__ row_q_len, int C, int seg_len,
                                                int segs) {
  const int row = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int used = min(segs, (row_q_len[row] + seg_len - 1) / seg_len);
  float* slot = state + (size_t)row_slot[row] * C + c;
  float s = *slot;
  for (int g = 0; g < used; ++g) {
    const size_t at = ((size_t)row * segs + g) * C + c;
    const float end = seg_state[at];
    seg_state[at] = s;
    s = fmaf(seg_decay[at], s, end);
  }
  *slot = s;
}

// One block per (row, head, slice of the value entries); thread j owns column j of the slice of S, which lies in shared memory
// as [dk][dvs].  Tokens in turn; q and k of a token are read into shared memory by all threads.
template <typename T>
__global__ void matrix_memory_kernel(const T* __restrict__ src, int src_stride, int q_off, int k_off, int v_off, float q_scale,
                                     const float* __restrict__ gates, const float* __restrict__ gate_bias, float cap, float guard,
                                     float* __restrict__ S_state, float* __restrict__ z_state, float* __restrict__ m_state,
                                     float* __restrict__ out, const int* __restrict__ row_slot, const int* __restrict__ row_q_start,
                                     const int* __restrict__ row_q_len, int H, int dk, int dv, int dvs, int keep_zm) {
  extern __shared__ float sm[];
  float* S = sm;                    // [dk][dvs]
  float* z = S + (size_t)dk * dvs;  // [dk]
  float* qs = z + dk;               // [dk]
  float* ks = qs + dk;              // [dk]
  const int row = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * dvs;
  const int j = threadIdx.x;
  const int width = min(dvs, dv - j0);
  const bool live = j < width;
  const int slot = row_slot[row], q0 = row_q_start[row], len = row_q_len[row];
  float* Sg = S_state + ((size_t)slot * H + h) * dk * dv;
  float* zg = z_state + ((size_t)slot * H + h) * dk;
  for (int i = 0; i < dk; ++i)
    if (live) S[(size_t)i * dvs + j] = Sg[(size_t)i * dv + j0 + j];
  for (int i = threadIdx.x; i < dk; i += blockDim.x) z[i] = zg[i];
  float m = m_state[(size_t)slot * H + h];
  for (int t = 0; t < len; ++t) {
    const size_t tok = (size_t)(q0 + t);
    const T* base = src + tok * src_stride;
    __syncthreads();
    const float gi = gates[tok * 2 * H + h] + gate_bias[h], gf = gates[tok * 2 * H + H + h] + gate_bias[H + h];
    const float li = cap * tanhf(gi / cap), lf = log_sigmoid_f(cap * tanhf(gf / cap));
    const float m_new = fmaxf(lf + m, li);
    const float keep = expf(lf + m - m_new), take = expf(li - m_new);
    m = m_new;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
      const float kv = to_f32<T>(base[k_off + h * dk + i]);
      qs[i] = to_f32<T>(base[q_off + h * dk + i]) * q_scale;
      ks[i] = take * kv;
      z[i] = fmaf(keep, z[i], take * kv);
    }
    __syncthreads();
    if (live) {
      const float vj = to_f32<T>(base[v_off + h * dv + j0 + j]);
      float acc = 0.f, zq = 0.f;
      for (int i = 0; i < dk; ++i) {
        const float s = fmaf(keep, S[(size_t)i * dvs + j], ks[i] * vj);
        S[(size_t)i * dvs + j] = s;
        acc = fmaf(s, qs[i], acc);
        zq = fmaf(z[i], qs[i], zq);
      }
      out[tok * H * dv + h * dv + j0 + j] = acc / (fmaxf(fabsf(zq), expf(-m)) + guard);
    }
  }
  __syncthreads();
  for (int i = 0; i < dk; ++i)
    if (live) Sg[(size_t)i * dv + j0 + j] = S[(size_t)i * dvs + j];
  if (keep_zm) {      // (with several slices every block still reads them: matrix_memory_sums_kernel stores them afterwards)
    for (int i = threadIdx.x; i < dk; i += blockDim.x) zg[i] = z[i];
    if (threadIdx.x == 0) m_state[(size_t)slot * H + h] = m;
  }
}

// The keys' sum z and the maximum m over a row's tokens, one block per (row, head): what matrix_memory_kernel leaves to a launch
// of its own when a head's value entries are spread over several blocks, all of which read z and m as the step found them.
template <typename T>
__global__ void matrix_memory_sums_kernel(const T* __restrict__ src, int src_stride, int k_off, const float* __restrict__ gates,
                                          const float* __restrict__ gate_bias, float cap, float* __restrict__ z_state,
                                          float* __restrict__ m_state, const int* __restrict__ row_slot, const int* __restrict__ row_q_start,
                                          const int* __restrict__ row_q_len, int H, int dk) {
  const int row = blockIdx.x, h = blockIdx.y;
  const int slot = row_slot[row], q0 = row_q_start[row], len = row_q_len[row];
  float* zg = z_state + ((size_t)slot * H + h) * dk;
  float m = m_state[(size_t)slot * H + h];
  __syncthreads();
  for (int t = 0; t < len; ++t) {
    const size_t tok = (size_t)(q0 + t);
    const float gi = gates[tok * 2 * H + h] + gate_bias[h], gf = gates[tok * 2 * H + H + h] + gate_bias[H + h];
    const float li = cap * tanhf(gi / cap), lf = log_sigmoid_f(cap * tanhf(gf / cap));
    const float m_new = fmaxf(lf + m, li);
    const float keep = expf(lf + m - m_new), take = expf(li - m_new);
    m = m_new;
    for (int i = threadIdx.x; i < dk; i += blockDim.x)
      zg[i] = fmaf(keep, zg[i], take * to_f32<T>(src[tok * src_stride + k_off + h * dk + i]));
  }
  if (threadIdx.x == 0) m_state[(size_t)slot * H + h] = m;
}

// ---- single tokens (decode steps): the memory streams through registers once ---------------------------------------------
// One block per (row, head): 8 groups of 32 lanes; a lane owns four neighbouring value entries (16-byte accesses), group g the key
// entries g, g + 8, ...; value entries beyond 128 are taken in turn.  S <- keep S + take k v^T is written back in place, o = S^T q
// is summed over the groups in shared memory and divided by the denominator, which every thread has from a sum over the block.
// The value size is a multiple of 4.
template <typename T>
__global__ void __launch_bounds__(256)
matrix_memory_step_kernel(const T* __restrict__ src, int src_stride, int q_off, int k_off, int v_off, float q_scale,
                          const float* __restrict__ gates, const float* __restrict__ gate_bias, float cap, float guard,
                          float* __restrict__ S_state, float* __restrict__ z_state, float* __restrict__ m_state, float* __restrict__ out,
                          const int* __restrict__ row_slot, const int* __restrict__ row_q_start, int H, int dk, int dv) {
  extern __shared__ __align__(16) float sm[];
  float4* red = reinterpret_cast<float4*>(sm);       // [8][32]
  float* scratch = sm + 8 * 32 * 4;                  // [36]
  float* q = scratch + 36;                           // [dk], scaled
  float* k = q + dk;                                 // [dk], times the input gate's weight
  const int row = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, grp = tid >> 5;
  const size_t t = (size_t)row_q_start[row], slot = (size_t)row_slot[row] * H + h;
  const T* tok = src + t * src_stride;
  const float gi = gates[t * 2 * H + h] + gate_bias[h], gf = gates[t * 2 * H + H + h] + gate_bias[H + h];
  const float li = cap * tanhf(gi / cap), lf = log_sigmoid_f(cap * tanhf(gf / cap));
  const float m_old = m_state[slot];
  const float m_new = fmaxf(lf + m_old, li);
  const float keep = expf(lf + m_old - m_new), take = expf(li - m_new);
  float* zg = z_state + slot * dk;
  float zq = 0.f;
  for (int i = tid; i < dk; i += 256) {
    const float qv = to_f32<T>(tok[q_off + (size_t)h * dk + i]) * q_scale, kv = take * to_f32<T>(tok[k_off + (size_t)h * dk + i]);
    const float zn = fmaf(keep, zg[i], kv);
    q[i] = qv;
    k[i] = kv;
    zg[i] = zn;
    zq = fmaf(zn, qv, zq);
  }
  zq = block_sum(zq, scratch);      // (its barriers also stand between every thread's read of m and the write below)
  const float den = fmaxf(fabsf(zq), expf(-m_new)) + guard;
  if (tid == 0) m_state[slot] = m_new;
  float* Sg = S_state + slot * dk * dv;
  for (int j0 = 0; j0 < dv; j0 += 128) {
    const int j = j0 + lane * 4;
    const bool live = j < dv;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f), o = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
      const T* vp = tok + v_off + (size_t)h * dv + j;
      v = make_float4(to_f32<T>(vp[0]), to_f32<T>(vp[1]), to_f32<T>(vp[2]), to_f32<T>(vp[3]));
      float* st = Sg + j;
#pragma unroll 4
      for (int i = grp; i < dk; i += 8) {
        float4 s4 = *reinterpret_cast<const float4*>(st + (size_t)i * dv);
        const float ki = k[i], qi = q[i];
        s4.x = fmaf(keep, s4.x, ki * v.x);
        s4.y = fmaf(keep, s4.y, ki * v.y);
        s4.z = fmaf(keep, s4.z, ki * v.z);
        s4.w = fmaf(keep, s4.w, ki * v.w);
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
      *reinterpret_cast<float4*>(out + t * ((size_t)H * dv) + (size_t)h * dv + j) = make_float4(a.x / den, a.y / den, a.z / den, a.w / den);
    }
    __syncthreads();
  }
}

constexpr size_t MM_SMEM_LIMIT = 200 * 1024;
size_t mm_smem(int dk, int dvs) { return ((size_t)dk * dvs + 3 * (size_t)dk) * sizeof(float); }

}  // namespace

// gates: for token t and block b of `block_size` channels the decay gate's products at t * g_tok + b * g_block, the input gate's
// block_size entries behind them ([T, 2C]: g_tok = 2C, g_block = 2 block_size; [blocks, T, 2 block_size]: g_tok = 2 block_size,
// g_block = T * 2 block_size).  seg_len > 0: rows are cut into segments of that many tokens that run in parallel (`segs` the most of any
// row; seg_state and seg_decay hold rows * segs * C floats each).
extern "C" int dk_gated_recurrence(const void* u, const float* gates, long long g_tok, long long g_block, int block_size, const float* rb, const float* ib, const float* decay,
                                   const void* y, int y_stride, const float* yb, int act, float* state, void* out, const int* row_slot,
                                   const int* row_q_start, const int* row_q_len, int rows, int C, int seg_len, int segs, float* seg_state,
                                   float* seg_decay, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && C > 0 && block_size > 0 && C % block_size == 0 && y_stride >= C,
             "gated_recurrence: bad sizes rows=%d C=%d block=%d stride=%d", rows, C, block_size, y_stride);
  DK_REQUIRE(rows <= 65535, "gated_recurrence: %d rows are above the grid's limit", rows);
  DK_REQUIRE(dtype == DK_F32 || dtype == DK_BF16, "gated_recurrence: unknown dtype %d", dtype);
  const int threads = 128;
  const int cb = (C + threads - 1) / threads;
#define LAUNCH(T, PHASE, grid)                                                                                                   \
  gated_recurrence_kernel<T, PHASE><<<grid, threads, 0, stream>>>((const T*)u, gates, g_tok, g_block, block_size, rb, ib, decay, (const T*)y, y_stride, \
                                                                  yb, act, state, (T*)out, row_slot, row_q_start, row_q_len, C,  \
                                                                  seg_len, segs, seg_state, seg_decay)
  if (seg_len <= 0) {
    const dim3 grid(cb, rows, 1);
    if (dtype == DK_F32) LAUNCH(float, 0, grid);
    else LAUNCH(__nv_bfloat16, 0, grid);
    return dk_check_launch("gated_recurrence");
  }
  DK_REQUIRE(segs > 0 && segs <= 65535 && seg_state != nullptr && seg_decay != nullptr, "gated_recurrence: bad segments (%d)", segs);
  const dim3 grid(cb, rows, segs), cgrid(cb, rows, 1);
  if (dtype == DK_F32) LAUNCH(float, 1, grid);
  else LAUNCH(__nv_bfloat16, 1, grid);
  gated_recurrence_combine_kernel<<<cgrid, threads, 0, stream>>>(state, seg_state, seg_decay, row_slot, row_q_len, C, seg_len, segs);
  if (dtype == DK_F32) LAUNCH(float, 2, grid);
  else LAUNCH(__nv_bfloat16, 2, grid);
#undef LAUNCH
  return dk_check_launch("gated_recurrence");
}

// The slice of value entries a block of matrix_memory takes.
extern "C" int dk_matrix_memory_slice(int rows, int H, int dk, int dv) {
  int dvs = dv < 128 ? dv : 128;
  while (dvs > 1 && mm_smem(dk, dvs) > MM_SMEM_LIMIT) dvs = (dvs + 1) / 2;
  const int sms = dk_sm_count();
  while (dvs > 32 && (long long)rows * H * ((dv + dvs - 1) / dvs) < sms) dvs = (dvs + 1) / 2;
  return dvs;
}

// src [T, stride] holds a token's q at q_off, k at k_off (H * dk each) and v at v_off (H * dv); gates [T, 2H] the input gates'
// products and behind them the forget gates'; gate_bias [2H] likewise.  out float [T, H * dv].
extern "C" int dk_matrix_memory(const void* src, int src_stride, int q_off, int k_off, int v_off, float q_scale, const float* gates,
                                const float* gate_bias, float cap, float guard, float* S_state, float* z_state, float* m_state,
                                float* out, const int* row_slot, const int* row_q_start, const int* row_q_len, int rows, int H, int dk,
                                int dv, int dvs, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && H > 0 && dk > 0 && dv > 0 && dvs > 0 && dvs <= 1024, "matrix_memory: bad sizes rows=%d H=%d dk=%d dv=%d slice=%d",
             rows, H, dk, dv, dvs);
  DK_REQUIRE(cap > 0.f, "matrix_memory: the gates' cap must be positive");
  const size_t smem = mm_smem(dk, dvs);
  DK_REQUIRE(smem <= MM_SMEM_LIMIT, "matrix_memory: a state slice of %d x %d does not fit the shared memory", dk, dvs);
  DK_REQUIRE(H <= 65535, "matrix_memory: %d heads are above the grid's limit", H);
  const dim3 grid(rows, H, (dv + dvs - 1) / dvs);
  const int threads = ((dvs + 31) / 32) * 32;
#define LAUNCH(T)                                                                                                                  \
  do {                                                                                                                             \
    if (smem > 48 * 1024 &&                                                                                                        \
        cudaFuncSetAttribute(matrix_memory_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {   \
      cudaGetLastError();                                                                                                          \
      DK_REQUIRE(false, "matrix_memory: %zu bytes of shared memory were not granted", smem);                                       \
    }                                                                                                                              \
    matrix_memory_kernel<T><<<grid, threads, smem, stream>>>((const T*)src, src_stride, q_off, k_off, v_off, q_scale, gates, gate_bias, \
                                                             cap, guard, S_state, z_state, m_state, out, row_slot, row_q_start,   \
                                                             row_q_len, H, dk, dv, dvs, grid.z == 1);                             \
    if (grid.z > 1)                                                                                                                \
      matrix_memory_sums_kernel<T><<<dim3(rows, H), 128, 0, stream>>>((const T*)src, src_stride, k_off, gates, gate_bias, cap, z_state, \
                                                                       m_state, row_slot, row_q_start, row_q_len, H, dk);         \
  } while (0)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "matrix_memory: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("matrix_memory");
}

// Decode steps: every row brings one token.  The value size is a multiple of 4 and the memory and the output are 16-byte aligned.
extern "C" int dk_matrix_memory_step_supported(int dk, int dv) { return dv % 4 == 0 && (size_t)(2 * dk + 36) * 4 + 8 * 32 * 16 <= 48 * 1024; }

extern "C" int dk_matrix_memory_step(const void* src, int src_stride, int q_off, int k_off, int v_off, float q_scale, const float* gates,
                                     const float* gate_bias, float cap, float guard, float* S_state, float* z_state, float* m_state,
                                     float* out, const int* row_slot, const int* row_q_start, int rows, int H, int dk, int dv, int dtype,
                                     cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && H > 0 && dk > 0 && dv > 0, "matrix_memory_step: bad sizes rows=%d H=%d dk=%d dv=%d", rows, H, dk, dv);
  DK_REQUIRE(cap > 0.f, "matrix_memory_step: the gates' cap must be positive");
  DK_REQUIRE(dk_matrix_memory_step_supported(dk, dv) && ((uintptr_t)S_state % 16) == 0 && ((uintptr_t)out % 16) == 0,
             "matrix_memory_step: heads of %d x %d are not taken (the value size must be a multiple of 4)", dk, dv);
  DK_REQUIRE(H <= 65535, "matrix_memory_step: %d heads are above the grid's limit", H);
  const dim3 grid(rows, H);
  const size_t smem = (size_t)(2 * dk + 36) * sizeof(float) + 8 * 32 * sizeof(float4);
#define LAUNCH(T)                                                                                                                      \
  matrix_memory_step_kernel<T><<<grid, 256, smem, stream>>>((const T*)src, src_stride, q_off, k_off, v_off, q_scale, gates, gate_bias, cap, \
                                                            guard, S_state, z_state, m_state, out, row_slot, row_q_start, H, dk, dv)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "matrix_memory_step: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("matrix_memory_step");
}
