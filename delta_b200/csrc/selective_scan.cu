// The selective state-space mixer (Mamba-1 kind): a short causal convolution per channel, and a
// diagonal linear recurrence whose step size, input and output maps depend on the token.
//
// A step brings, per batch row, q_len new tokens of a request; what the request left behind is its
// state in 32 bit, one slot per request:
//   conv_state [slot][taps-1][C]   the last taps-1 inputs of the convolution (oldest first)
//   scan_state [slot][C][N]        the recurrence's state
//
// Per token, channel c, state n (dt, the decay and the state in 32 bit):
//   x_c  = silu(bias_c + sum_j w[c][j] * in_c(t - (taps-1) + j))           (column taps-1: the current token)
//   dt_c = softplus(dtraw_c + dtbias_c)
//   S[c][n] <- exp(dt_c * A[c][n]) * S[c][n] + dt_c * x_c * B_n ,   A = -exp(A_log)
//   y_c  = (sum_n S[c][n] * C_n + D_c * x_c) * silu(z_c)
#include "common.cuh"

namespace {
constexpr int MAX_TAPS = 16;

// grid (tokens, ceil(C / blockDim)); one thread per (token, channel)
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ xin, int in_stride, const float* __restrict__ w, const float* __restrict__ bias,
                                 const float* __restrict__ conv_state, T* __restrict__ out, const int* __restrict__ tok_row,
                                 const int* __restrict__ row_slot, const int* __restrict__ row_q_start, int C, int taps,
                                 const float* __restrict__ in_bias, int act) {
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int row = tok_row[t];
  const int q0 = row_q_start[row];
  const int i = t - q0;
  const float* st = conv_state + (size_t)row_slot[row] * (taps - 1) * C;
  float acc = bias ? bias[c] : 0.f;
  const float ib = in_bias ? in_bias[c] : 0.f;      // a bias of the inputs themselves (the state holds it already)
  for (int j = 0; j < taps; ++j) {
    const int k = i - (taps - 1) + j;     // index among the row's tokens of this step; negative: before it
    const float v = k >= 0 ? to_f32<T>(xin[(size_t)(q0 + k) * in_stride + c]) + ib : st[(size_t)(taps - 1 + k) * C + c];
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
  }
  out[(size_t)t * C + c] = from_f32<T>(act ? acc / (1.f + expf(-acc)) : acc);
}

// grid (rows, ceil(C / blockDim)); one thread per (row, channel) reads what it needs, then writes
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ xin, int in_stride, float* __restrict__ conv_state,
                                  const int* __restrict__ row_slot, const int* __restrict__ row_q_start,
                                  const int* __restrict__ row_q_len, int C, int taps, const float* __restrict__ in_bias) {
  const int row = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int q0 = row_q_start[row], L = row_q_len[row];
  float* st = conv_state + (size_t)row_slot[row] * (taps - 1) * C;
  float v[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j < taps - 1) {
      const int k = L - (taps - 1) + j;
      v[j] = k >= 0 ? to_f32<T>(xin[(size_t)(q0 + k) * in_stride + c]) + (in_bias ? in_bias[c] : 0.f) : st[(size_t)(taps - 1 + k) * C + c];
    }
  }
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j)
    if (j < taps - 1) st[(size_t)j * C + c] = v[j];
}

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// Block: 128 threads = (128 / P) channels x P lanes; lane p of a channel keeps the states n = p, p + P, ...
// grid (ceil(C / (128 / P)), rows * segs).  Tokens go through shared memory TT at a time.
//
// A long row is cut into segments of `seg_len` tokens that run in parallel (MODE 1, 2); the recurrence is linear, so
//   MODE 1  runs every segment from a zero state and keeps its end state E_g and the sum of its step sizes d_g;
//   combine walks the segments of a row in order: start_0 = the request's state, start_{g+1} = exp(A d_g) start_g + E_g
//           (the decays of a segment multiply to exp(A * sum of dt)), and the last value is the request's new state;
//   MODE 2  runs every segment again from its start state and writes y.
// MODE 0 is the whole row in one block, from and into the request's state (single tokens, short portions).
constexpr int TT = 16;
template <typename T, int P, int MAXS, int MODE>
__global__ void __launch_bounds__(128) selective_scan_kernel(
    const T* __restrict__ x, const T* __restrict__ dtraw, const T* __restrict__ bc, int bc_stride, int b_off, int c_off,
    const T* __restrict__ z, int z_stride, const float* __restrict__ A_log, const float* __restrict__ Dw,
    const float* __restrict__ dt_bias, float* __restrict__ scan_state, T* __restrict__ out, const int* __restrict__ row_slot,
    const int* __restrict__ row_q_start, const int* __restrict__ row_q_len, int C, int N, int segs, int seg_len,
    float* __restrict__ seg_state, float* __restrict__ seg_dt) {
  constexpr int CH = 128 / P;
  extern __shared__ float sm[];
  float* s_dt = sm;                 // [TT][CH]
  float* s_x = s_dt + TT * CH;      // [TT][CH]
  float* s_g = s_x + TT * CH;       // [TT][CH]  silu(z)
  float* s_y = s_g + TT * CH;       // [TT][CH]
  float* s_B = s_y + TT * CH;       // [TT][N]
  float* s_C = s_B + TT * N;        // [TT][N]
  const int row = blockIdx.y / segs, seg = blockIdx.y % segs;
  const int c0 = blockIdx.x * CH;
  const int cl = threadIdx.x / P, part = threadIdx.x % P;
  const int c = c0 + cl;
  const bool live = c < C;
  const int row_len = row_q_len[row];
  if (seg * seg_len >= row_len) return;
  const int q0 = row_q_start[row] + seg * seg_len;
  const int L = MODE == 0 ? row_len : min(seg_len, row_len - seg * seg_len);
  float* st = MODE == 0 ? scan_state + ((size_t)row_slot[row] * C + (live ? c : 0)) * N
                        : seg_state + ((size_t)blockIdx.y * C + (live ? c : 0)) * N;
  float s[MAXS], a[MAXS];
#pragma unroll
  for (int k = 0; k < MAXS; ++k) {
    const int n = part + k * P;
    const bool on = live && n < N;
    s[k] = (on && MODE != 1) ? st[n] : 0.f;
    a[k] = on ? -expf(A_log[(size_t)c * N + n]) : 0.f;
  }
  const float dsk = live ? Dw[c] : 0.f;
  float dt_sum = 0.f;
  for (int t0 = 0; t0 < L; t0 += TT) {
    const int nt = min(TT, L - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * CH; idx += 128) {
      const int tt = idx / CH, cc = idx % CH;
      const size_t tok = (size_t)(q0 + t0 + tt);
      float dtv = 0.f, xv = 0.f, gv = 0.f;
      if (c0 + cc < C) {
        dtv = softplus_f(to_f32<T>(dtraw[tok * C + c0 + cc]) + dt_bias[c0 + cc]);
        xv = to_f32<T>(x[tok * C + c0 + cc]);
        if (MODE != 1) {
          const float zv = to_f32<T>(z[tok * z_stride + c0 + cc]);
          gv = zv / (1.f + expf(-zv));
        }
      }
      s_dt[idx] = dtv;
      s_x[idx] = xv;
      s_g[idx] = gv;
    }
    for (int idx = threadIdx.x; idx < nt * N; idx += 128) {
      const int tt = idx / N, n = idx % N;
      const size_t tok = (size_t)(q0 + t0 + tt);
      s_B[idx] = to_f32<T>(bc[tok * bc_stride + b_off + n]);
      if (MODE != 1) s_C[idx] = to_f32<T>(bc[tok * bc_stride + c_off + n]);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float dtv = s_dt[tt * CH + cl], xv = s_x[tt * CH + cl];
      const float dx = dtv * xv;
      dt_sum += dtv;
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < MAXS; ++k) {
        const int n = part + k * P;
        if (n < N) {
          s[k] = fmaf(expf(dtv * a[k]), s[k], dx * s_B[tt * N + n]);
          if (MODE != 1) acc = fmaf(s[k], s_C[tt * N + n], acc);
        }
      }
      if (MODE != 1) {
#pragma unroll
        for (int o = P / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (part == 0) s_y[tt * CH + cl] = (acc + dsk * xv) * s_g[tt * CH + cl];
      }
    }
    if (MODE != 1) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < nt * CH; idx += 128) {
        const int tt = idx / CH, cc = idx % CH;
        if (c0 + cc < C) out[(size_t)(q0 + t0 + tt) * C + c0 + cc] = from_f32<T>(s_y[idx]);
      }
    }
  }
  if (live && MODE != 2) {
#pragma unroll
    for (int k = 0; k < MAXS; ++k) {
      const int n = part + k * P;
      if (n < N) st[n] = s[k];
    }
    if (MODE == 1 && part == 0) seg_dt[(size_t)blockIdx.y * C + c] = dt_sum;
  }
}

// grid (ceil(C * N / 256), rows): thread (c, n) turns the segments' end states into their start states, in order
__global__ void scan_combine_kernel(const float* __restrict__ A_log, float* __restrict__ scan_state, float* __restrict__ seg_state,
                                    const float* __restrict__ seg_dt, const int* __restrict__ row_slot,
                                    const int* __restrict__ row_q_len, int C, int N, int segs, int seg_len) {
  const int row = blockIdx.y;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)C * N) return;
  const int c = (int)(i / N);
  const int used = (row_q_len[row] + seg_len - 1) / seg_len;
  float* slot = scan_state + (size_t)row_slot[row] * C * N + i;
  const float a = -expf(A_log[i]);
  float s = *slot;
  for (int g = 0; g < used && g < segs; ++g) {
    float* e = seg_state + ((size_t)(row * segs + g) * C) * N + i;
    const float end = *e;
    *e = s;
    s = fmaf(expf(a * seg_dt[(size_t)(row * segs + g) * C + c]), s, end);
  }
  *slot = s;
}
}  // namespace

extern "C" int dk_conv_silu(const void* xin, int in_stride, const float* w, const float* bias, float* conv_state, void* out,
                            const int* tok_row, const int* row_slot, const int* row_q_start, const int* row_q_len, int T_,
                            int rows, int C, int taps, const float* in_bias, int act, int dtype, cudaStream_t stream) {
  // in_bias [C] (or null) is added to every input as it is read, not to the zeros before a request's first token;
  // act 1: silu behind the convolution, 0: none
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && rows > 0 && C > 0 && in_stride >= C, "conv_silu: bad sizes T=%d rows=%d C=%d stride=%d", T_, rows, C, in_stride);
  DK_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "conv_silu: %d taps; this kernel takes 1 to %d", taps, MAX_TAPS);
  DK_REQUIRE(dtype == DK_F32 || dtype == DK_BF16, "conv_silu: unknown dtype %d", dtype);
  const int threads = C >= 256 ? 256 : 128;
  const dim3 g1(T_, (C + threads - 1) / threads), g2(rows, (C + threads - 1) / threads);
  DK_REQUIRE(g1.y <= 65535, "conv_silu: too many channels");
  if (dtype == DK_F32) {
    conv_silu_kernel<float><<<g1, threads, 0, stream>>>((const float*)xin, in_stride, w, bias, conv_state, (float*)out, tok_row,
                                                        row_slot, row_q_start, C, taps, in_bias, act);
    if (taps > 1)
      conv_state_kernel<float><<<g2, threads, 0, stream>>>((const float*)xin, in_stride, conv_state, row_slot, row_q_start, row_q_len, C, taps, in_bias);
  } else {
    conv_silu_kernel<__nv_bfloat16><<<g1, threads, 0, stream>>>((const __nv_bfloat16*)xin, in_stride, w, bias, conv_state,
                                                                (__nv_bfloat16*)out, tok_row, row_slot, row_q_start, C, taps, in_bias, act);
    if (taps > 1)
      conv_state_kernel<__nv_bfloat16><<<g2, threads, 0, stream>>>((const __nv_bfloat16*)xin, in_stride, conv_state, row_slot,
                                                                   row_q_start, row_q_len, C, taps, in_bias);
  }
  return dk_check_launch("conv_silu");
}

// seg_len > 0: rows longer than seg_len tokens are cut into segments that run in parallel (`segs` = the most segments of
// any row); seg_state holds rows * segs * C * N floats and seg_dt rows * segs * C.  seg_len == 0: every row in one block.
extern "C" int dk_selective_scan(const void* x, const void* dtraw, const void* bc, int bc_stride, int b_off, int c_off,
                                 const void* z, int z_stride, const float* A_log, const float* Dw, const float* dt_bias,
                                 float* scan_state, void* out, const int* row_slot, const int* row_q_start,
                                 const int* row_q_len, int rows, int C, int N, int dtype, int segs, int seg_len, float* seg_state,
                                 float* seg_dt, cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && C > 0 && N > 0, "selective_scan: bad sizes rows=%d C=%d N=%d", rows, C, N);
  DK_REQUIRE(N <= 256, "selective_scan: %d states per channel; this kernel takes up to 256", N);
  DK_REQUIRE(dtype == DK_F32 || dtype == DK_BF16, "selective_scan: unknown dtype %d", dtype);
  const bool cut = seg_len > 0;
  DK_REQUIRE(!cut || (segs >= 1 && seg_len % TT == 0 && seg_state != nullptr && seg_dt != nullptr),
             "selective_scan: segments of %d tokens (a multiple of %d) need their buffers", seg_len, TT);
  if (!cut) segs = 1;
  DK_REQUIRE((long long)rows * segs <= 65535, "selective_scan: too many rows or segments");
#define LAUNCH(T, P, MODE)                                                                                                    \
  do {                                                                                                                        \
    constexpr int CH = 128 / P;                                                                                               \
    const size_t smem = (size_t)(4 * TT * CH + 2 * TT * N) * sizeof(float);                                                  \
    selective_scan_kernel<T, P, 8, MODE><<<dim3((C + CH - 1) / CH, rows * segs), 128, smem, stream>>>(                        \
        (const T*)x, (const T*)dtraw, (const T*)bc, bc_stride, b_off, c_off, (const T*)z, z_stride, A_log, Dw, dt_bias,      \
        scan_state, (T*)out, row_slot, row_q_start, row_q_len, C, N, segs, cut ? seg_len : (1 << 30), seg_state, seg_dt);    \
  } while (0)
#define PICK(T, MODE)                       \
  do {                                      \
    if (N <= 32) LAUNCH(T, 4, MODE);        \
    else if (N <= 64) LAUNCH(T, 8, MODE);   \
    else LAUNCH(T, 32, MODE);               \
  } while (0)
#define BOTH(MODE)                          \
  do {                                      \
    if (dtype == DK_F32) PICK(float, MODE); \
    else PICK(__nv_bfloat16, MODE);         \
  } while (0)
  if (!cut) {
    BOTH(0);
    return dk_check_launch("selective_scan");
  }
  BOTH(1);
  scan_combine_kernel<<<dim3((unsigned)(((size_t)C * N + 255) / 256), rows), 256, 0, stream>>>(A_log, scan_state, seg_state, seg_dt,
                                                                                              row_slot, row_q_len, C, N, segs, seg_len);
  BOTH(2);
#undef BOTH
#undef PICK
#undef LAUNCH
  return dk_check_launch("selective_scan");
}
