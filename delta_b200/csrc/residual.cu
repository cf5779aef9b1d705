// A residual stream of one copy kept in 32 bit, for blocks whose sublayers run side by side:
//
//   embedding_pair   x = table[token] * scale + pair_table[hash(previous token, token)]
//                    (the previous token of a portion's first token comes from the request's state;
//                    a sequence's first token takes the pair table's last row);
//   remember_tokens  leaves every row's last token in that state;
//   residual_norm    the step between two layers, in one pass over the stream:
//                        x <- x + (y1 + y2)      what the last layer's sublayers gave (either may be absent)
//                        x <- x + e              a second 32-bit stream (the embedding output, at a re-entry)
//                        x <- x + vec            one vector for all tokens
//                    then out = norm(x) * w with the layer norm without bias, (x - mean) / sqrt(var + eps), var the
//                    mean of the squared deviations, or the RMS norm x / sqrt(mean(x^2) + eps); w == nullptr: out = x.
//                    A bias b (or null) is added behind the weight.
//                    All sums and statistics are 32 bit; only `out` is rounded to the compute type.
//   sublayer_norm_add  x <- x + norm(y) * w + b: the norm sits on a sublayer's output.
#include "common.cuh"

namespace {

template <typename T>
__global__ void embedding_pair_kernel(const int* __restrict__ tokens, const int* __restrict__ tok_row, const int* __restrict__ tok_pos,
                                      const int* __restrict__ row_q_start, const int* __restrict__ row_slot,
                                      const int* __restrict__ prev_state, const T* __restrict__ table, float scale,
                                      const T* __restrict__ pair_table, long long buckets, long long mul_prev, long long mul_cur,
                                      float* __restrict__ X, float* __restrict__ E, T* __restrict__ R, int d, int vocab, int* err) {
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const bool bad = tok < 0 || tok >= vocab;
  if (bad && threadIdx.x == 0) dk_report(err, DK_DEV_BAD_TOKEN, t, tok, vocab);
  const T* pair = nullptr;
  if (pair_table != nullptr && !bad) {
    const int row = tok_row[t];
    int prev = -1;
    if (tok_pos[t] > 0) prev = (t == row_q_start[row]) ? prev_state[row_slot[row]] : tokens[t - 1];
    long long b = buckets;
    if (prev >= 0) {
      b = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
      if (b < 0) b += buckets;
    }
    pair = pair_table + (size_t)b * d;
  }
  const T* src = table + (size_t)(bad ? 0 : tok) * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = bad ? 0.f : to_f32<T>(src[i]) * scale;
    if (pair != nullptr) v += to_f32<T>(pair[i]);
    X[(size_t)t * d + i] = v;
    if (E != nullptr) E[(size_t)t * d + i] = v;
    if (R != nullptr) R[(size_t)t * d + i] = from_f32<T>(v);      // the stream in the compute type, for a first sublayer that reads it
  }
}

__global__ void remember_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ row_q_start,
                                       const int* __restrict__ row_q_len, const int* __restrict__ row_slot, int* __restrict__ prev_state,
                                       int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < rows && row_q_len[r] > 0) prev_state[row_slot[r]] = tokens[row_q_start[r] + row_q_len[r] - 1];
}

// One block per output row r (token tk = rows ? rows[r] : r); the settled row is kept in shared memory between the passes.
template <typename T, typename TO>
__global__ void residual_norm_kernel(float* __restrict__ X, const T* __restrict__ y1, const T* __restrict__ y2, const float* __restrict__ e,
                                     const float* __restrict__ vec, const float* __restrict__ w, const float* __restrict__ b,
                                     TO* __restrict__ out, const int* __restrict__ rows, int d, float eps, int kind, int write_back) {
  extern __shared__ __align__(16) float xs[];   // d floats + 33
  float* scratch = xs + d;
  const int r = blockIdx.x;
  const int tk = rows ? rows[r] : r;
  float* x = X + (size_t)tk * d;
  float sum = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = x[i];
    if (y1 != nullptr) {
      float u = to_f32<T>(y1[(size_t)tk * d + i]);
      if (y2 != nullptr) u += to_f32<T>(y2[(size_t)tk * d + i]);
      v += u;
    }
    if (e != nullptr) v += e[(size_t)tk * d + i];
    if (vec != nullptr) v += vec[i];
    if (write_back) x[i] = v;
    xs[i] = v;
    sum += v;
  }
  if (out == nullptr) return;
  TO* o = out + (size_t)r * d;
  if (w == nullptr) {
    __syncthreads();
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f32<TO>(xs[i]);
    return;
  }
  float mean = 0.f;
  if (kind == 1) mean = block_sum(sum, scratch) / (float)d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float c = xs[i] - mean;
    ss += c * c;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f32<TO>((xs[i] - mean) * inv * w[i] + (b != nullptr ? b[i] : 0.f));
}

// The step behind a sublayer whose OUTPUT is normed (the sublayer itself read the stream as it was):
//     x <- x + norm(y) * w + b
// with the layer norm or the RMS norm of the sublayer's output y over the width and a bias b (or null), all in 32 bit; `out` (or null) takes the new x rounded to the compute type, for the next sublayer to read.
template <typename T, typename TO>
__global__ void sublayer_norm_add_kernel(float* __restrict__ X, const T* __restrict__ y, const float* __restrict__ w,
                                         const float* __restrict__ b, TO* __restrict__ out, int d, float eps, int kind) {
  extern __shared__ __align__(16) float ys[];   // d floats + 34
  float* scratch = ys + d;
  const size_t at = (size_t)blockIdx.x * d;
  float sum = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = to_f32<T>(y[at + i]);
    ys[i] = v;
    sum += v;
  }
  float mean = 0.f;
  if (kind == 1) mean = block_sum(sum, scratch) / (float)d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float c = ys[i] - mean;
    ss += c * c;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = X[at + i] + ((ys[i] - mean) * inv * w[i] + (b != nullptr ? b[i] : 0.f));
    X[at + i] = v;
    if (out != nullptr) out[at + i] = from_f32<TO>(v);
  }
}

// out = factor * sum over the branches k of  rms_norm(y_k + b_k) * w_k : sublayers that run side by side, each normed over the
// width with its own weight before they are summed.  One block per token, all in 32 bit.
__global__ void normed_sum_kernel(const float* __restrict__ y1, const float* __restrict__ b1, const float* __restrict__ w1,
                                  const float* __restrict__ y2, const float* __restrict__ b2, const float* __restrict__ w2,
                                  float* __restrict__ out, int d, float eps, float factor) {
  extern __shared__ __align__(16) float xs[];   // 2 d floats + 33
  float* scratch = xs + 2 * d;
  const size_t at = (size_t)blockIdx.x * d;
  float s1 = 0.f, s2 = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float a = y1[at + i] + (b1 ? b1[i] : 0.f);
    const float b = y2 ? y2[at + i] + (b2 ? b2[i] : 0.f) : 0.f;
    xs[i] = a;
    xs[d + i] = b;
    s1 += a * a;
    s2 += b * b;
  }
  s1 = block_sum(s1, scratch);
  s2 = block_sum(s2, scratch);
  const float i1 = 1.f / sqrtf(s1 / (float)d + eps), i2 = 1.f / sqrtf(s2 / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = xs[i] * i1 * w1[i];
    if (y2) v += xs[d + i] * i2 * w2[i];
    out[at + i] = factor * v;
  }
}

}  // namespace

extern "C" int dk_normed_sum(const float* y1, const float* b1, const float* w1, const float* y2, const float* b2, const float* w2,
                             float* out, int T_, int d, float eps, float factor, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && d > 0 && d <= 12000, "normed_sum: bad sizes T=%d d=%d (width up to 12000)", T_, d);
  DK_REQUIRE(y1 != nullptr && w1 != nullptr && (y2 == nullptr || w2 != nullptr), "normed_sum: a branch without its weight");
  const int threads = d >= 4096 ? 512 : (d >= 1024 ? 256 : 128);
  const size_t smem = (size_t)(2 * d + 36) * sizeof(float);
  if (smem > 48 * 1024) {
    static bool granted[DK_MAX_DEVICES] = {false};
    const int dev = dk_current_device();
    if (!granted[dev]) {
      if (cudaFuncSetAttribute(normed_sum_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (2 * 12000 + 36) * 4) != cudaSuccess) {
        cudaGetLastError();
        DK_REQUIRE(false, "normed_sum: %zu bytes of shared memory were not granted", smem);
      }
      granted[dev] = true;
    }
  }
  normed_sum_kernel<<<T_, threads, smem, stream>>>(y1, b1, w1, y2, b2, w2, out, d, eps, factor);
  return dk_check_launch("normed_sum");
}

extern "C" int dk_embedding_pair(const int* tokens, const int* tok_row, const int* tok_pos, const int* row_q_start, const int* row_slot,
                                 int* prev_state, const void* table, float scale, const void* pair_table, long long buckets,
                                 long long mul_prev, long long mul_cur, float* X, float* E, void* R, int T_, int d, int vocab, int dtype, int* err,
                                 cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && d > 0 && vocab > 0, "embedding_pair: bad sizes T=%d d=%d vocab=%d", T_, d, vocab);
  DK_REQUIRE(pair_table == nullptr || (buckets > 0 && prev_state != nullptr), "embedding_pair: a pair table needs buckets and the state of previous tokens");
  const int threads = d >= 1024 ? 256 : 128;
#define LAUNCH(T)                                                                                                               \
  embedding_pair_kernel<T><<<T_, threads, 0, stream>>>(tokens, tok_row, tok_pos, row_q_start, row_slot, prev_state, (const T*)table, \
                                                        scale, (const T*)pair_table, buckets, mul_prev, mul_cur, X, E, (T*)R, d, vocab, err)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "embedding_pair: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("embedding_pair");
}

extern "C" int dk_remember_tokens(const int* tokens, const int* row_q_start, const int* row_q_len, const int* row_slot, int* prev_state,
                                  int rows, cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && prev_state != nullptr, "remember_tokens: bad arguments rows=%d", rows);
  remember_tokens_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(tokens, row_q_start, row_q_len, row_slot, prev_state, rows);
  return dk_check_launch("remember_tokens");
}

extern "C" int dk_residual_norm(float* X, const void* y1, const void* y2, const float* e, const float* vec, const float* w, const float* b,
                                void* out, const int* rows, int n_rows, int d, float eps, int kind, int write_back, int y_dtype, int out_dtype,
                                cudaStream_t stream) {
  if (n_rows == 0) return 0;
  DK_REQUIRE(n_rows > 0 && d > 0, "residual_norm: bad sizes rows=%d d=%d", n_rows, d);
  DK_REQUIRE(d <= 12000, "residual_norm: width %d is above the 12000 this kernel keeps in shared memory", d);
  DK_REQUIRE(kind == 0 || kind == 1, "residual_norm: unknown norm kind %d", kind);
  DK_REQUIRE(y2 == nullptr || y1 != nullptr, "residual_norm: a second update is given without a first");
  const int threads = d >= 4096 ? 512 : (d >= 1024 ? 256 : 128);
  const size_t smem = (size_t)(d + 36) * sizeof(float);
#define LAUNCH(T, TO)                                                                                                          \
  residual_norm_kernel<T, TO><<<n_rows, threads, smem, stream>>>(X, (const T*)y1, (const T*)y2, e, vec, w, b, (TO*)out, rows, d, eps, \
                                                                 kind, write_back)
  if (y_dtype == DK_F32 && out_dtype == DK_F32) LAUNCH(float, float);
  else if (y_dtype == DK_BF16 && out_dtype == DK_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (y_dtype == DK_BF16 && out_dtype == DK_F32) LAUNCH(__nv_bfloat16, float);
  else if (y_dtype == DK_F32 && out_dtype == DK_BF16) LAUNCH(float, __nv_bfloat16);
  else DK_REQUIRE(false, "residual_norm: unsupported dtypes y=%d out=%d", y_dtype, out_dtype);
#undef LAUNCH
  return dk_check_launch("residual_norm");
}

// The same for a width that is a multiple of 8 with 16-byte aligned rows: a thread keeps V groups of eight entries of y and of
// x in registers from the start, so every load of the block is under way before the first sum is needed, and nothing is staged
// in shared memory.
template <typename T, typename TO, int V>
__global__ void sublayer_norm_add_vec_kernel(float* __restrict__ X, const T* __restrict__ y, const float* __restrict__ w,
                                             const float* __restrict__ b, TO* __restrict__ out, int d, float eps, int kind) {
  __shared__ float scratch[34];
  const size_t at = (size_t)blockIdx.x * d;
  const int groups = d / 8;
  float yv[V][8], xv[V][8];
  float sum = 0.f;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int c = threadIdx.x + v * blockDim.x;
    if (c < groups) {
      load8<T>(y + at + (size_t)c * 8, yv[v]);
      load8<float>(X + at + (size_t)c * 8, xv[v]);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += yv[v][e];
    }
  }
  float mean = 0.f;
  if (kind == 1) mean = block_sum(sum, scratch) / (float)d;
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int c = threadIdx.x + v * blockDim.x;
    if (c < groups) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        yv[v][e] -= mean;
        ss += yv[v][e] * yv[v][e];
      }
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)d + eps);
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int c = threadIdx.x + v * blockDim.x;
    if (c < groups) {
      float wv[8], bv[8];
      load8<float>(w + (size_t)c * 8, wv);
      if (b != nullptr) load8<float>(b + (size_t)c * 8, bv);
#pragma unroll
      for (int e = 0; e < 8; ++e) xv[v][e] += yv[v][e] * inv * wv[e] + (b != nullptr ? bv[e] : 0.f);
      store8<float>(X + at + (size_t)c * 8, xv[v]);
      if (out != nullptr) store8<TO>(out + at + (size_t)c * 8, xv[v]);
    }
  }
}

extern "C" int dk_sublayer_norm_add(float* X, const void* y, const float* w, const float* b, void* out, int T_, int d,
                                    float eps, int kind, int y_dtype, int out_dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && d > 0, "sublayer_norm_add: bad sizes T=%d d=%d", T_, d);
  DK_REQUIRE(d <= 12000, "sublayer_norm_add: width %d is above the 12000 this kernel keeps in shared memory", d);
  DK_REQUIRE(kind == 0 || kind == 1, "sublayer_norm_add: unknown norm kind %d", kind);
  DK_REQUIRE(w != nullptr, "sublayer_norm_add: the norm has no weight");
  const int threads = d >= 4096 ? 512 : (d >= 1024 ? 256 : 128);
  const size_t smem = (size_t)(d + 36) * sizeof(float);
  auto aligned = [](const void* q) { return q == nullptr || ((uintptr_t)q % 16) == 0; };
  const int groups = d / 8;
  const bool vec = d % 8 == 0 && groups <= 2048 && aligned(X) && aligned(y) && aligned(w) && aligned(b) && aligned(out);
  const int vthreads = groups <= 1024 ? (groups + 31) / 32 * 32 : 1024;      // one group of eight a thread up to a width of 8,192, then two
#define LAUNCH(T, TO)                                                                                                             \
  do {                                                                                                                            \
    if (vec && groups <= 1024) sublayer_norm_add_vec_kernel<T, TO, 1><<<T_, vthreads, 0, stream>>>(X, (const T*)y, w, b, (TO*)out, d, eps, kind); \
    else if (vec) sublayer_norm_add_vec_kernel<T, TO, 2><<<T_, vthreads, 0, stream>>>(X, (const T*)y, w, b, (TO*)out, d, eps, kind); \
    else sublayer_norm_add_kernel<T, TO><<<T_, threads, smem, stream>>>(X, (const T*)y, w, b, (TO*)out, d, eps, kind);           \
  } while (0)
  if (y_dtype == DK_F32 && out_dtype == DK_F32) LAUNCH(float, float);
  else if (y_dtype == DK_BF16 && out_dtype == DK_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (y_dtype == DK_BF16 && out_dtype == DK_F32) LAUNCH(__nv_bfloat16, float);
  else if (y_dtype == DK_F32 && out_dtype == DK_BF16) LAUNCH(float, __nv_bfloat16);
  else DK_REQUIRE(false, "sublayer_norm_add: unsupported dtypes y=%d out=%d", y_dtype, out_dtype);
#undef LAUNCH
  return dk_check_launch("sublayer_norm_add");
}
