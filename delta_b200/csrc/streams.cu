// A residual stream kept in 32 bit, as one copy or as several mixed copies ("hyper-connections"),
// with the kernels that read and write it:
//
//   embedding into S equal copies;
//   the fused  [update of the copies by the last sublayer's output] -> [weighted sum of the copies] -> RMSNorm,
//   which is what stands between two sublayers, so the copies are read and written once per sublayer;
//   the update alone (for callers that want the stream settled);
//   element-wise activations of a feed-forward and the soft cap of logits.
//
// With copies X_1..X_S of a token (each d floats), a sublayer with weights in[S], out[S], mix[S][S] does
//   u    = sum_s in[s] X_s                      (what the sublayer's norm reads)
//   y    = sublayer(norm(u))
//   X_t <- sum_s mix[s][t] X_s + out[t] y       (all t at once, from the old copies)
// One copy with in = out = mix = 1 is the ordinary residual sum.
#include "common.cuh"

namespace {
constexpr int MAX_STREAMS = 8;

template <typename T>
__global__ void embedding_streams_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ X,
                                         int S, int d, int vocab, int* err) {
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const bool bad = tok < 0 || tok >= vocab;
  if (bad && threadIdx.x == 0) dk_report(err, DK_DEV_BAD_TOKEN, t, tok, vocab);
  const T* src = table + (size_t)(bad ? 0 : tok) * d;
  float* dst = X + (size_t)t * S * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = bad ? 0.f : to_f32<T>(src[i]);
    for (int s = 0; s < S; ++s) dst[(size_t)s * d + i] = v;
  }
}

// One block per output row r (token tk = rows ? rows[r] : r).
//   y != nullptr: the copies of the token are updated with (mix, outw, y) first; write_back stores them.
//   u = sum_s inw[s] X_s (inw == nullptr: the plain sum); out[r] = u * rsqrt(mean(u^2) + eps) * w.
//   w == nullptr: out[r] = u, not normalised.
template <typename T, typename TO>
__global__ void stream_norm_kernel(float* __restrict__ X, const T* __restrict__ y, const float* __restrict__ mix,
                                   const float* __restrict__ outw, const float* __restrict__ inw, const float* __restrict__ w,
                                   TO* __restrict__ out, const int* __restrict__ rows, int S, int d, float eps, int write_back) {
  extern __shared__ __align__(16) float usm[];   // d floats + 33
  float* scratch = usm + d;
  __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_out[MAX_STREAMS], s_in[MAX_STREAMS];
  const int r = blockIdx.x;
  const int tk = rows ? rows[r] : r;
  if (threadIdx.x < S * S) s_mix[threadIdx.x] = mix ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    s_out[threadIdx.x] = outw ? outw[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = inw ? inw[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float* xs = X + (size_t)tk * S * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) v[s] = s < S ? xs[(size_t)s * d + i] : 0.f;
    if (y != nullptr) {
      const float yv = to_f32<T>(y[(size_t)tk * d + i]);
      float n[MAX_STREAMS];
#pragma unroll
      for (int t2 = 0; t2 < MAX_STREAMS; ++t2) {
        if (t2 < S) {
          float a = 0.f;
#pragma unroll
          for (int s = 0; s < MAX_STREAMS; ++s)
            if (s < S) a = fmaf(s_mix[s * S + t2], v[s], a);
          n[t2] = fmaf(s_out[t2], yv, a);
        }
      }
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) {
          v[s] = n[s];
          if (write_back) xs[(size_t)s * d + i] = n[s];
        }
    }
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s)
      if (s < S) u = fmaf(s_in[s], v[s], u);
    usm[i] = u;
    ss += u * u;
  }
  if (out == nullptr) return;
  TO* o = out + (size_t)r * d;
  if (w == nullptr) {
    __syncthreads();
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f32<TO>(usm[i]);
    return;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f32<TO>(usm[i] * inv * w[i]);
}

// The same for a width that is a multiple of 4 and a compile-time number of copies: 16-byte loads and stores, all
// copies of four neighbouring entries in registers at once.
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&a);
  raw.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T, typename TO, int S>
__global__ void stream_norm_vec_kernel(float* __restrict__ X, const T* __restrict__ y, const float* __restrict__ mix,
                                       const float* __restrict__ outw, const float* __restrict__ inw, const float* __restrict__ w,
                                       TO* __restrict__ out, const int* __restrict__ rows, int d, float eps, int write_back) {
  extern __shared__ __align__(16) float usm[];   // d floats + 33
  float* scratch = usm + d;
  const int r = blockIdx.x;
  const int tk = rows ? rows[r] : r;
  float c_mix[S][S], c_out[S], c_in[S];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    c_out[s] = outw ? outw[s] : 0.f;
    c_in[s] = inw ? inw[s] : 1.f;
#pragma unroll
    for (int t2 = 0; t2 < S; ++t2) c_mix[s][t2] = mix ? mix[s * S + t2] : 0.f;
  }
  float* xs = X + (size_t)tk * S * d;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
    float4 v[S];
#pragma unroll
    for (int s = 0; s < S; ++s) v[s] = *reinterpret_cast<const float4*>(xs + (size_t)s * d + i);
    if (y != nullptr) {
      const float4 yv = load4<T>(y + (size_t)tk * d + i);
      float4 n[S];
#pragma unroll
      for (int t2 = 0; t2 < S; ++t2) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < S; ++s) {
          a.x = fmaf(c_mix[s][t2], v[s].x, a.x);
          a.y = fmaf(c_mix[s][t2], v[s].y, a.y);
          a.z = fmaf(c_mix[s][t2], v[s].z, a.z);
          a.w = fmaf(c_mix[s][t2], v[s].w, a.w);
        }
        n[t2] = make_float4(fmaf(c_out[t2], yv.x, a.x), fmaf(c_out[t2], yv.y, a.y), fmaf(c_out[t2], yv.z, a.z), fmaf(c_out[t2], yv.w, a.w));
      }
#pragma unroll
      for (int s = 0; s < S; ++s) {
        v[s] = n[s];
        if (write_back) *reinterpret_cast<float4*>(xs + (size_t)s * d + i) = n[s];
      }
    }
    float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < S; ++s) {
      u.x = fmaf(c_in[s], v[s].x, u.x);
      u.y = fmaf(c_in[s], v[s].y, u.y);
      u.z = fmaf(c_in[s], v[s].z, u.z);
      u.w = fmaf(c_in[s], v[s].w, u.w);
    }
    *reinterpret_cast<float4*>(usm + i) = u;
    ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
  }
  if (out == nullptr) return;
  TO* o = out + (size_t)r * d;
  float inv = 1.f;
  if (w != nullptr) {
    ss = block_sum(ss, scratch);
    inv = 1.f / sqrtf(ss / (float)d + eps);
  }
  for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
    const float4 u = *reinterpret_cast<const float4*>(usm + i);
    const float4 wv = w != nullptr ? *reinterpret_cast<const float4*>(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
    store4<TO>(o + i, make_float4(u.x * inv * wv.x, u.y * inv * wv.y, u.z * inv * wv.z, u.w * inv * wv.w));
  }
}

// kind 0: relu(x)^2; 1: gelu with the tanh form; 2: silu.  Computed in float, rounded once.
template <typename T>
__global__ void activation_kernel(const T* __restrict__ in, T* __restrict__ out, size_t n, int kind) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float z = to_f32<T>(in[i]);
    float r;
    if (kind == 0) {
      const float p = fmaxf(z, 0.f);
      r = p * p;
    } else if (kind == 1) {
      r = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    } else {
      r = z / (1.f + expf(-z));
    }
    out[i] = from_f32<T>(r);
  }
}

// x <- x * scale, then x <- cap * tanh(x / cap) (cap <= 0: no cap)
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap, float scale) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = x[i] * scale;
    x[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

int grid_for(size_t n, int threads) {
  size_t b = (n + threads - 1) / threads;
  const size_t most = (size_t)dk_sm_count() * 16;
  return (int)(b < 1 ? 1 : (b > most ? most : b));
}
}  // namespace

extern "C" int dk_embedding_streams(const int* tokens, const void* table, float* X, int T_, int S, int d, int vocab, int dtype,
                                    int* err, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && d > 0 && vocab > 0 && S >= 1, "embedding_streams: bad sizes T=%d S=%d d=%d vocab=%d", T_, S, d, vocab);
  const int threads = d >= 1024 ? 256 : 128;
  if (dtype == DK_F32)
    embedding_streams_kernel<float><<<T_, threads, 0, stream>>>(tokens, (const float*)table, X, S, d, vocab, err);
  else if (dtype == DK_BF16)
    embedding_streams_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(tokens, (const __nv_bfloat16*)table, X, S, d, vocab, err);
  else
    DK_REQUIRE(false, "embedding_streams: unknown dtype %d", dtype);
  return dk_check_launch("embedding_streams");
}

extern "C" int dk_stream_norm(float* X, const void* y, const float* mix, const float* outw, const float* inw, const float* w,
                              void* out, const int* rows, int n_rows, int S, int d, float eps, int write_back, int y_dtype,
                              int out_dtype, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  DK_REQUIRE(n_rows > 0 && d > 0, "stream_norm: bad sizes rows=%d d=%d", n_rows, d);
  DK_REQUIRE(S >= 1 && S <= MAX_STREAMS, "stream_norm: %d copies of the stream; this kernel takes 1 to %d", S, MAX_STREAMS);
  DK_REQUIRE(d <= 12000, "stream_norm: width %d is above the 12000 this kernel keeps in shared memory", d);
  DK_REQUIRE(y == nullptr || (mix != nullptr && outw != nullptr), "stream_norm: an update is given without its weights");
  const int threads = d >= 4096 ? 512 : (d >= 1024 ? 256 : 128);
  const size_t smem = (size_t)(d + 36) * sizeof(float);
  const bool vec = (d % 4) == 0 && (S == 1 || S == 2 || S == 4) && ((uintptr_t)X % 16) == 0 && ((uintptr_t)y % 8) == 0 &&
                   ((uintptr_t)out % 8) == 0 && ((uintptr_t)w % 16) == 0;
#define VEC(T, TO, SS) \
  stream_norm_vec_kernel<T, TO, SS><<<n_rows, threads, smem, stream>>>(X, (const T*)y, mix, outw, inw, w, (TO*)out, rows, d, eps, write_back)
#define LAUNCH(T, TO)                                                                                                            \
  do {                                                                                                                           \
    if (vec && S == 1) VEC(T, TO, 1);                                                                                            \
    else if (vec && S == 2) VEC(T, TO, 2);                                                                                       \
    else if (vec && S == 4) VEC(T, TO, 4);                                                                                       \
    else                                                                                                                         \
      stream_norm_kernel<T, TO><<<n_rows, threads, smem, stream>>>(X, (const T*)y, mix, outw, inw, w, (TO*)out, rows, S, d, eps, \
                                                                   write_back);                                                  \
  } while (0)
  if (y_dtype == DK_F32 && out_dtype == DK_F32) LAUNCH(float, float);
  else if (y_dtype == DK_BF16 && out_dtype == DK_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (y_dtype == DK_BF16 && out_dtype == DK_F32) LAUNCH(__nv_bfloat16, float);
  else DK_REQUIRE(false, "stream_norm: unsupported dtypes y=%d out=%d", y_dtype, out_dtype);
#undef LAUNCH
#undef VEC
  return dk_check_launch("stream_norm");
}

extern "C" int dk_activation(const void* in, void* out, long long n, int kind, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  DK_REQUIRE(n > 0 && kind >= 0 && kind <= 2, "activation: bad arguments n=%lld kind=%d", n, kind);
  const int threads = 256;
  const int blocks = grid_for((size_t)n, threads);
  if (dtype == DK_F32) activation_kernel<float><<<blocks, threads, 0, stream>>>((const float*)in, (float*)out, (size_t)n, kind);
  else if (dtype == DK_BF16)
    activation_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, (size_t)n, kind);
  else DK_REQUIRE(false, "activation: unknown dtype %d", dtype);
  return dk_check_launch("activation");
}

extern "C" int dk_softcap(float* x, long long n, float cap, float scale, cudaStream_t stream) {
  if (n == 0) return 0;
  DK_REQUIRE(n > 0 && (cap > 0.f || scale != 1.f), "softcap: bad arguments n=%lld cap=%g scale=%g", n, cap, scale);
  softcap_kernel<<<grid_for((size_t)n, 256), 256, 0, stream>>>(x, (size_t)n, cap, scale);
  return dk_check_launch("softcap");
}
