// Paged attention over a cache of rows (see row_attention_params.h), in its plain form, and the kernels
// that fill such a cache.
//
// The plain kernel takes every size and both element types with float arithmetic throughout: one block
// per (token, head), causal, optionally a sliding window, optionally a sink in the softmax.  The faster
// kernels of this family are checked against it.
//
//   s_j  = (q . k_j) * scale          for the visible keys  max(0, i - window + 1) <= j <= i
//   s_j <- softcap * tanh(s_j / softcap)                      (softcap > 0)
//   s_j <- s_j + dist_bias[h][min(i - j, dist_max)]           (a table of biases by distance, one row a head)
//   p_j  = exp(s_j) / (sum_j' exp(s_j') [+ exp(sink_h)])
//   y    = sum_j p_j v_j
#include "common.cuh"
#include "row_attention_params.h"

extern "C" int dk_sizeof_row_attn_params() { return (int)sizeof(DkRowAttnParams); }

namespace {
constexpr int CH = 128;        // key slots per pass = threads per block
constexpr int MAX_DV = 1024;   // value size the plain kernel takes

template <typename T>
__global__ void __launch_bounds__(CH) attention_rows_plain_kernel(const DkRowAttnParams p) {
  extern __shared__ float smem[];
  float* qs = smem;                 // dk
  float* sc = qs + p.dk;            // CH
  float* scratch = sc + CH;         // 34
  long long* voff = (long long*)(scratch + 34 + ((p.dk + CH + 34) & 1));   // CH, 8-byte aligned
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int row = p.tok_row[t], pos = p.tok_pos[t];
  const int dk = p.dk, dv = p.dv, ps = p.ps, KV = p.KV;
  const int g = h / (p.H / KV);
  const T* q = (const T*)p.q + (size_t)t * p.q_stride + (size_t)h * p.q_head_stride;
  const T* cache = (const T*)p.cache;
  for (int i = tid; i < dk; i += CH) qs[i] = to_f32<T>(q[i]);
  const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  const int first_page = lo / ps;
  const int n_entries = pos / ps - first_page + 1;

  float m = -INFINITY, l = 0.f;
  if (p.sink != nullptr) {      // the sink: a key with this logit and no value
    m = p.sink[h];
    l = 1.f;
  }
  float acc[MAX_DV / CH];
#pragma unroll
  for (int dd = 0; dd < MAX_DV / CH; ++dd) acc[dd] = 0.f;
  const int pages_per_pass = CH / ps;
  __syncthreads();

  for (int e0 = 0; e0 < n_entries; e0 += pages_per_pass) {
    const int e = e0 + tid / ps, off = tid % ps;
    float s = -INFINITY;
    long long vo = -1;
    if (e < n_entries) {
      const int lp = first_page + e;
      const int key = lp * ps + off;
      if (lp < p.max_pages && key >= lo && key <= pos) {
        const int page = p.block_table[(size_t)row * p.max_pages + lp];
        if (page < 0 || page >= p.num_pages) {
          dk_report(p.err, DK_DEV_BAD_PAGE, t, lp, page);
        } else {
          const size_t base = (((size_t)page * KV + g) * ps + off) * p.row_width;
          const T* kr = cache + base + p.k_off;
          float d = 0.f;
          for (int i = 0; i < dk; ++i) d = fmaf(qs[i], to_f32<T>(kr[i]), d);
          s = d * p.scale;
          if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
          if (p.dist_bias != nullptr) s += p.dist_bias[(size_t)h * (p.dist_max + 1) + min(pos - key, p.dist_max)];
          vo = (long long)(base + p.v_off);
        }
      }
    }
    voff[tid] = vo;
    const float cmax = block_max(s, scratch);
    if (cmax == -INFINITY) {
      __syncthreads();
      continue;
    }
    const float m_new = fmaxf(m, cmax);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float pr = (vo >= 0) ? expf(s - m_new) : 0.f;
    sc[tid] = pr;
    const float psum = block_sum(pr, scratch);
    l = l * corr + psum;
    m = m_new;
#pragma unroll
    for (int dd = 0; dd < MAX_DV / CH; ++dd) {
      const int d = tid + dd * CH;
      if (d < dv) {
        float a = acc[dd] * corr;
        for (int k = 0; k < CH; ++k) {
          const long long o = voff[k];
          if (o >= 0) a = fmaf(sc[k], to_f32<T>(cache[o + d]), a);
        }
        acc[dd] = a;
      }
    }
    __syncthreads();
  }
  T* out = (T*)p.out + ((size_t)t * p.H + h) * dv;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int dd = 0; dd < MAX_DV / CH; ++dd) {
    const int d = tid + dd * CH;
    if (d < dv) out[d] = from_f32<T>(acc[dd] * inv);
  }
}

// The page and offset a token is appended at; -1 with an error record when the table has none.
__device__ __forceinline__ long long row_slot_of(const int* block_table, int max_pages, int num_pages, int b, int pos, int ps, int t,
                                                 int* err) {
  const int lp = pos / ps;
  const int page = lp < max_pages ? block_table[(size_t)b * max_pages + lp] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) dk_report(err, DK_DEV_BAD_PAGE, t, lp, page);
    return -1;
  }
  return (long long)page * ps + pos % ps;
}

// Pair j of the first rot_dims entries of a head: entries (2j, 2j+1) when interleaved, else (j, j + rot_dims/2).
__device__ __forceinline__ void pair_index(int j, int rot_dims, int interleaved, int& i0, int& i1) {
  i0 = interleaved ? 2 * j : j;
  i1 = interleaved ? 2 * j + 1 : j + rot_dims / 2;
}

// src[t] = [q (H*dk) | k (KV*dk) | v (KV*dv)].  q and k get rotary positions on their first rot_dims entries
// (table == nullptr: none), q in place; k and v go to the token's cache rows.
template <typename T>
__global__ void rows_append_kernel(T* __restrict__ src, int src_stride, const int* __restrict__ tok_pos, const int* __restrict__ tok_row,
                                   const int* __restrict__ block_table, int max_pages, T* __restrict__ cache, int num_pages,
                                   const float* __restrict__ table, int table_positions, int rot_dims, int interleaved, int H,
                                   int KV, int dk, int dv, int ps, int row_width, int k_off, int v_off, int* err) {
  const int t = blockIdx.x;
  const int pos = tok_pos[t], b = tok_row[t];
  T* base = src + (size_t)t * src_stride;
  if (pos < 0 || (table != nullptr && pos >= table_positions)) {
    if (threadIdx.x == 0) dk_report(err, DK_DEV_BAD_POSITION, t, pos, table_positions);
    return;
  }
  const long long at = cache != nullptr ? row_slot_of(block_table, max_pages, num_pages, b, pos, ps, t, err) : -1;
  const int half = rot_dims / 2;
  if (table != nullptr) {
    const float* cs = table + (size_t)pos * half * 2;
    for (int idx = threadIdx.x; idx < (H + KV) * half; idx += blockDim.x) {
      const int hs = idx / half, j = idx - hs * half;
      int i0, i1;
      pair_index(j, rot_dims, interleaved, i0, i1);
      T* hp = base + (size_t)hs * dk;
      const float u = to_f32<T>(hp[i0]), v = to_f32<T>(hp[i1]);
      const float c = cs[2 * j], s = cs[2 * j + 1];
      hp[i0] = from_f32<T>(u * c - v * s);
      hp[i1] = from_f32<T>(v * c + u * s);
    }
    __syncthreads();
  }
  if (at < 0) return;
  const long long page = at / ps, off = at % ps;
  const T* ksrc = base + (size_t)H * dk;
  const T* vsrc = ksrc + (size_t)KV * dk;
  for (int idx = threadIdx.x; idx < KV * dk; idx += blockDim.x) {
    const int g = idx / dk, i = idx - g * dk;
    cache[(((size_t)page * KV + g) * ps + off) * row_width + k_off + i] = ksrc[idx];
  }
  for (int idx = threadIdx.x; idx < KV * dv; idx += blockDim.x) {
    const int g = idx / dv, i = idx - g * dv;
    cache[(((size_t)page * KV + g) * ps + off) * row_width + v_off + i] = vsrc[idx];
  }
}

// The same step for designs that norm queries and keys: src[t] = [q (H*dk) | k (KV*dk) | v (KV*dv), absent when the
// value is the key].  One warp per head: the head is read into 32-bit shared memory, rotated on its first rot_dims
// entries (table == nullptr: not), then divided by its root mean square over dk, sqrt(mean(x^2) + eps) (unit_norm == 0:
// not), and rounded once.  q goes back in place, k to the cache row.  value_from_key: the value is the key as
// projected, before rotation and norm (its first dv entries), so no v is read.  bias (32 bit, laid out as a row of src) is
// added to q, k and v as they are read.  q_norm / k_norm [dk]: before the rotation the head is RMS-normed with this
// weight, x / sqrt(mean(x^2) + pre_eps) * w, the same weight for every head; norm_whole: the mean is taken over all columns of
// q (and of k) at once and the weights are [H*dk] and [KV*dk].  temp_every > 0: the query is multiplied by
// 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1).  KV may be 0 (no cache): src holds queries only.
template <typename T>
__global__ void rows_append_unit_kernel(T* __restrict__ src, int src_stride, const int* __restrict__ tok_pos, const int* __restrict__ tok_row,
                                        const int* __restrict__ block_table, int max_pages, T* __restrict__ cache, int num_pages,
                                        const float* __restrict__ table, int table_positions, int rot_dims, int interleaved, int H,
                                        int KV, int dk, int dv, int ps, int row_width, int k_off, int v_off, int unit_norm, float eps,
                                        int value_from_key, const float* __restrict__ bias, const float* __restrict__ q_norm,
                                        const float* __restrict__ k_norm, float pre_eps, int norm_whole, float temp_coef, int temp_every,
                                        int* err) {
  extern __shared__ float heads[];     // [warps][dk] (norm_whole: and 34 behind them)
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int pos = tok_pos[t], b = tok_row[t];
  T* base = src + (size_t)t * src_stride;
  if (pos < 0 || (table != nullptr && pos >= table_positions)) {
    if (threadIdx.x == 0) dk_report(err, DK_DEV_BAD_POSITION, t, pos, table_positions);
    return;
  }
  const long long at = cache != nullptr ? row_slot_of(block_table, max_pages, num_pages, b, pos, ps, t, err) : -1;
  const long long page = at >= 0 ? at / ps : 0, off = at >= 0 ? at % ps : 0;
  const int half = rot_dims / 2;
  float* x = heads + (size_t)warp * dk;
  float whole_q = 0.f, whole_k = 0.f;      // norm_whole: 1 / rms over all of q's columns, and over all of k's
  if (norm_whole) {
    float* scratch = heads + (size_t)warps * dk;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < (H + KV) * dk; i += blockDim.x) {
      const float v = to_f32<T>(base[i]) + (bias != nullptr ? bias[i] : 0.f);
      if (i < H * dk) sq += v * v;
      else sk += v * v;
    }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    whole_q = 1.f / sqrtf(sq / (float)(H * dk) + pre_eps);
    if (KV > 0) whole_k = 1.f / sqrtf(sk / (float)(KV * dk) + pre_eps);
  }
  // the factor on a query by its position: 1 + coef * ln(floor((pos + 1) / every) + 1)
  const float temp = temp_every > 0 ? 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f) : 1.f;
  for (int hs = warp; hs < H + KV; hs += warps) {
    T* hp = base + (size_t)hs * dk;
    const bool is_key = hs >= H;
    T* crow = (is_key && at >= 0) ? cache + (((size_t)page * KV + (hs - H)) * ps + off) * row_width : nullptr;
    float ss0 = 0.f;
    for (int i = lane; i < dk; i += 32) {
      const T raw = hp[i];
      const float v = to_f32<T>(raw) + (bias != nullptr ? bias[(size_t)hs * dk + i] : 0.f);
      x[i] = v;
      ss0 += v * v;
      if (crow != nullptr && value_from_key && i < dv) crow[v_off + i] = bias != nullptr ? from_f32<T>(v) : raw;
    }
    const float* pre_w = is_key ? k_norm : q_norm;
    if (pre_w != nullptr) {      // the RMS norm with a weight, before the rotation: over the head, or over all heads at once
      const float pre = norm_whole ? (is_key ? whole_k : whole_q) : 1.f / sqrtf(warp_sum(ss0) / (float)dk + pre_eps);
      const float* w = norm_whole ? pre_w + (size_t)(is_key ? hs - H : hs) * dk : pre_w;
      for (int i = lane; i < dk; i += 32) x[i] = x[i] * pre * w[i];
    }
    __syncwarp();
    if (table != nullptr) {
      const float* cs = table + (size_t)pos * half * 2;
      for (int j = lane; j < half; j += 32) {
        int i0, i1;
        pair_index(j, rot_dims, interleaved, i0, i1);
        const float u = x[i0], v = x[i1];
        const float c = cs[2 * j], s = cs[2 * j + 1];
        x[i0] = u * c - v * s;
        x[i1] = v * c + u * s;
      }
      __syncwarp();
    }
    float inv = 1.f;
    if (unit_norm) {
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) ss += x[i] * x[i];
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / (float)dk + eps);
    }
    if (!is_key) inv *= temp;
    for (int i = lane; i < dk; i += 32) {
      const T r = from_f32<T>(x[i] * inv);
      if (!is_key) hp[i] = r;
      else if (crow != nullptr) crow[k_off + i] = r;
    }
    __syncwarp();
  }
  if (at < 0 || value_from_key) return;
  const T* vsrc = base + (size_t)(H + KV) * dk;
  for (int idx = threadIdx.x; idx < KV * dv; idx += blockDim.x) {
    const int g = idx / dv, i = idx - g * dv;
    cache[(((size_t)page * KV + g) * ps + off) * row_width + v_off + i] =
        bias != nullptr ? from_f32<T>(to_f32<T>(vsrc[idx]) + bias[(size_t)(H + KV) * dk + idx]) : vsrc[idx];
  }
}

// Latent attention's step between its first product and the attention kernel.
// src[t] = [per head: q_plain (dq) | q_rot (dr)] x H, then [low (R) | k_rot (dr)].
//   c      = low * rsqrt(mean(low^2) + eps) * w      (32 bit)   -> cache row [0, R)
//   k_rot  rotated on its first rot_dims entries                 -> cache row [R, R + dr)
//   q_rot  of every head rotated                                  -> qabs[t][h][R, R + dr)
// The front part qabs[t][h][0, R) is filled by the product of q_plain with the key up-projection.
// low_src != nullptr: [low | k_rot] of token t lies at low_src + t * low_stride instead (queries that were made by a
// product of their own, from a latent), and src holds the heads' queries only.
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ src, int src_stride, const int* __restrict__ tok_pos,
                                      const int* __restrict__ tok_row, const int* __restrict__ block_table, int max_pages,
                                      T* __restrict__ cache, int num_pages, const float* __restrict__ table, int table_positions,
                                      int rot_dims, int interleaved, const float* __restrict__ w, float eps, T* __restrict__ qabs,
                                      int H, int dq, int dr, int R, int ps, const T* __restrict__ low_src, int low_stride, int* err) {
  __shared__ float scratch[34];
  const int t = blockIdx.x;
  const int pos = tok_pos[t], b = tok_row[t];
  if (pos < 0 || (table != nullptr && pos >= table_positions)) {
    if (threadIdx.x == 0) dk_report(err, DK_DEV_BAD_POSITION, t, pos, table_positions);
    return;
  }
  const T* base = src + (size_t)t * src_stride;
  const T* low = low_src != nullptr ? low_src + (size_t)t * low_stride : base + (size_t)H * (dq + dr);
  const int width = R + dr;
  const long long at = cache != nullptr ? row_slot_of(block_table, max_pages, num_pages, b, pos, ps, t, err) : -1;
  T* crow = at >= 0 ? cache + (size_t)at * width : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const float v = to_f32<T>(low[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)R + eps);
  if (crow != nullptr)
    for (int i = threadIdx.x; i < R; i += blockDim.x) crow[i] = from_f32<T>(to_f32<T>(low[i]) * inv * w[i]);
  // rotated parts: unit 0 is the shared key part, units 1..H the heads' query parts
  const int half = rot_dims / 2;
  const float* cs = table != nullptr ? table + (size_t)pos * half * 2 : nullptr;
  for (int idx = threadIdx.x; idx < (H + 1) * dr; idx += blockDim.x) {
    const int unit = idx / dr, i = idx - unit * dr;
    const T* in = unit == 0 ? low + R : base + (size_t)(unit - 1) * (dq + dr) + dq;
    float r = to_f32<T>(in[i]);
    if (cs != nullptr && i < rot_dims) {
      int j, first;
      if (interleaved) { j = i >> 1; first = !(i & 1); } else { j = i % half; first = i < half; }
      int i0, i1;
      pair_index(j, rot_dims, interleaved, i0, i1);
      const float u = to_f32<T>(in[i0]), v = to_f32<T>(in[i1]);
      const float c = cs[2 * j], s = cs[2 * j + 1];
      r = first ? u * c - v * s : v * c + u * s;
    }
    if (unit == 0) {
      if (crow != nullptr) crow[R + i] = from_f32<T>(r);
    } else {
      qabs[((size_t)t * H + (unit - 1)) * width + R + i] = from_f32<T>(r);
    }
  }
}
}  // namespace

static int check_row_params(const DkRowAttnParams& p, const char* who) {
  DK_REQUIRE(p.T > 0 && p.H > 0 && p.KV > 0 && p.dk > 0 && p.dv > 0, "%s: bad sizes T=%d H=%d KV=%d dk=%d dv=%d", who, p.T, p.H, p.KV, p.dk, p.dv);
  DK_REQUIRE(p.H % p.KV == 0, "%s: %d heads are no multiple of %d key-value heads", who, p.H, p.KV);
  DK_REQUIRE(p.ps >= 1 && p.ps <= 128 && (p.ps & (p.ps - 1)) == 0, "%s: page size %d must be a power of two <= 128", who, p.ps);
  DK_REQUIRE(p.k_off >= 0 && p.v_off >= 0 && p.k_off + p.dk <= p.row_width && p.v_off + p.dv <= p.row_width,
             "%s: key [%d, +%d) or value [%d, +%d) does not lie in a row of %d", who, p.k_off, p.dk, p.v_off, p.dv, p.row_width);
  DK_REQUIRE(p.dtype == DK_F32 || p.dtype == DK_BF16, "%s: unknown dtype %d", who, p.dtype);
  return 0;
}

extern "C" int dk_attention_rows_plain(const DkRowAttnParams* pp, cudaStream_t stream) {
  const DkRowAttnParams& p = *pp;
  if (p.T == 0) return 0;
  if (int e = check_row_params(p, "attention_rows")) return e;
  DK_REQUIRE(p.dv <= MAX_DV, "attention_rows: value size %d is above the %d the plain kernel takes", p.dv, MAX_DV);
  DK_REQUIRE(p.dk <= 8192, "attention_rows: key size %d is above the 8192 the plain kernel takes", p.dk);
  DK_REQUIRE(p.H <= 65535, "attention_rows: too many heads");
  const size_t smem = (size_t)(p.dk + CH + 36) * sizeof(float) + (size_t)CH * sizeof(long long);
  dim3 grid(p.T, p.H);
  if (p.dtype == DK_F32) attention_rows_plain_kernel<float><<<grid, CH, smem, stream>>>(p);
  else attention_rows_plain_kernel<__nv_bfloat16><<<grid, CH, smem, stream>>>(p);
  return dk_check_launch("attention_rows_plain");
}

extern "C" int dk_rows_append(void* src, int src_stride, const int* tok_pos, const int* tok_row, const int* block_table,
                              int max_pages, void* cache, int num_pages, const float* table, int table_positions, int rot_dims,
                              int interleaved, int T_, int H, int KV, int dk, int dv, int ps, int row_width, int k_off, int v_off,
                              int dtype, int* err, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && H > 0 && KV > 0 && dk > 0 && dv > 0 && ps > 0, "rows_append: bad sizes T=%d H=%d KV=%d dk=%d dv=%d ps=%d", T_, H, KV, dk, dv, ps);
  DK_REQUIRE(src_stride >= (H + KV) * dk + KV * dv, "rows_append: rows of %d elements do not hold q, k and v", src_stride);
  DK_REQUIRE(cache == nullptr || (block_table != nullptr && max_pages > 0 && num_pages > 0), "rows_append: a cache is given without a block table");
  DK_REQUIRE(table == nullptr || (rot_dims > 0 && rot_dims % 2 == 0 && rot_dims <= dk), "rows_append: %d rotated entries do not fit a head of %d", rot_dims, dk);
  DK_REQUIRE(k_off + dk <= row_width && v_off + dv <= row_width, "rows_append: key and value do not fit a row of %d", row_width);
  const int threads = (H + KV) * dk >= 2048 ? 256 : 128;
#define LAUNCH(T)                                                                                                              \
  rows_append_kernel<T><<<T_, threads, 0, stream>>>((T*)src, src_stride, tok_pos, tok_row, block_table, max_pages, (T*)cache, \
                                                     num_pages, table, table_positions, rot_dims, interleaved, H, KV, dk, dv, \
                                                     ps, row_width, k_off, v_off, err)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "rows_append: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("rows_append");
}

extern "C" int dk_rows_append_unit(void* src, int src_stride, const int* tok_pos, const int* tok_row, const int* block_table,
                                   int max_pages, void* cache, int num_pages, const float* table, int table_positions, int rot_dims,
                                   int interleaved, int T_, int H, int KV, int dk, int dv, int ps, int row_width, int k_off, int v_off,
                                   int unit_norm, float eps, int value_from_key, const float* bias, const float* q_norm,
                                   const float* k_norm, float pre_eps, int norm_whole, float temp_coef, int temp_every, int dtype,
                                   int* err, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && H > 0 && KV >= 0 && dk > 0 && dv > 0 && ps > 0, "rows_append_unit: bad sizes T=%d H=%d KV=%d dk=%d dv=%d ps=%d", T_, H, KV, dk, dv, ps);
  DK_REQUIRE(KV > 0 || cache == nullptr, "rows_append_unit: a cache is given and no keys to append");
  DK_REQUIRE(!norm_whole || q_norm != nullptr, "rows_append_unit: a norm over all heads needs its weights");
  DK_REQUIRE(temp_every >= 0, "rows_append_unit: bad temperature period %d", temp_every);
  DK_REQUIRE(src_stride >= (H + KV) * dk + (value_from_key ? 0 : KV * dv), "rows_append_unit: rows of %d elements do not hold q, k and v", src_stride);
  DK_REQUIRE(!value_from_key || dv <= dk, "rows_append_unit: a value of %d entries cannot be taken from a key of %d", dv, dk);
  DK_REQUIRE(cache == nullptr || (block_table != nullptr && max_pages > 0 && num_pages > 0), "rows_append_unit: a cache is given without a block table");
  DK_REQUIRE(table == nullptr || (rot_dims > 0 && rot_dims % 2 == 0 && rot_dims <= dk), "rows_append_unit: %d rotated entries do not fit a head of %d", rot_dims, dk);
  DK_REQUIRE(k_off + dk <= row_width && v_off + dv <= row_width, "rows_append_unit: key and value do not fit a row of %d", row_width);
  const int threads = (H + KV) >= 8 ? 256 : 128;
  const size_t smem = ((size_t)(threads / 32) * dk + 34) * sizeof(float);
  DK_REQUIRE(smem <= 48 * 1024, "rows_append_unit: heads of %d entries do not fit the shared memory", dk);
#define LAUNCH(T)                                                                                                                 \
  rows_append_unit_kernel<T><<<T_, threads, smem, stream>>>((T*)src, src_stride, tok_pos, tok_row, block_table, max_pages, (T*)cache, \
                                                            num_pages, table, table_positions, rot_dims, interleaved, H, KV, dk, dv, \
                                                            ps, row_width, k_off, v_off, unit_norm, eps, value_from_key, bias, q_norm, k_norm, pre_eps, norm_whole, temp_coef, temp_every, err)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "rows_append_unit: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("rows_append_unit");
}

extern "C" int dk_latent_prepare(const void* src, int src_stride, const int* tok_pos, const int* tok_row, const int* block_table,
                                 int max_pages, void* cache, int num_pages, const float* table, int table_positions,
                                 int rot_dims, int interleaved, const float* w, float eps, void* qabs, int T_, int H, int dq,
                                 int dr, int R, int ps, const void* low_src, int low_stride, int dtype, int* err, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && H > 0 && dq > 0 && dr >= 0 && R > 0 && ps > 0, "latent_prepare: bad sizes T=%d H=%d dq=%d dr=%d R=%d ps=%d", T_, H, dq, dr, R, ps);
  DK_REQUIRE(src_stride >= H * (dq + dr) + (low_src == nullptr ? R + dr : 0), "latent_prepare: rows of %d elements do not hold the queries and the latent", src_stride);
  DK_REQUIRE(low_src == nullptr || low_stride >= R + dr, "latent_prepare: rows of %d elements do not hold the latent", low_stride);
  DK_REQUIRE(cache == nullptr || (block_table != nullptr && max_pages > 0 && num_pages > 0), "latent_prepare: a cache is given without a block table");
  DK_REQUIRE(table == nullptr || (rot_dims > 0 && rot_dims % 2 == 0 && rot_dims <= dr), "latent_prepare: %d rotated entries do not fit a part of %d", rot_dims, dr);
  const int threads = 256;
#define LAUNCH(T)                                                                                                         \
  latent_prepare_kernel<T><<<T_, threads, 0, stream>>>((const T*)src, src_stride, tok_pos, tok_row, block_table, max_pages, \
                                                        (T*)cache, num_pages, table, table_positions, rot_dims, interleaved, \
                                                        w, eps, (T*)qabs, H, dq, dr, R, ps, (const T*)low_src, low_stride, err)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "latent_prepare: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("latent_prepare");
}
