// Paged attention over a cache of rows for bfloat16 on the tensor cores (warp-level MMA), for prompt portions and
// for single decoded tokens alike.
//
// A block takes one (batch row, key-value head) and a tile of its "query rows": the pairs (new token i, head hh of
// the group), numbered m = i * G + hh, so that every head that shares the key-value head shares the block's key
// tiles.  With one shared head (a latent cache) a 64-row tile is a few tokens times all heads and the cache is
// read once for all of them; a single decoded token is a tile of G rows.  Keys stream through shared memory in
// tiles (cp.async, two stages, 16-byte chunks swizzled for ldmatrix); a cached row holds key and value, so one
// copy brings both, and a value that is the front of its key is not copied twice.  Per tile and warp:
// S = Q K^T (mma.sync.m16n8k16, float accumulators), mask by position (causal, window), online softmax in
// float (scores may first be capped, s <- cap tanh(s / cap), and take a bias by distance and head), O += P V
// with P split into two bfloat16 parts (so the softmax weights keep 16 bits of mantissa; their sum is taken in
// float from the unrounded weights).  The sink joins the denominator when the result is finished.
//
// grid (tiles of query rows, splits, batch rows * KV).  With more than one split each block takes a share of the
// key tiles and stores (unnormalised O, running maximum, sum) per query row; a second kernel merges them.
#include "common.cuh"
#include "row_attention_params.h"
#include "mma_helpers.cuh"

namespace {
constexpr int PSTAGES = 2;
constexpr float LOG2E = 1.4426950408889634f;

__host__ __device__ inline int pad128(int bytes) { return (bytes + 127) / 128 * 128; }

// tanh(t) = 1 - 2 / (1 + e^(2t)) through the exponential and reciprocal units, without a branch: exact at both ends (e^(2t) of 0
// or infinity), absolute error about 3e-7 elsewhere, which a score made of bfloat16 queries and keys does not see.
__device__ __forceinline__ float tanh_by_exp(float t) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t * (2.f * LOG2E)));
  return 1.f - __fdividef(2.f, 1.f + e);
}

// part[((t*H + head) * splits + split) * (dv + 2)]: dv floats of O, then m (log2 units), then l
// RM: 16-row tiles of query rows per warp.  With two, every key and value fragment that a warp fetches from shared memory
// feeds two products, which is what bounds this kernel (it moves 512 bytes of fragments for every 2 x 4,096 FLOP product).
// SHAPED: scores are capped and take biases by distance (an instance of its own, so that the others keep their registers).
template <int WARPS, int KT, int DVMAX, int RM, bool SHAPED>
__global__ void __launch_bounds__(WARPS * 32) attention_rows_mma_kernel(const DkRowAttnParams p, float* __restrict__ part) {
  constexpr int QT = 16 * WARPS * RM, THREADS = WARPS * 32, NT = DVMAX / 8, WR = 16 * RM;
  extern __shared__ __align__(128) unsigned char smem[];
  const int row = blockIdx.z / p.KV, g = blockIdx.z % p.KV;
  const int q_len = p.row_q_len[row];
  if ((p.row_filter == 2 && q_len == 1) || (p.row_filter == 1 && q_len != 1)) return;
  const int G = p.H / p.KV;
  const int M = q_len * G;
  const int m0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * QT;      // late tiles have the most keys: start them first
  if (m0 >= M) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int dk = p.dk, dv = p.dv, ps = p.ps;
  const int KB = dk / 16;
  const int ROWS = pad128(p.row_width * 2), QS = pad128(dk * 2);   // bytes between rows of a key tile / of the query tile
  const int CPR = p.row_width / 8;                                  // 16-byte chunks of a cached row
  unsigned char* q_smem = smem;
  unsigned char* kv_smem = smem + QT * QS;
  const int nrows = min(QT, M - m0);
  const int q_start = p.row_q_start[row], pos_start = p.row_pos_start[row];
  const int first_pos = pos_start + m0 / G, last_pos = pos_start + (m0 + nrows - 1) / G;
  const int lo_tile = (p.window > 0 && first_pos - p.window + 1 > 0) ? first_pos - p.window + 1 : 0;
  const int kt_lo = lo_tile / KT, kt_hi = last_pos / KT;
  const int splits = gridDim.y, split = blockIdx.y;
  const int per = (kt_hi - kt_lo + 1 + splits - 1) / splits;
  const int kt_a = kt_lo + split * per, kt_b = min(kt_hi + 1, kt_a + per);   // this block's key tiles [kt_a, kt_b)
  const __nv_bfloat16* cache = reinterpret_cast<const __nv_bfloat16*>(p.cache);
  const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(p.q);

  // the tile's query rows into shared memory
  for (int c = tid; c < QT * (dk / 8); c += THREADS) {
    const int r = c / (dk / 8), part_c = c % (dk / 8);
    const int m = m0 + min(r, nrows - 1);
    const __nv_bfloat16* src = q + (size_t)(q_start + m / G) * p.q_stride + (size_t)(g * G + m % G) * p.q_head_stride + part_c * 8;
    cp_async_16(smem_u32(q_smem + r * QS + ((part_c ^ (r & 7)) * 16)), src, true);
  }
  auto load_tile = [&](int kt, int stage) {
    unsigned char* dst = kv_smem + (size_t)stage * KT * ROWS;
    for (int c = tid; c < KT * CPR; c += THREADS) {
      const int tok = c / CPR, part_c = c % CPR;
      const int key = kt * KT + tok;
      bool valid = false;
      size_t off = 0;
      if (key <= last_pos && key >= lo_tile) {
        const int lp = key / ps;
        const int page = lp < p.max_pages ? p.block_table[(size_t)row * p.max_pages + lp] : -1;
        if (page < 0 || page >= p.num_pages) {
          if (part_c == 0) dk_report(p.err, DK_DEV_BAD_PAGE, q_start, lp, page);
        } else {
          valid = true;
          off = (((size_t)page * p.KV + g) * ps + key % ps) * p.row_width + part_c * 8;
        }
      }
      cp_async_16(smem_u32(dst + tok * ROWS + ((part_c ^ (tok & 7)) * 16)), cache + off, valid);
    }
  };

  float o[RM][NT][4];
  float m_run[RM][2], l_run[RM][2];
  int pos_r[RM][2];     // positions of this thread's query rows: rows warp*WR + rm*16 + gq and + 8
  const float* bias_r[RM][2];   // and the rows of the bias table of their heads
  bool live_r[RM][2];           // whether the tile has these rows at all
  const float inv_cap = (SHAPED && p.softcap > 0.f) ? 1.f / p.softcap : 0.f;
#pragma unroll
  for (int rm = 0; rm < RM; ++rm) {
#pragma unroll
    for (int n = 0; n < NT; ++n) o[rm][n][0] = o[rm][n][1] = o[rm][n][2] = o[rm][n][3] = 0.f;
    m_run[rm][0] = m_run[rm][1] = -INFINITY;
    l_run[rm][0] = l_run[rm][1] = 0.f;
    pos_r[rm][0] = pos_start + (m0 + min(warp * WR + rm * 16 + gq, nrows - 1)) / G;
    pos_r[rm][1] = pos_start + (m0 + min(warp * WR + rm * 16 + gq + 8, nrows - 1)) / G;
    if constexpr (SHAPED) {
      live_r[rm][0] = warp * WR + rm * 16 + gq < nrows;
      live_r[rm][1] = warp * WR + rm * 16 + gq + 8 < nrows;
      const size_t head0 = g * G + (m0 + min(warp * WR + rm * 16 + gq, nrows - 1)) % G;
      const size_t head1 = g * G + (m0 + min(warp * WR + rm * 16 + gq + 8, nrows - 1)) % G;
      bias_r[rm][0] = p.dist_bias != nullptr ? p.dist_bias + head0 * (p.dist_max + 1) : nullptr;
      bias_r[rm][1] = p.dist_bias != nullptr ? p.dist_bias + head1 * (p.dist_max + 1) : nullptr;
    }
  }
  const float sc_log2 = p.scale * LOG2E;
  const int warp_first_pos = pos_start + (m0 + min(warp * WR, nrows - 1)) / G;
  const int warp_last_pos = pos_start + (m0 + min(warp * WR + WR - 1, nrows - 1)) / G;
  const int kc0 = p.k_off / 8, vc0 = p.v_off / 8;

  if (kt_a < kt_b) load_tile(kt_a, 0);
  cp_async_commit();
  for (int kt = kt_a; kt < kt_b; ++kt) {
    if (kt + 1 < kt_b) load_tile(kt + 1, (kt + 1 - kt_a) % PSTAGES);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t kbase = smem_u32(kv_smem + (size_t)((kt - kt_a) % PSTAGES) * KT * ROWS);
    const uint32_t qbase = smem_u32(q_smem);
    const int kt0 = kt * KT;
    const bool visible = warp * WR < nrows && kt0 <= warp_last_pos && (p.window <= 0 || kt0 + KT - 1 > warp_first_pos - p.window);
    if (visible) {
      float s[RM][KT / 8][4];
#pragma unroll
      for (int rm = 0; rm < RM; ++rm)
#pragma unroll
        for (int j = 0; j < KT / 8; ++j) s[rm][j][0] = s[rm][j][1] = s[rm][j][2] = s[rm][j][3] = 0.f;
      for (int kb = 0; kb < KB; kb += 2) {
        uint32_t qa[RM][4], qb[RM][4];
#pragma unroll
        for (int rm = 0; rm < RM; ++rm) {
          const int r = warp * WR + rm * 16 + (lane & 15);
          ldmatrix_x4(qa[rm][0], qa[rm][1], qa[rm][2], qa[rm][3], qbase + r * QS + (((2 * kb + (lane >> 4)) ^ (r & 7)) * 16));
          if (kb + 1 < KB)
            ldmatrix_x4(qb[rm][0], qb[rm][1], qb[rm][2], qb[rm][3], qbase + r * QS + (((2 * kb + 2 + (lane >> 4)) ^ (r & 7)) * 16));
        }
#pragma unroll
        for (int j = 0; j < KT / 8; ++j) {
          const int tok = j * 8 + (lane & 7);
          uint32_t b0, b1, b2, b3;
          // (an odd count of 16-element blocks: the second pair of the last load repeats the first and is not used)
          const int cj = kc0 + 2 * kb + (kb + 1 < KB ? (lane >> 3) : ((lane >> 3) & 1));
          ldmatrix_x4(b0, b1, b2, b3, kbase + tok * ROWS + ((cj ^ (tok & 7)) * 16));
#pragma unroll
          for (int rm = 0; rm < RM; ++rm) {
            mma_bf16(s[rm][j], qa[rm], b0, b1);
            if (kb + 1 < KB) mma_bf16(s[rm][j], qb[rm], b2, b3);
          }
        }
      }
#pragma unroll
      for (int rm = 0; rm < RM; ++rm) {
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int key = kt0 + j * 8 + 2 * tq + c;
            float v0, v1;
            if constexpr (SHAPED) {      // capped scores and biases by distance: in natural units first; rows the tile does not have are left out
              v0 = v1 = -INFINITY;
              if (live_r[rm][0]) {
                v0 = s[rm][j][c] * p.scale;
                if (p.softcap > 0.f) v0 = p.softcap * tanh_by_exp(v0 * inv_cap);
                // (a key behind the query is masked below: its huge unsigned distance takes the last entry)
                if (p.dist_bias != nullptr) v0 += bias_r[rm][0][min((unsigned)(pos_r[rm][0] - key), (unsigned)p.dist_max)];
                v0 *= LOG2E;
              }
              if (live_r[rm][1]) {
                v1 = s[rm][j][2 + c] * p.scale;
                if (p.softcap > 0.f) v1 = p.softcap * tanh_by_exp(v1 * inv_cap);
                if (p.dist_bias != nullptr) v1 += bias_r[rm][1][min((unsigned)(pos_r[rm][1] - key), (unsigned)p.dist_max)];
                v1 *= LOG2E;
              }
            } else {
              v0 = s[rm][j][c] * sc_log2;
              v1 = s[rm][j][2 + c] * sc_log2;
            }
            if (key > pos_r[rm][0] || (p.window > 0 && key <= pos_r[rm][0] - p.window)) v0 = -INFINITY;
            if (key > pos_r[rm][1] || (p.window > 0 && key <= pos_r[rm][1] - p.window)) v1 = -INFINITY;
            s[rm][j][c] = v0;
            s[rm][j][2 + c] = v1;
            tmax[0] = fmaxf(tmax[0], v0);
            tmax[1] = fmaxf(tmax[1], v1);
          }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
          tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
          const float m_new = fmaxf(m_run[rm][r], tmax[r]);
          m_use[r] = m_new == -INFINITY ? 0.f : m_new;
          corr[r] = m_run[rm][r] == -INFINITY ? 0.f : exp2f(m_run[rm][r] - m_use[r]);
          m_run[rm][r] = m_new;
          l_run[rm][r] *= corr[r];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          o[rm][n][0] *= corr[0];
          o[rm][n][1] *= corr[0];
          o[rm][n][2] *= corr[1];
          o[rm][n][3] *= corr[1];
        }
        // the weights, in float, take the scores' place
#pragma unroll
        for (int j = 0; j < KT / 8; ++j) {
          s[rm][j][0] = exp2f(s[rm][j][0] - m_use[0]);
          s[rm][j][1] = exp2f(s[rm][j][1] - m_use[0]);
          s[rm][j][2] = exp2f(s[rm][j][2] - m_use[1]);
          s[rm][j][3] = exp2f(s[rm][j][3] - m_use[1]);
          l_run[rm][0] += s[rm][j][0] + s[rm][j][1];
          l_run[rm][1] += s[rm][j][2] + s[rm][j][3];
        }
      }
      // O += P V with the weights kept to 16 bits of mantissa: P = P_hi + P_lo, both bfloat16, two products per value
      // fragment (a weight rounded to bfloat16 alone would carry 8 bits)
#pragma unroll
      for (int kb2 = 0; kb2 < KT / 16; ++kb2) {
        uint32_t hi[RM][4], lo[RM][4];
#pragma unroll
        for (int rm = 0; rm < RM; ++rm) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            // fragment register q4: rows (q4 & 1 ? +8 : +0), keys 2 tq, 2 tq + 1 of the 8-key block 2 kb2 + (q4 >> 1)
            const float w0 = s[rm][2 * kb2 + (q4 >> 1)][2 * (q4 & 1)], w1 = s[rm][2 * kb2 + (q4 >> 1)][2 * (q4 & 1) + 1];
            const __nv_bfloat162 h = __floats2bfloat162_rn(w0, w1);
            hi[rm][q4] = *reinterpret_cast<const uint32_t*>(&h);
            lo[rm][q4] = pack_bf16(w0 - __low2float(h), w1 - __high2float(h));
          }
        }
        const int tok = kb2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
          if (n * 8 < dv) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, kbase + tok * ROWS + (((vc0 + n + (lane >> 4)) ^ (tok & 7)) * 16));
#pragma unroll
            for (int rm = 0; rm < RM; ++rm) {
              mma_bf16(o[rm][n], hi[rm], b0, b1);
              mma_bf16(o[rm][n + 1], hi[rm], b2, b3);
              mma_bf16(o[rm][n], lo[rm], b0, b1);
              mma_bf16(o[rm][n + 1], lo[rm], b2, b3);
            }
          }
        }
      }
    }
    __syncthreads();   // every warp is done with this stage before the next load overwrites it
  }
  cp_async_wait<0>();

#pragma unroll
  for (int rm = 0; rm < RM; ++rm) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float ll = l_run[rm][half];
      ll += __shfl_xor_sync(0xffffffffu, ll, 1);
      ll += __shfl_xor_sync(0xffffffffu, ll, 2);
      const int r = warp * WR + rm * 16 + gq + 8 * half;
      if (r >= nrows) continue;
      const int m = m0 + r;
      const int t = q_start + m / G, head = g * G + m % G;
      const float mm = m_run[rm][half];
      if (splits > 1) {
        float* dst = part + (((size_t)t * p.H + head) * splits + split) * (dv + 2);
#pragma unroll
        for (int n = 0; n < NT; ++n)
          if (n * 8 < dv) {
            dst[n * 8 + 2 * tq] = o[rm][n][2 * half];
            dst[n * 8 + 2 * tq + 1] = o[rm][n][2 * half + 1];
          }
        if (tq == 0) {
          dst[dv] = mm;
          dst[dv + 1] = ll;
        }
        continue;
      }
      float f = 1.f;
      if (p.sink != nullptr) {      // the sink joins the denominator: a key with this logit and no value
        const float s2 = p.sink[head] * LOG2E;
        const float mf = fmaxf(mm, s2);
        f = mm == -INFINITY ? 0.f : exp2f(mm - mf);
        ll = ll * f + exp2f(s2 - mf);
      }
      const float inv = ll > 0.f ? f / ll : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)t * p.H + head) * dv;
#pragma unroll
      for (int n = 0; n < NT; ++n)
        if (n * 8 < dv) *reinterpret_cast<uint32_t*>(orow + n * 8 + 2 * tq) = pack_bf16(o[rm][n][2 * half] * inv, o[rm][n][2 * half + 1] * inv);
    }
  }
}

// one block per (token of a single-token row, head): sums the splits' partial results
__global__ void attention_rows_merge_kernel(const DkRowAttnParams p, const float* __restrict__ part, int splits) {
  const int t = blockIdx.x, head = blockIdx.y;
  const int row = p.tok_row[t];
  const int q_len = p.row_q_len[row];
  if ((p.row_filter == 2 && q_len == 1) || (p.row_filter == 1 && q_len != 1)) return;
  const int dv = p.dv;
  const float* src = part + ((size_t)t * p.H + head) * splits * (dv + 2);
  float mf = p.sink != nullptr ? p.sink[head] * LOG2E : -INFINITY;
  for (int s = 0; s < splits; ++s) mf = fmaxf(mf, src[(size_t)s * (dv + 2) + dv]);
  float l = p.sink != nullptr ? exp2f(p.sink[head] * LOG2E - mf) : 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = src[(size_t)s * (dv + 2) + dv];
    if (ms != -INFINITY) l += src[(size_t)s * (dv + 2) + dv + 1] * exp2f(ms - mf);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)t * p.H + head) * dv;
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = src[(size_t)s * (dv + 2) + dv];
      if (ms != -INFINITY) a = fmaf(src[(size_t)s * (dv + 2) + d], exp2f(ms - mf), a);
    }
    orow[d] = __float2bfloat16_rn(a * inv);
  }
}

template <int WARPS, int KT, int DVMAX, int RM, bool SHAPED>
int launch_as(const DkRowAttnParams& p, int max_m, int splits, float* part, cudaStream_t stream) {
  const int m_tiles = (max_m + 16 * WARPS * RM - 1) / (16 * WARPS * RM);
  const size_t smem = (size_t)16 * WARPS * RM * pad128(p.dk * 2) + (size_t)PSTAGES * KT * pad128(p.row_width * 2);
  if (smem > 220 * 1024) {
    dk_set_error("attention_rows_mma: rows of %d elements need more shared memory than a block has", p.row_width);
    return DK_ERR_ARG;
  }
  static size_t configured_on[DK_MAX_DEVICES] = {0};
  size_t& configured = configured_on[dk_current_device()];
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_rows_mma_kernel<WARPS, KT, DVMAX, RM, SHAPED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      dk_set_error("attention_rows_mma: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return DK_ERR_LAUNCH;
    }
    configured = smem;
  }
  dim3 grid(m_tiles, splits, p.rows * p.KV);
  attention_rows_mma_kernel<WARPS, KT, DVMAX, RM, SHAPED><<<grid, WARPS * 32, smem, stream>>>(p, part);
  return dk_check_launch("attention_rows_mma");
}

// RM_SHAPED: the 16-row tiles a warp takes when the scores are shaped (the shaping's registers leave room for fewer).
template <int WARPS, int KT, int DVMAX, int RM, int RM_SHAPED = RM>
int launch(const DkRowAttnParams& p, int max_m, int splits, float* part, cudaStream_t stream) {
  if (p.softcap > 0.f || p.dist_bias != nullptr) return launch_as<WARPS, KT, DVMAX, RM_SHAPED, true>(p, max_m, splits, part, stream);
  return launch_as<WARPS, KT, DVMAX, RM, false>(p, max_m, splits, part, stream);
}
}  // namespace

extern "C" int dk_attention_rows_mma_supported(const DkRowAttnParams* pp) {
  const DkRowAttnParams& p = *pp;
  if (p.dtype != DK_BF16 || p.KV <= 0 || p.H % p.KV != 0) return 0;
  if (p.dk % 16 || p.dv % 16 || p.dk < 16 || p.dv < 16 || p.dv > 256) return 0;
  if (p.row_width % 8 || p.k_off % 8 || p.v_off % 8 || p.q_stride % 8 || p.q_head_stride % 8) return 0;
  if (p.ps < 1 || p.ps > 128 || (p.ps & (p.ps - 1)) != 0) return 0;
  if ((size_t)128 * pad128(p.dk * 2) + (size_t)PSTAGES * 64 * pad128(p.row_width * 2) > 220 * 1024) return 0;
  return 1;
}

// Floats of scratch that `splits` > 1 need.
extern "C" long long dk_attention_rows_mma_scratch_floats(int T, int H, int dv, int splits) {
  return splits > 1 ? (long long)T * H * splits * (dv + 2) : 0;
}

// max_m: the most query rows (tokens * heads of a group) any batch row brings among those the filter lets through.
extern "C" int dk_attention_rows_mma(const DkRowAttnParams* pp, int max_m, int splits, float* part, cudaStream_t stream) {
  const DkRowAttnParams& p = *pp;
  if (p.T == 0 || p.rows == 0) return 0;
  DK_REQUIRE(dk_attention_rows_mma_supported(pp), "attention_rows_mma: sizes not taken (bfloat16; key and value sizes multiples of 16, value "
             "at most 256; offsets and strides multiples of 8): dk=%d dv=%d width=%d", p.dk, p.dv, p.row_width);
  DK_REQUIRE(max_m >= 1 && splits >= 1 && splits <= 65535, "attention_rows_mma: bad max_m %d or splits %d", max_m, splits);
  DK_REQUIRE(splits == 1 || part != nullptr, "attention_rows_mma: splits without scratch memory");
  DK_REQUIRE(p.row_q_start && p.row_q_len && p.row_pos_start && p.tok_row, "attention_rows_mma: the rows' arrays are missing");
  DK_REQUIRE((long long)p.rows * p.KV <= 65535, "attention_rows_mma: grid too large");
  int e;
  // a single token's heads: one warp; up to 64 query rows or a wide value: 16 rows a warp; else 32 rows a warp
  if (max_m <= 16) {
    if (p.dv <= 64) e = launch<1, 32, 64, 1>(p, max_m, splits, part, stream);
    else if (p.dv <= 128) e = launch<1, 32, 128, 1>(p, max_m, splits, part, stream);
    else e = launch<1, 32, 256, 1>(p, max_m, splits, part, stream);
  } else if (p.dv > 128) {
    // A wide value leaves room for one 16-row tile a warp, so the fragment loads are hidden by more warps instead: eight
    // warps on 128 query rows share a key tile.  Measured on latent attention (16 heads, key 320, value 256, 2,048 tokens):
    // 4 warps with 64-key tiles 0.62 ms a layer, 4 warps with 32-key tiles (two blocks an SM) 0.41, 8 warps with 32-key
    // tiles 0.33, 8 warps with 64-key tiles 0.30.
    e = launch<8, 64, 256, 1>(p, max_m, splits, part, stream);
  } else if (max_m <= 64) {
    e = p.dv <= 64 ? launch<4, 64, 64, 1>(p, max_m, splits, part, stream) : launch<4, 64, 128, 1>(p, max_m, splits, part, stream);
  } else {
    // (shaped scores with a value of 128: two tiles a warp spill 224 bytes; one tile a warp was measured against them)
    // Shaped scores with a value of 128: two tiles a warp spill 224 bytes.  Measured (16 heads on 4, key and value 128, 2,048
    // tokens, a layer): 4 warps x 2 tiles 0.69 ms, 4 warps x 1 tile 0.57, 8 warps x 1 tile on a shared key tile 0.49.
    if (p.dv > 64 && (p.softcap > 0.f || p.dist_bias != nullptr)) e = launch_as<8, 64, 128, 1, true>(p, max_m, splits, part, stream);
    else e = p.dv <= 64 ? launch<4, 64, 64, 2>(p, max_m, splits, part, stream) : launch<4, 64, 128, 2>(p, max_m, splits, part, stream);
  }
  if (e != 0 || splits == 1) return e;
  DK_REQUIRE(p.H <= 65535, "attention_rows_mma: too many heads");
  attention_rows_merge_kernel<<<dim3(p.T, p.H), 128, 0, stream>>>(p, part, splits);
  return dk_check_launch("attention_rows_merge");
}
