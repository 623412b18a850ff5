// Attention of single tokens over a window of keys and, in front of it, the pooled blocks: a token
// at position p sees the keys max(0, p - window + 1) .. p and one mean key and value for every block
// of `pool` positions that lies wholly before its window (block j if j pool + pool - 1 <= p - window),
// all in one softmax.  bfloat16 cache and queries; scores, softmax and the output sum are 32-bit.
//
// A step of single tokens has little work per token (a window and context / pool blocks), so the
// kernel is laid out for latency: a CTA takes one token and up to GH query heads that share a kv
// head, and walks the token's list (blocks first, then the window's keys) in passes of PASS entries.
//   scores:   a thread takes one entry and reads its whole key row with 16-byte loads that are all in
//             flight at once (the queries come from shared memory, every thread the same address); the
//             V row's address is kept for the third phase;
//   softmax:  warp g owns head g: the pass's maximum, the running maximum and sum, the weights;
//   values:   HD / 8 threads cover a value row, 16 bytes each; a slice of them takes every NS-th entry.
// The partial sums of the NS slices meet once, at the end.  The order of every sum depends on the
// token's position only: not on the batch, nor on how the sequence reached that position.
//
// Stores: cache [pages, 2, nkv, 64, HD]; pooled [pages, 2, nkv, pool_rows, HD], block j in the page
// of its first position at row j - ceil(that page's first position / pool).  -DHD=64 or 128.
#include "common.cuh"

G2B_DEFINE_LAST_ERROR

#ifndef HD
#define HD 128
#endif
static_assert(HD == 64 || HD == 128, "attn_pool_decode: head sizes 64 and 128");

namespace {
constexpr int PAGE = 64;
constexpr int THREADS = 256, WARPS = THREADS / 32;
constexpr int GH = 4;                       // query heads of one kv head that a CTA takes
constexpr int PASS = THREADS;               // entries (blocks or keys) per pass: one per thread
constexpr int TPR = HD / 8;                 // threads that cover a value row, 16 bytes each
constexpr int NS = THREADS / TPR;           // slices of a pass in the value phase
static_assert(GH <= WARPS, "a warp per head in the softmax phase");

// eight bfloat16 of one 16-byte load as floats
__device__ __forceinline__ void unpack8(const uint4 &v, float *f) {
  const unsigned int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[e]));
    f[2 * e] = a.x, f[2 * e + 1] = a.y;
  }
}
__device__ __forceinline__ void load8(const bf16 *p, float *f) {
  unpack8(__ldg(reinterpret_cast<const uint4 *>(p)), f);
}
}  // namespace

__global__ void __launch_bounds__(THREADS)
attn_pool_decode_kernel(const bf16 *__restrict__ q, bf16 *__restrict__ out, const bf16 *__restrict__ cache,
                        const bf16 *__restrict__ pooled, const int *__restrict__ tok_pos,
                        const int *__restrict__ tok_seq, const int *__restrict__ page_table, int P, int nh,
                        int nkv, int window, float scale, int q_stride, int pool, int pool_rows) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float qs[GH][HD];           // the queries
  __shared__ float sc[GH][PASS];                       // scores, then weights, of the pass
  __shared__ const bf16 *vrow[PASS];                   // where each entry's value row starts
  __shared__ float s_m[GH], s_l[GH], s_corr[GH];
  __shared__ float red[WARPS][GH][HD];

  const int t = blockIdx.x;
  const int group = nh / nkv, head_tiles = (group + GH - 1) / GH;
  const int kvh = blockIdx.y / head_tiles, h0 = kvh * group + (blockIdx.y % head_tiles) * GH;
  const int n_heads = min(GH, kvh * group + group - h0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = tok_pos[t], b = tok_seq[t];
  const int lo = max(0, pos - window + 1);
  const int n_blocks = max(0, pos - window + 1) / pool;
  const int n_entries = n_blocks + pos - lo + 1;
  const int *pt = page_table + (size_t)b * P;
  const size_t panel = (size_t)PAGE * HD, ppanel = (size_t)pool_rows * HD;

  for (int idx = threadIdx.x; idx < GH * HD; idx += THREADS) {
    const int g = idx / HD, d = idx % HD;
    qs[g][d] = g < n_heads ? __bfloat162float(q[(size_t)t * q_stride + (size_t)(h0 + g) * HD + d]) : 0.f;
  }
  if (threadIdx.x < GH) s_m[threadIdx.x] = -INFINITY, s_l[threadIdx.x] = 0.f;

  const int d8 = (threadIdx.x % TPR) * 8, slice = threadIdx.x / TPR;
  float acc[GH][8];
#pragma unroll
  for (int g = 0; g < GH; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;

  for (int i0 = 0; i0 < n_entries; i0 += PASS) {
    const int n_here = min(PASS, n_entries - i0);
    __syncthreads();                                   // the last pass's weights are used up; qs, s_m, s_l are set
    // ---- scores: a thread takes one entry and reads its whole key row, all loads in flight at once ----
    if (threadIdx.x < n_here) {
      const int i = i0 + threadIdx.x;
      const bf16 *krow, *vr;
      if (i < n_blocks) {
        const int home = (i * pool) / PAGE;
        const int row = i - (home * PAGE + pool - 1) / pool;
        krow = pooled + (((size_t)pt[home] * 2) * nkv + kvh) * ppanel + (size_t)row * HD;
        vr = krow + (size_t)nkv * ppanel;
      } else {
        const int key = lo + (i - n_blocks);
        krow = cache + (((size_t)pt[key / PAGE] * 2) * nkv + kvh) * panel + (size_t)(key % PAGE) * HD;
        vr = krow + (size_t)nkv * panel;
      }
      vrow[threadIdx.x] = vr;
      float dot[GH];
#pragma unroll
      for (int g = 0; g < GH; ++g) dot[g] = 0.f;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        float kf[8];
        load8(krow + 8 * c, kf);
#pragma unroll
        for (int g = 0; g < GH; ++g) {
          const float4 q0 = *reinterpret_cast<const float4 *>(&qs[g][8 * c]);      // every thread the same address
          const float4 q1 = *reinterpret_cast<const float4 *>(&qs[g][8 * c + 4]);
          dot[g] = fmaf(q0.x, kf[0], dot[g]), dot[g] = fmaf(q0.y, kf[1], dot[g]);
          dot[g] = fmaf(q0.z, kf[2], dot[g]), dot[g] = fmaf(q0.w, kf[3], dot[g]);
          dot[g] = fmaf(q1.x, kf[4], dot[g]), dot[g] = fmaf(q1.y, kf[5], dot[g]);
          dot[g] = fmaf(q1.z, kf[6], dot[g]), dot[g] = fmaf(q1.w, kf[7], dot[g]);
        }
      }
#pragma unroll
      for (int g = 0; g < GH; ++g) sc[g][threadIdx.x] = dot[g] * scale;
    }
    __syncthreads();
    // ---- softmax: warp g owns head g ----
    if (warp < n_heads) {
      float mx = -INFINITY;
      for (int r = lane; r < n_here; r += 32) mx = fmaxf(mx, sc[warp][r]);
      const float m_old = s_m[warp];
      const float m_new = fmaxf(m_old, warp_max(mx));  // finite: the pass has an entry
      float sum = 0.f;
      for (int r = lane; r < n_here; r += 32) {
        const float p = expf(sc[warp][r] - m_new);
        sc[warp][r] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float corr = expf(m_old - m_new);        // 0 in the first pass
        s_corr[warp] = corr;
        s_l[warp] = s_l[warp] * corr + sum;
        s_m[warp] = m_new;
      }
    }
    __syncthreads();
    // ---- values: TPR threads cover a row, slice s takes the entries s, s + NS, ... ----
#pragma unroll
    for (int g = 0; g < GH; ++g) {
      const float corr = g < n_heads ? s_corr[g] : 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= corr;
    }
    // every value row of the slice is asked for before the first is used: PASS / NS loads in flight
    uint4 vv[PASS / NS];
#pragma unroll
    for (int it = 0; it < PASS / NS; ++it) {
      const int r = slice + it * NS;
      vv[it] = r < n_here ? __ldg(reinterpret_cast<const uint4 *>(vrow[r] + d8)) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int it = 0; it < PASS / NS; ++it) {
      const int r = slice + it * NS;
      if (r >= n_here) break;
      float vf[8];
      unpack8(vv[it], vf);
#pragma unroll
      for (int g = 0; g < GH; ++g) {
        const float p = sc[g][r];                      // rows of heads that are not there hold zeros' scores: not written out
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(p, vf[e], acc[g][e]);
      }
    }
  }
  // the slices of one warp meet in its first TPR lanes, the warps in shared memory
#pragma unroll
  for (int off = TPR; off < 32; off <<= 1)
#pragma unroll
    for (int g = 0; g < GH; ++g)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], off);
  if (lane < TPR) {
#pragma unroll
    for (int g = 0; g < GH; ++g)
#pragma unroll
      for (int e = 0; e < 8; ++e) red[warp][g][d8 + e] = acc[g][e];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_heads * HD; idx += THREADS) {
    const int g = idx / HD, d = idx % HD;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) sum += red[w][g][d];
    out[(size_t)t * nh * HD + (size_t)(h0 + g) * HD + d] = __float2bfloat16(sum / s_l[g]);
  }
}

// q [T, >= nh*HD] bfloat16 (rows q_stride elements apart), out [T, nh*HD] bfloat16 contiguous; one token a row.
extern "C" int g2b_attn_pool_decode(const void *q, void *out, const void *cache, const void *pooled,
                                    const int *tok_pos, const int *tok_seq, const int *page_table, int P,
                                    int n_tokens, int nh, int nkv, int hd, int page_size, int window, float scale,
                                    int q_stride, int pool, int pool_rows, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd != HD) G2B_REFUSE("attn_pool_decode: built for head_dim %d, got %d", HD, hd);
  if (page_size != PAGE) G2B_REFUSE("attn_pool_decode: page size must be %d, got %d", PAGE, page_size);
  if (nkv <= 0 || nh % nkv) G2B_REFUSE("attn_pool_decode: %d heads are not a multiple of %d kv heads", nh, nkv);
  if (pool <= 0 || window <= 0 || !pooled || pool_rows < (PAGE + pool - 1) / pool)
    G2B_REFUSE("attn_pool_decode: pooled blocks of %d need a window, their store and %d rows a page", pool,
               pool > 0 ? (PAGE + pool - 1) / pool : 0);
  if (q_stride < nh * HD || ((uintptr_t)cache & 15) || ((uintptr_t)pooled & 15))
    G2B_REFUSE("attn_pool_decode: query rows %d elements apart; the stores 16-byte aligned", q_stride);
  const int group = nh / nkv;
  const long long tiles = (long long)nkv * ((group + GH - 1) / GH);
  if (tiles > 65535) G2B_REFUSE("attn_pool_decode: %lld head tiles are too many for one launch", tiles);
  g2b_launch(attn_pool_decode_kernel, dim3((unsigned)n_tokens, (unsigned)tiles), dim3(THREADS), 0, stream,
             (const bf16 *)q, (bf16 *)out, (const bf16 *)cache, (const bf16 *)pooled, tok_pos, tok_seq, page_table, P,
             nh, nkv, window, scale, q_stride, pool, pool_rows);
  return g2b_check_launch("attn_pool_decode");
}
