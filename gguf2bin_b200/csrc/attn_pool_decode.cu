// Attention of single tokens over a window of keys and, in front of it, the pooled blocks: a token
// at position p sees the keys max(0, p - window + 1) .. p and one mean key and value for every block
// of `pool` positions that lies wholly before its window (block j if j pool + pool - 1 <= p - window),
// all in one softmax.  bfloat16 cache and queries; scores, softmax and the output sum are 32-bit.
//
// A step of single tokens has little work per token (a window and context / pool blocks), so the
// kernel is laid out for latency: a CTA takes one token and up to GH query heads that share a kv
// head, and walks the token's list (blocks first, then the window's keys) in passes of PASS entries.
//   scores:   a warp takes every 8th entry; its lanes split the row (one 4- or 8-byte load each),
//             one warp sum per query head; the V row's address is kept for the third phase;
//   softmax:  warp g owns head g: the pass's maximum, the running maximum and sum, the weights;
//   values:   a thread owns two neighbouring value dimensions of every NS-th entry of the pass.
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
constexpr int PASS = 256;                   // entries (blocks or keys) per pass
constexpr int EPL = HD / 32;                // elements of a row per lane
constexpr int NS = THREADS / (HD / 2);      // slices of a pass in the value phase
static_assert(GH <= WARPS, "a warp per head in the softmax phase");

// N (2 or 4) neighbouring bfloat16 as floats, fetched with one load
template <int N> __device__ __forceinline__ void load_part(const bf16 *p, float *f) {
  if constexpr (N == 2) {
    const float2 a = __bfloat1622float2(__ldg(reinterpret_cast<const __nv_bfloat162 *>(p)));
    f[0] = a.x, f[1] = a.y;
  } else {
    const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.x));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.y));
    f[0] = a.x, f[1] = a.y, f[2] = c.x, f[3] = c.y;
  }
}
}  // namespace

__global__ void __launch_bounds__(THREADS)
attn_pool_decode_kernel(const bf16 *__restrict__ q, bf16 *__restrict__ out, const bf16 *__restrict__ cache,
                        const bf16 *__restrict__ pooled, const int *__restrict__ tok_pos,
                        const int *__restrict__ tok_seq, const int *__restrict__ page_table, int P, int nh,
                        int nkv, int window, float scale, int q_stride, int pool, int pool_rows) {
  pdl_launch();
  pdl_wait();
  __shared__ float sc[GH][PASS];                       // scores, then weights, of the pass
  __shared__ const bf16 *vrow[PASS];                   // where each entry's value row starts
  __shared__ float s_m[GH], s_l[GH], s_corr[GH];
  __shared__ float red[NS][GH][HD];

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

  float qr[GH][EPL];                                   // this lane's part of each head's query
#pragma unroll
  for (int g = 0; g < GH; ++g) {
    if (g < n_heads) {
      load_part<EPL>(q + (size_t)t * q_stride + (size_t)(h0 + g) * HD + lane * EPL, qr[g]);
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) qr[g][e] = 0.f;
    }
  }
  if (threadIdx.x < GH) s_m[threadIdx.x] = -INFINITY, s_l[threadIdx.x] = 0.f;

  const int dp = threadIdx.x % (HD / 2), slice = threadIdx.x / (HD / 2);
  float acc[GH][2];
#pragma unroll
  for (int g = 0; g < GH; ++g) acc[g][0] = acc[g][1] = 0.f;

  for (int i0 = 0; i0 < n_entries; i0 += PASS) {
    const int n_here = min(PASS, n_entries - i0);
    __syncthreads();                                   // the last pass's weights are used up; s_m, s_l are set
    // ---- scores ----
#pragma unroll 2
    for (int r = warp; r < n_here; r += WARPS) {
      const int i = i0 + r;
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
      float kf[EPL];
      load_part<EPL>(krow + lane * EPL, kf);
      float dot[GH];
#pragma unroll
      for (int g = 0; g < GH; ++g) {
        dot[g] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) dot[g] = fmaf(qr[g][e], kf[e], dot[g]);
      }
#pragma unroll
      for (int g = 0; g < GH; ++g) dot[g] = warp_sum(dot[g]);
      if (lane == 0) {
        vrow[r] = vr;
#pragma unroll
        for (int g = 0; g < GH; ++g) sc[g][r] = dot[g] * scale;
      }
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
    // ---- values ----
#pragma unroll
    for (int g = 0; g < GH; ++g) {
      const float corr = g < n_heads ? s_corr[g] : 0.f;
      acc[g][0] *= corr, acc[g][1] *= corr;
    }
#pragma unroll 4
    for (int r = slice; r < n_here; r += NS) {
      const float2 v = __bfloat1622float2(__ldg(reinterpret_cast<const __nv_bfloat162 *>(vrow[r]) + dp));
#pragma unroll
      for (int g = 0; g < GH; ++g) {
        const float p = sc[g][r];                      // rows of heads that are not there hold old numbers: not written out
        acc[g][0] = fmaf(p, v.x, acc[g][0]);
        acc[g][1] = fmaf(p, v.y, acc[g][1]);
      }
    }
  }
#pragma unroll
  for (int g = 0; g < GH; ++g) red[slice][g][2 * dp] = acc[g][0], red[slice][g][2 * dp + 1] = acc[g][1];
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_heads * HD; idx += THREADS) {
    const int g = idx / HD, d = idx % HD;
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < NS; ++s) sum += red[s][g][d];
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
  if (q_stride < nh * HD || q_stride % 4 || ((uintptr_t)q & 7) || ((uintptr_t)cache & 7) || ((uintptr_t)pooled & 7))
    G2B_REFUSE("attn_pool_decode: query rows %d elements apart; q and the stores 8-byte aligned", q_stride);
  const int group = nh / nkv;
  const long long tiles = (long long)nkv * ((group + GH - 1) / GH);
  if (tiles > 65535) G2B_REFUSE("attn_pool_decode: %lld head tiles are too many for one launch", tiles);
  g2b_launch(attn_pool_decode_kernel, dim3((unsigned)n_tokens, (unsigned)tiles), dim3(THREADS), 0, stream,
             (const bf16 *)q, (bf16 *)out, (const bf16 *)cache, (const bf16 *)pooled, tok_pos, tok_seq, page_table, P,
             nh, nkv, window, scale, q_stride, pool, pool_rows);
  return g2b_check_launch("attn_pool_decode");
}
