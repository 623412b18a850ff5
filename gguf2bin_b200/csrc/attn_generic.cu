// Causal grouped-query attention over the paged cache, 32-bit arithmetic, any head size
// up to 512: one warp per (token, query head).  It serves prompts and single tokens
// alike (every token carries its own position), is the attention of the float32 path,
// and the fallback of the bfloat16 path for head sizes the tensor-core kernels refuse.
//
// Formula (src/l5_model.c:518, 559-577 of AnonymoDGH/gguf2bin): kv head = head / group;
// s_t = (q . K_t) * scale for t <= pos (the loop bound is the causal mask); softmax with
// the maximum subtracted (src/l3_math.c:52-56); o = sum_t p_t V_t.  `window` > 0 keeps
// only the keys with pos - window < t <= pos; `chunk` > 0 keeps only the keys of the token's own
// chunk, floor(pos / chunk) * chunk <= t <= pos (chunks count from position 0 of the sequence).
//
// Keys are visited in chunks of 32 that start at absolute positions that are multiples
// of 32, with a running maximum and sum, so the arithmetic for a (token, head) depends
// only on its own position: not on how the tokens were cut into steps, nor on the batch.
//
// Two options for other kinds of attention.  `sink` (one float per query head, or null): the
// softmax's denominator is sum_j exp(s_j) + exp(sink_h): the sink takes probability, adds
// nothing to the output, and is used as it is (the score scale does not apply).  `planes` = 1: a page holds one panel per kv head that serves as keys AND as
// values (attention over cached latents); 2: a panel of keys and a panel of values.
// `q_stride`: elements between the query rows of two tokens (the queries may be columns of a wider
// product's output).  `gate` (one number per token and head, or null): the head's output is
// multiplied by its sigmoid.
//
// `softcap` > 0: a score s becomes softcap tanh(s / softcap) after the scale.  `keep_first` > 0 (with a
// window): the keys at positions below it stay visible to every later token, at their true
// positions; they are visited first, in chunks of 32 from position 0.  `v_heads` < nkv: key head g
// reads the values of head g mod v_heads (several score maps over one set of values).
//
// `pool` > 0 (with a window): in front of the window's keys a token also sees one key and value for
// every block of `pool` positions that lies wholly before the window, block b if
// b pool + pool - 1 <= pos - window; they come from a second store (`pooled`, [pages, 2, nkv,
// pool_rows, hd]; block b in the page of its first position at row b - ceil(that page's first
// position / pool)) and share the softmax with the window's keys.  Blocks are visited first, in
// chunks of 32 from block 0, so the order still depends on the token's position only.
#include "common.cuh"

G2B_DEFINE_LAST_ERROR

#define AG_MAX_HD 512
#define AG_WARPS 4

template <typename T>
__global__ void __launch_bounds__(AG_WARPS * 32)
attn_generic_kernel(const T *__restrict__ q, T *__restrict__ out, const T *__restrict__ cache,
                    const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
                    const int *__restrict__ page_table, int P, int n_tokens, int nh, int nkv,
                    int hd, int page_size, int window, float scale,
                    const float *__restrict__ sink, int planes, int q_stride,
                    const T *__restrict__ gate, int gate_stride, int chunk, const T *__restrict__ pooled,
                    int pool, int pool_rows, float softcap, int keep_first, int v_heads) {
  pdl_launch();
  pdl_wait();
  __shared__ float qs[AG_WARPS][AG_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * AG_WARPS + warp;
  if (item >= (long long)n_tokens * nh) return;
  const int t = (int)(item / nh), h = (int)(item % nh);
  const int pos = tok_pos[t], b = tok_seq[t];
  const int kvh = h / (nh / nkv);
  const int vh = kvh % v_heads;                                   // several key heads may share one value head
  const int lo = chunk > 0 ? (pos / chunk) * chunk : (window > 0 ? max(0, pos - window + 1) : 0);

  const T *qp = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int j = lane; j < hd; j += 32) qs[warp][j] = to_f32(qp[j]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[AG_MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] = 0.f;

  const size_t head_stride = (size_t)page_size * hd;              // one (page, K|V, kv head) panel
  if (pool > 0) {
    const int n_blocks = max(0, (pos - window + 1) / pool);       // window > 0 (the launcher checks)
    const size_t pstride = (size_t)pool_rows * hd;
    auto row_of = [&](int blk, const T *&kr, const T *&vr) {
      const int home = (blk * pool) / page_size;
      const int row = blk - (home * page_size + pool - 1) / pool;
      const size_t page = (size_t)page_table[(size_t)b * P + home];
      kr = pooled + ((page * 2 + 0) * nkv + kvh) * pstride + (size_t)row * hd;
      vr = pooled + ((page * 2 + 1) * nkv + kvh) * pstride + (size_t)row * hd;
    };
    for (int base = 0; base < n_blocks; base += 32) {
      const bool valid = base + lane < n_blocks;
      float s = -INFINITY;
      if (valid) {
        const T *kr, *vr;
        row_of(base + lane, kr, vr);
        float dot = 0.f;
        for (int j = 0; j < hd; ++j) dot = fmaf(qs[warp][j], to_f32(kr[j]), dot);
        s = dot * scale;
      }
      const float m_new = fmaxf(m, warp_max(s));                  // finite: block `base` is valid
      const float p = valid ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);
      l = l * corr + warp_sum(p);
#pragma unroll
      for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] *= corr;
      const int n_here = min(32, n_blocks - base);
      for (int j = 0; j < n_here; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const T *kr, *vr;
        row_of(base + j, kr, vr);
#pragma unroll
        for (int i = 0; i < AG_MAX_HD / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
        }
      }
      m = m_new;
    }
  }
  // keys base .. base + 31 that lie in first .. last
  auto visit = [&](int base, int first, int last) {
    const int page = page_table[(size_t)b * P + base / page_size];
    const T *kpanel = cache + (((size_t)page * planes + 0) * nkv + kvh) * head_stride;
    const T *vpanel = cache + (((size_t)page * planes + (planes - 1)) * nkv + (planes == 2 ? vh : kvh)) * head_stride;
    const int in_page = base % page_size;                         // chunk lies inside one page
    const int key = base + lane;
    const bool valid = key >= first && key <= last;
    float s = -INFINITY;
    if (valid) {
      const T *kr = kpanel + (size_t)(in_page + lane) * hd;
      float dot = 0.f;
      for (int j = 0; j < hd; ++j) dot = fmaf(qs[warp][j], to_f32(kr[j]), dot);
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    }
    const float m_new = fmaxf(m, warp_max(s));                    // finite: key `last` or `base` valid
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);                           // 0 on the first chunk
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] *= corr;
    const int n_keys = min(32, last - base + 1);
    for (int j = 0; j < n_keys; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      if (base + j < first) continue;
      const T *vr = vpanel + (size_t)(in_page + j) * hd;
#pragma unroll
      for (int i = 0; i < AG_MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
      }
    }
    m = m_new;
  };
  if (keep_first > 0 && lo > 0) {                                 // the first tokens stay visible behind the window
    const int last = min(keep_first, lo) - 1;
    for (int base = 0; base <= last; base += 32) visit(base, 0, last);
  }
  for (int base = (lo / 32) * 32; base <= pos; base += 32) visit(base, lo, pos);
  T *op = out + (size_t)t * nh * hd + (size_t)h * hd;
  if (sink) l += expf(sink[h] - m);                                // m is finite: the token's own key
  float inv_l = 1.f / l;
  if (gate) inv_l *= 1.f / (1.f + expf(-to_f32(gate[(size_t)t * gate_stride + h])));   // the head's output gate
#pragma unroll
  for (int i = 0; i < AG_MAX_HD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) op[d] = from_f32<T>(acc[i] * inv_l);
  }
}

extern "C" int g2b_attn_generic(const void *q, void *out, int dtype, const void *cache,
                                const int *tok_pos, const int *tok_seq, const int *page_table,
                                int P, int n_tokens, int nh, int nkv, int hd, int page_size,
                                int window, float scale, const float *sink, int planes, int q_stride,
                                const void *gate, int gate_stride, int chunk, const void *pooled, int pool,
                                int pool_rows, float softcap, int keep_first, int v_heads, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (pool < 0 || (pool > 0 && (window <= 0 || !pooled || planes != 2 || pool_rows < (page_size + pool - 1) / pool)))
    G2B_REFUSE("attn_generic: pooled blocks of %d need a window, their store and %d rows a page", pool,
               pool > 0 ? (page_size + pool - 1) / pool : 0);
  if (chunk < 0 || (chunk > 0 && window > 0)) G2B_REFUSE("attn_generic: a chunk of %d keys with a window of %d", chunk, window);
  if (v_heads <= 0) v_heads = nkv;
  if (v_heads > nkv || nkv % v_heads) G2B_REFUSE("attn_generic: %d key heads on %d value heads", nkv, v_heads);
  if (keep_first < 0 || (keep_first > 0 && (window <= 0 || pool > 0)))
    G2B_REFUSE("attn_generic: %d first tokens kept need a window, and go with no pooled blocks", keep_first);
  if (planes != 1 && planes != 2) G2B_REFUSE("attn_generic: %d panels per page and kv head (1 or 2)", planes);
  if (hd <= 0 || hd > AG_MAX_HD) G2B_REFUSE("attn_generic: head_dim %d outside 1..%d", hd, AG_MAX_HD);
  if (nkv <= 0 || nh % nkv) G2B_REFUSE("attn_generic: %d heads are not a multiple of %d kv heads", nh, nkv);
  if (page_size <= 0 || page_size % 32)
    G2B_REFUSE("attn_generic: page size %d must be a multiple of 32", page_size);
  const long long items = (long long)n_tokens * nh;
  const unsigned blocks = (unsigned)((items + AG_WARPS - 1) / AG_WARPS);
  if (dtype == G2B_F32)
    g2b_launch(attn_generic_kernel<float>, dim3(blocks), dim3(AG_WARPS * 32), 0, stream, 
        (const float *)q, (float *)out, (const float *)cache, tok_pos, tok_seq, page_table, P,
        n_tokens, nh, nkv, hd, page_size, window, scale, sink, planes, q_stride, (const float *)gate, gate_stride, chunk, (const float *)pooled, pool, pool_rows, softcap, keep_first, v_heads);
  else if (dtype == G2B_BF16)
    g2b_launch(attn_generic_kernel<bf16>, dim3(blocks), dim3(AG_WARPS * 32), 0, stream, 
        (const bf16 *)q, (bf16 *)out, (const bf16 *)cache, tok_pos, tok_seq, page_table, P,
        n_tokens, nh, nkv, hd, page_size, window, scale, sink, planes, q_stride, (const bf16 *)gate, gate_stride, chunk, (const bf16 *)pooled, pool, pool_rows, softcap, keep_first, v_heads);
  else
    G2B_REFUSE("attn_generic: unknown dtype %d", dtype);
  return g2b_check_launch("attn_generic");
}
