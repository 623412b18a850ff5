// Kernels of mixers that carry a matrix state per head instead of keys (linear attention with a
// decay, the gated delta rule), of the short causal convolution in front of them, and of an
// attention prologue whose norm spans the whole projection.  All arithmetic is 32-bit;
// activations are read and written in the compute type (float or bfloat16); states are float.
//
//   proj_norm_rope_cache  q, k, v of one product (+ bias); RMS norm of ALL of q (and of all of k)
//                         at once, times a weight; rotation of the first `rot` entries of every
//                         head, pairs (i, i + rot/2) or (2i, 2i + 1); q out, k and v into the
//                         layer's pages.  Key and value heads may differ in size: both are
//                         stored zero-filled to the larger, and so is q.  Options: the norm per
//                         head instead (a weight of one head's size), every head of q and k
//                         divided by its root mean square after the rotation, fewer value heads
//                         than key heads, and no keys and values at all (q only).
//   selective_scan        a state S [channels, N] per sequence with a decay per entry:
//                         S[c, n] = exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n, y_c = sum_n S[c, n] C_n,
//                         dt = softplus(. + bias); out = (y + D x) silu(z) times a constant
//   diff_combine          two attention maps per head: (a1 - lambda a2) / rms, times a constant
//   rotate_heads          the rotation alone, in place, then times a constant
//   short_conv            y_t = act(sum_j w[j, c] x_{t - taps + 1 + j}[c]); rows before the step's
//                         first come from a ring of `taps` rows per slot indexed by position mod
//                         taps; rows before position 0 are zero
//   conv_keep             the last taps - 1 input rows of every sequence of the step into its ring
//   state_scan            per head a state S [D, V], a token at a time:
//                           decay:  S = a S + k v^T;                     o = S^T q
//                           delta:  S = g S; u = b (v - S^T k); S += k u^T; o = S^T q
//                           gated:  S = g S + s k v^T;                   o = S^T q
//                         with a fixed per head, or g = exp(-exp(A) softplus(x + dt)) and
//                         b = sigmoid(y) per token and head, or g and s given per token and head
//                         (`scan_gates` makes them).  One more column whose value is always 1 may
//                         ride along (the sum of the weighted keys: a normaliser).  q and k are prepared while they are
//                         staged: rotated (then k times a constant), or made unit vectors.
//   head_norm_gate        o / sqrt(mean(o^2) + eps) per head (times a weight), times silu(gate)
//   gate_mul              o * sigmoid(gate) element by element, heads unpadded
//   norm_add              x += y / sqrt(mean(y^2) + eps) * w, and the sum again in the compute type
//
// A state column (all D entries that feed one output channel) never mixes with another, so a
// block owns a range of columns of one head of one sequence and walks the step's tokens in
// order: what it computes for a token depends on the tokens before it in the sequence only,
// not on how they were cut into steps or on the batch.
#include "common.cuh"

G2B_DEFINE_LAST_ERROR

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// Rotation of x[0..rot) in shared memory by one warp: pairs (i, i + rot/2), or (2i, 2i + 1).
__device__ __forceinline__ void rotate_in_place(float *x, const float2 *cs, int rot, int interleaved, int lane) {
  const int half = rot >> 1;
  for (int i = lane; i < half; i += 32) {
    const float2 r = cs[i];
    const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
    const float u = x[a], v = x[b];
    x[a] = u * r.x - v * r.y;
    x[b] = v * r.x + u * r.y;
  }
}

// ---------------------------------------------------------------------------
// attention prologue with a norm over the whole projection
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
proj_norm_rope_cache_kernel(const T *__restrict__ qkv, int row_stride, const float *__restrict__ bias,
                            int nh, int nkv, int D, int V, const float *__restrict__ q_w,
                            const float *__restrict__ k_w, float eps, const float2 *__restrict__ rope,
                            int rot, int interleaved, const int *__restrict__ tok_pos,
                            const int *__restrict__ tok_seq, const int *__restrict__ page_table, int P,
                            T *__restrict__ cache, int page_size, T *__restrict__ q_out, float v_norm_eps,
                            int norm_per_head, float unit_eps, int nvh) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float sm[];                     // q [nh*D], k [nkv*D], one factor per value head [nvh]
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int nq = nh * D, nk = nkv * D;
  const int hd = D > V ? D : V;
  const T *src = qkv + (size_t)t * row_stride;
  float *xq = sm, *xk = sm + nq;
  float sq = 0.f, sk = 0.f;
  for (int j = threadIdx.x; j < nq + nk; j += blockDim.x) {
    const float v = to_f32(src[j]) + (bias ? bias[j] : 0.f);
    sm[j] = v;
    if (j < nq) sq = fmaf(v, v, sq); else sk = fmaf(v, v, sk);
  }
  const bool whole = !norm_per_head;
  if (q_w && whole) sq = block_sum(sq, scratch);
  if (k_w && whole) sk = block_sum(sk, scratch);
  __syncthreads();
  if (q_w && whole) {
    const float inv = 1.f / sqrtf(sq / (float)nq + eps);
    for (int j = threadIdx.x; j < nq; j += blockDim.x) xq[j] = xq[j] * inv * q_w[j];
  }
  if (k_w && whole && nk) {
    const float inv = 1.f / sqrtf(sk / (float)nk + eps);
    for (int j = threadIdx.x; j < nk; j += blockDim.x) xk[j] = xk[j] * inv * k_w[j];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  if (rope || norm_per_head || unit_eps > 0.f) {
    // a warp per head: norm with a weight over the head, rotation, division by the root mean square
    const float2 *cs = rope ? rope + (size_t)t * (rot >> 1) : nullptr;
    for (int h = warp; h < nh + nkv; h += n_warps) {
      float *x = sm + (size_t)h * D;
      const float *w = h < nh ? q_w : k_w;
      if (norm_per_head && w) {
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = fmaf(x[d], x[d], ss);
        const float inv = 1.f / sqrtf(warp_sum(ss) / (float)D + eps);
        for (int d = lane; d < D; d += 32) x[d] = x[d] * inv * w[d];
        __syncwarp();
      }
      if (cs) {
        rotate_in_place(x, cs, rot, interleaved, lane);
        __syncwarp();
      }
      if (unit_eps > 0.f) {
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = fmaf(x[d], x[d], ss);
        const float inv = 1.f / sqrtf(warp_sum(ss) / (float)D + unit_eps);
        for (int d = lane; d < D; d += 32) x[d] *= inv;
      }
    }
    __syncthreads();
  }
  float *v_inv = sm + nq + nk;                      // value heads divided by their root mean square
  if (v_norm_eps > 0.f) {
    for (int h = warp; h < nvh; h += n_warps) {
      float ss = 0.f;
      for (int d = lane; d < V; d += 32) {
        const float v = to_f32(src[nq + nk + h * V + d]) + (bias ? bias[nq + nk + h * V + d] : 0.f);
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) v_inv[h] = 1.f / sqrtf(ss / (float)V + v_norm_eps);
    }
    __syncthreads();
  }
  for (int j = threadIdx.x; j < nh * hd; j += blockDim.x) {
    const int h = j / hd, d = j % hd;
    q_out[(size_t)t * nh * hd + j] = from_f32<T>(d < D ? xq[h * D + d] : 0.f);
  }
  if (nkv <= 0) return;                             // a layer that reads another layer's keys and values
  const int pos = tok_pos[t];
  const int page = page_table[(size_t)tok_seq[t] * P + pos / page_size];
  const int in_page = pos % page_size;
  for (int j = threadIdx.x; j < nkv * hd; j += blockDim.x) {
    const int h = j / hd, d = j % hd;
    T *kd = cache + ((((size_t)page * 2 + 0) * nkv + h) * page_size + in_page) * hd;
    kd[d] = from_f32<T>(d < D ? xk[h * D + d] : 0.f);
    if (h >= nvh) continue;                         // fewer value heads than key heads: the rest of the panel is unused
    T *vd = cache + ((((size_t)page * 2 + 1) * nkv + h) * page_size + in_page) * hd;
    float v = d < V ? to_f32(src[nq + nk + h * V + d]) + (bias ? bias[nq + nk + h * V + d] : 0.f) : 0.f;
    if (v_norm_eps > 0.f) v *= v_inv[h];
    vd[d] = from_f32<T>(v);
  }
}

// The same prologue where nothing spans the heads (no norm over the whole projection): a warp a (token, head),
// no block-wide wait.  Heads count through q (nh), then keys (nkv), then values (nvh); every warp stages its head
// in shared memory, norms it (a weight of one head's size), rotates it, may divide it by its root mean square,
// and writes it out: q into q_out, keys and values into the token's page, all zero-filled to hd = max(D, V).
#define HEADWISE_WARPS 8
template <typename T>
__global__ void __launch_bounds__(HEADWISE_WARPS * 32)
proj_rope_cache_headwise_kernel(const T *__restrict__ qkv, int row_stride, const float *__restrict__ bias, int nh,
                                int nkv, int D, int V, const float *__restrict__ q_w, const float *__restrict__ k_w,
                                float eps, const float2 *__restrict__ rope, int rot, int interleaved,
                                const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
                                const int *__restrict__ page_table, int P, T *__restrict__ cache, int page_size,
                                T *__restrict__ q_out, float v_norm_eps, int norm_per_head, float unit_eps, int nvh,
                                long long n_items) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float sm[];                     // a head per warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * HEADWISE_WARPS + warp;
  if (item >= n_items) return;
  const int heads = nh + nkv + nvh;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int hd = D > V ? D : V;
  const bool is_v = h >= nh + nkv;
  const int n = is_v ? V : D;                       // entries of this head
  const int col = is_v ? (nh + nkv) * D + (h - nh - nkv) * V : h * D;
  const T *src = qkv + (size_t)t * row_stride + col;
  float *x = sm + (size_t)warp * hd;
  for (int d = lane; d < n; d += 32) x[d] = to_f32(src[d]) + (bias ? bias[col + d] : 0.f);
  __syncwarp();
  if (!is_v) {
    const float *w = h < nh ? q_w : k_w;
    if (norm_per_head && w) {
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) ss = fmaf(x[d], x[d], ss);
      const float inv = 1.f / sqrtf(warp_sum(ss) / (float)D + eps);
      for (int d = lane; d < D; d += 32) x[d] = x[d] * inv * w[d];
      __syncwarp();
    }
    if (rope) {
      rotate_in_place(x, rope + (size_t)t * (rot >> 1), rot, interleaved, lane);
      __syncwarp();
    }
    if (unit_eps > 0.f) {
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) ss = fmaf(x[d], x[d], ss);
      const float inv = 1.f / sqrtf(warp_sum(ss) / (float)D + unit_eps);
      for (int d = lane; d < D; d += 32) x[d] *= inv;
      __syncwarp();
    }
  } else if (v_norm_eps > 0.f) {
    float ss = 0.f;
    for (int d = lane; d < V; d += 32) ss = fmaf(x[d], x[d], ss);
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float)V + v_norm_eps);
    for (int d = lane; d < V; d += 32) x[d] *= inv;
    __syncwarp();
  }
  T *dst;
  if (h < nh) {
    dst = q_out + ((size_t)t * nh + h) * hd;
  } else {
    const int pos = tok_pos[t];
    const size_t page = (size_t)page_table[(size_t)tok_seq[t] * P + pos / page_size];
    const int plane = is_v ? 1 : 0, kh = is_v ? h - nh - nkv : h - nh;
    dst = cache + (((page * 2 + plane) * nkv + kh) * page_size + pos % page_size) * hd;
  }
  for (int d = lane; d < hd; d += 32) dst[d] = from_f32<T>(d < n ? x[d] : 0.f);
}

extern "C" int g2b_proj_norm_rope_cache(const void *qkv, int dtype, int row_stride, int T_tokens,
                                        const float *bias, int nh, int nkv, int D, int V, const float *q_w,
                                        const float *k_w, float eps, const float *rope, int rot, int interleaved,
                                        const int *tok_pos, const int *tok_seq, const int *page_table, int P,
                                        void *cache, int page_size, void *q_out, float v_norm_eps,
                                        int norm_per_head, float unit_eps, int nvh, cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (rope && (rot <= 0 || rot > D || (rot & 1))) G2B_REFUSE("proj_norm_rope_cache: %d rotated entries of a head of %d", rot, D);
  if (nkv < 0 || nvh < 0 || nvh > nkv) G2B_REFUSE("proj_norm_rope_cache: %d value heads beside %d key heads", nvh, nkv);
  if (nkv > 0 && !cache) G2B_REFUSE("proj_norm_rope_cache: keys without pages to write them to");
  if (norm_per_head || (!q_w && !k_w)) {                // nothing spans the heads: a warp a (token, head)
    const int hd = D > V ? D : V;
    const long long n_items = (long long)T_tokens * (nh + nkv + nvh);
    const long long blocks = (n_items + HEADWISE_WARPS - 1) / HEADWISE_WARPS;
    const size_t smem_h = (size_t)HEADWISE_WARPS * hd * sizeof(float);
    if (blocks <= 0x7fffffffLL && smem_h <= 48 * 1024) {
      if (dtype == G2B_F32)
        g2b_launch(proj_rope_cache_headwise_kernel<float>, dim3((unsigned)blocks), dim3(HEADWISE_WARPS * 32), smem_h, stream,
                   (const float *)qkv, row_stride, bias, nh, nkv, D, V, q_w, k_w, eps, (const float2 *)rope, rot, interleaved,
                   tok_pos, tok_seq, page_table, P, (float *)cache, page_size, (float *)q_out, v_norm_eps, norm_per_head,
                   unit_eps, nvh, n_items);
      else if (dtype == G2B_BF16)
        g2b_launch(proj_rope_cache_headwise_kernel<bf16>, dim3((unsigned)blocks), dim3(HEADWISE_WARPS * 32), smem_h, stream,
                   (const bf16 *)qkv, row_stride, bias, nh, nkv, D, V, q_w, k_w, eps, (const float2 *)rope, rot, interleaved,
                   tok_pos, tok_seq, page_table, P, (bf16 *)cache, page_size, (bf16 *)q_out, v_norm_eps, norm_per_head,
                   unit_eps, nvh, n_items);
      else
        G2B_REFUSE("proj_norm_rope_cache: unknown dtype %d", dtype);
      return g2b_check_launch("proj_norm_rope_cache");
    }
  }
  const size_t smem = ((size_t)(nh + nkv) * D + nkv) * sizeof(float);
  if (smem > 200 * 1024) G2B_REFUSE("proj_norm_rope_cache: q and k of %d entries do not fit a block's shared memory", (nh + nkv) * D);
  if (dtype == G2B_F32) {
    auto k = proj_norm_rope_cache_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    g2b_launch(k, dim3(T_tokens), dim3(256), smem, stream, (const float *)qkv, row_stride, bias, nh, nkv, D, V, q_w, k_w,
               eps, (const float2 *)rope, rot, interleaved, tok_pos, tok_seq, page_table, P, (float *)cache, page_size,
               (float *)q_out, v_norm_eps, norm_per_head, unit_eps, nvh);
  } else if (dtype == G2B_BF16) {
    auto k = proj_norm_rope_cache_kernel<bf16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    g2b_launch(k, dim3(T_tokens), dim3(256), smem, stream, (const bf16 *)qkv, row_stride, bias, nh, nkv, D, V, q_w, k_w,
               eps, (const float2 *)rope, rot, interleaved, tok_pos, tok_seq, page_table, P, (bf16 *)cache, page_size,
               (bf16 *)q_out, v_norm_eps, norm_per_head, unit_eps, nvh);
  } else {
    G2B_REFUSE("proj_norm_rope_cache: unknown dtype %d", dtype);
  }
  return g2b_check_launch("proj_norm_rope_cache");
}

// ---------------------------------------------------------------------------
// rotation alone
// ---------------------------------------------------------------------------
#define ROT_MAX_D 512
template <typename T>
__global__ void __launch_bounds__(128)
rotate_heads_kernel(T *__restrict__ x, int row_stride, int T_tokens, int heads, int D,
                    const float2 *__restrict__ rope, int rot, int interleaved, float scale) {
  pdl_launch();
  pdl_wait();
  __shared__ float buf[4][ROT_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + warp;
  if (item >= (long long)T_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  T *p = x + (size_t)t * row_stride + (size_t)h * D;
  for (int j = lane; j < D; j += 32) buf[warp][j] = to_f32(p[j]);
  __syncwarp();
  rotate_in_place(buf[warp], rope + (size_t)t * (rot >> 1), rot, interleaved, lane);
  __syncwarp();
  for (int j = lane; j < D; j += 32) p[j] = from_f32<T>(buf[warp][j] * scale);
}

extern "C" int g2b_rotate_heads(void *x, int dtype, int row_stride, int T_tokens, int heads, int D,
                                const float *rope, int rot, int interleaved, float scale, cudaStream_t stream) {
  if (T_tokens <= 0 || heads <= 0) return 0;
  if (D <= 0 || D > ROT_MAX_D) G2B_REFUSE("rotate_heads: head size %d outside 1..%d", D, ROT_MAX_D);
  if (!rope || rot <= 0 || rot > D || (rot & 1)) G2B_REFUSE("rotate_heads: %d rotated entries of a head of %d", rot, D);
  const unsigned blocks = (unsigned)(((long long)T_tokens * heads + 3) / 4);
  if (dtype == G2B_F32)
    g2b_launch(rotate_heads_kernel<float>, dim3(blocks), dim3(128), 0, stream, (float *)x, row_stride, T_tokens, heads, D,
               (const float2 *)rope, rot, interleaved, scale);
  else if (dtype == G2B_BF16)
    g2b_launch(rotate_heads_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, (bf16 *)x, row_stride, T_tokens, heads, D,
               (const float2 *)rope, rot, interleaved, scale);
  else
    G2B_REFUSE("rotate_heads: unknown dtype %d", dtype);
  return g2b_check_launch("rotate_heads");
}

// ---------------------------------------------------------------------------
// short causal convolution over time, per channel
// ---------------------------------------------------------------------------
#define CONV_MAX_TAPS 16
// seq_meta [B,4]: first row of the step, rows, tokens before the step, slot; null: one token per sequence
template <typename T>
__global__ void __launch_bounds__(256)
short_conv_kernel(const T *__restrict__ x, int x_stride, const float *__restrict__ w, T *__restrict__ ring,
                  int taps, int C, int T_tokens, const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
                  const int *__restrict__ seq_slots, const int *__restrict__ seq_meta, int act,
                  T *__restrict__ out, int out_stride, const float *__restrict__ bias) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;                        // tokens along x: a step may bring more than 65,535
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = tok_seq[t], pos = tok_pos[t];
  const int first_row = seq_meta ? seq_meta[4 * b + 0] : t;
  const int past = seq_meta ? seq_meta[4 * b + 2] : pos;
  T *my_ring = ring + (size_t)seq_slots[b] * taps * C;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int p = pos - (taps - 1) + j;
    float v = 0.f;
    if (p >= past) v = to_f32(x[(size_t)(first_row + (p - past)) * x_stride + c]);
    else if (p >= 0) v = to_f32(my_ring[(size_t)(p % taps) * C + c]);
    acc = fmaf(w[(size_t)j * C + c], v, acc);
  }
  if (!seq_meta && taps > 1)      // one token per sequence: nobody else touches this slot's ring in this launch,
    my_ring[(size_t)(pos % taps) * C + c] = x[(size_t)t * x_stride + c];      // and place pos % taps is not read above
  out[(size_t)t * out_stride + c] = from_f32<T>(act ? silu_f(acc) : acc);
}

// The same in bfloat16 for channel counts and row strides that are multiples of eight: a thread takes
// eight neighbouring channels of a token, 16 bytes of every tap's row at a time.
__global__ void __launch_bounds__(128)
short_conv8_kernel(const bf16 *__restrict__ x, int x_stride, const float *__restrict__ w, bf16 *__restrict__ ring,
                   int taps, int C, const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
                   const int *__restrict__ seq_slots, const int *__restrict__ seq_meta, int act,
                   bf16 *__restrict__ out, int out_stride, const float *__restrict__ bias) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int b = tok_seq[t], pos = tok_pos[t];
  const int first_row = seq_meta ? seq_meta[4 * b + 0] : t;
  const int past = seq_meta ? seq_meta[4 * b + 2] : pos;
  bf16 *my_ring = ring + (size_t)seq_slots[b] * taps * C;
  float acc[8];
  if (bias) {
    const float4 b0 = *reinterpret_cast<const float4 *>(bias + c), b1 = *reinterpret_cast<const float4 *>(bias + c + 4);
    acc[0] = b0.x, acc[1] = b0.y, acc[2] = b0.z, acc[3] = b0.w, acc[4] = b1.x, acc[5] = b1.y, acc[6] = b1.z, acc[7] = b1.w;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  }
  for (int j = 0; j < taps; ++j) {
    const int p = pos - (taps - 1) + j;
    if (p < 0) continue;                               // zeros in front of the sequence
    const bf16 *src = p >= past ? x + (size_t)(first_row + (p - past)) * x_stride + c : my_ring + (size_t)(p % taps) * C + c;
    const uint4 xv = *reinterpret_cast<const uint4 *>(src);
    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(w + (size_t)j * C + c));
    const float4 w1 = __ldg(reinterpret_cast<const float4 *>(w + (size_t)j * C + c + 4));
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xv.x));
    const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xv.y));
    const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xv.z));
    const float2 x3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xv.w));
    acc[0] = fmaf(w0.x, x0.x, acc[0]), acc[1] = fmaf(w0.y, x0.y, acc[1]);
    acc[2] = fmaf(w0.z, x1.x, acc[2]), acc[3] = fmaf(w0.w, x1.y, acc[3]);
    acc[4] = fmaf(w1.x, x2.x, acc[4]), acc[5] = fmaf(w1.y, x2.y, acc[5]);
    acc[6] = fmaf(w1.z, x3.x, acc[6]), acc[7] = fmaf(w1.w, x3.y, acc[7]);
  }
  if (!seq_meta && taps > 1)      // one token per sequence: place pos % taps of the slot's ring is not read above
    *reinterpret_cast<uint4 *>(my_ring + (size_t)(pos % taps) * C + c) =
        *reinterpret_cast<const uint4 *>(x + (size_t)t * x_stride + c);
  unsigned int ow[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float a = act ? silu_f(acc[2 * e]) : acc[2 * e], d = act ? silu_f(acc[2 * e + 1]) : acc[2 * e + 1];
    const __nv_bfloat162 ob = __floats2bfloat162_rn(a, d);
    ow[e] = *reinterpret_cast<const unsigned int *>(&ob);
  }
  *reinterpret_cast<uint4 *>(out + (size_t)t * out_stride + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

template <typename T>
__global__ void __launch_bounds__(256)
conv_keep_kernel(const T *__restrict__ x, int x_stride, T *__restrict__ ring, int taps, int C, int n_seqs,
                 const int *__restrict__ seq_meta) {
  pdl_launch();
  pdl_wait();
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int first_row = seq_meta[4 * b + 0], n = seq_meta[4 * b + 1], past = seq_meta[4 * b + 2];
  T *my_ring = ring + (size_t)seq_meta[4 * b + 3] * taps * C;
  for (int r = max(0, n - (taps - 1)); r < n; ++r)
    my_ring[(size_t)((past + r) % taps) * C + c] = x[(size_t)(first_row + r) * x_stride + c];
}

extern "C" int g2b_short_conv(const void *x, int dtype, int x_stride, const float *w, void *ring, int taps, int C,
                              int T_tokens, int n_seqs, const int *tok_pos, const int *tok_seq, const int *seq_slots,
                              const int *seq_meta, int act, void *out, int out_stride, const float *bias,
                              cudaStream_t stream) {
  if (T_tokens <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > CONV_MAX_TAPS) G2B_REFUSE("short_conv: %d taps outside 1..%d", taps, CONV_MAX_TAPS);
  if (taps > 1 && !ring) G2B_REFUSE("short_conv: no ring for the rows before the step");
  const dim3 grid(T_tokens, (C + 255) / 256), keep_grid((C + 255) / 256, n_seqs);
  if (grid.y > 65535 || n_seqs > 65535) G2B_REFUSE("short_conv: %d channels or %d sequences are too many for one launch", C, n_seqs);
  if (dtype == G2B_F32) {
    g2b_launch(short_conv_kernel<float>, grid, dim3(256), 0, stream, (const float *)x, x_stride, w, (float *)ring, taps, C,
               T_tokens, tok_pos, tok_seq, seq_slots, seq_meta, act, (float *)out, out_stride, bias);
    if (seq_meta && taps > 1)
      g2b_launch(conv_keep_kernel<float>, keep_grid, dim3(256), 0, stream, (const float *)x, x_stride, (float *)ring, taps, C,
                 n_seqs, seq_meta);
  } else if (dtype == G2B_BF16) {
    const bool wide = C % 8 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 && (C + 1023) / 1024 <= 65535 &&
                      !(((uintptr_t)x | (uintptr_t)out | (uintptr_t)ring | (uintptr_t)w | (uintptr_t)bias) & 15);
    if (wide)
      g2b_launch(short_conv8_kernel, dim3(T_tokens, (C / 8 + 127) / 128), dim3(128), 0, stream, (const bf16 *)x, x_stride, w,
                 (bf16 *)ring, taps, C, tok_pos, tok_seq, seq_slots, seq_meta, act, (bf16 *)out, out_stride, bias);
    else
      g2b_launch(short_conv_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16 *)x, x_stride, w, (bf16 *)ring, taps, C,
                 T_tokens, tok_pos, tok_seq, seq_slots, seq_meta, act, (bf16 *)out, out_stride, bias);
    if (seq_meta && taps > 1)
      g2b_launch(conv_keep_kernel<bf16>, keep_grid, dim3(256), 0, stream, (const bf16 *)x, x_stride, (bf16 *)ring, taps, C,
                 n_seqs, seq_meta);
  } else {
    G2B_REFUSE("short_conv: unknown dtype %d", dtype);
  }
  return g2b_check_launch("short_conv");
}

// ---------------------------------------------------------------------------
// the state scan
// ---------------------------------------------------------------------------
// A column of the state (D entries) is held by L lanes of one warp, R = ceil(D / L) <= 16 entries
// each: lane l holds rows r * L + l.  The state is stored column by column ([slot, head, V, D]), so
// the L lanes of a column read L consecutive floats per r.
#define SCAN_THREADS 256
#define SCAN_R 16
#define SCAN_TILE 8           // tokens staged at a time (one warp prepares one token's q and k)
#define SCAN_MAX_D 512

struct ScanArgs {
  const void *q, *k, *v;      // compute type; rows of wider buffers
  int q_stride, k_stride, v_stride;
  int H, G, D, V;             // value heads, query/key heads, key size, columns of a head's state
  int Vin;                    // value size of a head in `v`; columns from there on take the value 1
  const float2 *rope;         // [T, rot/2] or null
  int rot, interleaved;
  float q_scale, k_scale;     // after rotation / after the unit norm
  int unit_norm;              // q and k divided by sqrt(sum x^2 + unit_eps) first
  float unit_eps;
  const float *decay;         // mode 0: [H]
  const float *ab;            // mode 1: [T, 2H] float: decay input x, then write-strength input y
                              // mode 2: [T, 2H] float: the decay g, then the strength s, as they are
  const float *A_log, *dt_bias;      // mode 1: [H]
  float *state;               // [slots, H, V, D]
  const int *tok_pos, *seq_slots, *seq_meta;
  float *out;                 // [T, H*V] float
  int n_tokens;
};

template <typename T, int MODE>
__global__ void __launch_bounds__(SCAN_THREADS)
state_scan_kernel(const ScanArgs a, int L) {
  pdl_launch();
  pdl_wait();
  __shared__ float sq[SCAN_TILE][SCAN_MAX_D];
  __shared__ float sk[SCAN_TILE][SCAN_MAX_D];
  __shared__ float sv[SCAN_TILE][SCAN_THREADS / 8];
  __shared__ float sg[SCAN_TILE], sb[SCAN_TILE];
  const int D = a.D, V = a.V, H = a.H;
  const int b = blockIdx.z, h = blockIdx.y;
  const int qk_head = h / (H / a.G);
  const int cols = SCAN_THREADS / L;
  const int lane_in_col = threadIdx.x % L;
  const int col_local = threadIdx.x / L;
  const int c = blockIdx.x * cols + col_local;
  const bool live = c < V;
  const int first_row = a.seq_meta ? a.seq_meta[4 * b + 0] : b;
  const int n = a.seq_meta ? a.seq_meta[4 * b + 1] : 1;
  const int slot = a.seq_slots[b];
  const int R = (D + L - 1) / L;
  float *sp = a.state + (((size_t)slot * H + h) * V + (live ? c : 0)) * D;
  float S[SCAN_R];
#pragma unroll
  for (int r = 0; r < SCAN_R; ++r) {
    const int d = r * L + lane_in_col;
    S[r] = (live && r < R && d < D) ? sp[d] : 0.f;
  }
  float decay = 1.f, A = 0.f, dt = 0.f;
  if (MODE == 0) decay = a.decay[h];
  else if (MODE == 1) { A = expf(a.A_log[h]); dt = a.dt_bias[h]; }
  const int Vin = a.Vin;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T *qg = (const T *)a.q, *kg = (const T *)a.k, *vg = (const T *)a.v;

  for (int t0 = 0; t0 < n; t0 += SCAN_TILE) {
    const int nt = min(SCAN_TILE, n - t0);
    __syncthreads();                              // the tile before is used up
    if (warp < nt) {                              // SCAN_TILE == warps of the block: one token each
      const int row = first_row + t0 + warp;
      const T *qp = qg + (size_t)row * a.q_stride + (size_t)qk_head * D;
      const T *kp = kg + (size_t)row * a.k_stride + (size_t)qk_head * D;
      float nq = 0.f, nk = 0.f;
      for (int j = lane; j < D; j += 32) {
        const float x = to_f32(qp[j]), y = to_f32(kp[j]);
        sq[warp][j] = x;
        sk[warp][j] = y;
        nq = fmaf(x, x, nq);
        nk = fmaf(y, y, nk);
      }
      __syncwarp();
      float fq = a.q_scale, fk = a.k_scale;
      if (a.unit_norm) {
        fq *= 1.f / sqrtf(warp_sum(nq) + a.unit_eps);
        fk *= 1.f / sqrtf(warp_sum(nk) + a.unit_eps);
      }
      if (a.rope) {
        const float2 *cs = a.rope + (size_t)row * (a.rot >> 1);
        rotate_in_place(sq[warp], cs, a.rot, a.interleaved, lane);
        rotate_in_place(sk[warp], cs, a.rot, a.interleaved, lane);
        __syncwarp();
      }
      for (int j = lane; j < D; j += 32) {
        sq[warp][j] *= fq;
        sk[warp][j] *= fk;
      }
      if (MODE != 0 && lane == 0) {
        const float x = a.ab[(size_t)row * 2 * H + h], y = a.ab[(size_t)row * 2 * H + H + h];
        sg[warp] = MODE == 1 ? expf(-A * softplus_f(x + dt)) : x;
        sb[warp] = MODE == 1 ? sigmoid_f(y) : y;
      }
    }
    for (int i = threadIdx.x; i < nt * cols; i += SCAN_THREADS) {
      const int tt = i / cols, cc = i % cols;
      const int col = blockIdx.x * cols + cc;
      sv[tt][cc] = col < Vin ? to_f32(vg[(size_t)(first_row + t0 + tt) * a.v_stride + (size_t)h * Vin + col])
                             : (col < V ? 1.f : 0.f);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float v = sv[tt][col_local];
      const float *kq = sk[tt], *qq = sq[tt];
      float o = 0.f;
      if (MODE == 0) {
#pragma unroll
        for (int r = 0; r < SCAN_R; ++r) {
          if (r < R) {
            const int d = r * L + lane_in_col;
            const float kd = d < D ? kq[d] : 0.f, qd = d < D ? qq[d] : 0.f;
            S[r] = fmaf(decay, S[r], kd * v);
            o = fmaf(S[r], qd, o);
          }
        }
      } else if (MODE == 2) {
        const float g = sg[tt], sv_ = sb[tt] * v;
#pragma unroll
        for (int r = 0; r < SCAN_R; ++r) {
          if (r < R) {
            const int d = r * L + lane_in_col;
            const float kd = d < D ? kq[d] : 0.f, qd = d < D ? qq[d] : 0.f;
            S[r] = fmaf(g, S[r], kd * sv_);
            o = fmaf(S[r], qd, o);
          }
        }
      } else {
        const float g = sg[tt], beta = sb[tt];
        float dot = 0.f;
#pragma unroll
        for (int r = 0; r < SCAN_R; ++r) {
          if (r < R) {
            const int d = r * L + lane_in_col;
            S[r] *= g;
            dot = fmaf(S[r], d < D ? kq[d] : 0.f, dot);
          }
        }
        for (int off = L >> 1; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float u = beta * (v - dot);
#pragma unroll
        for (int r = 0; r < SCAN_R; ++r) {
          if (r < R) {
            const int d = r * L + lane_in_col;
            const float kd = d < D ? kq[d] : 0.f, qd = d < D ? qq[d] : 0.f;
            S[r] = fmaf(kd, u, S[r]);
            o = fmaf(S[r], qd, o);
          }
        }
      }
      for (int off = L >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (live && lane_in_col == 0) a.out[(size_t)(first_row + t0 + tt) * H * V + (size_t)h * V + c] = o;
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < SCAN_R; ++r) {
      const int d = r * L + lane_in_col;
      if (r < R && d < D) sp[d] = S[r];
    }
  }
}

extern "C" int g2b_state_scan(int mode, int dtype, const void *q, int q_stride, const void *k, int k_stride,
                              const void *v, int v_stride, int H, int G, int D, int V, const float *rope, int rot,
                              int interleaved, float q_scale, float k_scale, int unit_norm, float unit_eps,
                              const float *decay, const float *ab, const float *A_log, const float *dt_bias,
                              float *state, const int *tok_pos, const int *seq_slots, const int *seq_meta,
                              int n_tokens, int n_seqs, float *out, int extra_one, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0) return 0;
  if (D <= 0 || D > SCAN_MAX_D) G2B_REFUSE("state_scan: key size %d outside 1..%d", D, SCAN_MAX_D);
  if (G <= 0 || H % G) G2B_REFUSE("state_scan: %d heads are not a multiple of %d query/key heads", H, G);
  if (rope && (rot <= 0 || rot > D || (rot & 1))) G2B_REFUSE("state_scan: %d rotated entries of a head of %d", rot, D);
  if (mode == 0 ? !decay : (mode == 1 ? (!ab || !A_log || !dt_bias) : !ab)) G2B_REFUSE("state_scan: mode %d lacks its decay inputs", mode);
  const int Vin = V;
  V += extra_one ? 1 : 0;
  int L = 8;
  while (L * SCAN_R < D) L <<= 1;                 // 8, 16 or 32 lanes a column
  ScanArgs a;
  a.q = q; a.k = k; a.v = v; a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
  a.H = H; a.G = G; a.D = D; a.V = V; a.Vin = Vin; a.rope = (const float2 *)rope; a.rot = rot; a.interleaved = interleaved;
  a.q_scale = q_scale; a.k_scale = k_scale; a.unit_norm = unit_norm; a.unit_eps = unit_eps; a.decay = decay;
  a.ab = ab; a.A_log = A_log; a.dt_bias = dt_bias; a.state = state; a.tok_pos = tok_pos; a.seq_slots = seq_slots;
  a.seq_meta = seq_meta; a.out = out; a.n_tokens = n_tokens;
  const int cols = SCAN_THREADS / L;
  const dim3 grid((V + cols - 1) / cols, H, n_seqs);
  if (dtype != G2B_F32 && dtype != G2B_BF16) G2B_REFUSE("state_scan: unknown dtype %d", dtype);
  if (mode == 0) {
    if (dtype == G2B_F32) g2b_launch(state_scan_kernel<float, 0>, grid, dim3(SCAN_THREADS), 0, stream, a, L);
    else g2b_launch(state_scan_kernel<bf16, 0>, grid, dim3(SCAN_THREADS), 0, stream, a, L);
  } else if (mode == 1) {
    if (dtype == G2B_F32) g2b_launch(state_scan_kernel<float, 1>, grid, dim3(SCAN_THREADS), 0, stream, a, L);
    else g2b_launch(state_scan_kernel<bf16, 1>, grid, dim3(SCAN_THREADS), 0, stream, a, L);
  } else if (mode == 2) {
    if (dtype == G2B_F32) g2b_launch(state_scan_kernel<float, 2>, grid, dim3(SCAN_THREADS), 0, stream, a, L);
    else g2b_launch(state_scan_kernel<bf16, 2>, grid, dim3(SCAN_THREADS), 0, stream, a, L);
  } else {
    G2B_REFUSE("state_scan: unknown mode %d", mode);
  }
  return g2b_check_launch("state_scan");
}

// ---------------------------------------------------------------------------
// the state scan for prompts: q and k prepared once by a kernel of their own, then a scan whose
// next tile of tokens is on its way into shared memory while the current one is computed
// ---------------------------------------------------------------------------
// scan_prep: one warp per (token, query/key head): rotation or unit norm, scales; float out.
template <typename T>
__global__ void __launch_bounds__(128)
scan_prep_kernel(const T *__restrict__ q, int q_stride, const T *__restrict__ k, int k_stride, int n_tokens, int G, int D,
                 const float2 *__restrict__ rope, int rot, int interleaved, float q_scale, float k_scale,
                 int unit_norm, float unit_eps, float *__restrict__ qf, float *__restrict__ kf) {
  pdl_launch();
  pdl_wait();
  __shared__ float sq[4][SCAN_MAX_D];
  __shared__ float sk[4][SCAN_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + warp;
  if (item >= (long long)n_tokens * G) return;
  const int t = (int)(item / G), g = (int)(item % G);
  const T *qp = q + (size_t)t * q_stride + (size_t)g * D;
  const T *kp = k + (size_t)t * k_stride + (size_t)g * D;
  float nq = 0.f, nk = 0.f;
  for (int j = lane; j < D; j += 32) {
    const float x = to_f32(qp[j]), y = to_f32(kp[j]);
    sq[warp][j] = x;
    sk[warp][j] = y;
    nq = fmaf(x, x, nq);
    nk = fmaf(y, y, nk);
  }
  __syncwarp();
  float fq = q_scale, fk = k_scale;
  if (unit_norm) {
    fq *= 1.f / sqrtf(warp_sum(nq) + unit_eps);
    fk *= 1.f / sqrtf(warp_sum(nk) + unit_eps);
  }
  if (rope) {
    const float2 *cs = rope + (size_t)t * (rot >> 1);
    rotate_in_place(sq[warp], cs, rot, interleaved, lane);
    rotate_in_place(sk[warp], cs, rot, interleaved, lane);
    __syncwarp();
  }
  for (int j = lane; j < D; j += 32) {
    qf[((size_t)t * G + g) * D + j] = sq[warp][j] * fq;
    kf[((size_t)t * G + g) * D + j] = sk[warp][j] * fk;
  }
}

__device__ __forceinline__ void cp_async_f4(float *smem, const float *g) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(addr), "l"(g));
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// 128 threads; a column of the state is held by L lanes, lane l the rows 4 (j L + l) .. + 3, j < 4
// (16 L >= D; rows from D on are zeros).  Shared memory: two buffers of `tile` tokens of q and k
// (rows of Dp = D rounded up to 4 L floats), of the columns' v, and of the tokens' two gates.
#define PSCAN_THREADS 128
struct PScanArgs {
  const float *qf, *kf;       // [T, G, D] prepared
  const void *v;              // compute type, rows of a wider buffer
  int v_stride, H, G, D, V, Vin;        // V: columns of a head's state; Vin: value size in `v` (columns beyond: 1)
  const float *decay, *ab, *A_log, *dt_bias;
  float *state;               // [slots, H, V, D]
  const int *seq_meta;
  float *out;                 // [T, H*V]
  int L, Dp, tile;
};

template <typename T, int MODE, int L>
__global__ void __launch_bounds__(PSCAN_THREADS)
state_scan_prompt_kernel(const PScanArgs a) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float psm[];
  constexpr int cols = PSCAN_THREADS / L;
  const int D = a.D, V = a.V, H = a.H, Dp = a.Dp, TT = a.tile;
  // two buffers, each: q [TT, Dp], k [TT, Dp]; behind them two of v [TT, cols], gate [TT], strength [TT]
  const int qk_buf = 2 * TT * Dp, small_buf = TT * (cols + 2);
  float *small = psm + 2 * qk_buf;
  float *po = small + 2 * small_buf;               // [TT, threads]: every lane's share of a token's read-out
  const int b = blockIdx.z, h = blockIdx.y;
  const int qk_head = h / (H / a.G);
  const int lane_in_col = threadIdx.x % L, col_local = threadIdx.x / L;
  const int c = blockIdx.x * cols + col_local;
  const bool live = c < V;
  const int first_row = a.seq_meta[4 * b + 0], n = a.seq_meta[4 * b + 1], slot = a.seq_meta[4 * b + 3];
  const int RG = Dp / (4 * L);                     // groups of four rows per lane, at most 4
  float *sp = a.state + (((size_t)slot * H + h) * V + (live ? c : 0)) * D;
  const bool vec = (D & 3) == 0;
  float S[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int d = 4 * (j * L + lane_in_col) + i;
      S[j][i] = (live && j < RG && d < D) ? sp[d] : 0.f;
    }
  float decay = 1.f, A = 0.f, dt = 0.f;
  if (MODE == 0) decay = a.decay[h];
  else if (MODE == 1) { A = expf(a.A_log[h]); dt = a.dt_bias[h]; }
  const int Vin = a.Vin;
  const T *vg = (const T *)a.v;
  for (int i = threadIdx.x; i < 2 * qk_buf; i += PSCAN_THREADS) psm[i] = 0.f;     // rows from D on stay zero
  __syncthreads();

  auto fetch_qk = [&](int t0, int nt, int buf) {
    const float *qsrc = a.qf + ((size_t)(first_row + t0) * a.G + qk_head) * D;
    const float *ksrc = a.kf + ((size_t)(first_row + t0) * a.G + qk_head) * D;
    const size_t row = (size_t)a.G * D;
    float *dq = psm + buf * qk_buf, *dk = dq + TT * Dp;
    if (vec) {                                     // a warp per token row: no division per copy
      const int per = D >> 2;
      for (int tt = threadIdx.x >> 5; tt < nt; tt += PSCAN_THREADS / 32)
        for (int p = threadIdx.x & 31; p < per; p += 32) {
          cp_async_f4(dq + tt * Dp + 4 * p, qsrc + tt * row + 4 * p);
          cp_async_f4(dk + tt * Dp + 4 * p, ksrc + tt * row + 4 * p);
        }
    } else {
      for (int i = threadIdx.x; i < nt * D; i += PSCAN_THREADS) {
        const int tt = i / D, p = i % D;
        dq[tt * Dp + p] = qsrc[tt * row + p];
        dk[tt * Dp + p] = ksrc[tt * row + p];
      }
    }
    cp_async_commit_group();
  };
  // the small per-token values go through registers: loaded before the tile in work is computed,
  // stored behind it
  float rv0 = 0.f, rv1 = 0.f, rg = 0.f, rb = 0.f;                   // TT * cols <= 256 = 2 * threads
  auto load_small = [&](int t0, int nt) {
    {
      const int i = threadIdx.x, tt = i / cols, col = blockIdx.x * cols + i % cols;
      rv0 = (tt < nt && col < Vin) ? to_f32(vg[(size_t)(first_row + t0 + tt) * a.v_stride + (size_t)h * Vin + col])
                                   : ((tt < nt && col < V) ? 1.f : 0.f);
    }
    {
      const int i = threadIdx.x + PSCAN_THREADS, tt = i / cols, col = blockIdx.x * cols + i % cols;
      rv1 = (tt < nt && col < Vin) ? to_f32(vg[(size_t)(first_row + t0 + tt) * a.v_stride + (size_t)h * Vin + col])
                                   : ((tt < nt && col < V) ? 1.f : 0.f);
    }
    if (MODE != 0 && threadIdx.x < nt) {
      const size_t row = (size_t)(first_row + t0 + threadIdx.x) * 2 * H;
      rg = a.ab[row + h];
      rb = a.ab[row + H + h];
    }
  };
  auto store_small = [&](int nt, int buf) {
    float *dv = small + buf * small_buf;
    if (threadIdx.x < TT * cols) dv[threadIdx.x] = rv0;
    if (threadIdx.x + PSCAN_THREADS < TT * cols) dv[threadIdx.x + PSCAN_THREADS] = rv1;
    if (MODE != 0 && threadIdx.x < nt) {
      dv[TT * cols + threadIdx.x] = MODE == 1 ? expf(-A * softplus_f(rg + dt)) : rg;
      dv[TT * cols + TT + threadIdx.x] = MODE == 1 ? sigmoid_f(rb) : rb;
    }
  };

  fetch_qk(0, min(TT, n), 0);
  load_small(0, min(TT, n));
  store_small(min(TT, n), 0);
  int buf = 0;
  const size_t out_row = (size_t)H * V;
  for (int t0 = 0; t0 < n; t0 += TT, buf ^= 1) {
    const int nt = min(TT, n - t0);
    const int next = t0 + TT, nn = min(TT, n - next);
    cp_async_wait_all();
    __syncthreads();                               // tile t0 is in `buf`; nobody reads buf ^ 1 any more
    if (next < n) {
      fetch_qk(next, nn, buf ^ 1);
      load_small(next, nn);
    }
    const float *qp = psm + buf * qk_buf + 4 * lane_in_col;
    const float *kp = qp + TT * Dp;
    const float *vp = small + buf * small_buf + col_local;
    const float *gp = small + buf * small_buf + TT * cols, *bp = gp + TT;
    float *pp = po + threadIdx.x;
#pragma unroll 4
    for (int tt = 0; tt < nt; ++tt, qp += Dp, kp += Dp, vp += cols, pp += PSCAN_THREADS) {
      const float v = *vp;
      float o[4] = {0.f, 0.f, 0.f, 0.f};
      if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < RG) {
            const float4 kd = *(const float4 *)(kp + 4 * j * L);
            const float4 qd = *(const float4 *)(qp + 4 * j * L);
            S[j][0] = fmaf(decay, S[j][0], kd.x * v);
            S[j][1] = fmaf(decay, S[j][1], kd.y * v);
            S[j][2] = fmaf(decay, S[j][2], kd.z * v);
            S[j][3] = fmaf(decay, S[j][3], kd.w * v);
            o[j] = fmaf(S[j][3], qd.w, fmaf(S[j][2], qd.z, fmaf(S[j][1], qd.y, S[j][0] * qd.x)));
          }
        }
      } else if (MODE == 2) {
        const float g = gp[tt], sv_ = bp[tt] * v;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < RG) {
            const float4 kd = *(const float4 *)(kp + 4 * j * L);
            const float4 qd = *(const float4 *)(qp + 4 * j * L);
            S[j][0] = fmaf(g, S[j][0], kd.x * sv_);
            S[j][1] = fmaf(g, S[j][1], kd.y * sv_);
            S[j][2] = fmaf(g, S[j][2], kd.z * sv_);
            S[j][3] = fmaf(g, S[j][3], kd.w * sv_);
            o[j] = fmaf(S[j][3], qd.w, fmaf(S[j][2], qd.z, fmaf(S[j][1], qd.y, S[j][0] * qd.x)));
          }
        }
      } else {
        const float g = gp[tt], beta = bp[tt];
        float dot[4] = {0.f, 0.f, 0.f, 0.f};
        float4 kd[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < RG) {
            kd[j] = *(const float4 *)(kp + 4 * j * L);
            S[j][0] *= g; S[j][1] *= g; S[j][2] *= g; S[j][3] *= g;
            dot[j] = fmaf(S[j][3], kd[j].w, fmaf(S[j][2], kd[j].z, fmaf(S[j][1], kd[j].y, S[j][0] * kd[j].x)));
          }
        }
        float dsum = (dot[0] + dot[1]) + (dot[2] + dot[3]);
#pragma unroll
        for (int off = L >> 1; off > 0; off >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, off);
        const float u = beta * (v - dsum);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < RG) {
            const float4 qd = *(const float4 *)(qp + 4 * j * L);
            S[j][0] = fmaf(kd[j].x, u, S[j][0]);
            S[j][1] = fmaf(kd[j].y, u, S[j][1]);
            S[j][2] = fmaf(kd[j].z, u, S[j][2]);
            S[j][3] = fmaf(kd[j].w, u, S[j][3]);
            o[j] = fmaf(S[j][3], qd.w, fmaf(S[j][2], qd.z, fmaf(S[j][1], qd.y, S[j][0] * qd.x)));
          }
        }
      }
      *pp = (o[0] + o[1]) + (o[2] + o[3]);           // the lanes' shares are added after the tile: nothing waits here
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt * cols; i += PSCAN_THREADS) {
      const int tt = i / cols, cc = i % cols;
      const float *src = po + tt * PSCAN_THREADS + cc * L;
      float sum = 0.f;
#pragma unroll
      for (int l = 0; l < L; ++l) sum += src[(l + cc) % L];          // started at another lane per column: no bank conflicts
      const int col = blockIdx.x * cols + cc;
      if (col < V) a.out[(size_t)(first_row + t0 + tt) * out_row + (size_t)h * V + col] = sum;
    }
    if (next < n) store_small(nn, buf ^ 1);
  }
  if (live) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d = 4 * (j * L + lane_in_col) + i;
        if (j < RG && d < D) sp[d] = S[j][i];
      }
  }
}

template <typename T, int MODE>
static void launch_scan_prompt(const PScanArgs &a, dim3 grid, size_t smem, cudaStream_t stream) {
  if (a.L == 8) g2b_launch(state_scan_prompt_kernel<T, MODE, 8>, grid, dim3(PSCAN_THREADS), smem, stream, a);
  else if (a.L == 16) g2b_launch(state_scan_prompt_kernel<T, MODE, 16>, grid, dim3(PSCAN_THREADS), smem, stream, a);
  else g2b_launch(state_scan_prompt_kernel<T, MODE, 32>, grid, dim3(PSCAN_THREADS), smem, stream, a);
}

extern "C" int g2b_state_scan_prompt(int mode, int dtype, const void *q, int q_stride, const void *k, int k_stride,
                                     const void *v, int v_stride, int H, int G, int D, int V, const float *rope, int rot,
                                     int interleaved, float q_scale, float k_scale, int unit_norm, float unit_eps,
                                     const float *decay, const float *ab, const float *A_log, const float *dt_bias,
                                     float *state, const int *seq_meta, int n_tokens, int n_seqs, float *qf, float *kf,
                                     float *out, int extra_one, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0) return 0;
  if (D <= 0 || D > SCAN_MAX_D) G2B_REFUSE("state_scan: key size %d outside 1..%d", D, SCAN_MAX_D);
  if (G <= 0 || H % G) G2B_REFUSE("state_scan: %d heads are not a multiple of %d query/key heads", H, G);
  if (rope && (rot <= 0 || rot > D || (rot & 1))) G2B_REFUSE("state_scan: %d rotated entries of a head of %d", rot, D);
  if (mode == 0 ? !decay : (mode == 1 ? (!ab || !A_log || !dt_bias) : !ab)) G2B_REFUSE("state_scan: mode %d lacks its decay inputs", mode);
  const int Vin = V;
  V += extra_one ? 1 : 0;
  if (!seq_meta) G2B_REFUSE("state_scan: the prompt kernel needs the step's table of sequences");
  if (dtype != G2B_F32 && dtype != G2B_BF16) G2B_REFUSE("state_scan: unknown dtype %d", dtype);
  const unsigned prep_blocks = (unsigned)(((long long)n_tokens * G + 3) / 4);
  if (dtype == G2B_F32)
    g2b_launch(scan_prep_kernel<float>, dim3(prep_blocks), dim3(128), 0, stream, (const float *)q, q_stride, (const float *)k,
               k_stride, n_tokens, G, D, (const float2 *)rope, rot, interleaved, q_scale, k_scale, unit_norm, unit_eps, qf, kf);
  else
    g2b_launch(scan_prep_kernel<bf16>, dim3(prep_blocks), dim3(128), 0, stream, (const bf16 *)q, q_stride, (const bf16 *)k,
               k_stride, n_tokens, G, D, (const float2 *)rope, rot, interleaved, q_scale, k_scale, unit_norm, unit_eps, qf, kf);
  PScanArgs a;
  a.qf = qf; a.kf = kf; a.v = v; a.v_stride = v_stride; a.H = H; a.G = G; a.D = D; a.V = V; a.Vin = Vin; a.decay = decay; a.ab = ab;
  a.A_log = A_log; a.dt_bias = dt_bias; a.state = state; a.seq_meta = seq_meta; a.out = out;
  // Lanes per column: at least D / 16; more while the step has few columns, so that every scheduler
  // of the GPU gets a few warps (a token's work in a warp is a chain of short dependent steps).
  a.L = 8;
  while (a.L * 16 < D) a.L <<= 1;
  {
    const long long columns = (long long)n_seqs * H * V;
    while (a.L < 32 && columns * a.L * 2 <= 32LL * 2400) a.L <<= 1;
  }
  a.Dp = (D + 4 * a.L - 1) / (4 * a.L) * (4 * a.L);
  a.tile = a.Dp <= 128 ? 16 : (a.Dp <= 256 ? 8 : 4);            // q and k of a tile: 16 KB a buffer
  const int cols = PSCAN_THREADS / a.L;
  const size_t smem = (size_t)(4 * a.tile * a.Dp + 2 * a.tile * (cols + 2) + a.tile * PSCAN_THREADS) * sizeof(float);
  const dim3 grid((V + cols - 1) / cols, H, n_seqs);
  if (mode == 0) {
    if (dtype == G2B_F32) launch_scan_prompt<float, 0>(a, grid, smem, stream);
    else launch_scan_prompt<bf16, 0>(a, grid, smem, stream);
  } else if (mode == 1) {
    if (dtype == G2B_F32) launch_scan_prompt<float, 1>(a, grid, smem, stream);
    else launch_scan_prompt<bf16, 1>(a, grid, smem, stream);
  } else if (mode == 2) {
    if (dtype == G2B_F32) launch_scan_prompt<float, 2>(a, grid, smem, stream);
    else launch_scan_prompt<bf16, 2>(a, grid, smem, stream);
  } else {
    G2B_REFUSE("state_scan: unknown mode %d", mode);
  }
  return g2b_check_launch("state_scan_prompt");
}

// ---------------------------------------------------------------------------
// per-head norm of the scan's output, times a gate
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float *__restrict__ o, int T_tokens, int H, int V, const float *__restrict__ w, float eps,
                      const T *__restrict__ gate, int gate_stride, float out_scale, T *__restrict__ out) {
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + warp;
  if (item >= (long long)T_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const float *p = o + (size_t)t * H * V + (size_t)h * V;
  float ss = 0.f;
  for (int j = lane; j < V; j += 32) ss = fmaf(p[j], p[j], ss);
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)V + eps);
  for (int j = lane; j < V; j += 32) {
    float y = p[j] * inv;
    if (w) y *= w[j];
    if (gate) y *= silu_f(to_f32(gate[(size_t)t * gate_stride + (size_t)h * V + j]));
    out[(size_t)t * H * V + (size_t)h * V + j] = from_f32<T>(y * out_scale);
  }
}

extern "C" int g2b_head_norm_gate(const float *o, int T_tokens, int H, int V, const float *w, float eps,
                                  const void *gate, int gate_stride, int dtype, float out_scale, void *out,
                                  cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  const unsigned blocks = (unsigned)(((long long)T_tokens * H + 3) / 4);
  if (dtype == G2B_F32)
    g2b_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, T_tokens, H, V, w, eps,
               (const float *)gate, gate_stride, out_scale, (float *)out);
  else if (dtype == G2B_BF16)
    g2b_launch(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, o, T_tokens, H, V, w, eps,
               (const bf16 *)gate, gate_stride, out_scale, (bf16 *)out);
  else
    G2B_REFUSE("head_norm_gate: unknown dtype %d", dtype);
  return g2b_check_launch("head_norm_gate");
}

// ---------------------------------------------------------------------------
// attention output times sigmoid(gate), element by element; heads lose their padding
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
gate_mul_kernel(const T *__restrict__ o, int hd, const T *__restrict__ gate, int gate_stride, int T_tokens, int H, int V,
                float out_scale, T *__restrict__ out) {
  pdl_launch();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int n = H * V;
  if (i >= (long long)T_tokens * n) return;
  const int t = (int)(i / n), r = (int)(i % n), h = r / V, j = r % V;
  float y = to_f32(o[(size_t)t * H * hd + (size_t)h * hd + j]);
  if (gate) y *= sigmoid_f(to_f32(gate[(size_t)t * gate_stride + r]));
  out[i] = from_f32<T>(y * out_scale);
}

extern "C" int g2b_gate_mul(const void *o, int hd, const void *gate, int gate_stride, int dtype, int T_tokens, int H,
                            int V, float out_scale, void *out, cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  const unsigned blocks = (unsigned)(((long long)T_tokens * H * V + 255) / 256);
  if (dtype == G2B_F32)
    g2b_launch(gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float *)o, hd, (const float *)gate,
               gate_stride, T_tokens, H, V, out_scale, (float *)out);
  else if (dtype == G2B_BF16)
    g2b_launch(gate_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16 *)o, hd, (const bf16 *)gate,
               gate_stride, T_tokens, H, V, out_scale, (bf16 *)out);
  else
    G2B_REFUSE("gate_mul: unknown dtype %d", dtype);
  return g2b_check_launch("gate_mul");
}

// ---------------------------------------------------------------------------
// x += norm(y) * w; the new x once more in the compute type
// ---------------------------------------------------------------------------
#define NORM_ADD_PER 16       // elements a thread keeps of a row of up to 4,096
template <typename T>
__global__ void __launch_bounds__(256)
norm_add_kernel(float *__restrict__ x, const float *__restrict__ y, const float *__restrict__ w, float eps, int Hw,
                T *__restrict__ cast_out) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  float *xr = x + (size_t)t * Hw;
  const bool held = Hw <= 256 * NORM_ADD_PER;          // the row of y stays in registers: one pass over it
  float keep[NORM_ADD_PER];
  float inv = 0.f;
  if (y) {
    const float *yr = y + (size_t)t * Hw;
    float ss = 0.f;
    if (held) {
#pragma unroll
      for (int i = 0; i < NORM_ADD_PER; ++i) {
        const int j = threadIdx.x + 256 * i;
        keep[i] = j < Hw ? yr[j] : 0.f;
        ss = fmaf(keep[i], keep[i], ss);
      }
    } else {
      for (int j = threadIdx.x; j < Hw; j += blockDim.x) ss = fmaf(yr[j], yr[j], ss);
    }
    ss = block_sum(ss, scratch);
    inv = 1.f / sqrtf(ss / (float)Hw + eps);
  }
  if (held) {
#pragma unroll
    for (int i = 0; i < NORM_ADD_PER; ++i) {
      const int j = threadIdx.x + 256 * i;
      if (j < Hw) {
        float v = xr[j];
        if (y) {
          v += (keep[i] * inv) * (w ? w[j] : 1.f);
          xr[j] = v;
        }
        if (cast_out) cast_out[(size_t)t * Hw + j] = from_f32<T>(v);
      }
    }
    return;
  }
  for (int j = threadIdx.x; j < Hw; j += blockDim.x) {
    float v = xr[j];
    if (y) {
      v += (y[(size_t)t * Hw + j] * inv) * (w ? w[j] : 1.f);
      xr[j] = v;
    }
    if (cast_out) cast_out[(size_t)t * Hw + j] = from_f32<T>(v);
  }
}

extern "C" int g2b_norm_add(float *x, const float *y, const float *w, float eps, int T_tokens, int Hw, void *cast_out,
                            int dtype, cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (dtype == G2B_F32)
    g2b_launch(norm_add_kernel<float>, dim3(T_tokens), dim3(256), 0, stream, x, y, w, eps, Hw, (float *)cast_out);
  else if (dtype == G2B_BF16)
    g2b_launch(norm_add_kernel<bf16>, dim3(T_tokens), dim3(256), 0, stream, x, y, w, eps, Hw, (bf16 *)cast_out);
  else
    G2B_REFUSE("norm_add: unknown dtype %d", dtype);
  return g2b_check_launch("norm_add");
}

// ---------------------------------------------------------------------------
// decays and strengths of the gated scan, per token and head, 32-bit
// ---------------------------------------------------------------------------
// Step size of a state-space head: dt = softplus(x + dt_bias); g = exp(-exp(A_log) dt); s = dt.
// gates [T, 2H]: g, then s.
template <typename T>
__global__ void __launch_bounds__(256)
scan_gates_step_kernel(const T *__restrict__ x, int x_stride, const float *__restrict__ A_log,
                       const float *__restrict__ dt_bias, int T_tokens, int H, float *__restrict__ gates) {
  pdl_launch();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)T_tokens * H) return;
  const int t = (int)(i / H), h = (int)(i % H);
  const float dt = softplus_f(to_f32(x[(size_t)t * x_stride + h]) + dt_bias[h]);
  gates[(size_t)t * 2 * H + h] = expf(-expf(A_log[h]) * dt);
  gates[(size_t)t * 2 * H + H + h] = dt;
}

extern "C" int g2b_scan_gates_step(const void *x, int dtype, int x_stride, const float *A_log, const float *dt_bias,
                                   int T_tokens, int H, float *gates, cudaStream_t stream) {
  if (T_tokens <= 0 || H <= 0) return 0;
  const unsigned blocks = (unsigned)(((long long)T_tokens * H + 255) / 256);
  if (dtype == G2B_F32)
    g2b_launch(scan_gates_step_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float *)x, x_stride, A_log, dt_bias,
               T_tokens, H, gates);
  else if (dtype == G2B_BF16)
    g2b_launch(scan_gates_step_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16 *)x, x_stride, A_log, dt_bias,
               T_tokens, H, gates);
  else
    G2B_REFUSE("scan_gates_step: unknown dtype %d", dtype);
  return g2b_check_launch("scan_gates_step");
}

// Exponential gates held stable by a running maximum m (kept per slot and head, from 0):
//   i = cap tanh((x_i + b_i) / cap);  f = logsigmoid(cap tanh((x_f + b_f) / cap));
//   m' = max(f + m, i);  g = exp(f + m - m');  s = exp(i - m').
// gates [T, 2H]: g, then s; m_out [T, H]: m' of every token.  A block walks the tokens of one sequence
// (and of some of its heads) in tiles: the gates of a tile side by side, the chain of maxima by one
// thread per head, then the exponentials side by side again; the chain depends on the tokens before in
// the sequence only.
#define GATES_TILE 1024       // (token, head) pairs of a tile
template <typename T>
__global__ void __launch_bounds__(256)
scan_gates_max_kernel(const T *__restrict__ xi, const T *__restrict__ xf, int x_stride, const float *__restrict__ bi,
                      const float *__restrict__ bf, float cap, int H, float *__restrict__ m_state,
                      const int *__restrict__ seq_slots, const int *__restrict__ seq_meta,
                      float *__restrict__ gates, float *__restrict__ m_out, int heads_per_block) {
  pdl_launch();
  pdl_wait();
  __shared__ float si[GATES_TILE], sf[GATES_TILE], sm_new[GATES_TILE], sm_old[GATES_TILE];
  const int b = blockIdx.x;
  const int first_row = seq_meta ? seq_meta[4 * b + 0] : b, n = seq_meta ? seq_meta[4 * b + 1] : 1;
  const int slot = seq_meta ? seq_meta[4 * b + 3] : seq_slots[b];
  const float inv_cap = 1.f / cap;
  // a block takes `heads_per_block` heads (at most a tile's worth) of one sequence: few heads a block
  // make the tiles long and the chains of many heads run side by side in other blocks
  {
    const int h0 = blockIdx.y * heads_per_block;
    const int Hn = min(heads_per_block, H - h0);
    const int tile = max(1, GATES_TILE / Hn);
    float m = threadIdx.x < Hn ? m_state[(size_t)slot * H + h0 + threadIdx.x] : 0.f;
    float m_hi[GATES_TILE / 256];                     // heads beyond the block's threads
#pragma unroll
    for (int e = 1; e < GATES_TILE / 256; ++e) {
      const int hh = threadIdx.x + 256 * e;
      m_hi[e] = hh < Hn ? m_state[(size_t)slot * H + h0 + hh] : 0.f;
    }
    for (int t0 = 0; t0 < n; t0 += tile) {
      const int nt = min(tile, n - t0);
      __syncthreads();
      for (int idx = threadIdx.x; idx < nt * Hn; idx += blockDim.x) {
        const int tt = idx / Hn, h = h0 + idx % Hn;
        const size_t row = (size_t)(first_row + t0 + tt) * x_stride;
        const float zi = to_f32(xi[row + h]) + bi[h], zf = to_f32(xf[row + h]) + bf[h];
        si[idx] = cap * tanhf(zi * inv_cap);
        const float u = cap * tanhf(zf * inv_cap);
        sf[idx] = fminf(u, 0.f) - log1pf(expf(-fabsf(u)));
      }
      __syncthreads();
#pragma unroll
      for (int e = 0; e < GATES_TILE / 256; ++e) {
        const int hh = threadIdx.x + 256 * e;
        if (hh < Hn) {
          float mm = e == 0 ? m : m_hi[e];
          // eight tokens' gates are fetched before their maxima are chained, so that a link of the
          // chain is an addition and a maximum, not a wait on shared memory
          int tt = 0;
          for (; tt + 8 <= nt; tt += 8) {
            float f8[8], i8[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) f8[u] = sf[(tt + u) * Hn + hh], i8[u] = si[(tt + u) * Hn + hh];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              sm_old[(tt + u) * Hn + hh] = mm;
              mm = fmaxf(f8[u] + mm, i8[u]);
              sm_new[(tt + u) * Hn + hh] = mm;
            }
          }
          for (; tt < nt; ++tt) {
            const int idx = tt * Hn + hh;
            sm_old[idx] = mm;
            mm = fmaxf(sf[idx] + mm, si[idx]);
            sm_new[idx] = mm;
          }
          if (e == 0) m = mm; else m_hi[e] = mm;
        }
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < nt * Hn; idx += blockDim.x) {
        const int tt = idx / Hn, h = h0 + idx % Hn;
        const size_t row = (size_t)(first_row + t0 + tt);
        gates[row * 2 * H + h] = expf(sf[idx] + sm_old[idx] - sm_new[idx]);
        gates[row * 2 * H + H + h] = expf(si[idx] - sm_new[idx]);
        m_out[row * H + h] = sm_new[idx];
      }
    }
    if (threadIdx.x < Hn) m_state[(size_t)slot * H + h0 + threadIdx.x] = m;
#pragma unroll
    for (int e = 1; e < GATES_TILE / 256; ++e) {
      const int hh = threadIdx.x + 256 * e;
      if (hh < Hn) m_state[(size_t)slot * H + h0 + hh] = m_hi[e];
    }
  }
}

extern "C" int g2b_scan_gates_max(const void *xi, const void *xf, int dtype, int x_stride, const float *bi,
                                  const float *bf, float cap, int H, float *m_state, const int *seq_slots,
                                  const int *seq_meta, int n_seqs, float *gates, float *m_out, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0) return 0;
  if (!(cap > 0.f)) G2B_REFUSE("scan_gates_max: the gates' cap must be positive");
  if (!seq_meta && !seq_slots) G2B_REFUSE("scan_gates_max: neither the step's table of sequences nor their slots");
  // prompts: a head a block (its chain is as long as the prompt); single tokens: a sequence's heads together
  const int hb = seq_meta ? 1 : (H < GATES_TILE ? H : GATES_TILE);
  const dim3 grid(n_seqs, (H + hb - 1) / hb);
  if (grid.y > 65535) G2B_REFUSE("scan_gates_max: %d heads are too many for one launch", H);
  if (dtype == G2B_F32)
    g2b_launch(scan_gates_max_kernel<float>, grid, dim3(256), 0, stream, (const float *)xi, (const float *)xf,
               x_stride, bi, bf, cap, H, m_state, seq_slots, seq_meta, gates, m_out, hb);
  else if (dtype == G2B_BF16)
    g2b_launch(scan_gates_max_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16 *)xi, (const bf16 *)xf,
               x_stride, bi, bf, cap, H, m_state, seq_slots, seq_meta, gates, m_out, hb);
  else
    G2B_REFUSE("scan_gates_max: unknown dtype %d", dtype);
  return g2b_check_launch("scan_gates_max");
}

// ---------------------------------------------------------------------------
// what is read out of a scan, made ready for the output product
// ---------------------------------------------------------------------------
// o [T, H, Vs] float, Vs >= V (a head's columns from V on are not output).  Per element j = h V + c:
//   y = o[h, c]
//   m given:      y /= max(|o[h, V]|, exp(-m[t, h])) + den_eps      (column V: the normaliser's read-out)
//   skip given:   y += skip_w[h] * x[j]
//   gate_first:   y *= act(gate[j])
//   y /= sqrt(mean over the element's group of `group` elements of y^2 + eps)
//   y *= w[j mod w_len];  not gate_first: y *= act(gate[j])
// act: 0 silu, 1 sigmoid.  One block per (token, group): a thread takes every 128th element, so that a
// group of a few hundred elements is a few dependent rounds of loads and not sixteen.
template <typename T>
__global__ void __launch_bounds__(128)
state_readout_kernel(const float *__restrict__ o, int T_tokens, int H, int V, int Vs, const float *__restrict__ m,
                     float den_eps, const T *__restrict__ x, int x_stride, const float *__restrict__ skip_w,
                     const T *__restrict__ gate, int gate_stride, int gate_act, int gate_first, int group, float eps,
                     const float *__restrict__ w, int w_len, T *__restrict__ out) {
  pdl_launch();
  pdl_wait();
  __shared__ float part[4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = H * V, groups = n / group;
  const long long item = blockIdx.x;
  const int t = (int)(item / groups), j0 = (int)(item % groups) * group;
  const float *ot = o + (size_t)t * H * Vs;
  auto value = [&](int j) -> float {
    const int h = j / V, c = j - h * V;
    float y = ot[h * Vs + c];
    if (m) y /= fmaxf(fabsf(ot[h * Vs + V]), expf(-m[(size_t)t * H + h])) + den_eps;
    if (skip_w) y = fmaf(skip_w[h], to_f32(x[(size_t)t * x_stride + j]), y);
    if (gate && gate_first) {
      const float z = to_f32(gate[(size_t)t * gate_stride + j]);
      y *= gate_act ? sigmoid_f(z) : silu_f(z);
    }
    return y;
  };
  float ss = 0.f;
  for (int e = threadIdx.x; e < group; e += 128) {
    const float y = value(j0 + e);
    ss = fmaf(y, y, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) part[warp] = ss;
  __syncthreads();
  const float inv = 1.f / sqrtf(((part[0] + part[1]) + (part[2] + part[3])) / (float)group + eps);
  for (int e = threadIdx.x; e < group; e += 128) {
    const int j = j0 + e;
    float y = value(j) * inv;
    if (w) y *= w[j % w_len];
    if (gate && !gate_first) {
      const float z = to_f32(gate[(size_t)t * gate_stride + j]);
      y *= gate_act ? sigmoid_f(z) : silu_f(z);
    }
    out[(size_t)t * n + j] = from_f32<T>(y);
  }
}

extern "C" int g2b_state_readout(const float *o, int T_tokens, int H, int V, int Vs, const float *m, float den_eps,
                                 const void *x, int x_stride, const float *skip_w, const void *gate, int gate_stride,
                                 int gate_act, int gate_first, int group, float eps, const float *w, int w_len,
                                 int dtype, void *out, cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (group <= 0 || (H * V) % group) G2B_REFUSE("state_readout: groups of %d do not divide %d outputs", group, H * V);
  if (Vs < V || (m && Vs <= V)) G2B_REFUSE("state_readout: %d stored columns a head for %d outputs", Vs, V);
  if (w && w_len <= 0) G2B_REFUSE("state_readout: a weight of %d entries", w_len);
  if (skip_w && !x) G2B_REFUSE("state_readout: a skip weight without its input");
  const long long items = (long long)T_tokens * (H * V / group);
  if (items > 0x7fffffffLL) G2B_REFUSE("state_readout: %lld (token, group) pairs are too many for one launch", items);
  const unsigned blocks = (unsigned)items;
  if (dtype == G2B_F32)
    g2b_launch(state_readout_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, T_tokens, H, V, Vs, m, den_eps,
               (const float *)x, x_stride, skip_w, (const float *)gate, gate_stride, gate_act, gate_first, group, eps, w,
               w_len, (float *)out);
  else if (dtype == G2B_BF16)
    g2b_launch(state_readout_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, o, T_tokens, H, V, Vs, m, den_eps,
               (const bf16 *)x, x_stride, skip_w, (const bf16 *)gate, gate_stride, gate_act, gate_first, group, eps, w,
               w_len, (bf16 *)out);
  else
    G2B_REFUSE("state_readout: unknown dtype %d", dtype);
  return g2b_check_launch("state_readout");
}

// ---------------------------------------------------------------------------
// means of whole blocks of keys and values, kept beside the pages
// ---------------------------------------------------------------------------
// A token that ends a block of `pool` positions (pos + 1 a multiple of pool) writes the mean of the
// block's keys and of its values, read back from the pages as they hold them.  Block b lies in the
// page of its first position, page_table[(b pool) / page_size], at row b - ceil(first position of
// that page / pool); a page of the pooled store has `rows` rows: [pages, 2, nkv, rows, hd].
template <typename T>
__global__ void __launch_bounds__(128)
pool_update_kernel(const T *__restrict__ cache, T *__restrict__ pooled, const int *__restrict__ tok_pos,
                   const int *__restrict__ tok_seq, const int *__restrict__ page_table, int P, int nkv, int hd,
                   int page_size, int pool, int rows) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, kvh = blockIdx.y;
  const int pos = tok_pos[t];
  if ((pos + 1) % pool) return;
  const int b = (pos + 1) / pool - 1;
  const int *pt = page_table + (size_t)tok_seq[t] * P;
  const int home = (b * pool) / page_size;
  const int row = b - (home * page_size + pool - 1) / pool;
  const size_t panel = (size_t)page_size * hd, ppanel = (size_t)rows * hd;
  const float inv = 1.f / (float)pool;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float sk = 0.f, sv = 0.f;
    for (int r = 0; r < pool; ++r) {
      const int p = b * pool + r;
      const size_t page = (size_t)pt[p / page_size];
      const size_t at = (size_t)(p % page_size) * hd + d;
      sk += to_f32(cache[((page * 2 + 0) * nkv + kvh) * panel + at]);
      sv += to_f32(cache[((page * 2 + 1) * nkv + kvh) * panel + at]);
    }
    const size_t page = (size_t)pt[home];
    pooled[((page * 2 + 0) * nkv + kvh) * ppanel + (size_t)row * hd + d] = from_f32<T>(sk * inv);
    pooled[((page * 2 + 1) * nkv + kvh) * ppanel + (size_t)row * hd + d] = from_f32<T>(sv * inv);
  }
}

extern "C" int g2b_pool_update(const void *cache, void *pooled, int dtype, const int *tok_pos, const int *tok_seq,
                               const int *page_table, int P, int T_tokens, int nkv, int hd, int page_size, int pool,
                               int rows, cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (pool <= 0 || rows < (page_size + pool - 1) / pool)
    G2B_REFUSE("pool_update: %d rows a page do not hold the blocks of %d positions of a page of %d", rows, pool, page_size);
  if (nkv > 65535) G2B_REFUSE("pool_update: %d kv heads are too many for one launch", nkv);
  const dim3 grid(T_tokens, nkv);
  if (dtype == G2B_F32)
    g2b_launch(pool_update_kernel<float>, grid, dim3(128), 0, stream, (const float *)cache, (float *)pooled, tok_pos, tok_seq,
               page_table, P, nkv, hd, page_size, pool, rows);
  else if (dtype == G2B_BF16)
    g2b_launch(pool_update_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16 *)cache, (bf16 *)pooled, tok_pos, tok_seq,
               page_table, P, nkv, hd, page_size, pool, rows);
  else
    G2B_REFUSE("pool_update: unknown dtype %d", dtype);
  return g2b_check_launch("pool_update");
}

// ---------------------------------------------------------------------------
// selective scan: a decay per state entry
// ---------------------------------------------------------------------------
// A channel's N state entries are held by L lanes of one warp, at most P each: lane l holds entries
// l, l + L, ...  A block owns SEL_THREADS / L channels of one sequence and walks the step's tokens
// in order, SEL_TILE at a time.  The whole block stages a tile in shared memory: (B_n, C_n) pairs, and per
// channel (dt, dt x) with the softplus applied, and x.  Then every lane runs its entries through the
// tile: the only chain from token to token is one multiply-add per entry; a lane's share of a read-out
// goes to shared memory, and after the tile one thread per (token, channel) adds the L shares in lane
// order (an order that depends on N and L only), adds the skip, applies the gate and the scale and
// writes the output.  What a token gets depends on the tokens before it in its sequence only.  The
// launcher picks P as small as the step's size allows, so that a prompt of one sequence still fills
// the GPU with threads (P = 1: a lane an entry).
#define SEL_THREADS 128
#define SEL_TILE 16

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// `AHEAD`: the next tile's rows are fetched into registers while the current tile is computed (two (token,
// channel) elements and eight B | C values a thread hold a tile when a channel has 8 to 32 lanes and at most 32
// entries); otherwise a tile is fetched when its turn comes.
template <typename T, int MAXP, bool AHEAD>
__global__ void __launch_bounds__(SEL_THREADS)
selective_scan_kernel(const T *__restrict__ x, int x_stride, const float *__restrict__ dt_raw, int dt_stride,
                      const float *__restrict__ dt_bias, const T *__restrict__ bc, int bc_stride,
                      const float *__restrict__ A, const float *__restrict__ skip, const T *__restrict__ z,
                      int z_stride, float *__restrict__ state, const int *__restrict__ seq_slots,
                      const int *__restrict__ seq_meta, int inner, int N, int L, int log_cpb, float out_scale,
                      T *__restrict__ out, int out_stride) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float sm[];
  const int cpb = 1 << log_cpb;                          // channels of this block: its threads / L
  const int n_threads = blockDim.x, n_warps = blockDim.x >> 5;
  float2 *bcs = reinterpret_cast<float2 *>(sm);          // [SEL_TILE][N]: (B_n, C_n)
  float2 *dtx = bcs + (size_t)SEL_TILE * N;              // [SEL_TILE][cpb]: (dt, dt x)
  float *xs = reinterpret_cast<float *>(dtx + SEL_TILE * cpb);       // [SEL_TILE][cpb]
  float *part = xs + SEL_TILE * cpb;                     // [SEL_TILE][cpb][L + 1]: the lanes' shares of y
  const int b = blockIdx.y;
  const int first = seq_meta ? seq_meta[4 * b + 0] : b;
  const int n_tok = seq_meta ? seq_meta[4 * b + 1] : 1;
  const int slot = seq_meta ? seq_meta[4 * b + 3] : seq_slots[b];
  const int c0 = blockIdx.x * cpb;
  const int cl = threadIdx.x / L, sub = threadIdx.x % L;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = c0 + cl;
  const bool live = c < inner;
  float S[MAXP], a[MAXP];
  float *my_state = state + ((size_t)slot * inner + (live ? c : 0)) * N;
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int n = sub + L * i;
    const bool has = live && n < N;
    S[i] = has ? my_state[n] : 0.f;
    a[i] = has ? A[(size_t)c * N + n] * 1.4426950408889634f : 0.f;     // exp(dt a) = 2^(dt a log2 e)
  }
  float *my_part = part + (size_t)cl * (L + 1) + sub;
  const int part_row = cpb * (L + 1);
  // AHEAD: element k of a thread is (token r, channel ch) with i = threadIdx.x + k * 128 = r * cpb + (ch - c0), and
  // B | C value k is row warp + 4 (k / 2), column lane + 32 (k % 2)
  float f_dt[2], f_x[2], f_z[2], z_now[2], f_bc[8], e_bias[2], e_skip[2];
  auto fetch = [&](int t0) {
    const int here = min(SEL_TILE, n_tok - t0);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = threadIdx.x + k * SEL_THREADS, r = i >> log_cpb, ch = c0 + (i & (cpb - 1));
      f_dt[k] = f_x[k] = f_z[k] = 0.f;
      if (i < (here << log_cpb) && ch < inner) {
        const size_t row = (size_t)(first + t0 + r);
        f_dt[k] = dt_raw[row * dt_stride + ch];
        f_x[k] = to_f32(x[row * x_stride + ch]);
        f_z[k] = to_f32(z[row * z_stride + ch]);
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int r = warp + 4 * (k >> 1), j = lane + 32 * (k & 1);
      f_bc[k] = (r < here && j < 2 * N) ? to_f32(bc[(size_t)(first + t0 + r) * bc_stride + j]) : 0.f;
    }
  };
  if (AHEAD) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int ch = c0 + ((threadIdx.x + k * SEL_THREADS) & (cpb - 1));
      e_bias[k] = ch < inner ? dt_bias[ch] : 0.f;
      e_skip[k] = ch < inner ? skip[ch] : 0.f;
    }
    fetch(0);
  }
  for (int t0 = 0; t0 < n_tok; t0 += SEL_TILE) {
    const int here = min(SEL_TILE, n_tok - t0);
    __syncthreads();                                     // the tile before has left shared memory
    if (AHEAD) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int r = warp + 4 * (k >> 1), j = lane + 32 * (k & 1);
        if (r < here && j < 2 * N)
          reinterpret_cast<float *>(bcs + (size_t)r * N)[j < N ? 2 * j : 2 * (j - N) + 1] = f_bc[k];
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int i = threadIdx.x + k * SEL_THREADS;
        if (i < (here << log_cpb)) {
          const float dt = softplus_f(f_dt[k] + e_bias[k]);
          dtx[i] = make_float2(dt, dt * f_x[k]);
          xs[i] = f_x[k];
        }
        z_now[k] = f_z[k];
      }
      __syncthreads();
      if (t0 + SEL_TILE < n_tok) fetch(t0 + SEL_TILE);   // under way while this tile is computed
    } else {
      for (int r = warp; r < here; r += n_warps) {                 // a warp a row of B | C
        const T *row = bc + (size_t)(first + t0 + r) * bc_stride;
        float *dst = reinterpret_cast<float *>(bcs + (size_t)r * N);
        for (int j = lane; j < 2 * N; j += 32) dst[j < N ? 2 * j : 2 * (j - N) + 1] = to_f32(row[j]);
      }
      for (int i = threadIdx.x; i < (here << log_cpb); i += n_threads) {
        const int r = i >> log_cpb, ch = c0 + (i & (cpb - 1));
        float dt = 0.f, xv = 0.f;
        if (ch < inner) {
          const size_t row = (size_t)(first + t0 + r);
          dt = softplus_f(dt_raw[row * dt_stride + ch] + dt_bias[ch]);
          xv = to_f32(x[row * x_stride + ch]);
        }
        dtx[i] = make_float2(dt, dt * xv);
        xs[i] = xv;
      }
      __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < SEL_TILE; ++r) {                 // lanes beyond the last channel run along on zeros
      if (r < here) {
        const float2 d = dtx[(r << log_cpb) + cl];
        float y = 0.f;
#pragma unroll
        for (int i = 0; i < MAXP; ++i) {
          const int n = sub + L * i;
          if (n < N) {
            const float2 bcn = bcs[(size_t)r * N + n];
            S[i] = fmaf(ex2_approx(d.x * a[i]), S[i], d.y * bcn.x);
            y = fmaf(S[i], bcn.y, y);
          }
        }
        my_part[r * part_row] = y;
      }
    }
    __syncthreads();
    if (AHEAD) {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int i = threadIdx.x + k * SEL_THREADS, r = i >> log_cpb, ch = c0 + (i & (cpb - 1));
        if (i < (here << log_cpb) && ch < inner) {
          const float *p = part + (size_t)i * (L + 1);
          float y = 0.f;
          for (int l = 0; l < L; ++l) y += p[l];
          out[(size_t)(first + t0 + r) * out_stride + ch] =
              from_f32<T>((y + e_skip[k] * xs[i]) * silu_f(z_now[k]) * out_scale);
        }
      }
    } else {
      for (int i = threadIdx.x; i < (here << log_cpb); i += n_threads) {
        const int r = i >> log_cpb, ch = c0 + (i & (cpb - 1));
        if (ch < inner) {
          const float *p = part + (size_t)i * (L + 1);
          float y = 0.f;
          for (int l = 0; l < L; ++l) y += p[l];
          const size_t row = (size_t)(first + t0 + r);
          const float g = to_f32(z[row * z_stride + ch]);
          out[row * out_stride + ch] = from_f32<T>((y + skip[ch] * xs[i]) * silu_f(g) * out_scale);
        }
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int n = sub + L * i;
      if (n < N) my_state[n] = S[i];
    }
  }
}

extern "C" int g2b_selective_scan(const void *x, int dtype, int x_stride, const float *dt_raw, int dt_stride,
                                  const float *dt_bias, const void *bc, int bc_stride, const float *A,
                                  const float *skip, const void *z, int z_stride, float *state,
                                  const int *seq_slots, const int *seq_meta, int T_tokens, int n_seqs, int inner,
                                  int N, float out_scale, void *out, int out_stride, cudaStream_t stream) {
  if (T_tokens <= 0 || inner <= 0) return 0;
  if (N <= 0 || N > 256) G2B_REFUSE("selective_scan: a state of %d entries a channel (1..256)", N);
  const int seqs = seq_meta ? n_seqs : T_tokens;
  if (seqs > 65535) G2B_REFUSE("selective_scan: %d sequences are too many for one launch", seqs);
  // entries a lane: as few as keep the launch within a few hundred thousand threads (what the GPU holds at
  // once), and at least what 32 lanes a channel leave; depends on the step's sizes only, never on its data
  int maxp = N > 128 ? 8 : N > 64 ? 4 : N > 32 ? 2 : 1;
  auto lanes = [&](int p) { int l = 1; while (l * p < N) l <<= 1; return l; };
  while (maxp < 8 && (long long)seqs * inner * lanes(maxp) > 300000LL) maxp <<= 1;
  const int L = lanes(maxp);                             // lanes a channel: 1 .. 32
  // 128 threads a block: blocks of 64 and 32 threads stage the same B and C rows for fewer channels and were
  // slower (2,048 tokens, 4,096 channels of 16 entries: 535 us against 750 and 1,010)
  const int threads = SEL_THREADS;
  const int cpb = threads / L;
  const dim3 grid((inner + cpb - 1) / cpb, seqs);
  int log_cpb = 0;
  while ((1 << log_cpb) < cpb) ++log_cpb;
  const size_t smem = ((size_t)SEL_TILE * 2 * N + 3 * (size_t)SEL_TILE * cpb + (size_t)SEL_TILE * cpb * (L + 1)) * sizeof(float);
  // a tile ahead in registers: prompts only, a (token, channel) tile of at most 256 elements, B | C rows of at most 64
  const bool ahead = seq_meta && T_tokens > seqs && L >= 8 && N <= 32;
#define G2B_SEL(TYPE, MAXP, AHEAD)                                                                                 \
  g2b_launch(selective_scan_kernel<TYPE, MAXP, AHEAD>, grid, dim3(threads), smem, stream, (const TYPE *)x,         \
             x_stride, dt_raw, dt_stride, dt_bias, (const TYPE *)bc, bc_stride, A, skip, (const TYPE *)z, z_stride, \
             state, seq_slots, seq_meta, inner, N, L, log_cpb, out_scale, (TYPE *)out, out_stride)
#define G2B_SEL_P(TYPE)                                                                                            \
  do {                                                                                                             \
    if (ahead && maxp == 1) G2B_SEL(TYPE, 1, true); else if (ahead && maxp == 2) G2B_SEL(TYPE, 2, true);           \
    else if (ahead) G2B_SEL(TYPE, 4, true);                                                                        \
    else if (maxp == 1) G2B_SEL(TYPE, 1, false); else if (maxp == 2) G2B_SEL(TYPE, 2, false);                      \
    else if (maxp == 4) G2B_SEL(TYPE, 4, false); else G2B_SEL(TYPE, 8, false);                                     \
  } while (0)
  if (dtype == G2B_F32) G2B_SEL_P(float);
  else if (dtype == G2B_BF16) G2B_SEL_P(bf16);
  else G2B_REFUSE("selective_scan: unknown dtype %d", dtype);
#undef G2B_SEL_P
#undef G2B_SEL
  return g2b_check_launch("selective_scan");
}

// ---------------------------------------------------------------------------
// two attention maps per head, the second subtracted
// ---------------------------------------------------------------------------
// a [T, 2 * heads * hd]: the first map's heads, then the second's (heads padded to hd entries, V in
// use); out[t, h] = (a1 - lambda a2) / sqrt(mean((a1 - lambda a2)^2) + eps) * post, heads unpadded.
template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const T *__restrict__ a, int heads, int hd, int V, float lambda, float eps, float post,
                    T *__restrict__ out, int n_items) {
  pdl_launch();
  pdl_wait();
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n_items) return;
  const int t = item / heads, h = item % heads;
  const T *a1 = a + ((size_t)t * 2 * heads + h) * hd, *a2 = a1 + (size_t)heads * hd;
  float ss = 0.f;
  for (int d = lane; d < V; d += 32) {
    const float o = to_f32(a1[d]) - lambda * to_f32(a2[d]);
    ss = fmaf(o, o, ss);
  }
  const float inv = post / sqrtf(warp_sum(ss) / (float)V + eps);
  T *op = out + ((size_t)t * heads + h) * V;
  for (int d = lane; d < V; d += 32) op[d] = from_f32<T>((to_f32(a1[d]) - lambda * to_f32(a2[d])) * inv);
}

extern "C" int g2b_diff_combine(const void *a, int dtype, int T_tokens, int heads, int hd, int V, float lambda,
                                float eps, float post, void *out, cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (V <= 0 || V > hd) G2B_REFUSE("diff_combine: %d values of a head stored in %d", V, hd);
  const int items = T_tokens * heads;
  if (dtype == G2B_F32)
    g2b_launch(diff_combine_kernel<float>, dim3((items + 3) / 4), dim3(128), 0, stream, (const float *)a, heads, hd, V,
               lambda, eps, post, (float *)out, items);
  else if (dtype == G2B_BF16)
    g2b_launch(diff_combine_kernel<bf16>, dim3((items + 3) / 4), dim3(128), 0, stream, (const bf16 *)a, heads, hd, V,
               lambda, eps, post, (bf16 *)out, items);
  else
    G2B_REFUSE("diff_combine: unknown dtype %d", dtype);
  return g2b_check_launch("diff_combine");
}
