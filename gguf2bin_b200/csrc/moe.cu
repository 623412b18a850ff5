// A routed feed-forward: every token goes through `top` of a layer's small feed-forwards.
//
//   moe_route    scores s = softmax(z) over all experts (or sigmoid(z), each by itself) in 32-bit;
//                optionally only the experts of the best groups of neighbours stay eligible; the `top` largest of s + c
//                (c: a stored correction that steers the choice only) are chosen, ties to the
//                lower index; the weights are the chosen experts' s as they are, or divided by
//                their sum; then times `scale`.  idx [T, top], weight [T, top].
//   moe_plan     the step's (token, choice) pairs grouped by expert: how many rows every expert
//                gets, where its rows start, which pair sits in which row, and the list of row
//                tiles that the products walk.  Experts from `n_real` on have no matrices (their
//                output is their input); their pairs get no row.
//   moe_gemm     one product per expert over its rows: out = A_rows . W_e^T, the rows of A
//                gathered by the plan; with `swiglu` W_e holds gate rows then up rows and the
//                output is silu(gate) * up.  32-bit accumulation; a row's sum runs over k in
//                ascending order whatever else is in the tile.
//   moe_combine  y_t = sum_j weight_tj * (row of pair (t, j), or the token's own input for an
//                expert without matrices), added in the order of j; stored, or added to what is there.
//
// Which row of an expert's range a pair lands in depends on the batch (the plan hands rows out
// with atomic counters); what is computed for the pair does not: a row of a product depends on
// that row alone, and the combination adds a token's choices in the order of the choice.
#include "common.cuh"
#include "mma.cuh"

G2B_DEFINE_LAST_ERROR

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// Row of a gate/up matrix [2N, K] that holds gate (s = 0) or up (s = 1) row n: all gates and then all ups
// (`blocked` = 0), or eight gates and the eight ups of the same outputs in turn (`blocked` = 1, the
// layout whose neighbours a tensor-core epilogue combines).  Plain matrices pass s = 0, blocked = 0.
__device__ __forceinline__ size_t gu_row(int s, int n, int N, int blocked) {
  return blocked ? (size_t)((n >> 3) << 4) + (s << 3) + (n & 7) : (size_t)s * N + n;
}

// rows gathered side by side, in the plan's order, for the kernels that fetch tiles by address
template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const T *__restrict__ A, int a_stride, const int *__restrict__ row_pair, int pairs_per_token,
                  const int *__restrict__ plan, int n_real, int K, T *__restrict__ out) {
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= plan[1 + n_real]) return;
  const T *src = A + (size_t)(row_pair[r] / pairs_per_token) * a_stride;
  T *dst = out + (size_t)r * K;
  if ((K * sizeof(T)) % 16 == 0 && (a_stride * sizeof(T)) % 16 == 0) {
    const int n16 = K * (int)sizeof(T) / 16;
    for (int i = threadIdx.x; i < n16; i += blockDim.x) ((uint4 *)dst)[i] = ((const uint4 *)src)[i];
  } else {
    for (int i = threadIdx.x; i < K; i += blockDim.x) dst[i] = src[i];
  }
}

extern "C" int g2b_moe_gather(const void *A, int dtype, int a_stride, const int *row_pair, int pairs_per_token,
                              const int *plan, int n_real, int n_rows, int K, void *out, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dtype == G2B_F32)
    g2b_launch(moe_gather_kernel<float>, dim3(n_rows), dim3(256), 0, stream, (const float *)A, a_stride, row_pair,
               pairs_per_token, plan, n_real, K, (float *)out);
  else if (dtype == G2B_BF16)
    g2b_launch(moe_gather_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, (const bf16 *)A, a_stride, row_pair,
               pairs_per_token, plan, n_real, K, (bf16 *)out);
  else
    G2B_REFUSE("moe_gather: unknown dtype %d", dtype);
  return g2b_check_launch("moe_gather");
}

// ---------------------------------------------------------------------------
// router
// ---------------------------------------------------------------------------
#define ROUTE_WARPS 4
// `sigmoid`: the scores are sigmoids of the logits, each by itself, instead of a softmax over all.
// `groups` > 1: the experts form that many equal groups of neighbours; a group's score is the sum of its
// two largest scores (of score + correction); only experts of the `keep` best groups can be chosen.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float *__restrict__ z, const float *__restrict__ correction, int T, int N, int top,
                 int renormalise, int *__restrict__ idx, float *__restrict__ weight, float scale, int sigmoid,
                 int groups, int keep) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float sm[];                 // per warp: s [N], pick [N], group scores [groups]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  float *s = sm + (size_t)warp * (2 * N + groups), *pick = s + N, *gs = pick + N;
  const float *zr = z + (size_t)t * N;
  if (sigmoid) {
    for (int j = lane; j < N; j += 32) {
      s[j] = 1.f / (1.f + expf(-zr[j]));
      pick[j] = s[j] + (correction ? correction[j] : 0.f);
    }
  } else {
    float m = -INFINITY;
    for (int j = lane; j < N; j += 32) m = fmaxf(m, zr[j]);
    m = warp_max(m);
    float sum = 0.f;
    for (int j = lane; j < N; j += 32) {
      const float e = expf(zr[j] - m);
      s[j] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int j = lane; j < N; j += 32) {
      s[j] *= inv;
      pick[j] = s[j] + (correction ? correction[j] : 0.f);
    }
  }
  __syncwarp();
  if (groups > 1) {
    const int per = N / groups;
    for (int g = lane; g < groups; g += 32) {     // the sum of a group's two best
      float a = -INFINITY, b = -INFINITY;
      for (int j = g * per; j < (g + 1) * per; ++j) {
        const float v = pick[j];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gs[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    for (int r = 0; r < keep; ++r) {              // the best groups, one after another; ties to the lower index
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (gs[g] > best) { best = gs[g]; at = g; }
      for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oa = __shfl_xor_sync(0xffffffffu, at, off);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (at >= groups) break;                    // nothing left (NaN scores): every lane agrees
      if (lane == 0) gs[at] = -INFINITY;          // taken: marked by the value no score has
      __syncwarp();
    }
    for (int j = lane; j < N; j += 32)
      if (gs[j / per] != -INFINITY) pick[j] = -INFINITY;      // its group was not kept
    __syncwarp();
  }
  float chosen_sum = 0.f;
  for (int r = 0; r < top; ++r) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int j = lane; j < N; j += 32)
      if (pick[j] > best) { best = pick[j]; at = j; }
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oa = __shfl_xor_sync(0xffffffffu, at, off);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at >= N) at = 0;                        // all NaN: never read outside
    if (lane == 0) {
      idx[(size_t)t * top + r] = at;
      weight[(size_t)t * top + r] = renormalise ? s[at] : s[at] * scale;
      pick[at] = -INFINITY;
    }
    chosen_sum += s[at];
    __syncwarp();
  }
  if (renormalise && lane == 0)
    for (int r = 0; r < top; ++r)
      weight[(size_t)t * top + r] = weight[(size_t)t * top + r] / (chosen_sum + 1e-20f) * scale;
}

extern "C" int g2b_moe_route(const float *z, const float *correction, int T, int N, int top, int renormalise,
                             int *idx, float *weight, float scale, int sigmoid, int groups, int keep,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top < 1 || top > N) G2B_REFUSE("moe_route: %d choices among %d experts", top, N);
  if (groups < 1) groups = 1;
  if (groups > 1 && (N % groups || keep < 1 || keep > groups || top > keep * (N / groups)))
    G2B_REFUSE("moe_route: %d experts in %d groups of which %d are kept, for %d choices", N, groups, keep, top);
  const size_t smem = (size_t)ROUTE_WARPS * (2 * N + groups) * sizeof(float);
  if (smem > 48 * 1024) G2B_REFUSE("moe_route: %d experts are more than a block's shared memory holds", N);
  g2b_launch(moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream, z,
             correction, T, N, top, renormalise, idx, weight, scale, sigmoid, groups, keep);
  return g2b_check_launch("moe_route");
}

// ---------------------------------------------------------------------------
// plan: one block
// ---------------------------------------------------------------------------
#define PLAN_MAX_EXPERTS 1024
// plan layout (int32): [0] tiles in use, [1..E+1] first row of each expert (and the end),
// then the tiles as (expert, first row, rows) triples from word PLAN_TILES_AT(E) on
#define PLAN_TILES_AT(E) ((E) + 2)

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int *__restrict__ idx, int n_pairs, int n_real, int tile_rows, int max_tiles,
                int *__restrict__ plan, int *__restrict__ row_pair, int *__restrict__ pair_row) {
  pdl_launch();
  pdl_wait();
  __shared__ int count[PLAN_MAX_EXPERTS], start[PLAN_MAX_EXPERTS + 1], cursor[PLAN_MAX_EXPERTS];
  for (int e = threadIdx.x; e < n_real; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < n_real) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    int *tl = plan + PLAN_TILES_AT(n_real);
    for (int e = 0; e < n_real; ++e) {
      start[e] = at;
      plan[1 + e] = at;
      for (int r = 0; r < count[e] && tiles < max_tiles; r += tile_rows, ++tiles) {
        tl[3 * tiles + 0] = e;
        tl[3 * tiles + 1] = at + r;
        tl[3 * tiles + 2] = min(tile_rows, count[e] - r);
      }
      at += count[e];
    }
    start[n_real] = at;
    plan[1 + n_real] = at;
    plan[0] = tiles;
  }
  for (int e = threadIdx.x; e < n_real; e += blockDim.x) cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    int row = -1;
    if (e >= 0 && e < n_real) {
      row = start[e] + atomicAdd(&cursor[e], 1);
      row_pair[row] = p;
    }
    pair_row[p] = row;
  }
}

extern "C" int g2b_moe_plan(const int *idx, int n_pairs, int n_real, int tile_rows, int max_tiles, int *plan,
                            int *row_pair, int *pair_row, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (n_real < 0 || n_real > PLAN_MAX_EXPERTS) G2B_REFUSE("moe_plan: %d experts outside 0..%d", n_real, PLAN_MAX_EXPERTS);
  g2b_launch(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, idx, n_pairs, n_real, tile_rows, max_tiles, plan, row_pair,
             pair_row);
  return g2b_check_launch("moe_plan");
}

// ---------------------------------------------------------------------------
// one product per expert over its rows (CUDA cores, any type)
// ---------------------------------------------------------------------------
#define MG_BM 32
#define MG_BN 64
#define MG_BK 16
// 128 threads: thread (ty, tx) = (i / 16, i % 16) owns rows ty*4..+3 and columns tx + 16*j, j < 4

template <typename T, bool SWIGLU>
__global__ void __launch_bounds__(128)
moe_gemm_kernel(const T *__restrict__ A, int a_stride, const int *__restrict__ row_pair, int pairs_per_token,
                const T *__restrict__ W, int N, int K, const int *__restrict__ plan, int n_real,
                void *__restrict__ out, int out_f32, int blocked) {
  pdl_launch();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int *tl = plan + PLAN_TILES_AT(n_real) + 3 * tile;
  const int e = tl[0], row0 = tl[1], rows = tl[2];
  const int n0 = blockIdx.x * MG_BN;
  __shared__ float As[MG_BK][MG_BM + 1];
  __shared__ float Bs[SWIGLU ? 2 : 1][MG_BK][MG_BN + 1];
  __shared__ int src_row[MG_BM];
  const int tid = threadIdx.x;
  if (tid < MG_BM) {
    int r = -1;
    if (tid < rows) r = row_pair ? row_pair[row0 + tid] / pairs_per_token : row0 + tid;
    src_row[tid] = r;
  }
  __syncthreads();
  const int ty = tid / 16, tx = tid % 16;
  const size_t w_rows = SWIGLU ? 2 * (size_t)N : (size_t)N;
  const T *We = W + (size_t)e * w_rows * K;
  float acc[SWIGLU ? 2 : 1][4][4];
#pragma unroll
  for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[s][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += MG_BK) {
    for (int i = tid; i < MG_BM * MG_BK; i += 128) {
      const int r = i / MG_BK, kk = i % MG_BK;
      const int sr = src_row[r];
      As[kk][r] = (sr >= 0 && k0 + kk < K) ? to_f32(A[(size_t)sr * a_stride + k0 + kk]) : 0.f;
    }
    for (int i = tid; i < MG_BN * MG_BK; i += 128) {
      const int c = i / MG_BK, kk = i % MG_BK;
      const bool in = n0 + c < N && k0 + kk < K;
      Bs[0][kk][c] = in ? to_f32(We[gu_row(0, n0 + c, N, SWIGLU ? blocked : 0) * K + k0 + kk]) : 0.f;
      if (SWIGLU) Bs[1][kk][c] = in ? to_f32(We[gu_row(1, n0 + c, N, blocked) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MG_BK; ++kk) {
      float av[4], bv[SWIGLU ? 2 : 1][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[s][j] = Bs[s][kk][tx + 16 * j];
#pragma unroll
      for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[s][i][j] = fmaf(av[i], bv[s][j], acc[s][i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx + 16 * j;
      if (c >= N) continue;
      const float v = SWIGLU ? silu_f(acc[0][i][j]) * acc[SWIGLU ? 1 : 0][i][j] : acc[0][i][j];
      const size_t at = (size_t)(row0 + r) * N + c;
      if (out_f32) ((float *)out)[at] = v;
      else ((T *)out)[at] = from_f32<T>(v);
    }
  }
}

// ---------------------------------------------------------------------------
// the same on the tensor cores (bfloat16, mma.sync m16n8k16): a tile of 32 rows x 64 columns,
// four warps side by side, each 32 x 16
// ---------------------------------------------------------------------------
#define MT_BK 32
#define MT_PAD 8
template <bool SWIGLU>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const bf16 *__restrict__ A, int a_stride, const int *__restrict__ row_pair, int pairs_per_token,
                    const bf16 *__restrict__ W, int N, int K, const int *__restrict__ plan, int n_real,
                    void *__restrict__ out, int out_f32, int blocked) {
  pdl_launch();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int *tl = plan + PLAN_TILES_AT(n_real) + 3 * tile;
  const int e = tl[0], row0 = tl[1], rows = tl[2];
  const int n0 = blockIdx.x * MG_BN;
  constexpr int S = SWIGLU ? 2 : 1;
  __shared__ __align__(16) bf16 As[MG_BM][MT_BK + MT_PAD];
  __shared__ __align__(16) bf16 Bs[S][MG_BN][MT_BK + MT_PAD];
  __shared__ int src_row[MG_BM];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < MG_BM) {
    int r = -1;
    if (tid < rows) r = row_pair ? row_pair[row0 + tid] / pairs_per_token : row0 + tid;
    src_row[tid] = r;
  }
  __syncthreads();
  const bf16 *We = W + (size_t)e * (size_t)S * N * K;
  float acc[S][2][2][4];                        // [gate|up][16-row block][8-column block][fragment]
#pragma unroll
  for (int s = 0; s < S; ++s)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int f = 0; f < 4; ++f) acc[s][i][j][f] = 0.f;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int k0 = 0; k0 < K; k0 += MT_BK) {       // K is a multiple of 8: 16-byte pieces
    for (int i = tid; i < MG_BM * (MT_BK / 8); i += 128) {
      const int r = i / (MT_BK / 8), p = i % (MT_BK / 8);
      const int sr = src_row[r];
      uint4 v = zero;
      if (sr >= 0 && k0 + p * 8 < K) v = *(const uint4 *)(A + (size_t)sr * a_stride + k0 + p * 8);
      *(uint4 *)&As[r][p * 8] = v;
    }
    for (int i = tid; i < S * MG_BN * (MT_BK / 8); i += 128) {
      const int s = i / (MG_BN * (MT_BK / 8)), c = (i / (MT_BK / 8)) % MG_BN, p = i % (MT_BK / 8);
      uint4 v = zero;
      if (n0 + c < N && k0 + p * 8 < K) v = *(const uint4 *)(We + gu_row(s, n0 + c, N, SWIGLU ? blocked : 0) * K + k0 + p * 8);
      *(uint4 *)&Bs[s][c][p * 8] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MT_BK; kk += 16) {
      const int g = lane >> 2, q = lane & 3;
      uint32_t a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        a[i][0] = *(const uint32_t *)&As[16 * i + g][kk + 2 * q];
        a[i][1] = *(const uint32_t *)&As[16 * i + g + 8][kk + 2 * q];
        a[i][2] = *(const uint32_t *)&As[16 * i + g][kk + 2 * q + 8];
        a[i][3] = *(const uint32_t *)&As[16 * i + g + 8][kk + 2 * q + 8];
      }
#pragma unroll
      for (int s = 0; s < S; ++s)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int c = warp * 16 + 8 * j + g;
          uint32_t b[2];
          b[0] = *(const uint32_t *)&Bs[s][c][kk + 2 * q];
          b[1] = *(const uint32_t *)&Bs[s][c][kk + 2 * q + 8];
#pragma unroll
          for (int i = 0; i < 2; ++i) mma_bf16_16816(acc[s][i][j], a[i], b[0], b[1]);
        }
    }
    __syncthreads();
  }
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int r = 16 * i + g + (f >> 1) * 8;
        const int c = n0 + warp * 16 + 8 * j + 2 * q + (f & 1);
        if (r >= rows || c >= N) continue;
        const float v = SWIGLU ? silu_f(acc[0][i][j][f]) * acc[S - 1][i][j][f] : acc[0][i][j][f];
        const size_t at = (size_t)(row0 + r) * N + c;
        if (out_f32) ((float *)out)[at] = v;
        else ((bf16 *)out)[at] = __float2bfloat16_rn(v);
      }
}

// ---------------------------------------------------------------------------
// many rows per expert: tiles of 128 rows x 64 columns, eight warps (4 x 2, each 32 x 32), operands
// fetched one k-step ahead with cp.async, fragments read with ldmatrix
// ---------------------------------------------------------------------------
#define MW_BM 128
#define MW_BK 32
#define MW_LD (MW_BK + 8)
template <bool SWIGLU>
__global__ void __launch_bounds__(256)
moe_gemm_wide_kernel(const bf16 *__restrict__ A, int a_stride, const int *__restrict__ row_pair, int pairs_per_token,
                     const bf16 *__restrict__ W, int N, int K, const int *__restrict__ plan, int n_real,
                     void *__restrict__ out, int out_f32, int blocked) {
  pdl_launch();
  pdl_wait();
  constexpr int S = SWIGLU ? 2 : 1;
  __shared__ __align__(16) bf16 As[2][MW_BM][MW_LD];
  __shared__ __align__(16) bf16 Bs[2][S][MG_BN][MW_LD];
  __shared__ int src_row[MW_BM];
  // the plan's tiles are MG_BM rows; this kernel takes MW_BM / MG_BM of them at a time when they follow
  // one another in ONE expert's range: blockIdx.y counts groups of plan tiles, and a group that starts
  // inside an expert's range but is not its first of this size is skipped
  const int per = MW_BM / MG_BM;
  const int tile = blockIdx.y;
  const int n_tiles = plan[0];
  if (tile >= n_tiles) return;
  const int *tl = plan + PLAN_TILES_AT(n_real) + 3 * tile;
  const int e = tl[0], row0 = tl[1];
  const int first = plan[1 + e], end = plan[2 + e];        // the expert's rows
  if ((row0 - first) % MW_BM) return;                      // not the first plan tile of a wide tile
  const int rows = min(MW_BM, end - row0);
  (void)per;
  const int n0 = blockIdx.x * MG_BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 1, wn = warp & 1;
  if (tid < MW_BM) {
    int r = -1;
    if (tid < rows) r = row_pair ? row_pair[row0 + tid] / pairs_per_token : row0 + tid;
    src_row[tid] = r;
  }
  __syncthreads();
  const bf16 *We = W + (size_t)e * (size_t)S * N * K;
  float acc[S][2][4][4];
#pragma unroll
  for (int s = 0; s < S; ++s)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int f = 0; f < 4; ++f) acc[s][i][j][f] = 0.f;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  auto load_stage = [&](int st, int k0) {
    for (int i = tid; i < MW_BM * (MW_BK / 8); i += 256) {
      const int r = i >> 2, p = i & 3;
      const int sr = src_row[r];
      bf16 *dst = &As[st][r][p * 8];
      if (sr >= 0 && k0 + p * 8 < K) cp_async_16(smem_u32(dst), A + (size_t)sr * a_stride + k0 + p * 8);
      else *(uint4 *)dst = zero;
    }
    for (int i = tid; i < S * MG_BN * (MW_BK / 8); i += 256) {
      const int s = i / (MG_BN * 4), c = (i >> 2) % MG_BN, p = i & 3;
      bf16 *dst = &Bs[st][s][c][p * 8];
      if (n0 + c < N && k0 + p * 8 < K) cp_async_16(smem_u32(dst), We + gu_row(s, n0 + c, N, SWIGLU ? blocked : 0) * K + k0 + p * 8);
      else *(uint4 *)dst = zero;
    }
    cp_async_commit();
  };
  const int KT = (K + MW_BK - 1) / MW_BK;
  load_stage(0, 0);
  for (int kt = 0; kt < KT; ++kt) {
    const int st = kt & 1;
    if (kt + 1 < KT) {
      load_stage(st ^ 1, (kt + 1) * MW_BK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MW_BK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        ldmatrix_x4(a[i], smem_u32(&As[st][wm * 32 + 16 * i + (lane & 15)][kk + (lane >> 4) * 8]));
#pragma unroll
      for (int s = 0; s < S; ++s)
#pragma unroll
        for (int j2 = 0; j2 < 2; ++j2) {
          uint32_t b[4];
          ldmatrix_x4(b, smem_u32(&Bs[st][s][wn * 32 + 16 * j2 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]));
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            mma_bf16_16816(acc[s][i][2 * j2], a[i], b[0], b[1]);
            mma_bf16_16816(acc[s][i][2 * j2 + 1], a[i], b[2], b[3]);
          }
        }
    }
    __syncthreads();
  }
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int r = wm * 32 + 16 * i + g + (f >> 1) * 8;
        const int c = n0 + wn * 32 + 8 * j + 2 * q + (f & 1);
        if (r >= rows || c >= N) continue;
        const float v = SWIGLU ? silu_f(acc[0][i][j][f]) * acc[S - 1][i][j][f] : acc[0][i][j][f];
        const size_t at = (size_t)(row0 + r) * N + c;
        if (out_f32) ((float *)out)[at] = v;
        else ((bf16 *)out)[at] = __float2bfloat16_rn(v);
      }
}

// ---------------------------------------------------------------------------
// the same for a step of few rows (decoding): a warp takes four output columns of one row and
// streams their weight rows with 16-byte loads, the row's K entries dealt to the lanes
// ---------------------------------------------------------------------------
__device__ __forceinline__ float dot_chunk(const uint4 &w, const uint4 &x, float acc, bf16) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w}, xx[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc = fmaf(__uint_as_float(ww[i] << 16), __uint_as_float(xx[i] << 16), acc);
    acc = fmaf(__uint_as_float(ww[i] & 0xffff0000u), __uint_as_float(xx[i] & 0xffff0000u), acc);
  }
  return acc;
}
__device__ __forceinline__ float dot_chunk(const uint4 &w, const uint4 &x, float acc, float) {
  acc = fmaf(__uint_as_float(w.x), __uint_as_float(x.x), acc);
  acc = fmaf(__uint_as_float(w.y), __uint_as_float(x.y), acc);
  acc = fmaf(__uint_as_float(w.z), __uint_as_float(x.z), acc);
  return fmaf(__uint_as_float(w.w), __uint_as_float(x.w), acc);
}

#define MV_COLS 4            // columns a warp computes at a time
template <typename T, bool SWIGLU>
__global__ void __launch_bounds__(128)
moe_gemv_kernel(const T *__restrict__ A, int a_stride, const int *__restrict__ row_pair, int pairs_per_token, int gather,
                const int *__restrict__ idx, const T *__restrict__ W, int N, int K, const int *__restrict__ plan,
                int n_real, void *__restrict__ out, int out_f32, int blocked) {
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.y;
  if (r >= plan[1 + n_real]) return;                     // rows in use
  const int pair = row_pair[r];
  const int e = idx[pair];
  constexpr int EPL = 16 / sizeof(T);                    // entries per 16-byte load
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * 4 + warp) * MV_COLS;
  if (n0 >= N) return;
  const T *a = A + (size_t)(gather ? pair / pairs_per_token : r) * a_stride;
  const T *We = W + (size_t)e * (SWIGLU ? 2 : 1) * N * K;
  const int chunks = K / EPL;
  float acc[SWIGLU ? 2 : 1][MV_COLS];
#pragma unroll
  for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
    for (int j = 0; j < MV_COLS; ++j) acc[s][j] = 0.f;
#pragma unroll 2
  for (int c = lane; c < chunks; c += 32) {
    const uint4 x = *(const uint4 *)(a + (size_t)c * EPL);
    uint4 w[SWIGLU ? 2 : 1][MV_COLS];
#pragma unroll
    for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
      for (int j = 0; j < MV_COLS; ++j) {
        const int n = min(n0 + j, N - 1);
        w[s][j] = *(const uint4 *)(We + gu_row(s, n, N, SWIGLU ? blocked : 0) * K + (size_t)c * EPL);
      }
#pragma unroll
    for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
      for (int j = 0; j < MV_COLS; ++j) acc[s][j] = dot_chunk(w[s][j], x, acc[s][j], T());
  }
#pragma unroll
  for (int j = 0; j < MV_COLS; ++j) {
    float v = warp_sum(acc[0][j]);
    if (SWIGLU) v = silu_f(v) * warp_sum(acc[SWIGLU ? 1 : 0][j]);
    if (lane == 0 && n0 + j < N) {
      const size_t at = (size_t)r * N + n0 + j;
      if (out_f32) ((float *)out)[at] = v;
      else ((T *)out)[at] = from_f32<T>(v);
    }
  }
}

extern "C" int g2b_moe_tile_rows() { return MG_BM; }

template <typename T>
static void launch_gemv(const void *A, int a_stride, const int *row_pair, int pairs_per_token, int gather, const int *idx,
                        const void *W, int N, int K, const int *plan, int n_real, int n_rows, int swiglu, void *out,
                        int out_f32, int blocked, cudaStream_t stream) {
  const dim3 grid((N + 4 * MV_COLS - 1) / (4 * MV_COLS), n_rows);
  if (swiglu)
    g2b_launch(moe_gemv_kernel<T, true>, grid, dim3(128), 0, stream, (const T *)A, a_stride, row_pair, pairs_per_token,
               gather, idx, (const T *)W, N, K, plan, n_real, out, out_f32, blocked);
  else
    g2b_launch(moe_gemv_kernel<T, false>, grid, dim3(128), 0, stream, (const T *)A, a_stride, row_pair, pairs_per_token,
               gather, idx, (const T *)W, N, K, plan, n_real, out, out_f32, blocked);
}

// Few rows: `row_pair` (row -> pair) and `idx` (pair -> expert) are both needed; `gather` says whether
// row r reads A[pair / pairs_per_token] or A[r].
extern "C" int g2b_moe_gemv(const void *A, int dtype, int a_stride, const int *row_pair, int pairs_per_token, int gather,
                            const int *idx, const void *W, int N, int K, const int *plan, int n_real, int n_rows,
                            int swiglu, void *out, int out_f32, int blocked, cudaStream_t stream) {
  if (n_rows <= 0 || N <= 0) return 0;
  const int epl = dtype == G2B_BF16 ? 8 : 4;
  if (K % epl || a_stride % epl || (((uintptr_t)A | (uintptr_t)W) & 15))
    G2B_REFUSE("moe_gemv: K = %d or the rows' distance %d is no multiple of %d, or a pointer is off 16 bytes", K, a_stride, epl);
  if (dtype == G2B_F32) launch_gemv<float>(A, a_stride, row_pair, pairs_per_token, gather, idx, W, N, K, plan, n_real, n_rows, swiglu, out, out_f32, blocked, stream);
  else if (dtype == G2B_BF16) launch_gemv<bf16>(A, a_stride, row_pair, pairs_per_token, gather, idx, W, N, K, plan, n_real, n_rows, swiglu, out, out_f32, blocked, stream);
  else G2B_REFUSE("moe_gemv: unknown dtype %d", dtype);
  return g2b_check_launch("moe_gemv");
}

extern "C" int g2b_moe_gemm(const void *A, int dtype, int a_stride, const int *row_pair, int pairs_per_token,
                            const void *W, int N, int K, const int *plan, int n_real, int max_tiles, int swiglu,
                            void *out, int out_f32, int blocked, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  const dim3 grid((N + MG_BN - 1) / MG_BN, max_tiles);
  if (dtype == G2B_F32) {
    if (swiglu)
      g2b_launch(moe_gemm_kernel<float, true>, grid, dim3(128), 0, stream, (const float *)A, a_stride, row_pair,
                 pairs_per_token, (const float *)W, N, K, plan, n_real, out, out_f32, blocked);
    else
      g2b_launch(moe_gemm_kernel<float, false>, grid, dim3(128), 0, stream, (const float *)A, a_stride, row_pair,
                 pairs_per_token, (const float *)W, N, K, plan, n_real, out, out_f32, blocked);
  } else if (dtype == G2B_BF16) {
    const bool mma = K % 8 == 0 && a_stride % 8 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0;
    // many rows an expert (a prompt step): the wide tiles
    const bool wide = mma && max_tiles > 3 * n_real + 8;
    if (wide && swiglu)
      g2b_launch(moe_gemm_wide_kernel<true>, grid, dim3(256), 0, stream, (const bf16 *)A, a_stride, row_pair,
                 pairs_per_token, (const bf16 *)W, N, K, plan, n_real, out, out_f32, blocked);
    else if (wide)
      g2b_launch(moe_gemm_wide_kernel<false>, grid, dim3(256), 0, stream, (const bf16 *)A, a_stride, row_pair,
                 pairs_per_token, (const bf16 *)W, N, K, plan, n_real, out, out_f32, blocked);
    else if (mma && swiglu)
      g2b_launch(moe_gemm_mma_kernel<true>, grid, dim3(128), 0, stream, (const bf16 *)A, a_stride, row_pair,
                 pairs_per_token, (const bf16 *)W, N, K, plan, n_real, out, out_f32, blocked);
    else if (mma)
      g2b_launch(moe_gemm_mma_kernel<false>, grid, dim3(128), 0, stream, (const bf16 *)A, a_stride, row_pair,
                 pairs_per_token, (const bf16 *)W, N, K, plan, n_real, out, out_f32, blocked);
    else if (swiglu)
      g2b_launch(moe_gemm_kernel<bf16, true>, grid, dim3(128), 0, stream, (const bf16 *)A, a_stride, row_pair,
                 pairs_per_token, (const bf16 *)W, N, K, plan, n_real, out, out_f32, blocked);
    else
      g2b_launch(moe_gemm_kernel<bf16, false>, grid, dim3(128), 0, stream, (const bf16 *)A, a_stride, row_pair,
                 pairs_per_token, (const bf16 *)W, N, K, plan, n_real, out, out_f32, blocked);
  } else {
    G2B_REFUSE("moe_gemm: unknown dtype %d", dtype);
  }
  return g2b_check_launch("moe_gemm");
}

// ---------------------------------------------------------------------------
// combination
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float *__restrict__ rows, const int *__restrict__ pair_row, const float *__restrict__ weight,
                   const float *__restrict__ x_self, int T, int top, int Hw, float *__restrict__ out, int accumulate) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  for (int j = threadIdx.x; j < Hw; j += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < top; ++r) {
      const int row = pair_row[(size_t)t * top + r];
      const float v = row >= 0 ? rows[(size_t)row * Hw + j] : x_self[(size_t)t * Hw + j];
      acc = fmaf(weight[(size_t)t * top + r], v, acc);
    }
    out[(size_t)t * Hw + j] = accumulate ? out[(size_t)t * Hw + j] + acc : acc;
  }
}

// The combination, then the sum's RMS norm (times a weight) added to the stream, and the new stream
// once more in the compute type: what a layer whose sublayer outputs are normed does behind its routed
// feed-forward, in one pass.  A thread keeps its share of the row (rows of up to 4,096 entries).
#define MCN_PER 16
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_norm_add_kernel(const float *__restrict__ rows, const int *__restrict__ pair_row,
                            const float *__restrict__ weight, float *__restrict__ x, const float *__restrict__ norm_w,
                            float eps, int top, int Hw, T *__restrict__ cast_out) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  float *xr = x + (size_t)t * Hw;
  float keep[MCN_PER], own[MCN_PER];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MCN_PER; ++i) {
    const int j = threadIdx.x + 256 * i;
    float acc = 0.f;
    own[i] = 0.f;
    if (j < Hw) {
      own[i] = xr[j];
      for (int r = 0; r < top; ++r) {
        const int row = pair_row[(size_t)t * top + r];
        acc = fmaf(weight[(size_t)t * top + r], row >= 0 ? rows[(size_t)row * Hw + j] : own[i], acc);
      }
    }
    keep[i] = acc;
    ss = fmaf(acc, acc, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)Hw + eps);
#pragma unroll
  for (int i = 0; i < MCN_PER; ++i) {
    const int j = threadIdx.x + 256 * i;
    if (j < Hw) {
      const float v = own[i] + (keep[i] * inv) * (norm_w ? norm_w[j] : 1.f);
      xr[j] = v;
      if (cast_out) cast_out[(size_t)t * Hw + j] = from_f32<T>(v);
    }
  }
}

extern "C" int g2b_moe_combine_norm_add(const float *rows, const int *pair_row, const float *weight, float *x,
                                        const float *norm_w, float eps, int T_tokens, int top, int Hw, void *cast_out,
                                        int dtype, cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (Hw > 256 * MCN_PER) G2B_REFUSE("moe_combine_norm_add: rows of %d entries (at most %d)", Hw, 256 * MCN_PER);
  if (dtype == G2B_F32)
    g2b_launch(moe_combine_norm_add_kernel<float>, dim3(T_tokens), dim3(256), 0, stream, rows, pair_row, weight, x, norm_w,
               eps, top, Hw, (float *)cast_out);
  else if (dtype == G2B_BF16)
    g2b_launch(moe_combine_norm_add_kernel<bf16>, dim3(T_tokens), dim3(256), 0, stream, rows, pair_row, weight, x, norm_w,
               eps, top, Hw, (bf16 *)cast_out);
  else
    G2B_REFUSE("moe_combine_norm_add: unknown dtype %d", dtype);
  return g2b_check_launch("moe_combine_norm_add");
}

extern "C" int g2b_moe_combine(const float *rows, const int *pair_row, const float *weight, const float *x_self, int T,
                               int top, int Hw, float *out, int accumulate, cudaStream_t stream) {
  if (T <= 0) return 0;
  g2b_launch(moe_combine_kernel, dim3(T), dim3(256), 0, stream, rows, pair_row, weight, x_self, T, top, Hw, out, accumulate);
  return g2b_check_launch("moe_combine");
}
