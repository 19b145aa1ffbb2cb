// A feed-forward of experts with a router: every token goes to `top` of `E` small feed-forwards.
//
// Everything that depends on the router's choice stays on the device, so the launches of a step depend
// on its number of rows alone (a decode step through it can be captured in a graph):
//   1. route:   one block per token takes the E router logits (float32 products of the token's vector with
//               the router's rows, summed in a fixed order), picks the `top` largest (the lower index wins a
//               tie) and gives them the softmax over the chosen logits as weights.  A second mode scores every
//               expert by itself: s = sigmoid(logit); the choice is made on s + correction (a float per expert),
//               optionally among the experts of the best `keep` of `groups` equal groups of neighbours (a
//               group's score: the sum of its two largest choice scores), and the weights are the chosen
//               experts' s over their sum (+ norm_eps), times a factor.  The router's matrix may carry further
//               rows behind the experts' (`extra`): their logits' sigmoids are handed out per token (a gate
//               of a sublayer that every token uses).
//   2. sort:    one CTA counts the (token, choice) pairs per expert, lays the experts' rows out one after
//               the other (`perm`: sorted place -> pair, `inv`: pair -> sorted place) and cuts every
//               expert's rows into tiles of RT_BM rows (`tiles`: expert and first row, -1 for unused).
//   3. experts: a grouped product over those tiles: tile rows are gathered through `perm`, the weights are
//               the tile's expert's; first gate and up with silu(gate) * up in the epilogue, then down.
//               A row's result does not depend on its place in a tile: every output element is one chain of
//               k = 0..K-1 (the FMA kernel) or a fixed tree (the tensor-core kernel).
//   4. combine: y[t] = sum over the token's choices, in the order of the choices, of weight * expert output.
#include <math_constants.h>

#include "common.cuh"

#define RT_BM 64
#define RT_BN 64
#define RT_BK 16

// ------------------------------------------------------------------------------------ 1. route
#define RK_WARPS 8
struct RouteOpts {
  int mode;                  // 0: softmax over the chosen logits; 1: sigmoid scores
  const float* correction;   // mode 1: added to the scores for the choice alone (null: nothing)
  int groups, keep;          // mode 1: the choice is made inside the best `keep` of `groups` groups (groups 0: everywhere)
  float scale, norm_eps;     // mode 1: weights = s / (sum s + norm_eps) * scale
  int extra;                 // rows of w behind the E experts' rows
  float* extra_out;          // [n, extra]: the sigmoids of those rows' logits
};

template <typename T>
__global__ void __launch_bounds__(RK_WARPS * 32)
route_topk_kernel(const T* __restrict__ x, const float* __restrict__ w, int* __restrict__ ids, float* __restrict__ weights, int n,
                  int d, int n_experts, int top, RouteOpts opt) {
  extern __shared__ float sm[];               // [RK_WARPS][E] partial logits, then [E] logits, [n_experts] scores, [groups] x 2
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int t = blockIdx.x;                   // a block per token: its warps share the token's vector
  int E = n_experts + opt.extra;              // rows of the router's matrix
  float* part = sm;
  float* z = sm + (size_t)RK_WARPS * E;
  float* score = z + E;
  float* gscore = score + n_experts;
  float* gkept = gscore + opt.groups;
  const T* xr = x + (size_t)t * d;
  for (int e0 = 0; e0 < E; e0 += 8) {          // eight experts per pass over the token's vector
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if ((d & 3) == 0 && (((uintptr_t)w | (uintptr_t)xr) & 15) == 0) {
      // four consecutive elements a thread: 16-byte reads of the router's rows, all eight experts' in flight together
      for (int i = threadIdx.x * 4; i < d; i += RK_WARPS * 32 * 4) {
        const float x0 = to_f32<T>(xr[i]), x1 = to_f32<T>(xr[i + 1]), x2 = to_f32<T>(xr[i + 2]), x3 = to_f32<T>(xr[i + 3]);
        float4 wv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          wv[j] = e0 + j < E ? *reinterpret_cast<const float4*>(w + (size_t)(e0 + j) * d + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(x3, wv[j].w, fmaf(x2, wv[j].z, fmaf(x1, wv[j].y, fmaf(x0, wv[j].x, acc[j]))));
      }
    } else {
      for (int i = threadIdx.x; i < d; i += RK_WARPS * 32) {
        const float xv = to_f32<T>(xr[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (e0 + j < E) acc[j] = fmaf(xv, w[(size_t)(e0 + j) * d + i], acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sum = warp_sum(acc[j]);
      if (lane == 0 && e0 + j < E) part[(size_t)wid * E + e0 + j] = sum;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += RK_WARPS * 32) {       // the warps' shares in warp order
    float sum = 0.f;
#pragma unroll
    for (int wv = 0; wv < RK_WARPS; ++wv) sum += part[(size_t)wv * E + e];
    z[e] = sum;
  }
  __syncthreads();
  if (wid != 0) return;
  E = n_experts;
  if (opt.mode == 1) {
    for (int e = lane; e < E; e += 32) {
      const float sc = 1.0f / (1.0f + expf(-z[e]));
      score[e] = sc;
      z[e] = opt.correction != nullptr ? sc + opt.correction[e] : sc;
    }
    for (int e = lane; e < opt.extra; e += 32) opt.extra_out[(size_t)t * opt.extra + e] = 1.0f / (1.0f + expf(-z[E + e]));
    __syncwarp();
    if (opt.groups > 0 && opt.keep < opt.groups) {
      const int size = E / opt.groups;
      for (int g = lane; g < opt.groups; g += 32) {          // a group's score: its two largest choice scores
        float a = -CUDART_INF_F, b = -CUDART_INF_F;
        for (int e = g * size; e < (g + 1) * size; ++e) {
          const float v = z[e];
          if (v > a) {
            b = a;
            a = v;
          } else if (v > b) {
            b = v;
          }
        }
        gscore[g] = size > 1 ? a + b : a;
        gkept[g] = 0.f;
      }
      __syncwarp();
      for (int k = 0; k < opt.keep; ++k) {                   // the best groups, the lower index winning a tie
        float best = -CUDART_INF_F;
        int bi = 0x7fffffff;
        for (int g = lane; g < opt.groups; g += 32) {
          const float v = gscore[g];
          if (gkept[g] == 0.f && (v > best || bi == 0x7fffffff)) {
            best = v;
            bi = g;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best, o);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) {
            best = ov;
            bi = oi;
          }
        }
        if (lane == 0 && bi < opt.groups) gkept[bi] = 1.f;
        __syncwarp();
      }
      for (int e = lane; e < E; e += 32)
        if (gkept[e / size] == 0.f) z[e] = -CUDART_INF_F;
      __syncwarp();
    }
  }
  float first = 0.f, mine = 0.f, total = 0.f;
  int mine_id = 0;
  for (int k = 0; k < top; ++k) {
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best) {                          // ascending e: the first maximum of this lane
        best = v;
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (k == 0) first = best;
    // mode 0: the first chosen logit is the largest; mode 1: the expert's own score, without the correction
    const float p = opt.mode == 1 ? (bi < E ? score[bi] : 0.f) : expf(best - first);
    total += p;
    if (lane == (k & 31)) {                    // lane k keeps choice k (top <= 32)
      mine = p;
      mine_id = bi;
    }
    if (lane == 0 && bi < E) z[bi] = -CUDART_INF_F;
    __syncwarp();
  }
  if (lane < top) {
    ids[(size_t)t * top + lane] = mine_id < E ? mine_id : 0;
    weights[(size_t)t * top + lane] = opt.mode == 1 ? mine / (total + opt.norm_eps) * opt.scale : mine / total;
  }
}

HK_API int hk_route_topk(const void* x, int dtype, const float* w, int* ids, float* weights, int n, int d, int E, int top, int mode,
                         const float* correction, int groups, int keep, float scale, float norm_eps, int extra, float* extra_out,
                         void* stream) {
  if (n <= 0) return 0;
  if (E < 1 || top < 1 || top > E || top > 32 || E > 2048 || mode < 0 || mode > 1 || extra < 0 || extra > 64) return HK_ERR_UNSUPPORTED;
  if (mode == 0 && (correction != nullptr || groups != 0 || extra != 0)) return HK_ERR_UNSUPPORTED;
  if (groups < 0 || (groups > 0 && (E % groups || keep < 1 || keep > groups)) || (extra > 0 && extra_out == nullptr)) return HK_ERR_UNSUPPORTED;
  const RouteOpts opt = {mode, correction, groups, keep, scale, norm_eps, extra, extra_out};
  const size_t smem = ((size_t)(RK_WARPS + 1) * (E + extra) + E + 2 * groups) * sizeof(float);
  dim3 grid((unsigned)n);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == HK_F32) {
    static HkSmemCache cache;
    if (int e = hk_allow_smem(route_topk_kernel<float>, smem, cache)) return e;
    return hk_launch(route_topk_kernel<float>, grid, dim3(RK_WARPS * 32), smem, s, (const float*)x, w, ids, weights, n, d, E, top, opt);
  }
  if (dtype == HK_BF16) {
    static HkSmemCache cache;
    if (int e = hk_allow_smem(route_topk_kernel<bf16>, smem, cache)) return e;
    return hk_launch(route_topk_kernel<bf16>, grid, dim3(RK_WARPS * 32), smem, s, (const bf16*)x, w, ids, weights, n, d, E, top, opt);
  }
  return HK_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------ 2. sort
// offsets[E + 1], perm[pairs], inv[pairs], tiles[max_tiles][2].
__global__ void __launch_bounds__(1024)
route_sort_kernel(const int* __restrict__ ids, int pairs, int E, int bm, int* __restrict__ offsets, int* __restrict__ perm,
                  int* __restrict__ inv, int* __restrict__ tiles, int max_tiles) {
  extern __shared__ int smi[];                // counts[E], cursor[E]
  int* counts = smi;
  int* cursor = smi + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&counts[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tile = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      cursor[e] = at;
      for (int r = 0; r < counts[e] && tile < max_tiles; r += bm) {
        tiles[2 * tile] = e;
        tiles[2 * tile + 1] = at + r;
        ++tile;
      }
      at += counts[e];
    }
    offsets[E] = at;
    for (; tile < max_tiles; ++tile) {
      tiles[2 * tile] = -1;
      tiles[2 * tile + 1] = 0;
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int at = atomicAdd(&cursor[ids[p]], 1);
    perm[at] = p;
    inv[p] = at;
  }
}

HK_API int hk_route_sort(const int* ids, int pairs, int E, int* offsets, int* perm, int* inv, int* tiles, int max_tiles,
                         void* stream) {
  if (pairs <= 0) return 0;
  if (E > 4096) return HK_ERR_UNSUPPORTED;
  return hk_launch(route_sort_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), (cudaStream_t)stream, ids, pairs, E,
                   RT_BM, offsets, perm, inv, tiles, max_tiles);
}

HK_API int hk_route_tile_rows() { return RT_BM; }

// The padded layout for the tcgen05 grouped product: every expert's rows start on a multiple of `pad` (the product's
// 128-row tile), so a tile's rows all belong to one expert.  perm[M_max] (sorted place -> pair, -1 for padding),
// inv[pairs] (pair -> sorted place), groups[M_max / pad] (tile -> expert, -1 for tiles past the last expert).
__global__ void __launch_bounds__(1024)
route_sort_padded_kernel(const int* __restrict__ ids, int pairs, int E, int pad, int* __restrict__ perm, int* __restrict__ inv,
                         int* __restrict__ groups, int m_max) {
  extern __shared__ int smi[];                // counts[E], cursor[E]
  int* counts = smi;
  int* cursor = smi + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  for (int p = threadIdx.x; p < m_max; p += blockDim.x) perm[p] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&counts[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      cursor[e] = at;
      const int span = (counts[e] + pad - 1) / pad * pad;
      for (int r = 0; r < span && at + r < m_max; r += pad) groups[(at + r) / pad] = e;
      at += span;
    }
    for (int t = at / pad; t < m_max / pad; ++t) groups[t] = -1;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int at = atomicAdd(&cursor[ids[p]], 1);
    perm[at] = p;
    inv[p] = at;
  }
}

HK_API int hk_route_sort_padded(const int* ids, int pairs, int E, int pad, int* perm, int* inv, int* groups, int m_max, void* stream) {
  if (pairs <= 0) return 0;
  if (E > 4096 || pad < 1 || m_max % pad || m_max < pairs + E * (pad - 1)) return HK_ERR_UNSUPPORTED;
  return hk_launch(route_sort_padded_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), (cudaStream_t)stream, ids, pairs, E, pad,
                   perm, inv, groups, m_max);
}

// xs[p, :] = x[perm[p] / top, :], or zeros where perm[p] < 0: the tokens' vectors in the padded sorted order (bf16, d % 8 == 0).
__global__ void route_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ perm, int top, bf16* __restrict__ xs, int d) {
  const int p = blockIdx.x;
  const int src = perm[p];
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)p * d);
  const uint4* from = reinterpret_cast<const uint4*>(x + (size_t)(src < 0 ? 0 : src / top) * d);
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src < 0 ? make_uint4(0, 0, 0, 0) : from[i];
}

HK_API int hk_route_gather(const void* x, const int* perm, int top, void* xs, int m_max, int d, void* stream) {
  if (m_max <= 0) return 0;
  if ((d & 7) || (((uintptr_t)x | (uintptr_t)xs) & 15)) return HK_ERR_UNSUPPORTED;
  return hk_launch(route_gather_kernel, dim3((unsigned)m_max), dim3(d >= 2048 ? 256 : 128), 0, (cudaStream_t)stream, (const bf16*)x, perm,
                   top, (bf16*)xs, d);
}



// ------------------------------------------------------------------------------------ 3. experts
// out rows are sorted places.  GATED: w is [E][2N][K] = N gate rows then N up rows per expert, out[p, n] (type TO) =
// silu(gate) * up.  Otherwise w is [E][N][K] and out[p, n] (float) = a[p] . w[e][n].  `gather`: row p of `a` is row
// perm[p] / top of the tensor (the token's vector); else row p.
template <typename T, typename TO, bool GATED>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const T* __restrict__ a, const T* __restrict__ w, TO* __restrict__ out, const int* __restrict__ tiles,
                    const int* __restrict__ offsets, const int* __restrict__ perm, int top, int gather, int N, int K) {
  __shared__ float As[RT_BK][RT_BM + 4];
  __shared__ float Ws[GATED ? 2 : 1][RT_BK][RT_BN + 4];
  __shared__ int rows[RT_BM];
  const int e = tiles[2 * blockIdx.y];
  if (e < 0) return;
  const int p0 = tiles[2 * blockIdx.y + 1];
  const int p_end = min(p0 + RT_BM, offsets[e + 1]);
  const int tid = threadIdx.x;
  if (tid < RT_BM) {
    const int p = p0 + tid;
    rows[tid] = p < p_end ? (gather ? perm[p] / top : p) : -1;
  }
  __syncthreads();
  const int n0 = blockIdx.x * RT_BN;
  const int tx = tid & 15, ty = tid >> 4;
  const T* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
  float acc[GATED ? 2 : 1][4][4];
#pragma unroll
  for (int s = 0; s < (GATED ? 2 : 1); ++s)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[s][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += RT_BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + j * 256;
      const int r = i >> 4, c = i & 15;
      const int gk = k0 + c, gn = n0 + r;
      const int src = rows[r];
      As[c][r] = (src >= 0 && gk < K) ? to_f32<T>(a[(size_t)src * K + gk]) : 0.f;
      Ws[0][c][r] = (gn < N && gk < K) ? to_f32<T>(we[(size_t)gn * K + gk]) : 0.f;
      if (GATED) Ws[GATED ? 1 : 0][c][r] = (gn < N && gk < K) ? to_f32<T>(we[(size_t)(N + gn) * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < RT_BK; ++kk) {
      float av[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int s = 0; s < (GATED ? 2 : 1); ++s) {
        float wv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[j] = Ws[s][kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[s][i][j] = fmaf(av[i], wv[j], acc[s][i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int p = p0 + ty * 4 + i;
    if (p >= p_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float val = acc[0][i][j];
      if (GATED) {
        const float u = acc[GATED ? 1 : 0][i][j];
        val = val / (1.0f + expf(-val)) * u;
      }
      out[(size_t)p * N + gn] = from_f32<TO>(val);
    }
  }
}

// The same on the tensor cores (bf16 operands, fp32 accumulation; K a multiple of 8): a CTA takes a tile of RT_BM
// sorted rows and 128 weight rows: plain, 128 output columns; gated, 64 gate rows and the 64 up rows that match
// them, so that silu(gate) * up is taken in the epilogue.  Operands come through a three-stage cp.async ring in
// slices of 32 k (A rows gathered through `rows`), fragments by ldmatrix, products by mma.sync m16n8k16: eight
// warps as 2 (rows) x 4 (columns), a warp 32 rows x 32 weight rows.  An output element's sum runs over k in an
// order that does not depend on the row's place in its tile, so a token's result does not depend on the batch.
#define GM_BN 128
#define GM_BK 32
#define GM_LD (GM_BK + 8)

__device__ __forceinline__ uint32_t gm_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gm_cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(gm_smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gm_ldmatrix_x4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(gm_smem_u32(p)));
}
__device__ __forceinline__ void gm_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// GM_STAGES: slices in the ring (dynamic shared memory): all but one on their way while one is multiplied.
template <bool GATED, int GM_STAGES>
__global__ void __launch_bounds__(256)
grouped_gemm_mma_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, void* __restrict__ out_, const int* __restrict__ tiles,
                        const int* __restrict__ offsets, const int* __restrict__ perm, int top, int gather, int N, int K) {
  extern __shared__ __align__(16) uint8_t gm_smem[];
  typedef bf16 (*ATile)[RT_BM][GM_LD];
  typedef bf16 (*WTile)[GM_BN][GM_LD];
  ATile As = reinterpret_cast<ATile>(gm_smem);                                               // [GM_STAGES][RT_BM][GM_LD]
  WTile Ws = reinterpret_cast<WTile>(gm_smem + sizeof(bf16) * GM_STAGES * RT_BM * GM_LD);    // [GM_STAGES][GM_BN][GM_LD]
  __shared__ int rows[RT_BM];
  const int e = tiles[2 * blockIdx.y];
  if (e < 0) return;
  const int p0 = tiles[2 * blockIdx.y + 1];
  const int p_end = min(p0 + RT_BM, offsets[e + 1]);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < RT_BM) {
    const int p = p0 + tid;
    rows[tid] = p < p_end ? (gather ? perm[p] / top : p) : -1;
  }
  __syncthreads();
  constexpr int COLS = GATED ? 64 : 128;            // output columns of a tile
  const int n0 = blockIdx.x * COLS;
  const bf16* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
  // what this thread copies per stage: one 16-byte piece of A, two of W
  const int a_row = tid >> 2, a_k = (tid & 3) * 8;
  const int a_src = rows[a_row];
  const bf16* a_ptr = a + (size_t)max(a_src, 0) * K + a_k;
  const bf16* w_ptr[2];
  bool w_ok[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int r = (tid + j * 256) >> 2;              // row of the W tile
    const int col = GATED ? (r & 63) : r;
    const int gn = n0 + col;
    w_ok[j] = gn < N;
    const size_t wrow = GATED ? (size_t)(r >> 6) * N + min(gn, N - 1) : (size_t)min(gn, N - 1);
    w_ptr[j] = we + wrow * K + a_k;
  }
  auto load = [&](int stage, int k0) {
    const bool kin = k0 + a_k < K;
    gm_cp_async16(&As[stage][a_row][a_k], a_ptr + k0, kin && a_src >= 0);
#pragma unroll
    for (int j = 0; j < 2; ++j) gm_cp_async16(&Ws[stage][(tid + j * 256) >> 2][a_k], w_ptr[j] + k0, kin && w_ok[j]);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int wr = warp >> 2, wc = warp & 3;           // warp row (32 rows each), warp column
  // the W-tile row of this warp's n8 tile nt: gated, tiles 0 and 1 are gate rows and 2 and 3 the up rows that match them
  auto wn = [&](int nt) { return GATED ? ((nt >> 1) * 64 + wc * 16 + (nt & 1) * 8) : (wc * 32 + nt * 8); };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
  const int ksteps = (K + GM_BK - 1) / GM_BK;
#pragma unroll
  for (int pre = 0; pre < GM_STAGES - 1; ++pre) {      // one group per slice, also past the end: the counting below relies on it
    if (pre < ksteps) load(pre, pre * GM_BK); else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int ks = 0; ks < ksteps; ++ks) {
    asm volatile("cp.async.wait_group %0;" ::"n"(GM_STAGES - 2) : "memory");
    __syncthreads();                                  // stage ks has landed; stage ks - 1 is free for everyone
    if (ks + GM_STAGES - 1 < ksteps) load((ks + GM_STAGES - 1) % GM_STAGES, (ks + GM_STAGES - 1) * GM_BK);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const int st = ks % GM_STAGES;
#pragma unroll
    for (int kk = 0; kk < GM_BK; kk += 16) {
      uint32_t af[2][4], bfr[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        gm_ldmatrix_x4(af[mt], &As[st][wr * 32 + mt * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int np = 0; np < 2; ++np)                 // two n8 tiles per ldmatrix: (tile, k half) = (lane / 16, (lane / 8) & 1)
        gm_ldmatrix_x4(bfr[np], &Ws[st][wn(np * 2 + (lane >> 4)) + (lane & 7)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) gm_mma(acc[mt][nt], af[mt], bfr[nt >> 1][(nt & 1) * 2], bfr[nt >> 1][(nt & 1) * 2 + 1]);
    }
  }
  const int g = lane >> 2, t2 = (lane & 3) * 2;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int p = p0 + wr * 32 + mt * 16 + g + half * 8;
      if (p >= p_end) continue;
      if (GATED) {
        bf16* out = reinterpret_cast<bf16*>(out_);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int gn = n0 + wc * 16 + nt * 8 + t2 + c;
            if (gn >= N) continue;
            const float gate = acc[mt][nt][half * 2 + c], up = acc[mt][nt + 2][half * 2 + c];
            out[(size_t)p * N + gn] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
          }
      } else {
        float* out = reinterpret_cast<float*>(out_);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int gn = n0 + wc * 32 + nt * 8 + t2 + c;
            if (gn < N) out[(size_t)p * N + gn] = acc[mt][nt][half * 2 + c];
          }
      }
    }
}

template <bool GATED, int STAGES>
static int gm_launch(const void* a, const void* w, void* out, const int* tiles, int max_tiles, const int* offsets, const int* perm,
                     int top, int gather, int N, int K, cudaStream_t s) {
  const size_t smem = sizeof(bf16) * STAGES * (RT_BM + GM_BN) * GM_LD;
  static HkSmemCache cache;
  if (int e = hk_allow_smem(grouped_gemm_mma_kernel<GATED, STAGES>, smem, cache)) return e;
  dim3 grid((unsigned)((N + (GATED ? 63 : GM_BN - 1)) / (GATED ? 64 : GM_BN)), (unsigned)max_tiles);
  return hk_launch(grouped_gemm_mma_kernel<GATED, STAGES>, grid, dim3(256), smem, s, (const bf16*)a, (const bf16*)w, out, tiles, offsets,
                   perm, top, gather, N, K);
}

HK_API int hk_grouped_gemm(const void* a, const void* w, int dtype, void* out, const int* tiles, int max_tiles, const int* offsets,
                           const int* perm, int top, int gather, int N, int K, int gated, void* stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  if (max_tiles > 65535) return HK_ERR_UNSUPPORTED;
  dim3 grid((unsigned)((N + RT_BN - 1) / RT_BN), (unsigned)max_tiles);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == HK_F32) {
    if (gated)
      return hk_launch(grouped_gemm_kernel<float, float, true>, grid, dim3(256), 0, s, (const float*)a, (const float*)w, (float*)out,
                       tiles, offsets, perm, top, gather, N, K);
    return hk_launch(grouped_gemm_kernel<float, float, false>, grid, dim3(256), 0, s, (const float*)a, (const float*)w, (float*)out,
                     tiles, offsets, perm, top, gather, N, K);
  }
  if (dtype == HK_BF16 && (K & 7) == 0 && ((((uintptr_t)a | (uintptr_t)w) & 15) == 0)) {
    // few rows (decode steps): the products are bound by the experts' weight bytes, and a ring of six slices keeps more of
    // them on their way (width 4,096, 128 pairs: 88 and 45 us against 97 and 57 with three); many rows: three slices leave
    // room for four CTAs an SM (4,096 pairs: 546 and 297 us against 653 and 307 with six)
    const bool deep = max_tiles <= 40;       // tiles = pairs / 64 + experts: a few hundred pairs at most
    if (gated) return deep ? gm_launch<true, 6>(a, w, out, tiles, max_tiles, offsets, perm, top, gather, N, K, s)
                           : gm_launch<true, 3>(a, w, out, tiles, max_tiles, offsets, perm, top, gather, N, K, s);
    return deep ? gm_launch<false, 6>(a, w, out, tiles, max_tiles, offsets, perm, top, gather, N, K, s)
                : gm_launch<false, 3>(a, w, out, tiles, max_tiles, offsets, perm, top, gather, N, K, s);
  }
  if (dtype == HK_BF16) {
    if (gated)
      return hk_launch(grouped_gemm_kernel<bf16, bf16, true>, grid, dim3(256), 0, s, (const bf16*)a, (const bf16*)w, (bf16*)out, tiles,
                       offsets, perm, top, gather, N, K);
    return hk_launch(grouped_gemm_kernel<bf16, float, false>, grid, dim3(256), 0, s, (const bf16*)a, (const bf16*)w, (float*)out, tiles,
                     offsets, perm, top, gather, N, K);
  }
  return HK_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------ 4. combine
// y[t, :] (= or +=) sum_k weights[t, k] * ys[inv[t * top + k], :] (+ shared_gate[t] * shared[t, :], the result of a
// sublayer that every token uses, when `shared` is given; a null gate counts as 1)
__global__ void route_combine_kernel(const float* __restrict__ ys, const int* __restrict__ inv, const float* __restrict__ weights,
                                     float* __restrict__ y, int d, int top, int accumulate, const float* __restrict__ shared,
                                     const float* __restrict__ shared_gate) {
  const int t = blockIdx.x;
  const float sg = shared != nullptr ? (shared_gate != nullptr ? shared_gate[t] : 1.0f) : 0.f;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(weights[(size_t)t * top + k], ys[(size_t)inv[(size_t)t * top + k] * d + i], acc);
    if (shared != nullptr) acc = fmaf(sg, shared[(size_t)t * d + i], acc);
    float* o = y + (size_t)t * d + i;
    *o = accumulate ? *o + acc : acc;
  }
}

HK_API int hk_route_combine(const float* ys, const int* inv, const float* weights, float* y, int n, int d, int top, int accumulate,
                            const float* shared, const float* shared_gate, void* stream) {
  if (n <= 0) return 0;
  // a block per token; where the tokens alone do not fill the SMs (decode steps) a token's columns are spread over blocks
  const int threads = d >= 1024 ? 256 : 128;
  int split = 1;
  while (split < 16 && (long long)n * split < 2 * 148 && split * threads < d) split <<= 1;
  return hk_launch(route_combine_kernel, dim3((unsigned)n, (unsigned)split), dim3(threads), 0, (cudaStream_t)stream, ys, inv, weights,
                   y, d, top, accumulate, shared, shared_gate);
}
