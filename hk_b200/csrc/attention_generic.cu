// Generic attention over the paged cache, for every head size, group size and window, in
// float (the true 32-bit path) or bf16 storage with fp32 arithmetic.
//
// One block per (token, query head).  The token at position p of request slot s reads keys
// j in [max(0, p - window + 1), p] (window <= 0: all of [0, p]) through the slot's block table;
// its own key was written by the cache-write kernel earlier in the same step.  Four warps take
// the keys round-robin, each keeping an online softmax state (max, sum, weighted values); the
// four states are merged in a fixed order.  Nothing depends on which other tokens are in the
// batch, so the result at a position is the same under every way of cutting the work.
// Values may have another width than keys (`vd`: pages [page][G][page_tokens][vd], out [n, H * vd]).  With
// `sink` = 1 the softmax has one more term in its denominator, a key whose score is 0 and that has no value:
// p_j = exp(s_j) / (1 + sum exp(s_j)); with `sinks` (one float per query head) that key's score is sinks[h] instead of 0.
// Further options, each off at 0 or null:
//   softcap c   a score becomes c * tanh(score / c) before the softmax;
//   chunk s     a token also sees no key before the start of its own block of s positions, (p / s) * s, counted from
//               position 0 of the request;
//   v_stride    elements between the values of consecutive tokens of a page; when it is not vd the values lie inside
//               wider rows: a cache that keeps ONE tensor per token whose first vd dims are the value (v_pages = k_pages,
//               v_stride = hd);
//   gate        fp32 logits [n, gate_ld >= H * vd]: the output is multiplied by gate_scale * sigmoid(gate[t, h * vd + d]).
//
// Reference counterpart: `attention`, src/cuda_device.zig:1494-1594 (block per (token, head),
// warp per position, online softmax); scale on q first: src/engine/attention_kernel.zig:109.
#include <math_constants.h>

#include "common.cuh"

#define AG_WARPS 4

struct AgOptions {
  float softcap;
  int chunk;
  int v_stride;
  const float* sinks;
  const float* gate;
  long long gate_ld;
  float gate_scale;
};

// AG_MAX_PER_LANE: dims per lane, 8 for widths up to 256, 20 up to 640
template <typename T, int AG_MAX_PER_LANE>
__global__ void __launch_bounds__(AG_WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                         const T* __restrict__ v_pages, const int* __restrict__ block_table,
                         int table_stride, const int* __restrict__ positions,
                         const int* __restrict__ slot_of_token, T* __restrict__ out, int H, int G, int hd,
                         int page_tokens, int window, float scale, int vd, int sink, AgOptions opt) {
  extern __shared__ float smem[];  // [AG_WARPS][vd] values, then [AG_WARPS] max, [AG_WARPS] sum
  float* acc_s = smem;
  float* m_s = smem + AG_WARPS * vd;
  float* l_s = m_s + AG_WARPS;

  int t = blockIdx.x / H, h = blockIdx.x % H;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int g = h / (H / G);
  int pos = positions[t];
  const int* bt = block_table + (size_t)slot_of_token[t] * table_stride;
  int lo = window > 0 ? max(0, pos - window + 1) : 0;
  if (opt.chunk > 0) lo = max(lo, (pos / opt.chunk) * opt.chunk);
  const float cap = opt.softcap, inv_cap = opt.softcap > 0.f ? 1.0f / opt.softcap : 0.f;

  float qr[AG_MAX_PER_LANE], acc[AG_MAX_PER_LANE];
  const T* qp = q + ((size_t)t * H + h) * hd;
#pragma unroll
  for (int i = 0; i < AG_MAX_PER_LANE; ++i) {
    int d = lane + 32 * i;
    qr[i] = d < hd ? to_f32<T>(qp[d]) * scale : 0.f;
    acc[i] = 0.f;
  }
  float m = -CUDART_INF_F, l = 0.f;
  for (int j = lo + wid; j <= pos; j += AG_WARPS) {
    int page = bt[j / page_tokens];
    if (page < 0) continue;  // never scheduled by the host; keeps the reads in bounds
    const size_t at = ((size_t)page * G + g) * page_tokens + (j % page_tokens);
    const T* kp = k_pages + at * hd;
    const T* vp = v_pages + at * opt.v_stride;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < AG_MAX_PER_LANE; ++i) {
      int d = lane + 32 * i;
      if (d < hd) s = fmaf(qr[i], to_f32<T>(kp[d]), s);
    }
    s = warp_sum(s);
    if (cap > 0.f) s = cap * tanhf(s * inv_cap);
    float mn = fmaxf(m, s);
    float corr = expf(m - mn);
    float p = expf(s - mn);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < AG_MAX_PER_LANE; ++i) {
      int d = lane + 32 * i;
      if (d < vd) acc[i] = acc[i] * corr + p * to_f32<T>(vp[d]);
    }
    m = mn;
  }
#pragma unroll
  for (int i = 0; i < AG_MAX_PER_LANE; ++i) {
    int d = lane + 32 * i;
    if (d < vd) acc_s[wid * vd + d] = acc[i];
  }
  if (lane == 0) {
    m_s[wid] = m;
    l_s[wid] = l;
  }
  __syncthreads();
  const float sink_score = sink && opt.sinks ? opt.sinks[h] : 0.f;
  float mm = sink ? sink_score : m_s[0];   // the sink's score takes part in the maximum
#pragma unroll
  for (int w = sink ? 0 : 1; w < AG_WARPS; ++w) mm = fmaxf(mm, m_s[w]);
  float f[AG_WARPS], lt = 0.f;
#pragma unroll
  for (int w = 0; w < AG_WARPS; ++w) {
    f[w] = m_s[w] == -CUDART_INF_F ? 0.f : expf(m_s[w] - mm);
    lt += l_s[w] * f[w];
  }
  if (sink) lt += expf(sink_score - mm);
  T* op = out + ((size_t)t * H + h) * vd;
  for (int d = threadIdx.x; d < vd; d += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < AG_WARPS; ++w) a += acc_s[w * vd + d] * f[w];
    a /= lt;
    if (opt.gate) a = a * opt.gate_scale / (1.0f + expf(-opt.gate[(size_t)t * opt.gate_ld + (size_t)h * vd + d]));
    op[d] = from_f32<T>(a);
  }
}

template <typename T, int PER>
static int ag_launch(const void* q, const void* k_pages, const void* v_pages, const int* block_table, int table_stride,
                     const int* positions, const int* slot_of_token, void* out, int n, int H, int G, int hd, int page_tokens,
                     int window, float scale, int vd, int sink, AgOptions opt, cudaStream_t s) {
  size_t smem = (size_t)(AG_WARPS * vd + 2 * AG_WARPS) * sizeof(float);
  unsigned blocks = (unsigned)((long long)n * H);
  attention_generic_kernel<T, PER><<<blocks, AG_WARPS * 32, smem, s>>>(
      (const T*)q, (const T*)k_pages, (const T*)v_pages, block_table, table_stride, positions, slot_of_token, (T*)out, H, G, hd,
      page_tokens, window, scale, vd, sink, opt);
  return hk_launch_status();
}

HK_API int hk_attention_generic(const void* q, const void* k_pages, const void* v_pages, int dtype,
                                const int* block_table, int table_stride, const int* positions,
                                const int* slot_of_token, void* out, int n, int H, int G, int hd,
                                int page_tokens, int window, float scale, int vd, int sink, const float* sinks, float softcap,
                                int chunk, int v_stride, const float* gate, long long gate_ld, float gate_scale, void* stream) {
  if (n <= 0) return 0;
  const int widest = hd > vd ? hd : vd;
  if (widest > 640 || hd < 1 || G < 1 || H % G != 0 || vd < 1 || v_stride < vd || softcap < 0.f || chunk < 0) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  AgOptions opt = {softcap, chunk, v_stride, sinks, gate, gate_ld, gate_scale};
  if (dtype != HK_F32 && dtype != HK_BF16) return HK_ERR_UNSUPPORTED;
#define AG_GO(T, PER) ag_launch<T, PER>(q, k_pages, v_pages, block_table, table_stride, positions, slot_of_token, out, n, H, G, hd, \
                                        page_tokens, window, scale, vd, sink, opt, s)
  if (widest <= 256) return dtype == HK_F32 ? AG_GO(float, 8) : AG_GO(bf16, 8);
  return dtype == HK_F32 ? AG_GO(float, 20) : AG_GO(bf16, 20);
#undef AG_GO
}
