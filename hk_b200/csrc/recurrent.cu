// Recurrent mixers: scans over the rows of every request of a step, with the state of a request kept in
// float32 in its state slot between steps.
//
// A step's batch is described by a segment table int32 [n_seg, 3] = (state slot, first row, rows): the rows
// of a request are consecutive and in increasing position.  Every scan walks a segment's rows in order, one
// token after the other, whatever the cut of the prompt was, so the state after a token (and every sum's
// order) depends on the tokens before it alone: never on the portion sizes, the batch or the slot.
//
//   * generalised delta rule (per head a matrix state S [dk, dv]):
//         S_t = diag(d_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,   o_t = S_t^T r_t
//     with the decay d_t = exp(-decay_scale * sigmoid(wl_t + w0)), the removal rate a_t = sigmoid(al_t + a0) and
//     the unit key u_t = k_t / sqrt(sum(k_t^2) + key_eps).  The columns of S (one per value channel) never mix:
//     a thread group owns one column, its dk entries spread over L lanes in registers, so a token costs two
//     dot products over dk and no synchronisation.  What a token brings (d, a*u, u, k, r, v) is prepared for all
//     tokens at once by a kernel of its own and reaches the scan in chunks through shared memory.
//   * gate of the delta rule's output: each head's o over its root mean square, times a weight, times
//     sigmoid(g), narrowed to the compute type for the output projection.
//   * minGRU (one scalar state per channel): S_t = (1 - z_t) S_(t-1) + z_t c_t with z_t = sigmoid(zl_t + bz),
//     c_t = x + 1/2 for x >= 0 and sigmoid(x) below, x = xl_t + bx; output S_t * silu(g_t).
//
// All arithmetic is float32; the projections that feed the scans arrive as float32.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------ generalised delta rule: what a token brings
// One warp per (token, head) writes the record that the scan reads: five vectors of P = L * RPT floats (d, a*u, u, k, r;
// P >= dk, the rest zero) and the dv values.  Inside a vector, entry i sits at (i % L) * RPT + i / L: lane `sub` of a
// column's L lanes owns the entries i = sub, sub + L, ... and finds them side by side.  Everything that does not depend
// on the state is computed here, for all tokens at once.
__global__ void delta_rule_prep_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                                       const float* __restrict__ al, long long ld, const float* __restrict__ wl, long long ldw,
                                       const float* __restrict__ a_bias, const float* __restrict__ w_bias, float* __restrict__ rec,
                                       long long items, int H, int dk, int dv, int L, int RPT, float decay_scale, float key_eps) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const size_t row = (size_t)(item / H);
  const int h = (int)(item % H);
  const size_t hoff = (size_t)h * dk;
  const float* kp = k + row * ld + hoff;
  float ss = 0.f;
  for (int i = lane; i < dk; i += 32) {
    const float kv = kp[i];
    ss = fmaf(kv, kv, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + key_eps);
  const int P = L * RPT;
  float* out = rec + (size_t)item * (5 * P + dv);
  for (int j = lane; j < P; j += 32) {
    const int i = (j % RPT) * L + j / RPT;       // the entry that sits at place j
    float d = 0.f, au = 0.f, u = 0.f, kv = 0.f, rv = 0.f;
    if (i < dk) {
      kv = kp[i];
      u = kv * inv;
      au = sigmoid_f(al[row * ld + hoff + i] + a_bias[hoff + i]) * u;
      d = expf(-decay_scale * sigmoid_f(wl[row * ldw + hoff + i] + w_bias[hoff + i]));
      rv = r[row * ld + hoff + i];
    }
    out[j] = d;
    out[P + j] = au;
    out[2 * P + j] = u;
    out[3 * P + j] = kv;
    out[4 * P + j] = rv;
  }
  for (int c = lane; c < dv; c += 32) out[5 * P + c] = v[row * ld + (size_t)h * dv + c];
}

// ------------------------------------------------------------------ generalised delta rule: the scan
// A block owns `cols` columns of one head's state for one segment; a column's state entries are spread over L lanes, RPT
// per lane, in registers.  Records arrive in chunks of `chunk` tokens through a two-stage cp.async ring (the next chunk is
// on its way while this one is walked) and are read with 16-byte loads.  Per token the chain that the next token waits
// for is: u . S (four partial sums, then L lanes by shuffle), then one fused update per state entry; the output's dot
// product hangs off that chain.  How many lanes share a column is chosen by the launcher: one lane (no shuffle, the fewest
// instructions) when requests and heads alone give the SMs enough warps, more when a single request must be spread out.
__device__ __forceinline__ void dr_cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int RPT, int L, int CPT>     // CPT: columns a lane group owns (they share every load of the token's vectors)
__global__ void __launch_bounds__(256)
delta_rule_scan_kernel(const float* __restrict__ rec, const int* __restrict__ segs, float* __restrict__ state,
                       float* __restrict__ out, int H, int dk, int dv, int cols, int chunk) {
  extern __shared__ __align__(16) float sm[];   // [2][chunk][5 P + dv]
  constexpr int P = L * RPT;
  const int R = 5 * P + dv;
  const int seg = blockIdx.x / H, h = blockIdx.x % H;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const int col0 = blockIdx.y * cols;
  const int tid = threadIdx.x;
  const int sub = tid % L, cidx = (tid / L) * CPT;           // first of this lane group's columns, within the block
  bool col_ok[CPT];
  int col[CPT];
  float S[CPT][RPT];
  float* sp = state + ((size_t)slot * H + h) * dk * dv;
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    col[c] = col0 + cidx + c;
    col_ok[c] = cidx + c < cols && col[c] < dv;
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
      const int i = sub + L * m;
      S[c][m] = (col_ok[c] && i < dk) ? sp[(size_t)i * dv + col[c]] : 0.f;
    }
  }
  const int pieces = R >> 2;                    // records are whole 16-byte pieces: P is a multiple of 8, dv of 4
  auto fetch = [&](int c) {                     // chunk c -> stage c & 1
    const int t0 = c * chunk, tc = min(chunk, count - t0);
    float* dst = sm + (size_t)(c & 1) * chunk * R;
    const float* src = rec + ((size_t)(row0 + t0) * H + h) * R;
    for (int t = 0; t < tc; ++t)
      for (int p = tid; p < pieces; p += blockDim.x) dr_cp_async16(dst + (size_t)t * R + 4 * p, src + (size_t)t * H * R + 4 * p);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int nchunks = (count + chunk - 1) / chunk;
  float* op = out + (size_t)row0 * H * dv + (size_t)h * dv + col[0];
  const size_t ostep = (size_t)H * dv;
  const bool lead = sub == 0;
  const int mine = sub * RPT, vat = 5 * P + min(col[0], dv - CPT);
  fetch(0);
  for (int c = 0; c < nchunks; ++c) {
    if (c + 1 < nchunks) {
      fetch(c + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int tc = min(chunk, count - c * chunk);
    const float* buf = sm + (size_t)(c & 1) * chunk * R + mine;
    const float* vbuf = sm + (size_t)(c & 1) * chunk * R + vat;
#pragma unroll 2
    for (int t = 0; t < tc; ++t) {
      const float* tok = buf + (size_t)t * R;
      float du[CPT][2];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) du[cc][0] = du[cc][1] = 0.f;
#pragma unroll
      for (int q = 0; q < RPT / 4; ++q) {
        const float4 u = *reinterpret_cast<const float4*>(tok + 2 * P + 4 * q);
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          du[cc][0] = fmaf(u.y, S[cc][4 * q + 1], fmaf(u.x, S[cc][4 * q], du[cc][0]));
          du[cc][1] = fmaf(u.w, S[cc][4 * q + 3], fmaf(u.z, S[cc][4 * q + 2], du[cc][1]));
        }
      }
      float dus[CPT];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) dus[cc] = du[cc][0] + du[cc][1];
#pragma unroll
      for (int o = L >> 1; o > 0; o >>= 1)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) dus[cc] += __shfl_xor_sync(0xffffffffu, dus[cc], o);
      float v[CPT], acc[CPT][2];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        v[cc] = vbuf[(size_t)t * R + cc];
        acc[cc][0] = acc[cc][1] = 0.f;
      }
#pragma unroll
      for (int q = 0; q < RPT / 4; ++q) {
        const float4 d = *reinterpret_cast<const float4*>(tok + 4 * q);
        const float4 au = *reinterpret_cast<const float4*>(tok + P + 4 * q);
        const float4 k = *reinterpret_cast<const float4*>(tok + 3 * P + 4 * q);
        const float4 r = *reinterpret_cast<const float4*>(tok + 4 * P + 4 * q);
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          float* Sc = S[cc];
          Sc[4 * q] = fmaf(k.x, v[cc], fmaf(-au.x, dus[cc], d.x * Sc[4 * q]));
          Sc[4 * q + 1] = fmaf(k.y, v[cc], fmaf(-au.y, dus[cc], d.y * Sc[4 * q + 1]));
          Sc[4 * q + 2] = fmaf(k.z, v[cc], fmaf(-au.z, dus[cc], d.z * Sc[4 * q + 2]));
          Sc[4 * q + 3] = fmaf(k.w, v[cc], fmaf(-au.w, dus[cc], d.w * Sc[4 * q + 3]));
          acc[cc][0] = fmaf(r.y, Sc[4 * q + 1], fmaf(r.x, Sc[4 * q], acc[cc][0]));
          acc[cc][1] = fmaf(r.w, Sc[4 * q + 3], fmaf(r.z, Sc[4 * q + 2], acc[cc][1]));
        }
      }
      float o_[CPT];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) o_[cc] = acc[cc][0] + acc[cc][1];
#pragma unroll
      for (int o = L >> 1; o > 0; o >>= 1)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) o_[cc] += __shfl_xor_sync(0xffffffffu, o_[cc], o);
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc)
        if (lead && col_ok[cc]) op[(size_t)t * ostep + cc] = o_[cc];
    }
    op += (size_t)tc * ostep;
    __syncthreads();                            // the stage may be filled again
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
      const int i = sub + L * m;
      if (col_ok[c] && i < dk) sp[(size_t)i * dv + col[c]] = S[c][m];
    }
}

// The plain form of the scan for value sizes that are no multiple of 4 (records that are not whole 16-byte pieces):
// the same recurrence, the state in shared memory, records read with plain loads, one token at a time.
__global__ void delta_rule_scan_plain_kernel(const float* __restrict__ rec, const int* __restrict__ segs, float* __restrict__ state,
                                             float* __restrict__ out, int H, int dk, int dv, int L, int RPT, int cols) {
  extern __shared__ __align__(16) float sm[];   // [blockDim / L][P] the state columns; then one record
  const int P = L * RPT, R = 5 * P + dv;
  const int seg = blockIdx.x / H, h = blockIdx.x % H;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const int tid = threadIdx.x, sub = tid % L, cidx = tid / L, col = blockIdx.y * cols + cidx;
  const bool col_ok = cidx < cols && col < dv;
  float* Sc = sm + (size_t)cidx * P;             // this column's state, in the record's order of entries
  float* recs = sm + (size_t)(blockDim.x / L) * P;
  float* sp = state + ((size_t)slot * H + h) * dk * dv;
  for (int m = 0; m < RPT; ++m) {
    const int i = sub + L * m;
    Sc[sub * RPT + m] = (col_ok && i < dk) ? sp[(size_t)i * dv + col] : 0.f;
  }
  for (int t = 0; t < count; ++t) {
    __syncthreads();
    const float* src = rec + ((size_t)(row0 + t) * H + h) * R;
    for (int p = tid; p < R; p += blockDim.x) recs[p] = src[p];
    __syncthreads();
    const float* mine = recs + sub * RPT;
    float du0 = 0.f, du1 = 0.f;
    for (int m = 0; m < RPT; m += 2) {
      du0 = fmaf(mine[2 * P + m], Sc[sub * RPT + m], du0);
      if (m + 1 < RPT) du1 = fmaf(mine[2 * P + m + 1], Sc[sub * RPT + m + 1], du1);
    }
    float du = du0 + du1;
    for (int o = L >> 1; o > 0; o >>= 1) du += __shfl_xor_sync(0xffffffffu, du, o);
    const float vj = recs[5 * P + min(col, dv - 1)];
    float a0 = 0.f, a1 = 0.f;
    for (int m = 0; m < RPT; ++m) {
      const float sn = fmaf(mine[3 * P + m], vj, fmaf(-mine[P + m], du, mine[m] * Sc[sub * RPT + m]));
      Sc[sub * RPT + m] = sn;
      if (m & 1) a1 = fmaf(mine[4 * P + m], sn, a1); else a0 = fmaf(mine[4 * P + m], sn, a0);
    }
    float acc = a0 + a1;
    for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (col_ok && sub == 0) out[(size_t)(row0 + t) * H * dv + (size_t)h * dv + col] = acc;
  }
  for (int m = 0; m < RPT; ++m) {
    const int i = sub + L * m;
    if (col_ok && i < dk) sp[(size_t)i * dv + col] = Sc[sub * RPT + m];
  }
}

// How a column's dk state entries are laid over lanes: L lanes with RPT entries each (RPT in 8, 16, 32, 64; L * RPT >= dk
// with as little padding as there can be).  `spread` asks for at least that many lanes: more warps for a small batch.
static void dr_layout(int dk, int spread, int* L_out, int* rpt_out) {
  int L = 1;
  while (L < 32 && (dk + L - 1) / L > 64) L <<= 1;
  while (L < 32 && L < spread && (dk + 2 * L - 1) / (2 * L) >= 8) L <<= 1;
  int rpt = 8;
  while (rpt < 64 && rpt * L < dk) rpt <<= 1;
  *L_out = L;
  *rpt_out = rpt * L >= dk ? rpt : 0;           // 0: dk above 2,048
}

// The most scratch floats per (token, head) that `hk_delta_rule_scan` may need in `rec`, whatever layout it chooses.
HK_API int hk_delta_rule_record(int dk, int dv) {
  int most = 0;
  for (int spread = 1; spread <= 32; spread <<= 1) {
    int L, rpt;
    dr_layout(dk, spread, &L, &rpt);
    if (rpt && 5 * L * rpt + dv > most) most = 5 * L * rpt + dv;
  }
  return most;
}

template <int RPT, int CPT>
static int dr_launch(int L, dim3 grid, int threads, size_t smem, cudaStream_t s, const float* rec, const int* segs, float* state,
                     float* out, int H, int dk, int dv, int cols, int chunk) {
#define DR_LAUNCH(LL)                                                                                                       \
  do {                                                                                                                      \
    static HkSmemCache cache;                                                                                               \
    int e = hk_allow_smem(delta_rule_scan_kernel<RPT, LL, CPT>, smem, cache);                                               \
    if (e) return e;                                                                                                        \
    return hk_launch(delta_rule_scan_kernel<RPT, LL, CPT>, grid, dim3(threads), smem, s, rec, segs, state, out, H, dk, dv, cols, \
                     chunk);                                                                                                \
  } while (0)
  switch (L) {
    case 1: DR_LAUNCH(1);
    case 2: DR_LAUNCH(2);
    case 4: DR_LAUNCH(4);
    case 8: DR_LAUNCH(8);
    case 16: DR_LAUNCH(16);
    default: DR_LAUNCH(32);
  }
#undef DR_LAUNCH
}

// Lanes per column for a step: one where requests x heads x columns alone give every SM four warps or more, else as many
// as that takes.  Returns 0 for a key size that no layout holds.
static int dr_plan(int n_seg, int H, int dk, int dv, int* L_out, int* rpt_out) {
  const long long warps1 = ((long long)n_seg * H * dv + 31) / 32;
  int spread = 1;
  while (spread < 32 && warps1 * spread < 4 * 148) spread <<= 1;
  dr_layout(dk, spread, L_out, rpt_out);
  return *rpt_out;
}

// The scan over records that a prep kernel wrote with the layout (L, rpt) of `dr_plan`.
static int dr_scan_records(const float* rec, const int* segs, int n_seg, float* state, float* out, int H, int dk, int dv, int L,
                           int rpt, cudaStream_t s) {
  const int R = 5 * L * rpt + dv;
  if (dv & 3) {
    const int cols = max(1, min(dv, 128 / L));
    const int threads = ((cols * L + 31) / 32) * 32;      // whole warps: the lanes of a column meet by shuffle
    const size_t smem = (size_t)(threads * rpt + R) * sizeof(float);
    static HkSmemCache cache;
    int e = hk_allow_smem(delta_rule_scan_plain_kernel, smem, cache);
    if (e) return e;
    return hk_launch(delta_rule_scan_plain_kernel, dim3((unsigned)(n_seg * H), (unsigned)((dv + cols - 1) / cols)), dim3(threads), smem, s,
                     rec, segs, state, out, H, dk, dv, L, rpt, cols);
  }
  // a block takes as many columns as 256 threads hold (they share the records that the ring brings), fewer while the
  // blocks do not yet fill the SMs twice: one request of 2,048 tokens at 32 heads of 64 runs 808 us with 8 columns a
  // block (256 blocks of 64 threads) against 1,096 with 32 and 839 with 4; below 4 every block fetches too much
  int cols = max(1, min(dv, 256 / L));
  while (cols > 8 && cols * L > 64 && (long long)n_seg * H * ((dv + cols - 1) / cols) < 2 * 148) cols >>= 1;
  // two columns a lane group where a lane holds 8 state entries a column (they share the loads of the token's vectors,
  // and their two chains of arithmetic hide each other's latency) and the block's columns are even
  // (one request of 2,048 tokens: 64 heads of 64, 512 blocks: 1.00 ms against 1.12; 32 heads, 256 blocks: 0.89 against 0.78,
  // so only where the blocks fill the SMs twice)
  const bool many = (long long)n_seg * H * ((dv + cols - 1) / cols) >= 2 * 148;
  const int cpt = (rpt == 8 && many && (cols & 1) == 0 && (dv & 1) == 0) ? 2 : 1;
  const int threads = ((cols / cpt * L + 31) / 32) * 32;
  int chunk = 16;
  while (chunk > 2 && (size_t)2 * chunk * R * sizeof(float) > 64 * 1024) chunk >>= 1;
  const size_t smem = (size_t)2 * chunk * R * sizeof(float);
  dim3 grid((unsigned)(n_seg * H), (unsigned)((dv + cols - 1) / cols));
  if (rpt == 8 && cpt == 2) return dr_launch<8, 2>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
  if (rpt == 8) return dr_launch<8, 1>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
  if (rpt == 16) return dr_launch<16, 1>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
  if (rpt == 32) return dr_launch<32, 1>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
  return dr_launch<64, 1>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
}

// `rec`: scratch of n_rows * H * hk_delta_rule_record(dk, dv) floats (16-byte aligned) that the call fills and reads.
HK_API int hk_delta_rule_scan(const float* r, const float* k, const float* v, const float* al, long long ld, const float* wl,
                              long long ldw, const float* a_bias, const float* w_bias, const int* segs, int n_seg, int n_rows,
                              float* rec, float* state, float* out, int H, int dk, int dv, float decay_scale, float key_eps,
                              void* stream) {
  if (n_seg <= 0 || n_rows <= 0) return 0;
  if (H < 1 || dk < 1 || dv < 1 || dk > 2048 || ((uintptr_t)rec & 15)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  int L, rpt;
  if (!dr_plan(n_seg, H, dk, dv, &L, &rpt)) return HK_ERR_UNSUPPORTED;
  {
    const long long items = (long long)n_rows * H;
    int e = hk_launch(delta_rule_prep_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, s, r, k, v, al, ld, wl, ldw, a_bias,
                      w_bias, rec, items, H, dk, dv, L, rpt, decay_scale, key_eps);
    if (e) return e;
  }
  return dr_scan_records(rec, segs, n_seg, state, out, H, dk, dv, L, rpt, s);
}

// ------------------------------------------------------------------ generalised delta rule: the output's gate
// One warp per (token, head): y = o / sqrt(mean(o^2) + eps) * weight * sigmoid(g), narrowed to T.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ g, long long ldg,
                                      const float* __restrict__ weight, T* __restrict__ out, long long items, int H, int dv,
                                      float eps) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const long long t = item / H;
  const int h = (int)(item % H);
  const float* src = o + (size_t)item * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) {
    const float a = src[i];
    ss = fmaf(a, a, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int i = lane; i < dv; i += 32) {
    const float gate = sigmoid_f(g[(size_t)t * ldg + (size_t)h * dv + i]);
    out[(size_t)item * dv + i] = from_f32<T>(src[i] * inv * weight[(size_t)h * dv + i] * gate);
  }
}

HK_API int hk_head_norm_gate(const float* o, const float* g, long long ldg, const float* weight, void* out, int out_dtype, int n,
                             int H, int dv, float eps, void* stream) {
  if (n <= 0) return 0;
  const long long items = (long long)n * H;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == HK_F32)
    return hk_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, s, o, g, ldg, weight, (float*)out, items, H, dv, eps);
  if (out_dtype == HK_BF16)
    return hk_launch(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, s, o, g, ldg, weight, (bf16*)out, items, H, dv, eps);
  return HK_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------ minGRU
// proj[n, 3W] = [z logits | candidate inputs | gate inputs].  A block owns 32 channels of a segment and walks it in
// chunks of MG_CHUNK tokens: all threads turn the chunk's inputs into a = 1 - z, b = z * c and silu(g) (in parallel,
// the next chunk's inputs already on their way in registers), one warp runs the recurrence S <- a S + b down the
// chunk, a channel per lane, and all threads write S * silu(g).
#define MG_CHUNK 64
#define MG_LANES 8      // token lanes: a thread takes every 8th token of a chunk in the parallel phases
#define MG_PER (MG_CHUNK / MG_LANES)

template <typename T>
__global__ void __launch_bounds__(32 * MG_LANES)
mingru_scan_kernel(const float* __restrict__ proj, long long ld, const float* __restrict__ z_bias,
                   const float* __restrict__ x_bias, const int* __restrict__ segs, float* __restrict__ state,
                   T* __restrict__ out, int W) {
  __shared__ float sa[MG_CHUNK][32], sb[MG_CHUNK][32], sg[MG_CHUNK][32];
  const int seg = blockIdx.x;
  const int ch = threadIdx.x & 31, tl = threadIdx.x >> 5;
  const int c = blockIdx.y * 32 + ch;
  const bool ok = c < W;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const float bz = (ok && z_bias) ? z_bias[c] : 0.f, bx = (ok && x_bias) ? x_bias[c] : 0.f;
  float S = (ok && tl == 0) ? state[(size_t)slot * W + c] : 0.f;
  if (count == 1) {                              // a decoded token: nothing to stage, one lane per channel does it all
    if (ok && tl == 0) {
      const float* p = proj + (size_t)row0 * ld + c;
      const float z = sigmoid_f(p[0] + bz);
      const float x = p[W] + bx;
      const float g = p[2 * (size_t)W];
      S = fmaf(1.0f - z, S, z * (x >= 0.f ? x + 0.5f : sigmoid_f(x)));
      out[(size_t)row0 * W + c] = from_f32<T>(S * (g * sigmoid_f(g)));
      state[(size_t)slot * W + c] = S;
    }
    return;
  }
  float zl[MG_PER], xl[MG_PER], gl[MG_PER];
  auto fetch = [&](int t0) {
#pragma unroll
    for (int j = 0; j < MG_PER; ++j) {
      const int t = t0 + tl + j * MG_LANES;
      const bool in = ok && t < count;
      const float* p = proj + (size_t)(row0 + (in ? t : 0)) * ld + (ok ? c : 0);
      zl[j] = in ? p[0] : 0.f;
      xl[j] = in ? p[W] : 0.f;
      gl[j] = in ? p[2 * (size_t)W] : 0.f;
    }
  };
  fetch(0);
  for (int t0 = 0; t0 < count; t0 += MG_CHUNK) {
    const int tc = min(MG_CHUNK, count - t0);
#pragma unroll
    for (int j = 0; j < MG_PER; ++j) {
      const int t = tl + j * MG_LANES;
      const float z = sigmoid_f(zl[j] + bz);
      const float x = xl[j] + bx;
      const float cand = x >= 0.f ? x + 0.5f : sigmoid_f(x);
      sa[t][ch] = 1.0f - z;
      sb[t][ch] = z * cand;
      sg[t][ch] = gl[j] * sigmoid_f(gl[j]);
    }
    __syncthreads();
    if (t0 + MG_CHUNK < count) fetch(t0 + MG_CHUNK);      // in flight while the recurrence runs
    if (tl == 0) {
      for (int t = 0; t < tc; ++t) {
        S = fmaf(sa[t][ch], S, sb[t][ch]);
        sa[t][ch] = S;
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < MG_PER; ++j) {
      const int t = tl + j * MG_LANES;
      if (ok && t < tc) out[(size_t)(row0 + t0 + t) * W + c] = from_f32<T>(sa[t][ch] * sg[t][ch]);
    }
    __syncthreads();                                     // the chunk's arrays are free again
  }
  if (ok && tl == 0) state[(size_t)slot * W + c] = S;
}

HK_API int hk_mingru_scan(const float* proj, long long ld, const float* z_bias, const float* x_bias, const int* segs, int n_seg,
                          float* state, void* out, int out_dtype, int W, void* stream) {
  if (n_seg <= 0 || W <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((unsigned)n_seg, (unsigned)((W + 31) / 32));
  if (out_dtype == HK_F32)
    return hk_launch(mingru_scan_kernel<float>, grid, dim3(32 * MG_LANES), 0, s, proj, ld, z_bias, x_bias, segs, state, (float*)out, W);
  if (out_dtype == HK_BF16)
    return hk_launch(mingru_scan_kernel<bf16>, grid, dim3(32 * MG_LANES), 0, s, proj, ld, z_bias, x_bias, segs, state, (bf16*)out, W);
  return HK_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------ short causal convolution per channel
// y[t, c] = act(sum_j w[c, j] * x[t - (taps - 1) + j, c]) over the rows of every segment, with act = silu (1) or the
// identity (0): the last column of w is the current token's.  The inputs before a segment's first row come from the request's tail
// (state [slots, taps - 1, C], the last taps - 1 inputs of the request, zero at its start), which the same call
// moves on.  x and y are column slices [n, C] of wider float32 matrices.  A thread owns one channel of one chunk
// of a segment's tokens; the threads of the first chunk read the old tail before they write the new one, and
// nobody else touches it.
#define SC_TOKENS 32
#define SC_GROUP 8
#define SC_MAX_TAPS 16

// The thread walks its tokens in groups of SC_GROUP: the group's inputs are loaded at once (each input is read once; the
// taps - 1 before them stay in registers from the group before), then the group's outputs are summed, oldest tap first.
__global__ void __launch_bounds__(128)
short_conv_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w, const int* __restrict__ segs,
                  float* __restrict__ tail, float* __restrict__ y, long long ldy, int C, int taps, int act) {
  const int seg = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const int t0 = blockIdx.z * SC_TOKENS;
  if (c >= C || t0 >= count) return;
  const int back = taps - 1;
  float* tl = tail + (size_t)slot * back * C + c;
  auto input = [&](int r) -> float {            // the request's input r rows from the segment's first (r may be negative)
    return r >= 0 ? x[(size_t)(row0 + r) * ldx + c] : tl[(size_t)(back + r) * C];
  };
  float wr[SC_MAX_TAPS];                        // wr[s]: the weight of the input s tokens back
  float hist[SC_MAX_TAPS];                      // hist[s], s >= 1: the input s tokens before the group's first
#pragma unroll
  for (int s = 0; s < SC_MAX_TAPS; ++s) {
    wr[s] = s <= back ? w[(size_t)c * taps + back - s] : 0.f;
    hist[s] = (s >= 1 && s <= back) ? input(t0 - s) : 0.f;
  }
  const int t1 = min(count, t0 + SC_TOKENS);
  for (int tg = t0; tg < t1; tg += SC_GROUP) {
    float nw[SC_GROUP];
#pragma unroll
    for (int u = 0; u < SC_GROUP; ++u) nw[u] = tg + u < t1 ? x[(size_t)(row0 + tg + u) * ldx + c] : 0.f;
    float acc[SC_GROUP];
#pragma unroll
    for (int u = 0; u < SC_GROUP; ++u) acc[u] = 0.f;
#pragma unroll
    for (int s = SC_MAX_TAPS - 1; s >= 0; --s) {
      if (s <= back) {
#pragma unroll
        for (int u = 0; u < SC_GROUP; ++u) acc[u] = fmaf(wr[s], u >= s ? nw[u - s] : hist[s - u], acc[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < SC_GROUP; ++u)
      if (tg + u < t1) y[(size_t)(row0 + tg + u) * ldy + c] = act ? acc[u] / (1.0f + expf(-acc[u])) : acc[u];
    float next[SC_MAX_TAPS];
#pragma unroll
    for (int s = 1; s < SC_MAX_TAPS; ++s) next[s] = s <= SC_GROUP ? nw[SC_GROUP - s] : hist[s - SC_GROUP];
#pragma unroll
    for (int s = 1; s < SC_MAX_TAPS; ++s) hist[s] = next[s];
  }
  if (blockIdx.z == 0 && back > 0) {
    float keep[SC_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS; ++j)
      if (j < back) keep[j] = input(count - back + j);
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS; ++j)
      if (j < back) tl[(size_t)j * C] = keep[j];
  }
}

HK_API int hk_short_conv(const float* x, long long ldx, const float* w, const int* segs, int n_seg, int n_rows, float* tail,
                         float* y, long long ldy, int C, int taps, int act, void* stream) {
  if (n_seg <= 0 || n_rows <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > SC_MAX_TAPS || act < 0 || act > 1) return HK_ERR_UNSUPPORTED;
  dim3 grid((unsigned)n_seg, (unsigned)((C + 127) / 128), (unsigned)((n_rows + SC_TOKENS - 1) / SC_TOKENS));
  return hk_launch(short_conv_kernel, grid, dim3(128), 0, (cudaStream_t)stream, x, ldx, w, segs, tail, y, ldy, C, taps, act);
}

// ------------------------------------------------------------------ gated delta rule
// Per head a matrix state S [dk, dv] and per token a scalar decay g and a scalar write strength beta:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with q and k unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times q_scale, g = exp(-exp(A_log) *
// softplus(a_logit + dt_bias)), beta = sigmoid(b_logit).  Query/key head h / (H / G) serves value head h.  Written out,
// S_new = g S - (g beta k)(k^T S) + k (beta v)^T, which is the generalised rule's record (d, a*u, u, k, r, v) =
// (g, g beta k, k, k, q, beta v): the scan above runs it.
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__global__ void gated_delta_prep_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                        long long ld, const float* __restrict__ bl, const float* __restrict__ al, long long ldg,
                                        const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ rec,
                                        long long items, int H, int G, int dk, int dv, int L, int RPT, float q_scale,
                                        float unit_eps) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const size_t row = (size_t)(item / H);
  const int h = (int)(item % H);
  const int g = h / (H / G);
  const float* qp = q + row * ld + (size_t)g * dk;
  const float* kp = k + row * ld + (size_t)g * dk;
  float sq = 0.f, sk = 0.f;
  for (int i = lane; i < dk; i += 32) {
    const float a = qp[i], b = kp[i];
    sq = fmaf(a, a, sq);
    sk = fmaf(b, b, sk);
  }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  const float qinv = q_scale / sqrtf(sq + unit_eps), kinv = 1.0f / sqrtf(sk + unit_eps);
  const float beta = sigmoid_f(bl[row * ldg + h]);
  const float decay = expf(-expf(a_log[h]) * softplus_f(al[row * ldg + h] + dt_bias[h]));
  const int P = L * RPT;
  float* out = rec + (size_t)item * (5 * P + dv);
  for (int j = lane; j < P; j += 32) {
    const int i = (j % RPT) * L + j / RPT;       // the entry that sits at place j
    float d = 0.f, au = 0.f, u = 0.f, rv = 0.f;
    if (i < dk) {
      u = kp[i] * kinv;
      au = decay * beta * u;
      d = decay;
      rv = qp[i] * qinv;
    }
    out[j] = d;
    out[P + j] = au;
    out[2 * P + j] = u;
    out[3 * P + j] = u;
    out[4 * P + j] = rv;
  }
  for (int c = lane; c < dv; c += 32) out[5 * P + c] = beta * v[row * ld + (size_t)h * dv + c];
}

// q, k [n, G*dk] and v [n, H*dv] are column slices of one float32 matrix (row stride ld), already convolved and
// activated; b_logit and a_logit [n, H] slices of one (row stride ldg).  `rec` as for hk_delta_rule_scan.
HK_API int hk_gated_delta_scan(const float* q, const float* k, const float* v, long long ld, const float* bl, const float* al,
                               long long ldg, const float* a_log, const float* dt_bias, const int* segs, int n_seg, int n_rows,
                               float* rec, float* state, float* out, int H, int G, int dk, int dv, float q_scale, float unit_eps,
                               void* stream) {
  if (n_seg <= 0 || n_rows <= 0) return 0;
  if (H < 1 || G < 1 || H % G || dk < 1 || dv < 1 || dk > 2048 || ((uintptr_t)rec & 15)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  int L, rpt;
  if (!dr_plan(n_seg, H, dk, dv, &L, &rpt)) return HK_ERR_UNSUPPORTED;
  const long long items = (long long)n_rows * H;
  int e = hk_launch(gated_delta_prep_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, s, q, k, v, ld, bl, al, ldg, a_log,
                    dt_bias, rec, items, H, G, dk, dv, L, rpt, q_scale, unit_eps);
  if (e) return e;
  return dr_scan_records(rec, segs, n_seg, state, out, H, dk, dv, L, rpt, s);
}

// ------------------------------------------------------------------ retention
// Linear attention with a fixed decay per head and neither softmax nor denominator:
//     S <- decay_h S + k v^T;   o = S^T q
// q and k [n, H * dk] are first turned by position on their first `rot` dims (dim i paired with i + rot / 2, angle from
// the tables cos, sin [positions, rot / 2]; rot = 0: no rotation), k then times k_scale.  The preparation writes, per
// (token, head), either the lean record [k | q | v] (2 P + dv floats, the vectors in the scan's lane layout) for the scan
// below, or (value sizes that are no multiple of 4) the generalised rule's record (d, a*u, u, k, r, v) =
// (decay_h, 0, 0, k, q, v), which that rule's plain scan runs.
__global__ void retention_prep_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                      long long ld, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                                      const int* __restrict__ positions, const float* __restrict__ decay, float* __restrict__ rec,
                                      long long items, int H, int dk, int dv, int L, int RPT, float k_scale, int lean) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const size_t row = (size_t)(item / H);
  const int h = (int)(item % H);
  const float* qp = q + row * ld + (size_t)h * dk;
  const float* kp = k + row * ld + (size_t)h * dk;
  const int half = rot >> 1;
  const float* c = cos_t + (size_t)positions[row] * half;
  const float* s = sin_t + (size_t)positions[row] * half;
  const float dec = decay[h];
  const int P = L * RPT;
  float* out = rec + (size_t)item * ((lean ? 2 : 5) * P + dv);
  for (int j = lane; j < P; j += 32) {
    const int i = (j % RPT) * L + j / RPT;       // the entry that sits at place j
    float kv = 0.f, qv = 0.f;
    if (i < dk) {
      if (i < half) {
        kv = kp[i] * c[i] - kp[i + half] * s[i];
        qv = qp[i] * c[i] - qp[i + half] * s[i];
      } else if (i < rot) {
        kv = kp[i] * c[i - half] + kp[i - half] * s[i - half];
        qv = qp[i] * c[i - half] + qp[i - half] * s[i - half];
      } else {
        kv = kp[i];
        qv = qp[i];
      }
      kv *= k_scale;
    }
    if (lean) {
      out[j] = kv;
      out[P + j] = qv;
    } else {
      out[j] = i < dk ? dec : 0.f;
      out[P + j] = 0.f;
      out[2 * P + j] = 0.f;
      out[3 * P + j] = kv;
      out[4 * P + j] = qv;
    }
  }
  float* vo = out + (lean ? 2 : 5) * P;
  for (int cidx = lane; cidx < dv; cidx += 32) vo[cidx] = v[row * ld + (size_t)h * dv + cidx];
}

// The scan over lean records: the delta rule's layout of the state (a block owns `cols` columns of one head's state for
// one segment, a column's entries spread over L lanes, RPT per lane, in registers; records through a two-stage cp.async
// ring), but the chain that the next token waits for is one multiply and one fused multiply-add per state entry: no dot
// product with the old state, no shuffle before the update.  The read-out's dot product hangs off that chain, and its sum
// over a column's L lanes is put off: every lane leaves its share of a token's output in shared memory, and after a chunk
// of tokens the block adds the shares (lane 0 first, in order) and writes the chunk's outputs, neighbours side by side.
template <int RPT, int L, int CPT>
__global__ void __launch_bounds__(256)
retention_scan_kernel(const float* __restrict__ rec, const int* __restrict__ segs, const float* __restrict__ decay,
                      float* __restrict__ state, float* __restrict__ out, int H, int dk, int dv, int cols, int chunk) {
  extern __shared__ __align__(16) float sm[];   // [2][chunk][2 P + dv] records, then [2][chunk][W] the lanes' shares
  constexpr int P = L * RPT;
  const int R = 2 * P + dv;
  const int W = blockDim.x * CPT;               // shares a token: one per (column of the block, lane)
  float* part = sm + (size_t)2 * chunk * R;
  const int seg = blockIdx.x / H, h = blockIdx.x % H;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const int col0 = blockIdx.y * cols;
  const int tid = threadIdx.x;
  const int sub = tid % L, cidx = (tid / L) * CPT;
  const float dec = decay[h];
  bool col_ok[CPT];
  int col[CPT];
  float S[CPT][RPT];
  float* sp = state + ((size_t)slot * H + h) * dk * dv;
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    col[c] = col0 + cidx + c;
    col_ok[c] = cidx + c < cols && col[c] < dv;
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
      const int i = sub + L * m;
      S[c][m] = (col_ok[c] && i < dk) ? sp[(size_t)i * dv + col[c]] : 0.f;
    }
  }
  const int pieces = R >> 2;                    // records are whole 16-byte pieces: P is a multiple of 8, dv of 4
  auto fetch = [&](int c) {                     // chunk c -> stage c & 1
    const int t0 = c * chunk, tc = min(chunk, count - t0);
    float* dst = sm + (size_t)(c & 1) * chunk * R;
    const float* src = rec + ((size_t)(row0 + t0) * H + h) * R;
    for (int t = 0; t < tc; ++t)
      for (int p = tid; p < pieces; p += blockDim.x) dr_cp_async16(dst + (size_t)t * R + 4 * p, src + (size_t)t * H * R + 4 * p);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int nchunks = (count + chunk - 1) / chunk;
  float* op = out + (size_t)row0 * H * dv + (size_t)h * dv + col0;
  const size_t ostep = (size_t)H * dv;
  const int ncols = min(cols, dv - col0);       // columns of this block that exist
  const int mine = sub * RPT, vat = 2 * P + min(col[0], dv - CPT);
  fetch(0);
  for (int c = 0; c < nchunks; ++c) {
    if (c + 1 < nchunks) {
      fetch(c + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int tc = min(chunk, count - c * chunk);
    const float* buf = sm + (size_t)(c & 1) * chunk * R + mine;
    const float* vbuf = sm + (size_t)(c & 1) * chunk * R + vat;
    float* pw = part + (size_t)(c & 1) * chunk * W + (size_t)cidx * L + sub;
#pragma unroll 4
    for (int t = 0; t < tc; ++t) {
      const float* tok = buf + (size_t)t * R;
      float v[CPT], acc[CPT][2];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        v[cc] = vbuf[(size_t)t * R + cc];
        acc[cc][0] = acc[cc][1] = 0.f;
      }
#pragma unroll
      for (int q = 0; q < RPT / 4; ++q) {
        const float4 k = *reinterpret_cast<const float4*>(tok + 4 * q);
        const float4 r = *reinterpret_cast<const float4*>(tok + P + 4 * q);
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          float* Sc = S[cc];
          Sc[4 * q] = fmaf(k.x, v[cc], dec * Sc[4 * q]);
          Sc[4 * q + 1] = fmaf(k.y, v[cc], dec * Sc[4 * q + 1]);
          Sc[4 * q + 2] = fmaf(k.z, v[cc], dec * Sc[4 * q + 2]);
          Sc[4 * q + 3] = fmaf(k.w, v[cc], dec * Sc[4 * q + 3]);
          acc[cc][0] = fmaf(r.y, Sc[4 * q + 1], fmaf(r.x, Sc[4 * q], acc[cc][0]));
          acc[cc][1] = fmaf(r.w, Sc[4 * q + 3], fmaf(r.z, Sc[4 * q + 2], acc[cc][1]));
        }
      }
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) pw[(size_t)t * W + cc * L] = acc[cc][0] + acc[cc][1];
    }
    __syncthreads();                            // the shares are written; the stage may be filled again
    // (the shares of chunk c + 2 go to this buffer again, behind the barrier of chunk c + 1, which every thread reaches
    // only after it has read what it needs here)
    const float* pr = part + (size_t)(c & 1) * chunk * W;
    for (int e = tid; e < tc * ncols; e += blockDim.x) {
      const int t = e / ncols, cl = e % ncols;
      const float* shares = pr + (size_t)t * W + (size_t)cl * L;
      float sum = shares[0];
#pragma unroll
      for (int l = 1; l < L; ++l) sum += shares[l];
      op[(size_t)t * ostep + cl] = sum;
    }
    op += (size_t)tc * ostep;
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
      const int i = sub + L * m;
      if (col_ok[c] && i < dk) sp[(size_t)i * dv + col[c]] = S[c][m];
    }
}

template <int RPT, int CPT>
static int ret_launch(int L, dim3 grid, int threads, size_t smem, cudaStream_t s, const float* rec, const int* segs,
                      const float* decay, float* state, float* out, int H, int dk, int dv, int cols, int chunk) {
#define RET_LAUNCH(LL)                                                                                                      \
  do {                                                                                                                      \
    static HkSmemCache cache;                                                                                               \
    int e = hk_allow_smem(retention_scan_kernel<RPT, LL, CPT>, smem, cache);                                                \
    if (e) return e;                                                                                                        \
    return hk_launch(retention_scan_kernel<RPT, LL, CPT>, grid, dim3(threads), smem, s, rec, segs, decay, state, out, H, dk, dv, \
                     cols, chunk);                                                                                          \
  } while (0)
  switch (L) {
    case 1: RET_LAUNCH(1);
    case 2: RET_LAUNCH(2);
    case 4: RET_LAUNCH(4);
    case 8: RET_LAUNCH(8);
    case 16: RET_LAUNCH(16);
    default: RET_LAUNCH(32);
  }
#undef RET_LAUNCH
}

// q, k [n, H*dk] and v [n, H*dv] are column slices of one float32 matrix (row stride ld); decay float32 [H]; `rec` as for
// hk_delta_rule_scan.  Blocks, columns a block and columns a lane group are chosen as for the delta rule's scan.
HK_API int hk_retention_scan(const float* q, const float* k, const float* v, long long ld, const float* cos_t, const float* sin_t,
                             int rot, const int* positions, const float* decay, const int* segs, int n_seg, int n_rows, float* rec,
                             float* state, float* out, int H, int dk, int dv, float k_scale, void* stream) {
  if (n_seg <= 0 || n_rows <= 0) return 0;
  if (H < 1 || dk < 1 || dv < 1 || dk > 2048 || rot < 0 || rot > dk || (rot & 1) || ((uintptr_t)rec & 15)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  int L, rpt;
  if (!dr_plan(n_seg, H, dk, dv, &L, &rpt)) return HK_ERR_UNSUPPORTED;
  const long long items = (long long)n_rows * H;
  const int lean = (dv & 3) == 0;
  int e = hk_launch(retention_prep_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, s, q, k, v, ld, cos_t, sin_t, rot,
                    positions, decay, rec, items, H, dk, dv, L, rpt, k_scale, lean);
  if (e) return e;
  if (!lean) return dr_scan_records(rec, segs, n_seg, state, out, H, dk, dv, L, rpt, s);
  const int R = 2 * L * rpt + dv;
  int cols = max(1, min(dv, 256 / L));
  while (cols > 8 && cols * L > 64 && (long long)n_seg * H * ((dv + cols - 1) / cols) < 2 * 148) cols >>= 1;
  const bool many = (long long)n_seg * H * ((dv + cols - 1) / cols) >= 2 * 148;
  const int cpt = (rpt == 8 && many && (cols & 1) == 0 && (dv & 1) == 0) ? 2 : 1;
  const int threads = ((cols / cpt * L + 31) / 32) * 32;
  int chunk = 16;
  while (chunk > 2 && (size_t)2 * chunk * (R + threads * cpt) * sizeof(float) > 64 * 1024) chunk >>= 1;
  const size_t smem = (size_t)2 * chunk * (R + threads * cpt) * sizeof(float);       // records, and the lanes' shares of the outputs
  dim3 grid((unsigned)(n_seg * H), (unsigned)((dv + cols - 1) / cols));
  if (rpt == 8 && cpt == 2) return ret_launch<8, 2>(L, grid, threads, smem, s, rec, segs, decay, state, out, H, dk, dv, cols, chunk);
  if (rpt == 8) return ret_launch<8, 1>(L, grid, threads, smem, s, rec, segs, decay, state, out, H, dk, dv, cols, chunk);
  if (rpt == 16) return ret_launch<16, 1>(L, grid, threads, smem, s, rec, segs, decay, state, out, H, dk, dv, cols, chunk);
  if (rpt == 32) return ret_launch<32, 1>(L, grid, threads, smem, s, rec, segs, decay, state, out, H, dk, dv, cols, chunk);
  return ret_launch<64, 1>(L, grid, threads, smem, s, rec, segs, decay, state, out, H, dk, dv, cols, chunk);
}

// ------------------------------------------------------------------ matrix memory with exponential gates (mLSTM)
// Per head a matrix S [dk, dv], a vector n [dk] and a running maximum m (0 at a request's start).  With the log input
// gate i = cap tanh((il + bi) / cap) and the log forget gate f = logsigmoid(cap tanh((fl + bf) / cap)):
//     m_t = max(f + m_(t-1), i);  S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T;  n_t likewise with k alone
//     o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + den_eps)
// The maxima are a scalar recurrence per (request, head): one warp walks it and leaves, per token, the three
// exponentials.  n rides along as one more column of S whose value is always 1 (the state is [dk, dvp] with
// dvp = dv + 1 rounded up to 4; the columns past dv + 1 stay zero), so the delta rule's scan runs the matrix part
// with the record (d, a*u, u, k, r, v) = (keep, 0, 0, take k, q, [v | 1 | 0..]) and hands back S^T q and n . q together.
__device__ __forceinline__ float logsigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// A warp per (request, head) walks the maxima: 32 tokens at a time every lane turns its token's logits into the two
// log gates (the next 32 tokens' logits already on their way), then the chain m' = max(f + m, i) runs down the 32
// tokens in order, in every lane alike, and every lane writes its token's three exponentials.
__global__ void __launch_bounds__(128)
mlstm_gates_kernel(const float* __restrict__ il, const float* __restrict__ fl, long long ld, const float* __restrict__ i_bias,
                   const float* __restrict__ f_bias, const int* __restrict__ segs, float* __restrict__ m_state,
                   float* __restrict__ gates, int n_seg, int H, float cap) {
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (idx >= n_seg * H) return;
  const int seg = idx / H, h = idx % H;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const float bi = i_bias[h], bf = f_bias[h];
  float m = m_state[(size_t)slot * H + h];
  float xi = 0.f, xf = 0.f;
  if (lane < count) {
    xi = il[(size_t)(row0 + lane) * ld + h];
    xf = fl[(size_t)(row0 + lane) * ld + h];
  }
  for (int t0 = 0; t0 < count; t0 += 32) {
    const int tc = min(32, count - t0);
    float ni = 0.f, nf = 0.f;
    if (t0 + 32 + lane < count) {
      ni = il[(size_t)(row0 + t0 + 32 + lane) * ld + h];
      nf = fl[(size_t)(row0 + t0 + 32 + lane) * ld + h];
    }
    const float ig = cap * tanhf((xi + bi) / cap);
    const float fg = logsigmoid_f(cap * tanhf((xf + bf) / cap));
    float before = 0.f, after = 0.f;
#pragma unroll 8
    for (int j = 0; j < tc; ++j) {
      const float fj = __shfl_sync(0xffffffffu, fg, j), ij = __shfl_sync(0xffffffffu, ig, j);
      const float mn = fmaxf(fj + m, ij);
      if (lane == j) {
        before = m;
        after = mn;
      }
      m = mn;
    }
    if (lane < tc) {
      float* o = gates + ((size_t)(row0 + t0 + lane) * H + h) * 3;
      o[0] = expf(fg + before - after);
      o[1] = expf(ig - after);
      o[2] = expf(-after);
    }
    xi = ni;
    xf = nf;
  }
  if (lane == 0) m_state[(size_t)slot * H + h] = m;
}

__global__ void mlstm_prep_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                  long long ld, const float* __restrict__ gates, float* __restrict__ rec, long long items, int H,
                                  int dk, int dv, int dvp, int L, int RPT, float q_scale) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const size_t row = (size_t)(item / H);
  const int h = (int)(item % H);
  const float keep = gates[item * 3], take = gates[item * 3 + 1];
  const float* qp = q + row * ld + (size_t)h * dk;
  const float* kp = k + row * ld + (size_t)h * dk;
  const int P = L * RPT;
  float* out = rec + (size_t)item * (5 * P + dvp);
  for (int j = lane; j < P; j += 32) {
    const int i = (j % RPT) * L + j / RPT;
    const bool in = i < dk;
    out[j] = in ? keep : 0.f;
    out[P + j] = 0.f;
    out[2 * P + j] = 0.f;
    out[3 * P + j] = in ? take * kp[i] : 0.f;
    out[4 * P + j] = in ? qp[i] * q_scale : 0.f;
  }
  for (int c = lane; c < dvp; c += 32) out[5 * P + c] = c < dv ? v[row * ld + (size_t)h * dv + c] : (c == dv ? 1.0f : 0.f);
}

// The padded value size of the mLSTM's state and scan output.
HK_API int hk_mlstm_padded(int dv) { return (dv + 1 + 3) & ~3; }

// q, k [n, H*dk], v [n, H*dv], il, fl [n, H]: column slices of one float32 matrix (row stride ld).  state
// [slots, H, dk, dvp], m_state [slots, H], gates scratch [n, H, 3] (kept: the output's gate reads e^(-m)), out [n, H*dvp].
HK_API int hk_mlstm_scan(const float* q, const float* k, const float* v, const float* il, const float* fl, long long ld,
                         const float* i_bias, const float* f_bias, const int* segs, int n_seg, int n_rows, float* rec,
                         float* gates, float* state, float* m_state, float* out, int H, int dk, int dv, float cap, float q_scale,
                         void* stream) {
  if (n_seg <= 0 || n_rows <= 0) return 0;
  if (H < 1 || dk < 1 || dv < 1 || dk > 2048 || !(cap > 0.f) || ((uintptr_t)rec & 15)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const int dvp = hk_mlstm_padded(dv);
  int L, rpt;
  if (!dr_plan(n_seg, H, dk, dvp, &L, &rpt)) return HK_ERR_UNSUPPORTED;
  int e = hk_launch(mlstm_gates_kernel, dim3((unsigned)((n_seg * H + 3) / 4)), dim3(128), 0, s, il, fl, ld, i_bias, f_bias, segs,
                    m_state, gates, n_seg, H, cap);
  if (e) return e;
  const long long items = (long long)n_rows * H;
  e = hk_launch(mlstm_prep_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, s, q, k, v, ld, (const float*)gates, rec, items,
                H, dk, dv, dvp, L, rpt, q_scale);
  if (e) return e;
  return dr_scan_records(rec, segs, n_seg, state, out, H, dk, dvp, L, rpt, s);
}

// ------------------------------------------------------------------ the output of a head of a recurrent mixer
// One warp per (token, head): y = N(o / den) * weight * act(g), narrowed to T.  N divides by the root mean square over the
// head's dv values (eps inside the root).  o is read from rows of `ldo` floats per head (dv of them used).  `den`:
// with gates != null the head's values are first divided by max(|o[dv]|, gates[item, 2]) + den_eps (the mLSTM's
// normaliser: o[dv] is n . q, gates[.., 2] is e^(-m)).  The weight is [H, dv], or [dv] shared by the heads, or null (a
// norm without a weight); act is the logistic function or silu.
template <typename T>
__global__ void head_out_gate_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ g, long long ldg,
                                     const float* __restrict__ weight, int shared_weight, int act, const float* __restrict__ gates,
                                     float den_eps, T* __restrict__ out, long long items, int H, int dv, float eps) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const long long t = item / H;
  const int h = (int)(item % H);
  const float* src = o + (size_t)item * ldo;
  float scale = 1.0f;
  if (gates != nullptr) scale = 1.0f / (fmaxf(fabsf(src[dv]), gates[item * 3 + 2]) + den_eps);
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) {
    const float a = src[i] * scale;
    ss = fmaf(a, a, ss);
  }
  ss = warp_sum(ss);
  const float inv = scale / sqrtf(ss / (float)dv + eps);
  const float* wp = weight == nullptr ? nullptr : weight + (shared_weight ? 0 : (size_t)h * dv);
  for (int i = lane; i < dv; i += 32) {
    const float gl = g[(size_t)t * ldg + (size_t)h * dv + i];
    const float gate = act == 0 ? sigmoid_f(gl) : gl * sigmoid_f(gl);
    out[(size_t)item * dv + i] = from_f32<T>(src[i] * inv * (wp ? wp[i] : 1.0f) * gate);
  }
}

HK_API int hk_head_out_gate(const float* o, int ldo, const float* g, long long ldg, const float* weight, int shared_weight,
                            int act, const float* gates, float den_eps, void* out, int out_dtype, int n, int H, int dv, float eps,
                            void* stream) {
  if (n <= 0) return 0;
  if (ldo < dv || (gates != nullptr && ldo < dv + 1) || act < 0 || act > 1) return HK_ERR_UNSUPPORTED;
  const long long items = (long long)n * H;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == HK_F32)
    return hk_launch(head_out_gate_kernel<float>, dim3(blocks), dim3(256), 0, s, o, ldo, g, ldg, weight, shared_weight, act, gates,
                     den_eps, (float*)out, items, H, dv, eps);
  if (out_dtype == HK_BF16)
    return hk_launch(head_out_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, s, o, ldo, g, ldg, weight, shared_weight, act, gates,
                     den_eps, (bf16*)out, items, H, dv, eps);
  return HK_ERR_UNSUPPORTED;
}
