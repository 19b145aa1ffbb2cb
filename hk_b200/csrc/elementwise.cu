// Row-wise kernels of the decoder: embedding gather, RMS norm, the fused per-head
// norm + rotation + paged cache write, and SwiGLU.  Each is templated on the storage
// type (float for the true 32-bit path, bf16 for serving); all arithmetic is fp32.
//
// Reference counterparts (one launch each there, none fused): `rms_norm`
// src/cuda_device.zig:1393-1403, `head_norm` :1406-1415, `rope` :1420-1441,
// `kv_write` :1453-1477, `swiglu` :1824-1829; host-side embedding
// src/cuda/engine.zig:724-737.  The fusion of norm + rotation + cache write follows
// the idea of shaders/rope_kv.comp:2-7.
#include "common.cuh"

// ----------------------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] widened to fp32 (the residual stream is fp32) and multiplied by `scale` (1 for
// none).  `narrow` (or null) receives the same row rounded to bf16: the input of a first sublayer that reads the
// residual stream itself.
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int n, int d, int vocab, float scale, bf16* __restrict__ narrow) {
  int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;  // the host validates ids; this only keeps the read in bounds
  const T* src = table + (size_t)id * d;
  float* dst = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = to_f32<T>(src[i]) * scale;
    dst[i] = v;
    if (narrow) narrow[(size_t)t * d + i] = __float2bfloat16_rn(v);
  }
}

// The same with 16-byte loads (8 bf16 or 4 floats per thread and step), all issued before any is used.
template <typename T, int PER>
__global__ void embedding_vec_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                     int d, int vocab, float scale, bf16* __restrict__ narrow) {
  constexpr int E = 16 / sizeof(T);   // elements per 16-byte load
  pdl_launch_dependents();
  pdl_wait();
  int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * d);
  float* dst = out + (size_t)t * d;
  const int chunks = d / E;
  uint4 v[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) v[k] = src[c];
  }
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    int c = threadIdx.x + k * blockDim.x;
    if (c >= chunks) continue;
    const T* e = reinterpret_cast<const T*>(&v[k]);
    float f[E];
#pragma unroll
    for (int i = 0; i < E; ++i) f[i] = to_f32<T>(e[i]) * scale;
#pragma unroll
    for (int i = 0; i < E; i += 4) *reinterpret_cast<float4*>(dst + c * E + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
    if (narrow) {
#pragma unroll
      for (int i = 0; i < E; i += 2)
        *reinterpret_cast<__nv_bfloat162*>(narrow + (size_t)t * d + c * E + i) = __floats2bfloat162_rn(f[i], f[i + 1]);
    }
  }
}

HK_API int hk_embedding(const void* table, int table_dtype, const int* ids, float* out, int n, int d,
                        int vocab, float scale, void* narrow_out, void* stream) {
  bf16* narrow = (bf16*)narrow_out;
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  {
    const int e = table_dtype == HK_F32 ? 4 : 8;
    if (d % e == 0 && ((uintptr_t)table & 15) == 0 && ((uintptr_t)out & 15) == 0 && d / e <= 4 * 256) {
      if (table_dtype == HK_F32)
        return hk_launch(embedding_vec_kernel<float, 4>, dim3(n), dim3(256), 0, s, (const float*)table, ids, out, d, vocab, scale, narrow);
      else if (table_dtype == HK_BF16)
        return hk_launch(embedding_vec_kernel<bf16, 4>, dim3(n), dim3(256), 0, s, (const bf16*)table, ids, out, d, vocab, scale, narrow);
      else
        return HK_ERR_UNSUPPORTED;
      return hk_launch_status();
    }
  }
  int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == HK_F32)
    embedding_kernel<float><<<n, threads, 0, s>>>((const float*)table, ids, out, n, d, vocab, scale, narrow);
  else if (table_dtype == HK_BF16)
    embedding_kernel<bf16><<<n, threads, 0, s>>>((const bf16*)table, ids, out, n, d, vocab, scale, narrow);
  else
    return HK_ERR_UNSUPPORTED;
  return hk_launch_status();
}

// ----------------------------------------------------------------------------- rms norm
// out[r, :] = x[row(r), :] * rsqrt(mean(x^2) + eps) * w, with row(r) = rows ? rows[r] : r.
// The sum of squares runs in a fixed order (thread-strided partials, warp tree, then
// warps in order), so a row's result does not depend on what else is in the batch.
template <typename TO>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                const int* __restrict__ rows, TO* __restrict__ out, int d, float eps) {
  __shared__ float warp_part[32];
  __shared__ float inv_s;
  int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = src[i];
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) warp_part[wid] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < nw; ++i) tot += warp_part[i];
    inv_s = 1.0f / sqrtf(tot / (float)d + eps);
  }
  __syncthreads();
  float inv = inv_s;
  TO* dst = out + (size_t)r * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f32<TO>(src[i] * inv * w[i]);
}

// The same for widths that are a multiple of 4 and at most 4 * PER * 256: the row is read once with 16-byte
// loads that are all in flight together, and stays in registers between the two passes.  The order of the
// sum depends on the width alone.
template <typename TO, int PER>
__global__ void __launch_bounds__(256)
rms_norm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, const int* __restrict__ rows,
                    TO* __restrict__ out, int d, float eps) {
  __shared__ float warp_part[8];
  __shared__ float inv_s;
  const int r = blockIdx.x;
  const float4* wv = reinterpret_cast<const float4*>(w);
  const int chunks = d >> 2;
  float4 v[PER], g[PER];
  pdl_launch_dependents();
#pragma unroll
  for (int k = 0; k < PER; ++k) {     // the norm's weight does not depend on the kernel before
    const int c = threadIdx.x + k * 256;
    if (c < chunks) g[k] = wv[c];
  }
  pdl_wait();
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * 256;
    v[k] = c < chunks ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    ss = fmaf(v[k].x, v[k].x, ss);
    ss = fmaf(v[k].y, v[k].y, ss);
    ss = fmaf(v[k].z, v[k].z, ss);
    ss = fmaf(v[k].w, v[k].w, ss);
  }
  ss = warp_sum(ss);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) warp_part[wid] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += warp_part[i];
    inv_s = 1.0f / sqrtf(tot / (float)d + eps);
  }
  __syncthreads();
  const float inv = inv_s;
  TO* dst = out + (size_t)r * d;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * 256;
    if (c >= chunks) continue;
    const float a0 = v[k].x * inv * g[k].x, a1 = v[k].y * inv * g[k].y, a2 = v[k].z * inv * g[k].z, a3 = v[k].w * inv * g[k].w;
    if (sizeof(TO) == 4) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + 4 * c) = make_float4(a0, a1, a2, a3);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a0, a1), hi = __floats2bfloat162_rn(a2, a3);
      *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(dst) + 4 * c) =
          make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

template <int PER>
static int rms_norm_vec(const float* x, const float* w, const int* rows, void* out, int out_dtype, int n_out, int d, float eps,
                        cudaStream_t s) {
  if (out_dtype == HK_F32)
    return hk_launch_pdl(rms_norm_vec_kernel<float, PER>, dim3(n_out), dim3(256), 0, s, x, w, rows, (float*)out, d, eps);
  if (out_dtype == HK_BF16)
    return hk_launch_pdl(rms_norm_vec_kernel<bf16, PER>, dim3(n_out), dim3(256), 0, s, x, w, rows, (bf16*)out, d, eps);
  return HK_ERR_UNSUPPORTED;
}

HK_API int hk_rms_norm(const float* x, const float* w, const int* rows, void* out, int out_dtype,
                       int n_out, int d, float eps, void* stream) {
  if (n_out <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if ((d & 3) == 0 && d >= 1024 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0) {
    const int chunks = d >> 2;
    if (chunks <= 2 * 256) return rms_norm_vec<2>(x, w, rows, out, out_dtype, n_out, d, eps, s);
    if (chunks <= 4 * 256) return rms_norm_vec<4>(x, w, rows, out, out_dtype, n_out, d, eps, s);
    if (chunks <= 8 * 256) return rms_norm_vec<8>(x, w, rows, out, out_dtype, n_out, d, eps, s);
  }
  int threads = d >= 2048 ? 256 : 128;
  if (out_dtype == HK_F32)
    rms_norm_kernel<float><<<n_out, threads, 0, s>>>(x, w, rows, (float*)out, d, eps);
  else if (out_dtype == HK_BF16)
    rms_norm_kernel<bf16><<<n_out, threads, 0, s>>>(x, w, rows, (bf16*)out, d, eps);
  else
    return HK_ERR_UNSUPPORTED;
  return hk_launch_status();
}

// ------------------------------------------------- per-head norm + rotation + cache write
// One warp per (token, head) of the fused projection output qkv[n, (H + G) * hd + G * vd] (fp32; the value heads may
// have a width vd of their own):
//   q heads: optional RMS norm over hd (weight shared by the heads), rotate-half rotation of
//            the first `rot` dims by the token's position, stored to q_out[n, H*hd];
//   k heads: the same with the key norm weight, stored into the token's cache page;
//   v heads: stored into the cache page unchanged.
// `bias` (or null) [(H + 2G) * hd] is added to the projection output first.  `pairing` 0 rotates dims
// (i, i + rot/2) ("rotate-half"), 1 rotates dims (2i, 2i + 1) ("adjacent"); both read angle i of the tables.
// Page of a token: block_table[slot_of_token[t]][pos / page_tokens]; the cache layout is
// [page][G][page_tokens][hd] for keys and [page][G][page_tokens][vd] for values.  With write_kv == 0 only q is
// produced (a layer that reads another layer's cache).
// `norm_after` = 1 moves the per-head norm behind the rotation, where a null weight means a weight of ones
// (x over its root mean square).  `tied_v` = 1: the projection has no v heads (a row holds H + G heads) and a
// token's value is its key as projected, before rotation and norm, of which the first `vd` dims are kept.
#define QKR_MAX_HD 256
#define QKR_WARPS 4

template <typename T>
__global__ void qk_norm_rope_kv_write_kernel(
    const float* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_w,
    const float* __restrict__ k_w, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, int rot, const int* __restrict__ positions,
    const int* __restrict__ slot_of_token, const int* __restrict__ block_table, int table_stride,
    T* __restrict__ k_pages, T* __restrict__ v_pages, int n, int H, int G, int hd, int page_tokens,
    int write_kv, const float* __restrict__ bias, int pairing, int norm_after, int tied_v, int vd, long long ld) {
  __shared__ float buf[QKR_WARPS][QKR_MAX_HD];
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int kv_heads = tied_v ? G : 2 * G;
  int heads_total = H + (write_kv ? kv_heads : 0);
  long long item = (long long)blockIdx.x * QKR_WARPS + wid;
  if (item >= (long long)n * heads_total) return;
  int t = (int)(item / heads_total);
  int hh = (int)(item % heads_total);
  int kind = hh < H ? 0 : (hh < H + G ? 1 : 2);  // q, k, v
  // a row holds H + G heads of hd, then (unless the values are the keys) G value heads of vd
  const size_t row = (size_t)ld;   // at least (H + G) * hd + (tied_v ? 0 : G * vd): further columns are not read
  const size_t col = kind == 2 ? (size_t)(H + G) * hd + (size_t)(hh - H - G) * vd : (size_t)hh * hd;
  const int width_in = kind == 2 ? vd : hd;
  const float* src = qkv + (size_t)t * row + col;
  float* v = buf[wid];
  float ss = 0.f;
  for (int i = lane; i < width_in; i += 32) {
    float a = src[i];
    if (bias) a += bias[col + i];
    v[i] = a;
    ss = fmaf(a, a, ss);
  }
  __syncwarp();
  int pos = positions[t];
  int page = -1;
  if (kind != 0) {
    page = block_table[(size_t)slot_of_token[t] * table_stride + pos / page_tokens];
    if (page < 0) return;  // the host never schedules this; keeps a stale table from writing out of bounds
    if (kind == 1 && tied_v) {   // the value is the key as projected
      T* vdst = v_pages + (((size_t)page * G + (hh - H)) * page_tokens + (pos % page_tokens)) * vd;
      for (int i = lane; i < vd; i += 32) vdst[i] = from_f32<T>(v[i]);
    }
  }
  if (kind != 2) {
    const float* w = kind == 0 ? q_w : k_w;
    if (w && !norm_after) {
      ss = warp_sum(ss);
      float inv = 1.0f / sqrtf(ss / (float)hd + eps);
      for (int i = lane; i < hd; i += 32) v[i] = v[i] * inv * w[i];
      __syncwarp();
    }
    if (rot > 0) {
      int half = rot >> 1;
      const float* c = cos_t + (size_t)pos * half;
      const float* s = sin_t + (size_t)pos * half;
      for (int i = lane; i < half; i += 32) {
        const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
        float a = v[ia], b = v[ib];
        float ci = c[i], si = s[i];
        v[ia] = a * ci - b * si;
        v[ib] = a * si + b * ci;
      }
      __syncwarp();
    }
    if (norm_after) {
      float s2 = 0.f;
      for (int i = lane; i < hd; i += 32) s2 = fmaf(v[i], v[i], s2);
      s2 = warp_sum(s2);
      const float inv = 1.0f / sqrtf(s2 / (float)hd + eps);
      for (int i = lane; i < hd; i += 32) v[i] = v[i] * inv * (w ? w[i] : 1.0f);
      __syncwarp();
    }
  }
  T* dst;
  int width = hd;
  if (kind == 0) {
    dst = q_out + (size_t)t * H * hd + (size_t)hh * hd;
  } else if (kind == 1) {
    dst = k_pages + (((size_t)page * G + (hh - H)) * page_tokens + (pos % page_tokens)) * hd;
  } else {
    width = vd;
    dst = v_pages + (((size_t)page * G + (hh - H - G)) * page_tokens + (pos % page_tokens)) * vd;
  }
  for (int i = lane; i < width; i += 32) dst[i] = from_f32<T>(v[i]);
}

// The same for head sizes up to 128 that are a multiple of 4 (and a rotary width that is a multiple of 8):
// a lane holds 4 consecutive dims, read with one 16-byte load; the rotation partner (dim + rot/2) sits
// (rot/8) lanes away and comes by shuffle, so nothing goes through shared memory.
#define QKV_WARPS 8
template <typename T>
__global__ void __launch_bounds__(QKV_WARPS * 32)
qk_norm_rope_kv_write_vec_kernel(
    const float* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_w,
    const float* __restrict__ k_w, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, int rot, const int* __restrict__ positions,
    const int* __restrict__ slot_of_token, const int* __restrict__ block_table, int table_stride,
    T* __restrict__ k_pages, T* __restrict__ v_pages, int n, int H, int G, int hd, int page_tokens,
    int write_kv, const float* __restrict__ bias, int pairing, int norm_after, int tied_v, int vd, long long ld) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int kv_heads = tied_v ? G : 2 * G;
  const int heads_total = H + (write_kv ? kv_heads : 0);
  const long long item = (long long)blockIdx.x * QKV_WARPS + wid;
  if (item >= (long long)n * heads_total) return;
  const int t = (int)(item / heads_total);
  const int hh = (int)(item % heads_total);
  const int d0 = lane * 4;
  const int kind = hh < H ? 0 : (hh < H + G ? 1 : 2);
  const size_t row = (size_t)ld;   // at least (H + G) * hd + (tied_v ? 0 : G * vd): further columns are not read
  const size_t col = kind == 2 ? (size_t)(H + G) * hd + (size_t)(hh - H - G) * vd : (size_t)hh * hd;
  const bool active = d0 < (kind == 2 ? vd : hd);
  const float* src = qkv + (size_t)t * row + col;
  float4 v = active ? *reinterpret_cast<const float4*>(src + d0) : make_float4(0.f, 0.f, 0.f, 0.f);
  if (bias && active) {
    const float4 b = *reinterpret_cast<const float4*>(bias + col + d0);
    v = make_float4(v.x + b.x, v.y + b.y, v.z + b.z, v.w + b.w);
  }
  const int pos = positions[t];
  int page = 0;
  if (kind != 0) page = block_table[(size_t)slot_of_token[t] * table_stride + pos / page_tokens];
  if (kind == 1 && tied_v && page >= 0 && d0 < vd) {      // the value is the key as projected
    T* vdst = v_pages + (((size_t)page * G + (hh - H)) * page_tokens + (pos % page_tokens)) * vd;
    if (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(vdst) + d0) = v;
    } else {
      __nv_bfloat162 lo2 = __floats2bfloat162_rn(v.x, v.y), hi2 = __floats2bfloat162_rn(v.z, v.w);
      *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(vdst) + d0) =
          make_uint2(*reinterpret_cast<uint32_t*>(&lo2), *reinterpret_cast<uint32_t*>(&hi2));
    }
  }
  if (kind != 2) {
    const float* w = kind == 0 ? q_w : k_w;
    if (w && !norm_after) {
      float ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
      if (active) {
        const float4 g = *reinterpret_cast<const float4*>(w + d0);
        v = make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
      }
    }
    if (rot > 0 && pairing) {
      // adjacent pairs: a lane's four dims are the pairs d0/2 and d0/2 + 1, both its own
      if (d0 < rot) {
        const int half = rot >> 1;
        const float2 c = *reinterpret_cast<const float2*>(cos_t + (size_t)pos * half + (d0 >> 1));
        const float2 sn = *reinterpret_cast<const float2*>(sin_t + (size_t)pos * half + (d0 >> 1));
        v = make_float4(v.x * c.x - v.y * sn.x, v.x * sn.x + v.y * c.x, v.z * c.y - v.w * sn.y, v.z * sn.y + v.w * c.y);
      }
    } else if (rot > 0) {
      const int half = rot >> 1, shift = half >> 2;        // partner lanes are `shift` apart
      const bool low = d0 < half, in_rot = d0 < rot;
      const int partner = low ? lane + shift : lane - shift;
      const int src_lane = in_rot ? partner : lane;
      float4 p;
      p.x = __shfl_sync(0xffffffffu, v.x, src_lane);
      p.y = __shfl_sync(0xffffffffu, v.y, src_lane);
      p.z = __shfl_sync(0xffffffffu, v.z, src_lane);
      p.w = __shfl_sync(0xffffffffu, v.w, src_lane);
      if (in_rot) {
        const int i0 = low ? d0 : d0 - half;                // index into the tables
        const float4 c = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + i0);
        const float4 sn = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + i0);
        // low half: x' = a c - b s (a = own, b = partner); high half: x' = a s + b c (a = partner, b = own)
        if (low)
          v = make_float4(v.x * c.x - p.x * sn.x, v.y * c.y - p.y * sn.y, v.z * c.z - p.z * sn.z, v.w * c.w - p.w * sn.w);
        else
          v = make_float4(p.x * sn.x + v.x * c.x, p.y * sn.y + v.y * c.y, p.z * sn.z + v.z * c.z, p.w * sn.w + v.w * c.w);
      }
    }
    if (norm_after) {
      float ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
      if (active) {
        const float4 g = w ? *reinterpret_cast<const float4*>(w + d0) : make_float4(1.f, 1.f, 1.f, 1.f);
        v = make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
      }
    }
  }
  if (!active || page < 0) return;
  T* dst;
  if (kind == 0) {
    dst = q_out + (size_t)t * H * hd + (size_t)hh * hd;
  } else if (kind == 1) {
    dst = k_pages + (((size_t)page * G + (hh - H)) * page_tokens + (pos % page_tokens)) * hd;
  } else {
    dst = v_pages + (((size_t)page * G + (hh - H - G)) * page_tokens + (pos % page_tokens)) * vd;
  }
  if (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + d0) = v;
  } else {
    __nv_bfloat162 lo2 = __floats2bfloat162_rn(v.x, v.y), hi2 = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(dst) + d0) =
        make_uint2(*reinterpret_cast<uint32_t*>(&lo2), *reinterpret_cast<uint32_t*>(&hi2));
  }
}

HK_API int hk_qk_norm_rope_kv_write(const float* qkv, void* q_out, int dtype, const float* q_w,
                                    const float* k_w, float eps, const float* cos_t, const float* sin_t,
                                    int rot, const int* positions, const int* slot_of_token,
                                    const int* block_table, int table_stride, void* k_pages,
                                    void* v_pages, int n, int H, int G, int hd, int page_tokens,
                                    int write_kv, const float* bias, int pairing, int norm_after, int tied_v, int vd,
                                    long long ld, void* stream) {
  if (ld <= 0) ld = (long long)(H + G) * hd + (tied_v ? 0 : (long long)G * vd);
  if (n <= 0) return 0;
  if (hd > QKR_MAX_HD || hd < 2 || rot > hd || (rot & 1) || pairing < 0 || pairing > 1) return HK_ERR_UNSUPPORTED;
  if (vd < 1 || vd > QKR_MAX_HD || (tied_v && vd > hd)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  long long items = (long long)n * (H + (write_kv ? (tied_v ? G : 2 * G) : 0));
  const bool aligned = ((((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)q_w |
                          (uintptr_t)k_w | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)bias) & 15) == 0);
  if (hd <= 128 && vd <= 128 && (hd & 3) == 0 && (vd & 3) == 0 && (rot & 7) == 0 && (ld & 3) == 0 && aligned) {
    unsigned vblocks = (unsigned)((items + QKV_WARPS - 1) / QKV_WARPS);
    if (dtype == HK_F32)
      return hk_launch_pdl(qk_norm_rope_kv_write_vec_kernel<float>, dim3(vblocks), dim3(QKV_WARPS * 32), 0, s, qkv, (float*)q_out,
                       q_w, k_w, eps, cos_t, sin_t, rot, positions, slot_of_token, block_table, table_stride, (float*)k_pages,
                       (float*)v_pages, n, H, G, hd, page_tokens, write_kv, bias, pairing, norm_after, tied_v, vd, ld);
    if (dtype == HK_BF16)
      return hk_launch_pdl(qk_norm_rope_kv_write_vec_kernel<bf16>, dim3(vblocks), dim3(QKV_WARPS * 32), 0, s, qkv, (bf16*)q_out, q_w,
                       k_w, eps, cos_t, sin_t, rot, positions, slot_of_token, block_table, table_stride, (bf16*)k_pages,
                       (bf16*)v_pages, n, H, G, hd, page_tokens, write_kv, bias, pairing, norm_after, tied_v, vd, ld);
    return HK_ERR_UNSUPPORTED;
  }
  unsigned blocks = (unsigned)((items + QKR_WARPS - 1) / QKR_WARPS);
  if (dtype == HK_F32)
    return hk_launch(qk_norm_rope_kv_write_kernel<float>, dim3(blocks), dim3(QKR_WARPS * 32), 0, s, qkv, (float*)q_out, q_w,
                         k_w, eps, cos_t, sin_t, rot, positions, slot_of_token, block_table, table_stride, (float*)k_pages,
                         (float*)v_pages, n, H, G, hd, page_tokens, write_kv, bias, pairing, norm_after, tied_v, vd, ld);
  if (dtype == HK_BF16)
    return hk_launch(qk_norm_rope_kv_write_kernel<bf16>, dim3(blocks), dim3(QKR_WARPS * 32), 0, s, qkv, (bf16*)q_out, q_w,
                         k_w, eps, cos_t, sin_t, rot, positions, slot_of_token, block_table, table_stride, (bf16*)k_pages,
                         (bf16*)v_pages, n, H, G, hd, page_tokens, write_kv, bias, pairing, norm_after, tied_v, vd, ld);
  return HK_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------- bias
// out[t, j] += bias[j] for a projection with a bias whose product kernel has no such epilogue.
__global__ void add_bias_kernel(float* __restrict__ out, const float* __restrict__ bias, long long total, int N) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] += bias[i % N];
}

HK_API int hk_add_bias(float* out, const float* bias, int n, int N, void* stream) {
  if (n <= 0 || N <= 0) return 0;
  long long total = (long long)n * N;
  return hk_launch(add_bias_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, out, bias, total, N);
}

// ----------------------------------------------------------------------------- swiglu
// out[t, j] = silu(gate_j) * up_j for the fused projection gu[n, 2F], laid out in blocks of
// `block` gates followed by the matching `block` ups (block == F: all gates, then all ups).
// `act` chooses the gate's activation: 0 = silu (SwiGLU), 1 = the tanh form of gelu (GeGLU), 2 = the clamped form
// min(g, p0) * sigmoid(p1 * min(g, p0)) * (clamp(u, -p0, p0) + 1) with the limit p0 and the sigmoid's slope p1.
__device__ __forceinline__ float glu_pair(float g, float u, int act, float p0, float p1) {
  if (act == 0) return g / (1.0f + expf(-g)) * u;
  if (act == 1) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  g = fminf(g, p0);
  u = fminf(fmaxf(u, -p0), p0);
  return g / (1.0f + expf(-p1 * g)) * (u + 1.0f);
}

template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gu, TO* __restrict__ out, long long total, int F, int block, int act,
                              float p0, float p1) {
  pdl_launch_dependents();
  pdl_wait();
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  long long t = i / F;
  int j = (int)(i % F);
  long long gi = t * 2 * F + (long long)(j / block) * 2 * block + (j % block);
  float g = gu[gi];
  float u = gu[gi + block];
  out[i] = from_f32<TO>(glu_pair(g, u, act, p0, p1));
}

HK_API int hk_swiglu(const float* gu, void* out, int out_dtype, int n, int F, int block, int act, float p0, float p1, void* stream) {
  if (n <= 0) return 0;
  if (block <= 0 || F % block || act < 0 || act > 2) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  long long total = (long long)n * F;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dtype == HK_F32) return hk_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, s, gu, (float*)out, total, F, block, act, p0, p1);
  if (out_dtype == HK_BF16) return hk_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, s, gu, (bf16*)out, total, F, block, act, p0, p1);
  return HK_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------- norm of a sublayer's output, added
// residual[r, :] += y[r, :] * rsqrt(mean(y^2) + eps) * w: the norm AFTER a mixer or feed-forward of a layer that
// norms both sides of its sublayers, fused with the residual sum (which stays fp32).  Same summation order as
// `rms_norm_kernel`.  `narrow` (or null) receives the new residual row rounded to bf16: the input of a next sublayer
// that reads the residual stream itself (a layer that norms only behind its sublayers).
__global__ void rms_norm_add_kernel(const float* __restrict__ y, const float* __restrict__ w, float* __restrict__ residual,
                                    int d, float eps, bf16* __restrict__ narrow) {
  __shared__ float warp_part[32];
  __shared__ float inv_s;
  const int r = blockIdx.x;
  const float* src = y + (size_t)r * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = src[i];
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) warp_part[wid] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < nw; ++i) tot += warp_part[i];
    inv_s = 1.0f / sqrtf(tot / (float)d + eps);
  }
  __syncthreads();
  const float inv = inv_s;
  float* dst = residual + (size_t)r * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = dst[i] + src[i] * inv * w[i];
    dst[i] = v;
    if (narrow) narrow[(size_t)r * d + i] = __float2bfloat16_rn(v);
  }
}

// The same for widths that are a multiple of 4 and at most 4 * PER * 256: the row is read once with 16-byte loads that
// are all in flight together and stays in registers between the two passes (as `rms_norm_vec_kernel`).
template <int PER>
__global__ void __launch_bounds__(256)
rms_norm_add_vec_kernel(const float* __restrict__ y, const float* __restrict__ w, float* __restrict__ residual, int d, float eps,
                        bf16* __restrict__ narrow) {
  __shared__ float warp_part[8];
  __shared__ float inv_s;
  const int r = blockIdx.x;
  const int chunks = d >> 2;
  const float4* src = reinterpret_cast<const float4*>(y + (size_t)r * d);
  const float4* wv = reinterpret_cast<const float4*>(w);
  float4* dst = reinterpret_cast<float4*>(residual + (size_t)r * d);
  float4 v[PER], g[PER], x[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * 256;
    const bool in = c < chunks;
    v[k] = in ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    g[k] = in ? wv[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    x[k] = in ? dst[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    ss = fmaf(v[k].x, v[k].x, ss);
    ss = fmaf(v[k].y, v[k].y, ss);
    ss = fmaf(v[k].z, v[k].z, ss);
    ss = fmaf(v[k].w, v[k].w, ss);
  }
  ss = warp_sum(ss);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) warp_part[wid] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += warp_part[i];
    inv_s = 1.0f / sqrtf(tot / (float)d + eps);
  }
  __syncthreads();
  const float inv = inv_s;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * 256;
    if (c < chunks) {
      const float4 o = make_float4(x[k].x + v[k].x * inv * g[k].x, x[k].y + v[k].y * inv * g[k].y, x[k].z + v[k].z * inv * g[k].z,
                                   x[k].w + v[k].w * inv * g[k].w);
      dst[c] = o;
      if (narrow) {
        __nv_bfloat162 lo2 = __floats2bfloat162_rn(o.x, o.y), hi2 = __floats2bfloat162_rn(o.z, o.w);
        *reinterpret_cast<uint2*>(narrow + (size_t)r * d + 4 * c) =
            make_uint2(*reinterpret_cast<uint32_t*>(&lo2), *reinterpret_cast<uint32_t*>(&hi2));
      }
    }
  }
}

HK_API int hk_rms_norm_add(const float* y, const float* w, float* residual, int n, int d, float eps, void* narrow_out,
                           void* stream) {
  if (n <= 0) return 0;
  bf16* narrow = (bf16*)narrow_out;
  if ((d & 3) == 0 && d >= 512 && (((uintptr_t)y | (uintptr_t)w | (uintptr_t)residual) & 15) == 0 && ((uintptr_t)narrow & 7) == 0) {
    const int chunks = d >> 2;
    cudaStream_t s = (cudaStream_t)stream;
    if (chunks <= 256) return hk_launch(rms_norm_add_vec_kernel<1>, dim3((unsigned)n), dim3(256), 0, s, y, w, residual, d, eps, narrow);
    if (chunks <= 2 * 256) return hk_launch(rms_norm_add_vec_kernel<2>, dim3((unsigned)n), dim3(256), 0, s, y, w, residual, d, eps, narrow);
    if (chunks <= 4 * 256) return hk_launch(rms_norm_add_vec_kernel<4>, dim3((unsigned)n), dim3(256), 0, s, y, w, residual, d, eps, narrow);
    if (chunks <= 8 * 256) return hk_launch(rms_norm_add_vec_kernel<8>, dim3((unsigned)n), dim3(256), 0, s, y, w, residual, d, eps, narrow);
  }
  return hk_launch(rms_norm_add_kernel, dim3((unsigned)n), dim3(d >= 2048 ? 256 : 128), 0, (cudaStream_t)stream, y, w, residual, d,
                   eps, narrow);
}

// ----------------------------------------------------------------------------- polynomial activation with norms
// out[r, :] = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 over a row z of F values, powers element by element and
// N(v) = v / sqrt(mean(v^2) + eps): three sums of the row (z^2, z^4, z^6) in fp32, then one pass.  `coef` holds the
// four numbers on the device.
template <typename TO>
__global__ void polynorm_kernel(const float* __restrict__ z, const float* __restrict__ coef, TO* __restrict__ out, int F,
                                float eps) {
  __shared__ float part[3][32];
  __shared__ float inv_s[3];
  const int r = blockIdx.x;
  const float* src = z + (size_t)r * F;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = src[i], v2 = v * v, v3 = v2 * v;
    s1 = fmaf(v, v, s1);
    s2 = fmaf(v2, v2, s2);
    s3 = fmaf(v3, v3, s3);
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  s3 = warp_sum(s3);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) {
    part[0][wid] = s1;
    part[1][wid] = s2;
    part[2][wid] = s3;
  }
  __syncthreads();
  if (threadIdx.x < 3) {
    float tot = 0.f;
    for (int i = 0; i < nw; ++i) tot += part[threadIdx.x][i];
    inv_s[threadIdx.x] = 1.0f / sqrtf(tot / (float)F + eps);
  }
  __syncthreads();
  const float a = coef[0] * inv_s[0], b = coef[1] * inv_s[1], c = coef[2] * inv_s[2], e = coef[3];
  TO* dst = out + (size_t)r * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = src[i], v2 = v * v;
    dst[i] = from_f32<TO>(a * v + b * v2 + c * (v2 * v) + e);
  }
}

// The same for F a multiple of 4 and at most 4 * PER * 256, the row in registers between the two passes.
template <typename TO, int PER>
__global__ void __launch_bounds__(256)
polynorm_vec_kernel(const float* __restrict__ z, const float* __restrict__ coef, TO* __restrict__ out, int F, float eps) {
  __shared__ float part[3][8];
  __shared__ float inv_s[3];
  const int r = blockIdx.x;
  const int chunks = F >> 2;
  const float4* src = reinterpret_cast<const float4*>(z + (size_t)r * F);
  float4 v[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * 256;
    v[k] = c < chunks ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const float e[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = e[i], a2 = a * a, a3 = a2 * a;
      s1 = fmaf(a, a, s1);
      s2 = fmaf(a2, a2, s2);
      s3 = fmaf(a3, a3, s3);
    }
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  s3 = warp_sum(s3);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) {
    part[0][wid] = s1;
    part[1][wid] = s2;
    part[2][wid] = s3;
  }
  __syncthreads();
  if (threadIdx.x < 3) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += part[threadIdx.x][i];
    inv_s[threadIdx.x] = 1.0f / sqrtf(tot / (float)F + eps);
  }
  __syncthreads();
  const float a = coef[0] * inv_s[0], b = coef[1] * inv_s[1], c3 = coef[2] * inv_s[2], e0 = coef[3];
  TO* dst = out + (size_t)r * F;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * 256;
    if (c >= chunks) continue;
    const float in[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x = in[i], x2 = x * x;
      o[i] = a * x + b * x2 + c3 * (x2 * x) + e0;
    }
    if (sizeof(TO) == 4) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + 4 * c) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
      *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(dst) + 4 * c) =
          make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

template <typename TO>
static int polynorm_vec(const float* z, const float* coef, TO* out, int n, int F, float eps, cudaStream_t s) {
  const int chunks = F >> 2;
  if (chunks <= 2 * 256) return hk_launch(polynorm_vec_kernel<TO, 2>, dim3((unsigned)n), dim3(256), 0, s, z, coef, out, F, eps);
  if (chunks <= 4 * 256) return hk_launch(polynorm_vec_kernel<TO, 4>, dim3((unsigned)n), dim3(256), 0, s, z, coef, out, F, eps);
  if (chunks <= 8 * 256) return hk_launch(polynorm_vec_kernel<TO, 8>, dim3((unsigned)n), dim3(256), 0, s, z, coef, out, F, eps);
  return hk_launch(polynorm_vec_kernel<TO, 16>, dim3((unsigned)n), dim3(256), 0, s, z, coef, out, F, eps);
}

HK_API int hk_polynorm(const float* z, const float* coef, void* out, int out_dtype, int n, int F, float eps, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if ((F & 3) == 0 && F >= 512 && F <= 4 * 16 * 256 && (((uintptr_t)z | (uintptr_t)out) & 15) == 0) {
    if (out_dtype == HK_F32) return polynorm_vec<float>(z, coef, (float*)out, n, F, eps, s);
    if (out_dtype == HK_BF16) return polynorm_vec<bf16>(z, coef, (bf16*)out, n, F, eps, s);
    return HK_ERR_UNSUPPORTED;
  }
  const int threads = F >= 2048 ? 256 : 128;
  if (out_dtype == HK_F32) return hk_launch(polynorm_kernel<float>, dim3((unsigned)n), dim3(threads), 0, s, z, coef, (float*)out, F, eps);
  if (out_dtype == HK_BF16) return hk_launch(polynorm_kernel<bf16>, dim3((unsigned)n), dim3(threads), 0, s, z, coef, (bf16*)out, F, eps);
  return HK_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------- tanh of some columns
// out[t, j] = tanh(x[t * ld + j]) for j < R, narrowed to TO: the hidden layer of a low-rank projection that sits in
// a slice of a fused projection's output.
template <typename TO>
__global__ void tanh_cols_kernel(const float* __restrict__ x, long long ld, TO* __restrict__ out, long long total, int R) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / R;
  const int j = (int)(i % R);
  out[i] = from_f32<TO>(tanhf(x[t * ld + j]));
}

HK_API int hk_tanh_cols(const float* x, long long ld, void* out, int out_dtype, int n, int R, void* stream) {
  if (n <= 0 || R <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const long long total = (long long)n * R;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dtype == HK_F32) return hk_launch(tanh_cols_kernel<float>, dim3(blocks), dim3(256), 0, s, x, ld, (float*)out, total, R);
  if (out_dtype == HK_BF16) return hk_launch(tanh_cols_kernel<bf16>, dim3(blocks), dim3(256), 0, s, x, ld, (bf16*)out, total, R);
  return HK_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------- output gate of a mixer
// out[t, j] = x[t, j] * scale * sigmoid(gate[t, j]) for x [n, W] (fp32, or the storage type) and the gate's logits as a column
// slice of a fused projection's fp32 output (row stride ld).
template <typename TI, typename TO>
__global__ void sigmoid_gate_kernel(const TI* __restrict__ x, const float* __restrict__ gate, long long ld, TO* __restrict__ out,
                                    long long total, int W, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / W;
  const int j = (int)(i % W);
  const float g = gate[t * ld + j];
  out[i] = from_f32<TO>(to_f32<TI>(x[i]) * scale / (1.0f + expf(-g)));
}

HK_API int hk_sigmoid_gate(const void* x, int x_dtype, const float* gate, long long ld, void* out, int out_dtype, int n, int W,
                           float scale, void* stream) {
  if (n <= 0 || W <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const long long total = (long long)n * W;
  const dim3 grid((unsigned)((total + 255) / 256)), block(256);
  if (x_dtype == HK_F32 && out_dtype == HK_F32)
    return hk_launch(sigmoid_gate_kernel<float, float>, grid, block, 0, s, (const float*)x, gate, ld, (float*)out, total, W, scale);
  if (x_dtype == HK_F32 && out_dtype == HK_BF16)
    return hk_launch(sigmoid_gate_kernel<float, bf16>, grid, block, 0, s, (const float*)x, gate, ld, (bf16*)out, total, W, scale);
  if (x_dtype == HK_BF16 && out_dtype == HK_BF16)
    return hk_launch(sigmoid_gate_kernel<bf16, bf16>, grid, block, 0, s, (const bf16*)x, gate, ld, (bf16*)out, total, W, scale);
  return HK_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------- latent attention: what a token brings
// A mixer that caches one compressed vector per token instead of keys and values.  One warp per (token, item) of the fused
// projection's fp32 output row [H query heads of (dn + dr) | r + dr compressed | ...] (row stride ld):
//   query head h: its first dn dims go unchanged to q_plain[t, h, :dn] (they are multiplied with the keys' up-projection
//                 afterwards); its last dr dims are rotated by the token's position into q_full[t, h, r : r + dr];
//   the compressed row: its first r dims are RMS-normed with `c_w` (the latent), its last dr dims are rotated (the one
//                 rotated key part that all heads share); both go to the token's cache row [page][1][page_tokens][r + dr].
// The rotation turns the first `rot` of the dr dims, pairing 0: (i, i + rot/2), 1: (2i, 2i + 1); the tables carry any
// magnitude factor.  With write_kv == 0 only the queries are produced.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const float* __restrict__ proj, long long ld, T* __restrict__ q_plain, T* __restrict__ q_full,
                   const float* __restrict__ c_w, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                   int rot, int pairing, const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                   const int* __restrict__ block_table, int table_stride, T* __restrict__ pages, int n, int H, int dn, int dr,
                   int r, int page_tokens, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int items = H + (write_kv ? 1 : 0);
  const long long item = (long long)blockIdx.x * 4 + wid;
  if (item >= (long long)n * items) return;
  const int t = (int)(item / items), it = (int)(item % items);
  const int pos = positions[t];
  const float* row = proj + (size_t)t * ld;
  const int half = rot >> 1;
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;
  const float* src;   // the dr dims to rotate
  T* dst;             // where they go
  if (it < H) {
    const float* qh = row + (size_t)it * (dn + dr);
    T* qp = q_plain + ((size_t)t * H + it) * dn;
    for (int i = lane; i < dn; i += 32) qp[i] = from_f32<T>(qh[i]);
    src = qh + dn;
    dst = q_full + ((size_t)t * H + it) * (r + dr) + r;
  } else {
    const int page = block_table[(size_t)slot_of_token[t] * table_stride + pos / page_tokens];
    if (page < 0) return;   // the host never schedules this; keeps a stale table from writing out of bounds
    const float* cp = row + (size_t)H * (dn + dr);
    T* out = pages + ((size_t)page * page_tokens + (pos % page_tokens)) * (r + dr);
    float ss = 0.f;
    for (int i = lane; i < r; i += 32) ss = fmaf(cp[i], cp[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)r + eps);
    for (int i = lane; i < r; i += 32) out[i] = from_f32<T>(cp[i] * inv * c_w[i]);
    src = cp + r;
    dst = out + r;
  }
  for (int i = lane; i < half; i += 32) {
    const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
    const float a = src[ia], b = src[ib];
    dst[ia] = from_f32<T>(a * c[i] - b * s[i]);
    dst[ib] = from_f32<T>(a * s[i] + b * c[i]);
  }
  for (int i = rot + lane; i < dr; i += 32) dst[i] = from_f32<T>(src[i]);
}

HK_API int hk_latent_prep(const float* proj, long long ld, void* q_plain, void* q_full, int dtype, const float* c_w, float eps,
                          const float* cos_t, const float* sin_t, int rot, int pairing, const int* positions,
                          const int* slot_of_token, const int* block_table, int table_stride, void* pages, int n, int H, int dn,
                          int dr, int r, int page_tokens, int write_kv, void* stream) {
  if (n <= 0) return 0;
  if (rot < 0 || rot > dr || (rot & 1) || pairing < 0 || pairing > 1 || H < 1 || dn < 1 || dr < 0 || r < 1) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const long long items = (long long)n * (H + (write_kv ? 1 : 0));
  const dim3 grid((unsigned)((items + 3) / 4)), block(128);
  if (dtype == HK_F32)
    return hk_launch_pdl(latent_prep_kernel<float>, grid, block, 0, s, proj, ld, (float*)q_plain, (float*)q_full, c_w, eps, cos_t,
                         sin_t, rot, pairing, positions, slot_of_token, block_table, table_stride, (float*)pages, n, H, dn, dr, r,
                         page_tokens, write_kv);
  if (dtype == HK_BF16)
    return hk_launch_pdl(latent_prep_kernel<bf16>, grid, block, 0, s, proj, ld, (bf16*)q_plain, (bf16*)q_full, c_w, eps, cos_t,
                         sin_t, rot, pairing, positions, slot_of_token, block_table, table_stride, (bf16*)pages, n, H, dn, dr, r,
                         page_tokens, write_kv);
  return HK_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------- sums of float32 streams
// out = (accumulate ? out : 0) + alpha * a + beta * b, element by element (b may be null): the sum of two mixers that
// read the same input, each with a factor of its own; a stream that is added to the residual again.
__global__ void scaled_sum_kernel(float* __restrict__ out, const float* __restrict__ a, float alpha, const float* __restrict__ b,
                                  float beta, long long total4, long long total, int accumulate) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total4) {
    const float4 x = reinterpret_cast<const float4*>(a)[i];
    float4 r = accumulate ? reinterpret_cast<float4*>(out)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    r.x = fmaf(alpha, x.x, r.x); r.y = fmaf(alpha, x.y, r.y); r.z = fmaf(alpha, x.z, r.z); r.w = fmaf(alpha, x.w, r.w);
    if (b != nullptr) {
      const float4 y = reinterpret_cast<const float4*>(b)[i];
      r.x = fmaf(beta, y.x, r.x); r.y = fmaf(beta, y.y, r.y); r.z = fmaf(beta, y.z, r.z); r.w = fmaf(beta, y.w, r.w);
    }
    reinterpret_cast<float4*>(out)[i] = r;
  }
  if (i < total - 4 * total4) {                  // the last one to three elements
    const long long j = 4 * total4 + i;
    float r = accumulate ? out[j] : 0.f;
    r = fmaf(alpha, a[j], r);
    if (b != nullptr) r = fmaf(beta, b[j], r);
    out[j] = r;
  }
}

HK_API int hk_scaled_sum(float* out, const float* a, float alpha, const float* b, float beta, long long total, int accumulate,
                         void* stream) {
  if (total <= 0) return 0;
  const bool vec = !(((uintptr_t)out | (uintptr_t)a | (uintptr_t)b) & 15);
  const long long total4 = vec ? total / 4 : 0;
  const long long threads = total4 > total - 4 * total4 ? total4 : total - 4 * total4;
  return hk_launch(scaled_sum_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, out, a, alpha, b,
                   beta, total4, total, accumulate);
}

// ----------------------------------------------------------------------------- a float32 stream rounded to the storage type
template <typename T>
__global__ void narrow_kernel(const float* __restrict__ x, T* __restrict__ out, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = from_f32<T>(x[i]);
}

HK_API int hk_narrow(const float* x, void* out, int out_dtype, long long total, void* stream) {
  if (total <= 0) return 0;
  const dim3 grid((unsigned)((total + 255) / 256));
  if (out_dtype == HK_BF16) return hk_launch(narrow_kernel<bf16>, grid, dim3(256), 0, (cudaStream_t)stream, x, (bf16*)out, total);
  if (out_dtype == HK_F32) return hk_launch(narrow_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, x, (float*)out, total);
  return HK_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------- a gate times a token's own vector
// out[t, j] = act(z[t, j]) * table[ids[t], col0 + j] for j < W: z is a float32 column slice (row stride ld) of a
// projection's output, the table [vocab, table_cols] holds one vector per token id of which a layer reads W columns
// from col0 on.  act 0: gelu in its tanh form, 1: silu.
template <typename TT, typename TO>
__global__ void token_gate_kernel(const float* __restrict__ z, long long ld, const TT* __restrict__ table, long long table_cols,
                                  int col0, const int* __restrict__ ids, TO* __restrict__ out, long long total, int W, int act) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / W;
  const int j = (int)(i % W);
  const float g = z[t * ld + j];
  const float a = act == 0 ? 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) : g / (1.0f + expf(-g));
  out[i] = from_f32<TO>(a * to_f32<TT>(table[(size_t)ids[t] * table_cols + col0 + j]));
}

HK_API int hk_token_gate(const float* z, long long ld, const void* table, int table_dtype, long long table_cols, int col0,
                         const int* ids, void* out, int out_dtype, int n, int W, int act, void* stream) {
  if (n <= 0 || W <= 0) return 0;
  if (act < 0 || act > 1 || col0 < 0 || col0 + W > table_cols) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const long long total = (long long)n * W;
  const dim3 grid((unsigned)((total + 255) / 256)), block(256);
  if (table_dtype == HK_F32 && out_dtype == HK_F32)
    return hk_launch(token_gate_kernel<float, float>, grid, block, 0, s, z, ld, (const float*)table, table_cols, col0, ids, (float*)out,
                     total, W, act);
  if (table_dtype == HK_BF16 && out_dtype == HK_BF16)
    return hk_launch(token_gate_kernel<bf16, bf16>, grid, block, 0, s, z, ld, (const bf16*)table, table_cols, col0, ids, (bf16*)out, total,
                     W, act);
  if (table_dtype == HK_F32 && out_dtype == HK_BF16)
    return hk_launch(token_gate_kernel<float, bf16>, grid, block, 0, s, z, ld, (const float*)table, table_cols, col0, ids, (bf16*)out,
                     total, W, act);
  return HK_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------- attention with several score maps per head
// An attention whose heads carry M score maps over the same values (M = 2: a differential attention) runs on the
// ordinary paged attention kernels as H * M query heads over G key/value heads: a key/value head's cache row is the
// M maps' keys side by side [M * dk], and query head (h, j) is map j's query at its place in a row of M * dk numbers
// that is zero elsewhere, so its score with the row is q_j . k_j and every map of a head reads the same value.
// This kernel turns the projected (and convolved) float32 row x = [H * M * dk q | G * M * dk k | G * vd v] of every
// token into that layout: q and k are turned by position on the first `rot` dims of every map (dim i paired with
// i + rot / 2), the queries are written to q_out [n, H * M, M * dk], keys and values to the token's place in its pages
// [page, G, page_tokens, M * dk] and [page, G, page_tokens, vd].  One warp per (token, unit); a unit is a query map,
// a key map or a value head.
template <typename T>
__global__ void __launch_bounds__(128)
maps_rope_kv_write_kernel(const float* __restrict__ x, long long ld, T* __restrict__ q_out, const float* __restrict__ cos_t,
                          const float* __restrict__ sin_t, int rot, const int* __restrict__ positions,
                          const int* __restrict__ slot_of_token, const int* __restrict__ block_table, int table_stride,
                          T* __restrict__ k_pages, T* __restrict__ v_pages, int n, int H, int G, int M, int dk, int vd,
                          int page_tokens, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int qu = H * M, ku = G * M;
  const int units = qu + (write_kv ? ku + G : 0);
  const long long item = (long long)blockIdx.x * 4 + wid;
  if (item >= (long long)n * units) return;
  const int t = (int)(item / units), u = (int)(item % units);
  const int pos = positions[t];
  const float* row = x + (size_t)t * ld;
  const int half = rot >> 1;
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;
  size_t cache_at = 0;
  if (u >= qu) {
    const int page = block_table[(size_t)slot_of_token[t] * table_stride + pos / page_tokens];
    if (page < 0) return;   // the host never schedules this; keeps a stale table from writing out of bounds
    const int g = u < qu + ku ? (u - qu) / M : u - qu - ku;
    cache_at = ((size_t)page * G + g) * page_tokens + (pos % page_tokens);
  }
  if (u >= qu + ku) {       // a value head: copied
    const float* src = row + (size_t)(qu + ku) * dk + (size_t)(u - qu - ku) * vd;
    T* dst = v_pages + cache_at * vd;
    for (int i = lane; i < vd; i += 32) dst[i] = from_f32<T>(src[i]);
    return;
  }
  const float* src = row + (size_t)u * dk;       // q maps and k maps follow one another in x
  const int j = u % M;
  T* dst = u < qu ? q_out + ((size_t)t * qu + u) * M * dk : k_pages + cache_at * M * dk;
  if (u < qu)               // a query row is zero outside its own map
    for (int i = lane; i < M * dk; i += 32)
      if (i / dk != j) dst[i] = from_f32<T>(0.f);
  dst += (size_t)j * dk;
  for (int i = lane; i < dk; i += 32) {
    float v;
    if (i < half) v = src[i] * c[i] - src[i + half] * s[i];
    else if (i < rot) v = src[i] * c[i - half] + src[i - half] * s[i - half];
    else v = src[i];
    dst[i] = from_f32<T>(v);
  }
}

HK_API int hk_maps_rope_kv_write(const float* x, long long ld, void* q_out, int dtype, const float* cos_t, const float* sin_t, int rot,
                                 const int* positions, const int* slot_of_token, const int* block_table, int table_stride,
                                 void* k_pages, void* v_pages, int n, int H, int G, int M, int dk, int vd, int page_tokens,
                                 int write_kv, void* stream) {
  if (n <= 0) return 0;
  if (rot < 0 || rot > dk || (rot & 1) || H < 1 || G < 1 || M < 1 || dk < 1 || vd < 1) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const long long items = (long long)n * (H * M + (write_kv ? G * M + G : 0));
  const dim3 grid((unsigned)((items + 3) / 4)), block(128);
  if (dtype == HK_F32)
    return hk_launch_pdl(maps_rope_kv_write_kernel<float>, grid, block, 0, s, x, ld, (float*)q_out, cos_t, sin_t, rot, positions,
                         slot_of_token, block_table, table_stride, (float*)k_pages, (float*)v_pages, n, H, G, M, dk, vd, page_tokens,
                         write_kv);
  if (dtype == HK_BF16)
    return hk_launch_pdl(maps_rope_kv_write_kernel<bf16>, grid, block, 0, s, x, ld, (bf16*)q_out, cos_t, sin_t, rot, positions,
                         slot_of_token, block_table, table_stride, (bf16*)k_pages, (bf16*)v_pages, n, H, G, M, dk, vd, page_tokens,
                         write_kv);
  return HK_ERR_UNSUPPORTED;
}

// The heads' outputs of a differential attention: with a1 = a[t, 2h] and a2 = a[t, 2h + 1] the two maps' weighted values,
//     o = a1 - lambda * a2;   out[t, h] = o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate[t, h])
// (gate: float32 logits, one per head, row stride ldg; null: no gate).  One warp per (token, head), float32 arithmetic.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
diff_heads_out_kernel(const TI* __restrict__ a, const float* __restrict__ gate, long long ldg, TO* __restrict__ out, long long items,
                      int H, int vd, float lambda, float eps, float out_scale) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const long long t = item / H;
  const int h = (int)(item % H);
  const TI* a1 = a + (size_t)item * 2 * vd;
  const TI* a2 = a1 + vd;
  float ss = 0.f;
  for (int i = lane; i < vd; i += 32) {
    const float o = fmaf(-lambda, to_f32<TI>(a2[i]), to_f32<TI>(a1[i]));
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  float f = out_scale / sqrtf(ss / (float)vd + eps);
  if (gate != nullptr) f /= 1.0f + expf(-gate[(size_t)t * ldg + h]);
  for (int i = lane; i < vd; i += 32)
    out[(size_t)item * vd + i] = from_f32<TO>(fmaf(-lambda, to_f32<TI>(a2[i]), to_f32<TI>(a1[i])) * f);
}

HK_API int hk_diff_heads_out(const void* a, int a_dtype, const float* gate, long long ldg, void* out, int out_dtype, int n, int H,
                             int vd, float lambda, float eps, float out_scale, void* stream) {
  if (n <= 0) return 0;
  if (H < 1 || vd < 1) return HK_ERR_UNSUPPORTED;
  const long long items = (long long)n * H;
  const dim3 grid((unsigned)((items + 7) / 8)), block(256);
  cudaStream_t s = (cudaStream_t)stream;
  if (a_dtype == HK_F32 && out_dtype == HK_F32)
    return hk_launch(diff_heads_out_kernel<float, float>, grid, block, 0, s, (const float*)a, gate, ldg, (float*)out, items, H, vd,
                     lambda, eps, out_scale);
  if (a_dtype == HK_BF16 && out_dtype == HK_BF16)
    return hk_launch(diff_heads_out_kernel<bf16, bf16>, grid, block, 0, s, (const bf16*)a, gate, ldg, (bf16*)out, items, H, vd,
                     lambda, eps, out_scale);
  if (a_dtype == HK_F32 && out_dtype == HK_BF16)
    return hk_launch(diff_heads_out_kernel<float, bf16>, grid, block, 0, s, (const float*)a, gate, ldg, (bf16*)out, items, H, vd,
                     lambda, eps, out_scale);
  return HK_ERR_UNSUPPORTED;
}
