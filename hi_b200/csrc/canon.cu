// Small steps of a block whose sub-layers read the norm's output through a short causal convolution
// over time, and of a model that runs a range of its layers several times.
//
//   canon_conv     y_a[t] = h[t] + sum_j taps_a[:, j] * h[t - (K-1) + j]   for up to two sets of taps at once
//                  (the mixer's and the feed-forward's); rows before a portion's first token come from the
//                  request's state ([K-1, W] float32: the last K-1 rows of h it has seen, zero at its start)
//   stream_add     x += d1 + d2 + e + v   (any of them absent): what is added to the stream between two
//                  passes over a range of layers (sub-layer results still open, the embedding output, a
//                  vector per pass)
//   rmsnorm_mean2  out = (a / rms(a) * w_a + b / rms(b) * w_b) / 2: two mixers side by side
//
// Sums and statistics are float32; h stays float32 between the norm and the convolution.
#include <stdint.h>

#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float ld_any(const void* p, int dtype, size_t i) {
  return dtype == HB_DTYPE_F32 ? reinterpret_cast<const float*>(p)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st_any(void* p, int dtype, size_t i, float v) {
  if (dtype == HB_DTYPE_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// grid (tokens, channel groups); a thread per channel.
__global__ void canon_conv_kernel(const float* __restrict__ h, const float* __restrict__ taps_a,
                                  const float* __restrict__ taps_b, float* state,
                                  long long state_stride, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                  void* __restrict__ out_a, void* __restrict__ out_b, int dtype, int width, int K,
                                  int fuse_tail) {
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const int start = cu_seqlens[s];
  const int local = t - start;
  const float* tail = state + (size_t)slots[s] * state_stride;      // [K-1, W]
  float* tail_w = state + (size_t)slots[s] * state_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    float own = 0.f, a = 0.f, b = 0.f;
    for (int j = 0; j < K; ++j) {
      const int rel = local - (K - 1) + j;
      const float x = rel >= 0 ? h[(size_t)(start + rel) * width + c] : tail[(size_t)(K - 1 + rel) * width + c];
      own = x;                                     // the last tap's row is the token's own
      // the request's only token of the step: its inputs move up a row in the state (row j - 1 is read no more)
      if (fuse_tail && j >= 1) tail_w[(size_t)(j - 1) * width + c] = x;
      a = fmaf(taps_a[(size_t)c * K + j], x, a);
      if (taps_b) b = fmaf(taps_b[(size_t)c * K + j], x, b);
    }
    st_any(out_a, dtype, (size_t)t * width + c, own + a);
    if (taps_b) st_any(out_b, dtype, (size_t)t * width + c, own + b);
  }
}

// The same with four channels a thread (width a multiple of 4) and kTokensPerThread consecutive rows of the step a
// thread: the taps of its four channels ([4][K] floats, contiguous) are read once into registers, a request's rows
// slide through a window of K float4 (one new 16-byte load a row; after a request's first row of the run, or
// where the next row belongs to another request, the window is filled anew, rows before the portion from the
// state), results leave as 8- or 16-byte stores. Steps of few rows take one row a thread.
template <int K, int kTokensPerThread>
__global__ void canon_conv_vec_kernel(const float* __restrict__ h, const float* __restrict__ taps_a,
                                      const float* __restrict__ taps_b, float* state,
                                      long long state_stride, const int* __restrict__ cu_seqlens,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                      void* __restrict__ out_a, void* __restrict__ out_b, int dtype, int width,
                                      int n_tokens, int fuse_tail) {
  const int t0 = blockIdx.x * kTokensPerThread;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= width) return;
  float wa[4 * K], wb[4 * K];
#pragma unroll
  for (int i = 0; i < K; ++i) {
    *reinterpret_cast<float4*>(wa + 4 * i) = *reinterpret_cast<const float4*>(taps_a + (size_t)c * K + 4 * i);
    *reinterpret_cast<float4*>(wb + 4 * i) = taps_b ? *reinterpret_cast<const float4*>(taps_b + (size_t)c * K + 4 * i)
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  auto emit = [&](const float* w, const float4 (&x)[K], void* out, int t) {
    float4 y = x[K - 1];
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      a0 = fmaf(w[j], x[j].x, a0);
      a1 = fmaf(w[K + j], x[j].y, a1);
      a2 = fmaf(w[2 * K + j], x[j].z, a2);
      a3 = fmaf(w[3 * K + j], x[j].w, a3);
    }
    y.x += a0; y.y += a1; y.z += a2; y.w += a3;
    if (dtype == HB_DTYPE_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)t * width + c) = y;
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
      uint2 pack = make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)t * width + c) = pack;
    }
  };
  float4 x[K];
  int prev_seq = -1;
#pragma unroll 1
  for (int i = 0; i < kTokensPerThread; ++i) {
    const int t = t0 + i;
    if (t >= n_tokens) break;
    const int s = seq_of_token[t];
    if (s == prev_seq) {                           // the next row of the same request: slide
#pragma unroll
      for (int j = 0; j + 1 < K; ++j) x[j] = x[j + 1];
      x[K - 1] = *reinterpret_cast<const float4*>(h + (size_t)t * width + c);
    } else {
      const int start = cu_seqlens[s];
      const int local = t - start;
      const float* tail = state + (size_t)slots[s] * state_stride;      // [K-1, W]
#pragma unroll
      for (int j = 0; j < K; ++j) {
        const int rel = local - (K - 1) + j;
        x[j] = *reinterpret_cast<const float4*>(rel >= 0 ? h + (size_t)(start + rel) * width + c
                                                         : tail + (size_t)(K - 1 + rel) * width + c);
      }
      prev_seq = s;
    }
    emit(wa, x, out_a, t);
    if (taps_b) emit(wb, x, out_b, t);
    if (kTokensPerThread == 1 && fuse_tail) {      // the request's only token of the step: this thread alone reads
      float* tw = state + (size_t)slots[s] * state_stride;   // and writes these channels of its state
#pragma unroll
      for (int j = 1; j < K; ++j) *reinterpret_cast<float4*>(tw + (size_t)(j - 1) * width + c) = x[j];
    }
  }
}

// The last K-1 rows of h of every request after this step's rows replace its state's.
__global__ void canon_tail_kernel(const float* __restrict__ h, float* __restrict__ state, long long state_stride,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int width, int K) {
  const int s = blockIdx.x;
  const int start = cu_seqlens[s], n = cu_seqlens[s + 1] - start;
  if (n <= 0) return;
  float* tail = state + (size_t)slots[s] * state_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    // new row i is input n - (K-1) + i of the portion; a negative one is row n + i of the old state, which lies
    // behind every row written so far
    for (int i = 0; i < K - 1; ++i) {
      const int rel = n - (K - 1) + i;
      tail[(size_t)i * width + c] = rel >= 0 ? h[(size_t)(start + rel) * width + c] : tail[(size_t)(n + i) * width + c];
    }
  }
}

__global__ void stream_add_kernel(float* __restrict__ x, const void* __restrict__ d1, int d1_dtype,
                                  const void* __restrict__ d2, int d2_dtype, const float* __restrict__ e,
                                  const float* __restrict__ vec, long long total, int width) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float s = x[i];
    if (d1) s += ld_any(d1, d1_dtype, (size_t)i);
    if (d2) s += ld_any(d2, d2_dtype, (size_t)i);
    if (e) s += e[i];
    if (vec) s += vec[i % width];
    x[i] = s;
  }
}

// A block per row.
__global__ void rmsnorm_mean2_kernel(const void* __restrict__ a, const void* __restrict__ b, int in_dtype,
                                     const void* __restrict__ wa, const void* __restrict__ wb, int w_dtype, float eps,
                                     void* __restrict__ out, int out_dtype, int width) {
  __shared__ float scratch[33];
  const size_t row = blockIdx.x;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float va = ld_any(a, in_dtype, row * width + c), vb = ld_any(b, in_dtype, row * width + c);
    sa += va * va;
    sb += vb * vb;
  }
  const float ia = rsqrtf(hb::block_sum(sa, scratch) / (float)width + eps);
  const float ib = rsqrtf(hb::block_sum(sb, scratch) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float va = ld_any(a, in_dtype, row * width + c) * ia * ld_any(wa, w_dtype, c);
    const float vb = ld_any(b, in_dtype, row * width + c) * ib * ld_any(wb, w_dtype, c);
    st_any(out, out_dtype, row * width + c, 0.5f * (va + vb));
  }
}

// four neighbouring elements as floats / from floats (16-byte loads of float32, 8-byte ones of bfloat16)
__device__ __forceinline__ float4 ld4_any(const void* p, int dtype, size_t i) {
  if (dtype == HB_DTYPE_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void st4_any(void* p, int dtype, size_t i, float4 v) {
  if (dtype == HB_DTYPE_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) =
        make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
  }
}

// The same, four channels a thread, a row's numbers kept in registers between the two passes (width a multiple of
// 4, at most 4 * kGroups * blockDim.x; pointers on 16-byte boundaries).
template <int kGroups>
__global__ void rmsnorm_mean2_vec_kernel(const void* __restrict__ a, const void* __restrict__ b, int in_dtype,
                                         const void* __restrict__ wa, const void* __restrict__ wb, int w_dtype, float eps,
                                         void* __restrict__ out, int out_dtype, int width) {
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * width;
  float4 va[kGroups], vb[kGroups];
  float sa = 0.f, sb = 0.f;
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    const int c = (g * blockDim.x + threadIdx.x) * 4;
    va[g] = vb[g] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < width) {
      va[g] = ld4_any(a, in_dtype, base + c);
      vb[g] = ld4_any(b, in_dtype, base + c);
    }
    sa += va[g].x * va[g].x + va[g].y * va[g].y + va[g].z * va[g].z + va[g].w * va[g].w;
    sb += vb[g].x * vb[g].x + vb[g].y * vb[g].y + vb[g].z * vb[g].z + vb[g].w * vb[g].w;
  }
  const float ia = 0.5f * rsqrtf(hb::block_sum(sa, scratch) / (float)width + eps);
  const float ib = 0.5f * rsqrtf(hb::block_sum(sb, scratch) / (float)width + eps);
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    const int c = (g * blockDim.x + threadIdx.x) * 4;
    if (c < width) {
      const float4 ga = ld4_any(wa, w_dtype, c), gb = ld4_any(wb, w_dtype, c);
      st4_any(out, out_dtype, base + c,
              make_float4(va[g].x * ia * ga.x + vb[g].x * ib * gb.x, va[g].y * ia * ga.y + vb[g].y * ib * gb.y,
                          va[g].z * ia * ga.z + vb[g].z * ib * gb.z, va[g].w * ia * ga.w + vb[g].w * ib * gb.w));
    }
  }
}

bool dt_ok(int d) { return d == HB_DTYPE_F32 || d == HB_DTYPE_BF16; }

}  // namespace

extern "C" int hb_canon_conv(const float* h, const float* taps_a, const float* taps_b, float* state,
                             long long state_stride, const int* cu_seqlens, const int* seq_of_token, const int* slots,
                             void* out_a, void* out_b, int dtype, int n_tokens, int n_seqs, int width, int taps_n,
                             int update_state, cudaStream_t stream) {
  if (!h || !taps_a || !state || !cu_seqlens || !seq_of_token || !slots || !out_a || (taps_b && !out_b) || !dt_ok(dtype))
    return HB_ERR_BAD_ARG;
  if (width <= 0 || taps_n < 1 || n_tokens < 0 || n_seqs < 0 || state_stride < (long long)(taps_n - 1) * width)
    return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  int per = (width + 255) / 256;
  if (per > 32) per = 32;
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  int fuse = update_state == 2;     // every request brings exactly one token: the kernel moves the state itself
  const bool vec = width % 4 == 0 && state_stride % 4 == 0 && taps_n <= 4 && (width / 4 + 127) / 128 <= 65535 &&
                   aligned16(h) && aligned16(state) && aligned16(taps_a) && aligned16(taps_b) && aligned16(out_a) &&
                   aligned16(out_b);
  if (vec) {
    const int per_thread = n_tokens >= 1024 ? 8 : 1;
    fuse = update_state == 2 && per_thread == 1;
    const dim3 grid((n_tokens + per_thread - 1) / per_thread, (width / 4 + 127) / 128);
#define HB_CANON_VEC(K)                                                                                          \
    do {                                                                                                         \
      if (per_thread == 8)                                                                                       \
        canon_conv_vec_kernel<K, 8><<<grid, 128, 0, stream>>>(h, taps_a, taps_b, state, state_stride, cu_seqlens, \
                                                              seq_of_token, slots, out_a, out_b, dtype, width, n_tokens, fuse); \
      else                                                                                                       \
        canon_conv_vec_kernel<K, 1><<<grid, 128, 0, stream>>>(h, taps_a, taps_b, state, state_stride, cu_seqlens, \
                                                              seq_of_token, slots, out_a, out_b, dtype, width, n_tokens, fuse); \
    } while (0)
    if (taps_n == 1) HB_CANON_VEC(1);
    else if (taps_n == 2) HB_CANON_VEC(2);
    else if (taps_n == 3) HB_CANON_VEC(3);
    else HB_CANON_VEC(4);
#undef HB_CANON_VEC
  } else {
    canon_conv_kernel<<<dim3(n_tokens, per), 256, 0, stream>>>(h, taps_a, taps_b, state, state_stride, cu_seqlens,
                                                              seq_of_token, slots, out_a, out_b, dtype, width, taps_n, fuse);
  }
  HB_LAUNCH_CHECK();
  if (update_state && !fuse && taps_n > 1 && n_seqs > 0) {
    canon_tail_kernel<<<dim3(n_seqs, per), 256, 0, stream>>>(h, state, state_stride, cu_seqlens, slots, width, taps_n);
    HB_LAUNCH_CHECK();
  }
  return HB_OK;
}

extern "C" int hb_stream_add(float* x, const void* d1, int d1_dtype, const void* d2, int d2_dtype, const float* e,
                             const float* vec, long long rows, int width, cudaStream_t stream) {
  if (!x || rows < 0 || width <= 0 || (d1 && !dt_ok(d1_dtype)) || (d2 && !dt_ok(d2_dtype))) return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  const long long total = rows * width;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  stream_add_kernel<<<(int)blocks, 256, 0, stream>>>(x, d1, d1_dtype, d2, d2_dtype, e, vec, total, width);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_rmsnorm_mean2(const void* a, const void* b, int in_dtype, const void* wa, const void* wb, int w_dtype,
                                float eps, void* out, int out_dtype, int rows, int width, cudaStream_t stream) {
  if (!a || !b || !wa || !wb || !out || rows < 0 || width <= 0 || !dt_ok(in_dtype) || !dt_ok(w_dtype) || !dt_ok(out_dtype))
    return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (width % 4 == 0 && width <= 4 * 4 * 256 && aligned16(a) && aligned16(b) && aligned16(wa) && aligned16(wb) && aligned16(out)) {
    // whole warps, about two groups of four channels a thread
    int threads = ((width / 8 + 31) / 32) * 32;
    threads = threads < 32 ? 32 : (threads > 256 ? 256 : threads);
    if (width <= 4 * 2 * threads)
      rmsnorm_mean2_vec_kernel<2><<<rows, threads, 0, stream>>>(a, b, in_dtype, wa, wb, w_dtype, eps, out, out_dtype, width);
    else
      rmsnorm_mean2_vec_kernel<4><<<rows, threads, 0, stream>>>(a, b, in_dtype, wa, wb, w_dtype, eps, out, out_dtype, width);
  } else {
    const int threads = width >= 2048 ? 512 : 256;
    rmsnorm_mean2_kernel<<<rows, threads, 0, stream>>>(a, b, in_dtype, wa, wb, w_dtype, eps, out, out_dtype, width);
  }
  HB_LAUNCH_CHECK();
  return HB_OK;
}
