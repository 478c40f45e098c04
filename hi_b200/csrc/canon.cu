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

constexpr int kMaxTaps = 8;

// grid (tokens, channel groups); a thread per channel.
__global__ void canon_conv_kernel(const float* __restrict__ h, const float* __restrict__ taps_a,
                                  const float* __restrict__ taps_b, const float* __restrict__ state,
                                  long long state_stride, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                  void* __restrict__ out_a, void* __restrict__ out_b, int dtype, int width, int K) {
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const int start = cu_seqlens[s];
  const int local = t - start;
  const float* tail = state + (size_t)slots[s] * state_stride;      // [K-1, W]
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    float x[kMaxTaps];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
      if (j < K) {
        const int rel = local - (K - 1) + j;
        x[j] = rel >= 0 ? h[(size_t)(start + rel) * width + c] : tail[(size_t)(K - 1 + rel) * width + c];
      }
    }
    const float own = x[K - 1];
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
      if (j < K) {
        a = fmaf(taps_a[(size_t)c * K + j], x[j], a);
        if (taps_b) b = fmaf(taps_b[(size_t)c * K + j], x[j], b);
      }
    }
    st_any(out_a, dtype, (size_t)t * width + c, own + a);
    if (taps_b) st_any(out_b, dtype, (size_t)t * width + c, own + b);
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
  if (taps_n > kMaxTaps) return HB_ERR_UNSUPPORTED;
  if (n_tokens == 0) return HB_OK;
  int per = (width + 255) / 256;
  if (per > 32) per = 32;
  canon_conv_kernel<<<dim3(n_tokens, per), 256, 0, stream>>>(h, taps_a, taps_b, state, state_stride, cu_seqlens,
                                                            seq_of_token, slots, out_a, out_b, dtype, width, taps_n);
  HB_LAUNCH_CHECK();
  if (update_state && taps_n > 1 && n_seqs > 0) {
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
  const int threads = width >= 2048 ? 512 : 256;
  rmsnorm_mean2_kernel<<<rows, threads, 0, stream>>>(a, b, in_dtype, wa, wb, w_dtype, eps, out, out_dtype, width);
  HB_LAUNCH_CHECK();
  return HB_OK;
}
