// Hyper-connections: the residual stream kept as S copies per token, float32 [N, S, W].
//
// A sub-layer reads one weighted sum of the copies and its result goes back into every copy, while the
// copies are mixed among themselves:
//     u      = sum_s in[s] x_s                       the sub-layer's input (before its norm)
//     x_t'   = sum_s mix[s, t] x_s + mult * out[t] * y     all copies at once, from the old ones
// One launch of `hyper_step_kernel` sits at every sub-layer boundary and does, for one token per block,
//   (1) y = delta + delta2 + sum_r routed[slot_of_entry[t, r]] * routed_weight[t, r]    (what the sub-layer before left)
//   (2) the update of the copies with that sub-layer's mix / out (skipped when mix is null),
//   (3) u of the NEXT sub-layer with its `in` (null: all ones, the plain sum of the copies),
//   (4) the RMS norm of u: u * rsqrt(mean(u^2) + eps) * w, rounded to the consumer's dtype (and, on request, unrounded).
// So the copies are read and written once per sub-layer. Everything is float32 but the rounded output.
// `broadcast`: the copies do not exist yet; all S of them equal the row of x_in [N, W] (the embedding output).
// `row_map`: only the listed rows are worked on, and nothing is written back (the last norm before the head).
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

struct HyperArgs {
  float* streams;             // [N, S, W]
  const float* x_in;          // [N, W] with broadcast, else null
  const void* delta;  int delta_dtype;
  const void* delta2; int delta2_dtype;
  const float* routed;        // [N * top_k, W] rows in expert order
  const int* slot_of_entry;   // [N * top_k]
  const float* routed_weight; // [N * top_k] or null
  int top_k;
  const float* mix;           // [S, S] indexed [from, to], or null: the copies stay as they are
  const float* out_coef;      // [S]
  float mult;
  const float* in_coef;       // [S] or null (ones)
  const void* w; int w_dtype; // the norm's weight as applied (float32 where the model stores it around zero)
  float eps;
  void* y; int y_dtype;       // [rows, W]
  float* y_f32;               // [rows, W] or null
  const int* row_map;         // [rows] or null
  int S, W;
};

constexpr int kMaxStreams = 16;

template <int MAXS>
__global__ void hyper_step_kernel(const HyperArgs a) {
  __shared__ float scratch[33];
  __shared__ float mix_s[MAXS * MAXS], out_s[MAXS], in_s[MAXS];
  extern __shared__ float u_row[];   // [W]
  const int S = a.S, W = a.W;
  const int r = blockIdx.x;
  const size_t src = a.row_map ? (size_t)a.row_map[r] : (size_t)r;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix_s[i] = a.mix ? a.mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    out_s[i] = a.mix ? a.out_coef[i] * a.mult : 0.f;
    in_s[i] = a.in_coef ? a.in_coef[i] : 1.f;
  }
  __syncthreads();
  const bool has_y = a.delta || a.delta2 || a.routed;
  const bool write = !a.row_map && (a.mix != nullptr || a.x_in != nullptr);
  float ss = 0.f;
  for (int j = threadIdx.x; j < W; j += blockDim.x) {
    float xs[MAXS];
    if (a.x_in) {
      const float v = a.x_in[src * W + j];
#pragma unroll
      for (int s = 0; s < MAXS; ++s) xs[s] = v;
    } else {
#pragma unroll
      for (int s = 0; s < MAXS; ++s) xs[s] = s < S ? a.streams[(src * S + s) * W + j] : 0.f;
    }
    float y = 0.f;
    if (has_y) {
      if (a.delta) y += ld_any(a.delta, a.delta_dtype, src * W + j);
      if (a.delta2) y += ld_any(a.delta2, a.delta2_dtype, src * W + j);
      if (a.routed)
        for (int q = 0; q < a.top_k; ++q)
          y += a.routed[(size_t)a.slot_of_entry[src * a.top_k + q] * W + j] *
               (a.routed_weight ? a.routed_weight[src * a.top_k + q] : 1.f);
    }
    float u = 0.f;
    if (a.mix) {
#pragma unroll
      for (int t = 0; t < MAXS; ++t) {
        if (t < S) {
          float nx = 0.f;
#pragma unroll
          for (int s = 0; s < MAXS; ++s)
            if (s < S) nx += mix_s[s * S + t] * xs[s];
          nx += out_s[t] * y;
          if (write) a.streams[(src * S + t) * W + j] = nx;
          u += in_s[t] * nx;
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < MAXS; ++t) {
        if (t < S) {
          if (write) a.streams[(src * S + t) * W + j] = xs[t];
          u += in_s[t] * xs[t];
        }
      }
    }
    u_row[j] = u;
    ss += u * u;
  }
  const float inv = rsqrtf(hb::block_sum(ss, scratch) / (float)W + a.eps);
  if (!a.y) return;
  for (int j = threadIdx.x; j < W; j += blockDim.x) {
    const float o = u_row[j] * inv * (a.w ? ld_any(a.w, a.w_dtype, j) : 1.f);
    st_any(a.y, a.y_dtype, (size_t)r * W + j, o);
    if (a.y_f32) a.y_f32[(size_t)r * W + j] = o;
  }
}

__device__ __forceinline__ float4 ld4_any(const void* p, int dtype, size_t i) {   // i % 4 == 0
  if (dtype == HB_DTYPE_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}
__device__ __forceinline__ void st4_any(void* p, int dtype, size_t i, float4 v) {
  if (dtype == HB_DTYPE_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = raw;
  }
}
__device__ __forceinline__ void axpy4(float4& acc, float c, const float4& v) {
  acc.x += c * v.x; acc.y += c * v.y; acc.z += c * v.z; acc.w += c * v.w;
}

// The same for widths that are a multiple of four: a thread takes four neighbouring columns of all copies with 16-byte
// loads, and the loads of its first columns are in flight before the block waits for the coefficients.
template <int MAXS>
__global__ void __launch_bounds__(512) hyper_step_vec_kernel(const HyperArgs a) {
  __shared__ float scratch[33];
  __shared__ float mix_s[MAXS * MAXS], out_s[MAXS], in_s[MAXS];
  extern __shared__ float4 u_row4[];   // [W / 4]
  const int S = a.S, W = a.W, W4 = a.W >> 2;
  const int r = blockIdx.x;
  const size_t src = a.row_map ? (size_t)a.row_map[r] : (size_t)r;
  const bool has_y = a.delta || a.delta2 || a.routed;
  const bool write = !a.row_map && (a.mix != nullptr || a.x_in != nullptr);
  const int top_k = a.routed ? a.top_k : 0;
  float4 xs[MAXS], y;
  auto fetch = [&](int j4) {
    const size_t col = (size_t)j4 * 4;
    if (a.x_in) {
      const float4 v = *reinterpret_cast<const float4*>(a.x_in + src * W + col);
#pragma unroll
      for (int s = 0; s < MAXS; ++s) xs[s] = v;
    } else {
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) xs[s] = *reinterpret_cast<const float4*>(a.streams + (src * S + s) * W + col);
    }
    y = make_float4(0.f, 0.f, 0.f, 0.f);
    if (has_y) {
      if (a.delta) axpy4(y, 1.f, ld4_any(a.delta, a.delta_dtype, src * W + col));
      if (a.delta2) axpy4(y, 1.f, ld4_any(a.delta2, a.delta2_dtype, src * W + col));
      for (int q = 0; q < top_k; ++q)
        axpy4(y, a.routed_weight ? a.routed_weight[src * top_k + q] : 1.f,
              *reinterpret_cast<const float4*>(a.routed + (size_t)a.slot_of_entry[src * top_k + q] * W + col));
    }
  };
  int j4 = threadIdx.x;
  if (j4 < W4) fetch(j4);
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix_s[i] = a.mix ? a.mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    out_s[i] = a.mix ? a.out_coef[i] * a.mult : 0.f;
    in_s[i] = a.in_coef ? a.in_coef[i] : 1.f;
  }
  __syncthreads();
  float ss = 0.f;
  for (; j4 < W4; j4 += blockDim.x) {
    if (j4 != (int)threadIdx.x) fetch(j4);
    const size_t col = (size_t)j4 * 4;
    float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < MAXS; ++t) {
      if (t < S) {
        float4 nx = xs[t];
        if (a.mix) {
          nx = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int s = 0; s < MAXS; ++s)
            if (s < S) axpy4(nx, mix_s[s * S + t], xs[s]);
          axpy4(nx, out_s[t], y);
        }
        if (write) *reinterpret_cast<float4*>(a.streams + (src * S + t) * W + col) = nx;
        axpy4(u, in_s[t], nx);
      }
    }
    u_row4[j4] = u;
    ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
  }
  const float inv = rsqrtf(hb::block_sum(ss, scratch) / (float)W + a.eps);
  if (!a.y) return;
  for (j4 = threadIdx.x; j4 < W4; j4 += blockDim.x) {
    const float4 u = u_row4[j4];
    const float4 wv = a.w ? ld4_any(a.w, a.w_dtype, (size_t)j4 * 4) : make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 o = make_float4(u.x * inv * wv.x, u.y * inv * wv.y, u.z * inv * wv.z, u.w * inv * wv.w);
    st4_any(a.y, a.y_dtype, (size_t)r * W + (size_t)j4 * 4, o);
    if (a.y_f32) *reinterpret_cast<float4*>(a.y_f32 + (size_t)r * W + (size_t)j4 * 4) = o;
  }
}

// out[t, :] = sum_s streams[t, s, :]
__global__ void hyper_sum_kernel(const float* __restrict__ streams, float* __restrict__ out, int S, int W) {
  const size_t t = blockIdx.x;
  for (int j = threadIdx.x; j < W; j += blockDim.x) {
    float u = 0.f;
    for (int s = 0; s < S; ++s) u += streams[(t * S + s) * W + j];
    out[t * W + j] = u;
  }
}

}  // namespace

extern "C" int hb_hyper_step(float* streams, const float* x_in, const void* delta, int delta_dtype, const void* delta2,
                             int delta2_dtype, const float* routed, const int* slot_of_entry, const float* routed_weight,
                             int top_k, const float* mix, const float* out_coef, float mult, const float* in_coef,
                             const void* w, int w_dtype, float eps, void* y, int y_dtype, float* y_f32,
                             const int* row_map, int rows, int n_streams, int width, cudaStream_t stream) {
  if (!streams || rows < 0 || n_streams <= 0 || width <= 0) return HB_ERR_BAD_ARG;
  if (n_streams > kMaxStreams) return HB_ERR_UNSUPPORTED;
  if (mix && !out_coef) return HB_ERR_BAD_ARG;
  if (routed && (!slot_of_entry || top_k <= 0)) return HB_ERR_BAD_ARG;
  if ((delta || delta2 || routed) && !mix) return HB_ERR_BAD_ARG;     // a result needs its coefficients
  if (row_map && x_in) return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  HyperArgs a;
  a.streams = streams; a.x_in = x_in; a.delta = delta; a.delta_dtype = delta_dtype; a.delta2 = delta2;
  a.delta2_dtype = delta2_dtype; a.routed = routed; a.slot_of_entry = slot_of_entry; a.routed_weight = routed_weight;
  a.top_k = top_k; a.mix = mix; a.out_coef = out_coef; a.mult = mult; a.in_coef = in_coef; a.w = w; a.w_dtype = w_dtype;
  a.eps = eps; a.y = y; a.y_dtype = y_dtype; a.y_f32 = y_f32; a.row_map = row_map; a.S = n_streams; a.W = width;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return HB_ERR_UNSUPPORTED;
  const bool vec = width % 4 == 0 && n_streams <= 8;      // sixteen copies of four columns do not fit a thread's registers
  int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  if (vec) {                       // a thread per four columns, up to 512
    threads = ((width / 4 + 31) / 32) * 32;
    if (threads > 512) threads = 512;
  }
#define HB_HYPER(MAXS)                                                                                     \
  do {                                                                                                     \
    if (smem > 48 * 1024) {                                                                                \
      cudaError_t e = cudaFuncSetAttribute(hyper_step_kernel<MAXS>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                     \
      if (e != cudaSuccess) return (int)e;                                                                 \
    }                                                                                                      \
    if (vec) {                                                                                             \
      if (smem > 48 * 1024) {                                                                              \
        cudaError_t e = cudaFuncSetAttribute(hyper_step_vec_kernel<MAXS>,                                  \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        if (e != cudaSuccess) return (int)e;                                                               \
      }                                                                                                    \
      hyper_step_vec_kernel<MAXS><<<rows, threads, smem, stream>>>(a);                                     \
    } else {                                                                                               \
      hyper_step_kernel<MAXS><<<rows, threads, smem, stream>>>(a);                                         \
    }                                                                                                      \
  } while (0)
  if (n_streams == 1) HB_HYPER(1);
  else if (n_streams <= 2) HB_HYPER(2);
  else if (n_streams <= 4) HB_HYPER(4);
  else if (n_streams <= 8) HB_HYPER(8);
  else HB_HYPER(16);
#undef HB_HYPER
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_hyper_sum(const float* streams, float* out, int rows, int n_streams, int width, cudaStream_t stream) {
  if (!streams || !out || rows < 0 || n_streams <= 0 || width <= 0) return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  hyper_sum_kernel<<<rows, 256, 0, stream>>>(streams, out, n_streams, width);
  HB_LAUNCH_CHECK();
  return HB_OK;
}
